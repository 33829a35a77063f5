"""`Module`: stateful description of a computation that turns into (variable factories, graph).

`build` is traced once per `create_graph`; every `add_variable_input` inside registers a graph input together with the
factory that will create its variables. Sub-modules assigned as attributes are inlined and contribute their inputs
under the attribute name; `call_module` outlines a sub-module into its own graph instead. A module may provide a
hand-written backward pass with `build_grad`, using `self.aux` to carry forward tensors and `self.var_grad` to name
the gradients of its variables.

Parity: popxl_addons/module.py:66-753.
"""
import contextlib
import inspect
import warnings
from typing import Any, Callable, Dict, List, Optional, Set, Tuple, Union

from . import xl
from .graph import BoundGraph, GraphWithNamedArgs
from .graph_cache import GraphCache
from .named_tensors import NamedTensors
from .utils import OrderedDict, duplicate_items, overrides
from .variable_factory import (NamedVariableFactories, VariableFactory, add_replica_sharded_variable_input,
                               add_variable_input)
from .xl.autodiff import ExpectedConnection, ExpectedConnectionType, GradGraphInfo

__all__ = ["Module", "NameScopeMeta", "NamedTensors", "NamedVariableFactories", "VariableFactory",
           "add_variable_input", "add_replica_sharded_variable_input", "GraphWithNamedArgs", "BoundGraph",
           "GraphCache", "create_grad_graph_info"]

_BUILD_STACK: List["Module"] = []
_BUILD_GRAD_STACK: List["Module"] = []


@contextlib.contextmanager
def _building(stack: List["Module"], module: "Module"):
    stack.append(module)
    try:
        yield
    finally:
        stack.pop()


def _current(stack):
    return stack[-1] if stack else None


class NameScopeMeta(type):
    """Wraps `build` of every subclass so that tensors created inside carry the module's attribute name as scope."""

    def __new__(mcls, name, bases, ns):
        build = ns.get("build")
        if build is not None and not getattr(build, "_scoped", False):
            def scoped_build(self, *args, __build=build, **kwargs):
                scope = getattr(self, "_name_scope", None)
                if scope:
                    with xl.name_scope(scope):
                        return __build(self, *args, **kwargs)
                return __build(self, *args, **kwargs)

            scoped_build._scoped = True
            scoped_build.__wrapped__ = build
            scoped_build.__signature__ = inspect.signature(build)
            scoped_build.__name__ = "build"
            scoped_build.__doc__ = build.__doc__
            ns["build"] = scoped_build
        return super().__new__(mcls, name, bases, ns)


class _Aux:
    """Forward tensors (or plain Python values) a hand-written backward pass needs.
    Written in `build`; read in `build_grad`, where the first read of a tensor creates the matching grad-graph input."""

    def __init__(self):
        self._values = OrderedDict()
        self._grad_inputs: "OrderedDict[str, xl.Tensor]" = OrderedDict()
        self._grad_to_fwd: "OrderedDict[xl.Tensor, xl.Tensor]" = OrderedDict()

    def __setitem__(self, key, value):
        self._values[key] = value

    def __getitem__(self, key):
        owner = _current(_BUILD_GRAD_STACK)
        if owner is None or owner.aux is not self:
            raise Exception("You can only get items within the `build_graph` method which must be called via "
                            "`create_grad_graph` or `autodiff`.")
        value = self._values[key]
        if not isinstance(value, xl.Tensor):
            return value
        if key not in self._grad_inputs:
            gi = xl.graph_input(value.shape, value.dtype, str(key), False, value.meta_shape)
            self._grad_inputs[key] = gi
            self._grad_to_fwd[gi] = value
        return self._grad_inputs[key]

    def __contains__(self, key):
        return key in self._values

    def __repr__(self):
        return repr(self._values)

    def copy(self) -> "_Aux":
        c = _Aux()
        c._values = self._values.copy()
        c._grad_inputs = self._grad_inputs.copy()
        c._grad_to_fwd = self._grad_to_fwd.copy()
        return c


class _VarGrads:
    """`var_grad[name] = tensor` inside `build_grad` declares the gradient of variable `name`."""

    _MSG = ("You can only use` var_grad` within the `build_graph` method which must be called via "
            "`create_grad_graph` or `autodiff`.")

    def __init__(self, required: Optional[Dict[str, xl.Tensor]] = None):
        self._grads = OrderedDict()
        self._required = required

    def _check(self):
        owner = _current(_BUILD_GRAD_STACK)
        if owner is None or owner.var_grad is not self or self._required is None:
            raise Exception(self._MSG)

    def __getitem__(self, key):
        self._check()
        return self._grads[key]

    def __setitem__(self, key, tensor):
        self._check()
        if not isinstance(tensor, xl.Tensor):
            raise TypeError(f"Not a tensor: {tensor}")
        if key not in self._required:
            raise KeyError(f"Not a variable: {key}. Possible inputs: {list(self._required.keys())}")
        var = self._required[key]
        if tuple(var.shape) != tuple(tensor.shape) or tuple(var.meta_shape) != tuple(tensor.meta_shape):
            raise ValueError("Shape or meta-shape of Tensor does not match variable. "
                             f"Tensor shape: {tensor.shape} meta-shape {tensor.meta_shape}. "
                             f"Variable shape {var.shape} meta-shape {var.meta_shape}.")
        self._grads[key] = tensor

    def __contains__(self, key):
        return key in self._grads

    def __repr__(self):
        return repr(self._grads)


def _as_graph(g) -> xl.Graph:
    return g.graph if isinstance(g, (GraphWithNamedArgs, BoundGraph)) else g


def _as_info(g) -> GradGraphInfo:
    return g.grad_graph_info if isinstance(g, GraphWithNamedArgs) else g


class _CalledGraphsGradInfoRefs:
    """`{forward graph: GradGraphInfo}` for outlined sub-graphs with custom gradients, kept as a tree of references so
    sub-modules can keep adding entries after they were attached to their parent."""

    def __init__(self, mapping=None):
        self.map: Dict[xl.Graph, GradGraphInfo] = {_as_graph(k): _as_info(v) for k, v in (mapping or {}).items()}
        self.submaps: List["_CalledGraphsGradInfoRefs"] = []

    def add(self, fwd_graph, grad_graph):
        self.map[_as_graph(fwd_graph)] = _as_info(grad_graph)

    def add_submap(self, other):
        if not isinstance(other, _CalledGraphsGradInfoRefs):
            other = _CalledGraphsGradInfoRefs(other)
        self.submaps.append(other)

    def consolidate(self) -> Dict[xl.Graph, GradGraphInfo]:
        out: Dict[xl.Graph, GradGraphInfo] = {}
        for sub in self.submaps:
            out.update(sub.consolidate())
        out.update(self.map)  # own entries win
        return out

    def clear(self):
        for sub in self.submaps:
            sub.clear()
        self.map = {}
        self.submaps = []


def create_grad_graph_info(ir: xl.Ir, fwd_graph: xl.Graph, grad_graph: xl.Graph,
                           grad_input_to_fwd_output: "OrderedDict[xl.Tensor, xl.Tensor]",
                           grad_output_to_fwd_input: "OrderedDict[xl.Tensor, xl.Tensor]",
                           fwd_tensors: Set[xl.Tensor]) -> GradGraphInfo:
    """Describe a hand-built gradient graph: its inputs are gradients of forward outputs (`FwdGrad`) except those
    whose forward tensor is in `fwd_tensors` (plain forward values, `Fwd`); its outputs are gradients of forward
    inputs, in order."""
    expected_inputs = [
        ExpectedConnection(fwd_t, ExpectedConnectionType.Fwd if fwd_t in fwd_tensors else ExpectedConnectionType.FwdGrad)
        for fwd_t in grad_input_to_fwd_output.values()]
    expected_outputs = [ExpectedConnection(fwd_t, ExpectedConnectionType.FwdGrad)
                        for fwd_t in grad_output_to_fwd_input.values()]
    return GradGraphInfo(grad_graph, fwd_graph, expected_inputs, expected_outputs)


class Module(metaclass=NameScopeMeta):
    def __init__(self, cache: bool = False, grad_inlining_error: str = "error"):
        """`cache`: `create_graph` re-uses a graph for identical argument specs. `grad_inlining_error`: what to do
        when a module that implements `build_grad` is inlined (`error` / `warning` / `none`), because inlining
        silently drops the custom gradient."""
        object.__setattr__(self, "_variable_factories", NamedVariableFactories())
        object.__setattr__(self, "_named_inputs", NamedTensors())
        object.__setattr__(self, "called_graphs_grad_info", _CalledGraphsGradInfoRefs())
        self._graph_cache = GraphCache() if cache else None
        self._args_cache: Dict[xl.Graph, Tuple[NamedVariableFactories, NamedTensors]] = {}
        self.aux = _Aux()
        self.var_grad = _VarGrads()
        self.grad_inlining_error = grad_inlining_error
        if cache and self.implements_grad_graph:
            raise ValueError("You cannot use graph caching if you have implemented `build_grad`.")
        if grad_inlining_error not in ("error", "warning", "none"):
            raise ValueError(
                f"grad_inlining_error should be one of 'error', 'warning', 'none'. Not: {grad_inlining_error}")

    # -- to be provided by subclasses ---------------------------------------------------------------------------
    def build(self, *args, **kwargs):
        raise NotImplementedError("Your Module must implement the `build` method")

    def build_grad(self, *args, **kwargs):
        """Hand-written backward pass. Takes one gradient per forward output (in order), returns one gradient per
        non-variable forward input (in order); gradients of variables are declared through `self.var_grad`."""
        raise NotImplementedError("Your Module must implement the `build_grad` method to create a gradient graph.")

    @property
    def implements_grad_graph(self) -> bool:
        return overrides(type(self), Module, "build_grad")

    # -- calling (inlining) -------------------------------------------------------------------------------------
    def __call__(self, *args, **kwargs):
        if self.implements_grad_graph and _current(_BUILD_STACK) is not self:
            msg = ("You are calling this module directly but `build_grad` has been implemented. If you call this "
                   "module directly `build_grad` will not be called when using autodiff. You need to create a graph "
                   "of this module first and call that graph e.g. use `self.call_module`. To disable this guardrail "
                   "set `grad_inlining_error` to `none`")
            if self.grad_inlining_error == "error":
                raise Exception(msg)
            if self.grad_inlining_error == "warning":
                warnings.warn(msg)
        return self.build(*args, **kwargs)

    def set_name_scope(self, name: str):
        object.__setattr__(self, "_name_scope", name)

    def __setattr__(self, key: str, value: Any) -> None:
        if isinstance(value, Module):
            value.set_name_scope(key)
            self._variable_factories.insert(key, value._variable_factories)
            self._named_inputs.insert(key, value._named_inputs)
            self.called_graphs_grad_info.add_submap(value.called_graphs_grad_info)
        object.__setattr__(self, key, value)

    def _reset(self):
        self._variable_factories._clear()
        self._named_inputs._clear()
        self.called_graphs_grad_info.clear()
        self.aux = _Aux()
        self.var_grad = _VarGrads()

    # -- graph creation -----------------------------------------------------------------------------------------
    def create_graph(self, *args, **kwargs) -> Tuple[NamedVariableFactories, GraphWithNamedArgs]:
        """Trace `build` into a new graph. Tensor / TensorSpec arguments become graph inputs. Returns the variable
        factories of all `add_variable_input` calls and the graph with its named inputs. The module itself keeps no
        state afterwards and can create further graphs."""
        if self._graph_cache is not None:
            graph = self._graph_cache.create_graph(self, *args, **kwargs)
            if graph not in self._args_cache:
                self._args_cache[graph] = (self._variable_factories.copy(), self._named_inputs.copy())
            factories, named_inputs = self._args_cache[graph]
        else:
            self.aux = _Aux()
            with _building(_BUILD_STACK, self):
                graph = xl.gcg().ir.create_graph(self, *args, **kwargs)
            if self.implements_grad_graph:
                graph.can_autodiff = False
            factories, named_inputs = self._variable_factories, self._named_inputs
        result = GraphWithNamedArgs(graph, named_inputs.copy(), from_module=self, aux=self.aux.copy(),
                                    called_graphs_grad_info=self.called_graphs_grad_info.consolidate())
        factories = factories.copy()
        self._reset()
        return factories, result

    # -- hand-written gradient graphs ---------------------------------------------------------------------------
    def _validate_grad_request(self, fwd: GraphWithNamedArgs, grads_provided, grads_required):
        sig = inspect.signature(self.build_grad, follow_wrapped=True)
        for pname, p in sig.parameters.items():
            if p.kind not in (inspect.Parameter.POSITIONAL_ONLY, inspect.Parameter.POSITIONAL_OR_KEYWORD):
                raise TypeError("The `build_grad` method signature must only have a fixed number of positional "
                                f"parameters as inputs. Not a positional parameter: {pname}")
        if grads_provided is None:
            provided = list(fwd.graph.outputs)
        else:
            provided = list(grads_provided)
            for t in provided:
                if not isinstance(t, xl.Tensor) or t not in fwd.graph.outputs:
                    raise ValueError(f"A Tensor specified in `grads_provided` is not a output of `fwd_graph` "
                                     f"or not a Tensor: {t}")
            if duplicate_items(provided):
                raise ValueError("A Tensor has been specified more than once in `grads_provided`. "
                                 f"Duplicates: {duplicate_items(provided)}")
        if grads_required is None:
            required = list(fwd.graph.inputs)
        else:
            required = list(grads_required)
            for t in required:
                if not isinstance(t, xl.Tensor) or t not in fwd.graph.inputs:
                    raise ValueError(f"A Tensor specified in `grads_required` is not a input of `fwd_graph` "
                                     f"or not a Tensor: {t}")
            if duplicate_items(required):
                raise ValueError("A Tensor has been specified more than once in `grads_required`. "
                                 f"Duplicates: {duplicate_items(required)}")
        name_of = {t: k for k, t in fwd.args.to_dict().items()}
        required_vars = OrderedDict((name_of[t], t) for t in required if t in name_of)
        required_other = [t for t in required if t not in name_of]
        return provided, required, required_other, required_vars

    def create_grad_graph(self, fwd_graph: GraphWithNamedArgs, grads_provided=None,
                          grads_required=None) -> GraphWithNamedArgs:
        """Trace `build_grad` into the gradient graph of `fwd_graph` (which this module created). The forward graph
        gains one output per `aux` tensor that `build_grad` read, so this must happen before the forward graph is
        called."""
        provided, required, required_other, required_vars = self._validate_grad_request(
            fwd_graph, grads_provided, grads_required)
        ir = fwd_graph.graph.ir
        self.aux = fwd_graph.aux.copy() if fwd_graph.aux is not None else _Aux()
        # any variable of the forward graph may be given a gradient; only the required ones become outputs
        self.var_grad = _VarGrads(OrderedDict(fwd_graph.args.to_dict()))
        with _building(_BUILD_GRAD_STACK, self):
            grad_graph = ir.create_graph(self.build_grad, *[t.spec for t in provided])
        grad_graph.name = fwd_graph.graph.name.split("_subgraph")[0] + "_grad" + grad_graph.name[
            grad_graph.name.index("_subgraph"):] if "_subgraph" in grad_graph.name else grad_graph.name
        missing = set(required_vars) - set(self.var_grad._grads)
        if missing:
            raise Exception("Not all variable gradients have been specified in self.var_grad. If you dont want to "
                            "output all gradients specify `grads_required` when calling autodiff. "
                            f"Variables missing gradients: {missing}")
        n_out = len(grad_graph.outputs)
        if n_out > len(required_other):
            raise Exception(f"Too many outputs in the grad graph. `grads_required` has {len(required_other)} "
                            "non-variable outputs. If you dont want to output all gradients specify "
                            "`grads_required` when calling autodiff.")
        if n_out < len(required_other):
            raise Exception("Not all forward graph inputs have been specified as outputs in the grad graph. If you "
                            "dont want to output all gradients specify `grads_required` when calling autodiff. "
                            f"Outputs missing: {required_other[n_out:]}")
        for i, (out, req) in enumerate(zip(grad_graph.outputs, required_other)):
            if tuple(out.shape) != tuple(req.shape) or tuple(out.meta_shape) != tuple(req.meta_shape):
                raise ValueError(
                    f"Shape or meta-shape of output Tensor at position {i} does not match the `grad_required` at "
                    f"position {i}. Output Tensor shape: {out.shape} meta-shape {out.meta_shape}. "
                    f"Grad required shape {req.shape} meta-shape {req.meta_shape}.")
        # gradients of variables become further outputs, in `grads_required` order
        grad_out_to_fwd_in = OrderedDict(zip(grad_graph.outputs, required_other))
        with grad_graph:
            for name, var_input in required_vars.items():
                g = self.var_grad._grads[name]
                if g in grad_graph.outputs or g in grad_graph.inputs:
                    g = xl.ops.identity(g)
                xl.graph_output(g)
                grad_out_to_fwd_in[g] = var_input
        # stitching: every aux tensor read by build_grad becomes a forward output
        n_provided = len(provided)
        grad_in_to_fwd_out = OrderedDict(zip(grad_graph.inputs[:n_provided], provided))
        aux_fwd: Set[xl.Tensor] = set()
        for gi in grad_graph.inputs[n_provided:]:
            fwd_t = self.aux._grad_to_fwd[gi]
            if fwd_t not in fwd_graph.graph._outputs:
                fwd_graph.graph._outputs.append(fwd_t)
            grad_in_to_fwd_out[gi] = fwd_t
            aux_fwd.add(fwd_t)
        info = create_grad_graph_info(ir, fwd_graph.graph, grad_graph, grad_in_to_fwd_out, grad_out_to_fwd_in,
                                      aux_fwd)
        self._reset()
        return GraphWithNamedArgs.from_grad_graph(info)

    # -- registering inputs -------------------------------------------------------------------------------------
    def add_variable_factory(self, variable_f: VariableFactory, name: Optional[str] = None,
                             overwrite: bool = False) -> xl.Tensor:
        name = name or variable_f.name
        if name is None:
            raise ValueError("A variable factory needs a name (its own or the `name` argument)")
        variable_f.name = variable_f.name or name
        tensor = variable_f.create_input()
        self._variable_factories.insert(name, variable_f, overwrite)
        self._named_inputs.insert(name, tensor, overwrite)
        return tensor

    def add_variable_input(self, name: str, data_iter, dtype: Optional[xl.dtype] = None, by_ref: bool = False,
                           replica_grouping: Optional[xl.ReplicaGrouping] = None,
                           overwrite: bool = False) -> xl.Tensor:
        """Add a graph input that will be fed by a variable. `data_iter` (callable or iterable) supplies the initial
        value of each variable created for it. Replicas in one group of `replica_grouping` share the value."""
        tensor, factory = add_variable_input(name, data_iter, dtype, by_ref, replica_grouping)
        self._variable_factories.insert(name, factory, overwrite)
        self._named_inputs.insert(name, tensor, overwrite)
        return tensor

    def add_replica_sharded_variable_input(self, name: str, data_iter, dtype: Optional[xl.dtype] = None,
                                           by_ref: bool = False,
                                           replica_grouping: Optional[xl.ReplicaGrouping] = None,
                                           shard_over: Optional[int] = None, overwrite: bool = False) -> xl.Tensor:
        """As `add_variable_input`, for a tensor stored as flat `1/shard_over` shards across the replicas of each
        group (gather it with `ops.collectives.replicated_all_gather` before use)."""
        tensor, factory = add_replica_sharded_variable_input(name, data_iter, dtype, by_ref, replica_grouping,
                                                             shard_over)
        self._variable_factories.insert(name, factory, overwrite)
        self._named_inputs.insert(name, tensor, overwrite)
        return tensor

    def add_variable_inputs(self, name: Union[str, int], variable_f: NamedVariableFactories,
                            overwrite: bool = False) -> NamedTensors:
        """Instantiate the variables of an outlined sub-graph as inputs of the current graph under `name`; the
        returned tensors can be bound to the sub-graph. Calling this twice with different names gives two sets of
        weights for one compute graph."""
        if isinstance(name, int):
            if name < 0:
                raise ValueError(f"Name of int type must be positive. Value: {name}")
            name = str(name)
        tensors = NamedTensors.from_dict({k: f.create_input() for k, f in variable_f.to_dict().items()})
        self._variable_factories.insert(name, variable_f.copy(), overwrite=overwrite)
        self._named_inputs.insert(name, tensors, overwrite=overwrite)
        return tensors

    # -- containers ---------------------------------------------------------------------------------------------
    @classmethod
    def from_list(cls, sub_modules: List["Module"]) -> "Module":
        self = cls()
        for i, m in enumerate(sub_modules):
            setattr(self, str(i), m)
        object.__setattr__(self, "_sub_modules", list(sub_modules))
        return self

    @classmethod
    def from_variable_factories(cls, inputs: List[VariableFactory]) -> "Module":
        self = cls()
        for i, f in enumerate(inputs):
            object.__setattr__(self, str(i), self.add_variable_factory(f, name=str(i)))
        return self

    def get(self, key: Union[str, int]):
        return getattr(self, str(key) if isinstance(key, int) else key)

    def __getitem__(self, item: Union[str, int]):
        return self.get(item)

    def __iter__(self):
        subs = self.__dict__.get("_sub_modules")
        if subs is None:
            raise AttributeError("Iterating over a Module that was not created with `Module.from_list` is not "
                                 "supported.")
        return iter(subs)

    def call_module(self, module: "Module", name: Optional[str] = None, autodiff: str = "auto",
                    grads_provided: Optional[Callable] = None, grads_required: Optional[Callable] = None):
        """Outline `module`: `self.call_module(Sub())(x)` creates Sub's graph, registers its variables under `name`
        (default: the class name), differentiates it first when it has (or is asked to have) a gradient graph, and
        calls it."""
        return _CallModule(self, module, name, autodiff, grads_provided, grads_required)


class _CallModule:
    def __init__(self, caller: Module, callee: Module, name, autodiff, grads_provided, grads_required):
        if autodiff not in ("auto", "build_grad", "autodiff", "none"):
            raise ValueError(f"autodiff should be one of 'auto', 'build_grad', 'autodiff', 'none'. Not: {autodiff}")
        self.caller, self.callee = caller, callee
        self.name = name or type(callee).__name__
        self.autodiff = autodiff
        self.grads_provided, self.grads_required = grads_provided, grads_required

    def __call__(self, *args, **kwargs) -> Tuple[xl.Tensor, ...]:
        factories, graph = self.callee.create_graph(*args, **kwargs)
        graph_vars = self.caller.add_variable_inputs(self.name, factories)
        self.caller.called_graphs_grad_info.add_submap(graph.called_graphs_grad_info)
        n_outputs = len(graph.graph.outputs)
        wants_grad = self.autodiff in ("build_grad", "autodiff") or (
            self.autodiff == "auto" and self.callee.implements_grad_graph)
        if wants_grad:
            provided = self.grads_provided(graph) if self.grads_provided else None
            required = self.grads_required(graph) if self.grads_required else None
            grad_graph = graph.autodiff(method=self.autodiff, grads_provided=provided, grads_required=required)
            self.caller.called_graphs_grad_info.add(graph, grad_graph)
        tensor_args = [a for a in args if isinstance(a, xl.Tensor)]
        tensor_kwargs = {k: v for k, v in kwargs.items() if isinstance(v, xl.Tensor)}
        bound = graph.bind(graph_vars)
        inputs_dict = {}
        if tensor_kwargs:
            by_name = {t.name.split("/")[-1]: t for t in graph.graph.inputs}
            for k, v in tensor_kwargs.items():
                inputs_dict[by_name[k]] = v
        outs = bound.call(*tensor_args, args=inputs_dict)
        self.var_factories, self.graph, self.n_outputs_pre_autodiff = factories, graph, n_outputs
        return tuple(outs[:n_outputs])
