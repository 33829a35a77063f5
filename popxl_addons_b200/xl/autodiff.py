"""Reverse-mode differentiation of a recorded graph into an explicit gradient graph.

The gradient graph is an ordinary `Graph`. Its leading inputs are described by `GradGraphInfo.expected_inputs`:
`FwdGrad` entries are gradients of forward outputs, `Fwd` entries are forward tensors (activations, weights) the
backward pass needs. Forward intermediates that are needed become extra outputs of the forward graph, so one
particular forward call site can feed one gradient call (`GradGraphInfo.inputs_dict(call_info)`), and so that
activations are explicit tensors which can be stashed, offloaded or recomputed by the transforms.

Parity: `popxl.transforms.autodiff` / `GradGraphInfo` / `ExpectedConnection` as used by
popxl_addons/transforms/autodiff.py:26-105, module.py:713-753 and transforms/recomputation.py:22-42.
"""
import enum
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

from .core import Constant, Graph, Tensor, constant, gcg, graph_input, graph_output, name_scope
from .opdef import emit


class ExpectedConnectionType(enum.Enum):
    Fwd = "Fwd"
    FwdGrad = "FwdGrad"


class ExpectedConnection:
    def __init__(self, fwd_tensor: Tensor, connection_type: ExpectedConnectionType):
        self.fwd_tensor = fwd_tensor
        self.connection_type = connection_type

    def __repr__(self):
        return f"({self.connection_type.value}, {self.fwd_tensor.id})"


class GradGraphInfo:
    def __init__(self, graph: Graph, forward_graph: Graph, expected_inputs: List[ExpectedConnection],
                 expected_outputs: List[ExpectedConnection]):
        self.graph = graph
        self.forward_graph = forward_graph
        self._expected_inputs = list(expected_inputs)
        self._expected_outputs = list(expected_outputs)

    @property
    def expected_inputs(self) -> Tuple[ExpectedConnection, ...]:
        return tuple(self._expected_inputs)

    @property
    def expected_outputs(self) -> Tuple[ExpectedConnection, ...]:
        return tuple(self._expected_outputs)

    @property
    def inputs(self) -> Tuple[Tensor, ...]:
        return tuple(ec.fwd_tensor for ec in self._expected_inputs)

    @property
    def outputs(self) -> Tuple[Tensor, ...]:
        return tuple(ec.fwd_tensor for ec in self._expected_outputs)

    def inputs_dict(self, fwd_call_info) -> Dict[Tensor, Tensor]:
        """`{grad graph input: tensor at the forward call site}` for every `Fwd` expected input."""
        out = {}
        for gi, ec in zip(self.graph._inputs, self._expected_inputs):
            if ec.connection_type == ExpectedConnectionType.Fwd:
                out[gi] = fwd_call_info.graph_to_parent(ec.fwd_tensor)
        return out

    def fwd_parent_ins_to_grad_parent_outs(self, fwd_call_info, grad_call_info) -> Dict[Tensor, Tensor]:
        """`{forward call-site input: gradient call-site output holding its gradient}`."""
        return {fwd_call_info.graph_to_parent(ec.fwd_tensor): grad_call_info.parent_output(i)
                for i, ec in enumerate(self._expected_outputs)}

    def fwd_graph_ins_to_grad_parent_outs(self, grad_call_info) -> Dict[Tensor, Tensor]:
        return {ec.fwd_tensor: grad_call_info.parent_output(i) for i, ec in enumerate(self._expected_outputs)}


class _Ctx:
    """State of one autodiff run; passed to the vjp rules."""

    def __init__(self, fwd_graph: Graph, grad_graph: Graph, called: Dict[Graph, GradGraphInfo], all_infos):
        self.fwd_graph = fwd_graph
        self.grad_graph = grad_graph
        self.called = called
        self.all_infos = all_infos
        self.fwd_inputs: Dict[Tensor, Tensor] = {}
        self.expected: List[ExpectedConnection] = []
        self.pending_fwd: List[Tuple[Tensor, Tensor]] = []

    def fwd(self, t: Tensor) -> Tensor:
        """Grad-graph tensor that carries the value of forward tensor `t`."""
        if t in self.fwd_inputs:
            return self.fwd_inputs[t]
        if isinstance(t, Constant):
            c = constant(t.data, t.dtype, t.id.split("/")[-1])
            self.fwd_inputs[t] = c
            return c
        gi = graph_input(t.shape, t.dtype, t.id.split("/")[-1], meta_shape=t.meta_shape)
        self.fwd_inputs[t] = gi
        self.pending_fwd.append((t, gi))
        return gi

    def vjp_call(self, op, gs):
        from .ops.control import _sync_call_outputs

        callee: Graph = op.attrs["graph"]
        info = self.called.get(callee)
        if info is None:
            if not callee.can_autodiff:
                raise RuntimeError(
                    f"The called graph {callee.name} is marked as unsafe to autodiff (it has a custom gradient). "
                    f"Provide its GradGraphInfo through `called_graphs_grad_info`.")
            info = _autodiff(callee, None, None, self.called, self.all_infos)
            self.called[callee] = info
        _sync_call_outputs(op)
        gg = info.graph
        inputs_dict = {}
        for gi, ec in zip(gg._inputs, info._expected_inputs):
            if ec.connection_type == ExpectedConnectionType.FwdGrad:
                idx = callee._outputs.index(ec.fwd_tensor)
                g = gs[idx] if idx < len(gs) else None
                if g is None:
                    g = constant(0, ec.fwd_tensor.dtype)
                    from .ops import expand

                    g = expand(g, ec.fwd_tensor.shape) if ec.fwd_tensor.shape else g
                inputs_dict[gi] = g
            else:
                t = ec.fwd_tensor
                if t in callee._inputs:
                    parent = op.inputs[callee._inputs.index(t)]
                else:
                    parent = op.outputs[callee._outputs.index(t)]
                inputs_dict[gi] = self.fwd(parent)
        if len(gg._inputs) > len(info._expected_inputs):
            raise RuntimeError(
                f"The gradient graph {gg.name} has inputs beyond its expected connections; it cannot be called "
                f"automatically from an enclosing gradient graph.")
        from .ops.control import call

        outs = call(gg, inputs_dict=inputs_dict)
        in_grads: List[Optional[Tensor]] = [None] * len(op.inputs)
        for o, ec in zip(outs, info._expected_outputs):
            in_grads[callee._inputs.index(ec.fwd_tensor)] = o
        return in_grads


def _relevant_ops(graph: Graph, provided: List[Tensor], required: List[Tensor]):
    """Ops that lie on a path from a required input to a provided output."""
    reach = set(required)
    fwd_ops = set()
    for op in graph.ops:
        if any(t in reach for t in op.inputs):
            fwd_ops.add(op.uid)
            reach.update(op.outputs)
    need = set(provided)
    out = set()
    for op in reversed(graph.ops):
        if op.uid in fwd_ops and any(t in need for t in op.outputs):
            out.add(op.uid)
            need.update(t for t in op.inputs if t in reach)
    return out, reach


def _autodiff(graph: Graph, grads_provided, grads_required, called, all_infos) -> GradGraphInfo:
    provided = list(grads_provided) if grads_provided is not None else list(graph._outputs)
    required = list(grads_required) if grads_required is not None else list(graph._inputs)
    for t in provided:
        if t not in graph._outputs:
            raise ValueError(f"{t} is not an output of the graph {graph.name}")
    for t in required:
        if t not in graph._inputs:
            raise ValueError(f"{t} is not an input of the graph {graph.name}")
    from .ops import add

    ir = graph.ir
    from ..utils import suffix_graph_name

    grad_graph = Graph(ir, suffix_graph_name(graph.name, "grad") + f"_subgraph({next(ir._graph_counter)})")
    ir.graphs.append(grad_graph)
    ctx = _Ctx(graph, grad_graph, called, all_infos)
    relevant, reach = _relevant_ops(graph, provided, required)
    expected_inputs: List[ExpectedConnection] = []
    grads: Dict[Tensor, Tensor] = {}
    with grad_graph, name_scope("grad"):
        for t in provided:
            gi = graph_input(t.shape, t.dtype, t.id.split("/")[-1] + "_grad", meta_shape=t.meta_shape)
            grads[t] = gi
            expected_inputs.append(ExpectedConnection(t, ExpectedConnectionType.FwdGrad))
        n_fwdgrad = len(expected_inputs)
        for op in reversed(graph.ops):
            if op.uid not in relevant:
                continue
            out_grads = [grads.get(o) for o in op.outputs]
            if all(g is None for g in out_grads):
                continue
            if op.opdef.vjp is None:
                raise NotImplementedError(f"Op `{op.opdef.name}` in graph {graph.name} has no gradient rule")
            if op.opdef.name != "call" and out_grads[0] is None:
                # secondary outputs (saved statistics, masks) carry no gradient of their own
                continue
            in_grads = op.opdef.vjp(ctx, op, out_grads)
            for inp, g in zip(op.inputs, in_grads):
                if g is None or inp not in reach:
                    continue
                if not inp.dtype.is_floating_point:
                    continue
                if g.dtype != inp.dtype:
                    from .ops import cast

                    g = cast(g, inp.dtype)
                grads[inp] = g if inp not in grads else add(grads[inp], g)
        expected_outputs = []
        for t in required:
            g = grads.get(t)
            if g is None:
                from .ops import init

                g = init(t.shape, t.dtype, t.id.split("/")[-1] + "_zero_grad", "zero")
            if g in grad_graph._inputs or g in grad_graph._outputs:
                from .ops import identity

                g = identity(g)
            graph_output(g)
            expected_outputs.append(ExpectedConnection(t, ExpectedConnectionType.FwdGrad))
    # order grad-graph inputs: FwdGrad first (creation order), then Fwd in creation order
    for t, gi in ctx.pending_fwd:
        expected_inputs.append(ExpectedConnection(t, ExpectedConnectionType.Fwd))
    # stitching: forward intermediates needed by the backward pass become forward-graph outputs
    for t, _ in ctx.pending_fwd:
        if t not in graph._inputs and t not in graph._outputs:
            graph._outputs.append(t)
    info = GradGraphInfo(grad_graph, graph, expected_inputs, expected_outputs)
    all_infos[graph] = info
    return info


def autodiff(graph: Graph, grads_provided: Optional[Iterable[Tensor]] = None,
             grads_required: Optional[Iterable[Tensor]] = None,
             called_graphs_grad_info: Optional[Mapping[Graph, GradGraphInfo]] = None,
             return_all_grad_graphs: bool = False):
    """Differentiate `graph`. Returns its `GradGraphInfo`, or with `return_all_grad_graphs` a dict
    `{forward graph: GradGraphInfo}` that also holds the gradient graphs created for called sub-graphs."""
    called = dict(called_graphs_grad_info or {})
    all_infos: Dict[Graph, GradGraphInfo] = {}
    info = _autodiff(graph, grads_provided, grads_required, called, all_infos)
    if return_all_grad_graphs:
        return all_infos
    return info
