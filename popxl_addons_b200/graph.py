"""`GraphWithNamedArgs` (a graph plus the names of its variable inputs) and `BoundGraph` (a graph plus tensors
already connected to some of its inputs).

Parity: popxl_addons/graph.py:18-294.
"""
from typing import Dict, Iterable, Mapping, Optional, Tuple

from . import xl
from .named_tensors import NamedTensors
from .xl import ops
from .xl.autodiff import ExpectedConnectionType, GradGraphInfo

__all__ = ["BoundGraph", "GraphWithNamedArgs"]


class BoundGraph:
    def __init__(self, graph: xl.Graph, args: Optional[Mapping[xl.Tensor, xl.Tensor]] = None):
        """`args` maps inputs of `graph` to tensors of the calling graph."""
        self.graph = graph
        self.args: Dict[xl.Tensor, xl.Tensor] = dict(args or {})

    def call_with_info(self, *targs, args: Optional[Mapping[xl.Tensor, xl.Tensor]] = None):
        """Call the graph: bound tensors first (overridable through `args`), positional tensors fill the rest."""
        merged = dict(self.args)
        if args:
            merged.update(args)
        return ops.call_with_info(self.graph, *targs, inputs_dict=merged)

    def call(self, *targs, args: Optional[Mapping[xl.Tensor, xl.Tensor]] = None) -> Tuple[xl.Tensor, ...]:
        return self.call_with_info(*targs, args=args).outputs

    def bind(self, args: Mapping[xl.Tensor, xl.Tensor]) -> "BoundGraph":
        """New BoundGraph with `args` (graph input -> caller tensor) connected on top of what is already bound."""
        merged = dict(self.args)
        merged.update(args)
        return BoundGraph(self.graph, merged)

    def subgraph_io_map(self, *targs, args: Optional[Mapping[xl.Tensor, xl.Tensor]] = None,
                        outs: Optional[Iterable[xl.Tensor]] = None):
        """`{graph input: caller tensor}` exactly as `call(*targs, args=args)` would connect them, plus
        `{graph output: caller tensor}` for the call's outputs `outs`, if given."""
        merged = dict(self.args)
        if args:
            merged.update(args)
        free = [t for t in self.graph.inputs if t not in merged]
        for g_in, t in zip(free, targs):
            merged[g_in] = t
        for g_out, t in zip(self.graph.outputs, outs or ()):
            merged[g_out] = t
        return merged


class GraphWithNamedArgs:
    def __init__(self, graph: xl.Graph, args: Optional[NamedTensors] = None,
                 grad_graph_info: Optional[GradGraphInfo] = None, from_module=None, aux=None,
                 called_graphs_grad_info: Optional[Dict[xl.Graph, GradGraphInfo]] = None):
        self.graph = graph
        self.args = args if args is not None else NamedTensors()
        self._grad_graph_info = grad_graph_info
        self.from_module = from_module
        self.aux = aux
        self.called_graphs_grad_info: Dict[xl.Graph, GradGraphInfo] = dict(called_graphs_grad_info or {})
        self._autodiff_applied = False

    @classmethod
    def from_grad_graph(cls, grad_graph_info: GradGraphInfo, args: Optional[NamedTensors] = None):
        return cls(grad_graph_info.graph, args, grad_graph_info)

    # -- binding / calling --------------------------------------------------------------------------------------
    def bind(self, args: Optional[NamedTensors] = None) -> BoundGraph:
        """Connect variables to the named inputs they share a name with."""
        mapping = self.args.to_mapping(args) if args is not None else {}
        return BoundGraph(self.graph, mapping)

    def call(self, *targs, args: Optional[Mapping[xl.Tensor, xl.Tensor]] = None) -> Tuple[xl.Tensor, ...]:
        return self.call_with_info(*targs, args=args).outputs

    def call_with_info(self, *targs, args: Optional[Mapping[xl.Tensor, xl.Tensor]] = None):
        return ops.call_with_info(self.graph, *targs, inputs_dict=dict(args or {}))

    # -- autodiff -----------------------------------------------------------------------------------------------
    def autodiff(self, grads_provided: Optional[Iterable[xl.Tensor]] = None,
                 grads_required: Optional[Iterable[xl.Tensor]] = None,
                 called_graphs_grad_info: Optional[Dict[xl.Graph, GradGraphInfo]] = None,
                 method: str = "auto", force: bool = False) -> "GraphWithNamedArgs":
        """Gradient graph of this graph. `method`: `build_grad` uses the module's hand-written `build_grad`,
        `autodiff` the automatic transform, `auto` picks `build_grad` when the module implements it."""
        if method not in ("auto", "build_grad", "autodiff"):
            raise ValueError(f"method should be one of 'auto', 'build_grad', 'autodiff'. Not: {method}")
        if self._autodiff_applied and not force:
            raise Exception(
                "Autodiff has already been applied to this graph. Applying it again changes the forward graph's "
                "outputs a second time; pass `force=True` if that is intended.")
        use_build_grad = method == "build_grad" or (
            method == "auto" and self.from_module is not None and self.from_module.implements_grad_graph)
        if use_build_grad:
            if self.from_module is None:
                raise Exception("`build_grad` can only be used if `from_module` is specified on the "
                                "GraphWithNamedArgs (graphs made by `Module.create_graph` have it).")
            grad = self.from_module.create_grad_graph(self, grads_provided, grads_required)
        else:
            from .transforms.autodiff import autodiff as _autodiff

            merged = dict(self.called_graphs_grad_info)
            merged.update(called_graphs_grad_info or {})
            grad = _autodiff(self, grads_provided, grads_required, merged)
        self._autodiff_applied = True
        return grad

    @property
    def grad_graph_info(self) -> GradGraphInfo:
        if self._grad_graph_info is None:
            raise AttributeError("`grad_graph_info` is only available on gradient graphs (the result of `autodiff`)")
        return self._grad_graph_info

    @grad_graph_info.setter
    def grad_graph_info(self, info: GradGraphInfo):
        self._grad_graph_info = info

    def copy(self) -> "GraphWithNamedArgs":
        g = GraphWithNamedArgs(self.graph, self.args.copy(), self._grad_graph_info, self.from_module, self.aux,
                               dict(self.called_graphs_grad_info))
        g._autodiff_applied = self._autodiff_applied
        return g

    def print_schedule(self) -> str:
        """Text dump: named inputs, other inputs, ops in execution order, outputs."""
        named = {t: k for k, t in self.args.to_dict().items()}
        lines = [f"Graph : {self.graph.name}", "  Named inputs:"]
        for t in self.graph.inputs:
            if t in named:
                lines.append(f"    {named[t]}: {t.dtype} {t.shape}" + (f" meta={t.meta_shape}" if t.meta_shape else ""))
        lines.append("  Inputs:")
        for t in self.graph.inputs:
            if t not in named:
                lines.append(f"    {t.id}: {t.dtype} {t.shape}")
        lines.append("  Ops:")
        for op in self.graph.ops:
            callee = op.attrs.get("graph")
            extra = f" -> {callee.name}" if isinstance(callee, xl.Graph) else ""
            lines.append(f"    {op.opdef.name}{extra}: ({', '.join(t.id for t in op.inputs)}) -> "
                         f"({', '.join(t.id for t in op.outputs)})")
        lines.append("  Outputs:")
        for t in self.graph.outputs:
            lines.append(f"    {t.id}: {t.dtype} {t.shape}")
        text = "\n".join(lines)
        print(text)
        return text
