"""Make a tensor of a parent graph available inside a (possibly deeply nested) called sub-graph.

Sub-graphs only see their own inputs. `route_tensor_into_graph` adds a graph input to the target graph and to every
graph on every call path between the tensor's graph and the target, and wires all call / repeat sites along those
paths, so the tensor arrives wherever the target is executed.

Parity: popxl_addons/route_tensor.py:11-221.
"""
from typing import Dict, Optional, Set, Tuple

from . import xl

__all__ = ["route_tensor_into_graph", "is_subgraph"]


def _called(op) -> Optional[xl.Graph]:
    g = op.attrs.get("graph")
    return g if isinstance(g, xl.Graph) and op.opdef.name in ("call", "repeat") else None


def is_subgraph(parent: xl.Graph, subgraph: xl.Graph) -> bool:
    """Is `subgraph` (transitively) called from `parent`?"""
    seen: Set[int] = set()
    stack = [parent]
    while stack:
        g = stack.pop()
        for op in g.ops:
            c = _called(op)
            if c is None or id(c) in seen:
                continue
            if c is subgraph:
                return True
            seen.add(id(c))
            stack.append(c)
    return False


def called_graph_paths(parent_graph: xl.Graph, subgraph: xl.Graph) -> Set[Tuple[xl.Graph, ...]]:
    """All chains of graphs `(g1, ..., subgraph)` such that `parent_graph` calls g1, g1 calls g2, ..."""
    paths: Set[Tuple[xl.Graph, ...]] = set()

    def walk(g: xl.Graph, prefix: Tuple[xl.Graph, ...]):
        for c in {id(_called(op)): _called(op) for op in g.ops if _called(op) is not None}.values():
            chain = prefix + (c,)
            if c is subgraph:
                paths.add(chain)
            elif c not in prefix:
                walk(c, chain)

    walk(parent_graph, ())
    return paths


def _add_call_input(op, tensor: xl.Tensor, modified: bool):
    op.inputs.append(tensor)
    if modified:
        op.attrs.setdefault("modified", set()).add(tensor)


def route_tensor_into_graph(tensor: xl.Tensor, graph: Optional[xl.Graph] = None,
                            modified: bool = False) -> xl.Tensor:
    """Tensor inside `graph` (default: the current graph) that carries the value of `tensor`, which lives in a graph
    that (transitively) calls `graph`. `modified=True` marks it as written by the sub-graph (by-reference)."""
    t = tensor
    graph = graph or xl.gcg()
    if not isinstance(t, xl.Tensor):
        raise TypeError(f"Not a tensor: {t}")
    if t.graph is graph:
        return t
    src = t.graph
    if t not in src._tensors:
        raise ValueError(f"{t} is not in the graph {src.name}")
    paths = called_graph_paths(src, graph)
    if not paths:
        raise ValueError(f"{t} is not in the graph {graph.name}. Additionally, the tensor is not in a known parent "
                         f"graph so cannot be moved into the graph ({src.name} does not, transitively, call it).")
    routed: Dict[xl.Graph, xl.Tensor] = {src: t}

    def already_passed(caller: xl.Graph, callee: xl.Graph) -> Optional[xl.Tensor]:
        """The input of `callee` that every call site in `caller` already feeds with the routed tensor, if any."""
        sites = [op for op in caller.ops if _called(op) is callee]
        index = None
        for op in sites:
            hits = [i for i, x in enumerate(op.inputs[:len(callee._inputs)]) if x is routed[caller]]
            if not hits or (index is not None and hits[0] != index):
                return None
            index = hits[0]
        return callee._inputs[index] if index is not None else None

    def input_of(caller: xl.Graph, callee: xl.Graph) -> xl.Tensor:
        if callee not in routed:
            existing = already_passed(caller, callee)
            if existing is not None:
                routed[callee] = existing
                if modified:
                    callee._by_ref.add(existing)
                    for op in caller.ops:
                        if _called(op) is callee:
                            op.attrs.setdefault("modified", set()).add(routed[caller])
            else:
                with callee:
                    routed[callee] = xl.graph_input(t.shape, t.dtype, t.name.split("/")[-1], by_ref=modified,
                                                    meta_shape=t.meta_shape)
        return routed[callee]

    wired: Set[int] = set()
    for chain in paths:
        caller = src
        for callee in chain:
            input_of(caller, callee)
            for op in caller.ops:
                if _called(op) is callee and op.uid not in wired:
                    # inputs are positional: a new graph input was appended last, so append the caller's tensor
                    if len(op.inputs) < len(callee._inputs):
                        _add_call_input(op, routed[caller], modified)
                    wired.add(op.uid)
            caller = callee
    return routed[graph]
