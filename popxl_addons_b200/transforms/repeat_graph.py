"""Turn the body of a graph into a loop executed `n` times.

Parity: popxl_addons/transforms/repeat_graph.py:11-81. On a GPU the repeated body is the unit that gets captured in
a CUDA graph and replayed, which removes per-launch host overhead from small-kernel loops.
"""
from .. import xl
from ..xl import ops

__all__ = ["repeat_graph"]


def repeat_graph(graph: xl.Graph, repeat_count: int) -> xl.Graph:
    """In place: move every op of `graph` into a new sub-graph and replace them by one `repeat` of it. Variables and
    graph inputs that the ops touch are passed by reference, so state carried between iterations lives in them."""
    n = int(repeat_count)
    if n < 1:
        raise ValueError("repeat_count must be >= 1")
    ir = graph.ir
    body = ir.create_empty_graph(graph.name + "_repeat_body")
    moved = list(graph.ops)
    produced = {t for op in moved for t in op.outputs}
    external = []
    for op in moved:
        for t in op.inputs:
            if t not in produced and t not in external and not isinstance(t, xl.Constant):
                external.append(t)
    mapping = {}
    with body:
        for t in external:
            mapping[t] = xl.graph_input(t.shape, t.dtype, t.name.split("/")[-1], by_ref=True,
                                        meta_shape=t.meta_shape)
    for op in moved:
        op.graph = body
        for i, t in enumerate(op.inputs):
            if t in mapping:
                op.inputs[i] = mapping[t]
            elif isinstance(t, xl.Constant):
                t.graph = body
        for t in op.outputs:
            t.graph = body
    body.ops = moved
    body._tensors.extend(t for op in moved for t in op.outputs)
    body._tensors.extend(t for op in moved for t in op.inputs if isinstance(t, xl.Constant))
    graph.ops = []
    outputs = list(graph._outputs)
    graph._outputs = []
    with graph:
        ops.repeat(body, n, inputs_dict={mapping[t]: t for t in external})
    if outputs:
        raise ValueError("repeat_graph cannot be applied to a graph with outputs: results must be stored to "
                         "variables, streams or remote buffers inside the loop")
    return body
