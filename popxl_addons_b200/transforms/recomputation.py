"""Activation recomputation: trade a second forward pass for not keeping activations alive.

Parity: popxl_addons/transforms/recomputation.py:10-98.
"""
from typing import Dict, List, Optional, Sequence, Tuple

from .. import xl
from ..graph import GraphWithNamedArgs
from ..named_tensors import NamedTensors
from ..utils import suffix_graph_name
from ..xl import ops
from ..xl.autodiff import ExpectedConnection, ExpectedConnectionType, GradGraphInfo
from ..xl.core import Constant, Tensor
from ..xl.opdef import emit

__all__ = ["recompute_graph", "add_recompute_inputs", "prune_graph"]

# ops with their own executor whose only effect is their output (collectives: every rank prunes the same graph the same
# way, so the ranks keep issuing the same sequence of collectives)
_PURE_SPECIAL = {"all_reduce", "all_gather", "reduce_scatter", "matmul_all_reduce", "matmul2_all_reduce",
                 "matmuls_reduce_scatter", "all_gather_matmul", "replica_sharded_slice", "init"}


def _is_pure(op, _seen=None) -> bool:
    """True if the op may be dropped when nothing reads its outputs. A call is pure if the called graph takes nothing by
    reference and holds only pure ops."""
    d = op.opdef
    if d.inplace or d.name.endswith("_") or op.attrs.get("inplace"):
        return False
    if d.name == "call":
        callee = op.attrs["graph"]
        seen = _seen if _seen is not None else set()
        if callee in seen:  # recursion: be conservative
            return False
        seen.add(callee)
        return not callee._by_ref and not op.attrs.get("modified") and all(_is_pure(o, seen) for o in callee.ops)
    return d.special is None or d.name in _PURE_SPECIAL


def _holds_tensor(value) -> bool:
    if isinstance(value, Tensor):
        return True
    if isinstance(value, (list, tuple, set, frozenset)):
        return any(_holds_tensor(v) for v in value)
    if isinstance(value, dict):
        return any(_holds_tensor(v) for v in value.values())
    return False


def prune_graph(graph: xl.Graph, needed: Sequence[Tensor], name: Optional[str] = None
                ) -> Optional[Tuple[xl.Graph, Dict[Tensor, Tensor]]]:
    """Copy of `graph` that computes only `needed` (tensors of `graph`): same inputs in the same order, outputs =
    `needed` minus the graph inputs, and only the ops those outputs depend on, plus every op that has an effect of its
    own (in-place updates, host and remote transfers, calls) with what it depends on. Returns `(copy, {tensor of graph:
    tensor of the copy})` for inputs and outputs, or None if the graph holds something that cannot be copied (an op
    attribute that refers to a tensor, a variable used directly)."""
    live = {t for t in needed}
    keep = []
    for op in reversed(graph.ops):
        if any(o in live for o in op.outputs) or not _is_pure(op):
            keep.append(op)
            live.update(op.inputs)
    keep.reverse()
    inputs = set(graph._inputs)
    for op in keep:
        if any(_holds_tensor(v) for v in op.attrs.values()):
            return None
        for t in op.inputs:
            if t.producer is None and t not in inputs and not isinstance(t, Constant):
                return None
    for t in needed:
        if t.graph is not graph:
            raise ValueError(f"{t} is not a tensor of graph {graph.name}")
        if t.producer is None and t not in inputs and not isinstance(t, Constant):
            return None
    new = graph.ir.create_empty_graph(name or suffix_graph_name(graph.name, "pruned"))
    tmap: Dict[Tensor, Tensor] = {}
    with new:
        for t in graph._inputs:
            tmap[t] = xl.graph_input(t.shape, t.dtype, t.name.split("/")[-1], by_ref=graph.is_by_ref(t),
                                     meta_shape=t.meta_shape)

        def mapped(t: Tensor) -> Tensor:
            if t not in tmap:  # a constant of the original graph
                tmap[t] = Constant(new, t.data, t.name.split("/")[-1])
            return tmap[t]

        for op in keep:
            specs = [xl.TensorSpec(o.shape, o.dtype, o.meta_shape) for o in op.outputs]
            outs = emit(op.opdef.name, [mapped(t) for t in op.inputs], dict(op.attrs),
                        [o.name.split("/")[-1] for o in op.outputs], out_specs=specs)
            copy = outs[0].producer if outs else new.ops[-1]
            copy.device_index, copy.device_explicit = op.device_index, op.device_explicit
            copy.tile_set, copy.stage, copy.debug, copy.attrs_hint = op.tile_set, op.stage, op.debug, op.attrs_hint
            for o, c in zip(op.outputs, outs):
                c.device_index, c.tile_set = o.device_index, o.tile_set
                tmap[o] = c
        done = set()
        for t in needed:
            if t not in inputs and t not in done:
                xl.graph_output(mapped(t))
                done.add(t)
    new.hints.update(graph.hints)
    new.can_autodiff = False
    return new, {t: tmap[t] for t in list(graph._inputs) + [t for t in needed if t in tmap]}


def add_recompute_inputs(grad_info: GradGraphInfo):
    """Inputs of the recomputing graph (created in the current graph): one per `FwdGrad` expected input of the
    original gradient graph, then one per forward-graph input. Returns
    `(grad_inputs {orig grad input: new input}, fwd_inputs {fwd input: new input}, expected connections)`."""
    fwd = grad_info.forward_graph
    gg = grad_info.graph
    grad_inputs: Dict[xl.Tensor, xl.Tensor] = {}
    expected: List[ExpectedConnection] = []
    for gi, ec in zip(gg._inputs, grad_info._expected_inputs):
        if ec.connection_type == ExpectedConnectionType.FwdGrad:
            grad_inputs[gi] = xl.graph_input(gi.shape, gi.dtype, gi.name.split("/")[-1], meta_shape=gi.meta_shape)
            expected.append(ExpectedConnection(ec.fwd_tensor, ExpectedConnectionType.FwdGrad))
    fwd_inputs: Dict[xl.Tensor, xl.Tensor] = {}
    for t in fwd._inputs:
        fwd_inputs[t] = xl.graph_input(t.shape, t.dtype, t.name.split("/")[-1], by_ref=fwd.is_by_ref(t),
                                       meta_shape=t.meta_shape)
        expected.append(ExpectedConnection(t, ExpectedConnectionType.Fwd))
    return grad_inputs, fwd_inputs, expected


def recompute_graph(grad_graph: GraphWithNamedArgs, prune_forward: bool = False) -> GraphWithNamedArgs:
    """New gradient graph that needs only the *inputs* of the forward graph: it calls the forward graph again to
    regenerate the activations and then calls the original gradient graph. Extra inputs of the gradient graph
    (accumulators, counters) are carried over by reference under the same names.

    With `prune_forward` the second forward pass is a copy of the forward graph reduced to what the gradient graph
    reads (`prune_graph`): the ops that only lead to the forward result are left out. For a transformer block that is
    the output projections, their tensor-parallel all-reduce and the residual add; the gradients are bit-identical."""
    info = grad_graph.grad_graph_info
    fwd, gg = info.forward_graph, info.graph
    ir = gg.ir
    pruned = None
    if prune_forward:
        wanted = [ec.fwd_tensor for ec in info._expected_inputs if ec.connection_type == ExpectedConnectionType.Fwd]
        pruned = prune_graph(fwd, wanted, suffix_graph_name(fwd.name, "recomp_fwd"))
    new = ir.create_empty_graph(suffix_graph_name(gg.name, "recomp"))
    n_expected = len(info._expected_inputs)
    extra_map: Dict[xl.Tensor, xl.Tensor] = {}
    with new:
        grad_inputs, fwd_inputs, expected = add_recompute_inputs(info)
        for t in gg._inputs[n_expected:]:
            extra_map[t] = xl.graph_input(t.shape, t.dtype, t.name.split("/")[-1], by_ref=True,
                                          meta_shape=t.meta_shape)
        inputs_dict = dict(grad_inputs)
        if pruned is None:
            fwd_call = ops.call_with_info(fwd, inputs_dict=fwd_inputs)
            to_parent = fwd_call.graph_to_parent
        else:
            pruned_graph, tmap = pruned
            pruned_call = ops.call_with_info(pruned_graph, inputs_dict={tmap[t]: fwd_inputs[t] for t in fwd._inputs})
            to_parent = lambda t: pruned_call.graph_to_parent(tmap[t])  # noqa: E731
        for gi, ec in zip(gg._inputs, info._expected_inputs):
            if ec.connection_type == ExpectedConnectionType.Fwd:
                inputs_dict[gi] = to_parent(ec.fwd_tensor)
        inputs_dict.update(extra_map)
        outs = ops.call(gg, inputs_dict=inputs_dict)
        for o in outs:
            xl.graph_output(o)
    new_info = GradGraphInfo(new, fwd, expected, list(info._expected_outputs))
    args = NamedTensors.from_dict({k: extra_map[t] for k, t in grad_graph.args.to_dict().items() if t in extra_map})
    return GraphWithNamedArgs(new, args, new_info)
