"""Automatic differentiation of `GraphWithNamedArgs`, optionally with in-graph gradient accumulation.

Parity: popxl_addons/transforms/autodiff.py:26-228.
"""
from typing import Iterable, Mapping, Optional, Tuple

import numpy as np

from .. import xl
from ..graph import GraphWithNamedArgs
from ..named_tensors import NamedTensors
from ..variable_factory import NamedVariableFactories, add_variable_input
from ..xl import ops
from ..xl.autodiff import ExpectedConnection, ExpectedConnectionType, GradGraphInfo
from ..xl.autodiff import autodiff as _xl_autodiff

__all__ = ["autodiff", "autodiff_with_accumulation", "remap_grad_info"]


def autodiff(graph: GraphWithNamedArgs, grads_provided: Optional[Iterable[xl.Tensor]] = None,
             grads_required: Optional[Iterable[xl.Tensor]] = None,
             called_graphs_grad_info: Optional[Mapping[xl.Graph, GradGraphInfo]] = None) -> GraphWithNamedArgs:
    """Gradient graph of `graph` (default: gradients of all inputs given gradients of all outputs). Entries of
    `called_graphs_grad_info` supply gradient graphs for called sub-graphs (those with a hand-written `build_grad`
    must be listed); they take precedence over the ones recorded on `graph`."""
    called = dict(graph.called_graphs_grad_info)
    for k, v in (called_graphs_grad_info or {}).items():
        called[k.graph if isinstance(k, GraphWithNamedArgs) else k] = (
            v.grad_graph_info if isinstance(v, GraphWithNamedArgs) else v)
    info = _xl_autodiff(graph.graph, grads_provided, grads_required, called)
    return GraphWithNamedArgs.from_grad_graph(info)


def autodiff_with_accumulation(graph: GraphWithNamedArgs, tensors_to_accumulate_grads: Iterable[xl.Tensor],
                               grads_provided: Optional[Iterable[xl.Tensor]] = None,
                               grads_required: Optional[Iterable[xl.Tensor]] = None,
                               called_graphs_grad_info: Optional[Mapping[xl.Graph, GradGraphInfo]] = None,
                               replica_groupings=None,
                               accum_dtype: Optional[xl.dtype] = None, fuse_matmul: bool = True
                               ) -> Tuple[NamedVariableFactories, GraphWithNamedArgs]:
    """Gradient graph that, instead of returning the gradients of `tensors_to_accumulate_grads`, folds them into
    by-reference accumulators `accum.<name>` as a *running mean* over calls, counted by the scalar
    `mean_accum_counter` (zero it to start a new mean). Other `grads_required` remain graph outputs.
    Accumulators have the dtype of their tensor unless `accum_dtype` is given (e.g. fp32 sums for bf16 weights).
    With `fuse_matmul`, a gradient that is the direct result of a matmul and is used for nothing else is never written
    out: the matmul and the accumulation become one `matmul_accumulate_mean_` op (GEMM with accumulating epilogue).

    Returns the factories for the accumulators/counter and the gradient graph (its `args` name them)."""
    accumulate = list(tensors_to_accumulate_grads)
    required = list(grads_required) if grads_required is not None else []
    all_required = list(required) + [t for t in accumulate if t not in required]
    grad = autodiff(graph, grads_provided, all_required, called_graphs_grad_info)
    info = grad.grad_graph_info
    g = grad.graph
    name_of = {t: k for k, t in graph.args.to_dict().items()}
    rgs = replica_groupings.to_dict() if replica_groupings is not None else {}
    factories, named = {}, {}
    with g:
        counter, counter_f = add_variable_input("mean_accum_counter", lambda: np.zeros((), np.float32), xl.float32,
                                                by_ref=True)
        factories["mean_accum_counter"] = counter_f
        named["mean_accum_counter"] = counter
        drop = []
        for idx, ec in enumerate(info._expected_outputs):
            t = ec.fwd_tensor
            if t not in accumulate:
                continue
            key = name_of.get(t, t.name.replace("/", "_").replace(".", "_"))
            grad_t = g._outputs[idx]
            a_dt = accum_dtype or t.dtype
            np_dtype = a_dt.as_numpy() if a_dt._numpy is not None else np.float32
            shape = tuple(t.shape)
            accum, accum_f = add_variable_input(f"accum.{key}", lambda s=shape, d=np_dtype: np.zeros(s, d), a_dt,
                                                by_ref=True, replica_grouping=rgs.get(key))
            if t.meta_shape:
                accum.meta_shape = tuple(t.meta_shape)
            factories[f"accum.{key}"] = accum_f
            named[f"accum.{key}"] = accum
            if t not in required:
                drop.append(idx)
            if fuse_matmul and t not in required and _fuse_matmul_into_accumulator(g, grad_t, accum, counter):
                continue
            ops.var_updates.accumulate_mean_(accum, grad_t, counter)
        ops.add_(counter, xl.constant(1.0, xl.float32))
        for idx in sorted(drop, reverse=True):
            del g._outputs[idx]
            del info._expected_outputs[idx]
    grad.args = NamedTensors.from_dict(named)
    return NamedVariableFactories.from_dict(factories), grad


def _fuse_matmul_into_accumulator(g: xl.Graph, grad_t: xl.Tensor, accum: xl.Tensor, counter: xl.Tensor) -> bool:
    """If `grad_t` comes straight out of a 2-D matmul and has no other consumer, replace that matmul by a
    `matmul_accumulate_mean_` emitted now (current graph must be `g`). Returns whether the rewrite happened."""
    op = grad_t.producer
    if op is None or op.opdef.name != "matmul" or op.graph is not g:
        return False
    a, b = op.inputs
    if a.rank != 2 or b.rank != 2 or tuple(grad_t.shape) != tuple(accum.shape):
        return False
    if any(grad_t in other.inputs for other in g.ops) or g._outputs.count(grad_t) > 1:
        return False
    g.ops.remove(op)
    ops.var_updates.matmul_accumulate_mean_(accum, a, b, counter)
    return True


def remap_grad_info(grad_info: GradGraphInfo, forward_graph: xl.Graph, backward_graph: xl.Graph) -> GradGraphInfo:
    """Re-express `grad_info` against another (forward, backward) graph pair with the same input/output positions
    (used after a transform wrapped both graphs)."""
    old_fwd = grad_info.forward_graph

    def translate(t: xl.Tensor) -> xl.Tensor:
        if t in old_fwd._inputs:
            return forward_graph._inputs[old_fwd._inputs.index(t)]
        return forward_graph._outputs[old_fwd._outputs.index(t)]

    ins = [ExpectedConnection(translate(ec.fwd_tensor), ec.connection_type) for ec in grad_info._expected_inputs]
    outs = [ExpectedConnection(translate(ec.fwd_tensor), ec.connection_type) for ec in grad_info._expected_outputs]
    return GradGraphInfo(backward_graph, forward_graph, ins, outs)
