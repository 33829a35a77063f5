"""Activation recomputation: trade a second forward pass for not keeping activations alive.

Parity: popxl_addons/transforms/recomputation.py:10-98.
"""
from typing import Dict, List

from .. import xl
from ..graph import GraphWithNamedArgs
from ..named_tensors import NamedTensors
from ..utils import suffix_graph_name
from ..xl import ops
from ..xl.autodiff import ExpectedConnection, ExpectedConnectionType, GradGraphInfo

__all__ = ["recompute_graph", "add_recompute_inputs"]


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


def recompute_graph(grad_graph: GraphWithNamedArgs) -> GraphWithNamedArgs:
    """New gradient graph that needs only the *inputs* of the forward graph: it calls the forward graph again to
    regenerate the activations and then calls the original gradient graph. Extra inputs of the gradient graph
    (accumulators, counters) are carried over by reference under the same names."""
    info = grad_graph.grad_graph_info
    fwd, gg = info.forward_graph, info.graph
    ir = gg.ir
    new = ir.create_empty_graph(suffix_graph_name(gg.name, "recomp"))
    n_expected = len(info._expected_inputs)
    extra_map: Dict[xl.Tensor, xl.Tensor] = {}
    with new:
        grad_inputs, fwd_inputs, expected = add_recompute_inputs(info)
        for t in gg._inputs[n_expected:]:
            extra_map[t] = xl.graph_input(t.shape, t.dtype, t.name.split("/")[-1], by_ref=True,
                                          meta_shape=t.meta_shape)
        fwd_call = ops.call_with_info(fwd, inputs_dict=fwd_inputs)
        inputs_dict = dict(grad_inputs)
        for gi, ec in zip(gg._inputs, info._expected_inputs):
            if ec.connection_type == ExpectedConnectionType.Fwd:
                inputs_dict[gi] = fwd_call.graph_to_parent(ec.fwd_tensor)
        inputs_dict.update(extra_map)
        outs = ops.call(gg, inputs_dict=inputs_dict)
        for o in outs:
            xl.graph_output(o)
    new_info = GradGraphInfo(new, fwd, expected, list(info._expected_outputs))
    args = NamedTensors.from_dict({k: extra_map[t] for k, t in grad_graph.args.to_dict().items() if t in extra_map})
    return GraphWithNamedArgs(new, args, new_info)
