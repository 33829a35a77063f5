"""Sub-graph ops: `call`, `repeat`, `conditional`, and the call-site info objects that map callee tensors to the
caller's tensors (needed to feed a gradient graph with the activations of one particular forward call).

Parity: popxl `ops.call/_with_info`, `ops.repeat/_with_info` as used by popxl_addons/graph.py:26-57 and
transforms/batch_serialisation.py:355-409.
"""
from typing import List, Mapping, Optional, Tuple

import numpy as np

from ..core import Graph, Tensor, constant, gcg
from ..opdef import OpDef, emit


class CallSiteInfo:
    """Describes one call site of a graph. Lookups are live: outputs appended to the callee later (autodiff
    stitching) are visible through an existing info object."""

    def __init__(self, op):
        self._op = op

    @property
    def called_graph(self) -> Graph:
        return self._op.attrs["graph"]

    @property
    def inputs(self) -> Tuple[Tensor, ...]:
        return tuple(self._op.inputs[: len(self.called_graph._inputs)])

    @property
    def outputs(self) -> Tuple[Tensor, ...]:
        return tuple(self._op.outputs)

    def parent_input(self, index: int) -> Tensor:
        return self._op.inputs[index]

    def parent_output(self, index: int) -> Tensor:
        return self._op.outputs[index]

    def graph_to_parent(self, graph_tensor: Tensor) -> Tensor:
        g = self.called_graph
        for i, t in enumerate(g._inputs):
            if t is graph_tensor:
                return self._op.inputs[i]
        for i, t in enumerate(g._outputs):
            if t is graph_tensor:
                _sync_call_outputs(self._op)
                return self._op.outputs[i]
        raise ValueError(f"Tensor {graph_tensor} is not an input or output of the called graph {g.name}")

    def parent_to_graph(self, parent_tensor: Tensor) -> Tensor:
        g = self.called_graph
        for i, t in enumerate(self._op.inputs[: len(g._inputs)]):
            if t is parent_tensor:
                return g._inputs[i]
        for i, t in enumerate(self._op.outputs):
            if t is parent_tensor:
                return g._outputs[i]
        raise ValueError(f"Tensor {parent_tensor} is not an input or output of the call site")

    def graph_to_parent_input_index(self, index: int) -> int:
        return index

    def graph_to_parent_output_index(self, index: int) -> int:
        return index

    def parent_to_graph_input_index(self, index: int) -> int:
        return index

    def parent_to_graph_output_index(self, index: int) -> int:
        return index

    def set_parent_input_modified(self, parent_tensor: Tensor, infer_modified_regions: bool = False):
        self._op.attrs.setdefault("modified", set()).add(parent_tensor)


RepeatSiteInfo = CallSiteInfo


def _sync_call_outputs(op):
    """If outputs were appended to the callee after this call op was recorded, give the op matching outputs."""
    g: Graph = op.attrs["graph"]
    if op.opdef.name != "call":
        return
    while len(op.outputs) < len(g._outputs):
        src = g._outputs[len(op.outputs)]
        # create in the op's graph without disturbing the build context
        from ..core import _STATE

        _STATE.graphs.append(op.graph)
        try:
            op.outputs.append(Tensor(op.graph, src.shape, src.dtype, src.id.split("/")[-1], src.meta_shape,
                                     producer=op))
        finally:
            _STATE.graphs.pop()


def _resolve_inputs(graph: Graph, inputs, inputs_dict) -> List[Tensor]:
    inputs_dict = dict(inputs_dict or {})
    for k in inputs_dict:
        if k not in graph._inputs:
            raise ValueError(f"{k} is not an input of the called graph {graph.name}")
    free = [t for t in graph._inputs if t not in inputs_dict]
    flat = []
    for a in inputs:
        if isinstance(a, (list, tuple)):
            flat.extend(a)
        else:
            flat.append(a)
    if len(flat) > len(free):
        raise ValueError(
            f"Too many inputs provided to graph {graph.name}: {len(flat)} positional for {len(free)} unbound "
            f"inputs. Unbound graph inputs: {[t.id for t in free]}")
    for g_in, a in zip(free, flat):
        inputs_dict[g_in] = a
    missing = [t for t in graph._inputs if t not in inputs_dict]
    if missing:
        raise ValueError(
            f"Not enough inputs provided to graph {graph.name}. Missing graph inputs: {[t.id for t in missing]}")
    resolved = []
    for g_in in graph._inputs:
        a = inputs_dict[g_in]
        if not isinstance(a, Tensor):
            a = constant(a, g_in.dtype)
        if tuple(a.shape) != tuple(g_in.shape) and not (a.nelms == g_in.nelms == 1):
            raise ValueError(f"Shape mismatch for graph input {g_in.id}: expected {g_in.shape}, got {a.shape}")
        if a.dtype != g_in.dtype:
            raise ValueError(f"Dtype mismatch for graph input {g_in.id}: expected {g_in.dtype}, got {a.dtype}")
        resolved.append(a)
    return resolved


def _infer_call(op):
    return [(t.shape, t.dtype, t.meta_shape) for t in op.attrs["graph"]._outputs]


def _special_call(ex, op, env):
    g: Graph = op.attrs["graph"]
    outs = ex.run_graph(g, [env[t] for t in op.inputs[: len(g._inputs)]])
    for t, v in zip(op.outputs, outs):
        env[t] = v


def _vjp_call(ctx, op, gs):
    return ctx.vjp_call(op, gs)


OpDef("call", infer=_infer_call, special=_special_call, vjp=_vjp_call)


def _place_outputs(outs, graph: Graph):
    """Device slot of a call's results: the slot the call was placed on explicitly (`with ipu(i)`), else wherever the
    called graph produces them (a graph may span slots, e.g. the copy graph of a pipeline)."""
    if outs and not outs[0].producer.device_explicit:
        for o, go in zip(outs, graph._outputs):
            o.device_index = go.device_index


def call_with_info(graph: Graph, *inputs, inputs_dict: Optional[Mapping[Tensor, Tensor]] = None,
                   check_inputs: bool = True) -> CallSiteInfo:
    """Call `graph`. Positional inputs fill, in order, the graph inputs that `inputs_dict` does not cover."""
    resolved = _resolve_inputs(graph, inputs, inputs_dict)
    outs = emit("call", resolved, {"graph": graph}, [t.id.split("/")[-1] for t in graph._outputs])
    _place_outputs(outs, graph)
    return CallSiteInfo(outs[0].producer if outs else gcg().ops[-1])


def call(graph: Graph, *inputs, inputs_dict: Optional[Mapping[Tensor, Tensor]] = None) -> Tuple[Tensor, ...]:
    return call_with_info(graph, *inputs, inputs_dict=inputs_dict).outputs


# ---- repeat --------------------------------------------------------------------------------------------------


def _special_repeat(ex, op, env):
    g: Graph = op.attrs["graph"]
    n_in = len(g._inputs)
    vals = [env[t] for t in op.inputs[:n_in]]
    ex.run_repeat(op, g, vals, env)


OpDef("repeat", infer=_infer_call, special=_special_repeat)


def repeat_with_info(graph: Graph, repeat_count: int, *inputs,
                     inputs_dict: Optional[Mapping[Tensor, Tensor]] = None,
                     check_inputs: bool = True, cuda_graph: bool = False) -> CallSiteInfo:
    """Run `graph` `repeat_count` times. Output `i` of one iteration feeds input `i` of the next (loop-carried);
    the remaining inputs keep their value. Returns the outputs of the last iteration.
    `cuda_graph=True` (body without outputs, state kept in by-reference inputs, no data-dependent host decisions)
    lets a CUDA session capture one iteration as a CUDA graph and replay it, removing per-kernel launch overhead."""
    if repeat_count < 0:
        raise ValueError("repeat_count must be >= 0")
    resolved = _resolve_inputs(graph, inputs, inputs_dict)
    if len(graph._outputs) > len(graph._inputs):
        raise ValueError("A repeated graph cannot have more outputs than inputs")
    outs = emit("repeat", resolved, {"graph": graph, "count": int(repeat_count), "cuda_graph": bool(cuda_graph)},
                [t.id.split("/")[-1] for t in graph._outputs])
    _place_outputs(outs, graph)
    return CallSiteInfo(outs[0].producer if outs else gcg().ops[-1])


def repeat(graph: Graph, repeat_count: int, *inputs, inputs_dict: Optional[Mapping[Tensor, Tensor]] = None,
           check_inputs: bool = True, cuda_graph: bool = False) -> Tuple[Tensor, ...]:
    return repeat_with_info(graph, repeat_count, *inputs, inputs_dict=inputs_dict, cuda_graph=cuda_graph).outputs


# ---- conditional ---------------------------------------------------------------------------------------------


def _special_cond(ex, op, env):
    cond_vals = env[op.inputs[0]]
    then_g, else_g = op.attrs["then_graph"], op.attrs["else_graph"]
    n_then = len(then_g._inputs)
    take_then = bool(cond_vals[0].reshape(-1)[0].item())
    if take_then:
        outs = ex.run_graph(then_g, [env[t] for t in op.inputs[1:1 + n_then]])
    else:
        outs = ex.run_graph(else_g, [env[t] for t in op.inputs[1 + n_then:]])
    for t, v in zip(op.outputs, outs):
        env[t] = v


OpDef("conditional", special=_special_cond,
      infer=lambda op: [(t.shape, t.dtype, t.meta_shape) for t in op.attrs["then_graph"]._outputs])


def conditional(cond: Tensor, then_branch: Graph, else_branch: Graph, then_inputs=(), else_inputs=(),
                then_inputs_dict=None, else_inputs_dict=None) -> Tuple[Tensor, ...]:
    """Run one of two graphs depending on a scalar boolean tensor (decided on the host at run time)."""
    ti = _resolve_inputs(then_branch, then_inputs, then_inputs_dict)
    ei = _resolve_inputs(else_branch, else_inputs, else_inputs_dict)
    return tuple(emit("conditional", [cond, *ti, *ei], {"then_graph": then_branch, "else_graph": else_branch}))
