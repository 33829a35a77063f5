"""Pipeline-parallel execution as a schedule transform.

Inside `with pipelined_execution(steps) as p:` every op is created under `p.stage(i)` (and a device slot,
`xl.ipu(j)`; several stages may share a slot, e.g. the forward and backward stage of the same layers). On exit the
recorded ops are partitioned into one graph per stage plus one graph holding *all* stage-boundary copies, and replaced
by the schedule

    ramp-up   : for i in 1..S-1:  run stages [0, i)   ; copy
    main      : repeat (steps - (S-1)) times:  run stages [0, S) ; copy      (copied tensors are loop-carried)
    ramp-down : for i in 1..S-1:  run stages [i, S)   ; copy   (no copy after the very last cycle)

so that in steady state all stages work concurrently on different micro-batches: stage `s` handles micro-batch
`c - s` in cycle `c`. With one process per GPU each rank runs the stages of its slot and the copy graph turns into
NCCL send/recv on a side stream. Activations needed by a later stage on the same slot are kept in circular stash
buffers (`stash_and_restore_tensor`) of depth `to_stage - from_stage + 1`.

Parity: popxl_addons/transforms/pipelining.py:26-508.
"""
from collections import defaultdict
from contextlib import contextmanager
from functools import partial
from typing import Dict, List, Optional

import numpy as np

from .. import xl
from ..module import Module
from ..xl import ops
from ..xl.autodiff import GradGraphInfo
from ..xl.ops.control import CallSiteInfo

__all__ = ["pipelined_execution", "Pipelining", "StageContext", "Stash", "Restore"]


def _placeholder(orig: xl.Tensor) -> xl.Tensor:
    """Zero tensor standing in for `orig` in cycles where its producer has not run yet (same device slot)."""
    v = ops.init(orig.shape, orig.dtype, orig.name.split("/")[-1] + "_dummy", "zero")
    v.device_index = orig.device_index
    v.producer.device_index = orig.device_index
    return v


def _input_like(t: xl.Tensor, by_ref: bool = False) -> xl.Tensor:
    """Graph input standing for `t`, on the same device slot."""
    g_in = xl.graph_input(t.shape, t.dtype, t.name.split("/")[-1], by_ref=by_ref, meta_shape=t.meta_shape)
    g_in.device_index = t.device_index
    return g_in


class _Part:
    """One piece of the pipeline (a stage's compute, or the copy graph) as a graph plus the original tensors its
    inputs and outputs stand for."""

    def __init__(self, graph: xl.Graph):
        self.graph = graph
        self.inputs: Dict[xl.Tensor, xl.Tensor] = {}   # original tensor -> graph input
        self.outputs: List[xl.Tensor] = []             # original tensors (now inside `graph`) exposed as outputs

    def call(self, cur: Dict[xl.Tensor, xl.Tensor]):
        inputs = {}
        for orig, g_in in self.inputs.items():
            v = cur.get(orig)
            if v is None:
                if orig.graph is xl.gcg():
                    v = orig
                else:
                    # produced by a part that has not run yet in this ramp-up cycle: placeholder
                    v = _placeholder(orig)
                    cur[orig] = v
            inputs[g_in] = v
        outs = ops.call(self.graph, inputs_dict=inputs)
        for orig, o in zip(self.outputs, outs):
            cur[orig] = o


class Pipelining:
    def __init__(self, graph: xl.Graph, steps: int):
        self.ir = graph.ir
        self.original_graph = graph
        self.steps = steps
        self.stages: Dict[int, _Part] = {}
        self.copies: Optional[_Part] = None
        self.num_stages = 0

    # -- partitioning -------------------------------------------------------------------------------------------
    def _move_ops(self, part: _Part, op_list: List, produced_elsewhere) -> None:
        g = part.graph
        produced = {t for op in op_list for t in op.outputs}
        const_clone: Dict[xl.Tensor, xl.Tensor] = {}
        for op in op_list:
            for i, t in enumerate(op.inputs):
                if t in produced:
                    continue
                if isinstance(t, xl.Constant):
                    if t not in const_clone:
                        with g:
                            const_clone[t] = xl.constant(t.data, t.dtype, t.name.split("/")[-1])
                    op.inputs[i] = const_clone[t]
                    continue
                if t not in part.inputs:
                    with g:
                        part.inputs[t] = _input_like(t, by_ref=True)
                op.inputs[i] = part.inputs[t]
            op.graph = g
            g.ops.append(op)
            for t in op.outputs:
                t.graph = g
                g._tensors.append(t)

    def construct_graphs(self, stage_ops: Dict[int, List]):
        stage_ids = sorted(stage_ops)
        if stage_ids != list(range(len(stage_ids))):
            raise ValueError(f"Pipeline stages must be numbered 0..S-1 without gaps, got {stage_ids}")
        self.num_stages = len(stage_ids)
        staged = {op.uid for lst in stage_ops.values() for op in lst}
        og = self.original_graph
        self._position = min(i for i, op in enumerate(og.ops) if op.uid in staged)
        og.ops = [op for op in og.ops if op.uid not in staged]
        compute = {s: [op for op in stage_ops[s] if op.opdef.name != "ipu_copy"] for s in stage_ids}
        copy_ops = [op for s in stage_ids for op in stage_ops[s] if op.opdef.name == "ipu_copy"]
        # consumers per tensor, to decide which produced tensors must leave their part
        part_of = {}
        for s in stage_ids:
            for op in compute[s]:
                part_of[op.uid] = s
        for op in copy_ops:
            part_of[op.uid] = "copy"
        consumers = defaultdict(set)
        for uid_list in list(compute.values()) + [copy_ops]:
            for op in uid_list:
                for t in op.inputs:
                    consumers[t].add(part_of[op.uid])
        # later ops of the original graph (after the pipeline block) may also read results
        for op in og.ops:
            for t in op.inputs:
                consumers[t].add("outside")
        for s in stage_ids:
            part = _Part(self.ir.create_empty_graph(f"pipeline_stage_{s}"))
            outs = [t for op in compute[s] for t in op.outputs if consumers[t] - {s}]
            self._move_ops(part, compute[s], None)
            with part.graph:
                for t in outs:
                    xl.graph_output(t)
            part.outputs = outs
            self.stages[s] = part
        cpart = _Part(self.ir.create_empty_graph("pipeline_copies"))
        outs = [t for op in copy_ops for t in op.outputs]
        self._move_ops(cpart, copy_ops, None)
        with cpart.graph:
            for t in outs:
                xl.graph_output(t)
        cpart.outputs = outs
        self.copies = cpart

    # -- schedule -----------------------------------------------------------------------------------------------
    def cycle(self, start: int, end: int, cur: Dict[xl.Tensor, xl.Tensor]):
        for s in range(start, end):
            self.stages[s].call(cur)
        if start == self.num_stages - 1:
            return  # nothing downstream is left to feed
        if self.copies.graph.ops:
            self.copies.call(cur)

    def build(self):
        S = self.num_stages
        parts = [self.stages[s] for s in range(S)] + [self.copies]
        cross = [t for p in parts for t in p.outputs]
        cross_set = set(cross)
        externals: List[xl.Tensor] = []
        for p in parts:
            for orig in p.inputs:
                if orig not in cross_set and orig not in externals:
                    externals.append(orig)
        og = self.original_graph
        tail = og.ops[self._position:]
        og.ops = og.ops[: self._position]
        with og, xl.in_sequence():
            cur: Dict[xl.Tensor, xl.Tensor] = {}
            for i in range(1, S):
                self.cycle(0, i, cur)
            # main loop graph: one full cycle with every cross-part tensor loop-carried
            loop = self.ir.create_empty_graph("pipeline_main_cycle")
            with loop:
                lcur: Dict[xl.Tensor, xl.Tensor] = {}
                for t in cross:
                    lcur[t] = _input_like(t)
                for e in externals:
                    lcur[e] = _input_like(e, by_ref=True)
                self.cycle(0, S, lcur)
                for t in cross:
                    v = lcur[t]
                    if v in loop._inputs:
                        v = ops.identity(v)
                    xl.graph_output(v)
            carried = []
            for t in cross:
                if t not in cur:
                    cur[t] = _placeholder(t)
                carried.append(cur[t])
            outs = ops.repeat(loop, self.steps - (S - 1), *carried, *externals)
            for t, o in zip(cross, outs):
                cur[t] = o
            for i in range(1, S):
                self.cycle(i, S, cur)
        # ops recorded after the pipeline block read the final values
        for op in tail:
            op.inputs = [cur.get(t, t) for t in op.inputs]
        og.ops.extend(tail)
        self.final_values = cur

    def apply(self, stage_ops: Dict[int, List]):
        if not stage_ops:
            return
        self.construct_graphs(stage_ops)
        if self.steps < 2 * self.num_stages:
            raise ValueError("Pipelining requires the steps at least 2x the number of stages in the pipeline. "
                             f"steps={self.steps} stages={self.num_stages}")
        self.build()


def get_op_pipeline_stage(op, op_dict: Dict[int, List]) -> Optional[int]:
    for stage, lst in op_dict.items():
        if any(o is op for o in lst):
            return stage
    return None


class StageContext:
    def __init__(self):
        self._stage: Optional[int] = None
        self.ops: Dict[int, List] = defaultdict(list)

    def hook(self, op):
        if self._stage is None:
            raise RuntimeError("Operation must be created in a stage context.")
        self.ops[self._stage].append(op)

    @contextmanager
    def stage(self, i: int):
        """Ops created inside belong to pipeline stage `i`."""
        prev, self._stage = self._stage, i
        try:
            yield
        finally:
            self._stage = prev

    def _is_external_input(self, t: xl.Tensor) -> bool:
        if t.producer is None:
            return True
        return get_op_pipeline_stage(t.producer, self.ops) is None

    def stash_and_restore_tensor(self, t: xl.Tensor, from_stage: Optional[int] = None) -> xl.Tensor:
        """Keep `t`, produced in `from_stage`, alive until the current stage processes the same micro-batch: a stash
        op in the producing stage writes it into a ring of `to - from + 1` slots, a restore op here reads the oldest."""
        if from_stage is None:
            if t.producer is None:
                raise RuntimeError("If the tensor to be stash does not have a producer `from_stage` must be "
                                   "specified to `stash_and_restore_tensor`")
            from_stage = get_op_pipeline_stage(t.producer, self.ops)
        to_stage = self._stage
        if to_stage is None:
            raise RuntimeError("`stash_and_restore_tensor` must be called in a stage context.")
        size = (to_stage - from_stage) + 1
        with self.stage(from_stage), xl.ipu(t.device_index):
            args, graph = Stash().create_graph(t, size)
            stash_vars = args.init()
            graph.bind(stash_vars).call(t)
        with self.stage(to_stage):
            args, graph = Restore().create_graph(stash_vars.stash)
            (restored,) = graph.bind(args.init()).call(stash_vars.stash)
        return restored

    def stash_and_restore_activations(self, call_info: CallSiteInfo,
                                      grad_info: GradGraphInfo) -> Dict[xl.Tensor, xl.Tensor]:
        """`grad_info.inputs_dict(call_info)` with every activation that was produced inside the pipeline (in an
        earlier stage than the current one) replaced by its stashed-and-restored value."""
        activations = grad_info.inputs_dict(call_info)
        from_stage = get_op_pipeline_stage(call_info._op, self.ops)
        if self._stage != from_stage:
            for g_in, act in list(activations.items()):
                if not self._is_external_input(act):
                    activations[g_in] = self.stash_and_restore_tensor(act, from_stage=from_stage)
        return activations


@contextmanager
def pipelined_execution(steps: int):
    """Ops created in the context run as a pipeline in which every stage executes `steps` times."""
    graph = xl.gcg()
    transform = Pipelining(graph, steps)
    stages = StageContext()
    handle = graph.register_op_created_hook(stages.hook)
    try:
        yield stages
    finally:
        graph.remove_op_created_hook(handle)
    transform.apply(stages.ops)


class Stash(Module):
    def build(self, t: xl.Tensor, stash_size: int):
        if stash_size <= 1:
            raise TypeError(f"Stash must be larger than 1. size={stash_size}, t={t}")
        counter = self.add_variable_input("counter", partial(np.zeros, (1,), np.uint32), xl.uint32, by_ref=True)
        shape = t.shape if t.shape else (1,)
        np_dt = t.dtype.as_numpy() if t.dtype._numpy is not None else np.float32
        stash = self.add_variable_input("stash", partial(np.zeros, (stash_size, *shape), np_dt), t.dtype, by_ref=True)
        ops.dynamic_update_(stash, counter, t.reshape((1, *shape)), axes=[0], sizes=[1])
        ops.increment_mod_(counter, 1, stash_size)


class Restore(Module):
    def build(self, stash: xl.TensorByRef):
        counter = self.add_variable_input("counter", partial(np.zeros, (1,), np.uint32), xl.uint32, by_ref=True)
        t = ops.dynamic_slice(stash, counter, axes=[0], sizes=[1])
        ops.increment_mod_(counter, 1, stash.shape[0])
        return t.reshape(t.shape[1:])
