"""Per-device GEMM workspace hints.

The reference sets the Poplar planner's "available memory proportion" of every matmul/conv on a given IPU. The GPU
analogue is a workspace / tile-configuration budget for the GEMM kernels of a device slot; it is recorded on the ops
(`op.attrs["available_memory_proportion"]`) and on the graph (`graph.hints`) for the kernel selector to read.

Parity: popxl_addons/transforms/available_memory_proportion.py:13-67.
"""
from typing import Dict

from .. import xl

__all__ = ["set_available_memory_proportion_by_ipu", "set_graph_available_memory_proportion_by_ipu"]

_GEMM_OPS = ("matmul", "conv", "linear_bias_act", "matmul_pow2scaled", "gather")


def _normalise(proportions) -> Dict[int, float]:
    if isinstance(proportions, (int, float)):
        return {-1: float(proportions)}
    if isinstance(proportions, dict):
        out = {int(k): float(v) for k, v in proportions.items()}
    else:
        out = {i: float(v) for i, v in enumerate(proportions)}
    for v in out.values():
        if not 0.0 < v <= 1.0:
            raise ValueError(f"available memory proportion must be in (0, 1], got {v}")
    return out


def set_graph_available_memory_proportion_by_ipu(graph: xl.Graph, proportions) -> None:
    table = _normalise(proportions)
    graph.hints["available_memory_proportion"] = table
    for op in graph.ops:
        if op.opdef.name in _GEMM_OPS:
            p = table.get(op.device_index, table.get(-1))
            if p is not None:
                op.attrs_hint = p
                graph.hints.setdefault("per_op", {})[op.uid] = p


def set_available_memory_proportion_by_ipu(ir: xl.Ir, proportions) -> None:
    for g in ir.graphs:
        set_graph_available_memory_proportion_by_ipu(g, proportions)
