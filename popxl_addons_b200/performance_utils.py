"""Static FLOP estimate of a program: walks the graphs, counts matmul-class, elementwise and normalisation ops,
multiplies loop bodies by their trip count and the total by the replication factor.
Parity: popxl_addons/performance_utils.py:15-257."""
from typing import Dict, Optional, Tuple

from . import xl

__all__ = ["total_FLOPs", "evaluate_ir_FLOPs", "evaluate_FLOPs", "print_FLOPs", "format_flops_scientific"]

_ELEMENTWISE = {"add", "sub", "mul", "div", "pow", "maximum", "minimum", "fmod", "add_", "scaled_add",
                "scaled_add_"}


def _op_flops(op) -> int:
    od = op.opdef
    if od.flops is not None:
        return int(od.flops(op))
    if od.name in _ELEMENTWISE:
        return op.outputs[0].nelms if op.outputs else op.inputs[0].nelms
    if od.name in ("group_norm", "layer_norm", "rms_norm"):
        return 5 * op.inputs[0].nelms  # mean, var, subtract, scale, affine
    return 0


def _merge(dst: Dict[str, int], src: Dict[str, int], factor: int = 1):
    for k, v in src.items():
        dst[k] = dst.get(k, 0) + v * factor


def evaluate_FLOPs(graph: xl.Graph, _seen: Optional[Dict[xl.Graph, Dict[str, int]]] = None) -> Dict[str, int]:
    """FLOPs of one execution of `graph`, by op type (`"<callee>/<type>"` for called graphs)."""
    seen = _seen if _seen is not None else {}
    if graph in seen:
        return seen[graph]
    out: Dict[str, int] = {}
    for op in graph.ops:
        callee = op.attrs.get("graph")
        if isinstance(callee, xl.Graph) and op.opdef.name in ("call", "repeat"):
            trips = op.attrs.get("count", 1)
            sub = evaluate_FLOPs(callee, seen)
            _merge(out, {f"{callee.name}/{k}": v for k, v in sub.items()}, trips)
            continue
        f = _op_flops(op)
        if f:
            out[op.opdef.name] = out.get(op.opdef.name, 0) + f
    seen[graph] = out
    return out


def evaluate_ir_FLOPs(ir) -> Dict[str, int]:
    """FLOPs of one run of the main graph across all replicas."""
    if isinstance(ir, xl.Graph):
        ir = ir.ir
    per_replica = evaluate_FLOPs(ir.main_graph)
    return {k: v * ir.replication_factor for k, v in per_replica.items()}


def total_FLOPs(ir: xl.Ir) -> int:
    return sum(evaluate_ir_FLOPs(ir).values())


def format_flops_scientific(val: float, format: str = "nearest3") -> str:
    units = {"K": 1e3, "M": 1e6, "G": 1e9, "T": 1e12, "P": 1e15}
    if format == "nearest3":
        unit = ""
        for u, scale in units.items():
            if val >= scale:
                unit = u
        if not unit:
            return f"{val:.0f}"
        return f"{val / units[unit]:.2f}{unit}"
    if format not in units:
        raise ValueError(f"format must be one of {list(units)} or 'nearest3'. Not: {format}")
    return f"{val / units[format]:.2f}{format}"


def print_FLOPs(ir: xl.Ir, mode: str = "type", format: str = "nearest3") -> Dict[str, int]:
    """Print the estimate. `mode="type"` aggregates by op type, `"flat"` keeps the call path."""
    flat = evaluate_ir_FLOPs(ir)
    if mode == "type":
        table: Dict[str, int] = {}
        for k, v in flat.items():
            t = k.split("/")[-1]
            table[t] = table.get(t, 0) + v
    elif mode == "flat":
        table = flat
    else:
        raise ValueError(f"mode must be 'type' or 'flat'. Not: {mode}")
    for k, v in sorted(table.items(), key=lambda kv: -kv[1]):
        print(f"{k:50s} {format_flops_scientific(v, format)}")
    print(f"{'total':50s} {format_flops_scientific(sum(table.values()), format)}")
    return table
