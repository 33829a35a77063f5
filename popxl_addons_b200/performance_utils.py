"""Static FLOP estimate of a program: walks the graphs, counts matmul-class, elementwise and normalisation ops,
multiplies loop bodies by their trip count and the total by the replication factor.

The breakdown has the reference's shape: `{op type: {op id: flops, "<Call|Loop>_<id>(<graph>)": {...}}, "TOT": total}`
with popart's type names for the ops the reference counts (`MatMul`, `Add`, `Sub`, `Div`, `Mul`,
`GroupNormalization`); fused ops of this package (attention, linear + bias + activation, ...) appear under their own
names. Parity: popxl_addons/performance_utils.py:15-257."""
import re
from collections import defaultdict
from math import floor, log10
from typing import Dict, Union

from . import xl
from .xl.core import pb_op_type
from .xl.utils import table_to_string

__all__ = ["total_FLOPs", "evaluate_ir_FLOPs", "evaluate_FLOPs", "print_FLOPs", "format_flops_scientific",
           "matmul_flops", "elementwise_binary_flops", "group_norm_flops"]

_ELEMENTWISE = {"add", "sub", "mul", "div", "pow", "maximum", "minimum", "fmod", "add_", "scaled_add", "scaled_add_"}


def _unwrap(op):
    return getattr(op, "_op", op)  # popart-style view (`graph._pb_graph.getOps()`) or the op itself


def matmul_flops(op) -> int:
    """`2 * K * (elements of the result)`: 2m for a dot product, 2mn for matrix x vector, 2bmnp batched."""
    op = _unwrap(op)
    return int(2 * op.inputs[0].shape[-1] * op.outputs[0].nelms)


def elementwise_binary_flops(op) -> int:
    return int(_unwrap(op).outputs[0].nelms)


def group_norm_flops(op) -> int:
    return _group_norm_flops(_unwrap(op))


def _group_norm_flops(op) -> int:
    # mean, variance (E[x^2] - E[x]^2), whiten (subtract, multiply), scale, bias
    x, out = op.inputs[0], op.outputs[0]
    groups = int(op.attrs.get("num_groups", 1))
    n_stats = x.shape[0] * groups
    averaged = int(x.shape[-1] * x.shape[-2] / groups) if x.rank >= 2 else x.nelms
    return averaged + 2 * averaged + 2 * n_stats + 4 * out.nelms


def _op_flops(op) -> int:
    od = op.opdef
    if od.flops is not None:
        return int(od.flops(op))
    if od.name in _ELEMENTWISE:
        return op.outputs[0].nelms if op.outputs else op.inputs[0].nelms
    if od.name == "group_norm":
        return _group_norm_flops(op)
    if od.name in ("layer_norm", "rms_norm"):
        return 5 * op.inputs[0].nelms  # mean, var, subtract, scale, affine
    return 0


def _multiply(v, factor):
    if isinstance(v, dict):
        return {k: _multiply(x, factor) for k, x in v.items()}
    return v * factor


def _sum(v):
    if isinstance(v, dict):
        return sum(_sum(x) for x in v.values())
    return v


def _evaluate(graph: xl.Graph, visited: Dict) -> Dict:
    if graph in visited:
        return visited[graph]
    total = 0
    out = defaultdict(dict)
    for op in graph.ops:
        callee = op.attrs.get("graph")
        if isinstance(callee, xl.Graph) and op.opdef.name in ("call", "repeat"):
            sub = _evaluate(callee, visited)
            if op.opdef.name == "repeat":
                sub = _multiply(sub, int(op.attrs.get("count", 1)))
            total += sub["TOT"]
            key = f"{pb_op_type(op)}_{op.id}({re.sub(r'_subgraph\(\d+\)', '', str(callee.id))})"
            for k, v in sub.items():
                out[k].update({key: v})
            continue
        f = _op_flops(op)
        if f:
            total += f
            out[pb_op_type(op)].update({op.id: f})
    out.update({"TOT": total})
    visited[graph] = out
    return out


def evaluate_FLOPs(graph: xl.Graph) -> Dict[str, Union[int, Dict]]:
    """FLOPs of one execution of `graph`: nested breakdown by op type, then op id (call sites nest the breakdown of
    the called graph, loops multiplied by their trip count); key `"TOT"` holds the total."""
    return _evaluate(graph, {})


def evaluate_ir_FLOPs(ir) -> Dict[str, Union[int, Dict]]:
    """FLOPs of one run of the main graph across all replicas."""
    if isinstance(ir, xl.Graph):
        ir = ir.ir
    return _multiply(evaluate_FLOPs(ir.main_graph), ir.replication_factor)


def total_FLOPs(ir: xl.Ir) -> int:
    return evaluate_ir_FLOPs(ir)["TOT"]


def format_flops_scientific(val: float, format: str = "nearest3") -> str:
    """`9.072E+03`: three decimals and an exponent that is a multiple of three (`nearest3`: the multiple of three
    nearest to the value's exponent) or fixed by `format` in `K M G T`."""
    if format not in ("K", "M", "G", "T", "nearest3"):
        raise ValueError("unknown format specified")
    if format == "nearest3":
        power = floor(log10(abs(val))) if val > 0.0 else 0
        exponent = 3 * (power // 3 + int(power % 3 == 2))
    else:
        exponent = {"K": 3, "M": 6, "G": 9, "T": 12}[format]
    sign = "-" if exponent < 0 else "+"
    return f"{val * 10 ** (-exponent):.3f}E{sign}{abs(exponent):02d}"


def _flatten(d: Dict, out: Dict, prefix: str = ""):
    for k, v in d.items():
        key = f"{prefix}.{k}" if prefix else str(k)
        if isinstance(v, dict):
            _flatten(v, out, key)
        else:
            out[key] = v


def print_FLOPs(flops_breakdown, mode: str = "type", numerical_format: str = "nearest3") -> Dict[str, int]:
    """Print a breakdown (as returned by `evaluate_FLOPs` / `evaluate_ir_FLOPs`; an `Ir` is evaluated first).
    `mode="type"`: one row per op type with its share; `mode="flat"`: one row per op, call paths joined with dots.
    Rows are sorted by FLOPs, descending. Returns the printed table as a dict."""
    if isinstance(flops_breakdown, (xl.Ir, xl.Graph)):
        flops_breakdown = evaluate_ir_FLOPs(flops_breakdown)
    if mode == "type":
        table = {k: _sum(v) for k, v in flops_breakdown.items()}
        tot = table.get("TOT", 0) or 1
        rows = [["Op Type", "FLOPs", "%"]]
        for k, v in sorted(table.items(), key=lambda kv: kv[1], reverse=True):
            rows.append([k, format_flops_scientific(v, numerical_format), f"{100 * v / tot:.1f}"])
    elif mode == "flat":
        table = {}
        _flatten(flops_breakdown, table)
        rows = [["Op Type", "FLOPs", "Op Name"]]
        for k, v in sorted(table.items(), key=lambda kv: kv[1], reverse=True):
            rows.append([k.split(".")[0], format_flops_scientific(v, numerical_format), k])
        rows.append(["TOT", format_flops_scientific(table.get("TOT", 0), numerical_format), ""])
    else:
        raise ValueError("Unknown mode specified. Please use `type` or `flat`.")
    print(table_to_string(rows))
    return table
