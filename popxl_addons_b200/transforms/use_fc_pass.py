"""Whether GEMM weights keep a pre-transposed copy for the backward passes.

For inference the extra copy is pure memory overhead, so it can be disabled for a whole Ir. Recorded as a hint on
every matmul-class op. Parity: popxl_addons/transforms/use_fc_pass.py:7-32.
"""
from .. import xl

__all__ = ["disable_fc_pass", "enable_fc_pass"]

_MATMUL_OPS = ("matmul", "linear_bias_act", "matmul_pow2scaled")


def _set(ir: xl.Ir, value: bool):
    ir.options["use_fc_pass"] = value
    for g in ir.graphs:
        for op in g.ops:
            if op.opdef.name in _MATMUL_OPS:
                g.hints.setdefault("fc_pass", {})[op.uid] = value


def disable_fc_pass(ir: xl.Ir) -> None:
    _set(ir, False)


def enable_fc_pass(ir: xl.Ir) -> None:
    _set(ir, True)
