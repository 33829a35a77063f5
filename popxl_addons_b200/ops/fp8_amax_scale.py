"""Power-of-two FP8 scale from the absolute maximum of a tensor.

Parity: popxl_addons/ops/fp8_amax_scale.py:13-45.
"""
from .. import xl
from ..xl import ops
from .fp8_utils import fp8_format

__all__ = ["fp8_amax_scale"]


def fp8_amax_scale(src: xl.Tensor, dtype: xl.dtype = xl.float8_143) -> xl.Tensor:
    """int32 scalar `clip(floor(log2(format_max / max|src|)), -31, 31)`: the largest power-of-two multiplier that
    keeps every element of `src` representable in `dtype`."""
    fmt = fp8_format(dtype)
    amax = ops.max(ops.abs(ops.cast(src, xl.float32)))
    ratio = ops.div(xl.constant(fmt["max"], xl.float32), amax)
    scale = ops.clip(ops.floor(ops.log2(ratio)), -31.0, 31.0)
    return ops.cast(scale, xl.int32)
