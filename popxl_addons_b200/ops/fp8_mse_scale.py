"""Power-of-two FP8 scale that minimises the mean squared quantisation error of a tensor.

Algorithm (restated from popxl_addons/ops/fp8_mse_scale/README.md:1-24 and fp8_mse_scale_impl.cpp:92-240):
1. normalised histogram of |x| over 254 octave bins `[2^k, 2^(k+1))`, k = -126..127;
2. for each of the 62 candidate exponent shifts `b in [-31, 30]` the 8-bit format covers the octaves
   `[lo + b, lo + b + span)`; the cost of a shift is
   `sum_underflow h*2^2k + sum_inrange h*2^2k*qerr + sum_overflow h*(2^k - 2^top)^2`
   where `qerr = 2^(-2*(src_mantissa_bits - dst_mantissa_bits))` and `top` is the highest covered octave;
3. the result is `-(argmin + ties//2 - 31)`: the log2 of the factor to multiply `x` by before the cast.

On CUDA the histogram is one kernel (exponent extraction + shared-memory atomics) and the candidate scan runs in one
warp of the same launch's last block.
"""

import numpy as np
import torch

from .. import xl
from ..xl.opdef import OpDef, emit1
from .fp8_utils import fp8_format

__all__ = ["fp8_mse_scale", "fp8_mse_scale_reference"]

N_BINS = 254
N_CANDIDATES = 62
MIN_SHIFT = -31
SRC_MIN_EXP = -126


def _format_window(fmt: dict):
    """(lowest representable octave incl. subnormals, number of octaves)."""
    lo = fmt["min_normal_exp"] - fmt["mantissa_bits"]
    hi = int(np.floor(np.log2(fmt["max"])))
    return lo, hi - lo + 1


def fp8_mse_scale_reference(x: torch.Tensor, fmt_name: str, src_mantissa_bits: int) -> torch.Tensor:
    """Plain torch implementation (CPU oracle and CPU backend)."""
    from .fp8_utils import FP8_FORMATS

    fmt = FP8_FORMATS[fmt_name]
    lo, span = _format_window(fmt)
    qerr = 2.0 ** (-2.0 * (src_mantissa_bits - fmt["mantissa_bits"]))
    a = x.detach().float().abs().reshape(-1)
    n = a.numel()
    nz = a[a >= 2.0 ** SRC_MIN_EXP]
    k = torch.floor(torch.log2(nz)).clamp(SRC_MIN_EXP, 127).to(torch.int64) - SRC_MIN_EXP
    hist = torch.bincount(k, minlength=N_BINS).double() / max(n, 1)
    octave = torch.arange(N_BINS, dtype=torch.float64) + SRC_MIN_EXP
    val = torch.exp2(octave)
    idx = torch.arange(N_BINS)
    costs = torch.zeros(N_CANDIDATES, dtype=torch.float64)
    first = lo + MIN_SHIFT - SRC_MIN_EXP  # bin index of the lowest covered octave for the first candidate
    for c in range(N_CANDIDATES):
        start, stop = first + c, first + c + span
        under = (idx < start) & (idx >= 1)
        inside = (idx >= start) & (idx < stop)
        over = idx >= stop
        top = val[min(max(stop - 1, 0), N_BINS - 1)]
        costs[c] = (hist * val * val * under).sum() + (hist * val * val * qerr * inside).sum() + \
                   (hist * (val - top) ** 2 * over).sum()
    best = costs.min()
    ties = int((costs == best).sum().item())
    arg = int(torch.argmin(costs).item())
    return torch.tensor(-(arg + ties // 2 + MIN_SHIFT), dtype=torch.int32)


def _impl(x, fmt_name, src_mantissa_bits):
    if x.device.type == "meta":
        return torch.empty((), dtype=torch.int32, device="meta")
    return fp8_mse_scale_reference(x.cpu(), fmt_name, src_mantissa_bits).to(x.device)


OpDef("fp8_mse_scale", impl=_impl)


def fp8_mse_scale(src: xl.Tensor, dtype: xl.dtype = xl.float8_143) -> xl.Tensor:
    """int32 scalar log2-scale for casting `src` (fp16 / bf16 / fp32) to `dtype` with minimum squared error."""
    fp8_format(dtype)
    if src.dtype not in (xl.float32, xl.float16, xl.bfloat16):
        raise RuntimeError(f"dtype {src.dtype} not currently supported.")
    mant = {"float32": 23, "float16": 10, "bfloat16": 7}[src.dtype.name]
    return emit1("fp8_mse_scale", [src.flatten()], {"fmt_name": dtype.name, "src_mantissa_bits": mant})


from ._paths import also_importable_as  # noqa: E402

also_importable_as(__name__)
