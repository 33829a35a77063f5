"""`xl.fp8_utils` (popxl/fp8_utils.py): host-side fp8 conversions and the host version of the MSE scale search.

fp8 data on the host is a uint8 array of the encoded bytes (numpy has no 8-bit float types); `float8_143` is OCP
e4m3fn and `float8_152` is e5m2, the encodings the device kernels use."""
from typing import Tuple

import numpy as np
import torch

from . import dtypes as _dt

__all__ = ["host_pow2scale_cast_to_fp8", "host_pow2scale_cast_from_fp8", "host_fp8_mse_scale"]

_TORCH_FP8 = {"float8_143": torch.float8_e4m3fn, "float8_152": torch.float8_e5m2}


def _fp8(dtype) -> torch.dtype:
    if getattr(dtype, "name", None) not in _TORCH_FP8:
        raise ValueError(f"dtype must be float8_143 or float8_152, got {dtype}")
    return _TORCH_FP8[dtype.name]


def host_pow2scale_cast_to_fp8(src: np.ndarray, dtype=_dt.float8_143, log2_scale: int = 0,
                               nan_on_overflow: bool = True) -> np.ndarray:
    """`src * 2**log2_scale` encoded as fp8 bytes. Values beyond the format's range become NaN (e5m2: infinity) if
    `nan_on_overflow`, else they saturate to the largest finite value."""
    t8 = _fp8(dtype)
    if not -32 <= int(log2_scale) < 32:
        raise ValueError(f"log2_scale must be in the range [-32, 31], got {log2_scale}")
    x = torch.as_tensor(np.asarray(src, dtype=np.float32)) * float(2.0 ** int(log2_scale))
    fmax = torch.finfo(t8).max
    over = x.abs() > fmax
    if not nan_on_overflow:
        x = x.clamp(-fmax, fmax)
    out = x.to(t8)
    if nan_on_overflow and over.any() and t8 == torch.float8_e4m3fn:
        out = torch.where(over, torch.tensor(float("nan")).to(t8), out)
    return out.view(torch.uint8).numpy()


def host_pow2scale_cast_from_fp8(src: np.ndarray, dtype=_dt.float16, log2_scale: int = 0,
                                 src_dtype=_dt.float8_143) -> np.ndarray:
    """Decode fp8 bytes (format `src_dtype`) and multiply by `2**log2_scale`; result in `dtype` (float16 / float32)."""
    if not -32 <= int(log2_scale) < 32:
        raise ValueError(f"log2_scale must be in the range [-32, 31], got {log2_scale}")
    x = torch.as_tensor(np.asarray(src, dtype=np.uint8)).view(_fp8(src_dtype)).float() * float(2.0 ** int(log2_scale))
    return x.numpy().astype(dtype.as_numpy() if hasattr(dtype, "as_numpy") else dtype)


def host_fp8_mse_scale(src: np.ndarray, dtype=_dt.float8_143) -> Tuple[np.ndarray, int]:
    """`(src converted to fp8 with the chosen scale, log2 scale)`: the scale that minimises the squared quantisation
    error of `src` (histogram of binary exponents, scan over the candidate scales), as the device op computes it."""
    from ..ops.fp8_mse_scale import fp8_mse_scale_reference

    arr = np.asarray(src)
    mantissa = {np.dtype("float16"): 10, np.dtype("float32"): 23, np.dtype("float64"): 23}.get(arr.dtype, 23)
    _fp8(dtype)
    scale = int(fp8_mse_scale_reference(torch.as_tensor(arr.astype(np.float32)), dtype.name, mantissa))
    return host_pow2scale_cast_to_fp8(arr, dtype, scale, nan_on_overflow=False), scale
