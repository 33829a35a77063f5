"""4-bit group quantisation: compress on the host (numpy), decompress on the device.

Packed layout: `uint16 (rows, groups, group_size/4)`, four 4-bit codes per word with the *first* element in the most
significant nibble; per-group `scale` and `bias` of shape `(rows, groups, 1)`; value = `code * scale + bias`.
The decompress op exists standalone (API parity, tests); in `LinearGQ` it is fused into the GEMM so the bf16 weights
never exist in memory.
Parity: popxl_addons/ops/group_quantize_decompress/group_quantize_decompress.py:23-196.
"""
from typing import Tuple

import numpy as np
import torch

from .. import xl
from ..xl import ops
from ..xl.opdef import OpDef, emit1

__all__ = ["group_quantize_decompress", "group_quantize_decompress_numpy", "group_quantize_compress_numpy"]

_SHIFTS = (12, 8, 4, 0)


def _decompress_ref(packed, scale, bias):
    if packed.device.type == "meta":
        r, g, w = packed.shape
        return torch.empty((r, g * w * 4), dtype=scale.dtype, device="meta")
    p = packed.view(torch.int16).to(torch.int32) & 0xFFFF
    codes = torch.stack([(p >> s) & 0xF for s in _SHIFTS], dim=-1)  # (R, G, W, 4)
    r, g, w, _ = codes.shape
    vals = codes.reshape(r, g, w * 4).to(torch.float32) * scale.float() + bias.float()
    return vals.reshape(r, g * w * 4).to(scale.dtype)


OpDef("group_quantize_decompress", impl=_decompress_ref)


def group_quantize_decompress(t: xl.Tensor, group_scale: xl.Tensor, group_bias: xl.Tensor,
                              dim: int = -1) -> xl.Tensor:
    """`(rows, groups, group_size/4) uint16` -> `(rows, groups*group_size)` in the dtype of the scales. With
    `dim == 0` the groups run along the first axis of the original matrix, i.e. the result is transposed back."""
    if t.dtype != xl.uint16:
        raise ValueError(f"Compressed tensor must be uint16, got {t.dtype}")
    if t.rank != 3 or group_scale.rank != 3 or group_bias.rank != 3:
        raise ValueError("Expected rank-3 compressed tensor, scales and biases")
    if tuple(group_scale.shape) != (t.shape[0], t.shape[1], 1) or tuple(group_bias.shape) != tuple(group_scale.shape):
        raise ValueError(f"Scales/biases must have shape {(t.shape[0], t.shape[1], 1)}; "
                         f"got {group_scale.shape} and {group_bias.shape}")
    out = emit1("group_quantize_decompress", [t, group_scale, group_bias])
    if dim not in (-1, 1):
        out = ops.transpose(out)
    return out


def group_quantize_decompress_numpy(t: np.ndarray, group_scale: np.ndarray, group_bias: np.ndarray,
                                    dim: int = -1) -> np.ndarray:
    """`(*leading, n_groups, group_size / 4)` packed uint16 -> `(*leading, n_groups * group_size)` values
    `code * scale + bias`, computed in the dtype of the scales (for float16 scales: product and sum each rounded to
    float16, as the reference's helper does). The decompressed axis is last; `dim != -1` moves it to `dim`."""
    t = np.asarray(t).astype(np.uint16)
    codes = np.stack([(t >> s) & 0xF for s in _SHIFTS], axis=-1)
    *lead, g, w, _ = codes.shape
    dt = np.asarray(group_scale).dtype
    vals = codes.reshape(*lead, g, w * 4).astype(dt) * group_scale + group_bias
    out = vals.reshape(*lead, g * w * 4).astype(dt)
    if dim != -1:
        out = np.moveaxis(out, -1, dim)
    return out


def group_quantize_compress_numpy(t: np.ndarray, group_size: int = 64,
                                  dim: int = -1) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Quantise to 4 bits in groups of `group_size` along axis `dim` (moved last in the result). Per group:
    `bias = min`, `scale = (max - min) / 15` (both rounded to float16, as in the reference's helper),
    `code = round((x - bias) / scale)`. Returns `(packed uint16 (*other, n_groups, group_size / 4), scale, bias
    (*other, n_groups, 1) float16)`."""
    if group_size % 4:
        raise ValueError("group_size must be a multiple of 4")
    x = np.asarray(t)
    if not np.issubdtype(x.dtype, np.floating):
        x = x.astype(np.float32)
    if dim != -1:
        x = np.moveaxis(x, dim, -1)
    if not np.isfinite(x).all():
        raise ValueError("Cannot compress t which contains non-finite values")
    *lead, c = x.shape
    if c % group_size:
        raise ValueError(f"The quantised axis ({c}) must be divisible by group_size ({group_size})")
    g = x.reshape(*lead, c // group_size, group_size)
    # scale and bias are float16, whatever the input's dtype: that is what the decompression op consumes
    lo = g.min(axis=-1, keepdims=True).astype(np.float16)
    hi = g.max(axis=-1, keepdims=True).astype(np.float16)
    scale = (hi - lo) / np.float16(15)
    safe = np.where(scale == 0, np.ones_like(scale), scale)
    codes = np.clip(np.rint((g - lo) / safe), 0, 15).astype(np.uint16)
    codes = codes.reshape(*lead, c // group_size, group_size // 4, 4)
    packed = np.zeros(codes.shape[:-1], dtype=np.uint16)
    for i, s in enumerate(_SHIFTS):
        packed |= codes[..., i] << s
    return packed, scale, lo


from ._paths import also_importable_as  # noqa: E402

also_importable_as(__name__)
