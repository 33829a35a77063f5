"""Rotary position embedding on interleaved feature pairs (GPT-J convention) and its sin/cos tables.

Parity: popxl_addons/ops/rotary_pos_embed/rotary_pos_embed.py:19-109.
"""
from typing import Optional, Tuple

import numpy as np

from .. import xl
from ..xl import ops

__all__ = ["rotary_pos_embed", "trig_tables", "trig_table_constants"]


def trig_tables(seq_len: int, rotary_dim: int, base: int = 10000, np_dtype="float32",
                dtype=None) -> Tuple[np.ndarray, np.ndarray]:
    """`(sin, cos)` of shape `(seq_len, rotary_dim/2)`: angle `m * theta_i` for position `m`, with
    `theta_i = base^(-2i/rotary_dim)`. Computed in `np_dtype` throughout, which for float32 reproduces the tables of the
    Hugging Face GPT-J code to the last bit or two (`dtype` is an older spelling of `np_dtype`)."""
    np_dtype = np.dtype(dtype if dtype is not None else np_dtype)
    theta = np.power(np_dtype.type(base), -np.arange(0, rotary_dim, 2).astype(np_dtype) / np_dtype.type(rotary_dim))
    angle = np.outer(np.arange(seq_len).astype(np_dtype), theta)
    return np.sin(angle), np.cos(angle)


def trig_table_constants(seq_len: int, rotary_dim: int, base: int = 10000, dtype: xl.dtype = xl.float32):
    """`(sin, cos)` constants of shape `(seq_len, rotary_dim/2)`."""
    sin, cos = trig_tables(seq_len, rotary_dim, base)
    return xl.constant(sin, dtype, "rotary_sin"), xl.constant(cos, dtype, "rotary_cos")


def rotary_pos_embed(t: xl.Tensor, sin: xl.Tensor, cos: xl.Tensor, rotary_dim: Optional[int] = None) -> xl.Tensor:
    """Rotate the first `rotary_dim` (default: all) features of `t (batch, seq, heads, head_dim)` pairwise:
    `(x0, x1) -> (x0 cos - x1 sin, x1 cos + x0 sin)` with the angle of the token's position; `sin` / `cos` are
    `(seq, rotary_dim/2)` or `(1|batch, seq, rotary_dim/2)`. The sequence axis is axis 1, as in the reference's op
    (rotary_pos_embedx.cpp:49-70 broadcasts the tables over axes 2 and 4 of the pair view) and in the Hugging Face GPT-J
    code it is tested against; the kernels of this package work on `(batch, heads, seq, head_dim)`
    (`xl.ops.rotary_pos_embed`, what the models call), so this wrapper swaps the two axes around that op."""
    if t.rank != 4:
        raise ValueError(f"rotary_pos_embed expects a rank-4 (batch, seq, heads, head_dim) tensor, got {t.shape}")
    if not rotary_dim:
        rotary_dim = t.shape[-1]
    if sin.rank == 2:
        sin = ops.reshape(sin, (1, *sin.shape))
    if cos.rank == 2:
        cos = ops.reshape(cos, (1, *cos.shape))
    if sin.rank != 3 or cos.rank != 3:
        raise ValueError(f"sin / cos must have rank 2 or 3, got {sin.shape}, {cos.shape}")
    y = ops.rotary_pos_embed(ops.transpose(t, (0, 2, 1, 3)), sin, cos, rotary_dim)
    return ops.transpose(y, (0, 2, 1, 3))


from ._paths import also_importable_as  # noqa: E402

also_importable_as(__name__)
