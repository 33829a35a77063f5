"""Rotary position embedding on interleaved feature pairs (GPT-J convention) and its sin/cos tables.

Parity: popxl_addons/ops/rotary_pos_embed/rotary_pos_embed.py:19-109.
"""
from typing import Tuple

import numpy as np

from .. import xl
from ..xl import ops

__all__ = ["rotary_pos_embed", "trig_tables", "trig_table_constants"]


def trig_tables(seq_len: int, rotary_dim: int, base: int = 10000, dtype=np.float32) -> Tuple[np.ndarray, np.ndarray]:
    """`(sin, cos)` of shape `(seq_len, rotary_dim/2)` with `theta_i = base^(-2i/rotary_dim)`."""
    inv_freq = 1.0 / (base ** (np.arange(0, rotary_dim, 2, dtype=np.float64) / rotary_dim))
    ang = np.outer(np.arange(seq_len, dtype=np.float64), inv_freq)
    return np.sin(ang).astype(dtype), np.cos(ang).astype(dtype)


def trig_table_constants(seq_len: int, rotary_dim: int, base: int = 10000, dtype: xl.dtype = xl.float32):
    sin, cos = trig_tables(seq_len, rotary_dim, base)
    return xl.constant(sin[None], dtype, "rotary_sin"), xl.constant(cos[None], dtype, "rotary_cos")


def rotary_pos_embed(t: xl.Tensor, sin: xl.Tensor, cos: xl.Tensor, rotary_dim: int) -> xl.Tensor:
    """Rotate the first `rotary_dim` features of `t (batch, heads, seq, head_dim)` pairwise:
    `(x0, x1) -> (x0 cos - x1 sin, x1 cos + x0 sin)`; `sin`/`cos` are `(1|batch, seq, rotary_dim/2)`."""
    return ops.rotary_pos_embed(t, sin, cos, rotary_dim)


from ._paths import also_importable_as  # noqa: E402

also_importable_as(__name__)
