"""Host-side (numpy) layout helpers for per-replica data.

Session inputs and outputs are laid out `[num_host_transfers, replication_factor, *shape]`; these functions build
and take apart such arrays for sharded and repeated tensors.
Parity: popxl_addons/array_munging.py:25-427 (same function names and semantics, independent implementation).
"""
from typing import Callable, List, Optional, Sequence, Tuple, Union

import numpy as np

__all__ = ["shard", "unshard_arrays", "unshard", "repeat", "repeat_axis", "split2D", "shard2D", "unshard2D",
           "repeat_shard", "tensor_parallel_input", "pad_axis", "squeeze_safe", "handle_negative_axis"]


def handle_negative_axis(x: np.ndarray, axis: int) -> int:
    """Non-negative equivalent of `axis` for array `x`."""
    if x.ndim == 0:
        raise IndexError("Array is 0-dimensional")
    if not -x.ndim <= axis < x.ndim:
        raise IndexError(f"Axis is out of range. Axis: {axis}. Array Rank: {x.ndim}")
    return axis % x.ndim


def shard(x: np.ndarray, n: int, axis: int) -> np.ndarray:
    """Cut `x` into `n` equal pieces along `axis` and stack the pieces on a new leading axis:
    `(.., L, ..) -> (n, .., L/n, ..)`."""
    axis = handle_negative_axis(x, axis)
    return np.stack(np.split(x, n, axis=axis), axis=0)


def unshard_arrays(xs: List[np.ndarray], axis: int) -> np.ndarray:
    """Arrays with a unit leading axis -> one array: concatenated along `axis` (which does not count the leading
    axis when non-negative) with the leading axis removed."""
    ranks = {a.ndim for a in xs}
    if len(ranks) > 1:
        raise ValueError(f"All arrays must be of the same rank. Ranks: {','.join(str(a.ndim) for a in xs)}")
    ax = axis + 1 if axis >= 0 else handle_negative_axis(xs[0], axis)
    return np.concatenate(xs, axis=ax).squeeze(0)


def unshard(x: np.ndarray, axis: int) -> np.ndarray:
    """Inverse of `shard`: `(n, .., L/n, ..) -> (.., L, ..)`."""
    return unshard_arrays(np.split(x, x.shape[0], axis=0), axis)


def repeat(x: np.ndarray, n: int, axis: int = 0) -> np.ndarray:
    """`n` copies of `x` along a *new* axis at position `axis`."""
    return np.repeat(np.expand_dims(x, axis), n, axis=axis)


def repeat_axis(x: np.ndarray, n: int, axis: int = 0) -> np.ndarray:
    """Tile `x` `n` times along the existing axis `axis`."""
    reps = [1] * x.ndim
    reps[axis] = n
    return np.tile(x, reps)


def split2D(x: np.ndarray, n_1: int, n_2: int, axis_1: int, axis_2: int) -> List[List[np.ndarray]]:
    """`n_1 x n_2` grid of blocks: outer split along `axis_1`, inner along `axis_2`."""
    return [np.split(row, n_2, axis_2) for row in np.split(x, n_1, axis_1)]


def shard2D(x: np.ndarray, n_1: int, n_2: int, axis_1: int, axis_2: int) -> np.ndarray:
    """Blocks of `split2D` stacked on a new leading axis, `axis_1` outermost: `(n_1*n_2, ...)`."""
    blocks = [b for row in split2D(x, n_1, n_2, axis_1, axis_2) for b in row]
    return np.stack(blocks, axis=0)


def unshard2D(x: np.ndarray, n_1: int, n_2: int, axis_1: int, axis_2: int) -> np.ndarray:
    """Inverse of `shard2D` (the axes do not count the leading block axis)."""
    assert x.shape[0] == n_1 * n_2
    blocks = np.split(x, x.shape[0], axis=0)
    rows = [unshard_arrays(blocks[i * n_2:(i + 1) * n_2], axis_2) for i in range(n_1)]
    return np.concatenate(rows, axis=axis_1)


def repeat_shard(x: np.ndarray, n_repeats: int, n_shards: int, shard_axis: int,
                 sharded_tensor: str = "contiguous") -> np.ndarray:
    """Shard into `n_shards`, then give every shard to `n_repeats` replicas. `contiguous`: the whole shard sequence
    repeats (`s0 s1 s0 s1`), i.e. shards are on consecutive replicas; `strided`: each shard repeats in place
    (`s0 s0 s1 s1`)."""
    pieces = shard(x, n_shards, shard_axis)
    if sharded_tensor == "contiguous":
        return repeat_axis(pieces, n_repeats, 0)
    if sharded_tensor == "strided":
        return np.repeat(pieces, n_repeats, axis=0)
    raise ValueError(f"sharded_tensor should be either 'contiguous' or 'strided'. Not: {sharded_tensor}")


def _check_tp(tp: int, rf: int):
    if tp > rf:
        raise ValueError(f"tensor parallel factor `tp` is not less than replication factor `rf`: {tp} > {rf}")
    if rf % tp:
        raise ValueError(f"tensor parallel factor `tp` does not equally divide replication factor `rf`: rf/tp={rf/tp}")


def tensor_parallel_input(input_data: np.ndarray, tp: int, rf: int,
                          repeat_fn: Optional[Callable[[np.ndarray, int], np.ndarray]] = None) -> np.ndarray:
    """`[samples, *shape]` -> `[num_host_transfers, rf, *shape]` where each run of `tp` consecutive replicas sees
    the same sample (`repeat_fn(copy, i)` may alter the copy for tensor-parallel rank `i`, e.g. subtract the shard's
    vocabulary offset). Unit transfer / replica axes are squeezed."""
    _check_tp(tp, rf)
    x = np.expand_dims(input_data, 1)
    copies = [repeat_fn(x.copy(), i) if repeat_fn else x for i in range(tp)]
    out = np.concatenate(copies, axis=1).reshape(-1, rf, *input_data.shape[1:])
    return squeeze_safe(out, [0, 1])


def tensor_parallel_output(output_data: np.ndarray, num_host_transfers: int, tp: int, rf: int,
                           data_shape: Tuple[int, ...], tp_identical: bool = True,
                           true_num_host_transfers: Optional[int] = None) -> np.ndarray:
    """Session output `[num_host_transfers, rf, *data_shape]` -> `[samples, *data_shape]` (first tensor-parallel rank
    only when `tp_identical`, else `[samples, tp, *data_shape]`). `true_num_host_transfers` drops unused slots."""
    _check_tp(tp, rf)
    out = output_data.reshape(num_host_transfers, rf // tp, tp, *data_shape)
    if true_num_host_transfers is not None:
        out = out[:true_num_host_transfers]
    out = out.reshape(-1, tp, *data_shape)
    return out[:, 0] if tp_identical else out


def pad_axis(x: np.ndarray, n: int, axis: int, value: Union[int, float] = 0) -> np.ndarray:
    """Extend `axis` to length `n` with `value`."""
    assert x.shape[axis] <= n
    widths = [(0, 0)] * x.ndim
    widths[axis] = (0, n - x.shape[axis])
    return np.pad(x, widths, constant_values=value)


def squeeze_safe(x: np.ndarray, axis: Optional[Union[int, Sequence[int]]] = None) -> np.ndarray:
    """`np.squeeze` that silently skips listed axes whose length is not 1."""
    if axis is None:
        return np.squeeze(x)
    axes = [axis] if isinstance(axis, int) else list(axis)
    for ax in sorted({handle_negative_axis(x, a) for a in axes}, reverse=True):
        if x.shape[ax] == 1:
            x = np.squeeze(x, axis=ax)
    return x
