"""`xl.utils`: host-side helpers under popxl's module path (popxl/utils.py)."""
from typing import Iterable, Optional

import numpy as np
import torch

from . import dtypes as _dt

__all__ = ["to_numpy", "table_to_string", "downcast_np_dtypes"]

# numpy types narrowed when host data becomes a tensor, unless `downcast=False`
downcast_np_dtypes = {np.dtype("int64"): np.dtype("int32"), np.dtype("uint64"): np.dtype("uint32"),
                      np.dtype("float64"): np.dtype("float32")}


def to_numpy(x, dtype: Optional["_dt.dtype"] = None, downcast: bool = True, copy: bool = True) -> np.ndarray:
    """Host data (numpy array, torch tensor, scalar or nested list) as a numpy array: converted to `dtype` if given,
    else 64-bit types are narrowed to 32 bits when `downcast`. bf16 / fp8 torch tensors come back as float32 (numpy
    has no such types). `copy=False` avoids the copy where the input already is the requested array."""
    if isinstance(x, torch.Tensor):
        arr = _dt.to_numpy(x)
    else:
        arr = np.asarray(x)
    if dtype is not None:
        if hasattr(dtype, "as_numpy"):
            try:
                want = dtype.as_numpy()
            except TypeError:  # bf16 / fp8: numpy cannot hold them; round through torch and keep float32
                return _dt.to_numpy(torch.as_tensor(arr.astype(np.float32)).to(dtype.as_torch()))
        else:
            want = np.dtype(dtype)
        if arr.dtype != want:
            return arr.astype(want)
    elif downcast and arr.dtype in downcast_np_dtypes:
        return arr.astype(downcast_np_dtypes[arr.dtype])
    return arr.copy() if copy else arr


def table_to_string(rows: Iterable[Iterable], delimiter: str = " | ") -> str:
    """Rows of cells as aligned text columns (first row = header, underlined)."""
    rows = [[str(c) for c in r] for r in rows]
    if not rows:
        return ""
    widths = [max(len(r[i]) if i < len(r) else 0 for r in rows) for i in range(max(len(r) for r in rows))]
    lines = [delimiter.join(c.ljust(w) for c, w in zip(r, widths)).rstrip() for r in rows]
    lines.insert(1, "-" * max(len(l) for l in lines))
    return "\n".join(lines) + "\n"
