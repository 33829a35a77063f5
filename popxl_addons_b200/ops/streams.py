"""One-line host IO: create the stream and the load/store op together.

Parity: popxl_addons/ops/streams.py:13-23.
"""

import numpy as np

from .. import xl
from ..xl import ops

__all__ = ["host_load", "host_store"]


def host_load(t, dtype: xl.dtype, name: str):
    """Returns `(host array cast to dtype, h2d stream, loaded tensor)` for a host array `t`."""
    arr = np.asarray(t)
    if dtype._numpy is not None:
        arr = arr.astype(dtype.as_numpy())
    stream = xl.h2d_stream(arr.shape, dtype, name=f"{name}_stream")
    return arr, stream, ops.host_load(stream, name)


def host_store(t: xl.Tensor) -> xl.DeviceToHostStream:
    stream = xl.d2h_stream(t.shape, t.dtype, name=f"{t.name}_stream")
    ops.host_store(stream, t)
    return stream
