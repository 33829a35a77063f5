"""Host streams and remote buffers.

A *remote buffer* is a named slab of `entries` rows, each row one tensor. The reference keeps such slabs in off-chip
streaming memory because IPU SRAM is small; on a GPU with 180 GB of HBM the slab normally lives in device memory
(`location="device"`) and can be placed in pinned host memory (`location="host"`) to offload optimizer state or
stashed activations. Rows of a replica-sharded buffer hold flat `1/shard_over` shards and remember the full
`meta_shape`.

Parity: popxl `h2d_stream/d2h_stream`, `remote_buffer`, `replica_sharded_buffer`, `remote_variable`,
`remote_replica_sharded_variable` as used by popxl_addons/remote.py:79-116 and variable_factory.py:134-154.
"""
import itertools
from typing import Iterable, Optional, Tuple

import numpy as np

from . import dtypes as _dt
from .core import ReplicaGrouping, TensorSpec, Variable, _host_array, _shard_grouping_within, gcg
from .dtypes import dtype

_stream_ids = itertools.count()


class _Stream:
    def __init__(self, shape, dt, name, prefix):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = _dt.dtype.as_dtype(dt)
        self.meta_shape = ()
        n = next(_stream_ids)
        self.name = name or f"{prefix}_{n}"
        self.tensor_id = f"{self.name}#{n}"

    @property
    def spec(self) -> TensorSpec:
        return TensorSpec(self.shape, self.dtype)

    def __repr__(self):
        return f"{type(self).__name__}[{self.name} {self.dtype} {self.shape}]"

    def __hash__(self):
        return hash(self.tensor_id)

    def __eq__(self, other):
        return self is other


class HostToDeviceStream(_Stream):
    pass


class DeviceToHostStream(_Stream):
    pass


def h2d_stream(shape: Iterable[int], dtype: dtype, name: Optional[str] = None) -> HostToDeviceStream:
    s = HostToDeviceStream(shape, dtype, name, "h2d")
    try:
        gcg().ir.streams.append(s)
    except RuntimeError:
        pass
    return s


def d2h_stream(shape: Iterable[int], dtype: dtype, name: Optional[str] = None) -> DeviceToHostStream:
    s = DeviceToHostStream(shape, dtype, name, "d2h")
    try:
        gcg().ir.streams.append(s)
    except RuntimeError:
        pass
    return s


class RemoteBuffer:
    _ids = itertools.count()

    def __init__(self, tensor_shape, tensor_dtype, entries: int = 1, meta_shape=None, shard_group=None,
                 location: str = "device"):
        self.tensor_shape: Tuple[int, ...] = tuple(int(s) for s in tensor_shape)
        self.tensor_dtype = _dt.dtype.as_dtype(tensor_dtype)
        self._entries = int(entries)
        self.meta_shape: Tuple[int, ...] = tuple(int(s) for s in meta_shape) if meta_shape else ()
        self.shard_group: Optional[ReplicaGrouping] = shard_group
        self.location = location
        self.remote_buffer_id = next(RemoteBuffer._ids)

    @property
    def entries(self) -> int:
        return self._entries

    @entries.setter
    def entries(self, n: int):
        self._entries = int(n)

    @property
    def replica_sharded(self) -> bool:
        return bool(self.meta_shape)

    def validate_tensor_matches_buffer(self, t, num_shards: int = 1):
        if tuple(t.shape) != self.tensor_shape and t.nelms != int(np.prod(self.tensor_shape)):
            raise ValueError(f"Tensor {t} does not match buffer row shape {self.tensor_shape}")
        if t.dtype != self.tensor_dtype:
            raise ValueError(f"Tensor {t} does not match buffer dtype {self.tensor_dtype}")

    def __repr__(self):
        return (f"RemoteBuffer(id={self.remote_buffer_id}, shape={self.tensor_shape}, dtype={self.tensor_dtype}, "
                f"entries={self._entries}, meta_shape={self.meta_shape})")

    def __hash__(self):
        return hash(("rb", self.remote_buffer_id))

    def __eq__(self, other):
        return self is other


def remote_buffer(tensor_shape: Iterable[int], tensor_dtype: dtype, entries: int = 1,
                  location: str = "device") -> RemoteBuffer:
    rb = RemoteBuffer(tensor_shape, tensor_dtype, entries, location=location)
    try:
        gcg().ir.remote_buffers.append(rb)
    except RuntimeError:
        pass
    return rb


def replica_sharded_buffer(full_tensor_shape: Iterable[int], tensor_dtype: dtype,
                           replica_group: Optional[ReplicaGrouping] = None, shard_over: Optional[int] = None,
                           entries: int = 1, location: str = "device", shard_grouping=None) -> RemoteBuffer:
    """Buffer whose rows are flat `nelms/shard_over` shards of tensors of `full_tensor_shape`. As in popxl, the shape
    is the host shape of the variable the buffer is for: when `replica_group` has more than one group it starts with
    the group axis, which is not part of a row."""
    ir = gcg().ir
    full = tuple(int(s) for s in full_tensor_shape)
    rg = replica_group or ir.replica_grouping()
    if rg.num_groups > 1:
        if not full or full[0] != rg.num_groups:
            raise ValueError(f"The shape of a buffer for a grouping with {rg.num_groups} groups must start with the "
                             f"group axis; got {full}")
        full = full[1:]
    if shard_grouping is None:
        shard_grouping = _shard_grouping_within(rg, shard_over or rg.group_size)
    n = shard_grouping.group_size
    nelms = int(np.prod(full)) if full else 1
    if nelms % n != 0:
        raise ValueError(f"Cannot shard {nelms} elements over {n} replicas")
    rb = RemoteBuffer((nelms // n,), tensor_dtype, entries, meta_shape=full, shard_group=shard_grouping,
                      location=location)
    ir.remote_buffers.append(rb)
    return rb


def remote_variable(data, remote_buffer: RemoteBuffer, offset: int = 0, dtype: Optional[dtype] = None,
                    name: Optional[str] = None, replica_grouping: Optional[ReplicaGrouping] = None,
                    retrieval_mode=None) -> Variable:
    """Variable whose storage is row `offset` of `remote_buffer`. It is read with `ops.remote_load`."""
    g = gcg()
    dt = _dt.dtype.as_dtype(dtype) if dtype is not None else remote_buffer.tensor_dtype
    host = data if isinstance(data, np.memmap) else _host_array(data, dt)
    rg = replica_grouping or g.ir.replica_grouping()
    shape = tuple(host.shape[1:]) if rg.num_groups > 1 else tuple(host.shape)
    if int(np.prod(shape)) != int(np.prod(remote_buffer.tensor_shape)):
        raise ValueError(f"Data of shape {shape} does not fit buffer rows of shape {remote_buffer.tensor_shape}")
    if offset >= remote_buffer.entries:
        raise ValueError(f"Offset {offset} is out of range for a buffer with {remote_buffer.entries} entries")
    v = Variable(g.ir.main_graph, shape, dt, name or "remote_variable", replica_grouping=rg,
                 remote_buffer=remote_buffer, entry=int(offset))
    g.ir.initial_values[v] = host
    if isinstance(host, np.memmap):
        v._memmap_arr = host
    return v


def remote_replica_sharded_variable(data, remote_buffer: RemoteBuffer, offset: int = 0,
                                    dtype: Optional[dtype] = None, name: Optional[str] = None,
                                    replica_grouping: Optional[ReplicaGrouping] = None,
                                    retrieval_mode=None) -> Variable:
    """Remote variable stored as one flat shard per replica of the buffer's shard group; host data is unsharded."""
    if not remote_buffer.meta_shape:
        raise ValueError("The remote buffer is not replica-sharded (no meta_shape)")
    g = gcg()
    dt = _dt.dtype.as_dtype(dtype) if dtype is not None else remote_buffer.tensor_dtype
    host = data if isinstance(data, np.memmap) else _host_array(data, dt)
    rg = replica_grouping or g.ir.replica_grouping()
    full = tuple(host.shape[1:]) if rg.num_groups > 1 else tuple(host.shape)
    if int(np.prod(full)) != int(np.prod(remote_buffer.meta_shape)):
        raise ValueError(f"Data of shape {full} does not match the buffer meta shape {remote_buffer.meta_shape}")
    v = Variable(g.ir.main_graph, remote_buffer.tensor_shape, dt, name or "remote_variable",
                 meta_shape=remote_buffer.meta_shape, replica_grouping=rg, remote_buffer=remote_buffer,
                 entry=int(offset), shard_group=remote_buffer.shard_group)
    g.ir.initial_values[v] = host
    if isinstance(host, np.memmap):
        v._memmap_arr = host
    return v
