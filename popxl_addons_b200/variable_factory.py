"""Variable factories: deferred constructors for the variables a graph takes as named inputs.

A `VariableFactory` knows the spec of a graph input and how to draw initial data for it, so one graph can be
instantiated several times (`args.init()` twice gives two independent sets of weights). Factories with
`shard_over > 1` describe replica-sharded tensors (flat `1/shard_over` shards with the full shape as `meta_shape`):
the ZeRO-style partitioning of parameters and optimizer state.

Parity: popxl_addons/variable_factory.py:29-332.
"""
import itertools
import logging
import os
from typing import Callable, Iterable, Iterator, Optional, Tuple, Union

import numpy as np

from . import xl
from .dot_tree import DotTree
from .named_replica_grouping import NamedReplicaGrouping
from .named_tensors import NamedTensors
from .xl.core import _shard_grouping_within

logger = logging.getLogger(__name__)

__all__ = ["VariableFactory", "NamedVariableFactories", "add_variable_input", "add_replica_sharded_variable_input"]


class _Peekable:
    """Iterator wrapper that can look at the next element without consuming it."""

    def __init__(self, it: Iterator):
        self._it = iter(it)
        self._head = []

    def peek(self):
        if not self._head:
            self._head.append(next(self._it))
        return self._head[0]

    def __next__(self):
        if self._head:
            return self._head.pop()
        return next(self._it)

    def __iter__(self):
        return self


def _repeat_call(fn: Callable):
    while True:
        yield fn()


def _barrier():
    """Host barrier between the processes of a distributed launch (no-op otherwise)."""
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()
    except Exception:  # pragma: no cover
        pass


def _process_rank() -> int:
    return int(os.environ.get("RANK", "0"))


_NPY_MAGIC = b"\x93NUMPY"


def open_variable_file(path: str, np_dtype, shape, mode: str = "r") -> np.memmap:
    """Memory-map the host file of a variable: a raw array (what `np.memmap` and the reference write) or a `.npy` file
    with a numpy header. Shape and dtype are checked against the variable (for raw files: the file size)."""
    np_dtype, shape = np.dtype(np_dtype), tuple(int(d) for d in shape)
    with open(path, "rb") as f:
        has_header = f.read(len(_NPY_MAGIC)) == _NPY_MAGIC
    if has_header:
        mm = np.lib.format.open_memmap(path, mode=mode)
        if tuple(mm.shape) != shape or mm.dtype != np_dtype:
            raise ValueError(f"Existing memmap {path} has shape {mm.shape} / dtype {mm.dtype}; "
                             f"expected {shape} / {np_dtype}")
        return mm
    nbytes = int(np.prod(shape, dtype=np.int64)) * np_dtype.itemsize
    if os.path.getsize(path) != nbytes:
        raise ValueError(f"Existing memmap {path} holds {os.path.getsize(path)} bytes; expected {nbytes} "
                         f"({shape} / {np_dtype})")
    return np.memmap(path, dtype=np_dtype, shape=shape, mode=mode)


class VariableFactory:
    def __init__(self, data_iter: Union[Callable[[], np.ndarray], Iterable[np.ndarray]],
                 dtype: Optional[xl.dtype] = None, name: Optional[str] = None, by_ref: bool = False,
                 replica_grouping: Optional[xl.ReplicaGrouping] = None, shard_over: Optional[int] = None):
        """`data_iter` is either a callable returning one array per call, or an iterable of arrays. A callable is
        invoked once immediately (to fail early and to learn the shape)."""
        if callable(data_iter):
            try:
                first = data_iter()
            except Exception as e:
                raise ValueError("Passed callable via `data_iter` throws error.") from e
            if not isinstance(first, (np.ndarray, np.generic, xl.LazyInit)) and not hasattr(first, "shape"):
                raise ValueError("`data_iter` must return an array. "
                                 f"Got {type(first)} from {getattr(data_iter, '__name__', data_iter)}")
            source = itertools.chain([first], _repeat_call(data_iter))
        elif isinstance(data_iter, Iterable) and not isinstance(data_iter, np.ndarray):
            source = iter(data_iter)
        else:
            raise ValueError("`data_iter` must be a callable or an iterable of arrays "
                             "(wrap a single array: `lambda: array`)")
        self.data_iter = _Peekable(source)
        self.name = name
        self.by_ref = by_ref
        ir = xl.gcg().ir
        self.replica_grouping = replica_grouping or ir.replica_grouping()
        example = self.data_iter.peek()
        if not isinstance(example, xl.LazyInit):
            example = np.asarray(example)
        self.dtype = xl.dtype.as_dtype(dtype) if dtype is not None else xl.dtype.as_dtype(
            np.float32 if example.dtype == np.float64 else example.dtype)
        full_shape = tuple(example.shape)
        self.shard_over = int(shard_over) if shard_over else 1
        self.replica_sharded = self.shard_over > 1
        if self.replica_sharded:
            nelms = int(np.prod(full_shape)) if full_shape else 1
            if nelms % self.shard_over != 0:
                raise ValueError(f"{nelms} elements cannot be sharded evenly over {self.shard_over} replicas")
            self.meta_shape: Optional[Tuple[int, ...]] = full_shape
            self.shape: Tuple[int, ...] = (nelms // self.shard_over,)
            self.shard_grouping = _shard_grouping_within(self.replica_grouping, self.shard_over)
        else:
            self.meta_shape = None
            self.shape = full_shape
            self.shard_grouping = None

    # -- graph side ---------------------------------------------------------------------------------------------
    def create_input(self, prefix: Optional[str] = None) -> xl.Tensor:
        """Graph input (in the current graph) that a variable made by this factory can be bound to."""
        name = self.name if prefix is None else (f"{prefix}.{self.name}" if self.name else prefix)
        return xl.graph_input(self.shape, self.dtype, name, by_ref=self.by_ref, meta_shape=self.meta_shape)

    # -- variable side ------------------------------------------------------------------------------------------
    def _host_shape(self):
        n = self.replica_grouping.num_groups
        full = self.meta_shape if self.replica_sharded else self.shape
        return (n, *full) if n > 1 else tuple(full)

    def next_data(self, empty: bool = False) -> np.ndarray:
        """Host data for the next variable: one draw per replica group, stacked on a leading axis when there is more
        than one group. `empty=True` skips the draws and returns uninitialised memory of the right shape."""
        n = self.replica_grouping.num_groups
        if empty:
            return np.empty(self._host_shape(), self.dtype.as_numpy() if self.dtype._numpy is not None else np.float32)
        first = next(self.data_iter)
        if isinstance(first, xl.LazyInit):
            return first.with_groups(n) if n > 1 else first
        if n > 1:
            return np.stack([np.asarray(first)] + [np.asarray(next(self.data_iter)) for _ in range(n - 1)])
        return np.asarray(first)

    def next_memmap(self, memmap_dir: str, name: str, empty: bool = False,
                    read_only_if_exists: bool = False) -> np.memmap:
        """Backing file `<memmap_dir>/<name>.npy` of the variable: opened if it exists, else created (by process 0)
        and filled with the next data. New files are raw arrays without a header, the layout the reference writes
        (`np.memmap`), so memmap directories and the memmap files inside checkpoints are interchangeable with it;
        files that carry a numpy header are read as well."""
        path = os.path.join(memmap_dir, name + ".npy")
        shape = self._host_shape()
        np_dtype = self.dtype.as_numpy()
        if os.path.exists(path):
            _barrier()
            return open_variable_file(path, np_dtype, shape, "r" if read_only_if_exists else "r+")
        if _process_rank() == 0:
            os.makedirs(memmap_dir, exist_ok=True)
            mm = np.memmap(path, dtype=np_dtype, shape=tuple(shape), mode="w+")
            if not empty:
                mm[...] = np.asarray(self.next_data()).astype(np_dtype).reshape(shape)
            mm.flush()
            _barrier()
        else:
            if not empty:
                self.next_data()  # keep the data stream aligned across processes
            _barrier()
            mm = open_variable_file(path, np_dtype, shape, "r+")
        return mm

    def _data_for(self, name, empty, memmap_dir, read_only_if_exists):
        if memmap_dir is not None:
            return self.next_memmap(memmap_dir, name, empty, read_only_if_exists)
        if empty:
            n = self.replica_grouping.num_groups
            full = self.meta_shape if self.replica_sharded else self.shape
            return np.zeros((n, *full) if n > 1 else tuple(full), dtype=self.dtype.as_numpy()
                            if self.dtype._numpy is not None else np.float32)
        return self.next_data()

    def create_tensor(self, name: Optional[str] = None, empty: bool = False, memmap_dir: Optional[str] = None,
                      read_only_if_exists: bool = False) -> xl.Variable:
        """New variable in the main graph, initialised with the next draw of `data_iter`."""
        name = name or self.name
        data = self._data_for(name, empty, memmap_dir, read_only_if_exists)
        with xl.gcg().ir.main_graph:
            if self.replica_sharded:
                v, _ = xl.replica_sharded_variable(data, self.dtype, name, replica_grouping=self.replica_grouping,
                                                   shard_grouping=self.shard_grouping)
                return v
            return xl.variable(data, self.dtype, name, replica_grouping=self.replica_grouping)

    def create_remote_tensor(self, buffer: xl.RemoteBuffer, entry: int, name: Optional[str] = None,
                             empty: bool = False, memmap_dir: Optional[str] = None,
                             read_only_if_exists: bool = False) -> xl.Variable:
        """New variable stored in row `entry` of `buffer` (replica-sharded when the buffer is)."""
        name = name or self.name
        data = self._data_for(name, empty, memmap_dir, read_only_if_exists)
        with xl.gcg().ir.main_graph:
            if buffer.meta_shape:
                return xl.remote_replica_sharded_variable(data, buffer, entry, self.dtype, name,
                                                          replica_grouping=self.replica_grouping)
            return xl.remote_variable(data, buffer, entry, self.dtype, name, replica_grouping=self.replica_grouping)


class NamedVariableFactories(DotTree):
    """DotTree of `VariableFactory`. `init*` turn it into `NamedTensors` of fresh variables."""

    def _sorted_items(self):
        # alphabetical order => the sequence of random draws does not depend on construction order
        return sorted(self.to_dict().items(), key=lambda kv: kv[0])

    def init(self, prefix: Optional[str] = None, empty: bool = False, memmap_dir: Optional[str] = None,
             read_only_if_exists: bool = False) -> NamedTensors:
        out = {}
        for key, f in self._sorted_items():
            name = f"{prefix}.{key}" if prefix else key
            out[key] = f.create_tensor(name, empty, memmap_dir, read_only_if_exists)
        return NamedTensors.from_dict(out)

    def init_remote(self, buffers, entry: int = 0, prefix: Optional[str] = None, empty: bool = False,
                    memmap_dir: Optional[str] = None, read_only_if_exists: bool = False) -> NamedTensors:
        """Create every variable inside its remote buffer (`buffers` has the same keys) at row `entry`."""
        buf = buffers.to_dict()
        out = {}
        for key, f in self._sorted_items():
            name = f"{prefix}.{key}" if prefix else key
            out[key] = f.create_remote_tensor(buf[key], entry, name, empty, memmap_dir, read_only_if_exists)
        return NamedTensors.from_dict(out)

    def _init_in_graph(self, kind: str, prefix) -> NamedTensors:
        from .xl import ops

        out = {}
        for key, f in self._sorted_items():
            name = f"{prefix}.{key}" if prefix else key
            out[key] = ops.init(f.shape, f.dtype, name, kind, meta_shape=f.meta_shape)
        return NamedTensors.from_dict(out)

    def init_zero(self, prefix: Optional[str] = None) -> NamedTensors:
        """Zero tensors created by ops in the *current* graph (not variables)."""
        return self._init_in_graph("zero", prefix)

    def init_undef(self, prefix: Optional[str] = None) -> NamedTensors:
        return self._init_in_graph("undef", prefix)

    @property
    def replica_groupings(self) -> NamedReplicaGrouping:
        return NamedReplicaGrouping.from_dict({k: f.replica_grouping for k, f in self.to_dict().items()})


def add_variable_input(name: str, data_iter, dtype: Optional[xl.dtype] = None, by_ref: bool = False,
                       replica_grouping: Optional[xl.ReplicaGrouping] = None
                       ) -> Tuple[xl.Tensor, VariableFactory]:
    """Graph input in the current graph plus the factory that makes variables for it."""
    f = VariableFactory(data_iter, dtype, name, by_ref, replica_grouping)
    return f.create_input(), f


def add_replica_sharded_variable_input(name: str, data_iter, dtype: Optional[xl.dtype] = None,
                                       by_ref: bool = False,
                                       replica_grouping: Optional[xl.ReplicaGrouping] = None,
                                       shard_over: Optional[int] = None) -> Tuple[xl.Tensor, VariableFactory]:
    """As `add_variable_input` for a tensor sharded over `shard_over` replicas of its group (default: all)."""
    rg = replica_grouping or xl.gcg().ir.replica_grouping()
    f = VariableFactory(data_iter, dtype, name, by_ref, rg, shard_over or rg.group_size)
    return f.create_input(), f
