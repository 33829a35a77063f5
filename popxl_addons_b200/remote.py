"""Named remote buffers and graphs that load / store all of them at one run-time row index.

A remote buffer row per layer is how phased execution keeps the weights and optimizer state of all layers outside
the working set and streams one layer in at a time (device HBM slab by default, pinned host memory for offload).

Parity: popxl_addons/remote.py:20-222.
"""
from typing import List, Mapping, Optional, Tuple, Union

import numpy as np

from . import xl
from .dot_tree import DotTree
from .graph import GraphWithNamedArgs
from .named_tensors import NamedTensors
from .utils import null_context
from .variable_factory import NamedVariableFactories
from .xl import ops

__all__ = ["load_remote_graph", "store_remote_graph", "named_buffers", "named_variable_buffers",
           "create_remote_buffer"]


class NamedRemoteBuffers(DotTree):
    """DotTree of remote buffers."""


def create_remote_buffer(spec: xl.TensorSpec, entries: int = 1,
                         replica_group: Optional[xl.ReplicaGrouping] = None,
                         shard_over: Optional[int] = None, location: str = "device") -> xl.RemoteBuffer:
    """Buffer for tensors of `spec`. A spec that is already sharded (has a `meta_shape`) gets rows of the shard
    shape; otherwise `shard_over > 1` (default: the whole replica group) makes a replica-sharded buffer."""
    ir = xl.gcg().ir
    rg = replica_group or ir.replica_grouping()
    shard_over = shard_over or rg.group_size
    if spec.meta_shape:
        from .xl.core import _shard_grouping_within

        n_shards = int(np.prod(spec.meta_shape)) // max(int(np.prod(spec.shape)), 1)
        rb = xl.remote_buffer(spec.shape, spec.dtype, entries, location=location)
        rb.meta_shape = tuple(spec.meta_shape)
        rb.shard_group = _shard_grouping_within(rg, n_shards) if rg.group_size % n_shards == 0 else rg
        return rb
    if shard_over > 1:
        nelms = int(np.prod(spec.shape)) if spec.shape else 1
        if nelms % shard_over != 0:
            raise ValueError(f"Can't shard tensor with {nelms} elements over {shard_over} replicas")
        shape = (rg.num_groups, *spec.shape) if rg.num_groups > 1 else tuple(spec.shape)  # host shape: group axis first
        return xl.replica_sharded_buffer(shape, spec.dtype, rg, shard_over, entries, location=location)
    return xl.remote_buffer(spec.shape, spec.dtype, entries, location=location)


def named_buffers(tensors: NamedTensors, entries: int = 1, location: str = "device") -> NamedRemoteBuffers:
    """One (unsharded-row) buffer per tensor, rows shaped like the tensor; a sharded tensor keeps its meta-shape."""
    out = {}
    for name, t in tensors.to_dict().items():
        rb = xl.remote_buffer(t.shape, t.dtype, entries, location=location)
        if t.meta_shape:
            rb.meta_shape = tuple(t.meta_shape)
        out[name] = rb
    return NamedRemoteBuffers.from_dict(out)


def named_variable_buffers(factories: NamedVariableFactories, entries: int = 1,
                           shard_over_dict: Union[Mapping[str, int], int, bool] = True,
                           location: str = "device") -> NamedRemoteBuffers:
    """One buffer per variable factory. `shard_over_dict`: `True` shards every variable over its whole replica
    group, `False`/1 disables sharding, an int shards over that many replicas, a dict gives it per name."""
    out = {}
    for name, f in factories.to_dict().items():
        spec = xl.TensorSpec(f.shape, f.dtype, f.meta_shape)
        if isinstance(shard_over_dict, Mapping):
            shard_over = shard_over_dict.get(name)
        elif isinstance(shard_over_dict, bool):
            shard_over = f.replica_grouping.group_size if shard_over_dict else 1
        elif isinstance(shard_over_dict, int):
            if not 1 <= shard_over_dict <= f.replica_grouping.group_size:
                raise ValueError(f"Invalid shard_over_dict int value: {shard_over_dict}")
            shard_over = shard_over_dict
        else:
            raise ValueError("shard_over_dict must be a dictionary, an integer or a boolean")
        nelms = int(np.prod(spec.shape)) if spec.shape else 1
        if shard_over and shard_over > 1 and not spec.meta_shape and nelms % shard_over != 0:
            shard_over = 1  # tensors that do not divide evenly stay unsharded
        out[name] = create_remote_buffer(spec, entries, f.replica_grouping, shard_over, location)
    return NamedRemoteBuffers.from_dict(out)


def load_remote_graph(buffers: NamedRemoteBuffers, entries: int = 1,
                      use_io_tiles: bool = False) -> Tuple[GraphWithNamedArgs, List[str]]:
    """Graph with one input (the row index) that loads that row of every buffer; outputs are in the order of the
    returned names: `ts = NamedTensors.pack(names, g.call(i))`."""
    ir = xl.gcg().ir
    graph = ir.create_empty_graph("load_remote")
    names: List[str] = []
    ctx = xl.io_tiles() if use_io_tiles else null_context()
    with graph, xl.transforms.merge_exchange(), xl.in_sequence(False), ctx:
        index = xl.graph_input([], xl.int32, "load_index")
        for name, rb in zip(*buffers.unpack()):
            rb.entries = max(rb.entries, entries)
            names.append(name)
            xl.graph_output(ops.remote_load(rb, index, name))
    return GraphWithNamedArgs(graph), names


def load_remote(buffers: NamedRemoteBuffers, entry: Union[int, xl.Tensor] = 0,
                use_io_tiles: bool = False) -> NamedTensors:
    ctx = xl.io_tiles() if use_io_tiles else null_context()
    with xl.transforms.merge_exchange(), xl.in_sequence(False), ctx:
        return NamedTensors.from_dict({n: ops.remote_load(rb, entry, n) for n, rb in buffers.to_dict().items()})


def store_remote_graph(buffers: NamedRemoteBuffers, entries: int = 1,
                       use_io_tiles: bool = False) -> GraphWithNamedArgs:
    """Graph whose first input is the row index and which has one named input per buffer:
    `g.bind(tensors).call(i)` writes every tensor to row `i` of its buffer."""
    ir = xl.gcg().ir
    graph = ir.create_empty_graph("store_remote")
    args = {}
    ctx = xl.io_tiles() if use_io_tiles else null_context()
    with graph, xl.transforms.merge_exchange(), xl.in_sequence(False), ctx:
        index = xl.graph_input([], xl.int32, "store_index")
        for name, rb in zip(*buffers.unpack()):
            rb.entries = max(rb.entries, entries)
            t = xl.graph_input(rb.tensor_shape, rb.tensor_dtype, name, meta_shape=rb.meta_shape)
            ops.remote_store(rb, index, t)
            args[name] = t
    return GraphWithNamedArgs(graph, NamedTensors.from_dict(args))


def store_remote(buffers: NamedRemoteBuffers, tensors: NamedTensors, entry: Union[int, xl.Tensor] = 0,
                 use_io_tiles: bool = False) -> None:
    ctx = xl.io_tiles() if use_io_tiles else null_context()
    with xl.transforms.merge_exchange(), xl.in_sequence(False), ctx:
        for rb, t in buffers.to_mapping(tensors).items():
            ops.remote_store(rb, entry, t)
