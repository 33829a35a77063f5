"""Replicated tensor sharding (RTS): parameters, gradients and optimizer state stored as flat `1/n` shards across a
replica group, gathered just before use and reduce-scattered after the backward pass (ZeRO-style).

Parity: popxl_addons/rts.py:27-206.
"""
from typing import List, Optional, Tuple

import numpy as np

from . import xl
from .graph import GraphWithNamedArgs
from .named_replica_grouping import NamedReplicaGrouping
from .named_tensors import NamedTensors
from .ops.replicated_strided_collectives import (replicated_all_gather_strided, replicated_all_reduce_strided,
                                                 replicated_reduce_scatter_strided)
from .utils import null_context
from .xl import ops

__all__ = ["replica_sharded_spec", "gather_replica_sharded_tensor", "all_gather_replica_sharded_graph",
           "reduce_replica_sharded_tensor", "reduce_replica_sharded_graph"]


def replica_sharded_spec(t: xl.Tensor, shard_over: xl.ReplicaGrouping) -> xl.TensorSpec:
    """Spec `t` has once sharded over `shard_over`: unchanged if already sharded, if the group has one member or if
    the element count does not divide evenly."""
    if t.meta_shape:
        return t.spec
    n = shard_over.group_size
    if n == 1 or t.nelms % n != 0:
        return t.spec
    return xl.TensorSpec((t.nelms // n,), t.dtype, t.shape)


def gather_replica_sharded_tensor(t: xl.Tensor, use_io_tiles: bool = False,
                                  replica_group: Optional[xl.ReplicaGrouping] = None) -> xl.Tensor:
    """All-gather `t` over `replica_group` if it is a shard (has a `meta_shape`); otherwise pass it through."""
    rg = replica_group or xl.gcg().ir.replica_grouping()
    ctx = xl.io_tiles() if use_io_tiles else null_context()
    if t.meta_shape:
        with ctx:
            t = replicated_all_gather_strided(t, group=rg)
    if use_io_tiles:
        t = ops.io_tile_copy(t)
    return t


def all_gather_replica_sharded_graph(tensors: NamedTensors, use_io_tiles: bool = False,
                                     replica_groups: Optional[NamedReplicaGrouping] = None
                                     ) -> Tuple[GraphWithNamedArgs, List[str]]:
    """Graph with one named input per tensor that gathers every sharded one:
    `gathered = NamedTensors.pack(names, g.bind(shards).call())`."""
    ir = xl.gcg().ir
    graph = ir.create_empty_graph("all_gather")
    groups = replica_groups.to_dict() if replica_groups else {}
    names, args = [], {}
    ctx = xl.io_tiles() if use_io_tiles else null_context()
    with graph, xl.in_sequence(False), ctx:
        for name, t in zip(*tensors.unpack()):
            gi = xl.graph_input(t.shape, t.dtype, t.name.split("/")[-1], meta_shape=t.meta_shape)
            args[name] = gi
            names.append(name)
            xl.graph_output(gather_replica_sharded_tensor(gi, use_io_tiles, groups.get(name)))
    return GraphWithNamedArgs(graph, NamedTensors.from_dict(args)), names


def reduce_replica_sharded_tensor(t: xl.Tensor, op: str = "add",
                                  replica_group: Optional[xl.ReplicaGrouping] = None,
                                  shard_group: Optional[xl.ReplicaGrouping] = None) -> xl.Tensor:
    """Reduce `t` over `replica_group` and leave each replica with its shard within `shard_group` (default: the
    same group). Equal groups use one reduce-scatter; otherwise all-reduce then local slice. A tensor whose element
    count does not divide by the shard group is all-reduced and left whole."""
    rg = replica_group or xl.gcg().ir.replica_grouping()
    sg = shard_group or rg
    if sg.group_size > 1 and t.nelms % sg.group_size == 0:
        if rg == sg and rg.group_size > 1:
            return replicated_reduce_scatter_strided(t, op=op, group=rg,
                                                     configure_output_for_replicated_tensor_sharding=True)
        if rg.group_size > 1:
            t = replicated_all_reduce_strided(t, group=rg, op=op)
        return ops.collectives.replica_sharded_slice(t, group=sg)
    return replicated_all_reduce_strided(t, group=rg, op=op)


def reduce_replica_sharded_graph(tensors: NamedTensors, op: str = "add", use_io_tiles: bool = False,
                                 shard_groups: Optional[NamedReplicaGrouping] = None,
                                 replica_group: Optional[xl.ReplicaGrouping] = None
                                 ) -> Tuple[GraphWithNamedArgs, List[str]]:
    """Graph with one named input per tensor that reduces each (see `reduce_replica_sharded_tensor`):
    `reduced = NamedTensors.pack(names, g.bind(grads).call())`."""
    ir = xl.gcg().ir
    graph = ir.create_empty_graph("replica_reduce")
    groups = shard_groups.to_dict() if shard_groups else {}
    names, args = [], {}
    ctx = xl.io_tiles() if use_io_tiles else null_context()
    with graph, xl.in_sequence(False), ctx:
        for name, t in zip(*tensors.unpack()):
            gi = xl.graph_input(t.shape, t.dtype, t.name.split("/")[-1], meta_shape=t.meta_shape)
            args[name] = gi
            names.append(name)
            x = ops.io_tile_copy(gi) if use_io_tiles else gi
            xl.graph_output(reduce_replica_sharded_tensor(x, op, replica_group, groups.get(name, replica_group)))
    return GraphWithNamedArgs(graph, NamedTensors.from_dict(args)), names
