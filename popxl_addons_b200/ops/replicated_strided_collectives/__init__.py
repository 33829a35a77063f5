"""Collectives over replica groups given by `(stride, group_size)` or any explicit rank list.

On an NVSwitch box every group is served at full bandwidth, so these are the ordinary group collectives; the graph
variants reduce a whole `NamedTensors` in one graph.
Parity: popxl_addons/ops/replicated_strided_collectives/*.py.
"""
from typing import List, Optional, Tuple

from ... import xl
from ...xl import ops
from ...xl.ops import collectives as _c

__all__ = ["replicated_all_reduce_strided", "replicated_all_reduce_strided_identical_inputs",
           "replicated_all_reduce_strided_identical_grad_inputs", "replicated_all_reduce_strided_graph",
           "replicated_reduce_scatter_strided", "replicated_all_gather_strided"]


def _check_op(op):
    name = _c._norm_op(op)
    if name not in ("add", "mean"):
        raise ValueError(f"Strided collectives support `add` and `mean` only, got {op}")
    return name


def replicated_all_reduce_strided(t: xl.Tensor, op="add", group: Optional[xl.ReplicaGrouping] = None) -> xl.Tensor:
    """All-reduce; the gradient is an all-reduce as well."""
    return _c.replicated_all_reduce(t, _check_op(op), group)


def replicated_all_reduce_strided_identical_inputs(t: xl.Tensor, op="add",
                                                   group: Optional[xl.ReplicaGrouping] = None) -> xl.Tensor:
    """Inputs are identical on all replicas of the group: identity forward, all-reduce backward."""
    return _c.replicated_all_reduce(t, _check_op(op), group, identical_inputs=True)


def replicated_all_reduce_strided_identical_grad_inputs(t: xl.Tensor, op="add",
                                                        group: Optional[xl.ReplicaGrouping] = None) -> xl.Tensor:
    """Gradients are identical on all replicas of the group: all-reduce forward, identity backward."""
    return _c.replicated_all_reduce(t, _check_op(op), group, identical_grad_inputs=True)


def replicated_reduce_scatter_strided(t: xl.Tensor, op="add", group: Optional[xl.ReplicaGrouping] = None,
                                      configure_output_for_replicated_tensor_sharding: bool = False) -> xl.Tensor:
    return _c.replicated_reduce_scatter(t, _check_op(op), group, configure_output_for_replicated_tensor_sharding)


def replicated_all_gather_strided(t: xl.Tensor, group: Optional[xl.ReplicaGrouping] = None) -> xl.Tensor:
    """Gathers flat shards; the result takes the shard's `meta_shape` when it has one."""
    return _c.replicated_all_gather(t, group)


def replicated_all_reduce_strided_graph(tensors, op="add", group: Optional[xl.ReplicaGrouping] = None,
                                        use_io_tiles: bool = False):
    """Graph with one named input per tensor that all-reduces each:
    `reduced = NamedTensors.pack(names, g.bind(ts).call())`."""
    from ...graph import GraphWithNamedArgs
    from ...named_tensors import NamedTensors
    from ...utils import null_context

    ir = xl.gcg().ir
    graph = ir.create_empty_graph("all_reduce")
    names, args = [], {}
    ctx = xl.io_tiles() if use_io_tiles else null_context()
    with graph, xl.in_sequence(False), ctx:
        for name, t in zip(*tensors.unpack()):
            gi = xl.graph_input(t.shape, t.dtype, t.name.split("/")[-1], meta_shape=t.meta_shape)
            args[name] = gi
            names.append(name)
            xl.graph_output(replicated_all_reduce_strided(gi, op=op, group=group))
    return GraphWithNamedArgs(graph, NamedTensors.from_dict(args)), names


# the reference keeps each collective in a submodule named after it; load those now so that importing one later
# (`from ...replicated_strided_collectives.replicated_all_reduce_strided import ...`) does not rebind the function
# names of this package to the submodules
def _load_submodules():
    import importlib

    keep = {name: globals()[name] for name in __all__}
    for sub in ("replicated_all_gather_strided", "replicated_all_reduce_strided", "replicated_reduce_scatter_strided"):
        importlib.import_module(f"{__name__}.{sub}")
    globals().update(keep)


_load_submodules()
del _load_submodules
