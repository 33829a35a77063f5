"""Batch serialisation: run a graph `steps` times over micro-batches inside one device-side loop, loading the inputs
of each step from host streams or remote buffers and storing selected tensors back.

Remote buffers used here are matrices of `rows x steps` entries: entry `row * steps + i` belongs to micro-batch `i` of
row `row` (a row per layer when the same graph serves many layers). The loop graph takes the row as its first input.

Three IO modes:
* `compute`        loads, compute and stores are issued on the compute stream, strictly in order;
* `io`             loads / stores are tagged for the IO (copy) stream;
* `io_overlapped`  the loop is software-pipelined: the inputs of step `i+1` are fetched while step `i` computes and the
                   results of step `i` drain while step `i+1` computes (needs `steps >= 2`).

Parity: popxl_addons/transforms/batch_serialisation.py:23-781.
"""
import logging
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

from .. import xl
from ..graph import GraphWithNamedArgs
from ..named_tensors import NamedTensors
from ..remote import create_remote_buffer
from ..rts import gather_replica_sharded_tensor
from ..utils import null_context, suffix_graph_name
from ..xl import ops
from ..xl.autodiff import ExpectedConnectionType
from .autodiff import remap_grad_info

__all__ = ["batch_serialise", "batch_serialise_fwd_and_grad", "batch_serial_buffer", "RemoteHandle",
           "BatchSerialResult"]

logger = logging.getLogger(__name__)


@dataclass
class RemoteHandle:
    """Where a tensor lives between steps: `buffer`, the row offset to add to the loop's row (an int, `None` for
    "always row 0", or a function of the row tensor), and the replica group it is sharded over (None: unsharded)."""

    buffer: xl.RemoteBuffer
    row_offset: Union[int, None, Callable[[xl.Tensor], xl.Tensor]] = 0
    shard_group: Optional[xl.ReplicaGrouping] = None


def _as_handle(h):
    """Accept the legacy tuple form `(buffer, row_offset[, shard_group])`."""
    if isinstance(h, (RemoteHandle, xl.HostToDeviceStream)):
        return h
    if isinstance(h, (tuple, list)) and len(h) >= 2 and isinstance(h[0], xl.RemoteBuffer) and (
            h[1] is None or isinstance(h[1], int) or callable(h[1])):
        return RemoteHandle(*h)
    raise TypeError(f"Incompatible handle: {h}")


@dataclass
class BatchSerialResult:
    """`graph`: the loop graph (first input: row index; named args: the original graph's named inputs that are passed
    through). `stored_buffers`: `{tensor of the original graph: RemoteHandle it was stored to / loaded from}`."""

    graph: GraphWithNamedArgs
    stored_buffers: Dict[xl.Tensor, RemoteHandle]
    _remap_dict: Dict[xl.Tensor, xl.Tensor]

    def remap_tensors(self, ts: NamedTensors) -> NamedTensors:
        """Translate tensors of the original graph into the matching inputs of the loop graph."""
        return ts.remap(self._remap_dict)


def batch_serial_buffer(t: Union[xl.Tensor, xl.TensorSpec], steps: int = 1, rows: int = 1,
                        shard_group: Optional[xl.ReplicaGrouping] = None) -> xl.RemoteBuffer:
    """Buffer with `steps * rows` entries for tensors like `t`, sharded over `shard_group` if given."""
    spec = t.spec if isinstance(t, xl.Tensor) else t
    shard_over = shard_group.group_size if shard_group else 1
    return create_remote_buffer(spec, entries=steps * rows, replica_group=shard_group, shard_over=shard_over)


# ---- index arithmetic -----------------------------------------------------------------------------------------


def _entry_index(index: xl.Tensor, handle: RemoteHandle, steps: int, rows: int) -> xl.Tensor:
    """Buffer entry for the running index `row*steps + i`, and grow the buffer to fit."""
    off = handle.row_offset
    if off is None:
        entry, size = ops.remainder(index, xl.constant(steps, xl.int32)), steps
    elif callable(off):
        steps_t = xl.constant(steps, xl.int32)
        i = ops.remainder(index, steps_t)
        row = ops.div(index, steps_t)
        entry, size = ops.add(ops.mul(off(row), steps_t), i), steps * rows
    elif off != 0:
        entry, size = ops.add(index, xl.constant(off * steps, xl.int32)), steps * (off + rows)
    else:
        entry, size = index, steps * rows
    handle.buffer.entries = max(handle.buffer.entries, size)
    return entry


def _load(index, tensors, handles, steps, rows, tiles) -> List[xl.Tensor]:
    out = []
    with tiles(), xl.transforms.merge_exchange(), xl.in_sequence(False):
        for t in tensors:
            h = handles[t]
            if isinstance(h, xl.HostToDeviceStream):
                out.append(ops.host_load(h, t.name.split("/")[-1]))
            else:
                out.append(ops.remote_load(h.buffer, _entry_index(index, h, steps, rows), t.name.split("/")[-1]))
    # shards are gathered right after loading
    gathered = []
    with tiles():
        for t, v in zip(tensors, out):
            h = handles[t]
            if isinstance(h, RemoteHandle) and h.shard_group is not None and h.shard_group.group_size > 1:
                v = gather_replica_sharded_tensor(v, use_io_tiles=False, replica_group=h.shard_group)
                if tuple(v.shape) != tuple(t.shape):
                    v = ops.reshape(v, t.shape)
            gathered.append(v)
    return gathered


def _store(index, tensors, values, streams, buffers, steps, rows, tiles):
    with tiles():
        sliced = []
        for t, v in zip(tensors, values):
            h = buffers.get(t)
            if h is not None and h.shard_group is not None and h.shard_group.group_size > 1:
                v_b = ops.collectives.replica_sharded_slice(v, group=h.shard_group)
            else:
                v_b = v
            sliced.append(v_b)
    with tiles(), xl.transforms.merge_exchange(), xl.in_sequence(False):
        for t, v, v_b in zip(tensors, values, sliced):
            if t in streams:
                ops.host_store(streams[t], v)
            if t in buffers:
                h = buffers[t]
                ops.remote_store(h.buffer, _entry_index(index, h, steps, rows), v_b)


# ---- the transform --------------------------------------------------------------------------------------------


def _classify(graph: GraphWithNamedArgs, load_handles, store_streams, store_buffers, seed_input):
    g = graph.graph
    loaded = [t for t in g.inputs if t in load_handles]

    def is_stored(t):
        from_buffer = t in load_handles and not isinstance(load_handles[t], xl.HostToDeviceStream)
        return not from_buffer and (t in store_streams or t in store_buffers)

    stored = [t for t in list(g.inputs) + list(g.outputs) if is_stored(t)]
    passed = [t for t in g.inputs if t is not seed_input and t not in load_handles]
    return loaded, stored, passed


def _build(graph: GraphWithNamedArgs, steps, load_handles, store_streams, store_buffers, seed_input, rows,
           io_mode) -> BatchSerialResult:
    if rows < 1:
        raise ValueError("rows must be >0")
    ir = graph.graph.ir
    use_io = io_mode in ("io", "io_overlapped")
    overlapped = io_mode == "io_overlapped"
    tiles = xl.io_tiles if use_io else null_context
    loaded_ts, stored_ts, passed_ts = _classify(graph, load_handles, store_streams, store_buffers, seed_input)
    g = graph.graph

    def io_copy(ts):
        return [ops.io_tile_copy(t) for t in ts] if use_io else list(ts)

    def compute_and_store(index, seed, loaded, passed):
        inputs = {}
        if seed_input is not None:
            inputs[seed_input] = seed
        inputs.update(zip(loaded_ts, io_copy(loaded)))
        inputs.update(zip(passed_ts, passed))
        info = graph.call_with_info(args=inputs)
        results = io_copy([info.graph_to_parent(t) for t in stored_ts])
        _store(index, stored_ts, results, store_streams, store_buffers, steps, rows, tiles)

    def micro_plain(index: xl.Tensor, seed: xl.Tensor, passed: List[xl.TensorByRef]):
        seed, next_seed = ops.split_random_seed(seed)
        loaded = _load(index, loaded_ts, load_handles, steps, rows, tiles)
        compute_and_store(index, seed, loaded, passed)
        with tiles():
            index = ops.add(index, xl.constant(1, xl.int32))
        return (index, next_seed)

    def micro_overlapped(index: xl.Tensor, seed: xl.Tensor, current: List[xl.Tensor], passed: List[xl.TensorByRef]):
        # prefetch step i+1 (IO stream), compute step i, drain step i (IO stream)
        seed, next_seed = ops.split_random_seed(seed)
        with tiles():
            nxt_index = ops.add(index, xl.constant(1, xl.int32))
        nxt = _load(nxt_index, loaded_ts, load_handles, steps, rows, tiles)
        compute_and_store(index, seed, current, passed)
        return (nxt_index, next_seed, *nxt)

    loop = ir.create_empty_graph(suffix_graph_name(g.name, "repeat_graph"))
    with loop, xl.in_sequence():
        row = xl.graph_input([], xl.int32, "batch_serial_loop_index")
        with tiles():
            index = ops.mul(ops.io_tile_copy(row) if use_io else row, xl.constant(steps, xl.int32))
        if seed_input is not None:
            seed = xl.graph_input(seed_input.shape, seed_input.dtype, "batch_serial_random_seed")
        else:
            seed = xl.constant((0, 0), xl.uint32, "dummy_random_seed")
        passed = [xl.graph_input(t.shape, t.dtype, t.name.split("/")[-1], g.is_by_ref(t), t.meta_shape)
                  for t in passed_ts]
        if not overlapped:
            micro = ir.create_graph(micro_plain, index, seed, passed)
            ops.repeat(micro, steps, index, seed, *passed)
        else:
            first = _load(index, loaded_ts, load_handles, steps, rows, tiles)
            micro = ir.create_graph(micro_overlapped, index, seed, first, passed)
            outs = ops.repeat(micro, steps - 1, index, seed, *first, *passed)
            last_index, last_seed, last_loaded = outs[0], outs[1], list(outs[2:])
            compute_and_store(last_index, last_seed, last_loaded, passed)
    remap = dict(zip(passed_ts, passed))
    named = GraphWithNamedArgs(loop, graph.args.remap(remap))
    stored_buffers = {}
    for t, h in store_buffers.items():
        if t.graph is not g:
            continue
        if t in load_handles and not isinstance(load_handles[t], xl.HostToDeviceStream):
            stored_buffers[t] = load_handles[t]
        else:
            stored_buffers[t] = h
    return BatchSerialResult(named, stored_buffers, remap)


def batch_serialise(graph: GraphWithNamedArgs, steps: int,
                    load_handles: Dict[xl.Tensor, Union[xl.HostToDeviceStream, RemoteHandle, tuple]],
                    store_streams: Dict[xl.Tensor, xl.DeviceToHostStream],
                    store_buffers: Dict[xl.Tensor, Union[RemoteHandle, tuple]],
                    seed_input: Optional[xl.Tensor] = None, rows: int = 1,
                    io_mode: str = "io") -> BatchSerialResult:
    """Wrap `graph` in a loop of `steps` iterations. Per iteration: load the inputs listed in `load_handles` (host
    stream, or remote buffer entry `row*steps + i` adjusted by the handle's row offset), gather the ones stored as
    shards, call `graph`, store the tensors listed in `store_streams` / `store_buffers` (slicing those with a shard
    group). Inputs without a load handle become inputs of the returned graph (by reference where the original was);
    outputs that are not stored are dropped. `seed_input`, if given, receives a fresh seed each iteration."""
    if io_mode not in ("compute", "io", "io_overlapped"):
        raise ValueError(f"Unknown 'io_mode' {io_mode}. Supported: (compute, io, io_overlapped)")
    if steps < 1:
        raise ValueError("steps must be >= 1")
    load_handles = {t: _as_handle(h) for t, h in load_handles.items()}
    store_buffers = {t: _as_handle(h) for t, h in store_buffers.items()}
    if io_mode == "io_overlapped" and steps < 2:
        logger.warning("batch_serialisation with io_mode='io_overlapped' requires at least 2 steps. "
                       "Falling back to io_mode='io'.")
        io_mode = "io"
    return _build(graph, steps, load_handles, store_streams, store_buffers, seed_input, rows, io_mode)


def batch_serialise_non_overlapped(graph: GraphWithNamedArgs, steps: int, load_handles, store_streams, store_buffers,
                                   seed_input: Optional[xl.Tensor] = None, rows: int = 1,
                                   use_io_tiles: bool = False) -> BatchSerialResult:
    """`batch_serialise` with loads, compute and stores of one micro-batch in sequence (`io_mode` "io" when
    `use_io_tiles`, else "compute")."""
    return batch_serialise(graph, steps, load_handles, store_streams, store_buffers, seed_input, rows,
                           "io" if use_io_tiles else "compute")


def batch_serialise_overlapped(graph: GraphWithNamedArgs, steps: int, load_handles, store_streams, store_buffers,
                               seed_input: Optional[xl.Tensor] = None, rows: int = 1) -> BatchSerialResult:
    """`batch_serialise` with the loop software-pipelined: load of micro-batch i+1, compute of i and store of i-1
    overlap (`io_mode="io_overlapped"`, needs at least 2 steps)."""
    if steps < 2:
        raise ValueError("Overlapped batch serialisation needs at least 2 steps")
    return batch_serialise(graph, steps, load_handles, store_streams, store_buffers, seed_input, rows, "io_overlapped")


def batch_serialise_fwd_and_grad(forward_graph: GraphWithNamedArgs, gradient_graph: GraphWithNamedArgs,
                                 named_inputs_for_grad_graph: NamedTensors, steps: int,
                                 load_handles: Dict[xl.Tensor, Any], store_streams: Dict[xl.Tensor, Any],
                                 store_buffers: Dict[xl.Tensor, Any], seed_input: Optional[xl.Tensor] = None,
                                 rows: int = 1, io_mode: str = "io"
                                 ) -> Tuple[BatchSerialResult, BatchSerialResult]:
    """Serialise a forward graph and its gradient graph together. Every forward tensor the gradient graph expects
    (`Fwd` connections) is either one of `named_inputs_for_grad_graph` (typically the weights: it becomes a named,
    passed-through input of the gradient loop) or is stored by the forward loop into a buffer (created here unless
    given) and loaded by the gradient loop. An entry `{activation: ReplicaGrouping}` in `store_buffers` asks for that
    activation to be stored sharded over the group. Every `FwdGrad` input needs a load handle."""
    shard_groups = {t: v for t, v in store_buffers.items() if isinstance(v, xl.ReplicaGrouping)}
    store_buffers = {t: _as_handle(v) for t, v in store_buffers.items() if not isinstance(v, xl.ReplicaGrouping)}
    load_handles = {t: _as_handle(h) for t, h in load_handles.items()}
    info = gradient_graph.grad_graph_info
    grad_inputs = gradient_graph.graph.inputs
    named_fwd = named_inputs_for_grad_graph.to_dict()
    named_fwd_tensors = set(named_fwd.values())
    activations = [(i, ec.fwd_tensor) for i, ec in enumerate(info.expected_inputs)
                   if ec.connection_type == ExpectedConnectionType.Fwd]
    for _, t in activations:
        if t in store_buffers or t in named_fwd_tensors:
            continue
        if t in load_handles and not isinstance(load_handles[t], xl.HostToDeviceStream):
            store_buffers[t] = load_handles[t]
        else:
            sg = shard_groups.get(t)
            store_buffers[t] = RemoteHandle(batch_serial_buffer(t, steps, rows, sg), 0, sg)
    fwd_result = batch_serialise(forward_graph, steps, load_handles, store_streams, store_buffers, seed_input, rows,
                                 io_mode)
    grad_handles: Dict[xl.Tensor, Any] = {}
    named_inputs = {}
    for idx, t in activations:
        if t in named_fwd_tensors:
            name = next(k for k, v in named_fwd.items() if v is t)
            named_inputs[name] = grad_inputs[idx]
        elif t in fwd_result.stored_buffers:
            grad_handles[grad_inputs[idx]] = fwd_result.stored_buffers[t]
        else:
            raise RuntimeError(f"Fwd Connection {t} missing. You need to provide it either in forward_variables or "
                               f"in load_handles")
    named_inputs.update(gradient_graph.args.named_tensors)
    gradient_graph.args = NamedTensors.from_dict(named_inputs)
    for idx, ec in enumerate(info.expected_inputs):
        if ec.connection_type != ExpectedConnectionType.FwdGrad:
            continue
        gi = grad_inputs[idx]
        if gi not in load_handles:
            raise ValueError(f"FwdGrad input (idx={idx} {gi}) to Gradient graph must have a load_handle specified")
        grad_handles[gi] = load_handles[gi]
    grad_result = batch_serialise(gradient_graph, steps, grad_handles, store_streams, store_buffers, None, rows,
                                  io_mode)
    grad_result.graph.grad_graph_info = remap_grad_info(info, forward_graph.graph, gradient_graph.graph)
    return fwd_result, grad_result
