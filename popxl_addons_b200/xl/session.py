"""Session: owns device state (variables, remote-buffer slabs, constants) and interprets the recorded graphs.

Execution model. Each op of a graph is run in recorded order for every *local* replica: all replicas when the whole
replica set is simulated in one process (CPU backend, used by tests and as oracle), exactly one when the program is
launched with one process per GPU. An op runs its native sm_100a kernel when one is registered for the device and
accepts the operands, else its torch reference implementation. Tensors are released as soon as their last consumer
in the graph has run. Host streams are staged through pinned memory.

Parity: the `popxl.Session` surface used by popxl_addons/task_session.py:52-53,89-98,320-329 and every test
(`run`, `get_tensor(s)_data`, `write_variable(s)_data`, context manager, `ir`, `is_attached`).
"""
import os
import sys
import time
from typing import Any, Dict, Iterable, List, Mapping, Optional

import numpy as np
import torch

from . import dtypes as _dt
from .buffers import DeviceToHostStream, HostToDeviceStream, RemoteBuffer
from .comm import DistComm, SimComm
from .core import Constant, Graph, Ir, LazyInit, Tensor, Variable
from .opdef import note_fallback as _note_fallback


# what `run` takes and returns (popxl/session.py exports the same two names)
h2dStreamBufferMaps = Mapping[HostToDeviceStream, Any]
d2hStreamBufferMaps = Mapping[DeviceToHostStream, np.ndarray]


def _resolve_device(device_desc: str) -> torch.device:
    d = (device_desc or "auto").lower()
    if d in ("cpu", "ipu_model"):
        return torch.device("cpu")
    if d.startswith("cuda"):
        if ":" in d:
            return torch.device(d)
        return torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    # "ipu_hw" / "auto": the accelerator when there is one
    if torch.cuda.is_available():
        return torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    return torch.device("cpu")


class Session:
    def __init__(self, ir: Ir, device_desc: str = "auto", use_native: Optional[bool] = None):
        self.ir = ir
        self.device = _resolve_device(device_desc)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        self.distributed = bool(ir.distributed) and int(os.environ.get("WORLD_SIZE", "1")) > 1
        self.num_replicas = ir.replication_factor
        if use_native is None:
            use_native = ir.options.native_kernels
        self.slots = int(getattr(ir, "devices_per_replica", 1)) if self.distributed else 1
        self.slot: Optional[int] = None  # device slot (pipeline stage GPU) this process executes; None: all of them
        self._frame_dev: List[Optional[int]] = []
        if self.distributed:
            if use_native and self.device.type == "cuda":
                from ..parallel.fused import FusedComm

                self.comm = FusedComm(self.num_replicas, self.device, self, devices_per_replica=self.slots)
            else:
                self.comm = DistComm(self.num_replicas, self.device, devices_per_replica=self.slots)
            self.num_local = 1
            self.replica_offset = self.comm.rank
            if self.slots > 1:
                self.slot = self.comm.slot
        else:
            self.comm = SimComm(self.num_replicas)
            self.num_local = self.num_replicas
            self.replica_offset = 0
        self.use_native = use_native and self.device.type == "cuda"
        if self.use_native:
            from ..ops import native as _native  # noqa: F401  (registers the CUDA kernels; raises if not built)

        self._vars: Dict[Variable, List[torch.Tensor]] = {}
        self._buffers: Dict[RemoteBuffer, List[torch.Tensor]] = {}
        self._consts: Dict[Constant, torch.Tensor] = {}
        self._liveness: Dict[Graph, Dict[int, List[Tensor]]] = {}
        self._inputs: Dict[HostToDeviceStream, List[List[torch.Tensor]]] = {}
        self._cursor: Dict[HostToDeviceStream, int] = {}
        self._outputs: Dict[DeviceToHostStream, List[List[torch.Tensor]]] = {}
        self.is_attached = False
        self.timestamps: Dict[str, Any] = {}
        self._captured: Dict[int, dict] = {}
        self._capture_inputs = None
        self._capture_outputs = None
        self.h2d_bytes = 0  # host->device / device->host traffic of `run` so far (bytes of the tensors copied)
        self.d2h_bytes = 0
        # per-op timing: None = off, else a list of (graph name, op name, start, end) with CUDA events (or host
        # timestamps on CPU); summarised by `profile_summary()`
        self.profile: Optional[list] = [] if ir.options.profile_ops else None
        self._nvtx = bool(ir.options.nvtx) and self.device.type == "cuda"
        # ops recorded under `io_tiles()` run on a second stream (loads, stores and exchanges that overlap the compute
        # stream); values cross between the streams through events
        self._io_stream = (torch.cuda.Stream(self.device) if self.device.type == "cuda"
                           and os.environ.get("XL_IO_STREAM", "1") != "0" else None)
        self._io_ready: Dict[int, tuple] = {}  # id(tensor) -> (event recorded on the IO stream, tensor)
        self._io_dirty = False                 # an op ran on the IO stream since the streams were last joined
        self._slab_events: Dict[RemoteBuffer, tuple] = {}  # last access of a remote-buffer slab: (event, stream id)
        self._slab_pending = None
        self._uncapturable: set = set()        # loops whose capture failed once: they run eagerly from then on
        self._init_state()

    # ------------------------------------------------------------------------------------------------------
    # replica helpers
    # ------------------------------------------------------------------------------------------------------
    def global_replica(self, local_index: int) -> int:
        return self.replica_offset + local_index

    # ------------------------------------------------------------------------------------------------------
    # state
    # ------------------------------------------------------------------------------------------------------
    def _alloc_buffer(self, rb: RemoteBuffer) -> List[torch.Tensor]:
        if rb not in self._buffers:
            dt = rb.tensor_dtype.as_torch()
            if rb.location == "host":
                slabs = [torch.zeros((rb.entries, *rb.tensor_shape), dtype=dt,
                                     pin_memory=self.device.type == "cuda") for _ in range(self.num_local)]
            else:
                slabs = [torch.zeros((rb.entries, *rb.tensor_shape), dtype=dt, device=self.device)
                         for _ in range(self.num_local)]
            self._buffers[rb] = slabs
        return self._buffers[rb]

    def _replica_slice_of_host(self, var: Variable, host, replica: int) -> torch.Tensor:
        """Host array (full `shape_on_host`) -> the value replica `replica` holds."""
        rg = var.replica_grouping
        data = host
        if isinstance(data, LazyInit):
            if data.kind == "copy":
                src = data.source
                local = replica - self.replica_offset
                full = self._vars[src][local]
                if src.shard_group is not None:
                    raise ValueError("LazyInit copy of a sharded variable is not supported")
                data = full.detach()
            else:
                data = data.materialize(self.device, var.dtype.as_torch(), rg.group_index(replica))
        elif rg.num_groups > 1:
            data = data[rg.group_index(replica)]
        if isinstance(data, np.ndarray):
            data = _dt.to_torch(np.asarray(data))
        if var.shard_group is not None:
            n = var.nelms
            i = var.shard_group.index_in_group(replica)
            data = data.reshape(-1)[i * n:(i + 1) * n]
        return data.reshape(var.shape).to(var.dtype.as_torch())

    def _write_var(self, var: Variable, host):
        vals = []
        for r in range(self.num_local):
            vals.append(self._replica_slice_of_host(var, host, self.global_replica(r)))
        if var.remote_buffer is not None:
            slabs = self._alloc_buffer(var.remote_buffer)
            for r, v in enumerate(vals):
                slabs[r][var.entry].copy_(v.reshape(var.remote_buffer.tensor_shape))
        else:
            if var in self._vars:
                for r, v in enumerate(vals):
                    self._vars[var][r].copy_(v)
            elif var.symmetric_group is not None and self.distributed and self.use_native:
                from ..parallel.fused import runtime

                store = runtime(self).context(var.symmetric_group).arena.alloc(var.shape, var.dtype.as_torch())
                store.copy_(vals[0])
                self._vars[var] = [store]
            else:
                self._vars[var] = [v.to(self.device, copy=True) for v in vals]

    def _variable_slots(self) -> Dict[Variable, set]:
        """Device slots whose ops read or write each variable (following call sites into the called graphs)."""
        owners: Dict[Variable, set] = {}

        def walk(graph, binding, frame):
            for op in graph.ops:
                dev = self._effective_device(op, frame)
                sub = op.attrs.get("graph") if op.opdef.name in ("call", "repeat") else None
                if sub is not None:
                    inner = {gi: binding.get(t, t) for gi, t in zip(sub._inputs, op.inputs)}
                    walk(sub, inner, dev if op.device_explicit else frame)
                    continue
                if op.opdef.name == "conditional":
                    for key in ("then_graph", "else_graph"):
                        g2 = op.attrs[key]
                        inner = {gi: binding.get(t, t) for gi, t in zip(g2._inputs, op.inputs[1:])}
                        walk(g2, inner, dev if op.device_explicit else frame)
                    continue
                for t in op.inputs:
                    root = binding.get(t, t)
                    if isinstance(root, Variable):
                        owners.setdefault(root, set()).add(dev)
        walk(self.ir.main_graph, {}, None)
        return owners

    @staticmethod
    def _effective_device(op, frame: Optional[int]) -> int:
        """Ops placed explicitly (`with ipu(i)`) run there; other ops run where the enclosing explicitly placed call
        runs, or, outside any such call, where their operands live."""
        if op.device_explicit or frame is None:
            return op.device_index
        return frame

    def owns(self, var: Variable) -> bool:
        """Whether this process holds `var` (always true unless replicas span several processes)."""
        return self.slot is None or var in self._vars or var.remote_buffer is not None

    def _init_state(self):
        for rb in self.ir.remote_buffers:
            self._alloc_buffer(rb)
        deferred = []
        skip = set()
        if self.slot is not None:
            owners = self._variable_slots()
            for var in self.ir.initial_values:
                slots = owners.get(var) or {var.device_index}
                if self.slot not in slots:
                    skip.add(var)
        if self.distributed and self.use_native:
            from ..parallel.fused import runtime

            for var in self.ir.initial_values:
                if var.symmetric_group is not None and var.remote_buffer is None:
                    runtime(self).reserve(var.symmetric_group, var.nelms * var.dtype.itemsize)
        for var, host in self.ir.initial_values.items():
            if var in skip:
                continue
            if isinstance(host, LazyInit) and host.kind == "copy":
                deferred.append((var, host))  # copies are made once their source exists
            else:
                self._write_var(var, host)
        for var, host in deferred:
            self._write_var(var, host)

    def _read_var_local(self, var: Variable) -> List[torch.Tensor]:
        if var.remote_buffer is not None:
            return [s[var.entry] for s in self._alloc_buffer(var.remote_buffer)]
        return self._vars[var]

    def get_tensor_data(self, tensor: Variable) -> np.ndarray:
        return self.get_tensors_data([tensor])[tensor]

    def get_tensors_data(self, tensors: Iterable[Variable]) -> Dict[Variable, np.ndarray]:
        """Host copies of variables in their `shape_on_host`: one entry per replica group; replica-sharded variables
        are re-assembled to their full `meta_shape`. Collective when distributed (every rank must call)."""
        out = {}
        for var in tensors:
            if isinstance(var, Constant):
                out[var] = _dt.to_numpy(var.data)
                continue
            if not isinstance(var, Variable):
                raise TypeError(f"{var} is not a variable")
            if not self.owns(var):
                raise KeyError(f"{var} lives on another device slot (this process holds slot {self.slot}); read it "
                               f"from the process that owns it (`Session.owns`)")
            per_replica = self.comm.gather_to_host(self._read_var_local(var))
            rg = var.replica_grouping
            per_group = []
            for members in rg.groups:
                if var.shard_group is not None:
                    # the replicas of this group that are in one shard group, in shard order
                    shard_members = [r for r in var.shard_group.group_of(members[0])]
                    full = torch.cat([per_replica[r].reshape(-1) for r in shard_members])
                    per_group.append(full.reshape(var.meta_shape))
                else:
                    per_group.append(per_replica[members[0]].reshape(var.shape))
            res = torch.stack(per_group) if rg.num_groups > 1 else per_group[0]
            if res.device.type == "cpu" and self.device.type == "cpu" and rg.num_groups == 1:
                res = res.clone()  # on the CPU backend the gathered value is the live storage: hand out a copy
            out[var] = _dt.to_numpy(res)
            mm = getattr(var, "_memmap_arr", None)
            if mm is not None and tuple(mm.shape) == tuple(out[var].shape):
                # memmap-backed variable: the host file is the variable's host copy
                if mm.flags.writeable:
                    mm[...] = out[var].astype(mm.dtype, copy=False)
                    out[var] = mm
                elif np.array_equal(mm, out[var]):
                    out[var] = mm
        return out

    def write_variable_data(self, tensor: Variable, data) -> None:
        self.write_variables_data({tensor: data})

    def write_variables_data(self, tensors: Mapping[Variable, Any]) -> None:
        for var, data in tensors.items():
            if not isinstance(var, Variable):
                raise TypeError(f"{var} is not a variable")
            host = _dt.to_torch(np.asarray(data)) if not isinstance(data, torch.Tensor) else data.detach().cpu()
            if tuple(host.shape) != tuple(var.shape_on_host):
                if host.numel() == int(np.prod(var.shape_on_host)):
                    host = host.reshape(var.shape_on_host)
                else:
                    raise ValueError(f"Data shape {tuple(host.shape)} does not match the variable's host shape "
                                     f"{var.shape_on_host} ({var})")
            self._write_var(var, host)

    # popxl names
    def weights_to_host(self):
        pass

    def weights_from_host(self):
        pass

    # -- the rest of popxl.Session's host interface -----------------------------------------------------------------
    def _streams(self, kind):
        seen, out = set(), []

        def walk(graph):
            if id(graph) in seen:
                return
            seen.add(id(graph))
            for op in graph.ops:
                st = op.attrs.get("stream")
                if isinstance(st, kind) and st not in out:
                    out.append(st)
                callee = op.attrs.get("graph")
                if callee is not None and hasattr(callee, "ops"):
                    walk(callee)

        walk(self.ir.main_graph)
        return out

    def expected_inputs(self) -> List[HostToDeviceStream]:
        """The host-to-device streams the program loads from, in order of first use."""
        return self._streams(HostToDeviceStream)

    def create_host_outputs(self) -> Dict[DeviceToHostStream, np.ndarray]:
        """Zero-filled arrays of the shapes `run` returns, one per device-to-host stream of the program."""
        T, R = int(self.ir.num_host_transfers), self.num_replicas
        lead = ((T,) if T > 1 else ()) + ((R,) if R > 1 else ())
        return {st: np.zeros(lead + tuple(st.shape), dtype=_dt.to_numpy(torch.zeros((), dtype=st.dtype.as_torch())).dtype)
                for st in self._streams(DeviceToHostStream)}

    def run_with_outputs(self, inputs: Optional[Mapping[HostToDeviceStream, Any]] = None,
                         outputs: Optional[Dict[DeviceToHostStream, np.ndarray]] = None,
                         downcast_inputs: bool = True) -> None:
        """`run`, with the results written into caller-provided arrays (`create_host_outputs()` makes them)."""
        res = self.run(inputs, downcast_inputs=downcast_inputs)
        for st, arr in (outputs or {}).items():
            if st not in res:
                raise ValueError(f"{st} is not written by this program")
            arr[...] = np.asarray(res[st]).reshape(arr.shape)

    @property
    def ir_(self):
        return self.ir

    def __enter__(self):
        self.is_attached = True
        return self

    def __exit__(self, *exc):
        self.is_attached = False
        return False

    # ------------------------------------------------------------------------------------------------------
    # host IO
    # ------------------------------------------------------------------------------------------------------
    def _stage_inputs(self, inputs: Mapping[HostToDeviceStream, Any]):
        T = int(self.ir.num_host_transfers)
        R = self.num_replicas
        self._inputs, self._cursor = {}, {}
        for stream, arr in (inputs or {}).items():
            if not isinstance(stream, HostToDeviceStream):
                raise TypeError(f"{stream} is not a host-to-device stream")
            host = arr if isinstance(arr, torch.Tensor) else _dt.to_torch(np.asarray(arr))
            self.h2d_bytes += host.numel() * host.element_size() if host.device.type == "cpu" else 0
            if host.dtype != stream.dtype.as_torch():
                host = host.to(stream.dtype.as_torch())
            n_local = self.num_local
            full = (T, R, *stream.shape)
            local = (T, n_local, *stream.shape)
            numel = host.numel()
            if numel == int(np.prod(full)) and (not self.distributed or R == 1):
                host = host.reshape(full)
            elif self.distributed and numel == int(np.prod(full)):
                host = host.reshape(full)[:, self.replica_offset:self.replica_offset + 1]
            elif numel == int(np.prod(local)):
                host = host.reshape(local)
            else:
                raise ValueError(
                    f"Input for stream {stream.name} has shape {tuple(host.shape)}; expected "
                    f"(num_host_transfers={T}, replication_factor={R}, *{stream.shape}) with unit axes optional")
            if self.device.type == "cuda" and host.device.type == "cpu":
                if not host.is_pinned():
                    host = host.contiguous().pin_memory()
                dev = host.to(self.device, non_blocking=True)
            else:
                dev = host  # already resident on the session's device
            self._inputs[stream] = dev
            self._cursor[stream] = 0

    def host_load(self, stream: HostToDeviceStream) -> List[torch.Tensor]:
        if getattr(self, "_capture_inputs", None) is not None:
            return [self._capture_inputs[stream]]
        if stream not in self._inputs:
            raise KeyError(f"No input was provided for host stream {stream.name}")
        i = self._cursor[stream]
        data = self._inputs[stream]
        if i >= data.shape[0]:
            raise RuntimeError(
                f"Stream {stream.name} was read more than num_host_transfers={data.shape[0]} times in one run")
        self._cursor[stream] = i + 1
        return [data[i, r] for r in range(self.num_local)]

    def host_store(self, stream: DeviceToHostStream, vals: List[torch.Tensor]):
        if getattr(self, "_capture_outputs", None) is not None:
            self._capture_outputs.append((stream, [v.detach().clone() for v in vals]))
            return
        self._outputs.setdefault(stream, []).append([v.detach().clone() for v in vals])

    def _collect_outputs(self, fetch: bool = True) -> Dict[DeviceToHostStream, np.ndarray]:
        T = int(self.ir.num_host_transfers)
        res = {}
        for stream, items in self._outputs.items():
            stacked = torch.stack([torch.stack(per_replica) for per_replica in items])  # (t, R_local, *shape)
            if not fetch:
                res[stream] = stacked
                continue
            self.d2h_bytes += stacked.numel() * stacked.element_size() if stacked.device.type != "cpu" else 0
            arr = _dt.to_numpy(stacked)
            if arr.shape[1] == 1:
                arr = arr[:, 0]
            if arr.shape[0] == 1 and T == 1:
                arr = arr[0]
            res[stream] = arr
        return res

    # ------------------------------------------------------------------------------------------------------
    # remote buffers / device copies
    # ------------------------------------------------------------------------------------------------------
    @staticmethod
    def _index(idx: torch.Tensor) -> int:
        return int(idx.reshape(-1)[0].item())

    def _row_index(self, rb: RemoteBuffer, idx: torch.Tensor):
        """Row selector of a slab access. Slabs in device memory are indexed on the device (no host read, so the access
        can sit in a captured loop): a CUDA index is clamped into range, since an out-of-range one cannot be reported
        without a synchronisation; on the CPU backend it is checked. Slabs in pinned host memory need the index on the
        host."""
        if rb.location == "host" or idx.device.type == "cpu":
            i = self._index(idx)
            if not 0 <= i < rb.entries:
                raise IndexError(f"remote buffer index {i} out of range for {rb}")
            return i
        return idx.reshape(-1)[:1].to(torch.int64).clamp(0, rb.entries - 1)

    def _order_slab_access(self, rb: RemoteBuffer):
        """A slab is not an operand the executor can see, so accesses from the two streams are ordered here: the
        stream that touches a slab first waits for the last access made from the other stream."""
        if self._io_stream is None:
            return
        cur = torch.cuda.current_stream(self.device)
        last = self._slab_events.get(rb)
        if last is not None and last[1] != cur.cuda_stream:
            cur.wait_event(last[0])
        ev = torch.cuda.Event()
        self._slab_pending = (rb, ev, cur)

    def _slab_access_done(self):
        pend = getattr(self, "_slab_pending", None)
        if pend is not None:
            rb, ev, cur = pend
            ev.record(cur)
            self._slab_events[rb] = (ev, cur.cuda_stream)
            self._slab_pending = None

    def remote_load(self, rb: RemoteBuffer, index: List[torch.Tensor]) -> List[torch.Tensor]:
        self._order_slab_access(rb)
        try:
            return self._remote_load(rb, index)
        finally:
            self._slab_access_done()

    def remote_store(self, rb: RemoteBuffer, index: List[torch.Tensor], vals: List[torch.Tensor]):
        self._order_slab_access(rb)
        try:
            self._remote_store(rb, index, vals)
        finally:
            self._slab_access_done()

    def _remote_load(self, rb: RemoteBuffer, index: List[torch.Tensor]) -> List[torch.Tensor]:
        slabs = self._alloc_buffer(rb)
        out = []
        for r in range(self.num_local):
            i = self._row_index(rb, index[r])
            if isinstance(i, int):
                out.append(slabs[r][i].to(self.device, non_blocking=True).clone() if rb.location == "host"
                           else slabs[r][i].clone())
            else:
                out.append(slabs[r].index_select(0, i).reshape(rb.tensor_shape))
        return out

    def _remote_store(self, rb: RemoteBuffer, index: List[torch.Tensor], vals: List[torch.Tensor]):
        slabs = self._alloc_buffer(rb)
        for r in range(self.num_local):
            i = self._row_index(rb, index[r])
            if isinstance(i, int):
                slabs[r][i].copy_(vals[r].reshape(rb.tensor_shape), non_blocking=True)
            else:
                slabs[r].index_copy_(0, i, vals[r].reshape(1, *rb.tensor_shape))

    def device_copy(self, vals, op):
        """Stage-boundary copy. One process per device slot: the source slot queues a send, the destination slot a
        receive (issued together, see `DistComm.flush_p2p`); elsewhere all slots share this process's memory."""
        if self.slot is None:
            return vals
        src, dst = op.attrs["source"], op.attrs["destination"]
        if src == dst:
            return vals
        if self.slot == src:
            self.comm.send_to_slot(vals[0], dst)
            return None
        if self.slot == dst:
            out = op.outputs[0]
            return [self.comm.recv_from_slot(out.shape, out.dtype.as_torch(), src)]
        return None

    def record_timestamp(self, name: str):
        if self.device.type == "cuda":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
        else:
            import time

            ev = time.perf_counter()
        self.timestamps[name] = ev

    def elapsed_ms(self, start: str, end: str) -> float:
        """Device time between two `ops.timestamp` marks of the last run (synchronises)."""
        a, b = self.timestamps[start], self.timestamps[end]
        if self.device.type == "cuda":
            b.synchronize()
            return a.elapsed_time(b)
        return (b - a) * 1e3

    # -- per-op profile ----------------------------------------------------------------------------------------------
    def _now(self):
        if self.device.type == "cuda":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            return ev
        return time.perf_counter()

    def start_profile(self):
        """Time every op from now on (loop bodies run eagerly while profiling, CUDA-graph replay is bypassed)."""
        self.profile = []

    def profile_summary(self, stop: bool = True) -> Dict[str, Dict[str, float]]:
        """`{op name: {"count", "ms"}}` over everything executed since profiling started, slowest first. On CUDA the
        times are between events on the launching stream: an op's time includes the wait for its own launch when the
        host runs behind the device."""
        if self.profile is None:
            raise RuntimeError("profiling is off: set `ir.options.profile_ops` or call `start_profile()`")
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        agg: Dict[str, Dict[str, float]] = {}
        for _g, name, a, b in self.profile:
            ms = a.elapsed_time(b) if self.device.type == "cuda" else (b - a) * 1e3
            e = agg.setdefault(name, {"count": 0, "ms": 0.0})
            e["count"] += 1
            e["ms"] += ms
        self.profile = None if stop else []
        return dict(sorted(agg.items(), key=lambda kv: -kv[1]["ms"]))

    def native_collective(self, name: str):
        """Fused compute+collective kernel registered under `name` for this session's transport, or None (then the
        op runs its reference composition over `self.comm`)."""
        if not self.use_native:
            return None
        from ..parallel import fused

        if not self.distributed and name not in fused.LOCAL_OK:
            return None
        fn = fused.lookup(name, self)
        if fn is None:
            return None

        def counted(*args, **kw):
            res = fn(*args, **kw)
            if res is NotImplemented:
                _note_fallback("fused:" + name)  # the op then runs as its own kernels + a library collective
            return res

        return counted

    # ------------------------------------------------------------------------------------------------------
    # interpreter
    # ------------------------------------------------------------------------------------------------------
    def _const(self, c: Constant) -> torch.Tensor:
        v = self._consts.get(c)
        if v is None:
            v = c.data.to(self.device)
            self._consts[c] = v
        return v

    def _last_uses(self, graph: Graph) -> Dict[int, List[Tensor]]:
        lv = self._liveness.get(graph)
        if lv is None or lv[-1] != (len(graph.ops), len(graph._outputs)):
            last: Dict[Tensor, int] = {}
            for i, op in enumerate(graph.ops):
                for t in op.inputs:
                    last[t] = i
                for t in op.outputs:
                    last.setdefault(t, i)
            keep = set(graph._outputs) | set(graph._inputs)
            table: Dict[int, List[Tensor]] = {}
            for t, i in last.items():
                if t in keep or isinstance(t, (Variable, Constant)):
                    continue
                table.setdefault(i, []).append(t)
            table[-1] = (len(graph.ops), len(graph._outputs))
            self._liveness[graph] = lv = table
        return lv

    def _value(self, t: Tensor, env) -> List[torch.Tensor]:
        v = env.get(t)
        if v is not None:
            return v
        if isinstance(t, Constant):
            c = self._const(t)
            v = [c] * self.num_local
            env[t] = v
            return v
        if isinstance(t, Variable):
            if t.remote_buffer is not None:
                raise RuntimeError(f"{t} is a remote variable: read it with ops.remote_load")
            if self.slot is not None and t not in self._vars:
                return None
            return self._vars[t]
        if self.slot is not None:
            return None  # lives on another device slot (another process)
        raise KeyError(f"Tensor {t} has no value: it was used before being produced, or belongs to another graph")

    def _exec_ops(self, graph: Graph, env: Dict[Tensor, List[torch.Tensor]]):
        frees = self._last_uses(graph)
        native_dev = self.device.type if self.use_native else None
        staged = self.slot is not None
        frame = self._frame_dev[-1] if self._frame_dev else None
        for i, op in enumerate(graph.ops):
            od = op.opdef
            if staged:
                name = od.name
                if name in ("call", "repeat", "conditional"):
                    # control flow runs everywhere; what it calls is filtered op by op
                    self.comm.flush_p2p()
                    for t in op.inputs:
                        if t not in env:
                            env[t] = self._value(t, env)
                    self._frame_dev.append(self._effective_device(op, frame) if op.device_explicit else frame)
                    try:
                        od.special(self, op, env)
                    finally:
                        self._frame_dev.pop()
                    self._free_dead(frees, i, env)
                    continue
                if name == "ipu_copy":
                    env[op.outputs[0]] = self.device_copy(env.get(op.inputs[0]), op)
                    self._free_dead(frees, i, env)
                    continue
                if self._effective_device(op, frame) != self.slot:
                    continue
                self.comm.flush_p2p()  # received tensors may be read from here on
            control = od.name in ("call", "repeat", "conditional")
            pending = self.comm.pending
            if pending and not control:
                # a collective or receive still in flight is joined right before the first op that reads its result
                for t in op.inputs:
                    for x in env.get(t) or ():
                        entry = pending.pop(id(x), None)
                        if entry is not None:
                            entry[0].wait()
            on_io = self._io_stream is not None and op.tile_set == "io" and not control
            io_ctx = None
            if on_io:
                compute = torch.cuda.current_stream(self.device)
                self._io_stream.wait_stream(compute)  # everything queued on the compute stream so far is visible
                self._io_dirty = True
                for t in op.inputs:
                    for x in env.get(t) or ():
                        if isinstance(x, torch.Tensor) and x.is_cuda:
                            x.record_stream(self._io_stream)
                io_ctx = torch.cuda.stream(self._io_stream)
                io_ctx.__enter__()
            elif self._io_ready and not control:
                # a value produced on the IO stream is awaited by the compute stream at its first reader
                for t in op.inputs:
                    for x in env.get(t) or ():
                        entry = self._io_ready.pop(id(x), None)
                        if entry is not None:
                            torch.cuda.current_stream(self.device).wait_event(entry[0])
            timed = self.profile is not None and not control
            if timed:
                t_start = self._now()
            if self._nvtx:
                torch.cuda.nvtx.range_push(f"{graph.name}/{od.name}")
            if od.special is not None:
                for t in op.inputs:
                    if t not in env:
                        env[t] = self._value(t, env)
                od.special(self, op, env)
            else:
                ins = [self._value(t, env) for t in op.inputs]
                fn = od.native.get(native_dev) if native_dev else None
                outs_per_replica = []
                for r in range(self.num_local):
                    args = [v[r] for v in ins]
                    res = NotImplemented
                    if fn is not None:
                        res = fn(*args, **op.attrs)
                        if res is NotImplemented:
                            _note_fallback(od.name, ", ".join(
                                f"{tuple(a.shape)} {str(a.dtype).replace('torch.', '')}" for a in args
                                if isinstance(a, torch.Tensor)))
                    if res is NotImplemented:
                        res = od.impl(*args, **op.attrs)
                    outs_per_replica.append((res,) if isinstance(res, torch.Tensor) else tuple(res or ()))
                for j, t in enumerate(op.outputs):
                    env[t] = [outs_per_replica[r][j] for r in range(self.num_local)]
            if self._nvtx:
                torch.cuda.nvtx.range_pop()
            if timed:
                self.profile.append((graph.name, od.name + (" [io]" if on_io else ""), t_start, self._now()))
            if on_io:
                ev = torch.cuda.Event()
                ev.record(self._io_stream)
                io_ctx.__exit__(None, None, None)
                for t in op.outputs:
                    for x in env.get(t) or ():
                        if isinstance(x, torch.Tensor) and x.is_cuda:
                            x.record_stream(compute)
                            self._io_ready[id(x)] = (ev, x)  # holding `x` keeps its id unique while the entry exists
            self._free_dead(frees, i, env)
        if staged:
            self.comm.flush_p2p()

    def _join_streams(self):
        """The compute stream waits for everything queued on the IO stream and for every collective in flight (end of a
        run, end of a loop iteration, end of a captured loop body)."""
        self.comm.wait_all()
        if not self._io_dirty:
            self._slab_events.clear()  # every access so far was made from the compute stream: already ordered
        if self._io_stream is not None and self._io_dirty:
            # only when an op ran there since the last join: inside a graph capture a wait on a stream that never forked
            # from the capturing stream would invalidate the capture
            torch.cuda.current_stream(self.device).wait_stream(self._io_stream)
            self._io_ready.clear()
            self._slab_events.clear()
            self._io_dirty = False

    @staticmethod
    def _free_dead(frees, i, env):
        dead = frees.get(i)
        if dead:
            for t in dead:
                env.pop(t, None)

    def run_graph(self, graph: Graph, inputs: List[List[torch.Tensor]]) -> List[List[torch.Tensor]]:
        env = dict(zip(graph._inputs, inputs))
        self._exec_ops(graph, env)
        return [self._value(t, env) for t in graph._outputs]

    # ops that read a device value on the host, or decide on the host what runs: a loop body holding one is not captured
    _HOST_SYNC_OPS = frozenset({"conditional", "print_tensor", "dropout", "random_uniform", "random_normal",
                                "shaped_dropout", "timestamp", "fp8_mse_scale", "histogram"})

    def _capture_safe(self, graph: Graph, _seen=None) -> bool:
        """Whether a loop body can be captured into a CUDA graph without being told so: nothing in it (or in the graphs
        it calls) reads a device value on the host or touches a slab in pinned host memory."""
        seen = _seen if _seen is not None else set()
        if id(graph) in seen:
            return True
        seen.add(id(graph))
        for o in graph.ops:
            name = o.opdef.name
            if name in self._HOST_SYNC_OPS:
                return False
            if name in ("remote_load", "remote_store") and o.attrs["buffer"].location == "host":
                return False
            for key in ("graph", "then_graph", "else_graph"):
                callee = o.attrs.get(key)
                if callee is not None and hasattr(callee, "ops") and not self._capture_safe(callee, seen):
                    return False
        return True

    def run_repeat(self, op, graph: Graph, vals: List[List[torch.Tensor]], env):
        n_out = len(graph._outputs)
        count = op.attrs["count"]
        want = op.attrs.get("cuda_graph") or (self.ir.options.capture_loops and count >= 3
                                              and self._capture_safe(graph))
        # values that live on another process (a pipeline stage of a replica spanning processes) are None here: such a
        # loop exchanges them by send / recv and runs eagerly
        local = all(v is not None and all(x is not None for x in v) for v in vals)
        if (want and local and self.device.type == "cuda" and self.num_local == 1 and self.ir.options.cuda_graphs
                and self.profile is None and op.uid not in self._uncapturable and not self._capturing):
            outs = self._run_repeat_captured(op, graph, vals, count)
            if outs is not None:
                for t, v in zip(op.outputs, outs):
                    env[t] = v
                return
            vals = self._repeat_resume  # the iterations that did run eagerly before the capture was given up
            count = count - self._repeat_done
        outs = vals[:n_out]
        for _ in range(count):
            outs = self.run_graph(graph, vals)
            self._join_streams()
            vals = list(outs) + list(vals[n_out:])
        for t, v in zip(op.outputs, outs):
            env[t] = v

    # -- CUDA-graph replay of a loop body -----------------------------------------------------------------------
    _capturing = False

    def _run_repeat_captured(self, op, graph: Graph, vals, count: int):
        """Loop body without host syncs or shape changes: the first iteration ever runs eagerly (lazy initialisation:
        arenas, workspaces, library handles), the second is captured into a CUDA graph, all later ones (in this and
        every following `run`) replay it. Loop-carried values live in static buffers: the captured body reads them and
        copies its outputs back into them, so a replay continues where the previous one stopped. Host-stream reads
        inside the body go through a static staging tensor that is refreshed before each replay; host-stream writes are
        copied out after it. Returns the outputs of the last iteration, or None if the body could not be captured (the
        loop then continues eagerly from `self._repeat_resume`)."""
        # a collective issued outside the loop may still be in flight: its join must not land inside the capture (a wait
        # on an event recorded outside a capture is not part of the replayed graph)
        self._join_streams()
        n_out = len(graph._outputs)
        state = self._captured.get(op.uid)
        it = 0
        debug = os.environ.get("XL_DEBUG_CAPTURE") == "1"

        def note(msg):
            if debug:
                torch.cuda.synchronize(self.device)
                print(f"[capture rank {os.environ.get('RANK', '0')}] {graph.name}: {msg}", file=sys.stderr, flush=True)

        if state is None:
            outs = self.run_graph(graph, vals)  # eager warm-up iteration
            self._join_streams()
            note("eager iteration done")
            it = 1
            vals = list(outs[:n_out]) + list(vals[n_out:])
            if count == 1:
                return outs
            carried = [[v[0].clone()] for v in vals[:n_out]]
            try:
                state = self._capture(op, graph, vals, carried)
            except Exception as e:  # an op that cannot be captured after all: remember it and go on eagerly
                if op.attrs.get("cuda_graph"):
                    raise
                note(f"capture given up: {type(e).__name__}: {e}")
                self._uncapturable.add(op.uid)
                self._repeat_resume, self._repeat_done = vals, 1
                return None
            note("captured and replayed once")
            self._captured[op.uid] = state
            self._after_replay(state)
            it = 2
        else:
            for buf, v in zip(state["carried"], vals[:n_out]):
                buf[0].copy_(v[0])
        ptrs = tuple(v[0].data_ptr() for v in vals[n_out:])
        if ptrs != state["ptrs"]:
            raise RuntimeError("inputs of a CUDA-graph-captured loop changed address between runs")
        from ..ops import native as _native

        for _ in range(it, count):
            for stream, static in state["static_in"].items():
                static.copy_(self._next_host_item(stream), non_blocking=True)
            state["graph"].replay()
            _native.count_replay(state["kernels"])
            self._after_replay(state)
        return [[buf[0].clone()] for buf in state["carried"]]

    def _next_host_item(self, stream):
        i = self._cursor[stream]
        data = self._inputs[stream]
        if i >= data.shape[0]:
            raise RuntimeError(f"Stream {stream.name} was read more than num_host_transfers={data.shape[0]} times")
        self._cursor[stream] = i + 1
        return data[i, 0]

    def _host_loads_of(self, graph: Graph, found=None, _seen=None):
        """Host-to-device streams read anywhere inside a loop body (also in the graphs it calls)."""
        found = found if found is not None else []
        seen = _seen if _seen is not None else set()
        if id(graph) in seen:
            return found
        seen.add(id(graph))
        for o in graph.ops:
            if o.opdef.name == "host_load" and o.attrs["stream"] not in found:
                found.append(o.attrs["stream"])
            callee = o.attrs.get("graph")
            if callee is not None and hasattr(callee, "ops"):
                self._host_loads_of(callee, found, seen)
        return found

    def _capture(self, op, graph: Graph, vals, carried):
        from ..ops import native as _native

        n_out = len(carried)
        static_in = {}
        cursors = dict(self._cursor)
        for st in self._host_loads_of(graph):
            static_in[st] = torch.empty_like(self._inputs[st][0, 0])
        for stream, static in static_in.items():
            static.copy_(self._next_host_item(stream), non_blocking=True)
        self._capture_inputs = static_in
        self._capture_outputs = []
        kernels: List[str] = []
        _native._RECORDING.append(kernels)
        g = torch.cuda.CUDAGraph()
        torch.cuda.synchronize(self.device)
        ok = False
        self._capturing = True
        try:
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                outs = self.run_graph(graph, carried + list(vals[n_out:]))
                # every stream forked inside the body joins before its results are read back and the capture ends
                self._join_streams()
                for buf, o in zip(carried, outs[:n_out]):
                    buf[0].copy_(o[0])
            ok = True
        finally:
            self._capturing = False
            _native._RECORDING.pop()
            outs_rec = self._capture_outputs
            self._capture_inputs, self._capture_outputs = None, None
            if not ok:
                self._cursor = cursors  # the failed capture executed nothing: its host items are still unread
                self._io_ready.clear()
        if os.environ.get("XL_DEBUG_CAPTURE") == "1":
            print(f"[capture rank {os.environ.get('RANK', '0')}] {graph.name}: capture ended, {len(kernels)} own kernels",
                  file=sys.stderr, flush=True)
        g.replay()  # capture records but does not execute
        _native.count_replay(kernels)
        return {"graph": g, "static_in": static_in, "outputs": outs_rec, "kernels": kernels, "carried": carried,
                "ptrs": tuple(v[0].data_ptr() for v in vals[n_out:])}

    def _after_replay(self, state):
        for stream, tensors in state["outputs"]:
            self._outputs.setdefault(stream, []).append([t.clone() for t in tensors])

    def run(self, inputs: Optional[Mapping[HostToDeviceStream, Any]] = None,
            downcast_inputs: bool = True, fetch: bool = True) -> Dict[DeviceToHostStream, np.ndarray]:
        """Execute the main graph once. `inputs[stream]` has shape
        `(num_host_transfers, replication_factor, *stream.shape)` (unit axes may be omitted; under one process per
        GPU the replica axis may hold only this rank's slice). Host inputs are staged through pinned memory; tensors
        already on the session's device are used as they are. With `fetch=False` the outputs stay on the device
        (stacked torch tensors) and the call does not synchronise."""
        self._outputs = {}
        self._stage_inputs(inputs or {})
        main = self.ir.main_graph
        env: Dict[Tensor, List[torch.Tensor]] = {}
        with torch.no_grad():
            self._exec_ops(main, env)
            self._join_streams()
        out = self._collect_outputs(fetch)
        if self.use_native and fetch:
            from ..ops import native as _native

            _native.check_gemm_errors()
            if getattr(self, "_fused_runtime", None) is not None:
                self._fused_runtime.check()
        return out
