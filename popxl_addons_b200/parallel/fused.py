"""Fused compute + collective kernels on one process per GPU, and the session-side plumbing they need (arenas per
replica group, placement of variables in symmetric memory, a communicator that serves small reductions from a one-shot
NVLink kernel and everything else from NCCL)."""
import ctypes
import os
from typing import Dict, Optional

import torch

from ..xl.comm import DistComm
from ..xl.core import ReplicaGrouping
from .symm import SymmArena

_SMALL_ALL_REDUCE_ELEMS = 16384  # fp32 elements served by the one-shot kernel (64 KiB)
_SMALL_ALL_REDUCE_16BIT_BYTES = 128 << 10  # 16-bit activations served by the one-shot multimem kernel


# multimem needs NVLS; tests that lose a rank on purpose switch it off together with NCCL's
_MC_ALL_REDUCE = os.environ.get("XL_MULTIMEM", "1") != "0"


class GroupContext:
    """Everything the fused kernels need for one replica group of this rank."""

    def __init__(self, session, grouping: ReplicaGrouping, nbytes: int):
        pg, members = session.comm.group_for(grouping)
        self.pg, self.members = pg, members
        self.arena = SymmArena(nbytes, pg, session.device)
        self.rank, self.world = self.arena.rank, self.arena.world
        self.stage = self.arena.alloc((_SMALL_ALL_REDUCE_ELEMS,), torch.float32)  # staging of the small fp32 all-reduce
        # two alternating halves for the one-shot 16-bit all-reduce
        self.stage16 = self.arena.alloc((2 * _SMALL_ALL_REDUCE_16BIT_BYTES,), torch.uint8)
        self.err = torch.zeros(1, dtype=torch.int32, device=session.device)

    def check(self):
        code = int(self.err.item())
        self.arena.check_guards()  # no-op unless the arena was built with canaries
        if code:
            self.err.zero_()
            names = {101: "a peer never consumed this rank's previous signal", 102: "a peer's signal never arrived",
                     103: "the start-of-kernel handshake with the peers did not complete"}
            raise CollectiveTimeout(f"collective on group {self.members} gave up waiting: {names.get(code, code)}")


class CollectiveTimeout(RuntimeError):
    """A bounded device-side wait on a peer ran out; the CUDA context is still usable."""


def _key(grouping: ReplicaGrouping):
    return tuple(tuple(g) for g in grouping.groups)


class FusedRuntime:
    def __init__(self, session):
        self.session = session
        self.groups: Dict[tuple, GroupContext] = {}
        self.budget: Dict[tuple, int] = {}

    def reserve(self, grouping: ReplicaGrouping, nbytes: int):
        k = _key(grouping)
        self.budget[k] = self.budget.get(k, 0) + int(nbytes) + 512

    def context(self, grouping: ReplicaGrouping) -> GroupContext:
        k = _key(grouping)
        if k not in self.groups:
            base = 256 << 20  # room for fused-GEMM output rings and staging
            self.groups[k] = GroupContext(self.session, grouping, self.budget.get(k, 0) + base)
        return self.groups[k]

    def check(self):
        for ctx in self.groups.values():
            ctx.check()


def runtime(session) -> FusedRuntime:
    rt = getattr(session, "_fused_runtime", None)
    if rt is None:
        rt = FusedRuntime(session)
        session._fused_runtime = rt
    return rt


# ---- native collectives looked up by the ops -------------------------------------------------------------------------


def _lib():
    from ..ops import native

    return native


def matmul_all_reduce(ex, op, a_vals, w_vals):
    ctx = runtime(ex).context(op.attrs["group"])
    out = _gemms_all_reduce(ctx, [(a_vals[0], w_vals[0])])
    return NotImplemented if out is None else [out]


# From this group size on, an all-reduce is done as reduce-scatter epilogue + all-gather: pushing every tile to all ranks
# (`multimem.red`) makes each GPU receive world x the output, the reduce-scatter form (world - 1) / world of it.
_RS_AG_FROM_WORLD = int(os.environ.get("XL_RS_AG_FROM_WORLD", "4"))


# GEMM + all-reduce by pulling (NVSwitch adds the ranks' partial tiles on the way into the rank that owns the rows, which
# multicasts the sums): the form used from this group size on; XL_AR_PULL=0 switches it off, XL_AR_PULL_CTAS sets the
# number of CTAs that only reduce
_AR_PULL = os.environ.get("XL_AR_PULL", "1") != "0"
_AR_PULL_FROM_WORLD = int(os.environ.get("XL_AR_PULL_FROM_WORLD", "2"))
_AR_PULL_CTAS = int(os.environ.get("XL_AR_PULL_CTAS", "8"))


def _pull_buffers(ctx: GroupContext, M: int, N: int, dtype):
    """Arena buffers of the pull all-reduce for one output shape: the partial-product buffer, a ring of two result
    buffers, and the flag words with their address on every rank."""
    cache = ctx.__dict__.setdefault("_pull", {})
    key = (M, N, dtype)
    if key not in cache:
        partial = ctx.arena.alloc((M, N), dtype)
        results = [ctx.arena.alloc((M, N), dtype) for _ in range(2)]
        tiles = (M // 128) * (-(-N // 128))  # enough for either tile width of the kernel
        flags = ctx.arena.alloc((2 * tiles,), torch.int32)
        flags.zero_()
        torch.cuda.synchronize(flags.device)
        torch.distributed.barrier(group=ctx.pg)  # nobody signals into flag words that are not zeroed yet
        cache[key] = {"partial": partial, "results": results, "flags": _peer_ptr_tensor(ctx, flags), "pos": 0}
    return cache[key]


def gemm_all_reduce_pull(ctx: GroupContext, pairs, n_red: Optional[int] = None, timestamps=None):
    """`all_reduce(sum of a @ w over pairs)` (one or two pairs) as one pulling kernel; the result lives in a ring of two
    arena buffers (valid until the second next call with the same shape). NotImplemented if unsupported."""
    nat = _lib()
    a0, w0 = pairs[0]
    M, N = a0.shape[0], w0.shape[-1]
    if not ctx.arena.mc_base or M % (128 * ctx.world) or N % 8 or a0.dtype not in (torch.bfloat16, torch.float16):
        return NotImplemented
    buf = _pull_buffers(ctx, M, N, a0.dtype)
    result = buf["results"][buf["pos"]]
    res = nat.gemm_all_reduce_pull(pairs, ctx, buf["partial"], result, buf["flags"],
                                   n_red=_AR_PULL_CTAS if n_red is None else n_red, timestamps=timestamps)
    if res is NotImplemented:
        return NotImplemented
    buf["pos"] ^= 1
    return result


def _gemms_all_reduce(ctx: GroupContext, pairs):
    """`all_reduce(sum of a @ w over pairs)` with the reduction fused into the GEMM; None if unsupported."""
    nat = _lib()
    a0, w0 = pairs[0]
    M, N = a0.shape[0], w0.shape[-1]
    if ctx.world == 1 or N % 8 or a0.dtype not in (torch.bfloat16, torch.float16):
        return None
    if any(a.dtype != a0.dtype or a.shape[0] != M or w.shape[-1] != N for a, w in pairs):
        return None
    if _AR_PULL and _MC_ALL_REDUCE and ctx.world >= _AR_PULL_FROM_WORLD and len(pairs) <= 2:
        out = gemm_all_reduce_pull(ctx, pairs)
        if out is not NotImplemented:
            return out.clone()  # the ring buffer is reused two calls later; the graph may keep this value longer
    if ctx.world >= _RS_AG_FROM_WORLD and M % ctx.world == 0:
        # every tile is added into the shard of the rank that owns its rows, then the shards are gathered
        shard = ctx.arena.ring((M // ctx.world, N), a0.dtype)
        shard.zero_()
        dst = _peer_ptr_tensor(ctx, shard)
        for i, (a, w) in enumerate(pairs):
            if nat.gemm(a, w, out=shard, accumulate=4, comm=ctx, rs_dst=dst) is NotImplemented:
                if i:
                    raise RuntimeError("a GEMM of a fused group was rejected after an earlier one ran")
                return None
        out = torch.empty((M, N), dtype=a0.dtype, device=a0.device)
        torch.distributed.all_gather_into_tensor(out, shard, group=ctx.pg)
        return out
    if not _MC_ALL_REDUCE or not ctx.arena.mc_base:
        return None
    out = ctx.arena.ring((M, N), a0.dtype)
    out.zero_()
    for i, (a, w) in enumerate(pairs):
        if nat.gemm(a, w, out=out, accumulate=3, comm=ctx) is NotImplemented:
            if i:
                raise RuntimeError("a GEMM of a fused group was rejected after an earlier one ran")
            return None
    return out.clone()


def matmul2_all_reduce(ex, op, a1_vals, w1_vals, a2_vals, w2_vals):
    """`all_reduce(a1 @ w1 + a2 @ w2)`: both GEMMs reduce into the same zeroed output from their epilogues."""
    ctx = runtime(ex).context(op.attrs["group"])
    out = _gemms_all_reduce(ctx, [(a1_vals[0], w1_vals[0]), (a2_vals[0], w2_vals[0])])
    return NotImplemented if out is None else [out]


def gemm_reduce_scatter_pull(ctx: GroupContext, pairs, n_red: Optional[int] = None):
    """Rows `[rank*M/world, (rank+1)*M/world)` of `sum over ranks (sum of a @ w over pairs)` as one pulling kernel: the
    partial products stay in each rank's buffer, the owner of a row block adds the ranks' copies inside NVSwitch
    (`multimem.ld_reduce`) and keeps the sums. Returns a fresh `(M / world, N)` tensor or NotImplemented."""
    nat = _lib()
    a0, w0 = pairs[0]
    M, N = a0.shape[0], w0.shape[-1]
    if not ctx.arena.mc_base or M % (128 * ctx.world) or N % 8 or a0.dtype not in (torch.bfloat16, torch.float16):
        return NotImplemented
    buf = _pull_buffers(ctx, M, N, a0.dtype)
    out = torch.empty((M // ctx.world, N), dtype=a0.dtype, device=a0.device)
    res = nat.gemm_all_reduce_pull(pairs, ctx, buf["partial"], out, buf["flags"],
                                   n_red=_AR_PULL_CTAS if n_red is None else n_red, scatter=True)
    return out if res is not NotImplemented else NotImplemented


def matmuls_reduce_scatter(ex, op, *vals):
    """`reduce_scatter(a1 @ w1 [+ a2 @ w2])` over the rows as one kernel: pulling (NVSwitch adds the partial tiles on the
    way into the owner of the rows) where multicast is available, else every GEMM's epilogue adds its tiles into the
    owner's shard (`red.add` over NVLink). Returns the flat shard."""
    nat = _lib()
    ctx = runtime(ex).context(op.attrs["group"])
    pairs = [(vals[i][0], vals[i + 1][0]) for i in range(0, len(vals), 2)]
    a0, w0 = pairs[0]
    M, N = a0.shape[0], w0.shape[-1]
    if ctx.world == 1 or M % ctx.world or N % 8 or a0.dtype not in (torch.bfloat16, torch.float16):
        return NotImplemented
    if _AR_PULL and _MC_ALL_REDUCE and len(pairs) <= 2:
        out = gemm_reduce_scatter_pull(ctx, pairs)
        if out is not NotImplemented:
            return [out.reshape(-1)]
    shard = ctx.arena.ring((M // ctx.world, N), a0.dtype)
    shard.zero_()
    dst = _peer_ptr_tensor(ctx, shard)
    for i, (a, w) in enumerate(pairs):
        if nat.gemm(a, w, out=shard, accumulate=4, comm=ctx, rs_dst=dst) is NotImplemented:
            if i:
                raise RuntimeError("a GEMM of a fused group was rejected after an earlier one ran")
            return NotImplemented
    return [shard.reshape(-1).clone()]


def all_gather_multicast(ctx: GroupContext, shard: torch.Tensor) -> Optional[torch.Tensor]:
    """All-gather of equally sized 16-byte-multiple shards along the first axis: every rank multicasts its shard into the
    full buffer of all ranks (`multimem.st`), one kernel including the closing barrier. The result lives in a ring of two
    arena buffers (valid until the second next gather of the same shape). None if unsupported."""
    nat = _lib()
    nbytes = shard.numel() * shard.element_size()
    if not ctx.arena.mc_base or not _MC_ALL_REDUCE or nbytes % 16 or not shard.is_contiguous() or shard.data_ptr() % 16:
        return None
    full = ctx.arena.ring((shard.shape[0] * ctx.world, *shard.shape[1:]), shard.dtype)
    state = ctx.arena.local_sync[12:13]
    rc = nat._symm_all_gather_mc(shard.data_ptr(), ctx.arena.multicast_ptr(full), nbytes, state.data_ptr(),
                                 ctx.arena.pads_dev.data_ptr(), ctx.rank, ctx.world, 3, ctx.err.data_ptr(), nat._stream())
    if rc == -1:
        return None
    nat._check(rc, "symm_all_gather_mc")
    nat._count("symm_all_gather_mc")
    return full


def all_gather_matmul(ex, op, hs_vals, w_vals):
    """`all_gather(h_s) @ w`. Returns `(product, gathered operand)`. Where multicast is available the rows are gathered by
    one multicast kernel (each rank stores its rows into every rank's buffer) and the product is a plain GEMM; else the
    GEMM's copy CTAs pull the peers' rows into this rank's full-size operand while its other CTAs start on the local
    rows."""
    nat = _lib()
    ctx = runtime(ex).context(op.attrs["group"])
    h_s, w = hs_vals[0], w_vals[0]
    rows, k = h_s.shape
    if ctx.world == 1 or h_s.dtype not in (torch.bfloat16, torch.float16) or w.dtype != h_s.dtype:
        return NotImplemented
    full = all_gather_multicast(ctx, h_s) if _AR_PULL else None
    if full is not None:
        y = nat.gemm(full, w)
        if y is NotImplemented:
            return NotImplemented
        return [y], [full.clone()]  # the ring buffer is reused two gathers later; the graph keeps this value longer
    if rows % 128:
        return NotImplemented
    full, own = gathered_operand(ctx, rows * ctx.world, k, h_s.dtype, 128, "sp")
    own.copy_(h_s)
    y = all_gather_gemm(ctx, full, w, sharded="a")
    if y is NotImplemented:
        return NotImplemented
    return [y], [full.clone()]


def _peer_ptr_tensor(ctx: GroupContext, t: torch.Tensor) -> torch.Tensor:
    """int64 device tensor with the address of arena tensor `t` in every rank's memory (cached per buffer)."""
    cache = ctx.__dict__.setdefault("_peer_ptr_cache", {})
    key = t.data_ptr()
    if key not in cache:
        cache[key] = torch.tensor(ctx.arena.peer_ptrs(t), dtype=torch.int64, device=t.device)
    return cache[key]


def gemm_reduce_scatter(ctx: GroupContext, a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                        zero: bool = True):
    """Rows `[rank*M/world, (rank+1)*M/world)` of `sum over ranks (a @ w)`, one kernel: every finished tile is added
    (`red.add` over NVLink) into the output shard of the rank that owns its rows. `out` (default: a ring buffer of the
    group's arena) must live in the arena; with `zero=False` the caller has zeroed it (or wants to add to it: several
    GEMMs may reduce into the same shard). Returns the shard (valid once the kernel has finished) or NotImplemented."""
    nat = _lib()
    M, N = a.shape[0], w.shape[-1]
    if ctx.world == 1 or M % ctx.world or N % 8 or a.dtype not in (torch.bfloat16, torch.float16):
        return NotImplemented
    if out is None:
        out = ctx.arena.ring((M // ctx.world, N), a.dtype)
    if zero:
        out.zero_()
    res = nat.gemm(a, w, out=out, accumulate=4, comm=ctx, rs_dst=_peer_ptr_tensor(ctx, out))
    return out if res is not NotImplemented else NotImplemented


def gathered_operand(ctx: GroupContext, rows: int, cols: int, dtype, block_rows: int, name: str = ""):
    """Arena matrix `(rows, cols)` for an operand that is row-sharded over the group: returns `(full, own)` where
    `own` is the view of this rank's row range. `rows / world` must be a multiple of `block_rows` (128 for the left
    operand, 64 for the right operand of the GEMM that gathers it)."""
    if rows % (ctx.world * block_rows):
        raise ValueError(f"{rows} rows cannot be split into {ctx.world} shards of whole {block_rows}-row blocks")
    cache = ctx.__dict__.setdefault("_gathered", {})
    key = (rows, cols, dtype, name)
    if key not in cache:
        cache[key] = ctx.arena.alloc((rows, cols), dtype)
    full = cache[key]
    per = rows // ctx.world
    return full, full[ctx.rank * per:(ctx.rank + 1) * per]


def all_gather_gemm(ctx: GroupContext, a_full: torch.Tensor, b: torch.Tensor, sharded: str = "a", n_copy: int = 16,
                    **gemm_kwargs):
    """`a_full @ b` where one operand is row-sharded over the group and only this rank's rows are present at launch
    (`sharded="a"`: `a_full (M, K)` split over M; `sharded="b"`: `b (K, N)` split over K, e.g. a weight whose shards
    live on the ranks of a data-parallel group). The kernel's copy CTAs pull the remote row blocks over NVLink while its
    GEMM CTAs work on the local rows first; afterwards the gathered operand is complete in this rank's memory."""
    nat = _lib()
    op = a_full if sharded == "a" else b
    if ctx.world == 1 or not ctx.arena.contains(op) or not op.is_contiguous():
        return NotImplemented
    block_rows = 128 if sharded == "a" else 64
    if op.shape[0] % (ctx.world * block_rows):
        return NotImplemented
    bps = op.shape[0] // ctx.world // block_rows
    flags = ctx.__dict__.get("_gather_flags")
    if flags is None:
        flags = ctx._gather_flags = torch.zeros(4096, dtype=torch.int32, device=op.device)
    if ctx.world * bps > flags.numel():
        return NotImplemented
    flags[:ctx.world * bps].zero_()
    res = nat.gemm(a_full, b, comm=ctx, gather=(1 if sharded == "a" else 2, _peer_ptr_tensor(ctx, op), flags, bps, n_copy),
                   **gemm_kwargs)
    return res


def small_all_reduce(ctx: GroupContext, t: torch.Tensor, op: str) -> Optional[torch.Tensor]:
    """fp32 add / max all-reduce of at most 64 KiB through peer loads (one kernel, two signal rounds)."""
    nat = _lib()
    n = t.numel()
    if t.dtype != torch.float32 or n > _SMALL_ALL_REDUCE_ELEMS or op not in ("add", "max") or ctx.world == 1:
        return None
    ctx.stage[:n].copy_(t.reshape(-1))
    out = torch.empty_like(t)
    off = ctx.arena.offset_of(ctx.stage) // 4
    rc = nat._symm_all_reduce(ctx.arena.bases_dev.data_ptr(), ctx.arena.pads_dev.data_ptr(), off, out.data_ptr(), n,
                              0 if op == "add" else 1, ctx.rank, ctx.world, 2, ctx.err.data_ptr(), nat._stream())
    nat._check(rc, "symm_all_reduce")
    nat._count("symm_all_reduce")
    return out


def small_all_reduce_16bit(ctx: GroupContext, t: torch.Tensor) -> Optional[torch.Tensor]:
    """Sum all-reduce of a small bf16/fp16 tensor (decode-step activations): every rank stages its input in symmetric
    memory and reads the sum of all replicas with `multimem.ld_reduce` (fp32 accumulation inside NVSwitch). One kernel
    (staging copy included), one signal round."""
    nat = _lib()
    nbytes = t.numel() * 2
    if t.dtype not in (torch.bfloat16, torch.float16) or nbytes > _SMALL_ALL_REDUCE_16BIT_BYTES or nbytes % 16 \
            or ctx.world == 1 or not ctx.arena.mc_base or t.data_ptr() % 16:
        return None
    out = torch.empty_like(t)
    state = ctx.arena.local_sync[4:6]
    rc = nat._symm_all_reduce_mc(t.data_ptr(), ctx.stage16.data_ptr(), ctx.arena.multicast_ptr(ctx.stage16),
                                 _SMALL_ALL_REDUCE_16BIT_BYTES, state.data_ptr(), ctx.arena.pads_dev.data_ptr(),
                                 out.data_ptr(), nbytes, nat._CODE[t.dtype], ctx.rank, ctx.world, 16, ctx.err.data_ptr(),
                                 nat._stream())
    if rc == -1:
        return None
    nat._check(rc, "symm_all_reduce_mc")
    nat._count("symm_all_reduce_mc")
    return out


class FusedComm(DistComm):
    """NCCL transport with small reductions served by the one-shot NVLink kernels."""

    def __init__(self, num_replicas: int, device: torch.device, session, devices_per_replica: int = 1):
        super().__init__(num_replicas, device, devices_per_replica)
        self._session = session

    def all_reduce(self, vals, grouping, op, inplace=False, async_ok=False):
        t = vals[0]
        if t.dtype == torch.float32 and t.numel() <= _SMALL_ALL_REDUCE_ELEMS and op in ("add", "max") \
                and grouping.group_size > 1 and t.is_contiguous():
            ctx = runtime(self._session).context(grouping)
            out = small_all_reduce(ctx, t, op)
            if out is not None:
                if inplace:
                    t.copy_(out)
                    return [t]
                return [out]
        if t.dtype in (torch.bfloat16, torch.float16) and op == "add" and grouping.group_size > 1 \
                and t.is_contiguous() and t.numel() * 2 <= _SMALL_ALL_REDUCE_16BIT_BYTES and _MC_ALL_REDUCE:
            ctx = runtime(self._session).context(grouping)
            out = small_all_reduce_16bit(ctx, t)
            if out is not None:
                if inplace:
                    t.copy_(out)
                    return [t]
                return [out]
        return super().all_reduce(vals, grouping, op, inplace, async_ok)


def _fused_all_gather(self, vals, grouping):
    """`DistComm.all_gather` served by the multicast kernel where it applies."""
    t = vals[0]
    if grouping.group_size > 1 and _AR_PULL and t.is_cuda:
        ctx = runtime(self._session).context(grouping)
        flat = t.reshape(-1).contiguous()
        full = all_gather_multicast(ctx, flat)
        if full is not None:
            return [full.clone()]
    return DistComm.all_gather(self, vals, grouping)


FusedComm.all_gather = _fused_all_gather


def group_barrier(ctx: GroupContext, channel: int = 4):
    nat = _lib()
    nat._check(nat._symm_barrier(ctx.arena.pads_dev.data_ptr(), ctx.rank, ctx.world, channel, ctx.err.data_ptr(),
                                 nat._stream()), "symm_barrier")
    nat._count("symm_barrier")


def rts_adam(ex, op, w_vals, acc_vals, master_vals, m_vals, v_vals, step_vals):
    """One kernel: reduce-scatter of the gradient accumulators + AdamW on the local shard + all-gather of the new
    16-bit weights, over peer pointers. Needs the weight and the accumulator in this group's symmetric arena."""
    nat = _lib()
    a = op.attrs
    ctx = runtime(ex).context(a["group"])
    w, acc, master, m, v, step = w_vals[0], acc_vals[0], master_vals[0], m_vals[0], v_vals[0], step_vals[0]
    if ctx.world == 1 or ctx.world > 8:
        return NotImplemented
    if not (ctx.arena.contains(w) and ctx.arena.contains(acc)):
        return NotImplemented
    if w.dtype not in (torch.bfloat16, torch.float16) or acc.dtype != torch.float32 or v.dtype != torch.float32 \
            or master.dtype != torch.float32 or step.dtype != torch.float32:
        return NotImplemented
    shard_n = master.numel()
    if shard_n % 4 or shard_n * ctx.world != w.numel():
        return NotImplemented
    grads = (ctypes.c_void_p * ctx.world)(*ctx.arena.peer_ptrs(acc))
    weights = (ctypes.c_void_p * ctx.world)(*ctx.arena.peer_ptrs(w))
    if a["sync_before"]:
        group_barrier(ctx, 4)
    rc = nat._rts_adam(grads, weights, nat._CODE[w.dtype], master.data_ptr(), m.data_ptr(), nat._CODE[m.dtype],
                       v.data_ptr(), step.data_ptr(), ctx.rank * shard_n, shard_n, ctx.world, a["lr"], a["beta1"],
                       a["beta2"], a["eps"], a["weight_decay"], a["grad_scale"], int(a["bias_correction"]),
                       nat._stream())
    if rc == -1:
        return NotImplemented
    nat._check(rc, "rts_adam")
    nat._count("rts_adam")
    if a["sync_after"]:
        group_barrier(ctx, 5)
    return True


def _rts_bucket_table(ctx: GroupContext, key, ws, accs, masters, ms, vs, decays):
    """Device table of the bucket's segments (64 bytes each, see RtsSegment in csrc/comm.cu), built once per op."""
    import struct

    cache = ctx.__dict__.setdefault("_rts_tables", {})
    if key in cache:
        return cache[key]
    blob, chunk = b"", 0
    for w, acc, master, m, v, decay in zip(ws, accs, masters, ms, vs, decays):
        shard_n = master.numel()
        blob += struct.pack("<qqQQQqqfi", ctx.arena.offset_of(acc), ctx.arena.offset_of(w), master.data_ptr(),
                            m.data_ptr(), v.data_ptr(), ctx.rank * shard_n, shard_n, float(decay), chunk)
        chunk += -(-shard_n // 4096)
    table = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(ws[0].device)
    nat = _lib()
    grid = nat._rts_multi_grid(chunk)
    entry = {"table": table, "chunks": chunk, "partials": torch.zeros(grid, dtype=torch.float32, device=ws[0].device),
             "keep": (ws, accs, masters, ms, vs)}
    cache[key] = entry
    return entry


def _rts_bucket_ok(ctx, ws, accs, masters, ms, vs):
    if ctx.world == 1 or ctx.world > 64:
        return False
    m_dtype = ms[0].dtype
    for w, acc, master, m, v in zip(ws, accs, masters, ms, vs):
        if not (ctx.arena.contains(w) and ctx.arena.contains(acc)):
            return False
        if w.dtype != ws[0].dtype or w.dtype not in (torch.bfloat16, torch.float16) or acc.dtype != torch.float32 \
                or v.dtype != torch.float32 or master.dtype != torch.float32 or m.dtype != m_dtype:
            return False
        if master.numel() % 4 or master.numel() * ctx.world != w.numel() or not (w.is_contiguous() and acc.is_contiguous()):
            return False
    return True


def rts_reduce_bucket(ex, op, acc_vals):
    """Mode 1 of the bucket kernel: group mean of every accumulator into its owned range + sum of squares."""
    nat = _lib()
    a = op.attrs
    ctx = runtime(ex).context(a["group"])
    accs = [v[0] for v in acc_vals]
    if ctx.world == 1 or any(not ctx.arena.contains(t) or t.dtype != torch.float32 or t.numel() % (4 * ctx.world)
                             for t in accs):
        return NotImplemented
    import struct

    cache = ctx.__dict__.setdefault("_rts_tables", {})
    key = ("reduce", op.uid)
    if key not in cache:
        blob, chunk = b"", 0
        for acc in accs:
            shard_n = acc.numel() // ctx.world
            blob += struct.pack("<qqQQQqqfi", ctx.arena.offset_of(acc), 0, 0, 0, 0, ctx.rank * shard_n, shard_n, 0.0, chunk)
            chunk += -(-shard_n // 4096)
        cache[key] = {"table": torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(accs[0].device), "chunks": chunk,
                      "partials": torch.zeros(nat._rts_multi_grid(chunk), dtype=torch.float32, device=accs[0].device)}
    e = cache[key]
    sumsq = torch.zeros((), dtype=torch.float32, device=accs[0].device)
    if a["sync_before"]:
        group_barrier(ctx, 4)
    rc = nat._rts_adam_multi(e["table"].data_ptr(), len(accs), e["chunks"], ctx.arena.bases_dev.data_ptr(), ctx.rank,
                             ctx.world, 1, nat.BF16, nat.F32, None, None, e["partials"].data_ptr(), sumsq.data_ptr(),
                             0.0, 0.0, 0.0, 0.0, a["grad_scale"], 0, nat._stream())
    nat._check(rc, "rts_adam_multi")
    nat._count("rts_reduce_bucket")
    return [sumsq]


def rts_adam_bucket(ex, op, w_vals, acc_vals, master_vals, m_vals, v_vals, step_vals, scale_vals):
    """One launch for the whole bucket: gradient reduce-scatter + AdamW on the owned ranges + all-gather of the new
    16-bit weights (or, after `rts_reduce_bucket`, AdamW + all-gather from the already reduced gradients)."""
    nat = _lib()
    a = op.attrs
    ctx = runtime(ex).context(a["group"])
    ws, accs, masters, ms, vs = ([v[0] for v in vals] for vals in (w_vals, acc_vals, master_vals, m_vals, v_vals))
    step = step_vals[0]
    if not _rts_bucket_ok(ctx, ws, accs, masters, ms, vs) or step.dtype != torch.float32:
        return NotImplemented
    e = _rts_bucket_table(ctx, ("adam", op.uid), ws, accs, masters, ms, vs, a["weight_decays"])
    scale = scale_vals[0] if scale_vals is not None else None
    if scale is not None and (scale.dtype != torch.float32 or scale.numel() != 1):
        return NotImplemented
    if a["sync_before"]:
        group_barrier(ctx, 4)
    rc = nat._rts_adam_multi(e["table"].data_ptr(), len(ws), e["chunks"], ctx.arena.bases_dev.data_ptr(), ctx.rank,
                             ctx.world, 2 if a["reduced"] else 0, nat._CODE[ws[0].dtype], nat._CODE[ms[0].dtype],
                             step.data_ptr(), scale.data_ptr() if scale is not None else None, None, None, a["lr"],
                             a["beta1"], a["beta2"], a["eps"], a["grad_scale"], int(a["bias_correction"]), nat._stream())
    if rc == -1:
        return NotImplemented
    nat._check(rc, "rts_adam_multi")
    nat._count("rts_adam_bucket")
    if a["sync_after"]:
        group_barrier(ctx, 5)
    return True


def layer_norm_distributed_fwd(ex, op, x_vals, w_vals, b_vals):
    """Hidden-sharded LayerNorm: local (sum, sum of squares) per row in one kernel, one small all-reduce over the group,
    normalisation with the group statistics in a second kernel."""
    nat = _lib()
    group = op.attrs["group"]
    for x, w, b in zip(x_vals, w_vals, b_vals):
        if x.dim() != 2 or not nat._ok(x, w, b) or w.dtype != x.dtype or b.dtype != x.dtype:
            return NotImplemented
    stats = [nat.row_sum_sumsq(x) for x in x_vals]
    stats = ex.comm.all_reduce(stats, group, "add", inplace=True)
    hidden = x_vals[0].shape[1] * group.group_size
    res = [nat.ln_apply_stats(x, st, w, b, hidden, op.attrs["eps"]) for x, st, w, b in zip(x_vals, stats, w_vals, b_vals)]
    return [r[0] for r in res], [r[1] for r in res], [r[2] for r in res]


def layer_norm_distributed_bwd(ex, op, x_vals, w_vals, mean_vals, rstd_vals, g_vals):
    """Backward of the hidden-sharded LayerNorm: per row the sums of `g*w` and `g*w*xhat` over the local columns in one
    kernel, one small all-reduce over the group, then `dx` and the (local) `dw`, `db` in a second kernel.
    Parity: popxl_addons/ops/layer_norm_distributed/layer_norm_distributedx.cpp:140-152."""
    nat = _lib()
    group = op.attrs["group"]
    for x, w, m, r, g in zip(x_vals, w_vals, mean_vals, rstd_vals, g_vals):
        if x.dim() != 2 or not nat._ok(x, w, g) or w.dtype != x.dtype or g.dtype != x.dtype \
                or m.dtype != torch.float32 or r.dtype != torch.float32 or x.shape[1] > 8192:
            return NotImplemented
    stats = [nat.ln_shard_bwd_stats(x, w, m, r, g) for x, w, m, r, g in zip(x_vals, w_vals, mean_vals, rstd_vals, g_vals)]
    stats = ex.comm.all_reduce(stats, group, "add", inplace=True)
    hidden = x_vals[0].shape[1] * group.group_size
    res = [nat.ln_shard_bwd_apply(x, w, m, r, g, st, hidden)
           for x, w, m, r, g, st in zip(x_vals, w_vals, mean_vals, rstd_vals, g_vals, stats)]
    if any(r is NotImplemented for r in res):
        return NotImplemented
    return [r[0] for r in res], [r[1] for r in res], [r[2] for r in res]


def _ce_group_stats(ex, group, logits, idx):
    """Per local replica: `(gmax, gsum, gpicked)` of the vocabulary-sharded rows. Two passes' worth of exchange: the
    row maxima (max over the group), then the rescaled sums and the picked logits (sum over the group)."""
    nat = _lib()
    stats = [nat.ce_shard_stats(l, i) for l, i in zip(logits, idx)]
    gmax = ex.comm.all_reduce([st[0].contiguous() for st in stats], group, "max")
    resc = [nat.ce_shard_rescale(st, gm) for st, gm in zip(stats, gmax)]
    resc = ex.comm.all_reduce(resc, group, "add", inplace=True)
    return [(gm, rs[0], rs[1]) for gm, rs in zip(gmax, resc)]


def _ce_operands_ok(logits, idx):
    nat = _lib()
    return all(l.dim() == 2 and nat._ok(l) and i.is_cuda and i.numel() == l.shape[0] for l, i in zip(logits, idx))


def ce_sharded_fwd(ex, op, logits, idx):
    """Vocabulary-sharded cross-entropy, forward: `(loss per row, negative log-softmax of the shard)`.
    Parity: popxl_addons/ops/cross_entropy_sharded_loss/crossentropyshardedx.cpp:88-214."""
    nat = _lib()
    if not _ce_operands_ok(logits, idx):
        return NotImplemented
    g = _ce_group_stats(ex, op.attrs["group"], logits, idx)
    res = [nat.ce_shard_nls(l, gm, gs, gp) for l, (gm, gs, gp) in zip(logits, g)]
    return [r[1] for r in res], [r[0] for r in res]


def ce_sharded_with_grad(ex, op, logits, idx, row_scale):
    """Loss per row and `d(loss * row_scale)/dlogits` of this shard without keeping the softmax: statistics pass, two
    small all-reduces, gradient pass."""
    nat = _lib()
    if not _ce_operands_ok(logits, idx):
        return NotImplemented
    row_scale = [rs.float().contiguous() for rs in row_scale]  # may arrive as a broadcast view of one scalar
    g = _ce_group_stats(ex, op.attrs["group"], logits, idx)
    res = [nat.ce_shard_grad_loss(l, gm, gs, gp, i, 0, rs) for l, i, rs, (gm, gs, gp) in zip(logits, idx, row_scale, g)]
    return [r[1] for r in res], [r[0] for r in res]


def ar_add_layer_norm(ex, op, x_vals, delta_vals, *rest):
    """All-reduce of the partial layer output + residual update + LayerNorm in one kernel (token-by-token decoding)."""
    nat = _lib()
    a = op.attrs
    ctx = runtime(ex).context(a["group"])
    x, delta = x_vals[0], delta_vals[0]
    rest = [r[0] for r in rest]
    bias = rest.pop(0) if a["has_bias"] else None
    w, b = rest
    if ctx.world == 1 or not _MC_ALL_REDUCE or not ctx.arena.mc_base or x.dim() != 2:
        return NotImplemented
    if x.dtype not in (torch.bfloat16, torch.float16) or not nat._ok(x, delta, bias, w, b):
        return NotImplemented
    if any(t is not None and t.dtype != x.dtype for t in (delta, bias, w, b)) or delta.shape != x.shape:
        return NotImplemented
    h = torch.empty_like(x)
    state = ctx.arena.local_sync[4:6]
    rc = nat._ar_add_ln(x.data_ptr(), delta.data_ptr(), bias.data_ptr() if bias is not None else None, w.data_ptr(),
                        b.data_ptr(), h.data_ptr(), x.shape[0], x.shape[1], float(a["eps"]), nat._CODE[x.dtype],
                        ctx.stage16.data_ptr(), ctx.arena.multicast_ptr(ctx.stage16), _SMALL_ALL_REDUCE_16BIT_BYTES,
                        state.data_ptr(), ctx.arena.pads_dev.data_ptr(), ctx.rank, ctx.world, 16, ctx.err.data_ptr(),
                        nat._stream())
    if rc == -1:
        return NotImplemented
    nat._check(rc, "ar_add_layer_norm")
    nat._count("ar_add_layer_norm")
    return [h]


# entries that only need `ex.comm` (no symmetric arena): also used when all replicas of a group live in this process
LOCAL_OK = {"layer_norm_distributed_fwd", "layer_norm_distributed_bwd", "ce_sharded_fwd", "ce_sharded_with_grad"}

_TABLE = {"matmul_all_reduce": matmul_all_reduce, "ar_add_layer_norm": ar_add_layer_norm,
          "layer_norm_distributed_fwd": layer_norm_distributed_fwd,
          "layer_norm_distributed_bwd": layer_norm_distributed_bwd,
          "ce_sharded_fwd": ce_sharded_fwd, "ce_sharded_with_grad": ce_sharded_with_grad,
          "matmuls_reduce_scatter": matmuls_reduce_scatter, "all_gather_matmul": all_gather_matmul, "matmul2_all_reduce": matmul2_all_reduce, "rts_adam": rts_adam,
          "rts_adam_bucket": rts_adam_bucket, "rts_reduce_bucket": rts_reduce_bucket}


def lookup(name: str, session):
    return _TABLE.get(name)
