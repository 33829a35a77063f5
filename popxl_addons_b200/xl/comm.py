"""Communicators: how the replicas of a session exchange data.

* `SimComm` — all replicas live in this process (CPU tests, oracles): collectives are plain tensor arithmetic over
  the per-replica value lists.
* `DistComm` — one replica per process, one process per GPU: collectives go through `torch.distributed` process
  groups (NCCL over NVLink/NVSwitch on GPUs, gloo on CPU), one group per distinct rank list. The package's fused
  NVLink kernels plug in above this class for the hot paths; this class is the portable transport.

Every `(stride, size)` grouping is just a rank list on an NVSwitch box, so none of the orthogonal / consecutive /
masked special cases of popxl_addons/ops/replicated_strided_collectives/mgcl.cpp:210-293 exist here.
"""
from typing import Dict, List, Tuple

import torch

from .core import ReplicaGrouping


def _reduce(stack: torch.Tensor, op: str) -> torch.Tensor:
    if op == "add":
        return stack.sum(dim=0)
    if op == "mean":
        return stack.float().mean(dim=0).to(stack.dtype) if not stack.dtype.is_floating_point else stack.mean(dim=0)
    if op == "max":
        return stack.amax(dim=0)
    if op == "min":
        return stack.amin(dim=0)
    if op == "mul":
        return stack.prod(dim=0)
    raise ValueError(op)


def _pad_flat(t: torch.Tensor, size: int) -> Tuple[torch.Tensor, int]:
    flat = t.reshape(-1)
    n = -(-flat.numel() // size)
    if n * size != flat.numel():
        flat = torch.cat([flat, flat.new_zeros(n * size - flat.numel())])
    return flat, n


class SimComm:
    """All replicas in one process. `vals[r]` is replica r's tensor."""

    pending: Dict[int, tuple] = {}  # collectives in flight: always empty here (the simulation is synchronous)

    def __init__(self, num_replicas: int):
        self.num_replicas = num_replicas
        self.rank = 0
        self.world_size = 1

    def wait_all(self):
        pass

    def all_reduce(self, vals: List[torch.Tensor], grouping: ReplicaGrouping, op: str, inplace: bool = False,
                   async_ok: bool = False):
        out = list(vals)
        for members in grouping.groups:
            acc_dtype = torch.float32 if vals[members[0]].dtype in (torch.float16, torch.bfloat16) else None
            stack = torch.stack([vals[r].to(acc_dtype) if acc_dtype else vals[r] for r in members])
            red = _reduce(stack, op).to(vals[members[0]].dtype)
            for r in members:
                if inplace:
                    vals[r].copy_(red)
                    out[r] = vals[r]
                else:
                    out[r] = red.clone()
        return out

    def reduce_scatter(self, vals, grouping, op):
        out = [None] * len(vals)
        size = grouping.group_size
        for members in grouping.groups:
            padded = [_pad_flat(vals[r], size) for r in members]
            n = padded[0][1]
            stack = torch.stack([p[0].float() if p[0].dtype in (torch.float16, torch.bfloat16) else p[0]
                                 for p in padded])
            red = _reduce(stack, op).to(vals[members[0]].dtype)
            for i, r in enumerate(members):
                out[r] = red[i * n:(i + 1) * n].clone()
        return out

    def all_gather(self, vals, grouping):
        out = [None] * len(vals)
        for members in grouping.groups:
            cat = torch.cat([vals[r].reshape(-1) for r in members])
            for r in members:
                out[r] = cat.clone()
        return out

    def gather_to_host(self, vals: List[torch.Tensor]) -> List[torch.Tensor]:
        """Values of *all* replicas (list indexed by global replica), on the host."""
        return [v.detach().cpu() for v in vals]

    def barrier(self):
        pass


class DistComm:
    """One replica per process. `vals` always has length 1."""

    _REDUCE = {"add": "SUM", "max": "MAX", "min": "MIN", "mul": "PRODUCT", "mean": "SUM"}

    def __init__(self, num_replicas: int, device: torch.device, devices_per_replica: int = 1):
        import torch.distributed as dist

        if not dist.is_initialized():
            backend = "nccl" if device.type == "cuda" else "gloo"
            import datetime
            import os

            # a collective that waits longer than this ends with an error instead of blocking the job for good
            from .core import Options

            timeout = datetime.timedelta(seconds=float(Options.from_env().collective_timeout_s))
            dist.init_process_group(backend=backend, device_id=device if device.type == "cuda" else None,
                                    timeout=timeout)
        self.dist = dist
        self.world_rank = dist.get_rank()
        self.world_size = dist.get_world_size()
        self.slots = int(devices_per_replica)  # processes per replica (pipeline device slots)
        if num_replicas * self.slots != self.world_size:
            raise ValueError(f"replication_factor={num_replicas} x devices_per_replica={self.slots} must equal the "
                             f"number of processes {self.world_size}")
        self.rank = self.world_rank // self.slots  # replica index of this process
        self.slot = self.world_rank % self.slots
        self.num_replicas = num_replicas
        self._p2p: list = []
        self.device = device
        self._groups: Dict[tuple, object] = {}
        # all-reduces as asynchronous operations that overlap the ops issued after them (off by default)
        self.async_collectives = False
        self.pending: Dict[int, tuple] = {}

    def group_for(self, grouping: ReplicaGrouping):
        """Process group of this rank within `grouping` (creating, collectively, all groups of the grouping)."""
        key = tuple(tuple(g) for g in grouping.groups)
        if key not in self._groups:
            mine = None
            for members in grouping.groups:
                for slot in range(self.slots):  # the same slot of every member replica forms one process group
                    ranks = [m * self.slots + slot for m in members]
                    if len(ranks) == self.world_size:
                        pg = self.dist.group.WORLD
                    else:
                        pg = self.dist.new_group(ranks=ranks)
                    if self.rank in members and slot == self.slot:
                        mine = (pg, list(members))
            self._groups[key] = mine
        return self._groups[key]

    def all_reduce(self, vals, grouping, op, inplace=False, async_ok=False):
        """`async_ok`: the caller does not read the result itself (the executor joins the operation before the first op
        that does), so with `async_collectives` the all-reduce may stay in flight when this returns."""
        pg, members = self.group_for(grouping)
        t = vals[0] if inplace else vals[0].clone()
        if len(members) > 1:
            if async_ok and self.async_collectives and op != "mean":
                # issued on the library's own stream; the executor waits right before the first op that reads `t`
                work = self.dist.all_reduce(t, op=getattr(self.dist.ReduceOp, self._REDUCE[op]), group=pg, async_op=True)
                self.pending[id(t)] = (work, t)  # holding `t` keeps its id unique while the entry exists
                return [t]
            self.dist.all_reduce(t, op=getattr(self.dist.ReduceOp, self._REDUCE[op]), group=pg)
            if op == "mean":
                t.div_(len(members))
        return [t]

    def wait_all(self):
        """Join every collective still in flight (end of a run, end of a captured loop body)."""
        while self.pending:
            _, (work, _t) = self.pending.popitem()
            work.wait()

    # -- point-to-point between the device slots of one replica (pipeline stage boundaries) ------------------------
    def send_to_slot(self, t: torch.Tensor, slot: int):
        self._p2p.append(self.dist.P2POp(self.dist.isend, t.contiguous(), self.rank * self.slots + slot))

    def recv_from_slot(self, shape, dtype, slot: int) -> torch.Tensor:
        t = torch.empty(tuple(shape), dtype=dtype, device=self.device)
        self._p2p.append(self.dist.P2POp(self.dist.irecv, t, self.rank * self.slots + slot))
        return t

    def flush_p2p(self):
        """Issue all queued sends and receives as one batch (concurrent, so their order between ranks cannot deadlock).
        They run on the communication library's own stream: a received tensor is joined right before the first op that
        reads it (`pending`, as for asynchronous all-reduces), a send is joined at the end of the loop iteration or run
        (`wait_all`), so compute that does not depend on a transfer is not held up by it."""
        if self._p2p:
            ops, self._p2p = self._p2p, []
            works = self.dist.batch_isend_irecv(ops)
            if len(works) == len(ops):
                for w, o in zip(works, ops):
                    self.pending[id(o.tensor)] = (w, o.tensor)
            else:  # the batch came back as one coalesced work item (NCCL): every tensor of the batch waits on it
                for o in ops:
                    self.pending[id(o.tensor)] = (works[0], o.tensor)
                for w in works[1:]:
                    self.pending[id(w)] = (w, None)

    def reduce_scatter(self, vals, grouping, op):
        pg, members = self.group_for(grouping)
        size = len(members)
        flat, n = _pad_flat(vals[0], size)
        if size == 1:
            return [flat.clone()]
        out = flat.new_empty(n)
        self.dist.reduce_scatter_tensor(out, flat.contiguous(), op=getattr(self.dist.ReduceOp, self._REDUCE[op]),
                                        group=pg)
        if op == "mean":
            out.div_(size)
        return [out]

    def all_gather(self, vals, grouping):
        pg, members = self.group_for(grouping)
        flat = vals[0].reshape(-1).contiguous()
        if len(members) == 1:
            return [flat.clone()]
        out = flat.new_empty(flat.numel() * len(members))
        self.dist.all_gather_into_tensor(out, flat, group=pg)
        return [out]

    def gather_to_host(self, vals):
        """Values of all replicas (indexed by replica), on the host: gathered over the processes that hold the same
        device slot of every replica."""
        t = vals[0].detach().contiguous()
        pg, _ = self.group_for(ReplicaGrouping(self.num_replicas))
        out = [torch.empty_like(t) for _ in range(self.num_replicas)]
        if self.num_replicas > 1:
            self.dist.all_gather(out, t, group=pg)
        else:
            out = [t]
        return [o.cpu() for o in out]

    def send(self, t: torch.Tensor, dst: int):
        self.dist.send(t.contiguous(), dst)

    def recv(self, t: torch.Tensor, src: int):
        self.dist.recv(t, src)

    def barrier(self):
        self.dist.barrier()
