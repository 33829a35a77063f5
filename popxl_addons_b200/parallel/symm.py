"""Symmetric-memory arenas.

One arena per replica group (communicator): every rank allocates a buffer of the same size, the ranks exchange handles
once (`torch.distributed._symmetric_memory` does the CUDA VMM export / import and, where the fabric supports it, binds
an NVLS multicast address), and afterwards tensors are carved out of the arena with a bump allocator. Because all ranks
run the same program they allocate in the same order, so a tensor has the same offset on every rank and a peer's copy
lives at `peer_base + offset`: no further handshakes are needed.

The first 64 KiB of an arena hold the signal pad (flags written by peers) and a few words of local scratch for kernels.
"""
import os
from typing import Dict, List, Optional, Tuple

import torch

_ALIGN = 256
_HEADER = 64 * 1024
PAD_WORDS = 8 * 1024          # uint32 signal slots at the start of the header
LOCAL_SYNC_OFFSET = 48 * 1024  # byte offset of the kernels' local scratch words inside the header


_GUARD_BYTES = 256
_GUARD_PATTERN = 0xA5


class BumpAllocator:
    """Carves aligned tensors out of one byte buffer, in call order. With `guards`, a 256-byte canary block filled with
    a fixed pattern follows every allocation; `check_guards()` reads them back on the host and names the allocation
    whose canary was overwritten (a kernel wrote past the end of its buffer, on this rank or from a peer). Guards
    change the offsets, so either every rank of a group uses them or none (`XL_DEBUG_CANARIES=1` in the environment
    of all ranks)."""

    def __init__(self, buf: torch.Tensor, start: int = 0, guards: bool = False):
        if buf.dtype != torch.uint8 or buf.dim() != 1:
            raise TypeError("BumpAllocator takes a flat uint8 buffer")
        self.buf = buf
        self.nbytes = buf.numel()
        self.cursor = start
        self.guards = guards
        self.allocations: List[Tuple[int, int, tuple, torch.dtype]] = []  # (start, nbytes, shape, dtype)

    def alloc(self, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = self.cursor
        end = start + ((nbytes + _ALIGN - 1) // _ALIGN) * _ALIGN
        if self.guards:
            end += _GUARD_BYTES
        if end > self.nbytes:
            raise MemoryError(f"symmetric arena exhausted: need {end} bytes, have {self.nbytes}")
        self.cursor = end
        if self.guards:
            self.buf[start + nbytes:end].fill_(_GUARD_PATTERN)  # alignment slack and the canary block
            self.allocations.append((start, nbytes, tuple(shape), dtype))
        return self.buf[start:start + nbytes].view(dtype).view(tuple(shape))

    def check_guards(self) -> None:
        """Raise if any canary differs from the pattern. Synchronises with the device the buffer lives on."""
        if not self.guards:
            return
        for i, (start, nbytes, shape, dtype) in enumerate(self.allocations):
            end = start + ((nbytes + _ALIGN - 1) // _ALIGN) * _ALIGN + _GUARD_BYTES
            guard = self.buf[start + nbytes:end]
            bad = (guard != _GUARD_PATTERN).nonzero()
            if bad.numel():
                first = int(bad[0])
                raise RuntimeError(
                    f"buffer overrun: allocation #{i} ({tuple(shape)}, {dtype}, {nbytes} bytes at offset {start}) was "
                    f"written {first} byte(s) past its end ({int(bad.numel())} guard bytes changed)")


class SymmArena:
    def __init__(self, nbytes: int, pg, device: torch.device, use_multicast: Optional[bool] = None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        self.pg = pg
        self.device = device
        self.nbytes = _HEADER + ((int(nbytes) + _ALIGN - 1) // _ALIGN) * _ALIGN
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.hdl = symm_mem.rendezvous(self.buf, pg)
        self.rank = int(self.hdl.rank)
        self.world = int(self.hdl.world_size)
        self.base_ptrs: List[int] = [int(p) for p in self.hdl.buffer_ptrs]
        if use_multicast is None:
            use_multicast = os.environ.get("XL_NVLS", "1") != "0"
        mc = int(getattr(self.hdl, "multicast_ptr", 0) or 0)
        self.mc_base = mc if use_multicast else 0
        self.buf[:_HEADER].zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=pg)
        self.pads_dev = torch.tensor(self.base_ptrs, dtype=torch.int64, device=device)  # pad = start of each arena
        self.bases_dev = self.pads_dev
        self.local_sync = self.buf[LOCAL_SYNC_OFFSET:LOCAL_SYNC_OFFSET + 64].view(torch.int32)
        self._bump = BumpAllocator(self.buf, _HEADER, guards=os.environ.get("XL_DEBUG_CANARIES") == "1")
        self.epoch = 0
        self._rings: Dict[Tuple, List[torch.Tensor]] = {}
        self._ring_pos: Dict[Tuple, int] = {}

    # -- allocation ----------------------------------------------------------------------------------------------
    @property
    def cursor(self) -> int:
        return self._bump.cursor

    def alloc(self, shape, dtype: torch.dtype) -> torch.Tensor:
        return self._bump.alloc(shape, dtype)

    def check_guards(self) -> None:
        """With `XL_DEBUG_CANARIES=1`: verify the canary after every tensor of the arena (host read; synchronises)."""
        self._bump.check_guards()

    def ring(self, shape, dtype: torch.dtype, depth: int = 2) -> torch.Tensor:
        """Next buffer of a small ring of same-shaped arena tensors (outputs of fused collectives)."""
        key = (tuple(shape), dtype)
        if key not in self._rings:
            self._rings[key] = [self.alloc(shape, dtype) for _ in range(depth)]
            self._ring_pos[key] = 0
        i = self._ring_pos[key]
        self._ring_pos[key] = (i + 1) % len(self._rings[key])
        return self._rings[key][i]

    # -- addressing ----------------------------------------------------------------------------------------------
    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base_ptrs[self.rank]
        if not 0 <= off < self.nbytes:
            raise ValueError("tensor does not live in this arena")
        return off

    def contains(self, t: torch.Tensor) -> bool:
        off = t.data_ptr() - self.base_ptrs[self.rank]
        return 0 <= off < self.nbytes

    def peer_ptrs(self, t: torch.Tensor) -> List[int]:
        off = self.offset_of(t)
        return [b + off for b in self.base_ptrs]

    def multicast_ptr(self, t: torch.Tensor) -> int:
        return self.mc_base + self.offset_of(t) if self.mc_base else 0

    def next_epoch(self) -> int:
        self.epoch = (self.epoch + 1) & 0x7FFFFFFF or 1
        return self.epoch
