"""Host-side failure detection between the ranks of a job.

Every rank publishes a heartbeat (its last completed step) in the job's key-value store after each step and, before it
launches the next one, checks that all peers have reached the same step within a timeout. A rank that raised, exited or
hung on the host is therefore noticed *between* steps, before any kernel or collective that would wait for it has been
launched, and the survivors can stop cleanly (checkpoint, exit) instead of waiting inside a collective.
The reference has no equivalent (it relies on the launcher's process supervision); recovery is a restart from the
latest `TaskSession` checkpoint.
"""
import time
from typing import Iterable, Optional


class PeerLost(RuntimeError):
    def __init__(self, missing, step, waited):
        super().__init__(f"ranks {sorted(missing)} did not reach step {step} within {waited:.1f}s")
        self.missing, self.step = sorted(missing), step


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, prefix: str = "xl/heartbeat"):
        self.store, self.rank, self.world_size, self.prefix = store, rank, world_size, prefix

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self, step: int, status: str = "ok") -> None:
        """Publish that this rank finished `step` (or failed in it: `status="failed"`)."""
        self.store.set(self._key(self.rank), f"{step}:{status}")

    def _read(self, rank: int):
        try:
            if not self.store.check([self._key(rank)]):
                return -1, "ok"
            raw = self.store.get(self._key(rank)).decode()
            step, status = raw.split(":")
            return int(step), status
        except Exception:
            return -1, "ok"

    def check_peers(self, step: int, timeout: float = 10.0, poll: float = 0.05,
                    peers: Optional[Iterable[int]] = None) -> None:
        """Return once every peer has published `step` or later; raise `PeerLost` otherwise."""
        todo = set(range(self.world_size) if peers is None else peers) - {self.rank}
        t0 = time.monotonic()
        while todo:
            for r in list(todo):
                s, status = self._read(r)
                if status == "failed":
                    raise PeerLost({r}, step, time.monotonic() - t0)
                if s >= step:
                    todo.discard(r)
            if todo and time.monotonic() - t0 > timeout:
                raise PeerLost(todo, step, time.monotonic() - t0)
            if todo:
                time.sleep(poll)
