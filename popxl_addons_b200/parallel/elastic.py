"""Restart-from-checkpoint supervision of a multi-process job.

    python -m popxl_addons_b200.parallel.elastic --nproc 8 --max-restarts 3 train.py --my-args ...

starts one worker per rank (environment `RANK`, `LOCAL_RANK`, `WORLD_SIZE`, `MASTER_ADDR`, `MASTER_PORT`, like
`torchrun`, plus `XL_RESTART_COUNT`). When a worker ends with a non-zero status (it raised, or it stopped after
`parallel.health` reported a lost peer) the remaining workers are stopped, by their own process ids, and the whole job
is started again with a fresh rendezvous port, up to `max_restarts` times. A worker resumes from
`latest_checkpoint(root)`: the newest complete `TaskSession` checkpoint under `root`.

Workers are expected to leave between steps (no kernel or collective in flight): with `Heartbeat.check_peers` before
every step the survivors of a failure notice it on the host and exit by themselves; the supervisor's stop signal is only
the fallback. The reference has no counterpart: it relies on its launcher (`poprun`) and a manual restart from
`TaskSession.load_checkpoint` (popxl_addons/task_session.py:175-283).
"""
import argparse
import json
import os
import signal
import socket
import subprocess
import sys
import time
from typing import Dict, List, Optional, Sequence

__all__ = ["latest_checkpoint", "Supervisor", "main"]


def latest_checkpoint(root: str) -> Optional[str]:
    """The complete checkpoint under `root` (one directory per checkpoint) with the most steps: it must hold a
    `session_info.json` with a `steps` entry and a `model` directory. Directories still being written (no
    `session_info.json`, which is written last) are skipped. None if there is none."""
    best, best_steps = None, -1
    if not os.path.isdir(root):
        return None
    for name in sorted(os.listdir(root)):
        path = os.path.join(root, name)
        info = os.path.join(path, "session_info.json")
        if not (os.path.isdir(os.path.join(path, "model")) and os.path.isfile(info)):
            continue
        try:
            with open(info) as f:
                steps = int(json.load(f).get("steps", -1))
        except (OSError, ValueError, TypeError):
            continue  # truncated or unreadable: not a usable checkpoint
        if steps > best_steps:
            best, best_steps = path, steps
    return best


def _free_port(addr: str) -> int:
    with socket.socket() as s:
        s.bind((addr, 0))
        return s.getsockname()[1]


class Supervisor:
    def __init__(self, argv: Sequence[str], nproc: int, max_restarts: int = 3, master_addr: str = "127.0.0.1",
                 env: Optional[Dict[str, str]] = None, poll_s: float = 0.1, grace_s: float = 15.0,
                 log=lambda msg: print(msg, file=sys.stderr, flush=True)):
        """`argv`: the worker's command line after the interpreter (script and its arguments). `grace_s`: how long the
        other workers get to leave by themselves after one failed before they are signalled."""
        self.argv, self.nproc, self.max_restarts = list(argv), int(nproc), int(max_restarts)
        self.master_addr, self.env, self.poll_s, self.grace_s, self.log = master_addr, dict(env or {}), poll_s, grace_s, log
        self.attempts: List[List[int]] = []  # exit codes of every attempt

    def _spawn(self, attempt: int) -> List[subprocess.Popen]:
        port = _free_port(self.master_addr)
        procs = []
        for rank in range(self.nproc):
            e = dict(os.environ)
            e.update(self.env)
            e.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(self.nproc), LOCAL_WORLD_SIZE=str(self.nproc),
                     MASTER_ADDR=self.master_addr, MASTER_PORT=str(port), XL_RESTART_COUNT=str(attempt))
            procs.append(subprocess.Popen([sys.executable, *self.argv], env=e))
        return procs

    def _stop(self, procs: List[subprocess.Popen]) -> None:
        """Give the workers that still run `grace_s` to finish, then signal exactly those processes."""
        deadline = time.monotonic() + self.grace_s
        while any(p.poll() is None for p in procs) and time.monotonic() < deadline:
            time.sleep(self.poll_s)
        for sig, wait in ((signal.SIGTERM, 5.0), (signal.SIGKILL, 5.0)):
            alive = [p for p in procs if p.poll() is None]
            if not alive:
                return
            for p in alive:
                p.send_signal(sig)
            end = time.monotonic() + wait
            while any(p.poll() is None for p in alive) and time.monotonic() < end:
                time.sleep(self.poll_s)

    def run(self) -> int:
        """Run the job; returns 0 once an attempt ends with every worker at status 0, else the failing status of the
        last attempt."""
        code = 1
        for attempt in range(self.max_restarts + 1):
            procs = self._spawn(attempt)
            failed = None
            while failed is None and any(p.poll() is None for p in procs):
                for rank, p in enumerate(procs):
                    rc = p.poll()
                    if rc not in (None, 0):
                        failed = (rank, rc)
                        break
                else:
                    time.sleep(self.poll_s)
            if failed is None:
                failed = next(((r, p.returncode) for r, p in enumerate(procs) if p.returncode != 0), None)
            if failed is not None:
                self._stop(procs)
            self.attempts.append([p.returncode for p in procs])
            if failed is None:
                return 0
            code = failed[1] if failed[1] > 0 else 1
            left = self.max_restarts - attempt
            self.log(f"[elastic] attempt {attempt}: rank {failed[0]} ended with status {failed[1]}; "
                     + (f"restarting ({left} restart(s) left)" if left else "no restarts left"))
        return code


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m popxl_addons_b200.parallel.elastic", description=__doc__.split("\n")[0])
    ap.add_argument("--nproc", type=int, required=True, help="workers (one per GPU)")
    ap.add_argument("--max-restarts", type=int, default=3)
    ap.add_argument("--master-addr", default="127.0.0.1")
    ap.add_argument("--grace", type=float, default=15.0, help="seconds the surviving workers get to leave by themselves")
    ap.add_argument("script")
    ap.add_argument("script_args", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    return Supervisor([a.script, *a.script_args], a.nproc, a.max_restarts, a.master_addr, grace_s=a.grace).run()


if __name__ == "__main__":
    sys.exit(main())
