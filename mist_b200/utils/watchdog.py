"""Failure detection on the host.

* :class:`Heartbeat`: every rank bumps a counter in the job's key-value store between
  steps; a rank that stops (crashed, hung in host code, never joined) is reported by its
  peers *before* they launch their next collective, so nobody waits inside a kernel.
* :func:`terminate_job`: on an unrecoverable error (e.g. out of memory) a rank ends the
  processes of *this job only* -- the PIDs its ranks registered in the store -- with SIGINT.
  (The reference kills every process whose command line matches the script name on every
  node through pdsh: benchmark/mist/exec/benchmark_one_case.py:434-441,
  mist/utils/common.py:631-656.)
* device side: every wait in the kernels is bounded and reports through a status word that
  ``mist_b200.ops.native.check_status`` turns into an exception.
"""
from __future__ import annotations

import os
import signal
import time
from typing import Dict, List, Optional


class Heartbeat:
    def __init__(self, store, rank: int, world: int, prefix: str = "hb"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix
        self.count = 0
        self.store.set(f"{prefix}/pid/{rank}", str(os.getpid()))
        self.beat()

    def beat(self):
        self.count += 1
        self.store.set(f"{self.prefix}/{self.rank}", f"{self.count}:{time.time():.3f}")

    def _read(self, r: int):
        try:
            c, t = self.store.get(f"{self.prefix}/{r}").decode().split(":")
            return int(c), float(t)
        except Exception:
            return 0, 0.0

    def stale_ranks(self, max_age_s: float, min_count: Optional[int] = None) -> List[int]:
        """Ranks whose last beat is older than ``max_age_s`` (or behind ``min_count``)."""
        now = time.time()
        out = []
        for r in range(self.world):
            if r == self.rank:
                continue
            c, t = self._read(r)
            if now - t > max_age_s or (min_count is not None and c < min_count):
                out.append(r)
        return out

    def check(self, max_age_s: float = 60.0):
        stale = self.stale_ranks(max_age_s)
        if stale:
            raise RuntimeError(f"ranks {stale} stopped responding (no heartbeat for {max_age_s:.0f} s)")

    def pids(self) -> Dict[int, int]:
        out = {}
        for r in range(self.world):
            try:
                out[r] = int(self.store.get(f"{self.prefix}/pid/{r}").decode())
            except Exception:
                pass
        return out


def terminate_job(heartbeat: Heartbeat, include_self: bool = False, sig=signal.SIGINT):
    """Signals the registered PIDs of this job's ranks on this host."""
    for r, pid in heartbeat.pids().items():
        if r == heartbeat.rank and not include_self:
            continue
        try:
            os.kill(pid, sig)
        except (ProcessLookupError, PermissionError):
            pass
