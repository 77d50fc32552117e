"""Failure detection on the host.

* :class:`Heartbeat`: every rank bumps a counter in the job's key-value store between
  steps; a rank that stops (crashed, hung in host code, never joined) is reported by its
  peers *before* they launch their next collective, so nobody waits inside a kernel.
* :func:`terminate_job`: on an unrecoverable error (e.g. out of memory) a rank ends the
  processes of *this job only* -- the PIDs its ranks registered in the store -- with SIGINT.
  Every rank registers its host name and its process start time beside its PID; only entries of
  the calling host are signalled, and only while the PID still belongs to the process that
  registered it (a PID recycled for an unrelated process is left alone).  Ranks on other hosts
  are ended by their own host's ranks, which see the ``abort`` key at their next heartbeat check.
  (The reference kills every process whose command line matches the script name on every
  node through pdsh: benchmark/mist/exec/benchmark_one_case.py:434-441,
  mist/utils/common.py:631-656.)
* device side: every wait in the kernels is bounded and reports through a status word that
  ``mist_b200.ops.native.check_status`` turns into an exception.
"""
from __future__ import annotations

import os
import signal
import socket
import time
from typing import Dict, List, Optional, Tuple


def _start_time(pid: int) -> Optional[str]:
    """Start time of a process in clock ticks since boot (field 22 of /proc/<pid>/stat)."""
    try:
        with open(f"/proc/{pid}/stat") as f:
            return f.read().rsplit(")", 1)[1].split()[19]
    except (OSError, IndexError):
        return None


class Heartbeat:
    def __init__(self, store, rank: int, world: int, prefix: str = "hb", host: Optional[str] = None):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix
        self.host = host or socket.gethostname()
        self.count = 0
        pid = os.getpid()
        self.store.set(f"{prefix}/pid/{rank}", f"{pid}|{self.host}|{_start_time(pid) or ''}")
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
        if self.aborted():
            raise RuntimeError("another rank asked the job to stop")
        stale = self.stale_ranks(max_age_s)
        if stale:
            raise RuntimeError(f"ranks {stale} stopped responding (no heartbeat for {max_age_s:.0f} s)")

    def request_abort(self):
        self.store.set(f"{self.prefix}/abort", "1")

    def aborted(self) -> bool:
        try:
            return self.store.check([f"{self.prefix}/abort"])
        except Exception:
            return False

    def entries(self) -> Dict[int, Tuple[int, str, str]]:
        """rank -> (pid, host, start time) as registered by the ranks."""
        out = {}
        for r in range(self.world):
            try:
                if not self.store.check([f"{self.prefix}/pid/{r}"]):
                    continue
                pid, host, start = self.store.get(f"{self.prefix}/pid/{r}").decode().split("|")
                out[r] = (int(pid), host, start)
            except Exception:
                pass
        return out

    def pids(self) -> Dict[int, int]:
        return {r: e[0] for r, e in self.entries().items()}


def terminate_job(heartbeat: Heartbeat, include_self: bool = False, sig=signal.SIGINT) -> List[int]:
    """Marks the job as aborted in the store and signals the ranks registered **on this host**
    whose PID still belongs to the registering process.  Returns the ranks that were signalled."""
    heartbeat.request_abort()
    signalled = []
    for r, (pid, host, start) in heartbeat.entries().items():
        if r == heartbeat.rank and not include_self:
            continue
        if host != heartbeat.host:
            continue                      # another machine: that PID means nothing here
        if start and _start_time(pid) != start:
            continue                      # the PID now belongs to some other process
        try:
            os.kill(pid, sig)
            signalled.append(r)
        except (ProcessLookupError, PermissionError):
            pass
    return signalled
