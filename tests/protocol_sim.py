"""Discrete-event machinery for model checks of the kernels' barrier protocols.

mbarrier semantics modelled: a phase bit that flips when the expected number of arrivals is in;
``wait(parity)`` passes while the current phase bit differs from ``parity`` (so a waiter that falls
two phases behind blocks, as on the device).  Buffers are :class:`Resource` objects that assert that
nothing is overwritten while it is read and nothing is read before it is written.  The tensor cores
are an in-order queue; a commit arrives on its barrier when everything issued before it is done.
"""
import heapq
import random


class Sim:
    def __init__(self, seed):
        self.t = 0.0
        self.q = []
        self.n = 0
        self.rng = random.Random(seed)
        self.blocked = {}

    def at(self, dt, fn):
        self.n += 1
        heapq.heappush(self.q, (self.t + dt, self.n, fn))

    def run(self):
        while self.q:
            self.t, _, fn = heapq.heappop(self.q)
            fn()

    def lat(self, lo, hi):
        return self.rng.uniform(lo, hi)


class MBar:
    def __init__(self, sim, name, count):
        self.sim, self.name, self.count = sim, name, count
        self.phase, self.pending = 0, count
        self.waiters = []
        self.completed = 0

    def arrive(self):
        assert self.pending > 0
        self.pending -= 1
        if self.pending == 0:
            self.phase ^= 1
            self.completed += 1
            self.pending = self.count
            ws, self.waiters = self.waiters, []
            for parity, resume in ws:
                if self.phase != parity:
                    self.sim.at(self.sim.lat(0.01, 0.3), resume)
                else:
                    self.waiters.append((parity, resume))

    def wait(self, parity, resume):
        if self.phase != parity:
            self.sim.at(0.0, resume)
        else:
            self.waiters.append((parity, resume))


class Resource:
    """A buffer with one logical content per iteration."""

    def __init__(self, name, writers=1):
        self.name, self.writers = name, writers
        self.version, self.writing, self.readers = None, 0, 0
        self.w_done = 0
        self.w_version = None

    def write_begin(self, v):
        assert self.readers == 0, f"{self.name}: write of {v} while {self.readers} readers of {self.version} active"
        if self.writing == 0 and self.w_done == 0:
            self.w_version = v
        assert self.w_version == v, f"{self.name}: writers disagree ({self.w_version} vs {v})"
        self.writing += 1
        self.version = None

    def write_end(self, v):
        self.writing -= 1
        self.w_done += 1
        if self.w_done == self.writers:
            self.version, self.w_done = v, 0

    def read_begin(self, v):
        assert self.writing == 0 and self.version == v, \
            f"{self.name}: read of {v} but buffer holds {self.version} (writing={self.writing})"
        self.readers += 1

    def read_end(self):
        self.readers -= 1


class Task:
    """Runs a generator; it yields ('wait', bar, parity) | ('sleep', dt) | ('barrier', GroupBarrier)."""

    def __init__(self, sim, gen, name):
        self.sim, self.gen, self.name, self.done = sim, gen, name, False
        sim.at(0.0, self.step)

    def step(self):
        try:
            cmd = next(self.gen)
        except StopIteration:
            self.done = True
            return
        if cmd[0] == "wait":
            cmd[1].wait(cmd[2], self.step)
        elif cmd[0] == "sleep":
            self.sim.at(cmd[1], self.step)
        elif cmd[0] == "barrier":
            cmd[1].arrive(self.step)


class GroupBarrier:
    def __init__(self, sim, n):
        self.sim, self.n, self.waiting = sim, n, []

    def arrive(self, resume):
        self.waiting.append(resume)
        if len(self.waiting) == self.n:
            ws, self.waiting = self.waiting, []
            for w in ws:
                self.sim.at(self.sim.lat(0.0, 0.05), w)


class TensorQueue:
    """In-order queue of tensor-core work; a commit arrives when everything before it is done."""

    def __init__(self, sim):
        self.sim, self.free_at = sim, 0.0

    def op(self, dur, on_start, on_end):
        start = max(self.sim.t, self.free_at)
        self.free_at = start + dur
        self.sim.at(start - self.sim.t, on_start)
        self.sim.at(self.free_at - self.sim.t, on_end)

    def commit(self, bar):
        self.sim.at(max(self.free_at - self.sim.t, 0.0) + 1e-6, bar.arrive)
