"""Timing helpers: host-clock and device-event timing of a callable, peak-memory sampling and the
mean / median / std summary the drivers print.

Reference: ``benchmark_func_walltime`` / ``benchmark_func_cuda_event`` (mist/utils/common.py:191-306),
``process_benchmarking_results`` (:535-571).  Differences: the device timer can flush the L2 cache
between repetitions (a buffer larger than L2 is rewritten), and both timers run on a machine without
a GPU (the device timer then falls back to the host clock), which is what the CPU tests use.
"""
from __future__ import annotations

import time
from typing import Callable, Optional, Sequence, Tuple

import numpy as np
import torch

MB = 1 << 20
_L2_FLUSH_BYTES = 256 << 20      # larger than the 126 MB L2 of a B200


def _call(func: Callable, prepare: Optional[Callable]):
    if prepare is None:
        return func()
    args, kwargs = prepare()
    return func(*args, **kwargs)


class _MemorySampler:
    """Peak allocated / reserved bytes of the first ``records`` timed calls (one value per call)."""

    def __init__(self, records: int):
        self.records = int(records) if torch.cuda.is_available() else 0
        self.allocated, self.reserved = [], []
        if self.records:
            torch.cuda.reset_peak_memory_stats()

    def sample(self):
        if len(self.allocated) < self.records:
            self.allocated.append(torch.cuda.max_memory_allocated())
            self.reserved.append(torch.cuda.max_memory_reserved())
            torch.cuda.reset_peak_memory_stats()

    def result(self) -> Tuple[np.ndarray, np.ndarray]:
        def uniq(v):
            return np.sort(np.unique(np.asarray(v, dtype=np.float64) / MB))
        return uniq(self.allocated), uniq(self.reserved)


def time_host(func: Callable, warmup: int, number: int, prepare: Optional[Callable] = None,
              sync: Optional[Callable] = None, memory_records: int = 0):
    """Seconds per call by ``time.perf_counter`` with ``sync()`` on both sides of every call.
    ``prepare()`` (untimed) returns ``(args, kwargs)`` for the call.  Returns
    ``(costs [number], (peak_allocated_MB, peak_reserved_MB))``."""
    sync = sync or (lambda: None)
    mem = _MemorySampler(memory_records)

    def once() -> float:
        inputs = prepare
        sync()
        t0 = time.perf_counter()
        _call(func, inputs)
        sync()
        dt = time.perf_counter() - t0
        mem.sample()
        return dt

    for _ in range(warmup):
        once()
    costs = np.array([once() for _ in range(number)], dtype=np.float64)
    return costs, mem.result()


def time_device(func: Callable, warmup: int, number: int, prepare: Optional[Callable] = None,
                memory_records: int = 0, flush_l2: bool = False):
    """Seconds per call by CUDA events on the current stream (one synchronize at the end, so
    consecutive calls queue back to back unless ``flush_l2`` separates them).  Without a GPU this is
    :func:`time_host`."""
    if not torch.cuda.is_available():
        return time_host(func, warmup, number, prepare, None, memory_records)
    mem = _MemorySampler(memory_records)
    flush = torch.empty(_L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda") if flush_l2 else None
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(number)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(number)]

    def once(i: int):
        if flush is not None:
            flush.zero_()
        if i >= 0:
            starts[i].record()
        _call(func, prepare)
        if i >= 0:
            ends[i].record()
        mem.sample()

    for _ in range(warmup):
        once(-1)
    for i in range(number):
        once(i)
    torch.cuda.synchronize()
    costs = np.array([s.elapsed_time(e) / 1e3 for s, e in zip(starts, ends)], dtype=np.float64)
    return costs, mem.result()


def format_time(seconds: float) -> str:
    for unit, scale in (("s", 1.0), ("ms", 1e-3), ("us", 1e-6)):
        if abs(seconds) >= scale:
            return f"{seconds / scale:.4f} {unit}"
    return f"{seconds / 1e-9:.4f} ns"


def format_size(num_bytes: float) -> str:
    for unit, scale in (("GB", 1 << 30), ("MB", 1 << 20), ("KB", 1 << 10)):
        if abs(num_bytes) >= scale:
            return f"{num_bytes / scale:.2f} {unit}"
    return f"{num_bytes:.0f} B"


def summarize(costs: Sequence[float], label: str = "", log: Optional[Callable] = None) -> Tuple[float, float, float]:
    """``(mean, median, std)`` of the measured costs; ``log`` (e.g. ``print``) gets one line."""
    c = np.asarray(costs, dtype=np.float64)
    mean, median, std = float(c.mean()), float(np.median(c)), float(c.std())
    if log is not None:
        head = f"[{label}]\t" if label else ""
        log(f"{head}Median: {format_time(median)}, Mean: {format_time(mean)}, Std: {std:.8f}")
    return mean, median, std
