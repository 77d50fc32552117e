"""Logging and profiler ranges.

Root logger format ``time [LEVEL] {file:line} message``; ranks other than the first of a
data-parallel group are silenced unless asked otherwise (reference: mist/logger.py:7-46).
``record(name)`` labels scheduler actions for ``torch.profiler`` / NVTX with the names the
reference uses (``<module>.unshard``, ``.post_backward_grad_reduce``, ``OPT-<module>.step``...).
"""
from __future__ import annotations

import contextlib
import logging
import os
import sys

import torch

_FMT = "%(asctime)s [%(levelname)5s] {%(filename)s:%(lineno)d} %(message)s"


def get_logger(name: str = "mist_b200", level=None) -> logging.Logger:
    log = logging.getLogger(name)
    if not log.handlers:
        h = logging.StreamHandler(sys.stdout)
        h.setFormatter(logging.Formatter(_FMT))
        log.addHandler(h)
        log.setLevel(level or os.environ.get("MIST_LOG_LEVEL", "INFO"))
        log.propagate = False
    return log


def set_rank_filter(dp_rank: int, tag: str = "", only_first_dp_rank: bool = True):
    """Prefixes messages with ``tag`` and silences every data-parallel rank but the first."""
    log = get_logger()
    if only_first_dp_rank and dp_rank != 0:
        log.setLevel(logging.ERROR)
    for h in log.handlers:
        h.setFormatter(logging.Formatter((f"[{tag}] " if tag else "") + _FMT))


_PROFILING = False


def enable_ranges(flag: bool = True):
    global _PROFILING
    _PROFILING = flag


@contextlib.contextmanager
def record(name: str):
    """Named range visible in torch.profiler traces and (on CUDA) as an NVTX range."""
    if not _PROFILING:
        yield
        return
    with torch.profiler.record_function(name):
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            if torch.cuda.is_available():
                torch.cuda.nvtx.range_pop()


def log_memory(tag: str = "", logger=None):
    """Allocated / reserved / peak device memory in MB."""
    logger = logger or get_logger()
    if not torch.cuda.is_available():
        return
    mb = 1 << 20
    logger.info("%s allocated %.0f MB (peak %.0f) reserved %.0f MB (peak %.0f)", tag,
                torch.cuda.memory_allocated() / mb, torch.cuda.max_memory_allocated() / mb,
                torch.cuda.memory_reserved() / mb, torch.cuda.max_memory_reserved() / mb)
