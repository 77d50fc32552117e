"""Bi-objective sampling of (stable, delta) cost pairs.

A stage configuration costs ``stable`` seconds per micro batch and ``delta`` seconds once
per iteration; which one matters more depends on the gradient-accumulation count and on
the other stages, so the intra-stage tuner hands the inter-stage solver a handful of
trade-off points instead of a single winner: for weights ``alpha`` evenly spaced in (0, 1)
the candidate minimising ``alpha / (1 - alpha) * stable + delta`` (reference:
mist/utils/pareto.py:8-148 sample_pareto_frontier, :162-216 fill_redundant_samples).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from ..ops import native


def sample_pareto_frontier(stable: np.ndarray, delta: np.ndarray, feasible: Optional[np.ndarray], samples: int,
                           use_native: bool = True) -> np.ndarray:
    """Indices (length ``samples``; -1 where nothing is feasible) into the candidate arrays."""
    stable = np.ascontiguousarray(stable, dtype=np.float64)
    delta = np.ascontiguousarray(delta, dtype=np.float64)
    n = stable.shape[0]
    out = np.full(samples, -1, dtype=np.int64)
    if n == 0:
        return out
    feas = None if feasible is None else np.ascontiguousarray(feasible, dtype=np.uint8)
    if use_native:
        try:
            lib = native.runtime()
            fn = lib.rt_pareto_sample
            fn.restype = C.c_int
            fn(stable.ctypes.data_as(C.c_void_p), delta.ctypes.data_as(C.c_void_p),
               feas.ctypes.data_as(C.c_void_p) if feas is not None else None, C.c_int64(n), C.c_int(samples),
               out.ctypes.data_as(C.c_void_p))
            return out
        except (OSError, AttributeError):
            pass
    mask = np.ones(n, dtype=bool) if feas is None else feas.astype(bool)
    if not mask.any():
        return out
    for s in range(samples):
        alpha = (s + 1) / (samples + 1)
        v = np.where(mask, alpha / (1 - alpha) * stable + delta, np.inf)
        out[s] = int(np.argmin(v))
    return out


def dedup_samples(idx: np.ndarray) -> np.ndarray:
    """Unique sampled indices, order preserved, -1 dropped."""
    seen, out = set(), []
    for i in idx.tolist():
        if i >= 0 and i not in seen:
            seen.add(i)
            out.append(i)
    return np.array(out, dtype=np.int64)


def pareto_filter(stable: np.ndarray, delta: np.ndarray) -> np.ndarray:
    """Indices of the non-dominated (stable, delta) points."""
    order = np.lexsort((delta, stable))
    keep, best = [], np.inf
    for i in order:
        if delta[i] < best - 1e-15:
            keep.append(i)
            best = delta[i]
    return np.array(keep, dtype=np.int64)
