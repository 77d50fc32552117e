"""Operator-latency database: measured (forward, backward) seconds per :class:`NodeSpec`.

Entries live in one JSON file per operator under ``cache_<device name>/<op>.json`` next to
this module (or under ``MIST_B200_OP_CACHE``), guarded by a lock file so concurrent ranks
can add entries.  A lookup order of: memory -> JSON file -> micro-benchmark on the local
GPU (when there is one and profiling is allowed) -> analytic estimate.

``FAKE_DEVICE_NAME`` selects another device's cache on any machine, which is how the tuner
plans for a GPU that is not present (reference: mist/node_database/node_spec.py:234-373
lookup / file-locked JSON, mist/utils/device.py:67-75 FAKE_DEVICE_NAME, the shipped
cache_NVIDIA_L4 directory).
"""
from __future__ import annotations

import fcntl
import json
import os
from pathlib import Path
from typing import Dict, Optional, Tuple

import torch

from . import analytic
from .node_spec import NodeSpec

_HERE = Path(__file__).resolve().parent


def device_name() -> str:
    fake = os.environ.get("FAKE_DEVICE_NAME")
    if fake:
        return fake.replace(" ", "_")
    if torch.cuda.is_available():
        return torch.cuda.get_device_name(0).replace(" ", "_")
    return "NVIDIA_B200"


class OpDatabase:
    def __init__(self, device: Optional[str] = None, root: Optional[os.PathLike] = None, allow_profile: bool = True,
                 refresh_unclocked: bool = False):
        self.device = (device or device_name()).replace(" ", "_")
        base = Path(root or os.environ.get("MIST_B200_OP_CACHE", _HERE))
        self.dir = base / f"cache_{self.device}"
        self.allow_profile = allow_profile and torch.cuda.is_available() and not os.environ.get("FAKE_DEVICE_NAME")
        #: measure again the entries that were stored without the SM clock they ran at
        self.refresh_unclocked = bool(refresh_unclocked) and self.allow_profile
        self.model = analytic.device_model(self.device)
        self._mem: Dict[str, Dict[str, Dict]] = {}
        # Entries are timed one operator at a time, in short bursts, and carry the SM clock that was
        # read while they ran (``sm_mhz``).  A training step keeps the tensor cores busy for seconds
        # and settles at a lower, power-capped clock; the time of an operator that is bound by the SMs
        # (tensor cores, exponentials) scales with the inverse of that clock, so such an entry is
        # multiplied by ``sm_mhz / sm_mhz_under_load``.  ``_meta.json`` beside the entries names the
        # operators this applies to and the clock measured under a training load (the median that
        # bench.py samples during its timed region).  Entries without a recorded clock fall back to the
        # fixed ``sustained_scale`` of the file.
        self.sustained_scale, self.scaled_ops, self.sm_mhz_under_load = 1.0, (), None
        self.fused_overlap = {}
        meta = self.dir / "_meta.json"
        if meta.exists():
            try:
                with open(meta) as f:
                    m = json.load(f)
                self.sustained_scale = float(m.get("sustained_scale", 1.0))
                self.scaled_ops = tuple(m.get("scaled_ops", ()))
                if m.get("sm_mhz_under_load"):
                    self.sm_mhz_under_load = float(m["sm_mhz_under_load"])
                # overlap of the fused GEMM + collective kernels: {"ag_gemm": {"kappa", "tau"}, ...}
                self.fused_overlap = dict(m.get("fused_overlap", {}))
            except (json.JSONDecodeError, OSError, ValueError):
                pass
        self.hits = self.misses = self.profiled = 0

    # ---------------------------------------------------------------------------- files
    def _path(self, op: str) -> Path:
        return self.dir / f"{op}.json"

    def _load(self, op: str) -> Dict[str, Dict]:
        if op not in self._mem:
            p = self._path(op)
            data = {}
            if p.exists():
                try:
                    with open(p) as f:
                        data = json.load(f)
                except (json.JSONDecodeError, OSError):
                    data = {}
            self._mem[op] = data
        return self._mem[op]

    def _store(self, op: str, key: str, entry: Dict):
        self.dir.mkdir(parents=True, exist_ok=True)
        p = self._path(op)
        lock = p.with_suffix(".lock")
        with open(lock, "w") as lf:
            fcntl.flock(lf, fcntl.LOCK_EX)
            data = {}
            if p.exists():
                try:
                    with open(p) as f:
                        data = json.load(f)
                except (json.JSONDecodeError, OSError):
                    data = {}
            data[key] = entry
            tmp = p.with_suffix(".tmp")
            with open(tmp, "w") as f:
                json.dump(data, f, indent=0, sort_keys=True)
            os.replace(tmp, p)
            fcntl.flock(lf, fcntl.LOCK_UN)
        self._mem[op] = data

    # --------------------------------------------------------------------------- lookup
    def latency(self, spec: NodeSpec, flops_fwd: float = 0.0, flops_bwd: float = 0.0, bytes_fwd: float = 0.0,
                bytes_bwd: float = 0.0) -> Tuple[float, float]:
        """(forward, backward) seconds of one operator instance."""
        entries = self._load(spec.op)
        key = spec.key()
        e = entries.get(key)
        if e is not None and self.refresh_unclocked and "sm_mhz" not in e and spec.op in self.scaled_ops:
            e = None
        if e is not None:
            self.hits += 1
            return float(e["fwd"]) * self._clock_scale(spec.op, e), float(e["bwd"]) * self._clock_scale(spec.op, e)
        self.misses += 1
        if self.allow_profile:
            from . import profiler
            measured = profiler.profile(spec)
            if measured is not None:
                self.profiled += 1
                entry = {"spec": spec.as_dict(), "fwd": measured[0], "bwd": measured[1], "flops_fwd": flops_fwd,
                         "flops_bwd": flops_bwd, "bytes_fwd": bytes_fwd, "bytes_bwd": bytes_bwd}
                mhz = profiler.median_clock()
                if mhz:
                    entry["sm_mhz"] = mhz
                self._store(spec.op, key, entry)
                return measured[0] * self._clock_scale(spec.op, entry), measured[1] * self._clock_scale(spec.op, entry)
        return analytic.estimate(spec, flops_fwd, flops_bwd, bytes_fwd, bytes_bwd, self.model)

    def _clock_scale(self, op: str, entry: Dict) -> float:
        """Factor from the entry's profiling conditions to a training step (see ``__init__``)."""
        if op not in self.scaled_ops:
            return 1.0
        mhz = entry.get("sm_mhz")
        if mhz and self.sm_mhz_under_load:
            return max(1.0, float(mhz) / self.sm_mhz_under_load)
        return self.sustained_scale

    def add(self, spec: NodeSpec, fwd: float, bwd: float, **extra):
        self._store(spec.op, spec.key(), dict({"spec": spec.as_dict(), "fwd": fwd, "bwd": bwd}, **extra))

    def all_entries(self) -> Dict[str, Dict]:
        out = {}
        if self.dir.exists():
            for p in self.dir.glob("*.json"):
                if not p.name.startswith("_"):
                    out.update(self._load(p.stem))
        return out

    def refit_model(self):
        self.model = analytic.refit(self.model, self.all_entries())
        return self.model
