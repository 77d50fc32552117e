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
        # An entry holds two timings of its operator: one cold call on a quiet chip (``fwd`` / ``bwd``,
        # boost clock, L2 flushed) and a quarter of a second of back-to-back calls (``fwd_sus`` /
        # ``bwd_sus``) with the SM clock that the chip settled at under that load (``sm_mhz_fwd`` /
        # ``sm_mhz_bwd``, kept for the record).  A training step keeps the chip at its power limit just as
        # the back-to-back loop does, so an operator that is bound by the SMs (tensor cores, exponentials;
        # ``scaled_ops`` in ``_meta.json``) is priced with its sustained timing, every other operator with
        # its cold timing.  Nothing in the meta file is fitted to a training-step time.  (Scaling the
        # sustained timing to one clock "under load" for all operators was tried and dropped: that clock
        # depends on the share of GEMM time in the step; it fitted the 2.7B step and was 18-20 % optimistic
        # on steps with larger GEMMs.)  Entries without sustained timings fall back to the fixed
        # ``sustained_scale`` of the file applied to the cold timing.
        self.sustained_scale, self.scaled_ops, self.sm_mhz_under_load = 1.0, (), None
        self.fused_overlap = {}
        #: host seconds per traced operator of a block (tools/profile_host_dispatch.py); empty: no host bound
        self.host_dispatch = {}
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
                self.host_dispatch = dict(m.get("host_dispatch", {}))
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
        if e is not None and self.refresh_unclocked and "fwd_sus" not in e and spec.op in self.scaled_ops:
            e = None
        if e is not None:
            self.hits += 1
            return self._in_step(spec.op, e)
        self.misses += 1
        if self.allow_profile:
            from . import profiler
            try:
                measured = profiler.profile(spec)
            except RuntimeError as e:      # a launch that the kernels refuse: say which operator, estimate it instead
                import warnings
                warnings.warn(f"could not time {spec.key()} on the device ({e}); using the analytic estimate")
                measured = None
            if measured is not None:
                self.profiled += 1
                entry = {"spec": spec.as_dict(), "fwd": measured[0], "bwd": measured[1], "flops_fwd": flops_fwd,
                         "flops_bwd": flops_bwd, "bytes_fwd": bytes_fwd, "bytes_bwd": bytes_bwd}
                sus = dict(profiler.last_sustained)
                if sus.get("fwd") and sus.get("mhz_fwd"):
                    entry["fwd_sus"], entry["sm_mhz_fwd"] = sus["fwd"], sus["mhz_fwd"]
                    if sus.get("both") and sus.get("mhz_both"):
                        # the forward + backward loop ran at its own clock: bring the forward part to that clock
                        # before taking it out
                        f_at = sus["fwd"] * sus["mhz_fwd"] / sus["mhz_both"]
                        entry["bwd_sus"], entry["sm_mhz_bwd"] = max(sus["both"] - f_at, 0.0), sus["mhz_both"]
                self._store(spec.op, key, entry)
                return self._in_step(spec.op, entry)
        return analytic.estimate(spec, flops_fwd, flops_bwd, bytes_fwd, bytes_bwd, self.model)

    def _in_step(self, op: str, e: Dict) -> Tuple[float, float]:
        """(forward, backward) seconds of an entry under training-step conditions (see ``__init__``)."""
        fwd, bwd = float(e["fwd"]), float(e["bwd"])
        if op not in self.scaled_ops:
            return fwd, bwd
        if e.get("fwd_sus"):
            return float(e["fwd_sus"]), float(e["bwd_sus"]) if e.get("bwd_sus") is not None else bwd * self.sustained_scale
        return fwd * self.sustained_scale, bwd * self.sustained_scale

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
