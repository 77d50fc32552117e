"""Roofline-style latency estimates for operators that are not in the measured database.

``time = max(FLOPs / (peak * eff_compute), bytes / (bandwidth * eff_memory)) + launch``
with per-operator efficiencies.  The defaults were read off microbenchmarks of this
framework's kernels on B200 (GEMM ~0.85 of the measured cuBLAS bf16 rate at large sizes,
flash attention forward ~0.3 / backward ~0.2 of it, normalisation and elementwise kernels
0.5-0.9 of the measured copy bandwidth); :func:`refit` re-derives them from database
entries.  It lets the analyzer and tuner run on a machine without a GPU; measured entries
always take precedence.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Tuple

from .node_spec import NodeSpec


@dataclass
class DeviceModel:
    name: str = "NVIDIA_B200"
    peak_tflops: float = 1340.0       # sustained dense bf16 (measured library GEMM under the power cap)
    hbm_gbs: float = 6500.0           # measured copy bandwidth
    launch_s: float = 4e-6
    # efficiency of the compute roof per operator (forward, backward)
    eff_compute: Dict[str, Tuple[float, float]] = field(default_factory=lambda: {
        "linear": (0.85, 0.85), "bmm": (0.6, 0.6), "flash_attention": (0.28, 0.22),
    })
    # efficiency of the memory roof per operator (forward, backward); "default" for the rest
    eff_memory: Dict[str, Tuple[float, float]] = field(default_factory=lambda: {
        "layer_norm": (0.45, 0.3), "rms_norm": (0.45, 0.3), "cross_entropy": (0.75, 0.75),
        "swiglu": (0.8, 0.8), "gelu": (0.8, 0.8), "embedding": (0.5, 0.2), "default": (0.6, 0.6),
    })
    # small GEMMs do not fill the machine: eff *= flops / (flops + gemm_half_flops)
    gemm_half_flops: float = 3.0e10


L4 = DeviceModel(name="NVIDIA_L4", peak_tflops=60.0, hbm_gbs=260.0, launch_s=8e-6)
A100 = DeviceModel(name="NVIDIA_A100-SXM4-40GB", peak_tflops=250.0, hbm_gbs=1400.0, launch_s=5e-6)
DEVICES = {"NVIDIA_B200": DeviceModel(), "NVIDIA_L4": L4, "NVIDIA_A100-SXM4-40GB": A100}


def device_model(name: str) -> DeviceModel:
    return DEVICES.get(name.replace(" ", "_"), DeviceModel(name=name))


def estimate(spec: NodeSpec, flops_fwd: float, flops_bwd: float, bytes_fwd: float, bytes_bwd: float,
             dev: DeviceModel) -> Tuple[float, float]:
    """(forward seconds, backward seconds)."""
    ec = dev.eff_compute.get(spec.op)
    em = dev.eff_memory.get(spec.op, dev.eff_memory["default"])
    out = []
    for i, (fl, by) in enumerate(((flops_fwd, bytes_fwd), (flops_bwd, bytes_bwd))):
        if fl <= 0 and by <= 0:
            out.append(0.0)
            continue
        t_mem = by / (dev.hbm_gbs * 1e9 * em[i]) if by > 0 else 0.0
        t_cmp = 0.0
        if ec is not None and fl > 0:
            eff = ec[i]
            if spec.op in ("linear", "bmm"):
                eff *= fl / (fl + dev.gemm_half_flops)
            t_cmp = fl / (dev.peak_tflops * 1e12 * eff)
        launches = 1 if i == 0 else (3 if spec.op == "linear" else 2)
        out.append(max(t_mem, t_cmp) + dev.launch_s * launches)
    return out[0], out[1]


def refit(dev: DeviceModel, entries: Dict[str, Dict]) -> DeviceModel:
    """Rescales the per-operator efficiencies so the model reproduces measured entries
    (each entry: ``{"spec": {...}, "fwd": s, "bwd": s, "flops_fwd", "flops_bwd",
    "bytes_fwd", "bytes_bwd"}``) in the least-squares sense of log ratios."""
    import math
    by_op: Dict[str, list] = {}
    for e in entries.values():
        by_op.setdefault(e["spec"]["op"], []).append(e)
    for op, es in by_op.items():
        for i, (tk, fk, bk) in enumerate((("fwd", "flops_fwd", "bytes_fwd"), ("bwd", "flops_bwd", "bytes_bwd"))):
            ratios = []
            for e in es:
                spec = NodeSpec.from_dict(e["spec"])
                pred = estimate(spec, e.get("flops_fwd", 0), e.get("flops_bwd", 0), e.get("bytes_fwd", 0),
                                e.get("bytes_bwd", 0), dev)[i]
                if e.get(tk, 0) > 0 and pred > 0:
                    ratios.append(math.log(pred / e[tk]))
            if not ratios:
                continue
            scale = math.exp(sum(ratios) / len(ratios))      # > 1: model too slow -> raise efficiency
            if op in dev.eff_compute:
                f = list(dev.eff_compute[op])
                f[i] = min(1.0, f[i] * scale)
                dev.eff_compute[op] = tuple(f)
            else:
                f = list(dev.eff_memory.get(op, dev.eff_memory["default"]))
                f[i] = min(1.0, f[i] * scale)
                dev.eff_memory[op] = tuple(f)
    return dev
