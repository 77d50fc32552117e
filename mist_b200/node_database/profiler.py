"""Micro-benchmarks one operator instance on the local GPU for the latency database.

Builds random inputs of the spec's shapes, runs the framework's own op (the same code
path training uses) forward and backward, and times both with CUDA events after warm-up,
writing a buffer larger than L2 between repetitions so every run starts cold
(reference: mist/node_database/benchmark_computation_latency.py:36-228; it re-materialises
the inputs to defeat L2, here L2 is flushed explicitly).
Out-of-memory during profiling yields ``None`` (the caller falls back to the analytic
estimate) instead of a fake huge latency.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Tuple

import torch

from .node_spec import NodeSpec

WARMUP, REPEAT = 3, 5
#: seconds an operator is run back to back for its sustained timing (long enough for the SM clock to
#: settle under the power cap and for NVML's clock reading to mean something)
SUSTAIN_S = 0.25
_flush = None
_nvml = None
#: SM clocks (MHz) read while the most recent operator was being timed
clock_samples = []


def _sm_mhz() -> Optional[float]:
    """Current SM clock of the device in use, read through NVML (None when NVML is not there)."""
    global _nvml
    try:
        import pynvml
        if _nvml is None:
            pynvml.nvmlInit()
            uuid = torch.cuda.get_device_properties(torch.cuda.current_device()).uuid
            _nvml = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
        return float(pynvml.nvmlDeviceGetClockInfo(_nvml, pynvml.NVML_CLOCK_SM))
    except Exception:      # noqa: BLE001 - clocks are an annotation, never a reason to fail
        _nvml = False if _nvml is None else _nvml
        return None


def median_clock() -> Optional[float]:
    """Median of the SM clocks sampled since the last :func:`profile` call started."""
    if not clock_samples:
        return None
    xs = sorted(clock_samples)
    return xs[len(xs) // 2]


def _flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def _time(fn: Callable[[], None]) -> float:
    for _ in range(WARMUP):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(REPEAT):
        _flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        mhz = _sm_mhz() if _nvml is not False else None      # read while the kernels are (still) running
        if mhz:
            clock_samples.append(mhz)
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e-3)
    ts.sort()
    return ts[len(ts) // 2]


#: (sustained forward seconds, sustained forward+backward seconds, median SM MHz) of the last profile() call
last_sustained = {}


def _sustained(fn: Callable[[], None], one: float) -> Tuple[float, Optional[float]]:
    """Seconds per call of ``fn`` run back to back for about SUSTAIN_S, and the median SM clock over the
    second half of that time.  A single cold call says how long the kernel takes at boost clock on a quiet
    chip; inside a training step the chip sits at its power-capped clock, which this loop reproduces."""
    reps = int(min(max(SUSTAIN_S / max(one, 1e-6), 3), 4000))
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    clocks = []
    import time
    t0 = time.perf_counter()
    while not b.query():
        mhz = _sm_mhz() if _nvml is not False else None
        if mhz and time.perf_counter() - t0 > 0.4 * reps * one:
            clocks.append(mhz)
        time.sleep(0.01)
    torch.cuda.synchronize()
    per = a.elapsed_time(b) * 1e-3 / reps
    clocks.sort()
    return per, (clocks[len(clocks) // 2] if clocks else None)


def _fwd_bwd(make_inputs, op) -> Tuple[float, float]:
    """Times ``op(*inputs)`` and the backward of its first output."""
    inputs = make_inputs()
    out = op(*inputs)
    first = out[0] if isinstance(out, (tuple, list)) else out
    g = torch.randn_like(first) if first.dtype.is_floating_point else None
    last_sustained.clear()
    with torch.no_grad():
        det = [t.detach() if isinstance(t, torch.Tensor) else t for t in inputs]
        fwd = _time(lambda: op(*det))
    if g is None or not first.requires_grad:
        with torch.no_grad():
            last_sustained["fwd"], last_sustained["mhz_fwd"] = _sustained(lambda: op(*det), fwd)
        return fwd, 0.0
    leaves = [t for t in inputs if isinstance(t, torch.Tensor) and t.requires_grad]

    def both():
        o = op(*inputs)
        o0 = o[0] if isinstance(o, (tuple, list)) else o
        torch.autograd.grad(o0, leaves, g, allow_unused=True)

    total = _time(both)
    # the sustained loops come after both cold timings: they leave the chip at its power-capped clock
    with torch.no_grad():
        last_sustained["fwd"], last_sustained["mhz_fwd"] = _sustained(lambda: op(*det), fwd)
    last_sustained["both"], last_sustained["mhz_both"] = _sustained(both, total)
    return fwd, max(total - fwd, 0.0)


def profile(spec: NodeSpec, dtype=torch.bfloat16) -> Optional[Tuple[float, float]]:
    from ..ops import functional as F
    dev = "cuda"
    op = spec.op
    g = spec.get
    del clock_samples[:]
    last_sustained.clear()

    def rnd(*shape, grad=True, scale=1.0):
        return (torch.randn(*shape, device=dev, dtype=dtype) * scale).requires_grad_(grad)

    try:
        if op == "linear":
            m, n, k = int(g("m")), int(g("n")), int(g("k"))
            act = g("act") or None
            return _fwd_bwd(lambda: (rnd(m, k), rnd(n, k, scale=0.02), rnd(n) if g("bias") else None),
                            lambda x, w, b: F.linear(x, w, b, activation=act))
        if op in ("layer_norm", "rms_norm"):
            rows, h = int(g("rows")), int(g("h"))
            res = bool(g("residual"))
            if op == "layer_norm":
                return _fwd_bwd(lambda: (rnd(rows, h), rnd(h), rnd(h), rnd(rows, h) if res else None),
                                lambda x, ga, be, r: F.layer_norm(x, ga, be, 1e-5, residual=r, prenorm=res))
            return _fwd_bwd(lambda: (rnd(rows, h), rnd(h), rnd(rows, h) if res else None),
                            lambda x, ga, r: F.rms_norm(x, ga, 1e-5, residual=r, prenorm=res))
        if op == "flash_attention":
            b, sq, nh, d = int(g("b")), int(g("sq")), int(g("nh")), int(g("d"))
            causal = bool(g("causal"))
            if int(g("sk")) == sq and int(g("nkv")) == nh:
                return _fwd_bwd(lambda: (rnd(b, sq, 3, nh, d),),
                                lambda qkv: F.attention_qkvpacked(qkv * 1.0, 1.0 / math.sqrt(d), causal))
            sk, nkv = int(g("sk")), int(g("nkv"))
            return _fwd_bwd(lambda: (rnd(b, sq, nh, d), rnd(b, sk, nkv, d), rnd(b, sk, nkv, d)),
                            lambda q, k, v: F.attention(q, k, v, 1.0 / math.sqrt(d), causal))
        if op == "swiglu":
            rows, f = int(g("rows")), int(g("f"))
            return _fwd_bwd(lambda: (rnd(rows, 2 * f),), F.swiglu)
        if op == "gelu":
            return None
        if op == "cross_entropy":
            rows, cols = int(g("rows")), int(g("cols"))
            labels = torch.randint(0, cols, (rows,), device=dev)
            # the backward pass overwrites the logits, so each run gets a fresh copy (timed apart)
            base = torch.randn(rows, cols, device=dev, dtype=dtype)
            copy_t = _time(lambda: base.clone())

            def run():
                x = base.clone().requires_grad_(True)
                F.cross_entropy(x, labels).mean().backward()

            with torch.no_grad():
                fwd = _time(lambda: F.cross_entropy(base, labels))
            total = _time(run) - copy_t
            return fwd, max(total - fwd, 0.0)
        if op == "embedding":
            tokens, h, vocab = int(g("tokens")), int(g("h")), int(g("vocab"))
            seq = min(tokens, 2048)
            ids = torch.randint(0, vocab, (tokens // seq, seq), device=dev)
            return _fwd_bwd(lambda: (rnd(vocab, h), rnd(seq, h)), lambda w, p: F.embedding(ids, w, p))
        if op == "bmm":
            bt, m, n, k = int(g("batch")), int(g("m")), int(g("n")), int(g("k"))
            return _fwd_bwd(lambda: (rnd(bt, m, k), rnd(bt, k, n)), torch.bmm)
        if op in ("causal_softmax", "softmax"):
            return None
    except torch.cuda.OutOfMemoryError:
        torch.cuda.empty_cache()
        return None
    return None
