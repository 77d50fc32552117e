"""Runs one hot kernel on a fixed, named workload a few times -- the program to put under a
profiler or a timer when looking at a single kernel.

    python -m mist_b200.tools.kernel_cases gemm_pair --repeat 4
    ncu --set full --clock-control none -k regex:gemm_pair -s 1 -c 2 -o prof \\
        python -m mist_b200.tools.kernel_cases gemm_pair

Every case builds random bf16 inputs whose total size exceeds the L2 cache, calls the
framework's own operator (the code path training uses) ``--repeat`` times and checks the
device status word.  The multi-rank kernels run in their single-GPU stand-in mode: the
"peers" are further buffers on the same GPU and their flags are pre-set, so the launch never
waits for another launch.  ``--time`` prints the median device time over the repeats
(CUDA events, L2 flushed between repeats).
"""
from __future__ import annotations

import argparse
from typing import Callable, Dict

import torch

from ..ops import functional as F
from ..ops import native

DEV = "cuda"
BF = torch.bfloat16


def _rand(*shape, scale=1.0, grad=False):
    t = torch.randn(*shape, device=DEV, dtype=BF) * scale
    return t.requires_grad_(True) if grad else t


def case_gemm(pair: bool) -> Callable[[], None]:
    M, N, K = 8192, 7680, 2560
    a, b = _rand(M, K), _rand(N, K, scale=0.02)
    out = torch.empty(M, N, device=DEV, dtype=BF)

    def run():
        F.Settings.gemm_pair = pair
        F.gemm(a, b, out=out)
    return run


def case_gemm_wgrad(pair: bool) -> Callable[[], None]:
    M, N, K = 8192, 7680, 2560           # dW[N, K] += dy[M, N]^T x[M, K], fp32 accumulate
    dy, x = _rand(M, N), _rand(M, K)
    dw = torch.zeros(N, K, device=DEV, dtype=torch.float32)

    def run():
        F.Settings.gemm_pair = pair
        F.gemm(dy, x, a_mn=True, b_mn=True, out=dw, flags=F.EPI_ACCUM)
    return run


def case_norm() -> Callable[[], None]:
    rows, h = 16384, 2560
    x, r = _rand(rows, h, grad=True), _rand(rows, h, grad=True)
    g = torch.ones(h, device=DEV, dtype=BF, requires_grad=True)
    be = torch.zeros(h, device=DEV, dtype=BF, requires_grad=True)

    def run():
        z, xs = F.layer_norm(x, g, be, 1e-5, residual=r, prenorm=True)
        torch.autograd.backward([z, xs], [torch.ones_like(z), torch.ones_like(xs)])
    return run


def case_attention(d: int, s: int, b: int, nh: int) -> Callable[[], None]:
    qkv = _rand(b, s, 3, nh, d, grad=True)

    def run():
        o = F.attention_qkvpacked(qkv * 1.0)
        o.backward(torch.ones_like(o))
    return run


def case_ag_gemm() -> Callable[[], None]:
    """All-gather -> GEMM of a TP2 column-parallel linear (Llama-7B QKV shape), ranks emulated."""
    from ..parallel import fused_tp
    ctx = fused_tp.FusedTPContext(None, 0, emulate_ranks=2)
    rows, K, N = 4096, 4096, 6144
    x, w = _rand(rows, K), _rand(N, K, scale=0.02)

    def run():
        fused_tp._ag_gemm(ctx, x, w, None, False, "case")
    return run


def case_gemm_rs() -> Callable[[], None]:
    """GEMM -> reduce-scatter of a TP2 row-parallel linear (Llama-7B MLP output shape)."""
    from ..parallel import fused_tp
    ctx = fused_tp.FusedTPContext(None, 0, emulate_ranks=2)
    T, K, N = 8192, 5504, 4096
    x, w = _rand(T, K), _rand(N, K, scale=0.02)

    def run():
        fused_tp._gemm_rs(ctx, x, w, False)
    return run


def case_param_ag_gemm() -> Callable[[], None]:
    """ZeRO-3 weight all-gather fused into the QKV GEMM of a 2.7B-sized block, two emulated ranks."""
    from ..parallel.fused_zero3 import ParamGatherContext
    h, M, R = 2560, 8192, 2
    numel = 12 * h * h + 13 * h
    padded = (numel + 128 * R - 1) // (128 * R) * (128 * R)
    ctx = ParamGatherContext(None, padded, emulate_ranks=R, n_slots=1)
    for t in ctx.slots[0][2]:
        t.normal_(0, 0.02)
    x = _rand(M, h)
    b_off = 2 * h // 128 * 128 + 128

    def run():
        ctx.gather_linear(0, x, b_off, 3 * h, h)
    return run


def case_fused_grad_adam() -> Callable[[], None]:
    """Adam step on 80 M parameters (the per-block optimizer update of the 2.7B model)."""
    n = 80 * 1000 * 1000 // 256 * 256
    master = torch.randn(n, device=DEV)
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    grad = _rand(n, scale=0.01)
    model = torch.empty(n, device=DEV, dtype=BF)
    step = [0]

    def run():
        step[0] += 1
        F.adam_step(master, m, v, grad, model, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                    step=step[0], inv_scale=1.0, adamw=True)
    return run


CASES: Dict[str, Callable[[], Callable[[], None]]] = {
    "gemm": lambda: case_gemm(False),
    "gemm_pair": lambda: case_gemm(True),
    "gemm_wgrad": lambda: case_gemm_wgrad(False),
    "gemm_pair_wgrad": lambda: case_gemm_wgrad(True),
    "norm": case_norm,
    "attn_d80": lambda: case_attention(80, 2048, 4, 32),
    "attn_d128": lambda: case_attention(128, 4096, 2, 32),
    "ag_gemm": case_ag_gemm,
    "gemm_rs": case_gemm_rs,
    "param_ag_gemm": case_param_ag_gemm,
    "adam": case_fused_grad_adam,
}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--repeat", type=int, default=4)
    ap.add_argument("--time", action="store_true", help="print the median device time of one repeat")
    args = ap.parse_args(argv)
    torch.manual_seed(0)
    run = CASES[args.case]()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV) if args.time else None
    times = []
    for _ in range(args.repeat):
        if flush is not None:
            flush.zero_()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            run()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        else:
            run()
    torch.cuda.synchronize()
    native.check_status()
    if times:
        times.sort()
        print(f"{args.case}: median {times[len(times) // 2]:.4f} ms over {len(times)} repeats")
    print("ok")


if __name__ == "__main__":
    main()
