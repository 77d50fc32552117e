"""Numerics of every CUDA kernel against a plain PyTorch fp32 reference of the same op."""
import math
import os

import pytest
import torch

from mist_b200.ops import functional as F

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (384, 640, 192), (1000, 520, 264), (2048, 2560, 2560)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_gemm_layouts(M, N, K, a_mn, b_mn, tile_n):
    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operand needs a leading dimension that is a multiple of 8")
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    out = F.gemm(a_in, b_in, a_mn=a_mn, b_mn=b_mn, tile_n=tile_n)
    assert _rel_err(out, ref) < 1e-2
    _check_edges(out, ref)


def _check_edges(out, ref, tol=0.02):
    """Element-wise check of the last rows and columns (the ragged tiles): a wrong vector there does not
    move a norm over the whole matrix.  bf16 output of a K-long dot product of unit-variance operands:
    the error per element stays far below ``tol`` times the largest reference magnitude."""
    scale = ref.abs().max().item()
    o, r = out.float(), ref.float()
    for region in (o[-130:] - r[-130:], o[:, -130:] - r[:, -130:], o[:8] - r[:8], o[:, :8] - r[:, :8]):
        assert region.abs().max().item() < tol * scale


@pytest.mark.parametrize("M,N,K", [(1000, 520, 264), (8192 + 40, 2560 + 8, 328), (300, 7680 + 24, 2560)])
def test_gemm_pair_ragged_edges(M, N, K):
    """Shapes large enough for the CTA-pair kernel with ragged last tiles in both directions."""
    torch.manual_seed(7)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    out = F.gemm(a, b)
    assert _rel_err(out, ref) < 1e-2
    _check_edges(out, ref)
    # weight-gradient layout with fp32 accumulation into an existing bucket
    dy = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    acc = torch.randn(N, K, device=DEV, dtype=torch.float32)
    ref2 = acc + dy.float().t() @ a.float()
    if M % 8 == 0:
        F.gemm(dy, a, a_mn=True, b_mn=True, out=acc, flags=F.EPI_ACCUM)
        assert _rel_err(acc, ref2) < 1e-3
        _check_edges(acc, ref2, tol=0.01)


def test_gemm_epilogues():
    torch.manual_seed(1)
    M, N, K = 512, 768, 320
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t() + bias.float()
    out = F.gemm(a, b, bias=bias)
    assert _rel_err(out, ref) < 1e-2
    pre = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    out = F.gemm(a, b, bias=bias, aux=pre, flags=F.EPI_GELU | F.EPI_SAVE_PRE)
    assert _rel_err(pre, ref) < 1e-2
    assert _rel_err(out, torch.nn.functional.gelu(ref, approximate="tanh")) < 1e-2
    # fp32 accumulate
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    ref2 = acc + a.float() @ b.float().t()
    F.gemm(a, b, out=acc, flags=F.EPI_ACCUM)
    assert _rel_err(acc, ref2) < 1e-3
    # bf16 accumulate + residual
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    out = F.gemm(a, b, aux=res, flags=F.EPI_RESIDUAL)
    assert _rel_err(out, a.float() @ b.float().t() + res.float()) < 1e-2


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("K", [320, 1088])
def test_gemm_cta_pair_layouts_and_epilogues(a_mn, b_mn, K):
    """256 x 256 tiles on CTA pairs: ragged bottom edge (the second CTA of the last pair has no
    live rows), ragged right edge, fewer and more k-blocks than pipeline stages."""
    from mist_b200.ops import native
    from mist_b200.ops.native import ptr, stream
    torch.manual_seed(3)
    M, N = 2176, 2624
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    ref = a.float() @ b.float().t()
    lib = native.kernels()

    def run(out, flags, bias_t=None, aux=None):
        rc = lib.mb_gemm_pair_bf16(ptr(a_in), ptr(b_in), ptr(out), M, N, K, a_in.stride(0), b_in.stride(0),
                                   out.stride(0), int(a_mn), int(b_mn), flags, ptr(bias_t), ptr(aux), 1.0, 0, stream())
        assert rc == 0, rc           # 1 would mean "use the single-CTA kernel": the pair kernel must take these
        torch.cuda.synchronize()
        native.check_status()

    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    run(out, 0)
    assert _rel_err(out, ref) < 1e-2
    pre = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    run(out, F.EPI_BIAS | F.EPI_GELU | F.EPI_SAVE_PRE, bias, pre)
    assert _rel_err(pre, ref + bias.float()) < 1e-2
    assert _rel_err(out, torch.nn.functional.gelu(ref + bias.float(), approximate="tanh")) < 1e-2
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    ref2 = acc + ref
    run(acc, F.EPI_OUT_FP32 | F.EPI_ACCUM)
    assert _rel_err(acc, ref2) < 1e-3


@pytest.mark.parametrize("M,h,f", [(2304, 2560, 2304), (300, 256, 520)])
def test_fused_gelu_mlp_matches_reference(M, h, f):
    """One autograd node for fc1 -> GELU -> fc2; the backward pass multiplies by gelu'(pre) in the
    epilogue of the dgrad GEMM (CTA-pair kernel for the large case, single-CTA for the small one)."""
    torch.manual_seed(6)
    x = (torch.randn(M, h, device=DEV, dtype=torch.bfloat16)).requires_grad_(True)
    w1 = (torch.randn(f, h, device=DEV, dtype=torch.bfloat16) * 0.03).requires_grad_(True)
    b1 = (torch.randn(f, device=DEV, dtype=torch.bfloat16) * 0.1).requires_grad_(True)
    w2 = (torch.randn(h, f, device=DEV, dtype=torch.bfloat16) * 0.03).requires_grad_(True)
    b2 = (torch.randn(h, device=DEV, dtype=torch.bfloat16) * 0.1).requires_grad_(True)
    y = F.mlp_gelu(x, w1, b1, w2, b2)
    g = torch.randn_like(y)
    grads = torch.autograd.grad(y, (x, w1, b1, w2, b2), g)
    ref_in = [t.detach().float().requires_grad_(True) for t in (x, w1, b1, w2, b2)]
    xr, w1r, b1r, w2r, b2r = ref_in
    yr = torch.nn.functional.gelu(xr @ w1r.t() + b1r, approximate="tanh") @ w2r.t() + b2r
    grads_r = torch.autograd.grad(yr, ref_in, g.float())
    assert _rel_err(y, yr) < 1e-2
    for name, a, b in zip(("dx", "dw1", "db1", "dw2", "db2"), grads, grads_r):
        assert _rel_err(a, b) < 2e-2, name


def test_gemm_cta_pair_residual_epilogue():
    from mist_b200.ops import native
    from mist_b200.ops.native import ptr, stream
    torch.manual_seed(7)
    M, N, K = 2176, 2624, 320
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    rc = native.kernels().mb_gemm_pair_bf16(ptr(a), ptr(b), ptr(out), M, N, K, K, K, N, 0, 0, F.EPI_RESIDUAL, None,
                                            ptr(res), 1.0, 0, stream())
    assert rc == 0
    torch.cuda.synchronize()
    native.check_status()
    assert _rel_err(out, a.float() @ b.float().t() + res.float()) < 1e-2


def test_linear_autograd_matches_reference():
    torch.manual_seed(2)
    x = torch.randn(4, 128, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(512, 256, device=DEV, dtype=torch.bfloat16) * 0.05).requires_grad_(True)
    b = torch.randn(512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = F.linear(x, w, b, activation="gelu")
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.gelu(torch.nn.functional.linear(xr, wr, br), approximate="tanh")
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 2e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2
    assert _rel_err(b.grad, br.grad) < 2e-2


@pytest.mark.parametrize("h", [256, 2048, 2560, 4096, 5120, 6144, 8192])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_fwd_bwd(h, rms):
    torch.manual_seed(3)
    rows = 777
    x0 = torch.randn(rows, h, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    res = torch.randn(rows, h, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    g = (1 + 0.1 * torch.randn(h, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    b = (0.1 * torch.randn(h, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    if rms:
        z, xs = F.rms_norm(x0, g, 1e-5, residual=res, prenorm=True)
    else:
        z, xs = F.layer_norm(x0, g, b, 1e-5, residual=res, prenorm=True)
    dz, dxs = torch.randn_like(z), torch.randn_like(xs)
    torch.autograd.backward([z, xs], [dz, dxs])

    x0r, resr, gr, br = (t.detach().float().requires_grad_(True) for t in (x0, res, g, b))
    xsr = (x0r + resr).to(torch.bfloat16).float()  # the kernel rounds the stream to bf16
    xsr_leaf = (x0r + resr)
    if rms:
        zr = xsr_leaf * torch.rsqrt(xsr_leaf.pow(2).mean(-1, keepdim=True) + 1e-5) * gr
    else:
        zr = torch.nn.functional.layer_norm(xsr_leaf, (h,), gr, br, 1e-5)
    torch.autograd.backward([zr, xsr_leaf], [dz.float(), dxs.float()])
    assert _rel_err(z, zr) < 1e-2
    assert _rel_err(xs, xsr) < 1e-2
    assert _rel_err(x0.grad, x0r.grad) < 1e-2
    assert _rel_err(res.grad, resr.grad) < 1e-2
    assert _rel_err(g.grad, gr.grad) < 2e-2
    if not rms:
        assert _rel_err(b.grad, br.grad) < 2e-2


def test_gelu_swiglu_bias_dropout_add():
    torch.manual_seed(4)
    x = torch.randn(333, 1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    bias = torch.randn(1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = F.gelu(x, bias)
    g = torch.randn_like(y)
    y.backward(g)
    xr, br = x.detach().float().requires_grad_(True), bias.detach().float().requires_grad_(True)
    yr = torch.nn.functional.gelu(xr + br, approximate="tanh")
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2 and _rel_err(x.grad, xr.grad) < 1e-2 and _rel_err(bias.grad, br.grad) < 2e-2

    x = torch.randn(333, 2 * 768, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = F.swiglu(x)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    a, u = xr.chunk(2, -1)
    yr = torch.nn.functional.silu(a) * u
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2 and _rel_err(x.grad, xr.grad) < 1e-2

    x = torch.randn(64, 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(64, 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = F.bias_dropout_add(x, b, r, 0.0)
    assert _rel_err(y, x.float() + b.float() + r.float()) < 1e-2
    y.sum().backward()
    assert torch.allclose(x.grad.float(), torch.ones_like(x.grad).float())
    # the incoming gradient is a stride-0 expansion here; the bias gradient must still sum 64 rows
    assert torch.allclose(b.grad.float(), torch.full_like(b.grad, 64.0).float())
    # dropout: mask regenerated identically in backward, keep-rate close to 1-p
    y = F.bias_dropout_add(x, None, None, 0.25, seed=1234)
    kept = (y != 0).float().mean().item()
    assert abs(kept - 0.75) < 0.02
    x.grad = None
    y.backward(torch.ones_like(y))
    assert torch.equal(x.grad != 0, y != 0)


@pytest.mark.parametrize("d,rot", [(128, 128), (128, 32), (80, 16), (64, 64)])
def test_rope(d, rot):
    torch.manual_seed(5)
    b, s, nh = 2, 96, 6
    qkv = torch.randn(b, s, 3, nh, d, device=DEV, dtype=torch.bfloat16)
    cos, sin = F.rope_tables(s, rot, 10000.0, DEV)
    ref = F._rope_apply(qkv.cpu(), cos.cpu(), sin.cpu(), rot, False, 2)
    out = F.apply_rotary_qkv_(qkv.clone(), cos, sin, rot)
    assert _rel_err(out.cpu(), ref) < 1e-2
    back = F.apply_rotary_qkv_(out.clone(), cos, sin, rot, conj=True)
    assert _rel_err(back, qkv) < 2e-2


@pytest.mark.parametrize("cols,v0", [(50304, 0), (12576, 12576), (32000, 0), (1000, 0)])
def test_cross_entropy(cols, v0):
    torch.manual_seed(6)
    rows = 300
    logits = (torch.randn(rows, cols, device=DEV) * 3).to(torch.bfloat16).requires_grad_(True)
    labels = torch.randint(v0, v0 + cols, (rows,), device=DEV)
    loss = F.cross_entropy(logits, labels, vocab_start=v0)
    ref_in = logits.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(ref_in, labels - v0, reduction="none")
    assert torch.allclose(loss, ref, atol=2e-2, rtol=1e-2)
    w = torch.rand(rows, device=DEV)
    (loss * w).sum().backward()
    (ref * w).sum().backward()
    assert _rel_err(logits.grad, ref_in.grad) < 2e-2


def test_embedding_fwd_bwd():
    torch.manual_seed(7)
    b, s, h, v = 3, 64, 256, 1000
    ids = torch.randint(0, v, (b, s), device=DEV)
    wte = torch.randn(v, h, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    wpe = torch.randn(s, h, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    out = F.embedding(ids, wte, wpe)
    ref = wte.float()[ids] + wpe.float()[None]
    assert _rel_err(out, ref) < 1e-2
    g = torch.randn_like(out)
    out.backward(g)
    wr = wte.detach().float().requires_grad_(True)
    pr = wpe.detach().float().requires_grad_(True)
    (wr[ids] + pr[None]).backward(g.float())
    assert _rel_err(wte.grad, wr.grad) < 1e-2 and _rel_err(wpe.grad, pr.grad) < 1e-2
    # vocab-parallel slice: ids outside [v0, v1) give zero rows
    half = F.embedding(ids, wte.detach()[500:], None, vocab_start=500)
    mask = (ids >= 500)[..., None].float()
    assert _rel_err(half, wte.detach().float()[ids] * mask) < 1e-2


def test_causal_softmax():
    torch.manual_seed(8)
    x = torch.randn(2, 4, 128, 128, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = F.scaled_causal_softmax(x, 0.125)
    xr = x.detach().float().requires_grad_(True)
    mask = torch.ones(128, 128, dtype=torch.bool, device=DEV).tril()
    yr = torch.softmax((xr * 0.125).masked_fill(~mask, float("-inf")), -1)
    assert _rel_err(y, yr) < 1e-2
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    assert _rel_err(x.grad, xr.grad) < 2e-2


def test_adam_matches_torch():
    torch.manual_seed(9)
    n = 100003
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV).to(torch.bfloat16)
    ref = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    model = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    for step in range(1, 4):
        ref.grad = g.float() * 0.5
        opt.step()
        F.adam_step(p, m, v, g, model, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                    step=step, inv_scale=0.5, adamw=True)
    assert torch.allclose(p, ref.detach(), atol=1e-5, rtol=1e-4)
    assert _rel_err(model, ref.detach()) < 1e-2


def test_cast_and_accumulate():
    src = torch.randn(10001, device=DEV)
    dst = torch.empty(10001, device=DEV, dtype=torch.bfloat16)
    F.cast_to_bf16(src, dst, 2.0)
    assert _rel_err(dst, src * 2) < 1e-2
    acc = torch.ones(10001, device=DEV)
    F.accumulate_grad(dst, acc, 0.5, True)
    assert _rel_err(acc, 1 + dst.float() * 0.5) < 1e-5


def _rc(a, b):
    return _rel_err(a.detach().cpu(), b.detach().cpu())


def _norm_cpu(args, kwargs):
    """The same autograd function on CPU copies in fp32 (the reference path of the operator)."""
    cpu = [None if a is None else (a.detach().cpu().float().requires_grad_(a.requires_grad) if a.is_floating_point() else a.cpu())
           for a in args]
    return cpu, F.parallel_residual_norm(*cpu, **kwargs)


@pytest.mark.parametrize("h", [1024, 2560, 4096, 8192])
@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("res_fp32", [False, True])
def test_pipelined_norm_plain_and_fp32_stream(h, rms, res_fp32):
    """Pipelined norm kernels (forward and backward), ragged row count, bf16 and fp32 residual streams."""
    torch.manual_seed(h + rms)
    rows = 1000
    x0 = torch.randn(rows, h, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    res = torch.randn(rows, h, device="cuda", dtype=torch.float32 if res_fp32 else torch.bfloat16, requires_grad=True)
    g = (1 + 0.1 * torch.randn(h, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    b = None if rms else (0.1 * torch.randn(h, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    fn = F.rms_norm if rms else F.layer_norm
    a = (x0, g) if rms else (x0, g, b)
    z, xs = fn(*a, 1e-5, residual=res, prenorm=True)
    assert xs.dtype == res.dtype
    wz, wx = torch.randn_like(z), torch.randn_like(xs)
    leaves = [t for t in (x0, res, g, b) if t is not None]
    grads = torch.autograd.grad([z, xs], leaves, [wz, wx])
    c = [t.detach().cpu().float().requires_grad_(True) for t in leaves]
    ca = (c[0], c[2]) if rms else (c[0], c[2], c[3])
    zr, xr = fn(*ca, 1e-5, residual=c[1], prenorm=True)
    gr = torch.autograd.grad([zr, xr], c, [wz.cpu().float(), wx.cpu().float()])
    assert _rc(z, zr) < 1e-2 and _rc(xs, xr) < 1e-2
    assert (z.float().cpu() - zr).abs().max().item() < 0.1
    for got, ref, name in zip(grads, gr, ("x0", "res", "gamma", "beta")):
        assert _rc(got, ref) < 2e-2, name
    from mist_b200.ops import native
    native.check_status()


@pytest.mark.parametrize("rms", [False, True])
def test_pipelined_norm_parallel_block_and_dropout(rms):
    """Two branches, two norms of one stream, dropout on both branches: the masks are read off the returned
    stream (x = m0 * x0 / (1 - p) + m1 * x1 / (1 - p) + residual) and everything else is checked against them."""
    torch.manual_seed(3)
    rows, h, p = 777, 2560, 0.25
    mk = lambda scale=1.0: (scale * torch.randn(rows, h, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    x0, x1, res = mk(), mk(), mk()
    g0 = torch.ones(h, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g1 = (1 + 0.1 * torch.randn(h, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    b0 = b1 = None
    if not rms:
        b0 = (0.1 * torch.randn(h, device="cuda")).to(torch.bfloat16).requires_grad_(True)
        b1 = (0.1 * torch.randn(h, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    # without dropout: against the CPU path
    z0, z1, xs = F.parallel_residual_norm(x0, x1, res, g0, b0, g1, b1, rms=rms)
    cpu, (r0, r1, rx) = _norm_cpu((x0, x1, res, g0, b0, g1, b1), dict(rms=rms))
    assert _rc(z0, r0) < 1e-2 and _rc(z1, r1) < 1e-2 and _rc(xs, rx) < 1e-2
    w = [torch.randn_like(z0) for _ in range(3)]
    leaves = [t for t in (x0, x1, res, g0, b0, g1, b1) if t is not None]
    got = torch.autograd.grad([z0, z1, xs], leaves, w)
    ref = torch.autograd.grad([r0, r1, rx], [t for t in cpu if t is not None], [t.cpu().float() for t in w])
    for a_, r_ in zip(got, ref):
        assert _rc(a_, r_) < 2e-2
    # with dropout: a zero residual makes the returned stream x0 * mask / (1 - p), which shows the mask
    zero = torch.zeros_like(res).requires_grad_(True)
    z0, z1, xs = F.parallel_residual_norm(x0, None, zero, g0, b0, g1, b1, rms=rms, dropout_p=p, seed=1234)
    kept = xs != 0
    frac = 1.0 - kept.float().mean().item()
    assert abs(frac - p) < 0.01, frac
    z0b, _, xsb = F.parallel_residual_norm(x0, None, zero, g0, b0, g1, b1, rms=rms, dropout_p=p, seed=1234)
    assert torch.equal(xs, xsb) and torch.equal(z0, z0b)          # same seed, same mask
    _, _, xsc = F.parallel_residual_norm(x0, None, zero, g0, b0, g1, b1, rms=rms, dropout_p=p, seed=99)
    assert not torch.equal(xs, xsc)                                # another seed, another mask
    assert _rc(xs, (x0.float() * kept / (1 - p))) < 5e-3
    # the same mask with a residual: stream, both norms and the gradients follow from it
    z0, z1, xs = F.parallel_residual_norm(x0, None, res, g0, b0, g1, b1, rms=rms, dropout_p=p, seed=1234)
    xr = (x0.float() * kept / (1 - p) + res.float()).to(torch.bfloat16)
    assert _rc(xs, xr) < 5e-3
    cpu2, (q0, q1, qx) = _norm_cpu((xr, None, None, g0, b0, g1, b1), dict(rms=rms))
    assert _rc(z0, q0) < 1e-2 and _rc(z1, q1) < 1e-2
    dx0, dres = torch.autograd.grad([xs], [x0, res], [w[2]])
    assert _rc(dres, w[2]) == 0.0
    assert _rc(dx0, (w[2].float() * kept / (1 - p))) < 5e-3
    from mist_b200.ops import native
    native.check_status()
