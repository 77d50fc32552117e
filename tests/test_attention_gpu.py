"""tcgen05 attention forward (and the backward path in use) against fp32 references."""
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


@pytest.mark.parametrize("d", [128, 80, 64, 96])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("block_n", [64, 128])
def test_attn_fwd_packed(d, causal, block_n):
    torch.manual_seed(0)
    b, s, nh = 2, 384, 3
    qkv = torch.randn(b, s, 3, nh, d, device=DEV, dtype=torch.bfloat16)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    scale = 1 / math.sqrt(d)
    o, lse = F.attn_fwd(q, k, v, scale, causal, block_n=block_n)
    o_ref, lse_ref = F._ref_attention(q.float(), k.float(), v.float(), scale, causal)
    assert _rel_err(o, o_ref) < 2e-2
    assert torch.allclose(lse, lse_ref, atol=2e-2, rtol=1e-3)


def test_attn_fwd_ragged_and_gqa():
    torch.manual_seed(1)
    b, sq, nh, nkv, d = 1, 200, 4, 2, 128
    q = torch.randn(b, sq, nh, d, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(b, sq, nkv, d, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(b, sq, nkv, d, device=DEV, dtype=torch.bfloat16)
    o, lse = F.attn_fwd(q, k, v, 0.1, True)
    o_ref, lse_ref = F._ref_attention(q.float(), k.float(), v.float(), 0.1, True)
    assert _rel_err(o, o_ref) < 2e-2
    assert torch.allclose(lse, lse_ref, atol=2e-2, rtol=1e-3)


def test_attn_fwd_long_sequence():
    torch.manual_seed(2)
    b, s, nh, d = 1, 2048, 2, 128
    qkv = torch.randn(b, s, 3, nh, d, device=DEV, dtype=torch.bfloat16)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    o, lse = F.attn_fwd(q, k, v, 1 / math.sqrt(d), True)
    o_ref = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True).transpose(1, 2)
    assert _rel_err(o, o_ref) < 2e-2


@pytest.mark.parametrize("d,rot", [(128, 32), (80, 0)])
def test_attention_qkvpacked_grad(d, rot):
    torch.manual_seed(3)
    b, s, nh = 2, 256, 2
    qkv = torch.randn(b, s, 3, nh, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    rotary = None
    if rot:
        cos, sin = F.rope_tables(s, rot, 10000.0, DEV)
        rotary = (cos, sin, rot)
    g = torch.randn(b, s, nh, d, device=DEV, dtype=torch.bfloat16)
    o = F.attention_qkvpacked(qkv.clone(), rotary=rotary)
    # gradient w.r.t. the clone's source
    qkv2 = qkv.detach().clone().requires_grad_(True)
    o2 = F.attention_qkvpacked(qkv2 * 1.0, rotary=rotary)
    o2.backward(g)
    ref_in = qkv.detach().cpu().float().requires_grad_(True)
    rot_cpu = None if rotary is None else (rotary[0].cpu(), rotary[1].cpu(), rot)
    o_ref = F.attention_qkvpacked(ref_in * 1.0, rotary=rot_cpu)
    o_ref.backward(g.cpu().float())
    assert _rel_err(o.cpu(), o_ref) < 2e-2
    assert _rel_err(qkv2.grad.cpu(), ref_in.grad) < 3e-2


def _check_grads(got, ref):
    """Norm-wise and element-wise: a wrong vector at a ragged edge must not hide in the norm."""
    for a, r in zip(got, ref):
        assert _rel_err(a, r) < 3e-2
        assert (a.float() - r.float()).abs().max().item() < 0.06 * r.float().abs().max().item() + 1e-3


@pytest.mark.parametrize("pipelined", [True, False])
@pytest.mark.parametrize("d", [80, 64, 96, 128])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("s", [64, 256, 1000, 2048])
def test_attn_bwd_matches_reference(d, causal, s, pipelined):
    """Both backward kernels (the pipelined one is the default) against the fp32 reference, at short,
    ragged and long sequences, every supported head size, causal and not."""
    from mist_b200.ops import attention_bwd, native
    torch.manual_seed(4)
    b, nh = (2, 3) if s <= 1000 else (1, 2)
    scale = 1 / math.sqrt(d)
    q, k, v, g = (torch.randn(b, s, nh, d, device=DEV, dtype=torch.bfloat16) for _ in range(4))
    o, lse = F.attn_fwd(q, k, v, scale, causal)
    old = F.Settings.attn_bwd_pipelined
    F.Settings.attn_bwd_pipelined = pipelined
    try:
        dq, dk, dv = attention_bwd.backward(g, q, k, v, o, lse, scale, causal)
        torch.cuda.synchronize()
        assert native.kernels().mb_attn_bwd_last_variant() == int(pipelined)
    finally:
        F.Settings.attn_bwd_pipelined = old
    native.check_status()
    _check_grads((dq, dk, dv), attention_bwd._reference(g, q, k, v, scale, causal))


@pytest.mark.parametrize("nh,nkv,d,s,causal", [(8, 2, 128, 1024, True), (4, 1, 64, 1000, True), (6, 3, 96, 520, False),
                                               (8, 4, 80, 1031, True)])
def test_attn_bwd_grouped_query_heads(nh, nkv, d, s, causal):
    """Grouped-query attention (several query heads per key/value head): dK and dV sum over the group."""
    from mist_b200.ops import attention_bwd, native
    torch.manual_seed(6)
    b = 2
    scale = 1 / math.sqrt(d)
    q, g = (torch.randn(b, s, nh, d, device=DEV, dtype=torch.bfloat16) for _ in range(2))
    k, v = (torch.randn(b, s, nkv, d, device=DEV, dtype=torch.bfloat16) for _ in range(2))
    o, lse = F.attn_fwd(q, k, v, scale, causal)
    dq, dk, dv = attention_bwd.backward(g, q, k, v, o, lse, scale, causal)
    torch.cuda.synchronize()
    native.check_status()
    _check_grads((dq, dk, dv), attention_bwd._reference(g, q, k, v, scale, causal))


@pytest.mark.parametrize("d", [64, 80, 128])
@pytest.mark.parametrize("causal", [True, False])
def test_right_padded_batch_runs_as_one_launch(d, causal):
    """Per-sample lengths on the device: padded keys are masked, padded query rows are zeros, gradients of
    padded positions are zeros -- against the fp32 reference with the same lengths, forward and backward."""
    from mist_b200.ops import attention_bwd, native
    torch.manual_seed(8)
    b, s, nh = 4, 700, 3
    lens = torch.tensor([700, 1, 333, 512], dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    q, k, v, g = (torch.randn(b, s, nh, d, device=DEV, dtype=torch.bfloat16) for _ in range(4))
    launches = native.launch_count
    o, lse = F.attn_fwd(q, k, v, scale, causal, seqlens_q=lens, seqlens_k=lens)
    assert native.launch_count - launches == 1
    o_ref, lse_ref = F._ref_attention(q.float(), k.float(), v.float(), scale, causal, lens, lens)
    assert _rel_err(o, o_ref) < 2e-2
    for i, n in enumerate(lens.tolist()):
        assert float(o[i, n:].abs().max()) == 0.0 if n < s else True
        assert torch.allclose(lse[i, :, :n], lse_ref[i, :, :n], atol=2e-2, rtol=1e-3)
    dq, dk, dv = attention_bwd.backward(g, q, k, v, o, lse, scale, causal, seqlens=(lens, lens))
    torch.cuda.synchronize()
    native.check_status()
    ref = attention_bwd._reference(g, q, k, v, scale, causal, (lens, lens))
    _check_grads((dq, dk, dv), ref)
    for i, n in enumerate(lens.tolist()):
        if n < s:
            assert float(dq[i, n:].abs().max()) == 0.0 and float(dk[i, n:].abs().max()) == 0.0
            assert float(dv[i, n:].abs().max()) == 0.0


def test_cross_attention_with_padded_keys_and_queries():
    """Decoder queries over encoder keys, both right-padded with their own lengths, through autograd."""
    torch.manual_seed(9)
    b, sq, sk, nh, d = 3, 200, 456, 4, 64
    lq = torch.tensor([200, 77, 130], dtype=torch.int32, device=DEV)
    lk = torch.tensor([456, 300, 9], dtype=torch.int32, device=DEV)
    q = torch.randn(b, sq, nh, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(b, sk, nh, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(b, sk, nh, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(b, sq, nh, d, device=DEV, dtype=torch.bfloat16)
    o = F.attention(q, k, v, None, False, seqlens_q=lq, seqlens_k=lk)
    dq, dk, dv = torch.autograd.grad(o, (q, k, v), g)
    qr, kr, vr = (t.detach().cpu().float().requires_grad_(True) for t in (q, k, v))
    o_ref = F.attention(qr, kr, vr, None, False, seqlens_q=lq.cpu(), seqlens_k=lk.cpu())
    rq, rk, rv = torch.autograd.grad(o_ref, (qr, kr, vr), g.cpu().float())
    assert _rel_err(o.cpu(), o_ref) < 2e-2
    _check_grads((dq.cpu(), dk.cpu(), dv.cpu()), (rq, rk, rv))


@pytest.mark.parametrize("nh,nkv,d,seq_len", [(8, 8, 128, 300), (8, 2, 64, 5), (4, 4, 80, 1), (16, 4, 256, 1031)])
def test_single_query_attention_over_kv_cache(nh, nkv, d, seq_len):
    """Decode step: one query per sequence against the first ``seq_len`` positions of a cache
    that is a strided view ([b, max_seq, 2, heads, d]), vs fp32 softmax(q K^T) V."""
    from mist_b200.ops import functional as F
    torch.manual_seed(5)
    b, max_seq = 3, 1100
    cache = torch.randn(b, max_seq, 2, nkv, d, device="cuda", dtype=torch.bfloat16)
    q = torch.randn(b, nh, d, device="cuda", dtype=torch.bfloat16)
    scale = d ** -0.5
    out = F.decode_attention(q, cache[:, :, 0], cache[:, :, 1], seq_len, scale)
    k = cache[:, :seq_len, 0].float().repeat_interleave(nh // nkv, dim=2)
    v = cache[:, :seq_len, 1].float().repeat_interleave(nh // nkv, dim=2)
    s = torch.einsum("bhd,bkhd->bhk", q.float(), k) * scale
    ref = torch.einsum("bhk,bkhd->bhd", torch.softmax(s, dim=-1), v)
    err = ((out.float() - ref).norm() / ref.norm()).item()
    assert err < 1e-2, err
