"""Attention backward dispatch.

Given ``dout`` and what the forward saved (q, k, v, o and the per-row logsumexp) this
produces dq, dk, dv.  On CUDA the tcgen05 backward kernel is used when the library
exports it; otherwise the gradients come from a library attention kernel
(``torch`` scaled-dot-product attention re-run under autograd), which is the A/B
baseline and the interim path.  On CPU a plain fp32 recomputation is used.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

import ctypes as C

from . import native
from .native import call, ptr, stream

native.register_signature("mb_attn_bwd_set_variant", [C.c_int], None)
native.register_signature("mb_attn_bwd_last_variant", [], C.c_int)


def _reference(dout, q, k, v, scale, causal, seqlens=(None, None)):
    from .functional import _ref_attention
    qq, kk, vv = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    with torch.enable_grad():
        out, _ = _ref_attention(qq, kk, vv, scale, causal, *seqlens)
    dq, dk, dv = torch.autograd.grad(out, (qq, kk, vv), dout.float())
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def _library(dout, q, k, v, scale, causal):
    qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, k, v))
    with torch.enable_grad():
        out = F.scaled_dot_product_attention(
            qq.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), is_causal=causal, scale=scale,
            enable_gqa=(q.shape[2] != k.shape[2]))
    return torch.autograd.grad(out, (qq, kk, vv), dout.transpose(1, 2))


def has_native_backward() -> bool:
    lib = native.kernels()
    return lib is not None and hasattr(lib, "mb_attn_bwd")


def backward(dout, q, k, v, o, lse, scale, causal, out=None, seqlens=(None, None)):
    """Returns (dq, dk, dv); with ``out=(dq, dk, dv)`` writes into those (possibly strided) views.
    ``seqlens``: (per-sample query lengths, per-sample key lengths) of a right-padded batch, or Nones."""
    padded = seqlens[0] is not None or seqlens[1] is not None
    if not q.is_cuda or (padded and not has_native_backward()):
        grads = _reference(dout, q, k, v, scale, causal, seqlens)
    elif has_native_backward():
        from .functional import Settings
        if Settings.attn_backend == "tcgen05":
            if q.shape[2] == k.shape[2]:
                return _native_backward(dout, q, k, v, o, lse, scale, causal, out, seqlens)
            # grouped-query heads: every query head gets its own copy of its group's key / value head,
            # and the gradients of the copies are summed over the group afterwards
            g = q.shape[2] // k.shape[2]
            dq, dk, dv = _native_backward(dout, q, k.repeat_interleave(g, dim=2), v.repeat_interleave(g, dim=2),
                                          o, lse, scale, causal, None, seqlens)
            b, sk, nkv, d = k.shape
            grads = (dq, dk.view(b, sk, nkv, g, d).float().sum(3).to(k.dtype),
                     dv.view(b, sk, nkv, g, d).float().sum(3).to(v.dtype))
        else:
            grads = _reference(dout, q, k, v, scale, causal, seqlens) if padded else _library(dout, q, k, v, scale, causal)
    else:
        grads = _library(dout, q, k, v, scale, causal)
    if out is not None:
        for dst, src in zip(out, grads):
            dst.copy_(src)
        return out
    return grads


def _native_backward(dout, q, k, v, o, lse, scale, causal, out, seqlens=(None, None)):
    b, sq, nh, d = q.shape
    sk = k.shape[1]
    if out is None:
        dq = torch.empty(b, sq, nh, d, dtype=q.dtype, device=q.device)
        dk = torch.empty(b, sk, nh, d, dtype=q.dtype, device=q.device)
        dv = torch.empty(b, sk, nh, d, dtype=q.dtype, device=q.device)
    else:
        dq, dk, dv = out
    dout = dout.contiguous()
    from .functional import Settings, _select_variant
    _select_variant("mb_attn_bwd_set_variant", 1 if Settings.attn_bwd_pipelined else 0)
    delta = torch.empty(b, nh, sq, dtype=torch.float32, device=q.device)
    dq_acc = torch.empty(b, nh, sq, d, dtype=torch.float32, device=q.device)   # zeroed by the launch wrapper
    call("mb_attn_bwd", ptr(dout), ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), ptr(delta), ptr(dq_acc),
         ptr(dq), ptr(dk), ptr(dv), b, sq, sk, nh, d,
         q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
         v.stride(0), v.stride(1), v.stride(2),
         dq.stride(0), dq.stride(1), dq.stride(2), dk.stride(0), dk.stride(1), dk.stride(2),
         dv.stride(0), dv.stride(1), dv.stride(2), float(scale), int(causal), ptr(seqlens[0]), ptr(seqlens[1]),
         stream())
    return dq, dk, dv
