"""Differentiable front ends of the sm_100a kernels.

Every op has two implementations with the same semantics:

* CUDA tensors run the hand-written kernels of ``mist_b200/csrc`` (through
  :mod:`mist_b200.ops.native`); a missing library on a GPU machine raises.
* CPU tensors run a plain PyTorch reference, which is also the oracle that the GPU
  numerics tests compare against.

The ops mirror the fused operators the reference's module library is built on
(reference: mist/modules/fused_dense.py:41-186 FusedDenseFunc, mist/modules/layer_norm.py:
19-118 dropout_add_layer_norm, mist/modules/rotary.py:44-65, mist/modules/activations.py:
115-149 swiglu, mist/modules/losses.py:48-176, mist/modules/flash_attn.py:46-213).
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import torch
import torch.nn.functional as F

from . import native
from .native import call, ptr, stream, use_native


def _sym(*xs):
    """True when any argument is a shape-symbolic tensor of the analyzer (then the op is
    recorded by its symbolic rule instead of being executed)."""
    for x in xs:
        if x is not None and type(x).__name__ == "SymTensor":
            return True
    return False


def _rules():
    from ..analyzer import rules
    return rules

# --------------------------------------------------------------------------- settings
EPI_BIAS, EPI_GELU, EPI_SAVE_PRE, EPI_ACCUM, EPI_DGELU, EPI_OUT_FP32, EPI_RESIDUAL = 1, 2, 4, 8, 16, 32, 64


class Settings:
    """Process-wide kernel selection switches."""
    gemm_backend = "tcgen05"      # "tcgen05" (ours) | "cublas" (library, A/B baseline)
    attn_backend = "tcgen05"      # "tcgen05" (ours) | "sdpa" (library, A/B baseline)
    attn_block_n = 64
    # Backward kernel that overlaps the next block's S / dP products with the current block's softmax
    # (6 % faster than the unpipelined kernel at head sizes 80 and 128; MIST_B200_ATTN_BWD_PIPELINED=0
    # selects the unpipelined one).
    attn_bwd_pipelined = os.environ.get("MIST_B200_ATTN_BWD_PIPELINED", "1") != "0"
    gemm_max_ctas = 0             # >0 leaves SMs free for a concurrent communication kernel
    gemm_pair = True              # large GEMMs on CTA pairs (256 x 256 tiles, tcgen05 cta_group::2)
    fuse_mlp_gelu = True          # GELU MLP as one autograd node (gelu' folded into a dgrad GEMM epilogue)
    tp_backend = "nccl"           # "nccl" | "fused": sequence-parallel linears on the GEMM+collective kernels
    # Norms on the bulk-copy pipelined kernels (csrc/norm_pipe.cu): "always", "never", or "auto" = only where
    # their extra options are used (dropout inside the kernel, two norms of one stream, an fp32 residual
    # stream); MB_NORM_PIPE=1 / 0 selects always / never.
    norm_pipe = {"1": "always", "0": "never"}.get(os.environ.get("MB_NORM_PIPE", ""), "auto")
    dropout_seed_offset = 0       # added to every drawn seed; differs per rank only where tokens are sharded


def next_dropout_seed() -> int:
    """Seed for one dropout call, drawn from torch's CPU generator.  The training session seeds that
    generator alike on every rank of a tensor-parallel group, so replicated activations get the same mask
    on every rank; and it is the generator whose state activation checkpointing saves and restores, so a
    recomputed forward pass draws the seeds of the original one."""
    s = int(torch.randint(0, 2 ** 31 - 1, (1,)).item())
    return (s + Settings.dropout_seed_offset) % (2 ** 31 - 1)


_scratch = {}


def _get_scratch(numel: int, device, key="default") -> torch.Tensor:
    """fp32 scratch that grows on demand; one buffer per (device, key)."""
    k = (device, key)
    buf = _scratch.get(k)
    if buf is None or buf.numel() < numel:
        buf = torch.empty(max(numel, 1 << 20), dtype=torch.float32, device=device)
        _scratch[k] = buf
    return buf


# ------------------------------------------------------------------------------ GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16, bias=None, aux=None,
         flags: int = 0, alpha: float = 1.0, tile_n: int = 0) -> torch.Tensor:
    """``C[M,N] = A * B^T`` on tcgen05.

    ``a`` is ``[M,K]`` (K-major) or, with ``a_mn``, stored ``[K,M]``; ``b`` is ``[N,K]``
    or, with ``b_mn``, stored ``[K,N]``.  Both must be 2-D bf16 with unit inner stride.
    """
    assert a.dim() == 2 and b.dim() == 2 and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(1) == 1 and b.stride(1) == 1
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else b.shape
    assert K == Kb, (a.shape, b.shape, a_mn, b_mn)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    assert out.stride(1) == 1 and out.shape == (M, N)
    if out.dtype == torch.float32:
        flags |= EPI_OUT_FP32
    if bias is not None:
        flags |= EPI_BIAS
    if Settings.gemm_pair and tile_n == 0:
        # returns 1 (nothing launched) when the shape or epilogue needs the single-CTA kernel
        rc = native.kernels().mb_gemm_pair_bf16(ptr(a), ptr(b), ptr(out), M, N, K, a.stride(0), b.stride(0),
                                                out.stride(0), int(a_mn), int(b_mn), flags, ptr(bias), ptr(aux),
                                                float(alpha), Settings.gemm_max_ctas, stream())
        if rc == 0:
            native.launch_count += 1
            return out
        if rc != 1:
            detail = ""
            if rc <= -21:        # a tensor map could not be encoded: the library kept the call's arguments
                info = native.kernels().mb_gemm_pair_last_error
                info.restype = ctypes.c_char_p
                detail = f" ({info().decode()})"
            raise RuntimeError(f"mb_gemm_pair_bf16 failed with code {rc}{detail}")
    call("mb_gemm_bf16", ptr(a), ptr(b), ptr(out), M, N, K, a.stride(0), b.stride(0), out.stride(0),
         int(a_mn), int(b_mn), flags, ptr(bias), ptr(aux), float(alpha), tile_n,
         Settings.gemm_max_ctas, stream())
    return out


def _ref_act(x, activation):
    if activation == "gelu":
        return F.gelu(x, approximate="tanh")
    return x


class _LinearFn(torch.autograd.Function):
    """y = act(x W^T + b); wgrad may accumulate straight into a flat gradient bucket."""

    @staticmethod
    def forward(ctx, x, weight, bias, activation, residual):
        ctx.activation = activation
        ctx.has_bias = bias is not None
        ctx.has_residual = residual is not None
        xs = x.shape
        x2 = x.reshape(-1, xs[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        pre = None
        if not use_native(x2):
            y = F.linear(x2.float(), weight.float(), None if bias is None else bias.float())
            if activation == "gelu":
                pre = y.to(x.dtype)
                y = _ref_act(pre.float(), activation)
            if residual is not None:
                y = y + residual.reshape(-1, weight.shape[0]).float()
            y = y.to(x.dtype)
        elif Settings.gemm_backend == "cublas":
            y = F.linear(x2, weight, bias)
            if activation == "gelu":
                pre = y
                y = F.gelu(pre, approximate="tanh")
            if residual is not None:
                y = y + residual.reshape(-1, weight.shape[0])
        else:
            flags = 0
            aux = None
            if activation == "gelu":
                pre = torch.empty(x2.shape[0], weight.shape[0], dtype=x.dtype, device=x.device)
                aux = pre
                flags |= EPI_GELU | EPI_SAVE_PRE
            elif residual is not None:
                aux = residual.reshape(-1, weight.shape[0])
                assert aux.is_contiguous()
                flags |= EPI_RESIDUAL
            fused_gather = getattr(weight, "param_gather", None)
            if fused_gather is not None and flags != 0:
                raise RuntimeError("the weight-gathering GEMM has no activation / residual epilogue")
            if fused_gather is not None:
                # ZeRO-3: this GEMM also brings in the block's remote weight shards
                weight.param_gather = None
                y = fused_gather(x2)
            else:
                y = gemm(x2, weight, bias=bias, aux=aux, flags=flags)
        ctx.save_for_backward(x2, weight, pre)
        return y.reshape(*xs[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight, pre = ctx.saved_tensors
        dys = dy.shape
        dy2 = dy.reshape(-1, dys[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        native_path = use_native(dy2)
        tc = native_path and Settings.gemm_backend != "cublas"
        d_res = dy if ctx.has_residual else None
        # activation backward (standalone kernel; the pre-activation was saved by the forward)
        if ctx.activation == "gelu":
            dy2 = gelu_bwd(dy2, pre)
        dbias = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            dbias = colsum(dy2)
        dx = None
        if ctx.needs_input_grad[0]:
            if tc:
                dx = gemm(dy2, weight, b_mn=True)
            else:
                dx = (dy2.float() @ weight.float()).to(dy.dtype) if not native_path else dy2 @ weight
            dx = dx.reshape(*dys[:-1], weight.shape[1])
        dw = None
        if ctx.needs_input_grad[1]:
            bucket = getattr(weight, "grad_bucket", None)
            if bucket is not None:
                accumulate = bool(getattr(weight, "grad_accumulate", False))
                if tc:
                    gemm(dy2, x2, a_mn=True, b_mn=True, out=bucket,
                         flags=EPI_ACCUM if accumulate else 0)
                else:
                    g = dy2.t().float() @ x2.float() if not native_path else dy2.t() @ x2
                    if accumulate:
                        bucket.add_(g.to(bucket.dtype))
                    else:
                        bucket.copy_(g)
                weight.grad_accumulate = True
            else:
                if tc:
                    dw = gemm(dy2, x2, a_mn=True, b_mn=True)
                else:
                    dw = (dy2.t().float() @ x2.float()).to(weight.dtype) if not native_path \
                        else dy2.t() @ x2
        return dx, dw, dbias, None, d_res


def linear(x, weight, bias=None, activation: Optional[str] = None, residual=None):
    """``act(x @ weight.T + bias) (+ residual)`` with the three GEMMs on tcgen05."""
    if _sym(x):
        return _rules().linear(x, weight, bias, activation, residual)
    return _LinearFn.apply(x, weight, bias, activation, residual)


class _MlpGeluFn(torch.autograd.Function):
    """``gelu(x W1^T + b1) W2^T + b2`` as one autograd node, so the backward pass can fold
    GELU's derivative into the epilogue of the GEMM that produces the gradient of the
    activations: ``dpre = (dy W2) * gelu'(pre)`` in one kernel instead of a GEMM followed by an
    elementwise pass over the ``[tokens, ffn]`` tensor (reference: the cuBLASLt ``DGELU_BGRAD``
    epilogue behind ``bias_act_linear_dgrad_bgrad``, csrc/fused_dense_lib/fused_dense_cuda.cu:
    407-520, used by mist/modules/fused_dense.py:386-480 ``FusedMLPFunc``)."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2):
        xs = x.shape
        x2 = x.reshape(-1, xs[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        pre = torch.empty(x2.shape[0], w1.shape[0], dtype=x.dtype, device=x.device)
        act = gemm(x2, w1, bias=b1, aux=pre, flags=EPI_GELU | EPI_SAVE_PRE)
        y = gemm(act, w2, bias=b2)
        ctx.save_for_backward(x2, w1, w2, pre, act)
        ctx.has_b1, ctx.has_b2 = b1 is not None, b2 is not None
        return y.reshape(*xs[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w1, w2, pre, act = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()

        def wgrad(g, inp, weight):
            bucket = getattr(weight, "grad_bucket", None)
            if bucket is None:
                return gemm(g, inp, a_mn=True, b_mn=True)
            gemm(g, inp, a_mn=True, b_mn=True, out=bucket,
                 flags=EPI_ACCUM if getattr(weight, "grad_accumulate", False) else 0)
            weight.grad_accumulate = True
            return None

        db2 = colsum(dy2) if (ctx.has_b2 and ctx.needs_input_grad[4]) else None
        dw2 = wgrad(dy2, act, w2) if ctx.needs_input_grad[3] else None
        dpre = gemm(dy2, w2, b_mn=True, aux=pre, flags=EPI_DGELU)      # (dy W2) * gelu'(pre)
        db1 = colsum(dpre) if (ctx.has_b1 and ctx.needs_input_grad[2]) else None
        dw1 = wgrad(dpre, x2, w1) if ctx.needs_input_grad[1] else None
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dpre, w1, b_mn=True).reshape(*dy.shape[:-1], w1.shape[1])
        return dx, dw1, db1, dw2, db2


def mlp_gelu_fused_available(x) -> bool:
    return (Settings.fuse_mlp_gelu and (not _sym(x)) and use_native(x) and Settings.gemm_backend == "tcgen05"
            and x.dtype == torch.bfloat16)


def mlp_gelu(x, w1, b1, w2, b2):
    """Two-layer GELU MLP; one fused autograd node on the tcgen05 path, two linears otherwise."""
    if mlp_gelu_fused_available(x):
        return _MlpGeluFn.apply(x, w1, b1, w2, b2)
    return linear(linear(x, w1, b1, activation="gelu"), w2, b2)


# ---------------------------------------------------------------- column sum (bias grad)
def colsum(x2: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False):
    rows, cols = x2.shape
    if not use_native(x2):
        s = x2.float().sum(0)
        if out is None:
            return s.to(x2.dtype)
        out.copy_(out.float() + s if accumulate else s)
        return out
    x2 = x2.contiguous()      # gradients of reductions arrive as stride-0 expansions
    if out is None:
        out = torch.empty(cols, dtype=x2.dtype, device=x2.device)
    parts = (rows + 255) // 256
    scratch = _get_scratch(parts * cols, x2.device, "colsum")
    call("mb_colsum", ptr(x2), ptr(out), ptr(scratch), rows, cols, int(out.dtype == torch.float32),
         int(accumulate), stream())
    return out


# ------------------------------------------------------------------------- activations
def gelu_fwd(x, bias=None):
    if not use_native(x):
        xx = x.float() if bias is None else x.float() + bias.float()
        return F.gelu(xx, approximate="tanh").to(x.dtype)
    x = x.contiguous()
    y = torch.empty_like(x)
    call("mb_gelu_fwd", ptr(x), ptr(bias), ptr(y), x.numel() // x.shape[-1], x.shape[-1], stream())
    return y


def gelu_bwd(dy, x, bias=None):
    if not use_native(dy):
        xx = (x.float() if bias is None else x.float() + bias.float()).requires_grad_(True)
        with torch.enable_grad():
            y = F.gelu(xx, approximate="tanh")
        (g,) = torch.autograd.grad(y, xx, dy.float())
        return g.to(dy.dtype)
    dy = dy.contiguous()
    dx = torch.empty_like(dy)
    call("mb_gelu_bwd", ptr(dy), ptr(x), ptr(bias), ptr(dx), dy.numel() // dy.shape[-1], dy.shape[-1],
         stream())
    return dx


class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias):
        ctx.save_for_backward(x, bias)
        return gelu_fwd(x, bias)

    @staticmethod
    def backward(ctx, dy):
        x, bias = ctx.saved_tensors
        dx = gelu_bwd(dy, x, bias)
        db = colsum(dx.reshape(-1, dx.shape[-1])) if bias is not None else None
        return dx, db


def gelu(x, bias=None):
    if _sym(x):
        return _rules().gelu(x, bias)
    return _GeluFn.apply(x, bias)


class _SwigluFn(torch.autograd.Function):
    """[..., 2F] = [gate | up]  ->  silu(gate) * up"""

    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        F_ = x.shape[-1] // 2
        if not use_native(x):
            g, u = x.float().chunk(2, dim=-1)
            return (F.silu(g) * u).to(x.dtype)
        x = x.contiguous()
        out = torch.empty(*x.shape[:-1], F_, dtype=x.dtype, device=x.device)
        call("mb_swiglu_fwd", ptr(x), ptr(out), x.numel() // x.shape[-1], F_, stream())
        return out

    @staticmethod
    def backward(ctx, dout):
        (x,) = ctx.saved_tensors
        F_ = x.shape[-1] // 2
        if not use_native(x):
            g, u = x.float().chunk(2, dim=-1)
            s = torch.sigmoid(g)
            d = dout.float()
            dg = d * u * (s + g * s * (1 - s))
            du = d * g * s
            return torch.cat([dg, du], dim=-1).to(x.dtype)
        dout = dout.contiguous()
        din = torch.empty_like(x)
        call("mb_swiglu_bwd", ptr(dout), ptr(x), ptr(din), x.numel() // x.shape[-1], F_, stream())
        return din


def swiglu(x):
    if _sym(x):
        return _rules().swiglu(x)
    return _SwigluFn.apply(x)


class _BiasDropoutAddFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, residual, p, seed):
        ctx.p, ctx.seed = p, seed
        ctx.has_bias, ctx.has_res = bias is not None, residual is not None
        if not use_native(x):
            y = x.float() if bias is None else x.float() + bias.float()
            if p > 0:
                gen = torch.Generator(device=x.device).manual_seed(seed)
                mask = (torch.rand(y.shape, generator=gen, device=x.device) >= p).float() / (1 - p)
                ctx.mask = mask
                y = y * mask
            if residual is not None:
                y = y + residual.float()
            return y.to(x.dtype)
        x = x.contiguous()
        out = torch.empty_like(x)
        call("mb_bias_dropout_add", ptr(x), ptr(bias), ptr(residual), ptr(out),
             x.numel() // x.shape[-1], x.shape[-1], float(p), int(seed), stream())
        return out

    @staticmethod
    def backward(ctx, dout):
        dres = dout if ctx.has_res else None
        if ctx.p > 0:
            if not use_native(dout):
                dx = (dout.float() * ctx.mask).to(dout.dtype)
            else:
                dout = dout.contiguous()
                dx = torch.empty_like(dout)
                call("mb_dropout_bwd", ptr(dout), ptr(dx), dout.numel(), float(ctx.p), int(ctx.seed),
                     stream())
        else:
            dx = dout
        db = colsum(dx.reshape(-1, dx.shape[-1])) if ctx.has_bias else None
        return dx, db, dres, None, None


def bias_dropout_add(x, bias, residual, p: float = 0.0, seed: int = 0):
    """``residual + dropout(x + bias, p)``; the mask is regenerated, not stored."""
    if _sym(x, residual):
        return _rules().bias_dropout_add(x, bias, residual, p, seed)
    return _BiasDropoutAddFn.apply(x, bias, residual, float(p), int(seed))


# ------------------------------------------------------------------------------- norms
def _ref_norm(x, gamma, beta, eps, rms):
    xf = x.float()
    if rms:
        rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        return (xf * rstd * gamma.float()), None, rstd
    mean = xf.mean(-1, keepdim=True)
    var = xf.var(-1, unbiased=False, keepdim=True)
    rstd = torch.rsqrt(var + eps)
    z = (xf - mean) * rstd * gamma.float()
    if beta is not None:
        z = z + beta.float()
    return z, mean, rstd


def _keep_mask(seed: int, shape, p: float, device, second: bool = False):
    """Dropout mask of the reference (CPU) path: reproducible from the seed, one stream per branch."""
    gen = torch.Generator(device="cpu").manual_seed((int(seed) + (0x5DEECE66D if second else 0)) & 0x7FFFFFFFFFFFFFFF)
    return (torch.rand(shape, generator=gen) >= p).to(device)


class _NormFn(torch.autograd.Function):
    """``z = norm(dropout(x0) [+ dropout(x1)] [+ residual])`` and, for parallel blocks, a second norm ``z1``
    of the same stream with its own weights; optionally returns the sum as the new residual stream.

    The residual stream may be fp32 while the branches and the outputs are bf16
    (``residual_in_fp32`` of the reference, mist/modules/layer_norm.py:28, 133, 241).  Dropout masks are
    not stored: the backward pass regenerates them from ``seed``.  One kernel per pass
    (csrc/norm_pipe.cu); shapes it does not take, and runs with ``MB_NORM_PIPE=0``, use the older
    kernels of csrc/norm.cu, which cover the plain form only."""

    @staticmethod
    def forward(ctx, x0, residual, gamma, beta, eps, rms, prenorm, x1=None, gamma1=None, beta1=None,
                dropout_p=0.0, seed=0):
        ctx.rms, ctx.prenorm = rms, prenorm
        ctx.has_res = residual is not None
        ctx.has_beta = beta is not None
        ctx.has_x1, ctx.parallel, ctx.has_beta1 = x1 is not None, gamma1 is not None, beta1 is not None
        ctx.p, ctx.seed = float(dropout_p), int(seed)
        shp = x0.shape
        h = shp[-1]
        x0_2 = x0.reshape(-1, h)
        rows = x0_2.shape[0]
        res_fp32 = residual is not None and residual.dtype == torch.float32
        ctx.res_fp32 = res_fp32
        extras = ctx.has_x1 or ctx.parallel or ctx.p > 0 or res_fp32
        z1 = None
        if not use_native(x0):
            xf = x0_2.float()
            if ctx.p > 0:
                xf = xf * _keep_mask(seed, xf.shape, ctx.p, xf.device) / (1.0 - ctx.p)
            if x1 is not None:
                yf = x1.reshape(-1, h).float()
                if ctx.p > 0:
                    yf = yf * _keep_mask(seed, yf.shape, ctx.p, yf.device, True) / (1.0 - ctx.p)
                xf = xf + yf
            if residual is not None:
                xf = xf + residual.reshape(-1, h).float()
            x = xf if res_fp32 else xf.to(x0.dtype)
            z, mean, rstd = _ref_norm(x, gamma, beta, eps, rms)
            z = z.to(x0.dtype)
            if gamma1 is not None:
                z1 = _ref_norm(x, gamma1, beta1, eps, rms)[0].to(x0.dtype)
            mean = None if mean is None else mean.reshape(-1)
            rstd = rstd.reshape(-1)
        else:
            x0_2 = x0_2.contiguous()
            res2 = None if residual is None else residual.reshape(-1, h).contiguous()
            x1_2 = None if x1 is None else x1.reshape(-1, h).contiguous()
            z = torch.empty_like(x0_2)
            z1 = torch.empty_like(x0_2) if gamma1 is not None else None
            need_x = residual is not None or extras
            x = (torch.empty(rows, h, dtype=torch.float32 if res_fp32 else x0.dtype, device=x0.device)
                 if need_x else x0_2)
            mean = None if rms else torch.empty(rows, dtype=torch.float32, device=x0.device)
            rstd = torch.empty(rows, dtype=torch.float32, device=x0.device)
            rc = 1
            ctx.pipe = Settings.norm_pipe == "always" or (Settings.norm_pipe == "auto" and extras)
            if ctx.pipe:
                rc = native.kernels().mb_norm_fwd_pipe(
                    ptr(x0_2), ptr(x1_2), ptr(res2), ptr(gamma), ptr(beta), ptr(gamma1), ptr(beta1), ptr(z), ptr(z1),
                    ptr(x) if need_x else 0, ptr(mean), ptr(rstd), rows, h, float(eps), int(rms), int(res_fp32),
                    float(ctx.p), int(seed) & 0xFFFFFFFFFFFFFFFF, stream())
                if rc == 0:
                    native.launch_count += 1
                elif rc != 1:
                    raise RuntimeError(f"mb_norm_fwd_pipe failed with code {rc}")
            if rc == 1:
                if extras:
                    raise NotImplementedError("dropout, a second branch, a second norm and an fp32 residual stream "
                                              "need the pipelined norm kernel (hidden size a multiple of 8)")
                call("mb_norm_fwd", ptr(x0_2), ptr(res2), ptr(gamma), ptr(beta), ptr(z),
                     ptr(x) if need_x else 0, ptr(mean), ptr(rstd), rows, h, float(eps), int(rms), stream())
        ctx.save_for_backward(x, gamma, mean, rstd, gamma1)
        ctx.branch_dtype = x0.dtype
        outs = [z.reshape(shp)]
        if gamma1 is not None:
            outs.append(z1.reshape(shp))
        if prenorm:
            outs.append(x.reshape(shp))
        return outs[0] if len(outs) == 1 else tuple(outs)

    @staticmethod
    def backward(ctx, dz, *args):
        x, gamma, mean, rstd, gamma1 = ctx.saved_tensors
        args = list(args)
        dz1 = args.pop(0) if ctx.parallel else None
        dres_in = args.pop(0) if (ctx.prenorm and args) else None
        shp = dz.shape
        h = shp[-1]
        dz2 = dz.reshape(-1, h)
        rows = dz2.shape[0]
        dgamma1 = dbeta1 = None
        bdt = ctx.branch_dtype
        split = ctx.p > 0 or ctx.res_fp32          # branch gradients differ from the stream's gradient
        if not use_native(dz):
            xf = x.reshape(-1, h).float()
            xh = xf * rstd[:, None] if ctx.rms else (xf - mean[:, None]) * rstd[:, None]
            dy = dz2.float() * gamma.float()
            if dz1 is not None:
                dy = dy + dz1.reshape(-1, h).float() * gamma1.float()
            m1 = 0.0 if ctx.rms else dy.mean(-1, keepdim=True)
            m2 = (dy * xh).mean(-1, keepdim=True)
            dxf = rstd[:, None] * (dy - m1 - xh * m2)
            if dres_in is not None:
                dxf = dxf + dres_in.reshape(-1, h).float()
            dx = dxf.to(x.dtype)
            dgamma = (dz2.float() * xh).sum(0).to(gamma.dtype)
            dbeta = dz2.float().sum(0).to(gamma.dtype) if ctx.has_beta else None
            if dz1 is not None:
                dgamma1 = (dz1.reshape(-1, h).float() * xh).sum(0).to(gamma.dtype)
                dbeta1 = dz1.reshape(-1, h).float().sum(0).to(gamma.dtype) if ctx.has_beta1 else None
            dx0 = dx1 = None
            if split:
                dx0 = dxf
                if ctx.p > 0:
                    dx0 = dxf * _keep_mask(ctx.seed, dxf.shape, ctx.p, dxf.device) / (1.0 - ctx.p)
                dx0 = dx0.to(bdt)
                if ctx.has_x1:
                    dx1 = dxf
                    if ctx.p > 0:
                        dx1 = dxf * _keep_mask(ctx.seed, dxf.shape, ctx.p, dxf.device, True) / (1.0 - ctx.p)
                    dx1 = dx1.to(bdt)
        else:
            dz2 = dz2.contiguous()
            dz1_2 = None if dz1 is None else dz1.reshape(-1, h).contiguous()
            dr = None if dres_in is None else dres_in.reshape(-1, h).contiguous()
            dgamma = torch.empty_like(gamma)
            dbeta = torch.empty_like(gamma) if ctx.has_beta else None
            lib = native.kernels()
            parts = lib.mb_norm_pipe_parts(rows, h, int(ctx.res_fp32), int(dz1 is not None), int(dr is not None),
                                           int(ctx.rms)) if getattr(ctx, "pipe", False) else 0
            dx0 = dx1 = None
            if parts > 0:
                need_stream = ctx.has_res or not split
                dx = torch.empty(rows, h, dtype=x.dtype, device=dz.device) if need_stream else None
                if split:
                    dx0 = torch.empty(rows, h, dtype=bdt, device=dz.device)
                    dx1 = torch.empty(rows, h, dtype=bdt, device=dz.device) if ctx.has_x1 else None
                nvecs = 2 * (2 if dz1 is not None else 1)
                scratch = _get_scratch(nvecs * parts * h, dz.device, "norm")
                pg, pb = scratch[: parts * h], scratch[parts * h: 2 * parts * h]
                pg1 = scratch[2 * parts * h: 3 * parts * h] if dz1 is not None else None
                pb1 = scratch[3 * parts * h: 4 * parts * h] if dz1 is not None else None
                call("mb_norm_bwd_pipe", ptr(dz2), ptr(dz1_2), ptr(x), ptr(dr), ptr(gamma), ptr(gamma1), ptr(mean),
                     ptr(rstd), ptr(dx), ptr(dx0), ptr(dx1), ptr(pg), ptr(pb), ptr(pg1), ptr(pb1), rows, h,
                     int(ctx.rms), int(ctx.res_fp32), float(ctx.p), ctx.seed & 0xFFFFFFFFFFFFFFFF, stream())
                call("mb_norm_bwd_finalize", ptr(pg), ptr(pb) if ctx.has_beta else 0, ptr(dgamma), ptr(dbeta), parts, h,
                     stream())
                if dz1 is not None:
                    dgamma1 = torch.empty_like(gamma)
                    dbeta1 = torch.empty_like(gamma) if ctx.has_beta1 else None
                    call("mb_norm_bwd_finalize", ptr(pg1), ptr(pb1) if ctx.has_beta1 else 0, ptr(dgamma1), ptr(dbeta1),
                         parts, h, stream())
            else:
                if split or dz1 is not None:
                    raise NotImplementedError("this shape needs the pipelined norm kernel for its options")
                dx = torch.empty_like(dz2)
                nrows = lib.mb_norm_bwd_scratch_rows(rows, h)
                scratch = _get_scratch(2 * nrows * h, dz.device, "norm")
                call("mb_norm_bwd", ptr(dz2), ptr(x), ptr(gamma), ptr(mean), ptr(rstd), ptr(dr), ptr(dx),
                     ptr(dgamma), ptr(dbeta), ptr(scratch), rows, h, int(ctx.rms), 0, stream())
        g_x0 = (dx0 if split else dx).reshape(shp)
        g_res = dx.reshape(shp) if ctx.has_res else None
        g_x1 = None
        if ctx.has_x1:
            g_x1 = (dx1 if split else dx).reshape(shp)
        return g_x0, g_res, dgamma, dbeta, None, None, None, g_x1, dgamma1, dbeta1, None, None


def layer_norm(x, gamma, beta, eps=1e-5, residual=None, prenorm=False, dropout_p: float = 0.0, seed: int = 0):
    """``norm(dropout(x) + residual)``; with ``prenorm`` also returns the sum (the new residual stream,
    in the residual's dtype: bf16 or fp32)."""
    if _sym(x):
        return _rules().norm(x, residual, gamma, beta, eps, False, prenorm)
    return _NormFn.apply(x, residual, gamma, beta, eps, False, prenorm, None, None, None, float(dropout_p), int(seed))


def rms_norm(x, gamma, eps=1e-5, residual=None, prenorm=False, dropout_p: float = 0.0, seed: int = 0):
    if _sym(x):
        return _rules().norm(x, residual, gamma, None, eps, True, prenorm)
    return _NormFn.apply(x, residual, gamma, None, eps, True, prenorm, None, None, None, float(dropout_p), int(seed))


def parallel_residual_norm(x0, x1, residual, gamma0, beta0, gamma1, beta1, eps=1e-5, rms=False,
                           dropout_p: float = 0.0, seed: int = 0):
    """Parallel blocks (attention and MLP read the same stream): ``x = dropout(x0) + dropout(x1) + residual``,
    ``z0 = norm(x; gamma0, beta0)``, ``z1 = norm(x; gamma1, beta1)``, one kernel.  Returns ``(z0, z1, x)``;
    ``x1`` and ``residual`` may be ``None``; ``gamma1 = None`` gives ``(z0, x)`` (reference:
    ``dropout_add_ln_parallel_residual_fwd / bwd``, csrc/layer_norm/ln_api.cpp:832-846, used at
    mist/modules/layer_norm.py:808)."""
    return _NormFn.apply(x0, residual, gamma0, None if rms else beta0, eps, rms, True, x1, gamma1,
                         None if rms else beta1, float(dropout_p), int(seed))


# ------------------------------------------------------------------------------ rotary
_rope_cache = {}


def rope_tables(seq: int, rot_dim: int, base: float, device):
    key = (seq, rot_dim, base, str(device))
    if key not in _rope_cache:
        inv = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device) / rot_dim))
        t = torch.arange(seq, dtype=torch.float32, device=device)
        fr = torch.outer(t, inv)
        _rope_cache[key] = (fr.cos().contiguous(), fr.sin().contiguous())
    return _rope_cache[key]


def _rope_apply(qkv, cos, sin, rot, conj, n_rot):
    # qkv: [b, s, 3, nh, d] (or [b, s, n, nh, d]); rotate slots [0, n_rot)
    b, s, n3, nh, d = qkv.shape
    if not use_native(qkv):
        out = qkv.clone()
        x = qkv[:, :, :n_rot, :, :rot].float()
        x1, x2 = x[..., : rot // 2], x[..., rot // 2:]
        c = cos[:s].view(1, s, 1, 1, rot // 2)
        sn = sin[:s].view(1, s, 1, 1, rot // 2)
        if conj:
            sn = -sn
        out[:, :, :n_rot, :, : rot // 2] = (x1 * c - x2 * sn).to(qkv.dtype)
        out[:, :, :n_rot, :, rot // 2: rot] = (x1 * sn + x2 * c).to(qkv.dtype)
        return out
    assert qkv.is_contiguous()
    call("mb_rope", ptr(qkv), ptr(cos), ptr(sin), b * s, s, nh, d, rot, int(conj), n_rot, n3 * nh * d,
         stream())
    return qkv


def apply_rotary_qkv_(qkv, cos, sin, rot_dim: int, conj: bool = False):
    """Rotates q and k of a packed ``[b, s, 3, heads, d]`` tensor (in place on CUDA).
    Not differentiable by itself: :func:`attention_qkvpacked` applies it inside its
    forward and its conjugate inside its backward."""
    return _rope_apply(qkv, cos, sin, rot_dim, conj, 2)


# --------------------------------------------------------------------------- attention
def decode_attention(q, k_cache, v_cache, seq_len: int, scale: Optional[float] = None):
    """One new query per sequence against the first ``seq_len`` cached positions (no autograd).

    ``q``: ``[b, nh, d]``; ``k_cache`` / ``v_cache``: ``[b, max_seq, nh_kv, d]`` (views with unit
    stride along ``d`` are fine).  Returns ``[b, nh, d]``."""
    b, nh, d = q.shape
    nkv = k_cache.shape[2]
    scale = float(scale if scale is not None else 1.0 / math.sqrt(d))
    if not (use_native(q) and q.dtype == torch.bfloat16 and d % 8 == 0 and d <= 256
            and k_cache.stride(3) == 1 and v_cache.stride(3) == 1
            and all(st % 8 == 0 for st in k_cache.stride()[:3] + v_cache.stride()[:3])):
        k = k_cache[:, :seq_len].float()
        v = v_cache[:, :seq_len].float()
        if nkv != nh:
            k = k.repeat_interleave(nh // nkv, dim=2)
            v = v.repeat_interleave(nh // nkv, dim=2)
        s = torch.einsum("bhd,bkhd->bhk", q.float(), k) * scale
        return torch.einsum("bhk,bkhd->bhd", torch.softmax(s, dim=-1), v).to(q.dtype)
    q = q.contiguous()
    out = torch.empty_like(q)
    ks, vs = k_cache.stride(), v_cache.stride()
    call("mb_decode_attn", ptr(q), ptr(k_cache), ptr(v_cache), ptr(out), b, nh, nkv, d, int(seq_len),
         ks[0], ks[1], ks[2], vs[0], vs[1], vs[2], scale, stream())
    return out


def _ref_attention(q, k, v, scale, causal, seqlens_q=None, seqlens_k=None):
    # q: [b, sq, nh, d]; k, v: [b, sk, nh_kv, d]; seqlens_*: [b] real tokens per sample (right padding)
    b, sq, nh, d = q.shape
    sk, nkv = k.shape[1], k.shape[2]
    if nkv != nh:
        k = k.repeat_interleave(nh // nkv, dim=2)
        v = v.repeat_interleave(nh // nkv, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    lq = torch.full((b,), sq, device=q.device) if seqlens_q is None else seqlens_q.to(q.device).long().clamp(max=sq)
    lk = torch.full((b,), sk, device=q.device) if seqlens_k is None else seqlens_k.to(q.device).long().clamp(max=sk)
    qi = torch.arange(sq, device=q.device)[None, :, None]
    kj = torch.arange(sk, device=q.device)[None, None, :]
    visible = kj < lk[:, None, None]
    if causal:      # aligned at the end of each sample's real tokens
        visible = visible & (kj <= qi + (lk - lq)[:, None, None])
    real_q = (qi < lq[:, None, None])
    s = s.masked_fill(~(visible & real_q)[:, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.softmax(s, dim=-1).nan_to_num(0.0)      # rows without a visible key (padding) give zeros
    o = torch.einsum("bhqk,bkhd->bqhd", p, v.float())
    return o.to(q.dtype), lse


_VARIANTS = {}


def _select_variant(setter: str, want: int):
    """Tells the library which kernel variant to launch; only called when the choice changes
    (the library starts with variant 0)."""
    if _VARIANTS.get(setter, 0) != want:
        getattr(native.kernels(), setter)(want)
        _VARIANTS[setter] = want


def attn_fwd(q, k, v, scale, causal, block_n=None, seqlens_q=None, seqlens_k=None):
    """Forward only: returns (o [b,sq,nh,d], lse [b,nh,sq] fp32).  ``seqlens_q`` / ``seqlens_k``: int32
    device tensors ``[b]`` with the number of real tokens of each sample of a right-padded batch."""
    if not use_native(q):
        return _ref_attention(q, k, v, scale, causal, seqlens_q, seqlens_k)
    b, sq, nh, d = q.shape
    sk, nkv = k.shape[1], k.shape[2]
    assert q.stride(3) == 1 and k.stride(3) == 1 and v.stride(3) == 1
    o = torch.empty(b, sq, nh, d, dtype=q.dtype, device=q.device)
    lse = torch.empty(b, nh, sq, dtype=torch.float32, device=q.device)
    call("mb_attn_fwd", ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), b, sq, sk, nh, nkv, d,
         q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
         v.stride(0), v.stride(1), v.stride(2), o.stride(0), o.stride(1), o.stride(2),
         float(scale), int(causal), block_n or Settings.attn_block_n, ptr(seqlens_q), ptr(seqlens_k), stream())
    return o, lse




class _AttnFn(torch.autograd.Function):
    """Attention over separate q / k / v tensors (views allowed)."""

    @staticmethod
    def forward(ctx, q, k, v, scale, causal, seqlens_q=None, seqlens_k=None):
        o, lse = attn_fwd(q, k, v, scale, causal, seqlens_q=seqlens_q, seqlens_k=seqlens_k)
        ctx.scale, ctx.causal = scale, causal
        ctx.seqlens = (seqlens_q, seqlens_k)
        ctx.save_for_backward(q, k, v, o, lse)
        return o

    @staticmethod
    def backward(ctx, dout):
        q, k, v, o, lse = ctx.saved_tensors
        from . import attention_bwd
        dq, dk, dv = attention_bwd.backward(dout, q, k, v, o, lse, ctx.scale, ctx.causal, seqlens=ctx.seqlens)
        return dq, dk, dv, None, None, None, None


def attention(q, k, v, scale: Optional[float] = None, causal: bool = True, seqlens_q=None, seqlens_k=None):
    """Multi-head attention; q ``[b,sq,nh,d]``, k/v ``[b,sk,nh_kv,d]`` (views allowed).

    ``seqlens_q`` / ``seqlens_k`` (int32 ``[b]``, on the device): real tokens per sample of a right-padded
    batch.  One launch covers the whole batch and nothing is read back to the host: padded keys are masked
    inside the kernels and padded query rows come out as zeros -- the result of removing the padding,
    running variable-length attention and padding again (reference: csrc/flash_attn/flash_api.cpp:427, 814
    ``varlen_fwd`` / ``varlen_bwd`` behind mist/modules/mha.py:1233-1243)."""
    if _sym(q):
        return _rules().attention(q, k, v, scale, causal)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return _AttnFn.apply(q, k, v, float(scale), bool(causal), seqlens_q, seqlens_k)


def attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k=None, scale: Optional[float] = None, causal: bool = True):
    """Attention over sequences packed back to back without padding: q ``[total_q, nh, d]``, k / v
    ``[total_k, nh_kv, d]``, ``cu_seqlens_*`` the ``batch + 1`` cumulative lengths (a tensor or a list;
    a tensor is read back to the host once).  Returns ``[total_q, nh, d]``.  Each sequence is one launch
    of the ordinary kernel on a view of the packed tensors (the interface of the reference's
    ``flash_attn_varlen`` entry points, csrc/flash_attn/flash_api.cpp ``varlen_fwd`` / ``varlen_bwd``)."""
    cq = cu_seqlens_q.tolist() if isinstance(cu_seqlens_q, torch.Tensor) else list(cu_seqlens_q)
    ck = cq if cu_seqlens_k is None else (
        cu_seqlens_k.tolist() if isinstance(cu_seqlens_k, torch.Tensor) else list(cu_seqlens_k))
    assert len(cq) == len(ck) and cq[0] == 0 and ck[0] == 0
    outs = []
    for i in range(len(cq) - 1):
        qi, ki, vi = q[cq[i]:cq[i + 1]], k[ck[i]:ck[i + 1]], v[ck[i]:ck[i + 1]]
        if qi.shape[0] == 0:
            continue
        if ki.shape[0] == 0:
            outs.append(torch.zeros_like(qi))
            continue
        outs.append(attention(qi.unsqueeze(0), ki.unsqueeze(0), vi.unsqueeze(0), scale, causal).squeeze(0))
    return torch.cat(outs, 0) if outs else q.new_zeros(q.shape)


class _PackedAttnFn(torch.autograd.Function):
    """Rotary embedding + attention on a packed ``[b, s, 3, heads, d]`` projection output.

    The rotation is applied in place on the projection output (nothing else keeps that
    tensor: the producing linear saves its input, not its output) and the gradient is
    produced as one packed tensor, so autograd never splits or re-concatenates q/k/v."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, rot, scale, causal):
        if rot:
            qkv = _rope_apply(qkv, cos, sin, rot, False, 2)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        o, lse = attn_fwd(q, k, v, scale, causal)
        ctx.rot, ctx.scale, ctx.causal = rot, scale, causal
        ctx.save_for_backward(qkv, o, lse, cos, sin)
        return o

    @staticmethod
    def backward(ctx, dout):
        qkv, o, lse, cos, sin = ctx.saved_tensors
        from . import attention_bwd
        dqkv = torch.empty_like(qkv)
        attention_bwd.backward(dout, qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], o, lse, ctx.scale,
                               ctx.causal, out=(dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]))
        if ctx.rot:
            dqkv = _rope_apply(dqkv, cos, sin, ctx.rot, True, 2)
        return dqkv, None, None, None, None, None


def attention_qkvpacked(qkv, scale: Optional[float] = None, causal: bool = True, rotary=None):
    """``rotary`` is ``None`` or ``(cos, sin, rot_dim)`` from :func:`rope_tables`."""
    if _sym(qkv):
        return _rules().attention_qkvpacked(qkv, scale, causal, rotary)
    if scale is None:
        scale = 1.0 / math.sqrt(qkv.shape[-1])
    cos, sin, rot = rotary if rotary is not None else (None, None, 0)
    if qkv.is_cuda and Settings.attn_backend == "sdpa":
        # library baseline for A/B runs: rotary out of place, attention by torch SDPA
        if rot:
            qkv = _RotaryFn.apply(qkv, cos, sin, int(rot))
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        return F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale).transpose(1, 2)
    return _PackedAttnFn.apply(qkv, cos, sin, int(rot), float(scale), bool(causal))


class _RotaryFn(torch.autograd.Function):
    """Out-of-place differentiable rotary embedding on packed qkv."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, rot):
        ctx.save_for_backward(cos, sin)
        ctx.rot = rot
        return _rope_apply(qkv.clone(), cos, sin, rot, False, 2)

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        return _rope_apply(g.contiguous().clone(), cos, sin, ctx.rot, True, 2), None, None, None


# ------------------------------------------------------- non-flash attention softmax
class _CausalSoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, causal):
        ctx.scale = scale
        sq, sk = x.shape[-2], x.shape[-1]
        if not use_native(x):
            s = x.float() * scale
            if causal:
                mask = torch.ones(sq, sk, dtype=torch.bool, device=x.device).tril(sk - sq)
                s = s.masked_fill(~mask, float("-inf"))
            y = torch.softmax(s, dim=-1).to(x.dtype)
        else:
            x = x.contiguous()
            y = torch.empty_like(x)
            call("mb_causal_softmax_fwd", ptr(x), ptr(y), x.numel() // sk, sq, sk, float(scale),
                 int(causal), stream())
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        sk = y.shape[-1]
        if not use_native(y):
            yf, df = y.float(), dy.float()
            dx = ctx.scale * yf * (df - (df * yf).sum(-1, keepdim=True))
            return dx.to(y.dtype), None, None
        dy = dy.contiguous()
        dx = torch.empty_like(y)
        call("mb_causal_softmax_bwd", ptr(dy), ptr(y), ptr(dx), y.numel() // sk, sk, float(ctx.scale),
             stream())
        return dx, None, None


def scaled_causal_softmax(x, scale: float, causal: bool = True):
    if _sym(x):
        return _rules().scaled_causal_softmax(x, scale, causal)
    return _CausalSoftmaxFn.apply(x, float(scale), bool(causal))


# ----------------------------------------------------------------------- cross entropy
class _XentFn(torch.autograd.Function):
    """Vocab-parallel cross entropy; logits ``[rows, v_local]`` are overwritten by the
    gradient in the backward pass (as in the reference's in-place variant)."""

    @staticmethod
    def forward(ctx, logits, labels, v0, group, ignore_index):
        rows, cols = logits.shape
        ctx.v0, ctx.ignore = v0, ignore_index
        tp = group is not None and torch.distributed.get_world_size(group) > 1
        if not use_native(logits):
            lf = logits.float()
            m = lf.max(-1).values
            if tp:
                torch.distributed.all_reduce(m, op=torch.distributed.ReduceOp.MAX, group=group)
            se = torch.exp(lf - m[:, None]).sum(-1)
            lab = labels - v0
            inr = (lab >= 0) & (lab < cols)
            tgt = torch.where(inr, lf.gather(1, lab.clamp(0, cols - 1)[:, None])[:, 0],
                              torch.zeros_like(m))
            if tp:
                torch.distributed.all_reduce(se, group=group)
                torch.distributed.all_reduce(tgt, group=group)
            lse = se.log() + m
            loss = torch.where(labels == ignore_index, torch.zeros_like(lse), lse - tgt)
        else:
            assert logits.stride(1) == 1
            stats = torch.empty(rows, 3, dtype=torch.float32, device=logits.device)
            call("mb_xent_stats", ptr(logits), ptr(labels), ptr(stats), rows, cols, logits.stride(0), v0,
                 stream())
            if tp:
                gm = stats[:, 0].clone()
                torch.distributed.all_reduce(gm, op=torch.distributed.ReduceOp.MAX, group=group)
                rest = stats[:, 1:].clone()
                rest[:, 0] *= torch.exp(stats[:, 0] - gm)
                torch.distributed.all_reduce(rest, group=group)
                stats = torch.cat([gm[:, None], rest], dim=1).contiguous()
            loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
            lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
            call("mb_xent_loss", ptr(stats), ptr(labels), ptr(loss), ptr(lse), rows, ignore_index,
                 stream())
        ctx.save_for_backward(logits, labels, lse)
        return loss

    @staticmethod
    def backward(ctx, gloss):
        logits, labels, lse = ctx.saved_tensors
        rows, cols = logits.shape
        if not use_native(logits):
            p = torch.exp(logits.float() - lse[:, None])
            lab = labels - ctx.v0
            inr = (lab >= 0) & (lab < cols)
            oh = torch.zeros_like(p)
            oh[inr, lab[inr]] = 1.0
            g = (p - oh) * gloss.float()[:, None]
            g = torch.where((labels == ctx.ignore)[:, None], torch.zeros_like(g), g)
            return g.to(logits.dtype), None, None, None, None
        gloss = gloss.contiguous().float()
        call("mb_xent_bwd", ptr(logits), ptr(labels), ptr(lse), ptr(gloss), 1.0, rows, cols,
             logits.stride(0), ctx.v0, ctx.ignore, 0, stream())
        return logits, None, None, None, None


def cross_entropy(logits, labels, vocab_start: int = 0, group=None, ignore_index: int = -100):
    """Per-row loss (fp32) of ``[rows, v_local]`` logits against global ``labels``."""
    if _sym(logits):
        return _rules().cross_entropy(logits, labels, vocab_start, group, ignore_index)
    return _XentFn.apply(logits, labels, int(vocab_start), group, int(ignore_index))


# --------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, wte, wpe, v0):
        b, s = ids.shape
        h = wte.shape[1]
        ctx.v0 = v0
        ctx.has_pos = wpe is not None
        ctx.save_for_backward(ids, wte, wpe)
        v1 = v0 + wte.shape[0]
        if not use_native(wte):
            loc = ids - v0
            inr = (loc >= 0) & (loc < wte.shape[0])
            out = wte[loc.clamp(0, wte.shape[0] - 1)].float() * inr[..., None].float()
            if wpe is not None:
                out = out + wpe[:s].float()[None]
            return out.to(wte.dtype)
        ids = ids.contiguous()
        out = torch.empty(b, s, h, dtype=wte.dtype, device=wte.device)
        call("mb_embedding_fwd", ptr(ids), ptr(wte), ptr(wpe), ptr(out), b * s, s, h, v0, v1, stream())
        return out

    @staticmethod
    def backward(ctx, dout):
        ids, wte, wpe = ctx.saved_tensors
        b, s = ids.shape
        h = wte.shape[1]
        v0, v1 = ctx.v0, ctx.v0 + wte.shape[0]
        dwte = torch.zeros(wte.shape, dtype=torch.float32, device=wte.device)
        dwpe = torch.zeros(wpe.shape, dtype=torch.float32, device=wte.device) if ctx.has_pos else None
        if not use_native(wte):
            loc = ids - v0
            inr = (loc >= 0) & (loc < wte.shape[0])
            d2 = dout.float().reshape(-1, h)
            sel = inr.reshape(-1)
            dwte.index_add_(0, loc.reshape(-1)[sel], d2[sel])
            if dwpe is not None:
                dwpe[:s] += dout.float().sum(0)
        else:
            dout = dout.contiguous()
            call("mb_embedding_bwd", ptr(ids.contiguous()), ptr(dout), ptr(dwte), ptr(dwpe), b, s, h, v0,
                 v1, stream())
        return None, dwte.to(wte.dtype), (None if dwpe is None else dwpe.to(wpe.dtype)), None


def embedding(ids, wte, wpe=None, vocab_start: int = 0):
    """``wte[ids - vocab_start]`` (zero outside this rank's slice) ``+ wpe[position]``."""
    if _sym(ids):
        return _rules().embedding(ids, wte, wpe, vocab_start)
    return _EmbeddingFn.apply(ids, wte, wpe, int(vocab_start))


# --------------------------------------------------------------------- optimizer / casts
def adam_step(master, exp_avg, exp_avg_sq, grad, model, *, lr, beta1, beta2, eps, weight_decay, step,
              inv_scale=1.0, adamw=True):
    """One fused Adam(W) step on a flat shard; writes the bf16 model copy when given."""
    if not use_native(master):
        g = grad.float() * inv_scale
        if not adamw and weight_decay:
            g = g + weight_decay * master
        exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
        exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        mh = exp_avg / (1 - beta1 ** step)
        vh = exp_avg_sq / (1 - beta2 ** step)
        upd = mh / (vh.sqrt() + eps)
        if adamw and weight_decay:
            upd = upd + weight_decay * master
        master.add_(upd, alpha=-lr)
        if model is not None:
            model.copy_(master)
        return
    n = master.numel()
    call("mb_adam_step", ptr(master), ptr(exp_avg), ptr(exp_avg_sq), ptr(grad),
         int(grad.dtype == torch.float32), ptr(model), n, float(lr), float(beta1), float(beta2),
         float(eps), float(weight_decay), int(step), float(inv_scale), int(adamw), stream())


def cast_to_bf16(src_f32, dst_bf16, scale: float = 1.0):
    if not use_native(src_f32):
        dst_bf16.copy_(src_f32 * scale)
        return dst_bf16
    call("mb_cast_f32_to_bf16", ptr(src_f32), ptr(dst_bf16), src_f32.numel(), float(scale), stream())
    return dst_bf16


def accumulate_grad(src_bf16, dst, scale: float = 1.0, accumulate: bool = True):
    """dst (fp32 or bf16) (+)= scale * src (bf16)."""
    if not use_native(src_bf16):
        v = src_bf16.float() * scale
        dst.copy_((dst.float() + v) if accumulate else v)
        return dst
    if dst.dtype == torch.float32:
        call("mb_axpy_bf16_to_f32", ptr(src_bf16), ptr(dst), src_bf16.numel(), float(scale),
             int(accumulate), stream())
    else:
        assert scale == 1.0 and accumulate
        call("mb_add_bf16", ptr(src_bf16), ptr(dst), src_bf16.numel(), stream())
    return dst
