"""Symbolic rules of the framework's fused operators.

Each rule mirrors one entry point of :mod:`mist_b200.ops.functional` /
:mod:`mist_b200.parallel.dist_ops`: given SymTensors it returns SymTensors of the right
shape and records a node stating what the CUDA kernel keeps for the backward pass, how
many FLOPs / bytes both passes move and which scratch they need.  The numbers follow the
kernels in ``mist_b200/csrc`` (e.g. the flash-attention forward keeps q, k, v, o and the
fp32 logsumexp; the norm backward needs a partial-sum scratch matrix).

Same role as the reference's rules for its pybind kernels (mist/modules/sym_register.py:
54-620: flash fwd/bwd, fused dense, dropout_add_ln, swiglu, rotary, scaled softmax).
"""
from __future__ import annotations

import sympy as sp
import torch

from .symtensor import (Comm, SymTensor, as_sym_param, contiguous, elementwise, index_select, prod, record,
                        simplify_int, unary)


def _p(x):
    return as_sym_param(x)


def linear(x, weight, bias, activation, residual):
    w, b = _p(weight), _p(bias)
    x2 = x
    tokens = prod(x.shape[:-1])
    k, n = x.shape[-1], w.shape[0]
    fl = 2 * tokens * k * n
    out_shape = tuple(x.shape[:-1]) + (n,)
    saved = [x2, w]
    outs = [(out_shape, x.dtype)]
    save_out = []
    if activation == "gelu":
        outs.append((out_shape, x.dtype))      # pre-activation written by the GEMM epilogue
        save_out = [1]
    res = record("linear", [x2, w, b, residual], outs, saved=saved, save_outputs=save_out, flops_fwd=fl,
                 flops_bwd=2 * fl, spec={"op": "linear", "m": tokens, "n": n, "k": k, "act": activation or "",
                                         "bias": b is not None},
                 bytes_fwd=(tokens * k + k * n + tokens * n * len(outs)) * 2,
                 bytes_bwd=(2 * tokens * n + 2 * k * n + 2 * tokens * k) * 2,
                 grad_inputs=[x2, residual])
    return res[0]


def gelu(x, bias):
    return unary("gelu", x, save="input")


def swiglu(x):
    f = simplify_int(sp.Integer(1) * x.shape[-1] / 2)
    n = prod(x.shape[:-1]) * f
    (out,) = record("swiglu", [x], [(tuple(x.shape[:-1]) + (f,), x.dtype)], saved=[x], flops_fwd=8 * n,
                    flops_bwd=14 * n, spec={"op": "swiglu", "rows": prod(x.shape[:-1]), "f": f})
    return out


def bias_dropout_add(x, bias, residual, p, seed):
    (out,) = record("bias_dropout_add", [x, _p(bias), residual], [(x.shape, x.dtype)], flops_fwd=3 * x.numel(),
                    flops_bwd=x.numel() if p > 0 else 0,
                    spec={"op": "bias_dropout_add", "rows": prod(x.shape[:-1]), "h": x.shape[-1]})
    return out


def norm(x0, residual, gamma, beta, eps, rms, prenorm):
    g, b = _p(gamma), _p(beta)
    rows, h = prod(x0.shape[:-1]), x0.shape[-1]
    outs = [(x0.shape, x0.dtype)]
    saved = [x0, g]
    save_out = []
    if residual is not None:
        outs.append((x0.shape, x0.dtype))    # the summed residual stream is a new tensor
        saved = [g]
        save_out = [1]
    stats = rows * 4 * (1 if rms else 2)
    res = record("rms_norm" if rms else "layer_norm", [x0, residual, g, b], outs, saved=saved,
                 save_outputs=save_out, saved_extra=stats, flops_fwd=8 * rows * h, flops_bwd=16 * rows * h,
                 bwd_workspace=2 * 296 * 8 * h * 4, spec={"op": "rms_norm" if rms else "layer_norm", "rows": rows, "h": h,
                                                           "residual": residual is not None})
    if prenorm:
        return (res[0], res[1]) if residual is not None else (res[0], x0)
    return res[0]


def rope_inplace(qkv, rot):
    # in place on the projection output: no new storage, no saved tensor (cos/sin tables are tiny)
    n = prod(qkv.shape[:2]) * 2 * qkv.shape[3] * rot
    record("rope", [qkv], [], flops_fwd=3 * n, flops_bwd=3 * n, bytes_fwd=2 * n * 2, bytes_bwd=2 * n * 2,
           spec={"op": "rope", "tokens": prod(qkv.shape[:2]), "heads": qkv.shape[3], "d": qkv.shape[4], "rot": rot})
    return qkv


def attention(q, k, v, scale, causal, packed_from=None):
    """q [b, sq, nh, d], k / v [b, sk, nkv, d] -> o [b, sq, nh, d]; saves q, k, v, o and lse."""
    b_, sq, nh, d = q.shape
    sk = k.shape[1]
    fl = 4 * b_ * nh * sq * sk * d
    if causal:
        fl = fl / 2
    lse_bytes = b_ * nh * sq * 4
    srcs = [packed_from] if packed_from is not None else [q, k, v]
    (o,) = record("flash_attention", srcs, [((b_, sq, nh, d), q.dtype)], saved=srcs, save_outputs=[0],
                  saved_extra=lse_bytes, flops_fwd=fl, flops_bwd=2.5 * fl,
                  bwd_workspace=b_ * nh * sq * d * 4 + lse_bytes,
                  bytes_fwd=(b_ * sq * nh * d * 2 + 2 * b_ * sk * k.shape[2] * d) * 2,
                  bytes_bwd=(4 * b_ * sq * nh * d + 4 * b_ * sk * k.shape[2] * d) * 2 + 2 * b_ * nh * sq * d * 4,
                  spec={"op": "flash_attention", "b": b_, "sq": sq, "sk": sk, "nh": nh, "nkv": k.shape[2], "d": d,
                        "causal": bool(causal)})
    return o


def attention_qkvpacked(qkv, scale, causal, rotary):
    if rotary is not None and rotary[2]:
        qkv = rope_inplace(qkv, rotary[2])
    q = qkv._view((qkv.shape[0], qkv.shape[1], qkv.shape[3], qkv.shape[4]), contiguous=False)
    return attention(q, q, q, scale, causal, packed_from=qkv)


def scaled_causal_softmax(x, scale, causal):
    return unary("causal_softmax", x, save="output", flops_per_elem=10)


def cross_entropy(logits, labels, vocab_start, group, ignore_index):
    rows, cols = logits.shape
    (loss,) = record("cross_entropy", [logits, labels], [((rows,), torch.float32)], saved=[logits, labels],
                     saved_extra=rows * 4, flops_fwd=4 * rows * cols, flops_bwd=4 * rows * cols,
                     bytes_fwd=rows * cols * 2, bytes_bwd=2 * rows * cols * 2, fwd_workspace=rows * 12,
                     grad_inputs=[],    # the backward kernel rewrites the logits in place
                     spec={"op": "cross_entropy", "rows": rows, "cols": cols})
    return loss


def embedding(ids, wte, wpe, vocab_start):
    w, pz = _p(wte), _p(wpe)
    b_, s = ids.shape
    h = w.shape[1]
    (out,) = record("embedding", [ids, w, pz], [((b_, s, h), w.dtype)], saved=[ids],
                    bytes_fwd=3 * b_ * s * h * 2, bytes_bwd=b_ * s * h * 2 + w.numel() * 6,
                    bwd_workspace=w.numel() * 4 + (pz.numel() * 4 if pz is not None else 0),
                    spec={"op": "embedding", "tokens": b_ * s, "h": h, "vocab": w.shape[0]})
    return out


# ------------------------------------------------------------------------- collectives
def _coll(kind_fwd, kind_bwd, x, group, out_shape):
    from ..parallel.dist_ops import group_size
    n = group_size(group)
    full = prod(x.shape) * 2 * (n if kind_fwd == "all_gather" else 1)
    (out,) = record(kind_fwd, [x], [(out_shape, x.dtype)], comm_fwd=Comm(kind_fwd, full) if kind_fwd != "copy" else None,
                    comm_bwd=Comm(kind_bwd, full) if kind_bwd != "copy" else None,
                    spec={"op": kind_fwd, "bytes": full, "group": n})
    return out


def all_gather(x, group):
    from ..parallel.dist_ops import group_size
    n = group_size(group)
    return _coll("all_gather", "reduce_scatter", x, group, (x.shape[0] * n,) + tuple(x.shape[1:]))


def reduce_scatter(x, group):
    from ..parallel.dist_ops import group_size
    n = group_size(group)
    return _coll("reduce_scatter", "all_gather", x, group,
                 (simplify_int(sp.Integer(1) * x.shape[0] / n),) + tuple(x.shape[1:]))


def all_reduce(x, group):
    return _coll("all_reduce", "copy", x, group, x.shape)


def copy_to_group(x, group):
    # identity in the forward pass; the gradient is all-reduced in the backward pass
    from ..parallel.dist_ops import group_size
    record("copy_to_group", [x], [], comm_bwd=Comm("all_reduce", prod(x.shape) * 2),
           spec={"op": "copy_to_group", "bytes": prod(x.shape) * 2, "group": group_size(group)}, bytes_fwd=0,
           bytes_bwd=0)
    return x
