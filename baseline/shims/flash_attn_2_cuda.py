"""Adapter with the call signatures of flash-attn 2.3.1's ``flash_attn_2_cuda`` (what the reference's
requirements pin and ``mist/modules/flash_attn.py`` calls) on top of the flash-attn 2.8 extension that
this image ships.  The 2.3.1 wheel itself rejects sm_100 and is not available offline.  Only used by the
reference arm of bench.py."""
import importlib.machinery
import importlib.util
import os
import sys

import torch  # noqa: F401  (the extension needs torch's libraries loaded first)


def _load_real():
    for p in sys.path:
        if not p or os.path.abspath(p) == os.path.dirname(os.path.abspath(__file__)):
            continue
        if not os.path.isdir(p):
            continue
        for f in os.listdir(p):
            if f.startswith("flash_attn_2_cuda.") and f.endswith(".so"):
                path = os.path.join(p, f)
                loader = importlib.machinery.ExtensionFileLoader("flash_attn_2_cuda", path)
                spec = importlib.util.spec_from_file_location("flash_attn_2_cuda", path, loader=loader)
                mod = importlib.util.module_from_spec(spec)
                loader.exec_module(mod)
                return mod
    raise ImportError("the flash-attn extension of this image was not found")


_real = _load_real()


def fwd(q, k, v, out, dropout_p, softmax_scale, causal, window_left, window_right, return_softmax, gen):
    o, lse, s_dmask, rng_state = _real.fwd(q, k, v, out, None, dropout_p, softmax_scale, causal,
                                           window_left, window_right, 0.0, return_softmax, gen)
    return o, q, k, v, o, lse, s_dmask, rng_state


def bwd(dout, q, k, v, out, lse, dq, dk, dv, dropout_p, softmax_scale, causal, window_left, window_right,
        gen, rng_state):
    return _real.bwd(dout, q, k, v, out, lse, dq, dk, dv, None, dropout_p, softmax_scale, causal,
                     window_left, window_right, 0.0, False, gen, rng_state)


def varlen_fwd(q, k, v, out, cu_q, cu_k, max_q, max_k, dropout_p, softmax_scale, zero_tensors, causal,
               window_left, window_right, return_softmax, gen):
    o, lse, s_dmask, rng_state = _real.varlen_fwd(q, k, v, out, cu_q, cu_k, None, None, None, None, max_q,
                                                  max_k, dropout_p, softmax_scale, zero_tensors, causal,
                                                  window_left, window_right, 0.0, return_softmax, gen)
    return o, q, k, v, o, lse, s_dmask, rng_state


def varlen_bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, max_q, max_k, dropout_p, softmax_scale,
               zero_tensors, causal, window_left, window_right, gen, rng_state):
    return _real.varlen_bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, None, max_q, max_k, dropout_p,
                            softmax_scale, zero_tensors, causal, window_left, window_right, 0.0, False, gen,
                            rng_state)


def fwd_kvcache(*args, **kwargs):
    raise NotImplementedError("fwd_kvcache is not adapted (inference only; the benchmark does not reach it)")
