import types

import torch

_lib = torch.library.Library("xformers", "DEF")
for _name in ("efficient_attention_forward_cutlass", "efficient_attention_backward_cutlass"):
    try:
        _lib.define(f"{_name}(Tensor query) -> Tensor")
    except RuntimeError:
        pass


class LowerTriangularMask:
    pass


def _unsupported(*args, **kwargs):
    raise NotImplementedError("xformers kernels are not available; this stand-in only satisfies imports")


class _FwOp:
    OPERATOR = staticmethod(_unsupported)
    SUPPORTED_ATTN_BIAS_TYPES = set()

    @classmethod
    def not_supported_reasons(cls, *args, **kwargs):
        return []


class _BwOp(_FwOp):
    OPERATOR = staticmethod(_unsupported)
    SUPPORTED_ATTN_BIAS_TYPES = set()


fmha = types.SimpleNamespace(cutlass=types.SimpleNamespace(FwOp=_FwOp, BwOp=_BwOp),
                             attn_bias=types.SimpleNamespace(LowerTriangularMask=LowerTriangularMask))


def memory_efficient_attention(query, key, value, attn_bias=None, p=0.0, scale=None, op=None):
    causal = isinstance(attn_bias, LowerTriangularMask)
    out = torch.nn.functional.scaled_dot_product_attention(
        query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), dropout_p=p, is_causal=causal, scale=scale)
    return out.transpose(1, 2)
