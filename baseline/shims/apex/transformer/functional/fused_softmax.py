"""Eager stand-ins for apex's fused softmax autograd functions (only the non-flash attention path of the
reference reaches them; the benchmarked configuration uses flash attention)."""
import torch

from apex.transformer.enums import AttnMaskType


class ScaledUpperTriangMaskedSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inputs, scale):
        sq, sk = inputs.shape[-2:]
        mask = torch.ones(sq, sk, dtype=torch.bool, device=inputs.device).triu(1)
        probs = torch.softmax((inputs.float() * scale).masked_fill(mask, float("-inf")), dim=-1).to(inputs.dtype)
        ctx.save_for_backward(probs)
        ctx.scale = scale
        return probs

    @staticmethod
    def backward(ctx, grad):
        (probs,) = ctx.saved_tensors
        p, g = probs.float(), grad.float()
        return ((g - (g * p).sum(-1, keepdim=True)) * p * ctx.scale).to(grad.dtype), None


class ScaledMaskedSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inputs, mask, scale):
        x = inputs.float() * scale
        if mask is not None:
            x = x.masked_fill(mask, -10000.0)
        probs = torch.softmax(x, dim=-1).to(inputs.dtype)
        ctx.save_for_backward(probs)
        ctx.scale = scale
        return probs

    @staticmethod
    def backward(ctx, grad):
        (probs,) = ctx.saved_tensors
        p, g = probs.float(), grad.float()
        return ((g - (g * p).sum(-1, keepdim=True)) * p * ctx.scale).to(grad.dtype), None, None


class ScaledSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inputs, scale):
        return ScaledMaskedSoftmax.forward(ctx, inputs, None, scale)

    @staticmethod
    def backward(ctx, grad):
        return ScaledMaskedSoftmax.backward(ctx, grad)[0], None


def scaled_upper_triang_masked_softmax(inputs, _, scale):
    b, np_, sq, sk = inputs.size()
    return ScaledUpperTriangMaskedSoftmax.apply(inputs.view(-1, sq, sk), scale).view(b, np_, sq, sk)


def scaled_masked_softmax(inputs, mask, scale):
    if mask is not None:
        return ScaledMaskedSoftmax.apply(inputs, mask, scale)
    return ScaledSoftmax.apply(inputs, scale)


class FusedScaleMaskSoftmax(torch.nn.Module):
    def __init__(self, input_in_fp16, input_in_bf16, attn_mask_type, scaled_masked_softmax_fusion,
                 mask_func, softmax_in_fp32, scale):
        super().__init__()
        self.attn_mask_type = attn_mask_type
        self.mask_func = mask_func
        self.scale = scale

    def forward(self, input, mask):
        scale = self.scale if self.scale is not None else 1.0
        if self.attn_mask_type == AttnMaskType.causal:
            return scaled_upper_triang_masked_softmax(input, mask, scale)
        return scaled_masked_softmax(input, mask, scale)
