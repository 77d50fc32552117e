"""Transformer block and stack shared by every model family.

A block is ``norm -> attention -> norm -> MLP`` with pre-norm residual streams; the
residual add is folded into the following norm kernel, so a block hands
``(hidden, residual)`` to the next one and only the final norm materialises the sum.
Falcon-style parallel blocks (attention and MLP fed by the same norm output) and
decoder blocks with cross attention are options of the same class.  Under sequence
parallelism hidden/residual are ``[batch*seq/tp, hidden]`` token shards.

Parity: reference mist/model/transformer.py:91-342 (ParallelTransformerLayer),
:345-500 (ParallelTransformer; its sequence-parallel branch raises NotImplementedError at
:477-479, here it is implemented), checkpoint key renames :502-511.
"""
from __future__ import annotations

import contextlib
from typing import List, Optional

import torch
import torch.nn as nn

from ..config import AttnMaskType, ModelConfig, PositionEmbeddingType
from ..modules.layers import ParallelGatedMlp, ParallelMHA, ParallelMLP, get_norm
from ..ops import functional as F


def _gate_activation(name: str) -> str:
    """Gate activation of a gated MLP: the tanh-GELU default of the plain MLP means "not set" there."""
    name = (name or "swiglu").lower()
    return "swiglu" if name in ("gelu_new", "gelu_fast", "gelu_approx", "gelu_pytorch_tanh") else name


class ParallelTransformerLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, process_group=None, is_decoder: bool = False,
                 attn_mask_type: AttnMaskType = AttnMaskType.causal, sequence_parallel: bool = False,
                 device=None, dtype=None):
        super().__init__()
        assert cfg.num_experts is None, "mixture-of-experts blocks are not part of this model zoo"
        assert cfg.prenorm or not cfg.parallel_block, "parallel blocks take their residual from the block input"
        self.cfg, self.layer_idx, self.is_decoder = cfg, layer_idx, is_decoder
        # prenorm = False: each residual connection starts from the *normalised* stream (the norm's
        # output) instead of the norm's input (reference: mist/model/transformer.py:260-264,309-314)
        self.residual_from_norm = not cfg.prenorm
        # the residual stream in fp32 while the branches stay in the parameter dtype (reference:
        # fp32_residual_connection, mist/model/transformer.py:120; residual_in_fp32 of its norm kernels)
        self.fp32_residual = bool(cfg.fp32_residual_connection)
        self.parallel_block = cfg.parallel_block
        self.tied_norm = cfg.parallel_block_tied_norm
        self.sequence_parallel = sequence_parallel
        self.hidden_dropout = cfg.hidden_dropout
        fk = dict(device=device, dtype=dtype)
        nk = dict(eps=cfg.normalization_eps, prenorm=True, sequence_parallel=sequence_parallel, **fk)
        rot_dim = 0
        if cfg.position_embedding_type is PositionEmbeddingType.rotary:
            rot_dim = int(cfg.head_dim * cfg.rotary_emb_fraction) // 16 * 16
        # softmax scale: 1/sqrt(head_dim) when scale_attn_weights, else 1; optionally divided by the
        # 1-based layer index (reference: mist/model/transformer.py:33-37)
        softmax_scale = cfg.head_dim ** -0.5 if cfg.scale_attn_weights else 1.0
        if cfg.scale_attn_by_inverse_layer_idx:
            softmax_scale /= float(layer_idx + 1)
        self.norm1 = get_norm(cfg.normalization, cfg.hidden_size, **nk)
        self.attn = ParallelMHA(
            cfg.hidden_size, cfg.num_attention_heads, cfg.num_heads_kv, process_group=process_group,
            qkv_proj_bias=cfg.qkv_proj_bias, out_proj_bias=cfg.out_proj_bias, dropout=cfg.attention_dropout,
            causal=attn_mask_type is AttnMaskType.causal, rotary_emb_dim=rot_dim,
            rotary_emb_base=cfg.rotary_emb_base, use_flash_attn=cfg.use_flash_attn, softmax_scale=softmax_scale,
            rotary_emb_interleaved=cfg.rotary_emb_interleaved, rotary_emb_scale_base=cfg.rotary_emb_scale_base,
            sequence_parallel=sequence_parallel, layer_idx=layer_idx, **fk)
        if is_decoder:
            self.norm_cross = get_norm(cfg.normalization, cfg.hidden_size, **nk)
            self.cross_attn = ParallelMHA(
                cfg.hidden_size, cfg.num_attention_heads, cfg.num_heads_kv, process_group=process_group,
                qkv_proj_bias=cfg.qkv_proj_bias, out_proj_bias=cfg.out_proj_bias, cross_attn=True,
                use_flash_attn=cfg.use_flash_attn, softmax_scale=softmax_scale,
                sequence_parallel=sequence_parallel, layer_idx=layer_idx, **fk)
        if not (self.parallel_block and self.tied_norm):
            self.norm2 = get_norm(cfg.normalization, cfg.hidden_size, **nk)
        if cfg.gated:
            self.mlp = ParallelGatedMlp(cfg.hidden_size, cfg.intermediate_size, process_group=process_group,
                                        bias1=cfg.mlp_fc1_bias, bias2=cfg.mlp_fc2_bias,
                                        activation=_gate_activation(cfg.activation_function),
                                        sequence_parallel=sequence_parallel, **fk)
        else:
            self.mlp = ParallelMLP(cfg.hidden_size, cfg.intermediate_size, process_group=process_group,
                                   bias1=cfg.mlp_fc1_bias, bias2=cfg.mlp_fc2_bias,
                                   activation=cfg.activation_function,
                                   sequence_parallel=sequence_parallel, **fk)

    def _drop(self, x):
        if self.hidden_dropout > 0 and self.training:
            seed = F.next_dropout_seed()
            return F.bias_dropout_add(x, None, None, self.hidden_dropout, seed)
        return x

    def _drop_args(self):
        """Keyword arguments that make a norm apply this block's hidden dropout to its input, inside the
        norm kernel, before the residual add (one pass instead of a separate element-wise kernel)."""
        if self.hidden_dropout > 0 and self.training:
            return dict(dropout_p=self.hidden_dropout, seed=F.next_dropout_seed())
        return {}

    def forward(self, hidden, residual=None, encoder_output=None, batch_size: Optional[int] = None,
                attn_mask=None, enc_mask=None):
        """Returns ``(hidden, residual)``; the caller's next norm adds them.  ``attn_mask`` /
        ``enc_mask``: prepared padding masks (:class:`~mist_b200.modules.layers.PaddingMask`) of this
        stack's tokens and of the encoder output that cross attention reads.

        Dropout of the attention and cross-attention outputs runs inside the norm that consumes them;
        the MLP output leaves the block already dropped out (its consumer is another block, the final
        norm or a pipeline boundary)."""
        bs = batch_size if batch_size is not None else hidden.shape[0]
        if self.fp32_residual and residual is None and isinstance(hidden, torch.Tensor) and not F._sym(hidden):
            if hidden.dtype == torch.float32 and self.norm1.weight.dtype != torch.float32:
                # the stream of the previous pipeline stage, handed over as one fp32 tensor
                residual, hidden = hidden, torch.zeros(hidden.shape, dtype=self.norm1.weight.dtype, device=hidden.device)
            else:
                residual = torch.zeros(hidden.shape, dtype=torch.float32, device=hidden.device)   # the fp32 stream starts here
        if not self.parallel_block:
            x, residual = self.norm1(hidden, residual)
            if self.residual_from_norm:
                residual = x
            hidden = self.attn(x, batch_size=bs, attention_mask=attn_mask)
            if hidden.shape != residual.shape:
                hidden = hidden.reshape(residual.shape)
            if self.is_decoder:
                x, residual = self.norm_cross(hidden, residual, **self._drop_args())
                if self.residual_from_norm:
                    residual = x
                hidden = self.cross_attn(x, x_kv=encoder_output, batch_size=bs, attention_mask=attn_mask,
                                         kv_mask=enc_mask).reshape(residual.shape)
            x, residual = self.norm2(hidden, residual, **self._drop_args())
            if self.residual_from_norm:
                residual = x
            hidden = self._drop(self.mlp(x)).reshape(residual.shape)
            return hidden, residual
        # parallel block: attention and MLP read the same stream; both norms of it come from one kernel
        if self.tied_norm or F._sym(hidden):
            x1, residual = self.norm1(hidden, residual)
            x2 = x1 if self.tied_norm else self.norm2(residual, None)[0]
        else:
            n1, n2 = self.norm1, self.norm2
            x1, x2, residual = F.parallel_residual_norm(hidden, None, residual, n1.weight, n1.bias, n2.weight, n2.bias,
                                                        eps=n1.eps, rms=n1.bias is None)
        a = self._drop(self.attn(x1, batch_size=bs, attention_mask=attn_mask)).reshape(residual.shape)
        m = self._drop(self.mlp(x2)).reshape(residual.shape)
        return a + m, residual


class ParallelTransformer(nn.Module):
    """A contiguous range of blocks, plus the final norm when it holds the last block.

    ``gradient_checkpointing = c`` recomputes the **last** ``c`` blocks of this stack in the
    backward pass (same convention as the strategy's ``gradient_checkpointing`` entry)."""

    def __init__(self, cfg: ModelConfig, process_groups: List, layer_range=None, is_decoder=False,
                 attn_mask_type=AttnMaskType.causal, post_norm=True, sequence_parallel=False,
                 device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        start, end = layer_range if layer_range is not None else (0, cfg.num_hidden_layers)
        self.layer_range = (start, end)
        self.sequence_parallel = sequence_parallel
        self.layers = nn.ModuleList([
            ParallelTransformerLayer(cfg, i, process_group=process_groups[i], is_decoder=is_decoder,
                                     attn_mask_type=attn_mask_type, sequence_parallel=sequence_parallel,
                                     device=device, dtype=dtype)
            for i in range(start, end)])
        self.final_norm = None
        if post_norm:
            self.final_norm = get_norm(cfg.normalization, cfg.hidden_size, eps=cfg.normalization_eps,
                                       prenorm=False, sequence_parallel=sequence_parallel, device=device, dtype=dtype)
        self.gradient_checkpointing = 0
        self.input_tensor = None
        #: set by the training engine: object with before_layer / after_layer callbacks
        self.hooks = None

    def set_input_tensor(self, t):
        """Pipeline stages other than the first take their input from the previous stage."""
        self.input_tensor = t

    def forward(self, hidden, residual=None, encoder_output=None, batch_size=None, attn_mask=None, enc_mask=None):
        if self.input_tensor is not None:
            hidden = self.input_tensor
        n = len(self.layers)
        first_ckpt = n - self.gradient_checkpointing
        hooks = self.hooks
        for i, layer in enumerate(self.layers):
            if hooks is not None:
                hidden, residual = hooks.before_layer(self, i, hidden, residual)
            ctx = hooks.layer_context(self, i) if hasattr(hooks, "layer_context") else contextlib.nullcontext()
            with ctx:
                if i >= first_ckpt and torch.is_grad_enabled():
                    from ..utils.checkpointing import checkpoint_block
                    hidden, residual = checkpoint_block(layer, hidden, residual, encoder_output, batch_size,
                                                        attn_mask, enc_mask)
                else:
                    hidden, residual = layer(hidden, residual, encoder_output, batch_size, attn_mask, enc_mask)
            if hooks is not None:
                hidden, residual = hooks.after_layer(self, i, hidden, residual)
        if self.final_norm is not None:
            return self.final_norm(hidden, residual)
        return hidden, residual

    # legacy key names accepted on load ("layernorm" -> "norm", ".attention." -> ".attn.")
    def load_state_dict(self, state_dict, strict=True):
        renamed = {}
        for k, v in state_dict.items():
            k2 = k.replace("input_layernorm", "norm1").replace("post_attention_layernorm", "norm2")
            k2 = k2.replace("final_layernorm", "final_norm").replace(".attention.", ".attn.")
            renamed[k2] = v
        return super().load_state_dict(renamed, strict=strict)
