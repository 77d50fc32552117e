"""Autoregressive generation with a key/value cache for the decoder-only models.

    from mist_b200.inference import generate
    tokens = generate(model, prompt_ids, max_new_tokens=32)

The prompt is processed in one causal forward pass that fills each attention layer's cache;
every further token is one forward pass over a single position whose attention is the
single-query kernel over the cache.  The cache is ``[batch, max_seq, 2, kv_heads, head_dim]``
per layer, allocated on first use.

Reference: ``InferenceParams`` and the cache update / single-query branches of
mist/modules/mha.py:531-575 (``_update_kv_cache``, ``_apply_rotary_single_query_attention``)
backed by csrc/ft_attention; generation utilities are not part of the reference's benchmark
drivers, which only train.
"""
from __future__ import annotations

import contextlib
from typing import Dict, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .modules.layers import ParallelMHA


class InferenceParams:
    def __init__(self, max_batch_size: int, max_seqlen: int):
        self.max_batch_size, self.max_seqlen = int(max_batch_size), int(max_seqlen)
        self.seqlen_offset = 0
        self.key_value_memory: Dict[int, torch.Tensor] = {}

    def cache_for(self, layer_idx, batch, kv_heads, head_dim, dtype, device) -> torch.Tensor:
        assert batch <= self.max_batch_size, "batch larger than the cache was sized for"
        t = self.key_value_memory.get(layer_idx)
        if t is None:
            t = torch.zeros(self.max_batch_size, self.max_seqlen, 2, kv_heads, head_dim, dtype=dtype, device=device)
            self.key_value_memory[layer_idx] = t
        return t

    def reset(self):
        self.seqlen_offset = 0


@contextlib.contextmanager
def kv_cache(model: nn.Module, max_batch_size: int, max_seqlen: int):
    """Attaches one :class:`InferenceParams` to every self-attention layer of ``model``."""
    ip = InferenceParams(max_batch_size, max_seqlen)
    layers = [m for m in model.modules() if isinstance(m, ParallelMHA) and not m.cross_attn]
    keys = [m.layer_idx for m in layers]
    assert len(set(keys)) == len(keys) and None not in keys, "attention layers need distinct layer_idx values"
    for m in layers:
        m.inference_params = ip
    try:
        yield ip
    finally:
        for m in layers:
            m.inference_params = None


@torch.no_grad()
def generate(model: nn.Module, input_ids: torch.Tensor, max_new_tokens: int, eos_token_id: Optional[int] = None,
             temperature: float = 0.0, top_k: int = 0, generator: Optional[torch.Generator] = None,
             tp_group=None, top_p: float = 0.0) -> torch.Tensor:
    """Greedy (``temperature == 0``) or sampled continuation of ``input_ids`` ``[batch, prompt]``
    (``top_k`` keeps the k most likely tokens, ``top_p`` the smallest set whose probability reaches p).
    Returns ``[batch, prompt + generated]``; sequences that hit ``eos_token_id`` keep emitting it.
    With a tensor-parallel model pass its group as ``tp_group``: the vocabulary-parallel logits of
    the last position are gathered so every rank picks the same token (sampling then needs the
    same ``generator`` state on every rank)."""
    was_training = model.training
    model.eval()
    b, s0 = input_ids.shape
    total = s0 + max_new_tokens
    out = input_ids
    done = torch.zeros(b, dtype=torch.bool, device=input_ids.device)
    try:
        with kv_cache(model, b, total) as ip:
            step_ids = input_ids
            for _ in range(max_new_tokens):
                pos = torch.arange(ip.seqlen_offset, ip.seqlen_offset + step_ids.shape[1], device=input_ids.device)
                logits = model(step_ids, position_ids=pos.unsqueeze(0).expand(b, -1))
                ip.seqlen_offset += step_ids.shape[1]
                last = logits.reshape(b, step_ids.shape[1], -1)[:, -1].float()
                if tp_group is not None and dist.get_world_size(tp_group) > 1:
                    parts = [torch.empty_like(last) for _ in range(dist.get_world_size(tp_group))]
                    dist.all_gather(parts, last.contiguous(), group=tp_group)
                    last = torch.cat(parts, dim=-1)
                if temperature > 0:
                    last = last / temperature
                    if top_k > 0:
                        kth = torch.topk(last, top_k, dim=-1).values[:, -1:]
                        last = last.masked_fill(last < kth, float("-inf"))
                    if 0.0 < top_p < 1.0:
                        srt, idx = torch.sort(last, dim=-1, descending=True)
                        cum = torch.softmax(srt, dim=-1).cumsum(-1)
                        drop = cum - torch.softmax(srt, dim=-1) >= top_p      # mass before this token already reaches p
                        last = last.masked_fill(drop.scatter(-1, idx, drop), float("-inf"))
                    nxt = torch.multinomial(torch.softmax(last, dim=-1), 1, generator=generator).squeeze(1)
                else:
                    nxt = last.argmax(dim=-1)
                if eos_token_id is not None:
                    nxt = torch.where(done, torch.full_like(nxt, eos_token_id), nxt)
                    done = done | (nxt == eos_token_id)
                out = torch.cat([out, nxt.unsqueeze(1)], dim=1)
                step_ids = nxt.unsqueeze(1)
                if eos_token_id is not None and bool(done.all()):
                    break
    finally:
        model.train(was_training)
    return out
