"""Embedding -> transformer stack(s) -> (pooler) and the LM head / loss helpers.

Pipeline stages instantiate the same class with ``pre_process`` / ``post_process`` flags
and a layer range, so stage 0 owns the embeddings and the last stage the final norm and
head (reference: mist/model/language_model.py:71-312; nested checkpoint layout :314-405).
"""
from __future__ import annotations


import torch
import torch.nn as nn

from ..config import ModelConfig, PositionEmbeddingType
from ..modules.layers import ColumnParallelLinear, PaddingMask, VocabParallelEmbedding, vocab_parallel_cross_entropy
from ..ops import functional as F
from ..parallel import dist_ops
from .transformer import ParallelTransformer


class Pooler(nn.Module):
    """tanh(dense(hidden[:, index])) -- BERT's sentence representation."""

    def __init__(self, hidden_size, device=None, dtype=None):
        super().__init__()
        self.dense = nn.Linear(hidden_size, hidden_size, device=device, dtype=dtype)
        if self.dense.weight.device.type != "meta":
            nn.init.normal_(self.dense.weight, std=0.02)
            nn.init.zeros_(self.dense.bias)

    def forward(self, hidden_states, sequence_index=0):
        return torch.tanh(self.dense(hidden_states[:, sequence_index]))


class TransformerLanguageModel(nn.Module):
    def __init__(self, cfg: ModelConfig, pre_process=True, post_process=True, process_groups=None,
                 pre_post_process_group=None, layer_range=None, sequence_parallel=False,
                 device=None, dtype=None, stacks=("encoder", "decoder")):
        """``stacks``: which of the model's stacks this pipeline stage holds (an encoder-decoder model
        split over stages gives its first stages encoder blocks only and its last stage the decoder;
        that last stage also gets an embedding, for the decoder's input tokens)."""
        super().__init__()
        self.cfg, self.pre_process, self.post_process = cfg, pre_process, post_process
        self.enc_hidden_input = None      # encoder output received from the previous pipeline stage
        dtype = dtype or cfg.params_dtype
        L = cfg.num_hidden_layers
        if not isinstance(process_groups, (list, tuple)):
            process_groups = [process_groups] * L
        self.process_groups = list(process_groups)
        self.pre_post_process_group = pre_post_process_group if pre_post_process_group is not None \
            else self.process_groups[0]
        self.sequence_parallel = sequence_parallel
        self.embedding = None
        if pre_process:
            learned = cfg.position_embedding_type is PositionEmbeddingType.absolute
            self.embedding = VocabParallelEmbedding(
                cfg.vocab_size, cfg.hidden_size, cfg.max_position_embeddings if learned else 0,
                cfg.num_tokentypes, process_group=self.pre_post_process_group,
                sequence_parallel=sequence_parallel, padding_idx=cfg.padding_idx, device=device, dtype=dtype)
        self.encoder = None
        if cfg.add_encoder and "encoder" in stacks:
            # the encoder's final norm sits with its last block: on the last stage of a single-stack model,
            # on the stage that also holds the decoder, or on the last encoder-only stage
            last_encoder_stage = layer_range is None or layer_range[1] == L
            self.encoder = ParallelTransformer(
                cfg, self.process_groups, layer_range=layer_range, attn_mask_type=cfg.encoder_attn_mask_type,
                post_norm=post_process or (cfg.add_decoder and last_encoder_stage), sequence_parallel=sequence_parallel,
                device=device, dtype=dtype)
        self.decoder = None
        if cfg.add_decoder and "decoder" in stacks:
            if "encoder" not in stacks:
                layer_range = None        # the decoder is never split
            self.decoder = ParallelTransformer(
                cfg, self.process_groups, layer_range=layer_range, is_decoder=True,
                attn_mask_type=cfg.decoder_attn_mask_type, post_norm=post_process,
                sequence_parallel=sequence_parallel, device=device, dtype=dtype)
        self.pooler = Pooler(cfg.hidden_size, device=device, dtype=dtype) if (post_process and cfg.add_pooler) else None

    def set_input_tensor(self, t):
        if self.encoder is not None:
            self.encoder.set_input_tensor(t)
        elif self.cfg.add_encoder and self.decoder is not None:
            self.enc_hidden_input = t      # decoder stage of an encoder-decoder pipeline: t is the encoder output
        else:
            self.decoder.set_input_tensor(t)

    def flop_estimate(self, batch_size: int, seq_len: int) -> float:
        """Training FLOPs of one micro-batch (forward + backward, no recomputation)."""
        c = self.cfg
        h, f, L, v = c.hidden_size, c.intermediate_size, c.num_hidden_layers, c.vocab_size
        per_layer = 2 * batch_size * seq_len * (c.params_per_block()) + 4 * batch_size * seq_len * seq_len * h
        return 3.0 * (L * per_layer + 2 * batch_size * seq_len * h * v)

    def forward(self, enc_input_ids, enc_position_ids=None, enc_attn_mask=None, dec_input_ids=None,
                dec_position_ids=None, tokentype_ids=None, pooling_sequence_index=0, enc_hidden_states=None,
                dec_attn_mask=None, enc_dec_attn_mask=None):
        """``enc_attn_mask`` / ``dec_attn_mask``: ``[batch, seq]`` key-padding masks (non-zero = real
        token) of the encoder / decoder tokens; ``enc_dec_attn_mask``: mask of the encoder tokens as
        cross attention sees them (defaults to ``enc_attn_mask``).  Masks without padding are dropped."""
        bs = enc_input_ids.shape[0] if enc_input_ids is not None else None
        if enc_hidden_states is None and self.encoder is None and self.enc_hidden_input is not None:
            enc_hidden_states = self.enc_hidden_input
        enc_mask = PaddingMask.prepare(enc_attn_mask)
        dec_mask = PaddingMask.prepare(dec_attn_mask)
        cross_mask = PaddingMask.prepare(enc_dec_attn_mask) if enc_dec_attn_mask is not None else enc_mask
        if self.pre_process and self.encoder is not None:
            hidden = self.embedding(enc_input_ids, enc_position_ids, tokentype_ids)
        else:
            hidden = None
        residual = None
        if self.encoder is not None and enc_hidden_states is None:
            out = self.encoder(hidden, residual, batch_size=bs, attn_mask=enc_mask)
            if not self.post_process and self.decoder is None:
                # handed to the next pipeline stage: (hidden, residual), or the normalised encoder output
                # after the last encoder block of an encoder-decoder model
                return out
            enc_out = out
        else:
            enc_out = enc_hidden_states
        if self.decoder is None:
            if self.pooler is not None:
                full = enc_out
                if self.sequence_parallel:
                    full = dist_ops.all_gather(enc_out, self.pre_post_process_group, replicated_consumer=True).view(
                        bs, -1, enc_out.shape[-1])
                return enc_out, self.pooler(full, pooling_sequence_index)
            return enc_out
        dec_hidden = self.embedding(dec_input_ids, dec_position_ids, None)
        dec_out = self.decoder(dec_hidden, None, encoder_output=enc_out, batch_size=dec_input_ids.shape[0],
                               attn_mask=dec_mask, enc_mask=cross_mask)
        return dec_out, enc_out

    # ------------------------------------------------------------------ checkpoint layout
    def state_dict_for_save_checkpoint(self, prefix="", keep_vars=False):
        sd = {}
        if self.embedding is not None:
            sd["embedding"] = self.embedding.state_dict_for_save_checkpoint(prefix, keep_vars)
        if self.encoder is not None:
            sd["encoder"] = self.encoder.state_dict(prefix=prefix, keep_vars=keep_vars)
        if self.decoder is not None:
            sd["decoder"] = self.decoder.state_dict(prefix=prefix, keep_vars=keep_vars)
        if self.pooler is not None:
            sd["pooler"] = self.pooler.state_dict(prefix=prefix, keep_vars=keep_vars)
        return sd

    def load_state_dict_from_checkpoint(self, sd, strict=True):
        if self.embedding is not None:
            emb = sd.get("embedding")
            if emb is None:  # legacy flat layout: keys prefixed with the sub-module name
                emb = {"word_embeddings": {k.split("word_embeddings.")[1]: v for k, v in sd.items()
                                           if "word_embeddings." in k}}
            self.embedding.load_state_dict_from_checkpoint(emb, strict=strict)
        if self.encoder is not None:
            enc = sd.get("encoder", sd.get("transformer"))
            self.encoder.load_state_dict(enc, strict=strict)
        if self.decoder is not None and "decoder" in sd:
            self.decoder.load_state_dict(sd["decoder"], strict=strict)
        if self.pooler is not None and "pooler" in sd:
            self.pooler.load_state_dict(sd["pooler"], strict=strict)


class LMHead(nn.Module):
    """Vocabulary projection (column parallel, no bias) + vocab-parallel cross entropy."""

    def __init__(self, cfg: ModelConfig, process_group=None, sequence_parallel=False, device=None, dtype=None):
        super().__init__()
        self.process_group = process_group
        self.proj = ColumnParallelLinear(cfg.hidden_size, cfg.vocab_size, process_group=process_group,
                                         bias=False, sequence_parallel=sequence_parallel, device=device,
                                         dtype=dtype or cfg.params_dtype)

    def forward(self, hidden, labels=None, weight=None):
        if weight is not None:   # tied embeddings
            x = hidden
            if self.proj.sequence_parallel:
                x = dist_ops.all_gather(x.reshape(-1, x.shape[-1]), self.process_group)
            else:
                x = dist_ops.copy_to_group(x, self.process_group)
            logits = F.linear(x, weight)
        else:
            logits = self.proj(hidden)
        if labels is None:
            return logits
        logits = logits.reshape(-1, logits.shape[-1])
        loss = vocab_parallel_cross_entropy(logits, labels.reshape(-1), self.process_group)
        return loss.mean()
