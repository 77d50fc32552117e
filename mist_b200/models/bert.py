"""BERT: bidirectional encoder, token types, pooler, masked-LM head and the binary
(next-sentence) head (reference: mist/model/bert.py:59-118 head, :165-392 model)."""
from __future__ import annotations

import torch
import torch.nn as nn

from ..config import AttnMaskType, ModelConfig
from ..modules.layers import get_norm, vocab_parallel_cross_entropy
from ..ops import functional as F
from ..parallel import dist_ops
from .language_model import TransformerLanguageModel


class BertLMHead(nn.Module):
    """dense -> gelu -> norm -> tied vocabulary projection (+ per-rank bias slice)."""

    def __init__(self, cfg: ModelConfig, local_vocab: int, process_group=None, device=None, dtype=None):
        super().__init__()
        self.process_group = process_group
        self.dense = nn.Linear(cfg.hidden_size, cfg.hidden_size, device=device, dtype=dtype)
        self.norm = get_norm(cfg.normalization, cfg.hidden_size, cfg.normalization_eps, device=device, dtype=dtype)
        self.bias = nn.Parameter(torch.zeros(local_vocab, device=device, dtype=dtype))
        if self.dense.weight.device.type != "meta":
            nn.init.normal_(self.dense.weight, std=0.02)
            nn.init.zeros_(self.dense.bias)

    def forward(self, hidden, word_embeddings_weight):
        x = F.linear(hidden, self.dense.weight, self.dense.bias, activation="gelu")
        x = self.norm(x)
        x = dist_ops.copy_to_group(x, self.process_group)
        return F.linear(x, word_embeddings_weight, self.bias)


class BertModel(nn.Module):
    def __init__(self, cfg: ModelConfig, num_tokentypes=2, add_binary_head=True, pre_process=True,
                 post_process=True, process_groups=None, pre_post_process_group=None, layer_range=None,
                 sequence_parallel=False, device=None, dtype=None):
        super().__init__()
        assert cfg.add_encoder and not cfg.add_decoder, "bert: encoder only"
        assert cfg.encoder_attn_mask_type is AttnMaskType.padding, "bert: bidirectional attention expected"
        self.cfg, self.pre_process, self.post_process = cfg, pre_process, post_process
        self.add_binary_head = add_binary_head and cfg.add_pooler
        dtype = dtype or cfg.params_dtype
        self.language_model = TransformerLanguageModel(
            cfg, pre_process, post_process, process_groups, pre_post_process_group, layer_range,
            sequence_parallel, device, dtype)
        if post_process:
            grp = self.language_model.pre_post_process_group
            self.lm_head = BertLMHead(cfg, cfg.vocab_size // dist_ops.group_size(grp), grp, device, dtype)
            self.binary_head = nn.Linear(cfg.hidden_size, 2, device=device, dtype=dtype) if self.add_binary_head else None
            # stages that own the head but not the embedding keep their own copy of the word table
            self.word_embeddings = None
            if not pre_process:
                self.word_embeddings = nn.Embedding(cfg.vocab_size // dist_ops.group_size(grp), cfg.hidden_size,
                                                    device=device, dtype=dtype)
                self.word_embeddings.weight._shared_params = True
        # the masked-LM head always uses the word table: split over pipeline stages, the two copies are
        # kept equal by the training session (one copy at start-up) and the engine (gradient sum)
        self.tied_across_stages = not (pre_process and post_process)
        if self.tied_across_stages:
            if pre_process:
                self.language_model.embedding.word_embeddings.weight._tied_across_stages = True
            elif post_process:
                self.word_embeddings.weight._tied_across_stages = True

    def set_input_tensor(self, t):
        self.language_model.set_input_tensor(t)

    def tied_parameter(self):
        """This stage's copy of the word table when the model is split over pipeline stages."""
        if not self.tied_across_stages:
            return None
        if self.pre_process:
            return self.language_model.embedding.word_embeddings.weight
        return self.word_embeddings.weight if self.post_process else None

    def forward(self, input_ids, attention_mask=None, tokentype_ids=None, lm_labels=None, labels=None,
                sentence_order=None):
        lm_labels = lm_labels if lm_labels is not None else labels
        out = self.language_model(input_ids, enc_attn_mask=attention_mask, tokentype_ids=tokentype_ids)
        if not self.post_process:
            return out
        pooled = None
        if self.cfg.add_pooler:
            hidden, pooled = out
        else:
            hidden = out
        if self.language_model.sequence_parallel:
            grp = self.language_model.pre_post_process_group
            # the head's dense + norm run on the full sequence on every rank and the vocabulary
            # projection behind them sums its input gradient over the group, so the gradient that
            # comes back here is complete on every rank
            hidden = dist_ops.all_gather(hidden, grp, replicated_consumer=True).view(
                input_ids.shape[0], -1, hidden.shape[-1])
        wte = (self.language_model.embedding.word_embeddings.weight if self.pre_process
               else self.word_embeddings.weight)
        logits = self.lm_head(hidden, wte)
        binary_logits = self.binary_head(pooled) if (self.add_binary_head and pooled is not None) else None
        if lm_labels is None:
            return logits, binary_logits
        loss = vocab_parallel_cross_entropy(logits.reshape(-1, logits.shape[-1]), lm_labels.reshape(-1),
                                            self.language_model.pre_post_process_group).mean()
        if binary_logits is not None and sentence_order is not None:
            loss = loss + torch.nn.functional.cross_entropy(binary_logits.float(), sentence_order)
        return loss

    def state_dict_for_save_checkpoint(self, prefix="", keep_vars=False):
        sd = {"language_model": self.language_model.state_dict_for_save_checkpoint(prefix, keep_vars)}
        if self.post_process:
            sd["lm_head"] = self.lm_head.state_dict(prefix=prefix, keep_vars=keep_vars)
            if self.binary_head is not None:
                sd["binary_head"] = self.binary_head.state_dict(prefix=prefix, keep_vars=keep_vars)
            if self.word_embeddings is not None:
                sd["word_embeddings_for_head"] = self.word_embeddings.state_dict(prefix=prefix, keep_vars=keep_vars)
        return sd

    def load_state_dict_from_checkpoint(self, sd, strict=True):
        self.language_model.load_state_dict_from_checkpoint(sd["language_model"], strict)
        if self.post_process:
            self.lm_head.load_state_dict(sd["lm_head"], strict=strict)
            if self.binary_head is not None and "binary_head" in sd:
                self.binary_head.load_state_dict(sd["binary_head"], strict=strict)
            if self.word_embeddings is not None and "word_embeddings_for_head" in sd:
                self.word_embeddings.load_state_dict(sd["word_embeddings_for_head"], strict=strict)


def bert_inputs_provider(batch_size, seq_len, vocab_size=None, device="cuda", seed=None, **_):
    gen = torch.Generator(device="cpu").manual_seed(int(seed)) if seed is not None else None
    hi = int(vocab_size or 1000)
    return {
        "input_ids": torch.randint(0, hi, (batch_size, seq_len), generator=gen).to(device),
        "tokentype_ids": torch.randint(0, 2, (batch_size, seq_len), generator=gen).to(device),
        "lm_labels": torch.randint(0, hi, (batch_size, seq_len), generator=gen).to(device),
        "sentence_order": torch.randint(0, 2, (batch_size,), generator=gen).to(device),
    }
