"""Decoder-only language models: GPT, LLaMA and Falcon share one implementation and
differ only in what their configuration must look like (reference: mist/model/gpt.py:48-163,
llama.py:18-59, falcon.py:18-59)."""
from __future__ import annotations

import torch
import torch.nn as nn

from ..config import AttnMaskType, MLPType, ModelConfig, PositionEmbeddingType
from .language_model import LMHead, TransformerLanguageModel


class GPTModel(nn.Module):
    family = "gpt"

    def __init__(self, cfg: ModelConfig, num_tokentypes=0, pre_process=True, post_process=True,
                 process_groups=None, pre_post_process_group=None, layer_range=None,
                 sequence_parallel=False, device=None, dtype=None):
        super().__init__()
        self.cfg, self.pre_process, self.post_process = cfg, pre_process, post_process
        self._verify_config(cfg)
        self.language_model = TransformerLanguageModel(
            cfg, pre_process, post_process, process_groups, pre_post_process_group, layer_range,
            sequence_parallel, device, dtype)
        self.lm_head = None
        if post_process:
            self.lm_head = LMHead(cfg, self.language_model.pre_post_process_group, sequence_parallel,
                                  device, dtype)
        # Tied embeddings with the embedding and the head on different pipeline stages: the first
        # stage keeps the table, the last stage a copy of it as its projection weight.  The training
        # session copies the table into the copy once and the engine sums the two gradients over
        # the (first stage, last stage) rank pairs before each optimizer step, so the two stay equal.
        self.tied_across_stages = bool(cfg.tie_word_embeddings) and not (pre_process and post_process)
        if self.tied_across_stages:
            if pre_process:
                self.language_model.embedding.word_embeddings.weight._tied_across_stages = True
            if post_process:
                self.lm_head.proj.weight._tied_across_stages = True

    def _verify_config(self, cfg: ModelConfig):
        assert cfg.add_encoder and not cfg.add_decoder and not cfg.add_pooler, \
            f"{self.family}: decoder-only stack without pooler expected"
        assert cfg.encoder_attn_mask_type is AttnMaskType.causal, f"{self.family}: causal mask expected"
        assert not cfg.parallel_block, f"{self.family}: sequential blocks expected"

    def set_input_tensor(self, t):
        self.language_model.set_input_tensor(t)

    def forward(self, input_ids, position_ids=None, attention_mask=None, labels=None, tokentype_ids=None):
        out = self.language_model(input_ids, enc_position_ids=position_ids, enc_attn_mask=attention_mask,
                                  tokentype_ids=tokentype_ids)
        if not self.post_process:
            return out
        tied = None
        if self.cfg.tie_word_embeddings and not self.tied_across_stages:
            tied = self.language_model.embedding.word_embeddings.weight
        return self.lm_head(out, labels, tied)

    def tied_parameter(self):
        """This stage's copy of the table tied across pipeline stages (``None`` on other stages)."""
        if not self.tied_across_stages:
            return None
        if self.pre_process:
            return self.language_model.embedding.word_embeddings.weight
        return self.lm_head.proj.weight if self.post_process else None

    def state_dict_for_save_checkpoint(self, prefix="", keep_vars=False):
        sd = {"language_model": self.language_model.state_dict_for_save_checkpoint(prefix, keep_vars)}
        if self.lm_head is not None and (not self.cfg.tie_word_embeddings or self.tied_across_stages):
            sd["lm_head"] = self.lm_head.state_dict(prefix=prefix, keep_vars=keep_vars)
        return sd

    def load_state_dict_from_checkpoint(self, sd, strict=True):
        self.language_model.load_state_dict_from_checkpoint(sd["language_model"], strict)
        if self.lm_head is not None and "lm_head" in sd:
            self.lm_head.load_state_dict(sd["lm_head"], strict=strict)


class LLamaModel(GPTModel):
    family = "llama"

    def _verify_config(self, cfg):
        super()._verify_config(cfg)
        assert cfg.mlp_type is MLPType.gated_mlp and cfg.normalization.lower() == "rmsnorm", \
            "llama: gated MLP and RMSNorm expected"
        assert cfg.position_embedding_type is PositionEmbeddingType.rotary, "llama: rotary positions expected"


class FalconModel(GPTModel):
    family = "falcon"

    def _verify_config(self, cfg):
        assert cfg.add_encoder and not cfg.add_decoder and not cfg.add_pooler
        assert cfg.encoder_attn_mask_type is AttnMaskType.causal
        assert cfg.parallel_block, "falcon: parallel attention/MLP blocks expected"
        assert cfg.position_embedding_type is PositionEmbeddingType.rotary, "falcon: rotary positions expected"


def gpt_inputs_provider(batch_size, seq_len, vocab_size=None, device="cuda", seed=None, **_):
    """Synthetic batch: token ids uniform over the vocabulary, labels likewise
    (reference: mist/model/gpt.py:165-193 uses ids in [0,1000) and labels in [0,10))."""
    gen = None
    if seed is not None:
        gen = torch.Generator(device="cpu").manual_seed(int(seed))
    hi = int(vocab_size or 1000)
    ids = torch.randint(0, hi, (batch_size, seq_len), generator=gen)
    labels = torch.randint(0, hi, (batch_size, seq_len), generator=gen)
    return {"input_ids": ids.to(device), "labels": labels.to(device)}
