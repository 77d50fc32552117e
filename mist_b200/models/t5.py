"""T5: encoder-decoder with cross attention and a tied LM head
(reference: mist/model/t5.py:43-72 head, :74-301 model)."""
from __future__ import annotations

import torch
import torch.nn as nn

from ..config import ModelConfig
from ..modules.layers import vocab_parallel_cross_entropy
from ..ops import functional as F
from ..parallel import dist_ops
from .language_model import TransformerLanguageModel


class T5LMHead(nn.Module):
    """Tied vocabulary projection with a per-rank bias slice."""

    def __init__(self, local_vocab, process_group=None, device=None, dtype=None, sequence_parallel=False):
        super().__init__()
        self.process_group = process_group
        self.sequence_parallel = sequence_parallel
        self.bias = nn.Parameter(torch.zeros(local_vocab, device=device, dtype=dtype))

    def forward(self, hidden, word_embeddings_weight):
        if self.sequence_parallel:      # token shards -> all tokens; the backward pass reduce-scatters
            x = dist_ops.all_gather(hidden.reshape(-1, hidden.shape[-1]), self.process_group)
        else:
            x = dist_ops.copy_to_group(hidden, self.process_group)
        return F.linear(x, word_embeddings_weight, self.bias)


class T5Model(nn.Module):
    def __init__(self, cfg: ModelConfig, num_tokentypes=0, pre_process=True, post_process=True,
                 process_groups=None, pre_post_process_group=None, layer_range=None,
                 sequence_parallel=False, device=None, dtype=None):
        """Over pipeline stages (``pre_process`` / ``post_process`` not both true) the encoder blocks
        ``layer_range`` go to the stages before the last, the last stage holds the whole decoder, its
        own copy of the word table (decoder input embedding and output projection) and the head."""
        super().__init__()
        assert cfg.add_encoder and cfg.add_decoder, "t5: encoder and decoder stacks expected"
        self.cfg, self.pre_process, self.post_process = cfg, pre_process, post_process
        dtype = dtype or cfg.params_dtype
        self.tied_across_stages = not (pre_process and post_process)
        stacks = ("encoder", "decoder") if not self.tied_across_stages else (("decoder",) if post_process else ("encoder",))
        self.language_model = TransformerLanguageModel(
            cfg, pre_process or post_process, post_process, process_groups, pre_post_process_group, layer_range,
            sequence_parallel, device, dtype, stacks=stacks)
        if self.tied_across_stages and (pre_process or post_process):
            # encoder and decoder share one embedding (word and position tables): both copies are tied
            for p in self.language_model.embedding.parameters():
                p._tied_across_stages = True
        if post_process:
            grp = self.language_model.pre_post_process_group
            self.lm_head = T5LMHead(cfg.vocab_size // dist_ops.group_size(grp), grp, device, dtype,
                                    sequence_parallel and dist_ops.group_size(grp) > 1)

    def set_input_tensor(self, t):
        self.language_model.set_input_tensor(t)

    def tied_parameters(self):
        """This stage's copies of the embedding tables when the model is split over pipeline stages."""
        if not self.tied_across_stages or not (self.pre_process or self.post_process):
            return []
        return list(self.language_model.embedding.parameters())

    def forward(self, encoder_input_ids, decoder_input_ids, encoder_attn_mask=None, decoder_attn_mask=None,
                encoder_decoder_attn_mask=None, tokentype_ids=None, lm_labels=None, labels=None,
                enc_hidden_states=None):
        lm_labels = lm_labels if lm_labels is not None else labels
        if self.language_model.decoder is None:      # encoder-only pipeline stage
            return self.language_model(encoder_input_ids, enc_attn_mask=encoder_attn_mask, tokentype_ids=tokentype_ids)
        dec_out, enc_out = self.language_model(
            encoder_input_ids, dec_input_ids=decoder_input_ids, tokentype_ids=tokentype_ids,
            enc_hidden_states=enc_hidden_states, enc_attn_mask=encoder_attn_mask, dec_attn_mask=decoder_attn_mask,
            enc_dec_attn_mask=encoder_decoder_attn_mask)
        if not self.post_process:
            return dec_out, enc_out
        logits = self.lm_head(dec_out, self.language_model.embedding.word_embeddings.weight)
        if lm_labels is None:
            return logits
        return vocab_parallel_cross_entropy(logits.reshape(-1, logits.shape[-1]), lm_labels.reshape(-1),
                                            self.language_model.pre_post_process_group).mean()

    def state_dict_for_save_checkpoint(self, prefix="", keep_vars=False):
        sd = {"language_model": self.language_model.state_dict_for_save_checkpoint(prefix, keep_vars)}
        if self.post_process:
            sd["lm_head"] = self.lm_head.state_dict(prefix=prefix, keep_vars=keep_vars)
        return sd

    def load_state_dict_from_checkpoint(self, sd, strict=True):
        self.language_model.load_state_dict_from_checkpoint(sd["language_model"], strict)
        if self.post_process and "lm_head" in sd:
            self.lm_head.load_state_dict(sd["lm_head"], strict=strict)


def t5_inputs_provider(batch_size, seq_len, vocab_size=None, device="cuda", seed=None, decoder_seq_len=None, **_):
    gen = torch.Generator(device="cpu").manual_seed(int(seed)) if seed is not None else None
    hi = int(vocab_size or 1000)
    dl = decoder_seq_len or seq_len
    return {
        "encoder_input_ids": torch.randint(0, hi, (batch_size, seq_len), generator=gen).to(device),
        "decoder_input_ids": torch.randint(0, hi, (batch_size, dl), generator=gen).to(device),
        "lm_labels": torch.randint(0, hi, (batch_size, dl), generator=gen).to(device),
    }
