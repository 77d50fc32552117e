"""Activation checkpointing of a transformer block.

The block's forward is re-run during the backward pass instead of keeping its
intermediate activations (reference: mist/utils/gradient_checkpointing.py:33-48, which
wraps ``torch.utils.checkpoint`` in re-entrant mode).  The non-re-entrant form is used
here so that module hooks and tensors that do not require grad behave as in a normal
forward; RNG state is preserved so dropout masks repeat.
"""
from __future__ import annotations

import torch
from torch.utils.checkpoint import checkpoint


def checkpoint_block(layer, hidden, residual, encoder_output, batch_size, attn_mask=None, enc_mask=None):
    # the padding masks travel in the closure: the recomputation must see this call's masks even when
    # later micro batches have run their forward in between
    def run(h, r, e):
        return layer(h, r, e, batch_size, attn_mask, enc_mask)

    return checkpoint(run, hidden, residual, encoder_output, use_reentrant=False, preserve_rng_state=True)
