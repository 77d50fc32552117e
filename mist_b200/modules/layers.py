"""Module library: tensor-parallel linears, norms, embeddings, attention and MLP blocks.

Activations are ``[batch, seq, hidden]``.  Under sequence parallelism the regions
between a row-parallel output and the next column-parallel input hold
``[batch * seq / tp, hidden]`` token shards (tokens flattened, dim 0 split), the
column-parallel linear all-gathers its input and the row-parallel linear
reduce-scatters its output.

Parity map (reference): ColumnParallelLinear / RowParallelLinear
mist/modules/fused_dense.py:221-327; ParallelMHA mist/modules/mha.py:1028-1337;
ParallelMLP / ParallelGatedMlp mist/modules/mlp.py:17-128; VocabParallelEmbedding /
ParallelEmbedding mist/modules/embedding.py:17-299; LayerNorm / RMSNorm
mist/modules/layer_norm.py:880-908, rms_norm.py:124-139; RotaryEmbedding
mist/modules/rotary.py:348-540.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as F
from ..parallel import dist_ops
from ..parallel.dist_ops import group_rank, group_size


def _empty_param(*shape, dtype, device):
    return nn.Parameter(torch.empty(*shape, dtype=dtype, device=device))


# ------------------------------------------------------------------------------- norms
class LayerNorm(nn.Module):
    """LayerNorm with the residual add folded in: ``forward(x, residual)`` returns
    ``(norm(x + residual), x + residual)`` when ``prenorm`` else ``norm(x + residual)``."""

    def __init__(self, hidden_size, eps=1e-5, prenorm=False, sequence_parallel=False, device=None, dtype=None):
        super().__init__()
        self.eps, self.prenorm = eps, prenorm
        self.weight = _empty_param(hidden_size, dtype=dtype, device=device)
        self.bias = _empty_param(hidden_size, dtype=dtype, device=device)
        self.weight._sequence_parallel = self.bias._sequence_parallel = sequence_parallel
        self.reset_parameters()

    def reset_parameters(self):
        if self.weight.device.type != "meta":
            nn.init.ones_(self.weight)
            nn.init.zeros_(self.bias)

    def forward(self, x, residual=None, dropout_p: float = 0.0, seed: int = 0):
        """``dropout_p`` / ``seed``: dropout applied to ``x`` before the residual add, inside the kernel."""
        return F.layer_norm(x, self.weight, self.bias, self.eps, residual=residual, prenorm=self.prenorm,
                            dropout_p=dropout_p, seed=seed)


class RMSNorm(nn.Module):
    def __init__(self, hidden_size, eps=1e-5, prenorm=False, sequence_parallel=False, device=None, dtype=None):
        super().__init__()
        self.eps, self.prenorm = eps, prenorm
        self.weight = _empty_param(hidden_size, dtype=dtype, device=device)
        self.weight._sequence_parallel = sequence_parallel
        self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self):
        if self.weight.device.type != "meta":
            nn.init.ones_(self.weight)

    def forward(self, x, residual=None, dropout_p: float = 0.0, seed: int = 0):
        return F.rms_norm(x, self.weight, self.eps, residual=residual, prenorm=self.prenorm,
                          dropout_p=dropout_p, seed=seed)


def get_norm(kind: str, hidden_size, eps, prenorm=False, sequence_parallel=False, device=None, dtype=None):
    cls = RMSNorm if kind.lower() == "rmsnorm" else LayerNorm
    return cls(hidden_size, eps=eps, prenorm=prenorm, sequence_parallel=sequence_parallel, device=device, dtype=dtype)


# ----------------------------------------------------------------------------- linears
class FusedDense(nn.Module):
    """``act(x W^T + b)``; all three GEMMs run on the tcgen05 kernel."""

    def __init__(self, in_features, out_features, bias=True, activation=None, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features, self.activation = in_features, out_features, activation
        self.weight = _empty_param(out_features, in_features, dtype=dtype, device=device)
        self.bias = _empty_param(out_features, dtype=dtype, device=device) if bias else None
        self.reset_parameters()

    def reset_parameters(self, std: float = 0.02):
        if self.weight.device.type != "meta":
            nn.init.normal_(self.weight, mean=0.0, std=std)
            if self.bias is not None:
                nn.init.zeros_(self.bias)

    def forward(self, x, residual=None):
        return F.linear(x, self.weight, self.bias, activation=self.activation, residual=residual)


class ColumnParallelLinear(FusedDense):
    """Output features split over the tensor-parallel group.  With sequence parallelism
    the input is a token shard that is all-gathered first (and its gradient
    reduce-scattered); without it the input is replicated and its gradient all-reduced."""

    def __init__(self, in_features, out_features, process_group=None, bias=True, activation=None,
                 sequence_parallel=False, multiple_of=1, device=None, dtype=None):
        ws, rk = group_size(process_group), group_rank(process_group)
        assert out_features % multiple_of == 0
        local_out = dist_ops.dim_for_rank(out_features, ws, rk, multiple_of)
        super().__init__(in_features, local_out, bias=bias, activation=activation, device=device, dtype=dtype)
        self.process_group, self.sequence_parallel = process_group, sequence_parallel
        self.global_out_features = out_features
        # each rank holds its own slice: not to be made equal over the tensor-parallel group
        self.weight._tp_sharded = True
        if self.bias is not None:
            self.bias._tp_sharded = True

    def _fused(self, x) -> bool:
        return (self.sequence_parallel and F.Settings.tp_backend == "fused" and isinstance(x, torch.Tensor)
                and x.is_cuda and group_size(self.process_group) > 1
                and not isinstance(self.process_group, dist_ops.FakeGroup))

    def forward(self, x, residual=None):
        if self._fused(x) and residual is None:
            from ..parallel import fused_tp
            y = fused_tp.ag_linear(x.reshape(-1, x.shape[-1]), self.weight, self.bias,
                                   fused_tp.context_for(self.process_group))
            return F.gelu(y) if self.activation == "gelu" else y
        if self.sequence_parallel:
            x = dist_ops.all_gather(x.reshape(-1, x.shape[-1]), self.process_group)
        else:
            x = dist_ops.copy_to_group(x, self.process_group)
        return F.linear(x, self.weight, self.bias, activation=self.activation, residual=residual)


class RowParallelLinear(FusedDense):
    """Input features split over the group; the partial outputs are summed by an
    all-reduce, or by a reduce-scatter over tokens under sequence parallelism.  The bias
    (if any) is applied by the first rank only so that the sum counts it once."""

    def __init__(self, in_features, out_features, process_group=None, bias=True, sequence_parallel=False,
                 multiple_of=1, device=None, dtype=None):
        ws, rk = group_size(process_group), group_rank(process_group)
        local_in = dist_ops.dim_for_rank(in_features, ws, rk, multiple_of)
        super().__init__(local_in, out_features, bias=bias and rk == 0, device=device, dtype=dtype)
        self.process_group, self.sequence_parallel = process_group, sequence_parallel
        self.weight._tp_sharded = True
        if self.bias is not None:
            self.bias._tp_sharded = True      # exists on the first rank only
        # the bias lives on the first rank only and its gradient there is already complete (the
        # backward pass of the reduce-scatter gathers the full output gradient), so it takes no
        # part in the tensor-parallel gradient sum

    def forward(self, x, residual=None):
        ws = group_size(self.process_group)
        if ws == 1:
            return F.linear(x, self.weight, self.bias, residual=residual)
        if (self.sequence_parallel and F.Settings.tp_backend == "fused" and isinstance(x, torch.Tensor) and x.is_cuda
                and not isinstance(self.process_group, dist_ops.FakeGroup)):
            from ..parallel import fused_tp
            res2 = None if residual is None else residual.reshape(-1, residual.shape[-1])
            return fused_tp.linear_rs(x.reshape(-1, x.shape[-1]), self.weight, self.bias,
                                      fused_tp.context_for(self.process_group), residual=res2)
        y = F.linear(x, self.weight, self.bias)
        if self.sequence_parallel:
            y = dist_ops.reduce_scatter(y.reshape(-1, y.shape[-1]), self.process_group)
        else:
            y = dist_ops.all_reduce(y, self.process_group)
        if residual is not None:
            y = y + residual.reshape(y.shape)
        return y


# -------------------------------------------------------------------------- embeddings
class VocabParallelEmbedding(nn.Module):
    """Word (+ learned position, + token type) embeddings; the vocabulary is split over the
    tensor-parallel group and out-of-slice ids contribute zeros before the all-reduce."""

    def __init__(self, vocab_size, hidden_size, max_position_embeddings=0, num_tokentypes=0,
                 process_group=None, sequence_parallel=False, padding_idx=None, device=None, dtype=None):
        super().__init__()
        ws, rk = group_size(process_group), group_rank(process_group)
        assert vocab_size % ws == 0, f"vocab {vocab_size} must divide by tp {ws}"
        self.process_group, self.sequence_parallel = process_group, sequence_parallel
        self.vocab_size, self.local_vocab = vocab_size, vocab_size // ws
        self.vocab_start = rk * self.local_vocab
        self.padding_idx = padding_idx
        self.word_embeddings = nn.Embedding(self.local_vocab, hidden_size, device=device, dtype=dtype)
        self.word_embeddings.weight._tp_sharded = True
        self.position_embeddings = (nn.Embedding(max_position_embeddings, hidden_size, device=device, dtype=dtype)
                                    if max_position_embeddings > 0 else None)
        self.tokentype_embeddings = (nn.Embedding(num_tokentypes, hidden_size, device=device, dtype=dtype)
                                     if num_tokentypes > 0 else None)
        # position / token-type tables are replicated but only the first rank adds them (before the
        # all-reduce or reduce-scatter), so only it sees their gradient: the engine sums these
        # gradients over the tensor-parallel group to keep the replicas identical
        for emb in (self.position_embeddings, self.tokentype_embeddings):
            if emb is not None and ws > 1:
                emb.weight._tp_partial_grad = True
        self.reset_parameters()

    def reset_parameters(self, std=0.02):
        for emb in (self.word_embeddings, self.position_embeddings, self.tokentype_embeddings):
            if emb is not None and emb.weight.device.type != "meta":
                nn.init.normal_(emb.weight, mean=0.0, std=std)

    def forward(self, input_ids, position_ids=None, tokentype_ids=None):
        ws = group_size(self.process_group)
        wpe = self.position_embeddings.weight if self.position_embeddings is not None else None
        if position_ids is not None and wpe is not None:
            # explicit position ids: gather rows, the fused kernel handles the arange case
            x = F.embedding(input_ids, self.word_embeddings.weight, None, self.vocab_start)
            pos = wpe[position_ids]
            x = x + (pos if ws == 1 or group_rank(self.process_group) == 0 else 0)
        else:
            use_pos = wpe is not None and (ws == 1 or group_rank(self.process_group) == 0)
            x = F.embedding(input_ids, self.word_embeddings.weight, wpe if use_pos else None, self.vocab_start)
        if tokentype_ids is not None and self.tokentype_embeddings is not None:
            tt = self.tokentype_embeddings(tokentype_ids)
            x = x + (tt if ws == 1 or group_rank(self.process_group) == 0 else 0)
        if ws > 1:
            if self.sequence_parallel:
                x = dist_ops.reduce_scatter(x.reshape(-1, x.shape[-1]), self.process_group)
            else:
                x = dist_ops.all_reduce(x, self.process_group)
        return x

    def state_dict_for_save_checkpoint(self, prefix="", keep_vars=False):
        sd = {"word_embeddings": self.word_embeddings.state_dict(prefix=prefix, keep_vars=keep_vars)}
        if self.position_embeddings is not None:
            sd["position_embeddings"] = self.position_embeddings.state_dict(prefix=prefix, keep_vars=keep_vars)
        if self.tokentype_embeddings is not None:
            sd["tokentype_embeddings"] = self.tokentype_embeddings.state_dict(prefix=prefix, keep_vars=keep_vars)
        return sd

    def load_state_dict_from_checkpoint(self, sd, strict=True):
        self.word_embeddings.load_state_dict(sd["word_embeddings"], strict=strict)
        if self.position_embeddings is not None and "position_embeddings" in sd:
            self.position_embeddings.load_state_dict(sd["position_embeddings"], strict=strict)
        if self.tokentype_embeddings is not None and "tokentype_embeddings" in sd:
            self.tokentype_embeddings.load_state_dict(sd["tokentype_embeddings"], strict=strict)


# --------------------------------------------------------------------------- attention
class PaddingMask:
    """Key-padding mask of a batch, prepared once per forward pass and shared by every layer.

    ``mask``: ``[batch, seq]``, non-zero = real token.  Attention then runs per sample over its real
    tokens only (the tokens are sliced out when the padding is on the right, gathered otherwise) and
    the rows of padded positions come back as zeros -- the same result as removing the padding,
    running variable-length attention and padding the output again (reference:
    ``unpad_input`` / ``pad_input`` around the attention core, mist/modules/mha.py:1233-1243,1332-1334).
    When every sample is padded on the right (the usual batch layout) the whole batch runs as one launch
    of the attention kernels with the per-sample lengths passed on the device (``lengths_dev``).
    Preparing the mask reads it back to the host once, to find out whether that is the case and whether
    there is any padding at all; with ``assume_right_padded`` (class attribute, or the argument) nothing
    is read back: the mask is taken to be right-padded and only the lengths are computed, on the device.
    """

    #: trust that masks are right-padded (no validation, no host read-back)
    assume_right_padded = False

    def __init__(self, mask: torch.Tensor, assume_right_padded: Optional[bool] = None):
        assert mask.dim() == 2, "padding mask: [batch, seq] expected"
        valid = mask != 0
        b, s = valid.shape
        lens = valid.sum(1)
        self.valid = valid
        self.seq_len = s
        #: real tokens per sample, int32 on the mask's device (what the kernels take)
        self.lengths_dev = lens.to(torch.int32)
        trust = PaddingMask.assume_right_padded if assume_right_padded is None else assume_right_padded
        if trust:
            self.lengths, self.is_prefix, self.indices = None, None, None
            self.right_padded, self.all_valid = True, False
            return
        prefix = (valid == (torch.arange(s, device=valid.device)[None, :] < lens[:, None])).all(1)
        host = torch.stack([lens, prefix.long()], 1).tolist()
        self.lengths = [int(n) for n, _ in host]
        self.is_prefix = [bool(p) for _, p in host]
        self.indices = [None if self.is_prefix[i] else valid[i].nonzero().squeeze(1) for i in range(b)]
        self.all_valid = all(n == s for n in self.lengths)
        self.right_padded = all(self.is_prefix)

    @staticmethod
    def prepare(mask) -> Optional["PaddingMask"]:
        """``None`` for no mask or a mask without padding; masks already prepared pass through."""
        if mask is None:
            return None
        pm = mask if isinstance(mask, PaddingMask) else PaddingMask(mask)
        return None if pm.all_valid else pm

    def select(self, x: torch.Tensor, i: int) -> torch.Tensor:
        """Real tokens of sample ``i`` of ``x`` ``[batch, seq, ...]`` as ``[1, n_i, ...]``."""
        if self.is_prefix[i]:
            return x[i:i + 1, :self.lengths[i]]
        return x[i:i + 1].index_select(1, self.indices[i])

    def restore(self, part: torch.Tensor, i: int) -> torch.Tensor:
        """``[1, n_i, ...]`` back to ``[1, seq, ...]`` with zeros at the padded positions."""
        n, s = self.lengths[i], self.seq_len
        if n == s:
            return part
        if self.is_prefix[i]:
            return torch.cat([part, part.new_zeros(1, s - n, *part.shape[2:])], 1)
        return part.new_zeros(1, s, *part.shape[2:]).index_copy(1, self.indices[i], part)


class ParallelMHA(nn.Module):
    """Multi-head (self or cross) attention with heads split over the tensor-parallel group.

    ``use_flash_attn`` selects the tcgen05 flash kernel; otherwise scores are
    materialised and normalised by the scaled (causal) softmax kernel, which is the
    O(s^2)-memory path the analyzer also models."""

    def __init__(self, hidden_size, num_heads, num_heads_kv=None, process_group=None, qkv_proj_bias=True,
                 out_proj_bias=True, dropout=0.0, softmax_scale=None, causal=False, cross_attn=False,
                 rotary_emb_dim=0, rotary_emb_base=10000.0, use_flash_attn=True, sequence_parallel=False,
                 layer_idx=None, device=None, dtype=None, rotary_emb_interleaved=False, rotary_emb_scale_base=None):
        super().__init__()
        # interleaved: pairs (2i, 2i+1) rotate together instead of (i, i + rot/2); scale_base: position
        # dependent scaling of the rotated q (up) and k (down) ("xpos").  Both take the general path
        # below (rotary out of place), not the in-kernel rotation of the packed fast path.
        self.rotary_interleaved = bool(rotary_emb_interleaved) and rotary_emb_dim > 0
        self.rotary_scale_base = float(rotary_emb_scale_base) if (rotary_emb_scale_base and rotary_emb_dim > 0) else None
        ws = group_size(process_group)
        self.hidden_size, self.causal, self.cross_attn = hidden_size, causal, cross_attn
        self.num_heads = num_heads
        self.num_heads_kv = num_heads_kv or num_heads
        assert num_heads % ws == 0 and self.num_heads_kv % ws == 0, "heads must divide by tp"
        assert hidden_size % num_heads == 0
        self.head_dim = hidden_size // num_heads
        self.local_heads, self.local_heads_kv = num_heads // ws, self.num_heads_kv // ws
        self.rotary_emb_dim, self.rotary_emb_base = int(rotary_emb_dim), rotary_emb_base
        self.use_flash_attn, self.dropout, self.layer_idx = use_flash_attn, dropout, layer_idx
        self.softmax_scale = softmax_scale or 1.0 / math.sqrt(self.head_dim)
        self.process_group, self.sequence_parallel = process_group, sequence_parallel
        kv_dim = self.num_heads_kv * self.head_dim
        fk = dict(process_group=process_group, sequence_parallel=sequence_parallel, device=device, dtype=dtype)
        if not cross_attn:
            self.Wqkv = ColumnParallelLinear(hidden_size, hidden_size + 2 * kv_dim, bias=qkv_proj_bias,
                                             multiple_of=self.head_dim * (self.num_heads // self.num_heads_kv + 2), **fk)
        else:
            self.Wq = ColumnParallelLinear(hidden_size, hidden_size, bias=qkv_proj_bias,
                                           multiple_of=self.head_dim, **fk)
            self.Wkv = ColumnParallelLinear(hidden_size, 2 * kv_dim, bias=qkv_proj_bias,
                                            multiple_of=2 * self.head_dim, **fk)
        self.out_proj = RowParallelLinear(hidden_size, hidden_size, bias=out_proj_bias,
                                          multiple_of=self.head_dim, **fk)

    def _attend(self, q, k, v, causal):
        if self.use_flash_attn:
            return F.attention(q, k, v, self.softmax_scale, causal)
        # materialised scores: [b, h, sq, sk]
        b, sq, nh, d = q.shape
        if k.shape[2] != nh:
            k = k.repeat_interleave(nh // k.shape[2], dim=2)
            v = v.repeat_interleave(nh // v.shape[2], dim=2)
        scores = torch.matmul(q.transpose(1, 2), k.permute(0, 2, 3, 1))
        probs = F.scaled_causal_softmax(scores, self.softmax_scale, causal)
        if self.dropout > 0 and self.training:
            probs = torch.nn.functional.dropout(probs, self.dropout)
        return torch.matmul(probs, v.transpose(1, 2)).transpose(1, 2)

    def _general_rotary(self, qk, num_q_heads: int):
        """Rotary embedding of ``qk`` ``[b, s, q heads + k heads, d]`` for the interleaved and the
        position-scaled forms.  Interleaved pairs are first moved to the half-split positions; q and
        k get the same permutation of their head dimension, which leaves every q . k unchanged, so
        nothing is permuted back."""
        b, s, H, d = qk.shape
        rot = self.rotary_emb_dim
        if self.rotary_interleaved:
            perm = torch.cat([torch.arange(0, rot, 2), torch.arange(1, rot, 2), torch.arange(rot, d)]).to(qk.device)
            qk = qk.index_select(-1, perm)
        cos, sin = F.rope_tables(s, rot, self.rotary_emb_base, qk.device)
        qk = _RotaryOutOfPlace.apply(qk.unsqueeze(2), cos, sin, rot, 1).squeeze(2)
        if self.rotary_scale_base is not None:
            base = (torch.arange(0, rot, 2, dtype=torch.float32, device=qk.device) + 0.4 * rot) / (1.4 * rot)
            power = (torch.arange(s, dtype=torch.float32, device=qk.device) - s // 2) / self.rotary_scale_base
            sc = base[None, :] ** power[:, None]                          # [s, rot / 2]
            full = torch.cat([sc, sc, torch.ones(s, d - rot, device=qk.device)], -1).to(qk.dtype)
            qk = torch.cat([qk[:, :, :num_q_heads] * full[None, :, None, :],
                            qk[:, :, num_q_heads:] / full[None, :, None, :]], 2)
        return qk

    def _attend_masked(self, q, k, v, causal, q_mask: Optional[PaddingMask], k_mask: Optional[PaddingMask]):
        """Attention over the real tokens of every sample; rows of padded queries are zero.  Right-padded
        batches run as one launch with the lengths on the device; other masks go sample by sample."""
        if (self.use_flash_attn and (q_mask is None or q_mask.right_padded)
                and (k_mask is None or k_mask.right_padded)):
            return F.attention(q, k, v, self.softmax_scale, causal,
                               seqlens_q=None if q_mask is None else q_mask.lengths_dev,
                               seqlens_k=None if k_mask is None else k_mask.lengths_dev)
        outs = []
        for i in range(q.shape[0]):
            qi = q_mask.select(q, i) if q_mask is not None else q[i:i + 1]
            ki = k_mask.select(k, i) if k_mask is not None else k[i:i + 1]
            vi = k_mask.select(v, i) if k_mask is not None else v[i:i + 1]
            if qi.shape[1] == 0 or ki.shape[1] == 0:
                oi = qi.new_zeros(1, qi.shape[1], q.shape[2], q.shape[3])
            else:
                oi = self._attend(qi, ki, vi, causal)
            outs.append(q_mask.restore(oi, i) if q_mask is not None else oi)
        return torch.cat(outs, 0)

    def _forward_cached(self, x, residual=None):
        """Inference with a key/value cache (``self.inference_params`` set by
        :mod:`mist_b200.inference`): the new keys and values are appended to this layer's cache;
        a multi-token call (the prompt) attends causally inside itself, a single-token call
        runs the single-query kernel over the cache (reference: the ``inference_params``
        branches of mist/modules/mha.py:531-575,1110-1170)."""
        ip = self.inference_params
        assert not self.cross_attn and not self.sequence_parallel and x.dim() == 3
        if self.rotary_interleaved or self.rotary_scale_base is not None:
            raise NotImplementedError("cached generation with interleaved or position-scaled rotary embeddings")
        qkv = self.Wqkv(x)
        b, s = qkv.shape[:2]
        hq, hk, d = self.local_heads, self.local_heads_kv, self.head_dim
        off = ip.seqlen_offset
        if hq == hk:
            qkv = qkv.view(b, s, 3, hq, d)
            if self.rotary_emb_dim > 0:
                cos, sin = F.rope_tables(ip.max_seqlen, self.rotary_emb_dim, self.rotary_emb_base, qkv.device)
                qkv = F.apply_rotary_qkv_(qkv.contiguous(), cos[off:off + s], sin[off:off + s], self.rotary_emb_dim)
            q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        else:
            qk = qkv[..., : (hq + hk) * d].reshape(b, s, 1, hq + hk, d)
            if self.rotary_emb_dim > 0:
                cos, sin = F.rope_tables(ip.max_seqlen, self.rotary_emb_dim, self.rotary_emb_base, qkv.device)
                qk = F._rope_apply(qk.contiguous().clone(), cos[off:off + s], sin[off:off + s], self.rotary_emb_dim,
                                   False, 1)
            qk = qk.reshape(b, s, hq + hk, d)
            q, k = qk[:, :, :hq], qk[:, :, hq:]
            v = qkv[..., (hq + hk) * d:].reshape(b, s, hk, d)
        cache = ip.cache_for(self.layer_idx, b, hk, d, qkv.dtype, qkv.device)      # [b, max_seq, 2, hk, d]
        cache[:b, off:off + s, 0].copy_(k)
        cache[:b, off:off + s, 1].copy_(v)
        if s == 1:
            ctx = F.decode_attention(q[:, 0], cache[:b, :, 0], cache[:b, :, 1], off + 1, self.softmax_scale)
            ctx = ctx.unsqueeze(1)
        else:
            assert off == 0, "a multi-token call must start the sequence (prompt processing)"
            ctx = self._attend(q, k, v, self.causal)
        ctx = ctx.reshape(b, s, -1)
        return self.out_proj(ctx, residual=residual)

    def forward(self, x, x_kv=None, batch_size=None, residual=None, attention_mask: Optional[PaddingMask] = None,
                kv_mask: Optional[PaddingMask] = None):
        """``x``: [b, s, h], or a [b*s/tp, h] token shard under sequence parallelism (then
        ``batch_size`` is needed to recover the sequence length).  ``attention_mask`` marks the
        real tokens of ``x`` (queries, and keys too in self attention); ``kv_mask`` those of ``x_kv``."""
        if getattr(self, "inference_params", None) is not None:
            return self._forward_cached(x, residual)
        masked = attention_mask is not None or kv_mask is not None
        if not self.cross_attn:
            qkv = self.Wqkv(x)
            if qkv.dim() == 2:
                qkv = qkv.view(batch_size, -1, qkv.shape[-1])
            b, s = qkv.shape[:2]
            if self.local_heads == self.local_heads_kv:
                qkv = qkv.view(b, s, 3, self.local_heads, self.head_dim)
                rotary = None
                # (the symbolic trace of the analyzer prices these forms like the plain rotation)
                general_rotary = (self.rotary_interleaved or self.rotary_scale_base is not None) and not F._sym(qkv)
                if general_rotary:
                    h = self.local_heads
                    qk = self._general_rotary(qkv[:, :, :2].reshape(b, s, 2 * h, self.head_dim), h)
                    if masked:
                        ctx = self._attend_masked(qk[:, :, :h], qk[:, :, h:], qkv[:, :, 2], self.causal,
                                                  attention_mask, attention_mask)
                    else:
                        ctx = self._attend(qk[:, :, :h], qk[:, :, h:], qkv[:, :, 2], self.causal)
                    ctx = ctx.reshape(ctx.shape[0], ctx.shape[1], -1)
                    return self.out_proj(ctx, residual=residual)
                if self.rotary_emb_dim > 0:
                    cos, sin = F.rope_tables(s, self.rotary_emb_dim, self.rotary_emb_base, qkv.device)
                    rotary = (cos, sin, self.rotary_emb_dim)
                if masked:
                    if rotary is not None:      # positions are those of the padded layout
                        qkv = _RotaryOutOfPlace.apply(qkv, *rotary)
                    ctx = self._attend_masked(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], self.causal,
                                              attention_mask, attention_mask)
                elif self.use_flash_attn:
                    ctx = F.attention_qkvpacked(qkv, self.softmax_scale, self.causal, rotary)
                else:
                    if rotary is not None:
                        qkv = _RotaryOutOfPlace.apply(qkv, *rotary)
                    ctx = self._attend(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], self.causal)
            else:
                hq, hk, d = self.local_heads, self.local_heads_kv, self.head_dim
                if (self.rotary_interleaved or self.rotary_scale_base is not None) and not F._sym(qkv):
                    qk = self._general_rotary(qkv[..., : (hq + hk) * d].reshape(b, s, hq + hk, d), hq)
                    q, k = qk[:, :, :hq], qk[:, :, hq:]
                elif self.rotary_emb_dim > 0:
                    # grouped-query layout [q heads | k heads | v heads]: rotate the q and k heads together
                    cos, sin = F.rope_tables(s, self.rotary_emb_dim, self.rotary_emb_base, qkv.device)
                    qk = qkv[..., : (hq + hk) * d].reshape(b, s, 1, hq + hk, d)
                    qk = _RotaryOutOfPlace.apply(qk, cos, sin, self.rotary_emb_dim, 1).reshape(b, s, hq + hk, d)
                    q, k = qk[:, :, :hq], qk[:, :, hq:]
                else:
                    q = qkv[..., : hq * d].reshape(b, s, hq, d)
                    k = qkv[..., hq * d: (hq + hk) * d].reshape(b, s, hk, d)
                v = qkv[..., (hq + hk) * d:].reshape(b, s, hk, d)
                if masked:
                    ctx = self._attend_masked(q, k, v, self.causal, attention_mask, attention_mask)
                else:
                    ctx = self._attend(q, k, v, self.causal)
        else:
            q = self.Wq(x)
            kv = self.Wkv(x_kv)
            if q.dim() == 2:
                q = q.view(batch_size, -1, q.shape[-1])
                kv = kv.view(batch_size, -1, kv.shape[-1])
            b, sq = q.shape[:2]
            q = q.view(b, sq, self.local_heads, self.head_dim)
            kv = kv.view(b, kv.shape[1], 2, self.local_heads_kv, self.head_dim)
            if masked:
                ctx = self._attend_masked(q, kv[:, :, 0], kv[:, :, 1], False, attention_mask, kv_mask)
            else:
                ctx = self._attend(q, kv[:, :, 0], kv[:, :, 1], False)
        ctx = ctx.reshape(ctx.shape[0], ctx.shape[1], -1)
        return self.out_proj(ctx, residual=residual)


class _RotaryOutOfPlace(torch.autograd.Function):
    """Differentiable rotary embedding for the non-flash attention path."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, rot, n_rot=2):
        """``qkv``: ``[b, s, n, heads, d]``; the first ``n_rot`` of the ``n`` slots are rotated."""
        ctx.save_for_backward(cos, sin)
        ctx.rot, ctx.n_rot = rot, n_rot
        return F._rope_apply(qkv.contiguous().clone(), cos, sin, rot, False, n_rot)

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        return F._rope_apply(g.contiguous().clone(), cos, sin, ctx.rot, True, ctx.n_rot), None, None, None, None


# --------------------------------------------------------------------------------- MLP
_TANH_GELU = ("gelu_new", "gelu_fast", "gelu_approx", "gelu_pytorch_tanh")


def get_activation(name: str):
    """Element-wise activation by its configuration name (reference: ``get_activation``,
    mist/modules/utils.py:39-53).  The tanh form of GELU is the one fused into the GEMM epilogues;
    the others run as separate element-wise operations."""
    import torch.nn.functional as TF
    name = (name or "gelu_new").lower()
    if name in _TANH_GELU:
        return lambda x: TF.gelu(x, approximate="tanh")
    if name in ("gelu", "geglu"):
        return TF.gelu
    if name == "relu":
        return TF.relu
    if name in ("sigmoid", "glu"):
        return torch.sigmoid
    if name == "sqrelu":
        return lambda x: TF.relu(x).square()
    if name in ("silu", "swiglu"):
        return TF.silu
    raise ValueError(f"activation '{name}' is not known")


class ParallelMLP(nn.Module):
    """fc1 (column parallel, tanh-GELU fused into the GEMM epilogue) -> fc2 (row parallel); other
    activations run between the two GEMMs as an element-wise operation."""

    def __init__(self, hidden_size, intermediate_size, process_group=None, bias1=True, bias2=True,
                 activation="gelu_new", sequence_parallel=False, device=None, dtype=None):
        super().__init__()
        fk = dict(process_group=process_group, sequence_parallel=sequence_parallel, device=device, dtype=dtype)
        self.activation = (activation or "gelu_new").lower()
        self.fused_gelu = self.activation in _TANH_GELU
        self.act = None if self.fused_gelu else get_activation(self.activation)
        self.fc1 = ColumnParallelLinear(hidden_size, intermediate_size, bias=bias1,
                                        activation="gelu" if self.fused_gelu else None, **fk)
        self.fc2 = RowParallelLinear(intermediate_size, hidden_size, bias=bias2, **fk)

    def forward(self, x, residual=None):
        fc1, fc2 = self.fc1, self.fc2
        if not self.fused_gelu:
            return fc2(self.act(fc1(x)), residual=residual)
        if (residual is None and isinstance(x, torch.Tensor) and F.mlp_gelu_fused_available(x)
                and not fc1._fused(x) and x.dtype == fc1.weight.dtype):
            # local compute as one autograd node (GELU's derivative rides on a GEMM epilogue in the
            # backward pass); the tensor-parallel collectives stay around it
            pg, ws = fc1.process_group, group_size(fc1.process_group)
            if fc1.sequence_parallel:
                x = dist_ops.all_gather(x.reshape(-1, x.shape[-1]), pg)
            else:
                x = dist_ops.copy_to_group(x, pg)
            y = F.mlp_gelu(x, fc1.weight, fc1.bias, fc2.weight, fc2.bias)
            if ws > 1:
                if fc2.sequence_parallel:
                    y = dist_ops.reduce_scatter(y.reshape(-1, y.shape[-1]), pg)
                else:
                    y = dist_ops.all_reduce(y, pg)
            return y
        return self.fc2(self.fc1(x), residual=residual)


class ParallelGatedMlp(nn.Module):
    """fc1 produces ``[gate | up]`` (each rank holds matching halves), SwiGLU, then fc2."""

    def __init__(self, hidden_size, intermediate_size, process_group=None, bias1=False, bias2=False,
                 activation="swiglu", sequence_parallel=False, device=None, dtype=None):
        super().__init__()
        fk = dict(process_group=process_group, sequence_parallel=sequence_parallel, device=device, dtype=dtype)
        self.activation = (activation or "swiglu").lower()
        # silu gates use the fused SwiGLU kernel; "geglu" / "glu" ... gate with their own activation
        self.gate_act = None if self.activation in ("silu", "swiglu") else get_activation(self.activation)
        self.fc1 = ColumnParallelLinear(hidden_size, 2 * intermediate_size, bias=bias1, multiple_of=2, **fk)
        self.fc2 = RowParallelLinear(intermediate_size, hidden_size, bias=bias2, **fk)

    def forward(self, x, residual=None):
        y = self.fc1(x)
        if self.gate_act is None:
            return self.fc2(F.swiglu(y), residual=residual)
        gate, up = y.chunk(2, dim=-1)
        return self.fc2(self.gate_act(gate) * up, residual=residual)


# -------------------------------------------------------------------------------- loss
def vocab_parallel_cross_entropy(logits, labels, process_group=None, ignore_index=-100, label_smoothing: float = 0.0):
    """Per-token loss of ``[tokens, vocab/tp]`` logits against global labels.

    ``label_smoothing`` = a moves the mass a from the label to the other K - 1 classes, evenly:
    ``loss = (1 - s) * nll - s * mean_j log p_j`` with ``s = a * K / (K - 1)`` (reference:
    mist/modules/losses.py:117-134).  The smoothing term is built from two row sums that are reduced
    over the tensor-parallel group; it is not on the path the benchmarks use."""
    ws = group_size(process_group)
    rk = group_rank(process_group)
    group = None if (ws == 1 or isinstance(process_group, dist_ops.FakeGroup)) else process_group
    loss = F.cross_entropy(logits, labels, vocab_start=rk * logits.shape[-1], group=group,
                           ignore_index=ignore_index)
    if label_smoothing <= 0.0 or not isinstance(logits, torch.Tensor):
        return loss
    assert label_smoothing < 1.0
    K = logits.shape[-1] * ws
    s = label_smoothing * K / (K - 1)
    lf = logits.float()
    lmax = lf.detach().max(-1).values
    if group is not None:
        torch.distributed.all_reduce(lmax, op=torch.distributed.ReduceOp.MAX, group=group)
    sum_logits = dist_ops.all_reduce(lf.sum(-1), group)
    sum_exp = dist_ops.all_reduce((lf - lmax[:, None]).exp().sum(-1), group)
    mean_log_prob = sum_logits / K - (lmax + sum_exp.log())
    smooth = (1.0 - s) * loss - s * mean_log_prob
    return torch.where(labels.reshape(-1) == ignore_index, torch.zeros_like(smooth), smooth)
