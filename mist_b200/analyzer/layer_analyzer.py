"""From a symbolic trace to per-layer memory / work summaries.

The model is traced once per tensor-parallel degree with a symbolic micro batch ``b``
(one transformer block is enough: blocks are identical).  The trace is cut into three
layers -- *pre* (embedding), *block* (one transformer block) and *post* (final norm, head,
loss) -- and each is summarised by a :class:`LayerInfo`:

* memory, as sympy expressions in ``b``: peak transient bytes of the forward pass, bytes
  saved for the backward pass (with and without activation checkpointing), output bytes,
  peak bytes of the backward pass, and the weight / gradient / optimizer-state bytes;
* work: the operator list with symbolic shape signatures (latency comes from the
  operator database) and the tensor-parallel collectives of both passes.

The memory numbers come from a liveness simulation over the recorded nodes: a tensor dies
after its last consumer unless a node declared it saved for backward; in the backward
simulation saved tensors die after the last node that needs them.

Parity: reference mist/analyzer/layer_analyzer.py:253-646 (LayerAnalyzer), :691-750
(analyze_blocks), mist/analyzer/info.py:179-222 (state sizes; Adam mixed precision keeps
fp32 master + two moments = 6x the 16-bit weight bytes), mist/memory_pool.py:20-226, and
mist/benchmark/common.py:35-217 (trace one hidden layer with symbolic b, cache the result).
"""
from __future__ import annotations

import os
import pickle
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import sympy as sp
import torch

from ..config import MistConfig, ModelConfig
from ..models.provider import base_model_provider, family_of
from ..parallel.dist_ops import FakeGroup
from ..symbols import SymbolManager
from .symtensor import Comm, Graph, Node, SymTensor, set_scope, tracing

OPT_STATE_MULTIPLIER = 6     # bytes of fp32 master + exp_avg + exp_avg_sq per byte of 16-bit weight


@dataclass
class PhaseInfo:
    peak: Any = 0            # peak transient bytes (beyond the layer input and what is saved)
    saved: Any = 0           # bytes kept for the backward pass (forward) / released (backward)
    output: Any = 0
    flops: Any = 0
    bytes: Any = 0
    comms: List[Comm] = field(default_factory=list)


@dataclass
class LayerInfo:
    name: str
    fwd: PhaseInfo
    bwd: PhaseInfo
    input_bytes: Any
    weight_bytes: int
    grad_bytes: int
    opt_bytes: int
    nodes: List[Node]
    num_params: int

    def saved_bytes(self, checkpointed: bool):
        """Activation bytes alive between this layer's forward and backward."""
        return self.input_bytes if checkpointed else self.fwd.saved


class _TraceHooks:
    """Scope markers driven by the transformer stack's per-block callbacks."""

    def before_layer(self, stack, i, hidden, residual):
        # the blocks of a decoder stack (the second stack of an encoder-decoder model) get their own scopes
        set_scope(f"{'dblock' if getattr(stack.layers[0], 'is_decoder', False) else 'block'}{i}")
        return hidden, residual

    def after_layer(self, stack, i, hidden, residual):
        if i + 1 == len(stack.layers):
            set_scope("post")
        return hidden, residual


def _simulate(nodes: List[Node], graph: Graph, layer_inputs: set, used_later: set) -> (PhaseInfo, PhaseInfo, Any):
    """Liveness simulation of one layer.  Returns (fwd, bwd, input_bytes).  ``used_later``
    holds the tensors that nodes of later layers read."""
    produced = {o.tid: o for n in nodes for o in n.outputs}
    last_use: Dict[int, int] = {}
    for idx, n in enumerate(nodes):
        for t in n.inputs:
            last_use[t] = idx
    saved_by: Dict[int, List[int]] = {}
    for idx, n in enumerate(nodes):
        for t in n.saved:
            saved_by.setdefault(t, []).append(idx)
    consumed = set(t for n in nodes for t in n.inputs)
    # tensors handed on: read by a later layer, or (for the last layer) the final result
    exported = {t for t in produced if t in used_later}
    if not used_later and nodes:
        exported = set(o.tid for o in nodes[-1].outputs)

    def nbytes(t):
        return graph.tensors[t].nbytes

    # ------------------------------------------------------------------------ forward
    live: Dict[int, Any] = {}
    saved_total = 0
    saved_seen = set()
    peak_candidates = [sp.Integer(0)]
    extra_saved = 0
    for idx, n in enumerate(nodes):
        for o in n.outputs:
            live[o.tid] = o.nbytes
        cur = sum(live.values(), sp.Integer(0)) + n.fwd_workspace + saved_total + extra_saved
        peak_candidates.append(cur)
        extra_saved = extra_saved + n.saved_extra
        for t in n.saved:
            if t in saved_seen or graph.tensors[t].is_param:
                continue
            saved_seen.add(t)
            if t in live:                       # moves from transient to saved
                saved_total = saved_total + live.pop(t)
            elif t in layer_inputs:
                saved_total = saved_total + nbytes(t)
        for t in list(live):
            if last_use.get(t, -1) <= idx and t not in exported and t not in saved_seen:
                if last_use.get(t, -1) == idx or t not in consumed:
                    del live[t]
    out_bytes = sum((nbytes(t) for t in exported if t in produced), sp.Integer(0))
    fwd_saved = saved_total + extra_saved
    fwd_peak = sp.Max(*peak_candidates) if len(peak_candidates) > 1 else peak_candidates[0]
    input_bytes = sum((nbytes(t) for t in layer_inputs if not graph.tensors[t].is_param), sp.Integer(0))
    fwd = PhaseInfo(peak=fwd_peak, saved=fwd_saved, output=out_bytes,
                    flops=sum((n.flops_fwd for n in nodes), sp.Integer(0)),
                    bytes=sum((n.bytes_fwd for n in nodes), sp.Integer(0)),
                    comms=[n.comm_fwd for n in nodes if n.comm_fwd is not None])

    # ----------------------------------------------------------------------- backward
    # starts with everything saved alive plus the gradient of the layer output
    alive_saved = {t: nbytes(t) for t in saved_seen}
    grad_live = out_bytes
    bwd_candidates = [sp.Integer(0)]
    remaining_extra = extra_saved
    for idx in range(len(nodes) - 1, -1, -1):
        n = nodes[idx]
        cur = sum(alive_saved.values(), sp.Integer(0)) + remaining_extra + grad_live + n.grad_bytes + n.bwd_workspace
        bwd_candidates.append(cur)
        # after this node's backward: its output grads die, its input grads live on
        out_b = sum((o.nbytes for o in n.outputs), sp.Integer(0))
        grad_live = sp.Max(grad_live - out_b, 0) + n.grad_bytes if n.grad_bytes != 0 else grad_live
        remaining_extra = remaining_extra - n.saved_extra
        for t in n.saved:
            users = saved_by.get(t, [])
            if users and min(users) == idx and t in alive_saved:
                del alive_saved[t]
    bwd_peak = sp.Max(*bwd_candidates) if len(bwd_candidates) > 1 else bwd_candidates[0]
    bwd = PhaseInfo(peak=bwd_peak, saved=fwd_saved, output=input_bytes,
                    flops=sum((n.flops_bwd for n in nodes), sp.Integer(0)),
                    bytes=sum((n.bytes_bwd for n in nodes), sp.Integer(0)),
                    comms=[n.comm_bwd for n in nodes if n.comm_bwd is not None])
    return fwd, bwd, input_bytes


def _layer_info(name: str, nodes: List[Node], graph: Graph, later_nodes: List[Node]) -> LayerInfo:
    produced = {o.tid for n in nodes for o in n.outputs}
    used_later = {t for n in later_nodes for t in n.inputs}
    layer_inputs = {t for n in nodes for t in n.inputs if t not in produced}
    param_ids = {t for t in layer_inputs if graph.tensors[t].is_param}
    act_inputs = {t for t in layer_inputs if t not in param_ids and graph.tensors[t].requires_grad}
    fwd, bwd, input_bytes = _simulate(nodes, graph, act_inputs, used_later)
    wbytes = int(sum(int(graph.tensors[t].nbytes) for t in param_ids))
    nparams = wbytes // 2
    return LayerInfo(name, fwd, bwd, input_bytes, wbytes, wbytes, OPT_STATE_MULTIPLIER * wbytes, nodes, nparams)


@dataclass
class ModelAnalysis:
    """Result of tracing one (model, tp, flags) combination."""
    pre: LayerInfo
    block: LayerInfo
    post: LayerInfo
    tp: int
    seq_len: int
    symbol_names: List[str]
    sequence_parallel: bool
    graph_nodes: int
    enc_block: Optional[LayerInfo] = None      # encoder-decoder models only
    dec_block: Optional[LayerInfo] = None

    def layer(self, which: str) -> LayerInfo:
        table = {"pre_layer": self.pre, "block_layer": self.block, "post_layer": self.post,
                 "enc_block_layer": getattr(self, "enc_block", None) or self.block,
                 "dec_block_layer": getattr(self, "dec_block", None) or self.block}
        return table[which]


def trace_and_analyze(model_cfg: ModelConfig, seq_len: int, tp: int = 1, sequence_parallel: bool = False,
                      manager: Optional[SymbolManager] = None) -> ModelAnalysis:
    """Traces a one-block copy of the model with symbolic micro batch ``b``."""
    mgr = manager or SymbolManager()
    b = mgr.symbols("b", 2)
    import copy
    cfg = copy.copy(model_cfg)
    group = FakeGroup(tp, 0) if tp > 1 else None
    dtype = cfg.params_dtype
    full_layers = cfg.num_hidden_layers
    cfg.num_hidden_layers = 2      # the second block sees (hidden, residual) like every middle block
    try:
        model = base_model_provider(cfg, process_groups=group, pre_post_process_group=group,
                                    sequence_parallel=sequence_parallel and tp > 1, device="meta", dtype=dtype)
    finally:
        cfg.num_hidden_layers = full_layers
    lm = model.language_model
    hooks = _TraceHooks()
    for stack in (lm.encoder, lm.decoder):
        if stack is not None:
            stack.hooks = hooks
    fam = family_of(cfg.name)
    with tracing() as graph:
        ids = SymTensor((b, seq_len), torch.int64, label="input_ids")
        labels = SymTensor((b, seq_len), torch.int64, label="labels")
        if fam == "t5":
            model(encoder_input_ids=ids, decoder_input_ids=SymTensor((b, seq_len), torch.int64), lm_labels=labels)
        elif fam == "bert":
            model(input_ids=ids, tokentype_ids=SymTensor((b, seq_len), torch.int64), lm_labels=labels)
        else:
            model(input_ids=ids, labels=labels)
    scopes = graph.scopes()
    block_scopes = [s for s in scopes if s.startswith("block")]
    dec_scopes = [s for s in scopes if s.startswith("dblock")]
    pre_nodes = graph.nodes_of("pre")
    post_nodes = graph.nodes_of("post")
    first_block_nodes = graph.nodes_of(block_scopes[0]) if block_scopes else []
    pre = _layer_info("pre_layer", pre_nodes, graph, first_block_nodes)
    post = _layer_info("post_layer", post_nodes, graph, [])
    enc_block = dec_block = None
    if dec_scopes:
        # Encoder-decoder models: one "layer" of a single-stage strategy is an encoder block plus a decoder
        # block (both stacks have the same depth); pipeline strategies put encoder blocks on the first stages
        # and the decoder on the last, so the two kinds are also kept apart.
        enc_nodes, dec_nodes = graph.nodes_of(block_scopes[-1]), graph.nodes_of(dec_scopes[-1])
        enc_block = _layer_info("enc_block_layer", enc_nodes, graph, post_nodes + graph.nodes_of(dec_scopes[0]))
        dec_block = _layer_info("dec_block_layer", dec_nodes, graph, post_nodes)
        block = _layer_info("block_layer", enc_nodes + dec_nodes, graph, post_nodes)
    else:
        block_nodes = graph.nodes_of(block_scopes[-1]) if block_scopes else []
        block = _layer_info("block_layer", block_nodes, graph, post_nodes)
    return ModelAnalysis(pre, block, post, tp, seq_len, ["b"], sequence_parallel and tp > 1, len(graph.nodes),
                         enc_block, dec_block)


# ------------------------------------------------------------------------------- caching
def analysis_cache_name(model_cfg: ModelConfig, seq_len: int, tp: int, sequence_parallel: bool) -> str:
    """Same naming scheme as the reference's analysis cache, extended by the fields that
    change the trace here (tp is traced concretely)."""
    return (f"model_{model_cfg.name}_ori_layers_{model_cfg.num_hidden_layers}_analyzed_layers_1"
            f"_f_{int(model_cfg.use_flash_attn)}_s_{seq_len}_v_{model_cfg.vocab_size}_tp_{tp}"
            f"_sp_{int(sequence_parallel)}.pkl")


def get_analysis(cfg: MistConfig, tp: int, cache_dir: Optional[str] = None, sequence_parallel: Optional[bool] = None
                 ) -> ModelAnalysis:
    sp_flag = bool(cfg.get("sequence_parallel", False)) if sequence_parallel is None else sequence_parallel
    seq = cfg.training.max_sequence_length
    if cache_dir:
        os.makedirs(cache_dir, exist_ok=True)
        path = os.path.join(cache_dir, analysis_cache_name(cfg.model, seq, tp, sp_flag))
        if os.path.exists(path):
            try:
                with open(path, "rb") as f:
                    return pickle.load(f)
            except Exception:
                pass
    res = trace_and_analyze(cfg.model, seq, tp, sp_flag)
    if cache_dir:
        with open(path, "wb") as f:
            pickle.dump(res, f)
    return res
