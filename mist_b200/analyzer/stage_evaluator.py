"""Batched cost model of one pipeline stage.

For a device mesh, a gradient-accumulation count and a stage shape (number of blocks,
number of checkpointed blocks, with/without embedding and head) this evaluates *every*
candidate strategy vector ``[b, dp, tp, wre, gre, ore, wo, go, oo, ao]`` at once with
numpy broadcasting and returns, per candidate,

* ``stable``: seconds per micro batch (forward + backward of all layers of the stage),
* ``delta`` : seconds paid once per iteration (gradient synchronisation that only happens
  at the last micro batch, optimizer step, weight refresh, optimizer-state swaps),
* peak memory of the forward and of the backward pass, and a feasibility flag.

Per layer and pass four channels run concurrently -- compute, GPU<->GPU collectives
(ZeRO all-gather / reduce-scatter), host->GPU and GPU->host copies (offloading) -- and
their combined time comes from the interference model; tensor-parallel collectives sit
on the critical path and are added on top.  Execution latencies come from the operator
database, memory terms from the symbolic layer analysis evaluated at ``b``.

Parity: reference mist/analyzer/batched_module_analyzer.py:417-536 (search space),
:687-3144 (batched_stage_analyze: memory :100-256, latencies :259-414, channel overlap
:1362-1902, stable / delta split :1910-2028, state memory with ring buffers :2091-2162,
peak memory :2755-3062, feasibility :2805-2812).  The schedule costed here is the one
:mod:`mist_b200.parallel.engine` executes (optimizer step overlapped with the backward pass
of the last micro batch rather than deferred into the next forward).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass
from typing import Dict, Optional, Sequence, Tuple

import numpy as np
import sympy as sp

from ..config import MistConfig
from ..node_database.database import OpDatabase
from ..node_database.node_spec import NodeSpec
from ..tools import comm_model
from .layer_analyzer import LayerInfo, ModelAnalysis, get_analysis

BATCH_SIZE_CANDIDATES = (1, 2, 4, 8)
OFFLOAD_RATIOS = (0.0, 0.25, 0.375, 0.5, 0.625, 0.75, 0.875, 1.0)
SPARSE_OFFLOAD_RATIOS = (0.0, 0.25, 0.375, 0.5, 0.75, 1.0)
GB = float(1 << 30)
#: allocator fragmentation allowance on top of the modelled peak
MEMORY_FACTOR = 1.06
ADAM_BYTES_PER_PARAM = 28.0     # fp32 master/m/v read+write (24) + bf16 grad read (2) + bf16 weight write (2)


# ------------------------------------------------------------------------------ search space
def create_search_space(num_nodes: int, gpus_per_node: int, global_batch: int, grad_accum: int, cfg: MistConfig,
                        tp_size: Optional[int] = None, batch_candidates: Sequence[int] = BATCH_SIZE_CANDIDATES
                        ) -> np.ndarray:
    """All strategy vectors for one stage on ``num_nodes x gpus_per_node`` devices: [N, 10]."""
    n_gpus = num_nodes * gpus_per_node
    per_micro = global_batch // grad_accum
    tun = cfg.tuning
    par = []
    for b in batch_candidates:
        if b > per_micro or per_micro % b:
            continue
        dp = per_micro // b
        if dp > n_gpus or n_gpus % dp:
            continue
        tp = n_gpus // dp
        if tp_size is not None and tp != tp_size:
            continue
        if tp > gpus_per_node or (cfg.get("disable_tp_tuning", False) and tp > 1 and tp_size is None):
            continue
        if cfg.model.num_attention_heads % tp or cfg.model.vocab_size % tp:
            continue
        if dp == 1 or not (tun and tun.zero_2_and_3_enabled):
            flags = [(0, 0, 1)]
        else:
            flags = [(0, 0, 1), (0, 1, 1), (1, 1, 1)]
        for f in flags:
            par.append((b, dp, tp) + f)
    if not par:
        return np.zeros((0, 10))
    state_on = bool(tun and tun.state_offloading_enabled)
    act_on = bool(tun and tun.activation_offloading_enabled)

    def fixed(name, default):
        v = cfg.get(name, None)
        return [float(v)] if v is not None else default

    wo = fixed("fixed_wo_ratio", list(SPARSE_OFFLOAD_RATIOS) if state_on and not cfg.get("disable_wo_tuning", False) else [0.0])
    go = fixed("fixed_go_ratio", list(SPARSE_OFFLOAD_RATIOS) if state_on and not cfg.get("disable_go_tuning", False) else [0.0])
    oo = fixed("fixed_oo_ratio", list(OFFLOAD_RATIOS) if state_on and not cfg.get("disable_oo_tuning", False) else [0.0])
    ao = fixed("fixed_ao_ratio", list(OFFLOAD_RATIOS) if act_on else [0.0])
    off = [o for o in itertools.product(wo, go, oo, ao) if not (o[0] > 0 and o[1] == 0)]
    space = np.array([p + o for p in par for o in off], dtype=np.float64)
    return space


# ------------------------------------------------------------------ per-(tp, b) layer numbers
@dataclass
class LayerNumbers:
    exec_fwd: float
    exec_bwd: float
    tp_fwd: float            # tensor-parallel collectives on the critical path, seconds
    tp_bwd: float
    fwd_peak: float          # bytes
    bwd_peak: float
    saved: float
    input_bytes: float
    output_bytes: float
    weight_bytes: float
    params: float
    first_gemm_fwd: float = 0.0      # forward seconds of the block's first GEMM (the one a fused weight gather rides on)
    # seconds the host needs to issue the layer's passes (Python, autograd, launches); a pass takes at least that
    host_fwd: float = 0.0
    host_bwd: float = 0.0
    host_recompute: float = 0.0


def fused_time(compute, comm, kappa: float, tau: float):
    """Seconds of a kernel that overlaps a GEMM with its collective tile by tile: the longer of the two,
    plus the share ``kappa`` of the shorter one that is not hidden, plus a fixed cost ``tau`` (flag rounds,
    the pass that sums the partial products).  ``kappa`` and ``tau`` are fitted to timings of the fused
    kernels on real peers (``fused_overlap`` in the operator database's ``_meta.json``)."""
    return np.maximum(compute, comm) + kappa * np.minimum(compute, comm) + tau


class StageEvaluator:
    def __init__(self, cfg: MistConfig, db: Optional[OpDatabase] = None, cache_dir: Optional[str] = None):
        self.cfg = cfg
        self.db = db or OpDatabase()
        self.cache_dir = cache_dir
        self.hw = cfg.hardware
        self._analysis: Dict[int, ModelAnalysis] = {}
        self._numbers: Dict[Tuple[int, int, str], LayerNumbers] = {}
        self._b = sp.Symbol("b", integer=True, positive=True)
        # Which collectives run on the fused kernels ("auto" = wherever the executor would use them: groups
        # inside one node).  The analyzer then prices a sequence-parallel linear together with the
        # collective next to it (reference: the collectives attached to an operator are priced inside
        # its spec, mist/node_database/node_spec.py:249-320).
        one_node_tp = True      # tensor-parallel groups never leave a node (the search space enforces it)
        tpb = str(cfg.get("tp_backend", "auto"))
        self.tp_fused = (tpb == "fused") or (tpb == "auto" and one_node_tp and bool(cfg.get("sequence_parallel", False))
                                             and str(self.hw.gpu_type or "").upper().find("B200") >= 0)
        z3 = str(cfg.get("zero3_gather", "auto"))
        self.zero3_fused = (z3 == "fused") or (z3 == "auto" and self.hw.num_nodes == 1
                                               and str(self.hw.gpu_type or "").upper().find("B200") >= 0)
        self.fused_overlap = dict(getattr(self.db, "fused_overlap", {}) or {})

    # ------------------------------------------------------------------------- analysis
    def analysis(self, tp: int) -> ModelAnalysis:
        if tp not in self._analysis:
            self._analysis[tp] = get_analysis(self.cfg, tp, self.cache_dir)
        return self._analysis[tp]

    def _val(self, expr, b: int) -> float:
        if isinstance(expr, sp.Basic):
            return float(expr.subs(self._b, b))
        return float(expr)

    def layer_numbers(self, tp: int, b: int, which: str) -> LayerNumbers:
        key = (tp, b, which)
        if key in self._numbers:
            return self._numbers[key]
        info: LayerInfo = self.analysis(tp).layer(which)
        ef = eb = 0.0
        tpf = tpb = 0.0
        first_gemm = 0.0

        def comm_t(comm) -> float:
            return float(comm_model.gpu_gpu_latency(comm.kind, np.array([self._val(comm.nbytes, b) / 1e9]), tp, 1,
                                                    self.hw.gpu_gpu_comm_params)[0])

        nodes = list(info.nodes)
        lat = {}
        for k, n in enumerate(nodes):
            if n.comm_fwd is None and n.comm_bwd is None:
                spec = NodeSpec.from_dict(n.spec, {"b": b})
                lat[k] = self.db.latency(spec, self._val(n.flops_fwd, b), self._val(n.flops_bwd, b),
                                         self._val(n.bytes_fwd, b), self._val(n.bytes_bwd, b))
                if n.spec.get("op") == "linear" and first_gemm == 0.0:
                    first_gemm = lat[k][0]
        fused_with = {}
        if self.tp_fused and tp > 1:
            # all-gather directly before a linear, reduce-scatter directly after one: one kernel each
            for k, n in enumerate(nodes):
                if n.comm_fwd is None or n.comm_fwd.kind not in ("all_gather", "reduce_scatter"):
                    continue
                j = k + 1 if n.comm_fwd.kind == "all_gather" else k - 1
                if 0 <= j < len(nodes) and j in lat and nodes[j].spec.get("op") == "linear" and j not in fused_with.values():
                    fused_with[k] = j
        ag = self.fused_overlap.get("ag_gemm", {"kappa": 1.0, "tau": 0.0})
        rs = self.fused_overlap.get("gemm_rs", {"kappa": 1.0, "tau": 0.0})
        done = set()
        for k, j in fused_with.items():
            n = nodes[k]
            f, w = lat[j]
            fo = ag if n.comm_fwd.kind == "all_gather" else rs          # forward kernel of this pair
            bo = rs if n.comm_fwd.kind == "all_gather" else ag          # backward: the roles swap
            ef += float(fused_time(f, comm_t(n.comm_fwd), fo["kappa"], fo["tau"]))
            # backward: the input-gradient GEMM (half of the linear's backward) carries the collective,
            # the weight-gradient GEMM runs beside it
            eb += 0.5 * w + float(fused_time(0.5 * w, comm_t(n.comm_bwd) if n.comm_bwd is not None else 0.0,
                                             bo["kappa"], bo["tau"]))
            done.update((k, j))
        for k, n in enumerate(nodes):
            if k in done:
                continue
            if k in lat:
                ef += lat[k][0]
                eb += lat[k][1]
            for comm, fwd in ((n.comm_fwd, True), (n.comm_bwd, False)):
                if comm is None:
                    continue
                if fwd:
                    tpf += comm_t(comm)
                else:
                    tpb += comm_t(comm)
        # The host issues a layer no faster than it can dispatch its operators.  Measured on a model with
        # negligible kernels (tools/profile_host_dispatch.py): seconds per block for forward + backward (a third
        # of it is charged to the forward pass) and for a recomputed forward pass under activation
        # checkpointing (which costs the host more than a plain one: saved-tensor hooks, RNG state), scaled by
        # the number of traced operators of this layer.
        hd = getattr(self.db, "host_dispatch", None) or {}
        host = (0.0, 0.0, 0.0)
        if hd.get("ops_per_block"):
            k_ops = len(nodes) / float(hd["ops_per_block"])
            both = float(hd.get("block_fwd_bwd_s", 0.0)) * k_ops
            host = (both / 3.0, both * 2.0 / 3.0, float(hd.get("block_recompute_s", 0.0)) * k_ops)
        num = LayerNumbers(ef, eb, tpf, tpb, self._val(info.fwd.peak, b), self._val(info.bwd.peak, b),
                           self._val(info.fwd.saved, b), self._val(info.input_bytes, b), self._val(info.fwd.output, b),
                           float(info.weight_bytes), float(info.num_params), first_gemm, *host)
        self._numbers[key] = num
        return num

    # --------------------------------------------------------------------------- helpers
    def _coll(self, kind: str, nbytes: np.ndarray, n: np.ndarray) -> np.ndarray:
        per_node = self.hw.num_gpus_per_node
        intra = np.minimum(n, per_node)
        inter = np.maximum(n // per_node, 1)
        return comm_model.gpu_gpu_latency(kind, nbytes / 1e9, intra, inter, self.hw.gpu_gpu_comm_params)

    def _h2d(self, nbytes):
        return comm_model.host_copy_latency(np.asarray(nbytes) / 1e9, self.hw.cpu_gpu_comm_params)

    def _d2h(self, nbytes):
        return comm_model.host_copy_latency(np.asarray(nbytes) / 1e9, self.hw.gpu_cpu_comm_params)

    def _interf(self, C, G2G, C2G, G2C):
        return comm_model.interference_estimate(C, G2G, C2G, G2C, self.hw.interference_model_params)

    # -------------------------------------------------------------------------- evaluate
    def evaluate(self, space: np.ndarray, num_layers: int, num_ckpt: int, grad_accum: int, has_pre: bool,
                 has_post: bool, inflight_extra: int = 0, pre_post_flags: Optional[Tuple[int, int, int]] = None,
                 block_kind: str = "block_layer", tied_copy: bool = False, has_prev_stage: bool = False,
                 has_next_stage: bool = False) -> Dict[str, np.ndarray]:
        """``space``: [N, 10].  ``inflight_extra``: additional micro batches whose activations are
        alive at the memory peak (1F1B warm-up depth of this stage).  ``pre_post_flags``: the
        (wre, gre, ore) flags of the strategy vector that the embedding / head units run under
        (``None``: ZeRO-1, what the tuner writes); the executor caps them at ZeRO-2, at ZeRO-1 when
        a table is tied across stages, and never offloads those units, and so does this model.
        ``has_prev_stage`` / ``has_next_stage``: the stage exchanges its boundary activation (and
        its gradient) with a neighbour, which the schedule waits for (reference: the stage-output
        p2p term of mist/analyzer/batched_module_analyzer.py:1299-1305, 2796, 2848).

        The stage is costed as the sequence of units the executor walks -- embedding, blocks
        (the checkpointed ones last), head -- with the executor's one-unit look-ahead: the
        collectives and copies issued for unit ``u +- 1`` run while unit ``u`` computes, the
        first gather of a pass and the last reduction of the iteration's last backward pass
        have nothing to hide behind (reference: first / middle / last layer and first / last
        micro batch priced apart, batched_module_analyzer.py:1432-1902)."""
        N = space.shape[0]
        b = space[:, 0].astype(int)
        dp = space[:, 1].astype(int)
        tp = space[:, 2].astype(int)
        wre, gre, ore = space[:, 3] > 0, space[:, 4] > 0, space[:, 5] > 0
        wo, go, oo, ao = space[:, 6], space[:, 7], space[:, 8], space[:, 9]
        L, c, G = int(num_layers), int(num_ckpt), int(grad_accum)
        zeros = np.zeros(N)
        # embedding / head units: flags as the executor applies them
        ppf = (0, 0, 1) if pre_post_flags is None else tuple(int(bool(v)) for v in pre_post_flags)
        pp_gre = np.full(N, bool(ppf[1]) and not tied_copy) & (dp > 1)
        pp_ore = np.full(N, bool(ppf[2]) or bool(ppf[1])) & (dp > 1)
        pp_wre = np.zeros(N, dtype=bool)

        def gather(which: str) -> Dict[str, np.ndarray]:
            fields = ("exec_fwd", "exec_bwd", "tp_fwd", "tp_bwd", "fwd_peak", "bwd_peak", "saved", "input_bytes",
                      "output_bytes", "weight_bytes", "params", "first_gemm_fwd", "host_fwd", "host_bwd", "host_recompute")
            out = {f: np.zeros(N) for f in fields}
            for (t, bb) in set(zip(tp.tolist(), b.tolist())):
                sel = (tp == t) & (b == bb)
                num = self.layer_numbers(t, bb, which)
                for f in fields:
                    out[f][sel] = getattr(num, f)
            return out

        def unit_terms(x: Dict[str, np.ndarray], ckpt: bool, block: bool) -> Dict[str, np.ndarray]:
            """Per-channel seconds of one unit: what its own passes compute, and what is issued on
            its behalf while a neighbour computes."""
            W = x["weight_bytes"]
            u_wre, u_gre, u_ore = (wre, gre, ore) if block else (pp_wre, pp_gre, pp_ore)
            u_wo, u_go, u_oo, u_ao = (wo, go, oo, ao) if block else (zeros, zeros, zeros, zeros)
            w_shard = np.where(u_wre, W / dp, W)
            g_shard = np.where(u_gre, W / dp, W)
            kept = x["input_bytes"] if ckpt else x["saved"]
            shard_params = np.where(u_ore, x["params"] / dp, x["params"])
            opt_bytes = 12.0 * shard_params * u_oo
            cf = np.maximum(x["exec_fwd"] + x["tp_fwd"], x["host_fwd"])
            ag_all = np.where(u_wre, self._coll("all_gather", W, dp), 0.0)
            ag_fwd = ag_all
            if block and self.zero3_fused and not (self.tp_fused and np.any(tp > 1)):
                # forward pass: the gather rides on the block's first GEMM instead of running one block ahead
                zo = self.fused_overlap.get("zero3_gather", {"kappa": 1.0, "tau": 0.0})
                g1 = x["first_gemm_fwd"]
                fused = fused_time(g1, ag_all, zo["kappa"], zo["tau"])
                plain = u_wre & (u_wo == 0) & (g1 > 0)
                cf = np.where(plain, cf - g1 + fused, cf)
                ag_fwd = np.where(plain, 0.0, ag_all)
            return dict(
                cf=cf, ag_fwd=ag_fwd,
                cb=np.maximum(x["exec_bwd"] + x["tp_bwd"], x["host_bwd"])
                + (np.maximum(x["exec_fwd"] + x["tp_fwd"], x["host_recompute"]) if ckpt else 0.0),
                ag=ag_all,
                rs=np.where(u_gre, self._coll("reduce_scatter", W, dp), 0.0),
                # only at the last micro batch: the reduction that waited for it, the refresh of the
                # other ranks' weights after the step, the optimizer kernel and the optimizer-state copies
                sync=np.where(u_gre, 0.0, np.where(u_ore, self._coll("reduce_scatter", W, dp),
                                                   self._coll("all_reduce", W, dp))),
                refresh=np.where(u_ore & ~u_wre, self._coll("all_gather", W, dp), 0.0),
                adam=shard_params * ADAM_BYTES_PER_PARAM / (self.db.model.hbm_gbs * 1e9),
                h2d_w=self._h2d(u_wo * w_shard),
                h2d_a=self._h2d(u_ao * kept),
                d2h_a=self._d2h(u_ao * kept),
                h2d_g=self._h2d(u_go * g_shard) if G > 1 else zeros,
                d2h_g=self._d2h(u_go * g_shard),
                h2d_o=self._h2d(opt_bytes), d2h_o=self._d2h(opt_bytes))

        blk = gather(block_kind)      # "enc_block_layer" / "dec_block_layer" for the stages of an encoder-decoder pipeline
        kinds = {"b0": unit_terms(blk, False, True), "b1": unit_terms(blk, True, True)}
        pre = post = None
        if has_pre:
            pre = gather("pre_layer")
            kinds["pre"] = unit_terms(pre, False, False)
        if has_post:
            post = gather("post_layer")
            kinds["post"] = unit_terms(post, False, False)
        seq = (["pre"] if has_pre else []) + ["b0"] * (L - c) + ["b1"] * c + (["post"] if has_post else [])
        none = {k: zeros for k in kinds["b0"]}

        memo: Dict[Tuple, np.ndarray] = {}

        def fwd_unit(u: str, nxt: Optional[str]) -> np.ndarray:
            key = ("f", u, nxt)
            if key not in memo:
                me, nx = kinds[u], (kinds[nxt] if nxt else none)
                memo[key] = self._interf(me["cf"], nx["ag_fwd"], nx["h2d_w"], me["d2h_a"])
            return memo[key]

        def bwd_unit(u: str, nxt: Optional[str], prv: Optional[str], last: bool) -> np.ndarray:
            """Backward pass of ``u`` while the unit that follows it in the model (``nxt``, whose backward
            pass has just ended) reduces its gradients and the one before it (``prv``) is fetched."""
            key = ("b", u, nxt, prv, last)
            if key not in memo:
                me, nx, pv = kinds[u], (kinds[nxt] if nxt else none), (kinds[prv] if prv else none)
                g2g = pv["ag"] + nx["rs"]
                c2g = pv["h2d_w"] + pv["h2d_a"] + me["h2d_g"]
                g2c = nx["d2h_g"]
                comp = me["cb"]
                if last:
                    g2g = g2g + nx["sync"] + nx["refresh"]
                    comp = comp + nx["adam"]
                    c2g = c2g + nx["h2d_o"]
                    g2c = g2c + nx["d2h_o"]
                memo[key] = self._interf(comp, g2g, c2g, g2c)
            return memo[key]

        n = len(seq)
        fwd = sum((fwd_unit(seq[i], seq[i + 1] if i + 1 < n else None) for i in range(n)), zeros)
        first_block = next((k for k in seq if k in ("b0", "b1")), None)
        if first_block is not None:
            fwd = fwd + kinds[first_block]["ag_fwd"] + kinds[first_block]["h2d_w"]     # nothing computes while it arrives
        bwd = sum((bwd_unit(seq[i], seq[i + 1] if i + 1 < n else None, seq[i - 1] if i > 0 else None, False)
                   for i in range(n)), zeros)
        bwd_last = sum((bwd_unit(seq[i], seq[i + 1] if i + 1 < n else None, seq[i - 1] if i > 0 else None, True)
                        for i in range(n)), zeros)
        head = kinds[seq[0]]
        # after the last backward pass of the iteration the first unit's reduction, optimizer step and weight
        # refresh run with nothing left to overlap; the next iteration's first forward waits for them
        tail_last = (self._interf(head["adam"], head["rs"] + head["sync"] + head["refresh"], head["h2d_o"],
                                  head["d2h_o"] + head["d2h_g"]))
        # boundary activations: the schedule waits for each receive and each send of a micro batch
        p2p = zeros
        if has_prev_stage or has_next_stage:
            per = comm_model.gpu_gpu_latency("p2p", blk["input_bytes"] / 1e9, None,
                                             2 if self.hw.num_nodes > 1 else 1, self.hw.gpu_gpu_comm_params)
            p2p = 2.0 * per * (int(has_prev_stage) + int(has_next_stage))     # activation forward + gradient backward
        stable = fwd + bwd + p2p
        delta = (bwd_last - bwd) + tail_last

        # ---- memory of the stage
        W = blk["weight_bytes"]
        w_res = L * np.where(wre, W / dp, W) * (1 - wo)
        w_ring = np.where(wre | (wo > 0), 2 * W, 0.0)
        g_res = L * np.where(gre, W / dp, W) * (1 - go) * (2.0 if G > 1 else 1.0)   # fp32 accumulation when G > 1
        g_ring = np.where(gre | (go > 0), 2 * W, 0.0)
        o_res = L * 6.0 * np.where(ore, W / dp, W) * (1 - oo)
        o_stage = np.where(oo > 0, 2 * 6.0 * np.where(ore, W / dp, W), 0.0)
        states = w_res + w_ring + g_res + g_ring + o_res + o_stage
        inflight = 1 + int(inflight_extra)
        acts = inflight * ((L - c) * blk["saved"] * (1 - ao) + c * blk["input_bytes"] * (1 - ao))
        peak_f = states + acts + blk["fwd_peak"]
        bwd_tr = np.maximum(blk["bwd_peak"], (blk["fwd_peak"] + blk["bwd_peak"]) if c > 0 else 0.0)
        peak_b = states + acts + bwd_tr

        for x in (pre, post):
            if x is None:
                continue
            Wp = x["weight_bytes"]
            # full weights, gradient bucket (full: these units reduce in place), optimizer state
            st = Wp + Wp * (2.0 if (G > 1 and not ppf[1]) else 1.0) + 6.0 * np.where(pp_ore, Wp / dp, Wp)
            peak_f = peak_f + st + inflight * x["saved"]
            peak_b = peak_b + st + inflight * x["saved"]
            peak_f = np.maximum(peak_f, states + acts + st + x["fwd_peak"])
            peak_b = np.maximum(peak_b, states + acts + st + x["bwd_peak"])

        if tied_copy:
            # last stage of a pipeline whose model ties the output projection to the word table: the stage
            # holds its own copy (bf16 weights and full-size gradients, optimizer state sharded like the rest)
            Wt = 2.0 * self.cfg.model.vocab_size * self.cfg.model.hidden_size / tp
            extra = Wt + Wt + 6.0 * np.where(pp_ore, Wt / dp, Wt)
            peak_f = peak_f + extra
            peak_b = peak_b + extra
        cap = self.hw.memory_capacity * GB
        feasible = np.maximum(peak_f, peak_b) * MEMORY_FACTOR <= cap
        return {"stable": stable, "delta": delta, "peak_fwd": peak_f, "peak_bwd": peak_b, "feasible": feasible}


# ------------------------------------------------------------------------------- pipeline
def pipeline_latency(stable: Sequence[float], delta: Sequence[float], grad_accum: int) -> float:
    """Iteration time of a 1F1B pipeline: ``sum T + (G - 1) max T + max_s (D_s - sum_{i<s} T_i)``;
    a single stage costs ``T * G + D``."""
    T, D = list(stable), list(delta)
    if len(T) == 1:
        return T[0] * grad_accum + D[0]
    prefix, worst = 0.0, -float("inf")
    for t, d in zip(T, D):
        worst = max(worst, d - prefix)
        prefix += t
    return sum(T) + (grad_accum - 1) * max(T) + max(worst, 0.0)


def ties_across_stages(cfg: MistConfig) -> bool:
    """Whether a pipeline of this model keeps a second copy of the word table on its last stage (models whose
    output projection is the word table; encoder-decoder models count their copy as the decoder stage's
    embedding instead)."""
    from ..models.provider import family_of
    if cfg.model.add_decoder:
        return False
    return bool(cfg.model.tie_word_embeddings) or family_of(cfg.model.name) == "bert"


def analyze_strategy(cfg: MistConfig, evaluator: Optional[StageEvaluator] = None) -> Dict:
    """Predicted cost of the strategy written in ``cfg.strategy`` (the analyze entry point)."""
    ev = evaluator or StageEvaluator(cfg)
    st = cfg.strategy
    S, G = st.num_stages, st.gradient_accumulation_steps
    stables, deltas, peaks = [], [], []
    for s in range(S):
        vec = np.array([st.stage_strategies[s]], dtype=np.float64)
        warm = min(S - 1 - s, max(G - 1, 0))
        kind = "block_layer"
        if cfg.model.add_decoder and S > 1:
            kind = "dec_block_layer" if s == S - 1 else "enc_block_layer"
        # the decoder stage of an encoder-decoder pipeline holds its own copy of the embedding tables
        has_pre = s == 0 or kind == "dec_block_layer"
        ppa = st.pre_post_vector(s)
        res = ev.evaluate(vec, st.layer_partitions[s], st.gradient_checkpointing[s], G, has_pre=has_pre,
                          has_post=(s == S - 1), inflight_extra=warm, block_kind=kind,
                          tied_copy=(S > 1 and s == S - 1 and ties_across_stages(cfg)),
                          pre_post_flags=(tuple(ppa[3:6]) if ppa is not None else None),
                          has_prev_stage=(s > 0), has_next_stage=(s < S - 1))
        stables.append(float(res["stable"][0]))
        deltas.append(float(res["delta"][0]))
        peaks.append((float(res["peak_fwd"][0]), float(res["peak_bwd"][0])))
    if S > 1 and bool(getattr(cfg, "disable_non_uniform_pp_micro_batch_analysis", False)):
        # Uniform micro batches: each stage is charged its average time per micro batch (the
        # once-per-iteration part spread over the G micro batches) and no stage has a delta
        # (benchmark/mist/analysis/run.py:126-148).
        stables = [t + d / G for t, d in zip(stables, deltas)]
        deltas = [0.0] * S
    total = pipeline_latency(stables, deltas, G)
    return {"total": total, "stable": stables, "delta": deltas, "peak_memories": peaks}
