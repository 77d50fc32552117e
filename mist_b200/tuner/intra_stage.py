"""Intra-stage tuning: for every (gradient-accumulation count, device mesh, stage kind,
number of layers, number of checkpointed layers) evaluate all strategy vectors at once
and keep ``sample_size`` Pareto-sampled (stable, delta) points with their vectors.

Stage kinds: 0 first (has the embedding), 1 middle, 2 last (has the head), 3 only stage.
Parity: reference mist/analyzer/intra_tuning.py:84-282 (IntraStageTuner; cost tensors
indexed (g, mesh, kind, layers, ckpt, sample)), :285-370 (intra_stage_tune with a pickle
cache), mist/analyzer/batched_module_analyzer.py:581-685 (batched_tune_best_latency_for_stage).
"""
from __future__ import annotations

import hashlib
import os
import pickle
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..analyzer.stage_evaluator import ties_across_stages, StageEvaluator, create_search_space
from ..config import MistConfig
from .pareto import dedup_samples, sample_pareto_frontier

KINDS = {0: (True, False), 1: (False, False), 2: (False, True), 3: (True, True)}   # (has_pre, has_post)
EXACT_MIDDLE = 10      # kind EXACT_MIDDLE + s: the middle stage at pipeline position s (see tuner/inter_stage.py)


@dataclass
class StagePoint:
    stable: float
    delta: float
    peak_fwd: float
    peak_bwd: float
    vector: Tuple[float, ...]
    num_ckpt: int


@dataclass
class IntraStageResult:
    """points[(g, mesh, kind, layers)] -> list of StagePoint (all checkpoint counts merged,
    Pareto-sampled again so at most ``sample_size`` survive)."""
    points: Dict[Tuple[int, Tuple[int, int], int, int], List[StagePoint]] = field(default_factory=dict)
    evaluated: int = 0

    def get(self, g, mesh, kind, layers) -> List[StagePoint]:
        return self.points.get((g, tuple(mesh), kind, layers), [])


def ckpt_candidates(layers: int, cfg: MistConfig) -> List[int]:
    fixed = cfg.get("fixed_ckpt_value", None)
    if fixed is not None:
        return [min(int(fixed), layers)]
    if cfg.tuning is not None and not cfg.tuning.activation_checkpointing_tuning_enabled:
        return [0, layers]
    return list(range(0, layers + 1))


def tune_stage_cell(ev: StageEvaluator, cfg: MistConfig, g: int, mesh: Tuple[int, int], kind: int, layers: int,
                    num_stages: int, stage_index: int, tp: Optional[int] = None, block_kind: str = "block_layer",
                    has_pre: Optional[bool] = None) -> Tuple[List[StagePoint], int]:
    """Pareto points (stable time, delta) of one stage cell.  ``block_kind`` / ``has_pre``: for the stages of an
    encoder-decoder pipeline (encoder or decoder blocks; the decoder stage keeps its own embedding tables)."""
    gbs = cfg.training.global_batch_size
    space = create_search_space(mesh[0], mesh[1], gbs, g, cfg, tp_size=tp)
    if space.shape[0] == 0:
        return [], 0
    kind_pre, has_post = KINDS[1 if kind >= EXACT_MIDDLE else kind]
    has_pre = kind_pre if has_pre is None else bool(has_pre)
    warm = min(num_stages - 1 - stage_index, max(g - 1, 0))
    S = cfg.tuning.sample_size if cfg.tuning else 30
    all_points: List[StagePoint] = []
    evaluated = 0
    for c in ckpt_candidates(layers, cfg):
        # kinds: 0 first stage of a pipeline, 1 middle (EXACT_MIDDLE + s: the one at position s), 2 last,
        # 3 the only stage (no neighbours to exchange with)
        res = ev.evaluate(space, layers, c, g, has_pre, has_post, inflight_extra=warm, block_kind=block_kind,
                          tied_copy=(kind == 2 and ties_across_stages(cfg)),
                          has_prev_stage=kind not in (0, 3), has_next_stage=kind not in (2, 3))
        evaluated += space.shape[0]
        idx = dedup_samples(sample_pareto_frontier(res["stable"], res["delta"], res["feasible"], S))
        for i in idx:
            all_points.append(StagePoint(float(res["stable"][i]), float(res["delta"][i]), float(res["peak_fwd"][i]),
                                         float(res["peak_bwd"][i]), tuple(float(x) for x in space[i]), c))
    if not all_points:
        return [], evaluated
    st = np.array([p.stable for p in all_points])
    dl = np.array([p.delta for p in all_points])
    keep = dedup_samples(sample_pareto_frontier(st, dl, None, S))
    return [all_points[i] for i in keep], evaluated


def _cache_key(cfg: MistConfig, extra: str) -> str:
    m, t = cfg.model, cfg.training
    raw = (f"{m.name}|{m.hidden_size}|{m.num_hidden_layers}|{m.num_attention_heads}|{m.intermediate_size}|"
           f"{t.global_batch_size}|{t.max_sequence_length}|{cfg.hardware.gpu_gpu_comm_params}|"
           f"{cfg.hardware.memory_capacity}|{cfg.tuning.__dict__ if cfg.tuning else ''}|{extra}")
    return hashlib.sha1(raw.encode()).hexdigest()[:16]


def intra_stage_tune(cfg: MistConfig, ev: Optional[StageEvaluator] = None, grad_accums: Optional[Sequence[int]] = None,
                     meshes: Optional[Sequence[Tuple[int, int]]] = None, layer_counts: Optional[Dict] = None,
                     tp: Optional[int] = None, cache_dir: Optional[str] = None, num_stages_for_mesh=None
                     ) -> IntraStageResult:
    """``layer_counts``: ``{(mesh, kind): iterable of layer counts}``; ``num_stages_for_mesh(mesh)``
    gives the pipeline depth implied by a mesh (for the 1F1B warm-up depth of middle stages the
    deepest case, stage index 0 for first/only, is assumed: it is the memory worst case)."""
    from .candidates import device_mesh_candidates, grad_accum_candidates
    ev = ev or StageEvaluator(cfg)
    hw = cfg.hardware
    grad_accums = list(grad_accums or grad_accum_candidates(cfg.training.global_batch_size))
    meshes = list(meshes or device_mesh_candidates(hw.num_nodes, hw.num_gpus_per_node))
    key = _cache_key(cfg, f"{grad_accums}|{meshes}|{sorted((str(k), list(v)) for k, v in (layer_counts or {}).items())}|{tp}")
    path = os.path.join(cache_dir, f"intra_stage_{key}.pkl") if cache_dir else None
    if path and os.path.exists(path):
        with open(path, "rb") as f:
            return pickle.load(f)
    out = IntraStageResult()
    total_devices = hw.num_devices
    L = cfg.model.num_hidden_layers
    for g in grad_accums:
        for mesh in meshes:
            n_dev = mesh[0] * mesh[1]
            S = num_stages_for_mesh(mesh) if num_stages_for_mesh else max(total_devices // n_dev, 1)
            kinds = [3] if S == 1 else [0, 1, 2]
            asked = sorted({k for (m, k) in (layer_counts or {}) if tuple(m) == tuple(mesh)})
            if asked:
                kinds = asked                      # the caller names the stage kinds it wants priced
            for kind in kinds:
                counts = (layer_counts or {}).get((tuple(mesh), kind))
                if counts is None:
                    counts = [L] if S == 1 else range(1, L - S + 2)
                stage_index = kind - EXACT_MIDDLE if kind >= EXACT_MIDDLE else {0: 0, 1: 1 if S > 2 else 0, 2: S - 1, 3: 0}[kind]
                for layers in counts:
                    pts, n = tune_stage_cell(ev, cfg, g, tuple(mesh), kind, int(layers), S, stage_index, tp)
                    out.evaluated += n
                    if pts:
                        out.points[(g, tuple(mesh), kind, int(layers))] = pts
    if path:
        os.makedirs(cache_dir, exist_ok=True)
        with open(path, "wb") as f:
            pickle.dump(out, f)
    return out
