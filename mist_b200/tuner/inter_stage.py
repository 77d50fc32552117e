"""Inter-stage tuning: choose the number of pipeline stages, the layers per stage and one
intra-stage point per stage, minimising the 1F1B iteration time

    (G - 1) * max_s T_s + sum_s T_s + max(0, max_s (D_s - sum_{j<s} T_j)).

Granularities (``tuning.tuning_granularity``):

* ``uniform-device-pp-mip`` (default): every stage gets the same device mesh, layers per
  stage within ``avg +- layers_offset``; solved exactly by the native dynamic program
  (the reference solves the same model as a MILP with PuLP/CBC,
  mist/analyzer/inter_tuning_mip.py:90-249, 308-425, Pareto preprocessing :428-535).
* ``inter-stage``: stages may use different meshes; dynamic program over
  (stage, first layer, devices left) as in mist/analyzer/inter_tuning.py:222-355.
* ``uniform-pp`` / ``uniform-device-pp``: uniform layers and devices, scan stage counts
  (mist/analyzer/inter_tuning_uniform.py:123-260, inter_tuning_uniform_device.py).
* ``no-pp``: a single stage.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Dict, List, Optional, Tuple

import numpy as np

from ..analyzer.stage_evaluator import StageEvaluator, ties_across_stages
from ..config import MistConfig
from ..ops import native
from .candidates import device_mesh_candidates, grad_accum_candidates, stage_count_candidates
from .intra_stage import intra_stage_tune

Solution = Tuple[int, List[Tuple[Tuple[Tuple[int, int], Tuple[int, int], int, int], Tuple[float, ...]]]]


#: stage kinds: 0 first, 1 any middle stage, 2 last, 3 the only stage; EXACT_MIDDLE + s: the middle stage at
#: pipeline position s, priced with that position's 1F1B warm-up depth (the reference's
#: pre_saved_micro_batches dimension, mist/analyzer/batched_module_analyzer.py:581-685)
EXACT_MIDDLE = 10


def uniform_mesh_for(num_stages: int, num_nodes: int, gpus_per_node: int) -> Optional[Tuple[int, int]]:
    total = num_nodes * gpus_per_node
    if total % num_stages:
        return None
    per = total // num_stages
    if per >= gpus_per_node:
        if per % gpus_per_node:
            return None
        return (per // gpus_per_node, gpus_per_node)
    if gpus_per_node % per:
        return None
    return (1, per)


def _solve_native(num_stages, total_layers, g, kinds, layers, T, D) -> Tuple[float, List[int]]:
    lib = native.runtime()
    fn = lib.rt_inter_stage_solve
    fn.restype = C.c_double
    n = len(T)
    k = np.ascontiguousarray(kinds, dtype=np.int32)
    l = np.ascontiguousarray(layers, dtype=np.int32)
    t = np.ascontiguousarray(T, dtype=np.float64)
    d = np.ascontiguousarray(D, dtype=np.float64)
    ids = np.arange(n, dtype=np.int32)
    chosen = np.full(num_stages, -1, dtype=np.int32)
    cost = fn(C.c_int(num_stages), C.c_int(total_layers), C.c_int(g), C.c_int64(n), k.ctypes.data_as(C.c_void_p),
              l.ctypes.data_as(C.c_void_p), t.ctypes.data_as(C.c_void_p), d.ctypes.data_as(C.c_void_p),
              ids.ctypes.data_as(C.c_void_p), chosen.ctypes.data_as(C.c_void_p))
    return float(cost), chosen.tolist()


def _solve_python(num_stages, total_layers, g, kinds, layers, T, D) -> Tuple[float, List[int]]:
    """Reference implementation of the native solver (exhaustive over stages with pruning);
    used when the runtime library is unavailable and by the tests as an oracle."""
    n = len(T)
    best = [math.inf, None]

    def kind_of(s):
        if num_stages == 1:
            return 3
        return 0 if s == 0 else (2 if s == num_stages - 1 else 1)

    by_kind = {k: [i for i in range(n) if kinds[i] == k and math.isfinite(T[i])] for k in set(kinds) | {0, 1, 2, 3}}

    def candidates(s):
        k = kind_of(s)
        if k == 1 and by_kind.get(EXACT_MIDDLE + s):
            return by_kind[EXACT_MIDDLE + s]      # priced for exactly this stage index (its own warm-up depth)
        return by_kind[k]

    def rec(s, used, sumT, worst, tmax, choice):
        if s == num_stages:
            if used == total_layers:
                cost = (g - 1) * tmax + sumT + max(worst, 0.0)
                if cost < best[0]:
                    best[0], best[1] = cost, list(choice)
            return
        if (g - 1) * tmax + sumT >= best[0]:
            return
        for i in candidates(s):
            nu = used + layers[i]
            if nu > total_layers or total_layers - nu < num_stages - 1 - s:
                continue
            choice.append(i)
            rec(s + 1, nu, sumT + T[i], max(worst, D[i] - sumT), max(tmax, T[i]), choice)
            choice.pop()

    rec(0, 0, 0.0, -math.inf, 0.0, [])
    return best[0], (best[1] or [])


def solve_stage_assignment(num_stages, total_layers, g, kinds, layers, T, D, use_native=True):
    if use_native:
        try:
            return _solve_native(num_stages, total_layers, g, kinds, layers, T, D)
        except (OSError, AttributeError):
            pass
    return _solve_python(num_stages, total_layers, g, kinds, layers, T, D)


def _layer_range(total_layers: int, num_stages: int, offset: int) -> range:
    avg = total_layers / num_stages
    lo = max(1, int(math.floor(avg)) - offset)
    hi = min(total_layers - (num_stages - 1), int(math.ceil(avg)) + offset)
    return range(lo, hi + 1)


def inter_stage_tune(cfg: MistConfig, ev: Optional[StageEvaluator] = None, cache_dir: Optional[str] = None,
                     tp: Optional[int] = None, verbose: bool = False, single_stage: bool = False
                     ) -> Tuple[float, Optional[Solution]]:
    """Returns ``(best_cost, solution)`` with ``solution = [G, [(((layer_start, layer_end),
    (nodes, gpus), num_ckpt, point_index), strategy_vector), ...]]``."""
    ev = ev or StageEvaluator(cfg, cache_dir=cache_dir)
    hw, tun = cfg.hardware, cfg.tuning
    gran = tun.tuning_granularity
    L = cfg.model.num_hidden_layers
    offset = int(getattr(tun, "layers_offset", 2))
    # Encoder-decoder models run over pipeline stages in one fixed form (encoder blocks on the first
    # stages, the whole decoder on the last): searched by a routine of its own, beside the one-stage case.
    if cfg.model.add_decoder and not single_stage:
        one = inter_stage_tune(cfg, ev, cache_dir, tp, verbose, single_stage=True)
        if gran == "no-pp":
            return one
        piped = _enc_dec_pipeline_tune(cfg, ev, tp, verbose)
        return piped if piped[0] < one[0] else one
    if single_stage:
        gran = "no-pp"
    if gran == "inter-stage":
        return _inter_stage_tune_nonuniform(cfg, ev, cache_dir, tp)
    if gran == "no-pp":
        stage_counts = [1]
    else:
        stage_counts = stage_count_candidates(hw.num_devices, L)
    uniform_layers = gran in ("uniform-pp", "uniform-device-pp", "uniform-pp-simple-heuristic-mem-opt")
    from ..models.provider import family_of
    tied = bool(cfg.model.tie_word_embeddings) or family_of(cfg.model.name) == "bert"
    best_cost, best_sol = math.inf, None
    for S in stage_counts:
        mesh = uniform_mesh_for(S, hw.num_nodes, hw.num_gpus_per_node)
        if mesh is None:
            continue
        if uniform_layers:
            if L % S:
                continue
            counts = [L // S]
        else:
            counts = list(_layer_range(L, S, offset)) if S > 1 else [L]
        # pipelines deeper than three stages price every middle position with its own warm-up depth
        kinds = [3] if S == 1 else ([0, 1, 2] if S <= 3 else [0] + [EXACT_MIDDLE + i for i in range(1, S - 1)] + [2])
        lc = {(mesh, k): counts for k in kinds}
        g_cands = [g for g in grad_accum_candidates(cfg.training.global_batch_size)]
        intra = intra_stage_tune(cfg, ev, grad_accums=g_cands, meshes=[mesh], layer_counts=lc, tp=tp,
                                 cache_dir=cache_dir, num_stages_for_mesh=lambda m, S=S: S)
        for g in g_cands:
            opt_kind, opt_layers, opt_T, opt_D, opt_ref = [], [], [], [], []
            for k in kinds:
                for l in counts:
                    for pi, p in enumerate(intra.get(g, mesh, k, l)):
                        opt_kind.append(k)
                        opt_layers.append(l)
                        opt_T.append(p.stable)
                        opt_D.append(p.delta)
                        opt_ref.append((k, l, pi, p))
            if not opt_T:
                continue
            if tied and S > 1:
                # tables tied across the first and the last stage pair the ranks of the two stages, which
                # needs the same dp x tp layout on both: solve once per layout of the end stages
                cost, chosen = math.inf, None
                layouts = {(int(r[3].vector[1]), int(r[3].vector[2])) for r in opt_ref if r[0] in (0, 2)}
                for lay in sorted(layouts):
                    keep = [i for i, r in enumerate(opt_ref)
                            if r[0] not in (0, 2) or (int(r[3].vector[1]), int(r[3].vector[2])) == lay]
                    c, ch = solve_stage_assignment(S, L, g, [opt_kind[i] for i in keep], [opt_layers[i] for i in keep],
                                                   [opt_T[i] for i in keep], [opt_D[i] for i in keep])
                    if ch and c < cost:
                        cost, chosen = c, [keep[i] for i in ch]
            else:
                cost, chosen = solve_stage_assignment(S, L, g, opt_kind, opt_layers, opt_T, opt_D)
            if verbose:
                print(f"  stages={S} mesh={mesh} G={g}: cost={cost:.6f}")
            if not chosen or not math.isfinite(cost) or cost >= best_cost:
                continue
            best_cost = cost
            start, stages = 0, []
            for ci in chosen:
                k, l, pi, p = opt_ref[ci]
                stages.append((((start, start + l - 1), mesh, p.num_ckpt, pi), p.vector))
                start += l
            best_sol = [g, stages]
    return best_cost, best_sol


def _enc_dec_pipeline_tune(cfg, ev, tp, verbose=False):
    """Encoder-decoder models over S >= 2 stages of equal meshes: the L encoder blocks are split over the
    first S - 1 stages (the split is searched), the last stage holds the L decoder blocks, the head and its own
    copies of the embedding tables (what the executor runs, ``StrategyConfig.verify_with_other_config``).
    Every stage cell is tuned with its own kind of block; the exact stage-assignment solver then picks one
    Pareto point per stage."""
    from .intra_stage import tune_stage_cell
    hw, tun = cfg.hardware, cfg.tuning
    L = cfg.model.num_hidden_layers
    offset = int(getattr(tun, "layers_offset", 2))
    uniform_layers = tun.tuning_granularity in ("uniform-pp", "uniform-device-pp", "uniform-pp-simple-heuristic-mem-opt")
    best_cost, best_sol = math.inf, None
    for S in stage_count_candidates(hw.num_devices, L + 1):
        if S < 2:
            continue
        mesh = uniform_mesh_for(S, hw.num_nodes, hw.num_gpus_per_node)
        if mesh is None:
            continue
        enc_stages = S - 1
        if uniform_layers:
            if L % enc_stages:
                continue
            counts = [L // enc_stages]
        else:
            counts = list(_layer_range(L, enc_stages, offset)) if enc_stages > 1 else [L]
        for g in grad_accum_candidates(cfg.training.global_batch_size):
            opt_kind, opt_layers, opt_T, opt_D, opt_ref = [], [], [], [], []
            cells = [(0, l, "enc_block_layer", None, 0) for l in counts]
            if enc_stages > 1:
                cells += [(1, l, "enc_block_layer", None, 1) for l in counts]
            cells.append((2, L, "dec_block_layer", True, S - 1))
            for kind, l, block_kind, has_pre, stage_index in cells:
                pts, _ = tune_stage_cell(ev, cfg, g, mesh, kind, l, S, stage_index, tp, block_kind=block_kind,
                                         has_pre=has_pre)
                for pi, p in enumerate(pts):
                    opt_kind.append(kind)
                    opt_layers.append(l)
                    opt_T.append(p.stable)
                    opt_D.append(p.delta)
                    opt_ref.append((kind, l, pi, p))
            if not any(k == 2 for k in opt_kind) or not any(k == 0 for k in opt_kind):
                continue
            # the solver counts layers over all stages: L encoder blocks plus the decoder stage's L
            cost, chosen = solve_stage_assignment(S, 2 * L, g, opt_kind, opt_layers, opt_T, opt_D)
            if verbose:
                print(f"  encoder-decoder stages={S} mesh={mesh} G={g}: cost={cost:.6f}")
            if not chosen or not math.isfinite(cost) or cost >= best_cost:
                continue
            best_cost = cost
            start, stages = 0, []
            for ci in chosen:
                k, l, pi, p = opt_ref[ci]
                rng = (0, L - 1) if k == 2 else (start, start + l - 1)
                stages.append(((rng, mesh, p.num_ckpt, pi), p.vector))
                start += l
            best_sol = [g, stages]
    return best_cost, best_sol


def _prune_dominated(labels: List[Tuple]) -> List[Tuple]:
    """Keeps the labels ``(sum T, max T, exposed delta, path)`` that no other label beats in all three
    numbers.  The iteration time ``(G - 1) max T + sum T + max(exposed, 0)`` grows with each of them, and
    appending a stage adds the same amounts to every label of a state, so a dominated label can never
    end up in the best complete pipeline: the search stays exact."""
    labels = sorted(labels, key=lambda x: (x[0], x[1], x[2]))
    kept: List[Tuple] = []
    for lab in labels:
        if not any(k[0] <= lab[0] and k[1] <= lab[1] and k[2] <= lab[2] for k in kept):
            kept.append(lab)
    return kept


def _inter_stage_tune_nonuniform(cfg, ev, cache_dir, tp):
    """Stages may differ in device count: dynamic program over (stage, layers assigned, devices used
    [, layout of the first stage]) that keeps every non-dominated (sum T, max T, exposed delta) summary
    per state for a fixed G; G is scanned outside (reference: the ``inter-stage`` dynamic program of
    mist/analyzer/inter_tuning.py:222-355).  Models that tie a table across the first and the last
    stage carry the first stage's dp x tp layout in the state, and the last stage only takes
    strategies with that layout (the executor pairs the ranks of the two stages)."""
    hw = cfg.hardware
    L = cfg.model.num_hidden_layers
    meshes = [m for m in device_mesh_candidates(hw.num_nodes, hw.num_gpus_per_node)]
    total_dev = hw.num_devices
    tied = ties_across_stages(cfg)
    best_cost, best_sol = math.inf, None
    max_stages = min(total_dev, L, 8)
    for g in grad_accum_candidates(cfg.training.global_batch_size):
        for S in range(1, max_stages + 1):
            kinds = [3] if S == 1 else [0, 1, 2]
            counts = list(_layer_range(L, S, int(getattr(cfg.tuning, "layers_offset", 2)))) if S > 1 else [L]
            lc = {(tuple(m), k): counts for m in meshes for k in kinds}
            intra = intra_stage_tune(cfg, ev, grad_accums=[g], meshes=meshes, layer_counts=lc, tp=tp,
                                     cache_dir=cache_dir, num_stages_for_mesh=lambda m, S=S: S)
            # state: (layers used, devices used, layout of the first stage or None) -> labels
            states: Dict = {(0, 0, None): [(0.0, 0.0, -math.inf, [])]}
            for s in range(S):
                k = 3 if S == 1 else (0 if s == 0 else (2 if s == S - 1 else 1))
                nxt: Dict = {}
                for (used, dev, first_layout), labels in states.items():
                    for m in meshes:
                        nd = m[0] * m[1]
                        if dev + nd > total_dev or (total_dev - dev - nd) < (S - 1 - s):
                            continue
                        for l in counts:
                            if used + l > L or (L - used - l) < (S - 1 - s):
                                continue
                            for pi, p in enumerate(intra.get(g, tuple(m), k, l)):
                                layout = (int(p.vector[1]), int(p.vector[2]))
                                if tied and S > 1:
                                    if s == S - 1 and layout != first_layout:
                                        continue
                                    key_layout = layout if s == 0 else first_layout
                                else:
                                    key_layout = None
                                key = (used + l, dev + nd, key_layout)
                                cur = nxt.setdefault(key, [])
                                for (sumT, maxT, worst, path) in labels:
                                    cur.append((sumT + p.stable, max(maxT, p.stable), max(worst, p.delta - sumT),
                                                path + [(((used, used + l - 1), tuple(m), p.num_ckpt, pi), p.vector)]))
                states = {key: _prune_dominated(labels) for key, labels in nxt.items()}
            for (used, dev, _), labels in states.items():
                if used != L or dev != total_dev:
                    continue
                for lab in labels:
                    cost = (g - 1) * lab[1] + lab[0] + max(lab[2], 0.0)
                    if cost < best_cost:
                        best_cost, best_sol = cost, [g, lab[3]]
    return best_cost, best_sol


def solution_to_strategy(cfg: MistConfig, solution: Solution) -> Dict:
    """The ``strategy`` block (as plain dict) that reproduces ``solution`` in exec / analyze."""
    g, stages = solution
    layer_partitions = [s[0][0][1] - s[0][0][0] + 1 for s in stages]
    vectors = [list(s[1]) for s in stages]
    for v in vectors:
        v[0], v[1], v[2] = int(v[0]), int(v[1]), int(v[2])
        v[3], v[4], v[5] = int(v[3]), int(v[4]), int(v[5])
    last = vectors[-1]
    return {
        "enabled": True,
        "layer_partitions": layer_partitions,
        "device_assignment": [list(s[0][1]) for s in stages],
        "gradient_checkpointing": [int(s[0][2]) for s in stages],
        "gradient_accumulation_steps": int(g),
        "stage_strategies": vectors,
        "pre_post_strategy": "preset",
        "pre_post_strategy_array": [last[0], last[1], last[2], 0, 0, 1, 0, 0, 0, 0],
    }
