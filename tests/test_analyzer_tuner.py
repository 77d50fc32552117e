"""Symbolic analysis, cost models and the tuner (CPU only)."""
import math
import os

import numpy as np
import pytest
import sympy as sp
import torch

from mist_b200.analyzer.layer_analyzer import trace_and_analyze
from mist_b200.analyzer.stage_evaluator import (StageEvaluator, analyze_strategy, create_search_space,
                                                pipeline_latency)
from mist_b200.analyzer.symtensor import SymTensor, tracing
from mist_b200.config import load_config
from mist_b200.node_database.database import OpDatabase
from mist_b200.node_database.node_spec import NodeSpec
from mist_b200.symbols import SymbolManager
from mist_b200.tools import comm_model
from mist_b200.tuner.candidates import device_mesh_candidates, grad_accum_candidates
from mist_b200.tuner.inter_stage import _solve_native, _solve_python, inter_stage_tune, solution_to_strategy
from mist_b200.tuner.pareto import pareto_filter, sample_pareto_frontier

B = sp.Symbol("b", integer=True, positive=True)


def _mb(expr, b):
    return float(sp.sympify(expr).subs(B, b)) / 2 ** 20


def test_symbol_manager():
    m = SymbolManager()
    b, t = m.symbols("b tp", (2, 4))
    assert m.map(b * 3 + t) == 10 and m.map(b * 3 + t, {"b": 5}) == 19
    assert m.verify(sp.Eq(b * 2, t)) and not m.verify(b > t)
    assert m.solve(sp.Eq(b * t, 8), "b") == [8 / t]
    f = m.lambdify(b * 2 + t, ["b"])
    assert list(f(np.array([1, 2]))) == [6, 8]


def test_symbolic_ops_shapes_and_saved_tensors():
    m = SymbolManager()
    b = m.symbols("b", 2)
    with tracing() as g:
        x = SymTensor((b, 128, 64), torch.bfloat16, requires_grad=True)
        w = torch.nn.Parameter(torch.empty(256, 64, dtype=torch.bfloat16, device="meta"))
        y = torch.nn.functional.linear(x, w)
        z = torch.tanh(y).reshape(-1, 256).transpose(0, 1)
        s = (z * 2.0).sum()
    assert y.shape == (b, 128, 256) and z.shape == (256, 128 * b)
    ops = [n.op for n in g.nodes]
    assert ops[:2] == ["linear", "tanh"] and "mul" in ops
    lin = g.nodes[0]
    assert sp.simplify(lin.flops_fwd - 2 * b * 128 * 64 * 256) == 0
    assert x.tid in lin.saved                      # autograd keeps the input of a linear
    assert g.nodes[1].saved == [g.nodes[1].outputs[0].tid]   # tanh keeps its output


def test_layer_memory_matches_hand_count_gpt27b():
    cfg, _ = load_config("config", check_world_size=False)
    a = trace_and_analyze(cfg.model, 2048, tp=1)
    unit = 16384 * 2560 * 2 / 2 ** 20                        # one [tokens, hidden] bf16 tensor at b = 8
    # saved per block: x, ln1 out, qkv (3x), attn out, summed residual, ln2 out, fc1 pre-act (4x), gelu out (4x)
    assert abs(_mb(a.block.fwd.saved, 8) - 16 * unit) < 0.02 * 16 * unit
    assert abs(_mb(a.block.input_bytes, 8) - 2 * unit) < 1e-6
    assert abs(_mb(a.block.fwd.output, 8) - 2 * unit) < 1e-6
    assert a.block.num_params == cfg.model.params_per_block() or abs(a.block.num_params - cfg.model.params_per_block()) < 16
    # the head keeps the logits
    assert _mb(a.post.fwd.saved, 8) > 16384 * 50304 * 2 / 2 ** 20
    # memory is linear in the micro batch
    assert abs(_mb(a.block.fwd.saved, 4) * 2 - _mb(a.block.fwd.saved, 8)) < 1.0


def test_tensor_and_sequence_parallel_trace():
    cfg, _ = load_config("config", ["experiment=b200-llama-7b-tp2sp-dp4"], check_world_size=False)
    a1 = trace_and_analyze(cfg.model, 4096, tp=1)
    a2 = trace_and_analyze(cfg.model, 4096, tp=2, sequence_parallel=True)
    assert [c.kind for c in a2.block.fwd.comms] == ["all_gather", "reduce_scatter", "all_gather", "reduce_scatter"]
    assert [c.kind for c in a2.block.bwd.comms] == ["reduce_scatter", "all_gather", "reduce_scatter", "all_gather"]
    assert a2.block.num_params < 0.51 * a1.block.num_params + 2 * 4096
    assert _mb(a2.block.fwd.saved, 2) < 0.62 * _mb(a1.block.fwd.saved, 2)
    a3 = trace_and_analyze(cfg.model, 4096, tp=2, sequence_parallel=False)
    assert [c.kind for c in a3.block.fwd.comms] == ["all_reduce", "all_reduce"]


def test_every_family_traces():
    for exp, over in (("gpt2-1.3b", []), ("llama-1.3b", [])):
        cfg, _ = load_config("config", [f"experiment={exp}"] + over, check_world_size=False)
        a = trace_and_analyze(cfg.model, cfg.training.max_sequence_length)
        assert a.block.nodes and a.pre.nodes and a.post.nodes
    from mist_b200.config import ModelConfig
    base = dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                max_position_embeddings=128, vocab_size=1024, params_dtype="bfloat16", add_encoder=True, use_flash_attn=True)
    for mc in (ModelConfig(name="falcon-t", add_decoder=False, encoder_attn_mask_type="causal", parallel_block=True,
                           position_embedding_type="rotary", rotary_emb_fraction=1.0, **base),
               ModelConfig(name="bert-t", add_decoder=False, encoder_attn_mask_type="padding", add_pooler=True,
                           num_tokentypes=2, **base),
               ModelConfig(name="t5-t", add_decoder=True, encoder_attn_mask_type="padding",
                           decoder_attn_mask_type="causal", **base)):
        a = trace_and_analyze(mc, 128)
        assert a.block.num_params > 0 and a.graph_nodes > 10


def test_comm_and_interference_models():
    table = [4.5, 0, 100, 1e-5, 200, 1e-5, 300, 2e-5] + [4.5, 0] * 12
    t = comm_model.gpu_gpu_latency("all_gather", np.array([0.3]), 8, 1, table)[0]
    assert abs(t - (0.3 / 300 * 7 / 8 + 2e-5)) < 1e-12
    assert comm_model.gpu_gpu_latency("all_reduce", np.array([0.3]), 8, 1, table)[0] == pytest.approx(2.1 * t)
    assert comm_model.gpu_gpu_latency("all_gather", np.array([0.3]), 1, 1, table)[0] == 0.0
    assert comm_model.host_copy_latency(np.array([0.5, 0.0]), [50.0, 1e-4]).tolist() == [0.5 / 50 + 1e-4, 0.0]
    p = np.ones(28)
    # with unit factors channels overlap perfectly: total = max
    assert comm_model.interference_estimate(1.0, 0.4, 0.2, 0.7, p) == pytest.approx(1.0)
    p[16:18] = [1.5, 1.0]              # compute stretches 1.5x while a collective runs
    assert comm_model.interference_estimate(1.0, 0.6, 0.0, 0.0, p) == pytest.approx(0.6 + (1.5 - 0.6) / 1.5)
    assert comm_model.interference_estimate(0.0, 0.6, 0.0, 0.0, p) == pytest.approx(0.6)


def test_search_space_rules():
    cfg, _ = load_config("test-small-base", check_world_size=False)
    sp_ = create_search_space(1, 2, 32, 2, cfg)
    assert sp_.shape[1] == 10 and len(sp_) > 100
    assert not np.any((sp_[:, 6] > 0) & (sp_[:, 7] == 0))            # weight offload implies grad offload
    assert np.all(sp_[:, 0] * sp_[:, 1] * 2 == 32) and np.all(sp_[:, 1] * sp_[:, 2] == 2)
    dp1 = sp_[sp_[:, 1] == 1]
    assert np.all(dp1[:, 3:6] == [0, 0, 1]) if len(dp1) else True     # no ZeRO choice without data parallelism


def test_stage_evaluator_monotonic_and_feasibility(monkeypatch):
    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_B200")
    cfg, _ = load_config("config", check_world_size=False)
    ev = StageEvaluator(cfg, OpDatabase(allow_profile=False))
    vec = np.array([[8, 8, 1, 0, 1, 1, 0, 0, 0, 0], [8, 8, 1, 1, 1, 1, 0, 0, 0, 0], [8, 8, 1, 0, 0, 1, 0, 0, 0, 0]], dtype=float)
    r0 = ev.evaluate(vec, 32, 0, 1, True, True)
    r1 = ev.evaluate(vec, 32, 32, 1, True, True)
    assert np.all(r1["stable"] > r0["stable"])               # recomputation costs time ...
    assert np.all(r1["peak_bwd"] < r0["peak_bwd"])           # ... and saves memory
    assert r0["peak_fwd"][1] < r0["peak_fwd"][0] < r0["peak_fwd"][2]    # ZeRO-3 < ZeRO-2 < ZeRO-1
    assert np.all(r0["feasible"])
    # a 40 GB device cannot hold it without sharding / checkpointing
    cfg.hardware.memory_capacity = 40 * 0.88
    assert not ev.evaluate(vec[2:], 32, 0, 1, True, True)["feasible"][0]


def test_pipeline_latency_formula():
    assert pipeline_latency([2.0], [0.5], 4) == pytest.approx(8.5)
    assert pipeline_latency([1.0, 2.0], [0.5, 0.1], 4) == pytest.approx(3.0 + 3 * 2.0 + 0.5)
    from mist_b200.ops import native
    import ctypes as C
    lib = native.runtime()
    lib.rt_simulate_1f1b.restype = C.c_double
    fwd = (C.c_double * 2)(0.4, 0.8)
    bwd = (C.c_double * 2)(0.6, 1.2)
    t = lib.rt_simulate_1f1b(2, 4, fwd, bwd, None, C.c_double(0.0), None)
    # the event simulation agrees with the closed form (stage time = fwd + bwd)
    assert t == pytest.approx(pipeline_latency([1.0, 2.0], [0.0, 0.0], 4), rel=0.08)


def test_uniform_micro_batch_analysis_flag(monkeypatch):
    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_B200")
    over = ["hardware.num_gpus_per_node=8", "strategy.enabled=true", "strategy.layer_partitions=[16,16]",
            "strategy.device_assignment=[[1,4],[1,4]]", "strategy.gradient_checkpointing=[0,0]",
            "strategy.gradient_accumulation_steps=4", "training.global_batch_size=32",
            "strategy.stage_strategies=[[2,4,1,0,1,1,0,0,0,0],[2,4,1,0,1,1,0,0,0,0]]",
            "strategy.pre_post_strategy=heuristic"]
    cfg, _ = load_config("config", over, check_world_size=False)
    from mist_b200.analyzer.stage_evaluator import analyze_strategy
    ev = StageEvaluator(cfg, OpDatabase(allow_profile=False))
    a = analyze_strategy(cfg, ev)
    cfg2, _ = load_config("config", over + ["+disable_non_uniform_pp_micro_batch_analysis=true"], check_world_size=False)
    b = analyze_strategy(cfg2, StageEvaluator(cfg2, OpDatabase(allow_profile=False)))
    assert any(d > 0 for d in a["delta"]) and all(d == 0 for d in b["delta"])
    for s in range(2):
        assert b["stable"][s] == pytest.approx(a["stable"][s] + a["delta"][s] / 4)
    assert b["total"] == pytest.approx(sum(b["stable"]) + 3 * max(b["stable"]))
    assert b["peak_memories"] == a["peak_memories"]


def test_pareto_sampling():
    rng = np.random.default_rng(0)
    x, y = rng.random(200), rng.random(200)
    feas = rng.random(200) > 0.3
    a = sample_pareto_frontier(x, y, feas, 7, use_native=True)
    b = sample_pareto_frontier(x, y, feas, 7, use_native=False)
    assert a.tolist() == b.tolist() and all(feas[i] for i in a)
    front = set(pareto_filter(np.where(feas, x, np.inf), np.where(feas, y, np.inf)).tolist())
    assert set(a.tolist()) <= front
    assert sample_pareto_frontier(x, y, np.zeros(200, dtype=bool), 3).tolist() == [-1, -1, -1]


def test_inter_stage_solver_matches_exhaustive():
    rng = np.random.default_rng(1)
    for _ in range(10):
        S, L, g = int(rng.integers(1, 5)), int(rng.integers(4, 9)), int(rng.integers(1, 9))
        kinds, layers, T, D = [], [], [], []
        for k in ([3] if S == 1 else [0, 1, 2]):
            for l in range(1, L + 1):
                for _ in range(3):
                    kinds.append(k)
                    layers.append(l)
                    T.append(float(rng.uniform(0.5, 1.5) * l))
                    D.append(float(rng.uniform(0, 2)))
        a = _solve_native(S, L, g, kinds, layers, T, D)
        b = _solve_python(S, L, g, kinds, layers, T, D)
        assert a[0] == pytest.approx(b[0])
        assert sum(layers[i] for i in a[1]) == L


def test_candidates():
    assert device_mesh_candidates(2, 8) == [(1, 1), (1, 2), (1, 4), (1, 8), (2, 8)]
    assert grad_accum_candidates(24) == [1, 2, 4, 8]


def test_tune_small_case_end_to_end(monkeypatch, tmp_path):
    """GPT-1.3B on 2 devices with the L4 calibration: the tuner must return a valid strategy that
    the analyzer prices at the tuner's own cost and that beats the hand-written base strategy."""
    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_L4")
    cfg, node = load_config("test-small-base", check_world_size=False)
    ev = StageEvaluator(cfg, OpDatabase(allow_profile=False))
    base = analyze_strategy(cfg, ev)["total"]
    cost, sol = inter_stage_tune(cfg, ev)
    assert sol is not None and math.isfinite(cost) and cost < base
    strat = solution_to_strategy(cfg, sol)
    assert sum(strat["layer_partitions"]) == 24
    plain = node.to_dict()
    plain["strategy"] = strat
    from mist_b200.utils import yamlconf
    yamlconf.dump(plain, tmp_path / "best.yaml")
    cfg2, _ = load_config("best", config_dirs=[tmp_path], check_world_size=False)    # validates the strategy
    again = analyze_strategy(cfg2, StageEvaluator(cfg2, OpDatabase(allow_profile=False)))["total"]
    assert again == pytest.approx(cost, rel=1e-6)


def test_every_tuning_granularity_returns_a_valid_strategy(monkeypatch):
    """Wider search spaces can only find cheaper strategies: no-pp >= uniform-pp >= uniform-device-pp-mip
    >= inter-stage (up to the Pareto sampling), and each result passes the strategy validation."""
    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_L4")
    costs = {}
    for gran in ("no-pp", "uniform-pp", "uniform-device-pp-mip", "inter-stage"):
        cfg, node = load_config("test-small-base", ["model.num_hidden_layers=8", "training.global_batch_size=8",
                                                    "strategy.enabled=false", f"tuning.tuning_granularity={gran}"],
                                check_world_size=False)
        cost, sol = inter_stage_tune(cfg, StageEvaluator(cfg, OpDatabase(allow_profile=False)))
        assert sol is not None and math.isfinite(cost)
        strat = solution_to_strategy(cfg, sol)
        assert sum(strat["layer_partitions"]) == 8
        assert sum(n * m for n, m in strat["device_assignment"]) == 2
        if gran == "no-pp":
            assert len(strat["layer_partitions"]) == 1
        costs[gran] = cost
    tol = 1.02
    assert costs["uniform-pp"] <= costs["no-pp"] * tol
    assert costs["uniform-device-pp-mip"] <= costs["uniform-pp"] * tol
    assert costs["inter-stage"] <= costs["uniform-device-pp-mip"] * tol


def test_op_database_roundtrip(tmp_path):
    db = OpDatabase(device="TEST_GPU", root=tmp_path, allow_profile=False)
    spec = NodeSpec.from_dict({"op": "linear", "m": 8 * B, "n": 16, "k": 32, "act": "", "bias": False}, {"b": 4})
    assert spec.key() == "linear(act=,bias=False,k=32,m=32,n=16)"
    est = db.latency(spec, 1e9, 2e9, 1e6, 2e6)
    db.add(spec, 1.5e-3, 3e-3)
    db2 = OpDatabase(device="TEST_GPU", root=tmp_path, allow_profile=False)
    assert db2.latency(spec) == (1.5e-3, 3e-3) and est != (1.5e-3, 3e-3)


def test_experiment_orchestration_tune_then_analyze(tmp_path):
    """tune -> analyze for two search spaces without GPUs; the analyzer must reproduce the cost
    the tuner reported for its best strategy, and an identical solution is not run twice."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "exp"
    r = subprocess.run([sys.executable, os.path.join(root, "benchmark/mist_b200/experiment/run.py"), "--model",
                        "gpt2/1.3b", "-m", "2", "--global-batch-size", "8", "--spaces", "mist", "zero1-only",
                        "--skip-exec", "--out", str(out)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    s = json.load(open(out / "mist" / "summary.json"))
    assert abs(float(s["tuning_best_cost"]) - float(s["analyzed_total_cost"])) <= 0.02 * float(s["tuning_best_cost"])
    assert (out / "mist" / "best_config.yaml").exists()


def test_prediction_accuracy_report(tmp_path, capsys):
    import importlib.util
    import json
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location(
        "acc", os.path.join(root, "benchmark/mist_b200/prediction-accuracy/get_mem_and_latency_accuracy.py"))
    acc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(acc)
    for name, pred, meas in (("a", 1.10, 1.00), ("b", 1.98, 2.00)):
        d = tmp_path / name
        d.mkdir()
        json.dump({"analyzed_total_cost": str(pred), "exec_total_cost": str(meas),
                   "analyzed_stage_peak_memories": "[1100 MB]", "exec_stage_peak_allocated_memories": "[1000 MB]"},
                  open(d / "summary.json", "w"))
    acc.main([str(tmp_path)])
    text = capsys.readouterr().out
    assert "2 cases" in text and "mean abs rel err 5.50 %" in text and "memory : mean abs rel err 10.00 %" in text


def test_encoder_decoder_blocks_are_priced_apart(monkeypatch):
    """T5: a single-stage "layer" is an encoder block plus a decoder block; pipeline stages are priced with the
    kind of block they hold, so an encoder stage costs less than a decoder stage of the same depth."""
    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_B200")
    from mist_b200.analyzer.layer_analyzer import trace_and_analyze
    from mist_b200.analyzer.stage_evaluator import analyze_strategy
    cfg, _ = load_config("config", ["experiment=gpt2-1.3b", "model=t5/1.7b"], check_world_size=False)
    a = trace_and_analyze(cfg.model, 512, 1, False)
    assert a.block.num_params == a.enc_block.num_params + a.dec_block.num_params
    assert a.dec_block.num_params > a.enc_block.num_params            # cross attention
    vec = "[4,1,1,0,0,0,0,0,0,0]"
    cfg2, _ = load_config("config", ["experiment=gpt2-1.3b", "model=t5/1.7b", "hardware.num_gpus_per_node=2",
                                     "training.global_batch_size=8", "strategy.layer_partitions=[16,16]",
                                     "strategy.device_assignment=[[1,1],[1,1]]", "strategy.gradient_checkpointing=[0,0]",
                                     "strategy.gradient_accumulation_steps=2", f"strategy.stage_strategies=[{vec},{vec}]",
                                     f"strategy.pre_post_strategy_array={vec}"], check_world_size=False)
    res = analyze_strategy(cfg2, StageEvaluator(cfg2, OpDatabase(allow_profile=False)))
    assert res["stable"][0] < res["stable"][1]


def test_nondominated_pruning_keeps_every_possible_winner():
    """The inter-stage dynamic program drops a partial pipeline only when another one of the same state is
    no worse in all three numbers the iteration time is built from."""
    from mist_b200.tuner.inter_stage import _prune_dominated
    labels = [(1.0, 0.5, 0.1, "a"), (1.0, 0.5, 0.2, "dominated by a"), (0.9, 0.6, 0.1, "b"), (1.2, 0.4, 0.0, "c"),
              (1.3, 0.6, 0.3, "dominated by all"), (0.9, 0.6, 0.1, "duplicate of b")]
    kept = {x[3] for x in _prune_dominated(labels)}
    assert kept == {"a", "b", "c"} or kept == {"a", "duplicate of b", "c"}
    # every label that wins for some gradient-accumulation count survives
    for g in (1, 2, 8, 64):
        best = min(labels, key=lambda x: (g - 1) * x[1] + x[0] + max(x[2], 0.0))
        cost = (g - 1) * best[1] + best[0] + max(best[2], 0.0)
        assert any(abs((g - 1) * k[1] + k[0] + max(k[2], 0.0) - cost) < 1e-12 for k in _prune_dominated(labels))


def test_inter_stage_search_respects_tied_table_layout(tmp_path, monkeypatch):
    """A model that ties its output projection to the word table needs the same dp x tp layout on the first and
    the last pipeline stage; the non-uniform search must only return such pipelines."""
    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_L4")
    cfg, _ = load_config("test-small-base", ["model.num_hidden_layers=8", "model.tie_word_embeddings=true",
                                             "hardware.num_gpus_per_node=4", "training.global_batch_size=16",
                                             "strategy.enabled=false", "tuning.tuning_granularity=inter-stage",
                                             "tuning.sample_size=6", "hardware.memory_capacity=8.0"],
                         check_world_size=False)
    cost, sol = inter_stage_tune(cfg, StageEvaluator(cfg, OpDatabase(allow_profile=False)), cache_dir=str(tmp_path))
    assert sol is not None and cost < float("inf")
    stages = sol[1]
    if len(stages) > 1:
        first, last = stages[0][1], stages[-1][1]
        assert (int(first[1]), int(first[2])) == (int(last[1]), int(last[2]))


def test_kick_the_tires_memory_account(monkeypatch):
    """GPT-1.3B on 2 x L4, DP 2, micro batch 8, G = 2, every block checkpointed, no flash attention (the
    reference's README walk-through: 19 255 / 19 503 MB predicted, 19 274 MB measured there).  This executor
    differs from the reference's in three accountable ways, and the analyzer must price them:

    * gradients accumulated over micro steps are kept in fp32 (the reference accumulates in fp16): + one more
      copy of the fp16 weights, 2 705 MB;
    * a checkpointed block keeps its (hidden, residual) input pair, not one tensor: + 24 x 64 MB = 1 536 MB;
    * the recomputation of a block in the backward pass holds the block's forward and backward working sets
      together.

    The numbers below pin the analyzer's own account (states 16 230 MB, block inputs 3 072 MB) so that a change
    of the memory model shows up here."""
    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_L4")
    cfg, _ = load_config("test-small-base", check_world_size=False)
    ev = StageEvaluator(cfg, OpDatabase(allow_profile=False))
    res = analyze_strategy(cfg, ev)
    fwd, bwd = (x / 2 ** 20 for x in res["peak_memories"][0])
    blk = ev.layer_numbers(1, 8, "block_layer")
    pre, post = ev.layer_numbers(1, 8, "pre_layer"), ev.layer_numbers(1, 8, "post_layer")
    mb = 2 ** 20
    weights = (24 * blk.weight_bytes + pre.weight_bytes + post.weight_bytes) / mb
    assert weights == pytest.approx(2705.0, rel=0.01)                      # fp16 weights of 1.3 B parameters
    states = weights + 2 * weights + 6 * weights / 2                       # + fp32 gradients + Adam state / dp
    assert states == pytest.approx(16230.0, rel=0.01)
    assert 24 * blk.input_bytes / mb == pytest.approx(3072.0, rel=0.01)    # kept inputs of the 24 checkpointed blocks
    assert fwd == pytest.approx(states + 3072.0 + blk.fwd_peak / mb + post.saved / mb, rel=0.02)
    assert fwd == pytest.approx(23372.6, rel=0.02) and bwd == pytest.approx(26892.7, rel=0.02)
    # the same account with the reference's executor choices lands on its own prediction
    ref_like = (weights + weights + 6 * weights / 2) + 24 * blk.input_bytes / 2 / mb + (fwd - states - 3072.0)
    assert ref_like == pytest.approx(19255.0, rel=0.04)


def test_sm_bound_operators_are_priced_with_their_sustained_timing(tmp_path):
    """An entry with a back-to-back timing gives that timing for operators the meta file lists as bound by the
    SMs and its cold timing for every other operator; nothing is scaled by a clock."""
    import json
    d = tmp_path / "cache_TEST_GPU"
    d.mkdir()
    (d / "_meta.json").write_text(json.dumps({"scaled_ops": ["linear"], "sustained_scale": 1.0, "sm_mhz_under_load": 1530.0}))
    db = OpDatabase(device="TEST_GPU", root=tmp_path, allow_profile=False)
    lin = NodeSpec.from_dict({"op": "linear", "m": 64, "n": 16, "k": 32, "act": "", "bias": False}, {})
    norm = NodeSpec.from_dict({"op": "layer_norm", "rows": 64, "h": 32, "residual": True}, {})
    db.add(lin, 1.0e-3, 2.0e-3, fwd_sus=1.2e-3, bwd_sus=2.6e-3, sm_mhz_fwd=1100.0, sm_mhz_bwd=1200.0)
    db.add(norm, 1.0e-4, 2.0e-4, fwd_sus=0.8e-4, bwd_sus=1.5e-4, sm_mhz_fwd=1900.0, sm_mhz_bwd=1900.0)
    assert db.latency(lin) == (1.2e-3, 2.6e-3)
    assert db.latency(norm) == (1.0e-4, 2.0e-4)


def test_fused_overlap_fit_recovers_its_parameters():
    rows = []
    for kind, kappa, tau in (("AG->GEMM qkv", 0.25, 40e-6), ("GEMM->RS fc2 (store)", 0.5, 0.0)):
        for g, c in ((0.5, 0.2), (0.1, 0.12), (1.0, 0.21), (0.06, 0.1), (0.3, 0.3)):
            fused = max(g, c) + kappa * min(g, c) + tau * 1e3
            rows.append(dict(kernel=kind, fused_ms=fused, gemm_ms=g, collective_ms=c))
    rows.append(dict(kernel="GEMM->RS fc2 (add)", fused_ms=9.0, gemm_ms=0.1, collective_ms=0.1))    # ignored form
    fit = comm_model.fit_fused_overlap(rows)
    assert abs(fit["ag_gemm"]["kappa"] - 0.25) < 1e-3 and abs(fit["ag_gemm"]["tau"] - 40e-6) < 1e-6
    assert abs(fit["gemm_rs"]["kappa"] - 0.5) < 1e-3 and fit["gemm_rs"]["tau"] < 1e-6 and fit["gemm_rs"]["rows"] == 5


def test_host_dispatch_bounds_a_block_from_below(monkeypatch):
    """With the host's seconds per block in the operator database's meta data, a block whose kernels are
    faster than the host can issue them is charged the host time; a recomputed block pays the (larger)
    host cost of a checkpointed forward pass."""
    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_B200")
    cfg, _ = load_config("config", check_world_size=False)
    vec = np.array([[1, 8, 1, 0, 1, 1, 0, 0, 0, 0]], dtype=float)      # one sequence per micro batch: small kernels
    db = OpDatabase(allow_profile=False)
    db.host_dispatch = {}
    base = StageEvaluator(cfg, db)
    t0 = base.evaluate(vec, 32, 0, 1, True, True)["stable"][0]
    c0 = base.evaluate(vec, 32, 32, 1, True, True)["stable"][0]
    nodes = len(base.analysis(1).layer("block_layer").nodes)
    slow = OpDatabase(allow_profile=False)
    slow.host_dispatch = {"block_fwd_bwd_s": 0.3, "block_recompute_s": 0.5, "ops_per_block": nodes}
    ev = StageEvaluator(cfg, slow)
    num = ev.layer_numbers(1, 1, "block_layer")
    assert (num.host_fwd, num.host_bwd, num.host_recompute) == pytest.approx((0.1, 0.2, 0.5))
    t1 = ev.evaluate(vec, 32, 0, 1, True, True)["stable"][0]
    c1 = ev.evaluate(vec, 32, 32, 1, True, True)["stable"][0]
    assert t1 >= 32 * 0.3 and t1 > t0
    assert c1 - t1 == pytest.approx(32 * 0.5, rel=0.05) and c1 > c0
    quick = OpDatabase(allow_profile=False)
    quick.host_dispatch = {"block_fwd_bwd_s": 1e-9, "block_recompute_s": 1e-9, "ops_per_block": nodes}
    assert StageEvaluator(cfg, quick).evaluate(vec, 32, 0, 1, True, True)["stable"][0] == pytest.approx(t0)


def test_encoder_decoder_models_are_searched_over_pipeline_stages(monkeypatch, tmp_path):
    """T5 on 4 devices with too little memory for one stage's worth of replicas: the tuner may put the encoder
    blocks on the first stages and the decoder on the last.  Whatever it returns must load as a strategy
    (encoder blocks split over all stages but the last, which holds all decoder blocks) and be priced by the
    analyzer at the tuner's own cost; the pipelined search alone must agree with the analyzer as well."""
    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_B200")
    from mist_b200.tuner.inter_stage import _enc_dec_pipeline_tune
    from mist_b200.utils import yamlconf
    over = ["experiment=gpt2-1.3b", "model=t5/1.7b", "model.num_hidden_layers=8", "hardware.num_gpus_per_node=4",
            "training.global_batch_size=16", "training.max_sequence_length=512", "strategy.enabled=false",
            "tuning.tuning_granularity=uniform-device-pp-mip", "tuning.sample_size=6"]
    cfg, node = load_config("config", over, check_world_size=False)
    ev = StageEvaluator(cfg, OpDatabase(allow_profile=False))

    def check(cost, sol, name):
        assert sol is not None and math.isfinite(cost)
        strat = solution_to_strategy(cfg, sol)
        S = len(strat["layer_partitions"])
        if S > 1:
            assert strat["layer_partitions"][-1] == 8 and sum(strat["layer_partitions"][:-1]) == 8
        assert sum(n * m for n, m in strat["device_assignment"]) == 4
        plain = node.to_dict()
        plain["strategy"] = strat
        yamlconf.dump(plain, tmp_path / f"{name}.yaml")
        cfg2, _ = load_config(name, config_dirs=[tmp_path], check_world_size=False)       # validates the layout
        again = analyze_strategy(cfg2, StageEvaluator(cfg2, OpDatabase(allow_profile=False)))["total"]
        assert again == pytest.approx(cost, rel=1e-6)
        return S

    piped_cost, piped = _enc_dec_pipeline_tune(cfg, ev, None)
    assert check(piped_cost, piped, "piped") >= 2
    cost, sol = inter_stage_tune(cfg, ev)
    check(cost, sol, "best")
    one_cost, _ = inter_stage_tune(cfg, ev, single_stage=True)
    assert cost == pytest.approx(min(one_cost, piped_cost))


def test_middle_stages_are_priced_with_their_own_warm_up_depth(monkeypatch, tmp_path):
    """A four-stage pipeline: stage 1 keeps the activations of two extra micro batches alive, stage 2 of one.
    Both solvers take the options priced for exactly a stage's position when there are some; the tuner's cost
    on a memory-tight four-GPU case equals the analyzer's, which prices every stage at its own depth (the
    four-stage layout itself is forced in the next test)."""
    from mist_b200.tuner.inter_stage import EXACT_MIDDLE
    # options: first, exact middles for positions 1 and 2, a generic middle that must be ignored, last
    kinds = [0, EXACT_MIDDLE + 1, EXACT_MIDDLE + 2, 1, 2]
    layers = [2, 2, 2, 2, 2]
    T = [1.0, 3.0, 2.0, 0.1, 1.0]
    D = [0.0, 0.0, 0.0, 0.0, 0.0]
    for solve in (_solve_native, _solve_python):
        cost, chosen = solve(4, 8, 3, kinds, layers, T, D)
        assert chosen == [0, 1, 2, 4]                          # the cheap generic middle option is not eligible
        assert cost == pytest.approx(sum(T[i] for i in chosen) + 2 * 3.0)
    # without exact options the generic one serves every middle position
    cost, chosen = _solve_python(4, 8, 3, [0, 1, 2], [2, 2, 2], [1.0, 0.5, 1.0], [0.0, 0.0, 0.0])
    assert chosen == [0, 1, 1, 2]

    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_B200")
    from mist_b200.utils import yamlconf
    over = ["experiment=gpt2-1.3b", "model.num_hidden_layers=8", "hardware.num_gpus_per_node=4",
            "training.global_batch_size=16", "training.max_sequence_length=512", "strategy.enabled=false",
            "tuning.tuning_granularity=uniform-pp", "tuning.sample_size=4", "hardware.memory_capacity=6.0"]
    cfg, node = load_config("config", over, check_world_size=False)
    ev = StageEvaluator(cfg, OpDatabase(allow_profile=False))
    cost, sol = inter_stage_tune(cfg, ev)
    assert sol is not None and math.isfinite(cost)
    strat = solution_to_strategy(cfg, sol)
    plain = node.to_dict()
    plain["strategy"] = strat
    yamlconf.dump(plain, tmp_path / "deep.yaml")
    cfg2, _ = load_config("deep", config_dirs=[tmp_path], check_world_size=False)
    again = analyze_strategy(cfg2, StageEvaluator(cfg2, OpDatabase(allow_profile=False)))["total"]
    assert again == pytest.approx(cost, rel=1e-6)


def test_four_stage_pipeline_cost_matches_the_analyzer(monkeypatch):
    """The uniform search restricted to four stages (1 GPU each): what the solver adds up for its chosen
    Pareto points equals what the analyzer computes for the resulting strategy, stage by stage."""
    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_B200")
    from mist_b200.tuner import inter_stage as IS
    over = ["experiment=gpt2-1.3b", "model.num_hidden_layers=8", "hardware.num_gpus_per_node=4",
            "training.global_batch_size=16", "training.max_sequence_length=512", "strategy.enabled=false",
            "tuning.tuning_granularity=uniform-pp", "tuning.sample_size=4"]
    cfg, node = load_config("config", over, check_world_size=False)
    monkeypatch.setattr(IS, "stage_count_candidates", lambda n, L: [4])
    ev = StageEvaluator(cfg, OpDatabase(allow_profile=False))
    cost, sol = IS.inter_stage_tune(cfg, ev)
    assert sol is not None and len(sol[1]) == 4
    strat = solution_to_strategy(cfg, sol)
    plain = node.to_dict()
    plain["strategy"] = strat
    import tempfile
    from mist_b200.utils import yamlconf
    with tempfile.TemporaryDirectory() as d:
        yamlconf.dump(plain, os.path.join(d, "four.yaml"))
        cfg2, _ = load_config("four", config_dirs=[d], check_world_size=False)
    again = analyze_strategy(cfg2, StageEvaluator(cfg2, OpDatabase(allow_profile=False)))["total"]
    assert again == pytest.approx(cost, rel=1e-6)


def test_tuned_configurations_stay_within_tolerance_of_their_measured_runs(monkeypatch):
    """Regression harness on the shipped tuned strategies (measured on 8 x B200): the installed cost model
    prices each of them within 10 % of the measured iteration time and 5 % of the measured peak memory, and
    reproduces the predictions recorded beside the measurements."""
    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_B200")
    import importlib.util
    import json
    root = os.path.join(os.path.dirname(__file__), "..", "benchmark", "mist_b200", "tuned_configs")
    spec = importlib.util.spec_from_file_location("tuned_accuracy", os.path.join(root, "test_performance_accuracy.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    folder = os.path.join(root, "b200-180gb")
    rows = mod.report(folder, fresh=True)
    recorded = json.load(open(os.path.join(folder, "expected_summary.json")))
    assert len(rows) == 4
    for r in rows:
        assert abs(r["time_error"]) < 0.10, r
        assert abs(r["memory_error"]) < 0.05, r
        assert r["predicted_s"] == pytest.approx(recorded[r["name"]]["tuned_predicted_s"], rel=5e-3), r


def test_hand_written_b200_workloads_stay_within_tolerance_of_their_measured_runs(monkeypatch):
    """The four 8 x B200 workloads with hand-written strategies: predicted iteration time within 10 % and
    predicted peak memory per stage within 10 % of what the exec entry point measured."""
    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_B200")
    import json
    path = os.path.join(os.path.dirname(__file__), "..", "benchmark", "mist_b200", "prediction-accuracy", "measured_b200.json")
    for w in json.load(open(path))["workloads"]:
        cfg, _ = load_config("config", w["overrides"], check_world_size=False)
        res = analyze_strategy(cfg, StageEvaluator(cfg))
        assert abs(res["total"] / w["measured_s"] - 1.0) < 0.10, (w["name"], res["total"])
        if w["measured_peak_mb"]:
            for (pf, pb), m in zip(res["peak_memories"], w["measured_peak_mb"]):
                assert abs(max(pf, pb) / 2 ** 20 / m - 1.0) < 0.10, (w["name"], pf, pb, m)
