"""Configuration composition and validation (CPU)."""
import os

import pytest

from mist_b200.config import (MistConfig, StageStrategy, StrategyConfig, ZeroLevel, expand_comm_table,
                              load_config)
from mist_b200.utils import yamlconf


def test_packaged_tree_loads_every_experiment():
    root = os.path.join(os.path.dirname(__file__), "..", "mist_b200", "configs", "experiment")
    names = [f[:-5] for f in os.listdir(root) if f.endswith(".yaml") and not f.startswith("template")]
    assert len(names) >= 10
    for n in names:
        cfg, _ = load_config("config", [f"experiment={n}"], check_world_size=False)
        assert cfg.model.hidden_size % cfg.model.num_attention_heads == 0
        assert cfg.strategy.num_stages == len(cfg.strategy.layer_partitions)


def test_defaults_interpolation_and_overrides():
    cfg, node = load_config("config", ["experiment=gpt2-1.3b", "training.global_batch_size=128",
                                       "strategy.stage_strategies=[[8,8,1,0,0,1,0,0,0,0]]",
                                       "strategy.pre_post_strategy_array=[8,8,1,0,0,1,0,0,0,0]",
                                       "+output_path=/tmp/x.yaml"], check_world_size=False)
    assert cfg.strategy.layer_partitions == [24]          # ${model.num_hidden_layers}
    assert node.output_path == "/tmp/x.yaml"
    assert cfg.training.global_batch_size == 128
    assert cfg.model.max_position_embeddings == cfg.training.max_sequence_length
    assert cfg.overlap is True and cfg.get("nonexistent", 7) == 7


def test_small_base_matches_kick_the_tires_case():
    cfg, _ = load_config("test-small-base", check_world_size=False)
    s = cfg.strategy.stage(0)
    assert (s.micro_batch_size, s.dp, s.tp) == (8, 2, 1) and s.zero is ZeroLevel.OPT
    assert cfg.strategy.gradient_accumulation_steps == 2 and cfg.strategy.gradient_checkpointing == [24]
    assert abs(cfg.hardware.memory_capacity - 22.488 * 0.88) < 1e-9
    assert len(cfg.hardware.gpu_gpu_comm_params) == 32 and len(cfg.hardware.interference_model_params) == 28
    assert not cfg.model.use_flash_attn


def test_strategy_validation_errors():
    with pytest.raises(AssertionError):
        load_config("test-small-base", ["strategy.gradient_accumulation_steps=3"], check_world_size=False)
    with pytest.raises(AssertionError):
        load_config("test-small-base", ["strategy.layer_partitions=[23]"], check_world_size=False)
    with pytest.raises(AssertionError):
        load_config("test-small-base", ["strategy.stage_strategies=[[8,2,2,0,0,1,0,0,0,0]]"], check_world_size=False)
    with pytest.raises(AssertionError):
        StrategyConfig([24], [(1, 2)], [0], 2, [[8, 2, 1, 0, 0, 1, 0, 0, 0]])   # 9 elements


def test_zero_level_and_vector_roundtrip():
    s = StageStrategy.from_vector([4, 2, 1, 1, 1, 1, 0.5, 0, 0.25, 0])
    assert s.zero is ZeroLevel.FULL and s.to_vector()[6] == 0.5
    assert StageStrategy.from_vector([4, 2, 1, 0, 1, 1, 0, 0, 0, 0]).zero is ZeroLevel.OPT_GRAD
    assert StageStrategy.from_vector([4, 2, 1, 0, 0, 0, 0, 0, 0, 0]).zero is ZeroLevel.NONE


def test_world_size_check(monkeypatch):
    monkeypatch.setenv("WORLD_SIZE", "4")
    with pytest.raises(AssertionError):
        load_config("test-small-base")
    load_config("test-small-base", check_world_size=False)


def test_legacy_comm_table_expansion():
    t = expand_comm_table([1.0, 0.1, 2.0, 0.2, 3.0, 0.3], [7.0, 0.0])
    assert len(t) == 32 and t[2:4] == [1.0, 0.1] and t[6:8] == [3.0, 0.3] and t[8:10] == [7.0, 0.0]


def test_yaml_roundtrip(tmp_path):
    cfg, node = load_config("test-small", check_world_size=False)
    p = tmp_path / "out.yaml"
    yamlconf.dump(node, p)
    cfg2, _ = load_config("out", config_dirs=[tmp_path], check_world_size=False)
    assert cfg2.strategy.stage_strategies == cfg.strategy.stage_strategies
    assert cfg2.strategy.num_stages == 2


def test_memory_snapshot_summary():
    from mist_b200.tools.parse_memory_snapshot import summarise
    snap = {"segments": [
        {"segment_type": "large", "total_size": 100, "allocated_size": 60, "active_size": 60, "blocks": [
            {"state": "active_allocated", "size": 60, "requested_size": 50,
             "frames": [{"filename": "/x/engine.py", "line": 12, "name": "alloc"}]},
            {"state": "inactive", "size": 40}]},
        {"segment_type": "small", "total_size": 10, "allocated_size": 10, "active_size": 10, "blocks": [
            {"state": "active_allocated", "size": 10}]}]}
    r = summarise(snap, top=1)
    assert r["reserved"] == 110 and r["allocated"] == 70 and r["largest_free_block"] == 40
    assert r["by_kind"]["large"] == (1, 100, 60)
    assert r["top_blocks"][0][0] == 60 and "engine.py:12" in r["top_blocks"][0][2]


def test_merge_calibration_records(tmp_path):
    import json
    from mist_b200.tools.merge_json_results import main
    a = [{"intra": 2, "inter": 1, "g2g_gbytes": 0.5, "c2g_gbytes": 0.0, "g2c_gbytes": 0.0, "C": 0.0, "latency": 1.0}]
    b = [dict(a[0], latency=2.0), dict(a[0], intra=8)]
    for name, recs in (("a.json", a), ("b.json", b)):
        json.dump(recs, open(tmp_path / name, "w"))
    out = main([str(tmp_path / "a.json"), str(tmp_path / "b.json"), "-o", str(tmp_path / "m.json")])
    assert len(out) == 2 and {(r["intra"], r["latency"]) for r in out} == {(2, 2.0), (8, 1.0)}


def test_collect_results_table(tmp_path):
    import importlib.util
    import json
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("collect", os.path.join(root, "benchmark/scripts/collect_single_node_results.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    (tmp_path / "a").mkdir()
    json.dump({"analyzed_total_cost": "1.10", "exec_total_cost": "1.00", "exec_throughput": "10.0"}, open(tmp_path / "a" / "summary.json", "w"))
    (tmp_path / "b").mkdir()
    json.dump({"mist": {"tuning_best_cost": "2.0", "analyzed_total_cost": "2.0"}}, open(tmp_path / "b" / "summary.json", "w"))
    rows = mod.main([str(tmp_path), "--csv", str(tmp_path / "out.csv")])
    assert len(rows) == 2 and rows[0]["prediction_error_pct"] == "+10.0" and rows[1]["run"].endswith("mist")
    assert (tmp_path / "out.csv").read_text().startswith("run,")


def test_named_pre_post_strategies_set_the_redundancy_flags():
    """`preset` takes the array, the reference's named choices map to its flag triples
    (mist/analyzer/batched_module_analyzer.py:799-839) on the stage's own mesh, `heuristic` follows the stage."""
    cfg, _ = load_config("config", ["experiment=b200-gpt3-2.7b-dp8-zero2"], check_world_size=False)
    st = cfg.strategy
    assert st.pre_post_strategy == "preset" and tuple(st.pre_post_vector(0)) == tuple(st.pre_post_strategy_array)
    b, dp, tp = st.stage_strategies[0][:3]
    for name, flags in (("dp", (0, 0, 1)), ("intra-node-tp-with-ore", (0, 1, 1)), ("intra-node-tp-without-ore", (0, 1, 0))):
        st.pre_post_strategy = name
        v = st.pre_post_vector(0)
        assert tuple(v[:3]) == (b, dp, tp) and tuple(int(x) for x in v[3:6]) == flags and not any(v[6:])
    st.pre_post_strategy = "heuristic"
    assert st.pre_post_vector(0) is None
