"""analyze: predicted iteration latency and per-stage peak memory of a fixed strategy.

    python benchmark/mist_b200/analysis/run.py --config-name test-small-base

Prints and records (``summary.json``) the total latency, per-stage stable / delta latencies
and per-stage peak forward / backward memory (reference: benchmark/mist/analysis/run.py:
37-243; output keys :236-241).  Runs on CPU; operator latencies come from the database of
the target GPU (``FAKE_DEVICE_NAME`` or the ``hardware.gpu_type`` of the configuration).
With ``MIST_B200_PROFILE_OPS=1`` on a machine that has that GPU, operators the database does
not know yet are measured and added (``MIST_B200_OP_CACHE`` chooses where);
``MIST_B200_PROFILE_OPS=2`` also measures again the entries that carry no SM clock yet.
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from common import load_from_cli, output_dir  # noqa: E402

from mist_b200.analyzer.stage_evaluator import StageEvaluator, analyze_strategy  # noqa: E402
from mist_b200.node_database.database import OpDatabase  # noqa: E402
from mist_b200.utils.summary import fmt_cost, fmt_costs, fmt_memories, update_summary  # noqa: E402


def analyze(cfg, cache_dir=None):
    assert cfg.strategy is not None, "analyze needs strategy.enabled=true"
    # MIST_B200_PROFILE_OPS=1 (on a machine with the target GPU): operators missing from the
    # database are timed on the device and stored, so later CPU-only runs find them.
    mode = os.environ.get("MIST_B200_PROFILE_OPS", "0")
    profile_ops = mode in ("1", "2")
    if cfg.hardware.gpu_type and not os.environ.get("FAKE_DEVICE_NAME") and not profile_ops:
        os.environ["FAKE_DEVICE_NAME"] = str(cfg.hardware.gpu_type)
    ev = StageEvaluator(cfg, OpDatabase(allow_profile=profile_ops, refresh_unclocked=(mode == "2")), cache_dir=cache_dir)
    return analyze_strategy(cfg, ev)


def main(argv=None):
    cfg, node = load_from_cli(argv, check_world_size=False)
    out = output_dir(node)
    res = analyze(cfg, cache_dir=os.path.join(out, "model_tracing_and_analysis_results"))
    print(f"Total latency: {res['total']:.6f}")
    print(f"Stage stable latencies: {fmt_costs(res['stable'])}")
    print(f"Stage delta latencies: {fmt_costs(res['delta'])}")
    for s, (pf, pb) in enumerate(res["peak_memories"]):
        print(f"Stage {s} peak fwd memory: {pf / (1 << 20):.3f} MB, peak bwd memory: {pb / (1 << 20):.3f} MB")
    update_summary(os.path.join(out, "summary.json"), {
        "analyzed_total_cost": fmt_cost(res["total"]),
        "analyzed_stage_stable_latencies": fmt_costs(res["stable"]),
        "analyzed_stage_delta_latencies": fmt_costs(res["delta"]),
        "analyzed_stage_peak_memories": fmt_memories([max(p) for p in res["peak_memories"]]),
    })
    return res


if __name__ == "__main__":
    main()
