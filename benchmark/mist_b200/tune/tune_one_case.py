"""tune: search the strategy space and write the best strategy as a YAML that analyze and
exec consume.

    python benchmark/mist_b200/tune/tune_one_case.py --config-name test-small-base +output_path=best.yaml

(reference: benchmark/mist/tune/tune_one_case.py:104-451; best-solution YAML :62-101,
summary keys :445-448).
"""
from __future__ import annotations

import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from common import load_from_cli, output_dir  # noqa: E402

from mist_b200.analyzer.stage_evaluator import StageEvaluator  # noqa: E402
from mist_b200.node_database.database import OpDatabase  # noqa: E402
from mist_b200.tuner.inter_stage import inter_stage_tune, solution_to_strategy  # noqa: E402
from mist_b200.utils import yamlconf  # noqa: E402
from mist_b200.utils.summary import update_summary  # noqa: E402


def tune(cfg, cache_dir=None, verbose=False):
    assert cfg.tuning is not None, "tune needs tuning.enabled=true"
    if cfg.hardware.gpu_type and not os.environ.get("FAKE_DEVICE_NAME"):
        os.environ["FAKE_DEVICE_NAME"] = str(cfg.hardware.gpu_type)
    ev = StageEvaluator(cfg, OpDatabase(allow_profile=False), cache_dir=cache_dir)
    per_node = cfg.hardware.num_gpus_per_node
    tps = [1] if cfg.get("disable_tp_tuning", False) else [t for t in (1, 2, 4, 8) if t <= per_node]
    best = (float("inf"), None)
    for tp in tps:
        cost, sol = inter_stage_tune(cfg, ev, cache_dir=None, tp=tp, verbose=verbose)
        if sol is not None and cost < best[0]:
            best = (cost, sol)
    return best


def main(argv=None):
    cfg, node = load_from_cli(argv, check_world_size=False)
    node["strategy"]["enabled"] = False
    out = output_dir(node)
    t0 = time.time()
    cost, sol = tune(cfg, cache_dir=os.path.join(out, "model_tracing_and_analysis_results"),
                     verbose=not os.environ.get("DISABLE_TQDM"))
    dt = time.time() - t0
    if sol is None:
        print("No feasible strategy found")
        return None
    print(f"Best cost: {cost:.8f}")
    print(f"Best solution: {sol}")
    print(f"Tuning time: {dt:.2f} s")
    strategy = solution_to_strategy(cfg, sol)
    plain = node.to_dict()
    plain["strategy"] = strategy
    out_path = node.get("output_path") or os.path.join(out, "best_config.yaml")
    yamlconf.dump(plain, out_path)
    print(f"Wrote {out_path}")
    update_summary(os.path.join(out, "summary.json"), {
        "tuning_best_cost": f"{cost:.4f}", "tuning_best_solution": str(sol), "tuning_time": f"{dt:.2f}"})
    return cost, sol


if __name__ == "__main__":
    main()
