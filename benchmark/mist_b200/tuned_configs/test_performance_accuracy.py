"""Predicted against measured iteration time and peak memory of the tuned configurations of one folder.

    python benchmark/mist_b200/tuned_configs/test_performance_accuracy.py [b200-180gb] [--reanalyze]

Reads ``<folder>/expected_summary.json`` (measured on the machine the folder is named for) and prints, per
configuration, predicted / measured time and memory with their relative errors, then the mean absolute errors.
``--reanalyze`` prices every configuration again with the installed cost model instead of using the recorded
predictions (CPU only; set ``FAKE_DEVICE_NAME`` to the GPU the operator database was profiled on).

Counterpart in the reference: benchmark/mist/tuned_configs/test_performance_accuracy.py (analyzed / executed
ratios over its ``expected_summary.json``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def reanalyze(folder: str, name: str):
    from mist_b200.analyzer.stage_evaluator import StageEvaluator, analyze_strategy
    from mist_b200.config import load_config
    path = os.path.join(folder, name + ".yaml")
    cfg, _ = load_config(os.path.basename(name), config_dirs=[os.path.dirname(path)], check_world_size=False)
    res = analyze_strategy(cfg, StageEvaluator(cfg))
    return float(res["total"]), max(max(p) for p in res["peak_memories"]) / 2 ** 20


def report(folder: str, fresh: bool = False):
    with open(os.path.join(folder, "expected_summary.json")) as f:
        expected = json.load(f)
    rows = []
    for name, e in expected.items():
        pred_s, pred_mb = e.get("tuned_predicted_s"), e.get("tuned_predicted_peak_mb")
        if fresh:
            pred_s, pred_mb = reanalyze(folder, name)
        meas_s, meas_mb = e.get("tuned_measured_s"), e.get("tuned_measured_peak_mb")
        rows.append(dict(name=name, predicted_s=pred_s, measured_s=meas_s,
                         time_error=None if not meas_s else pred_s / meas_s - 1.0,
                         predicted_mb=pred_mb, measured_mb=meas_mb,
                         memory_error=None if not (meas_mb and pred_mb) else pred_mb / meas_mb - 1.0))
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("folder", nargs="?", default="b200-180gb")
    ap.add_argument("--reanalyze", action="store_true")
    args = ap.parse_args(argv)
    folder = args.folder if os.path.isabs(args.folder) else os.path.join(HERE, args.folder)
    rows = report(folder, args.reanalyze)
    te, me = [], []
    for r in rows:
        t = "   n/a" if r["time_error"] is None else f"{100 * r['time_error']:+6.1f} %"
        m = "   n/a" if r["memory_error"] is None else f"{100 * r['memory_error']:+6.1f} %"
        print(f"{r['name']:52s} {r['predicted_s']:8.4f} s / {r['measured_s'] or float('nan'):8.4f} s {t}   "
              f"{(r['predicted_mb'] or 0) / 1024:6.1f} GB / {(r['measured_mb'] or 0) / 1024:6.1f} GB {m}")
        if r["time_error"] is not None:
            te.append(abs(r["time_error"]))
        if r["memory_error"] is not None:
            me.append(abs(r["memory_error"]))
    if te:
        print(f"mean absolute error: time {100 * sum(te) / len(te):.1f} %, memory {100 * sum(me) / max(len(me), 1):.1f} %")
    return 0


if __name__ == "__main__":
    sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..", "..")))
    sys.exit(main())
