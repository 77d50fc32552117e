"""Analyzer accuracy: walks ``summary.json`` files that hold both analyzed and executed
numbers and reports the mean absolute relative error of latency (raw, and after removing
the mean offset as the reference does) and of peak memory (reference:
benchmark/mist/prediction-accuracy/get_mem_and_latency_accuracy.py:68-76)."""
from __future__ import annotations

import json
import os
import re
import sys


def _nums(s):
    return [float(x) for x in re.findall(r"[-+]?\d*\.?\d+", str(s))]


def collect(root):
    rows = []
    for d, _, files in os.walk(root):
        if "summary.json" not in files:
            continue
        with open(os.path.join(d, "summary.json")) as f:
            s = json.load(f)
        for key, val in (s.items() if "analyzed_total_cost" not in s else [("", s)]):
            if not isinstance(val, dict) or "analyzed_total_cost" not in val or "exec_total_cost" not in val:
                continue
            rows.append({"name": os.path.join(d, key), "pred": float(val["analyzed_total_cost"]),
                         "meas": float(val["exec_total_cost"]),
                         "pred_mem": _nums(val.get("analyzed_stage_peak_memories", "")),
                         "meas_mem": _nums(val.get("exec_stage_peak_allocated_memories", ""))})
    return rows


def collect_measured(path):
    """Rows for a file of measured runs (``measured_b200.json`` beside this script): every workload is priced
    again with the installed cost model (CPU only; set ``FAKE_DEVICE_NAME`` to the GPU of the operator database)."""
    sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..")))
    from mist_b200.analyzer.stage_evaluator import StageEvaluator, analyze_strategy
    from mist_b200.config import load_config
    rows = []
    with open(path) as f:
        workloads = json.load(f)["workloads"]
    for w in workloads:
        cfg, _ = load_config("config", w["overrides"], check_world_size=False)
        res = analyze_strategy(cfg, StageEvaluator(cfg))
        rows.append({"name": w["name"], "pred": float(res["total"]), "meas": float(w["measured_s"]),
                     "pred_mem": [max(p) / 2 ** 20 for p in res["peak_memories"]] if w.get("measured_peak_mb") else [],
                     "meas_mem": [float(m) for m in (w.get("measured_peak_mb") or [])]})
    return rows


def main(argv=None):
    """``<folder>``: walk its ``summary.json`` files; ``<file>.json``: a list of measured runs to price again."""
    root = (argv or sys.argv[1:] or ["."])[0]
    rows = collect_measured(root) if root.endswith(".json") else collect(root)
    if not rows:
        print("no summary.json with both analyzed and exec results under", root)
        return
    rel = [(r["pred"] - r["meas"]) / r["meas"] for r in rows]
    mean = sum(rel) / len(rel)
    print(f"{len(rows)} cases")
    for r, e in zip(rows, rel):
        print(f"  {r['name']}: predicted {r['pred']:.4f} s  measured {r['meas']:.4f} s  error {100 * e:+.1f} %")
    print(f"latency: mean abs rel err {100 * sum(abs(e) for e in rel) / len(rel):.2f} %, "
          f"after removing the mean offset {100 * sum(abs(e - mean) for e in rel) / len(rel):.2f} %")
    mem = [abs(p - m) / m for r in rows for p, m in zip(r["pred_mem"], r["meas_mem"]) if m > 0]
    if mem:
        print(f"memory : mean abs rel err {100 * sum(mem) / len(mem):.2f} %")


if __name__ == "__main__":
    main()
