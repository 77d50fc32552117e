"""Collects the ``summary.json`` files under a results folder into one table.

    python benchmark/scripts/collect_single_node_results.py results/ --csv results.csv

One row per run directory (or per top-level key of an orchestrated run): tuner cost and time,
analyzer prediction, measured iteration time, throughput, peak memory, and the prediction error
where both numbers exist (reference: benchmark/scripts/collect_single_node_results_v1.py, which
tabulates the same keys).
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import sys
from typing import Dict, List

COLUMNS = ["run", "tuning_best_cost", "tuning_time", "analyzed_total_cost", "exec_total_cost", "exec_throughput",
           "exec_stage_peak_allocated_memories", "prediction_error_pct"]


def _rows_of(path: str, summary: Dict) -> List[Dict]:
    entries = [("", summary)] if any(k in summary for k in COLUMNS) else \
        [(k, v) for k, v in summary.items() if isinstance(v, dict)]
    rows = []
    for key, s in entries:
        row = {"run": os.path.join(path, key) if key else path}
        for c in COLUMNS[1:-1]:
            row[c] = s.get(c, "")
        try:
            pred, meas = float(s["analyzed_total_cost"]), float(s["exec_total_cost"])
            row["prediction_error_pct"] = f"{100.0 * (pred - meas) / meas:+.1f}"
        except (KeyError, ValueError, ZeroDivisionError):
            row["prediction_error_pct"] = ""
        rows.append(row)
    return rows


def collect(root: str) -> List[Dict]:
    rows: List[Dict] = []
    for d, _, files in sorted(os.walk(root)):
        if "summary.json" in files:
            with open(os.path.join(d, "summary.json")) as f:
                rows.extend(_rows_of(os.path.relpath(d, root), json.load(f)))
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("root")
    ap.add_argument("--csv", default=None)
    args = ap.parse_args(argv)
    rows = collect(args.root)
    if not rows:
        print("no summary.json under", args.root)
        return rows
    try:
        from tabulate import tabulate
        print(tabulate([[r[c] for c in COLUMNS] for r in rows], headers=COLUMNS))
    except ImportError:
        print("\t".join(COLUMNS))
        for r in rows:
            print("\t".join(str(r[c]) for c in COLUMNS))
    if args.csv:
        with open(args.csv, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=COLUMNS)
            w.writeheader()
            w.writerows(rows)
    return rows


if __name__ == "__main__":
    main(sys.argv[1:])
