"""Tuning time over model sizes and GPU counts (CPU only).

    python benchmark/mist_b200/benchmark-tuning-time/run.py --models gpt2/1.3b gpt2/2.7b gpt2/7b --gpus 2 4 8

For every (model, GPU count) the tuner searches the full space of the hardware template and the
wall time, the number of strategies it scored and the best predicted iteration time are written
to ``tuning_time.json`` / printed as a table (reference: benchmark/mist/benchmark-tuning-time/run.py,
which times the same call for its paper's tuning-time figure).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
BENCH = os.path.dirname(HERE)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--models", nargs="+", default=["gpt2/1.3b", "gpt2/2.7b", "gpt2/7b"])
    ap.add_argument("--gpus", nargs="+", type=int, default=[2, 4, 8])
    ap.add_argument("--experiment", default="template-b200")
    ap.add_argument("--batch-per-gpu", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--out", default="tuning_time_results")
    args = ap.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)
    rows = []
    for model in args.models:
        for m in args.gpus:
            tag = f"{model.replace('/', '-')}-m{m}"
            out = os.path.join(args.out, tag)
            cmd = [sys.executable, os.path.join(BENCH, "tune", "tune_one_case.py"), f"experiment={args.experiment}",
                   f"model={model}", "hardware.num_nodes=1", f"hardware.num_gpus_per_node={m}",
                   f"training.global_batch_size={args.batch_per_gpu * m}", f"training.max_sequence_length={args.seq_len}",
                   "strategy.enabled=false", f"output_dir={out}", f"+output_path={os.path.join(out, 'best.yaml')}"]
            t0 = time.perf_counter()
            r = subprocess.run(cmd, capture_output=True, text=True)
            wall = time.perf_counter() - t0
            row = {"model": model, "gpus": m, "wall_s": round(wall, 2), "ok": r.returncode == 0}
            for line in r.stdout.splitlines():
                if line.startswith("Best cost:"):
                    row["best_cost_s"] = float(line.split(":")[1])
                elif line.startswith("Tuning time:"):
                    row["tuning_time_s"] = float(line.split(":")[1].split()[0])
                elif line.startswith("Best solution:"):
                    row["solution"] = line.split(":", 1)[1].strip()
            if not row["ok"]:
                row["error"] = (r.stderr or r.stdout)[-400:]
            rows.append(row)
            print(row, flush=True)
    with open(os.path.join(args.out, "tuning_time.json"), "w") as f:
        json.dump(rows, f, indent=1)
    try:
        from tabulate import tabulate
        print(tabulate([[r["model"], r["gpus"], r.get("tuning_time_s"), r.get("best_cost_s")] for r in rows],
                       headers=["model", "gpus", "tuning time (s)", "predicted s / iteration"]))
    except ImportError:
        pass
    return rows


if __name__ == "__main__":
    main()
