"""Tuning time over model sizes, GPU counts and search spaces of growing size (CPU only).

    python benchmark/mist_b200/benchmark-tuning-time/run.py --models gpt2/22b -n 4 --gpus 8
    python benchmark/mist_b200/benchmark-tuning-time/run.py --models gpt2/1.3b gpt2/7b --gpus 4 8 --spaces full

For every (model, nodes x GPUs, search space) the tuner runs once; wall time, the tuner's own
timer and the best predicted iteration time go to ``tuning_time.json`` and a table.  The search
spaces grow step by step: ``base`` (parallelism and micro batch only), ``+ckpt`` (activation
checkpointing), ``+zero`` (ZeRO-2/3), ``full`` (host offloading of weights, gradients, optimizer
state and activations) (reference: benchmark/mist/benchmark-tuning-time/run.py, which times the
tuner the same way, GPT-22B on 4 x 8 GPUs, while enlarging the space).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

SPACES = {
    "base": ["tuning.zero_2_and_3_enabled=false", "tuning.activation_checkpointing_tuning_enabled=false",
             "tuning.state_offloading_enabled=false", "tuning.activation_offloading_enabled=false"],
    "+ckpt": ["tuning.zero_2_and_3_enabled=false", "tuning.activation_checkpointing_tuning_enabled=true",
              "tuning.state_offloading_enabled=false", "tuning.activation_offloading_enabled=false"],
    "+zero": ["tuning.zero_2_and_3_enabled=true", "tuning.activation_checkpointing_tuning_enabled=true",
              "tuning.state_offloading_enabled=false", "tuning.activation_offloading_enabled=false"],
    "full": ["tuning.zero_2_and_3_enabled=true", "tuning.activation_checkpointing_tuning_enabled=true",
             "tuning.state_offloading_enabled=true", "tuning.activation_offloading_enabled=true"],
}

HERE = os.path.dirname(os.path.abspath(__file__))
BENCH = os.path.dirname(HERE)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--models", nargs="+", default=["gpt2/1.3b", "gpt2/2.7b", "gpt2/7b"])
    ap.add_argument("--gpus", nargs="+", type=int, default=[2, 4, 8], help="GPUs per node")
    ap.add_argument("-n", "--nnodes", type=int, default=1)
    ap.add_argument("--spaces", nargs="+", default=list(SPACES), choices=list(SPACES))
    ap.add_argument("--experiment", default="template-b200")
    ap.add_argument("--batch-per-gpu", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--out", default="tuning_time_results")
    args = ap.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)
    rows = []
    for model in args.models:
        for m, space in [(m, sp) for m in args.gpus for sp in args.spaces]:
            tag = f"{model.replace('/', '-')}-n{args.nnodes}-m{m}-{space.strip('+')}"
            out = os.path.join(args.out, tag)
            cmd = [sys.executable, os.path.join(BENCH, "tune", "tune_one_case.py"), f"experiment={args.experiment}",
                   f"model={model}", f"hardware.num_nodes={args.nnodes}", f"hardware.num_gpus_per_node={m}",
                   f"training.global_batch_size={args.batch_per_gpu * m * args.nnodes}",
                   f"training.max_sequence_length={args.seq_len}", "strategy.enabled=false", *SPACES[space],
                   f"output_dir={out}", f"+output_path={os.path.join(out, 'best.yaml')}"]
            t0 = time.perf_counter()
            r = subprocess.run(cmd, capture_output=True, text=True)
            wall = time.perf_counter() - t0
            row = {"model": model, "nodes": args.nnodes, "gpus": m, "space": space, "wall_s": round(wall, 2),
                   "ok": r.returncode == 0}
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
        print(tabulate([[r["model"], f"{r['nodes']} x {r['gpus']}", r["space"], r.get("tuning_time_s"), r.get("best_cost_s")]
                        for r in rows],
                       headers=["model", "nodes x gpus", "space", "tuning time (s)", "predicted s / iteration"]))
    except ImportError:
        pass
    return rows


if __name__ == "__main__":
    main()
