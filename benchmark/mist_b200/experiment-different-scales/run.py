"""Weak-scaling study: tune -> analyze (-> exec) a model family over growing model sizes and
GPU counts, global batch = ``factor`` x GPUs.

    python benchmark/mist_b200/experiment-different-scales/run.py --family gpt2 \\
        --cases 1.3b:1x2 2.7b:1x4 7b:1x8 --skip-exec

Each case ``size:NxM`` runs the orchestrator (``benchmark/mist_b200/experiment/run.py``) for that
model on ``N`` nodes of ``M`` GPUs; the per-case summaries are merged into one table
(reference: benchmark/mist/experiment-different-scales/run.py and its scripts/base.sh, which
loop the same way over (hosts, devices, model size)).
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BENCH = os.path.dirname(HERE)


def _orchestrator():
    spec = importlib.util.spec_from_file_location("mist_b200_experiment_run", os.path.join(BENCH, "experiment", "run.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--family", default="gpt2")
    ap.add_argument("--cases", nargs="+", default=["1.3b:1x2", "2.7b:1x4", "7b:1x8"])
    ap.add_argument("--experiment", default="template-b200")
    ap.add_argument("--global-batch-size-factor", "-f", type=int, default=8)
    ap.add_argument("--seq-len", "-s", type=int, default=2048)
    ap.add_argument("--spaces", nargs="*", default=["mist"])
    ap.add_argument("--skip-exec", action="store_true")
    ap.add_argument("--out", default="scales_results")
    args = ap.parse_args(argv)
    run = _orchestrator()
    table = {}
    for case in args.cases:
        size, shape = case.split(":")
        n, m = (int(x) for x in shape.lower().split("x"))
        out = os.path.join(args.out, f"{args.family}-{size}-n{n}-m{m}")
        argv2 = ["--model", f"{args.family}/{size}", "--experiment", args.experiment, "-n", str(n), "-m", str(m),
                 "--global-batch-size", str(args.global_batch_size_factor * n * m), "--seq-len", str(args.seq_len),
                 "--spaces", *args.spaces, "--out", out] + (["--skip-exec"] if args.skip_exec else [])
        run.main(argv2)
        with open(os.path.join(out, "summary.json")) as f:
            table[case] = json.load(f)
    with open(os.path.join(args.out, "summary.json"), "w") as f:
        json.dump(table, f, indent=2)
    for case, spaces in table.items():
        for space, s in spaces.items():
            print(f"{case:>12} {space:>14}: tuned {s.get('tuning_best_cost', '-')} s, analyzed "
                  f"{s.get('analyzed_total_cost', '-')} s, measured {s.get('exec_total_cost', '-')} s")
    return table


if __name__ == "__main__":
    main(sys.argv[1:])
