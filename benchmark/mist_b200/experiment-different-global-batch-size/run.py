"""Global-batch-size study: tune -> analyze (-> exec) one model on a fixed machine for several
global batch sizes.

    python benchmark/mist_b200/experiment-different-global-batch-size/run.py --model gpt2/2.7b \\
        -n 1 -m 8 --global-batch-sizes 32 64 128 256 --skip-exec

(reference: benchmark/mist/experiment-different-global-batch-size/run.py and scripts/run.sh.)
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BENCH = os.path.dirname(HERE)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="gpt2/2.7b")
    ap.add_argument("--experiment", default="template-b200")
    ap.add_argument("-n", "--nnodes", type=int, default=1)
    ap.add_argument("-m", "--nproc-per-node", type=int, default=8)
    ap.add_argument("--global-batch-sizes", nargs="+", type=int, default=[32, 64, 128, 256])
    ap.add_argument("--seq-len", "-s", type=int, default=2048)
    ap.add_argument("--spaces", nargs="*", default=["mist"])
    ap.add_argument("--skip-exec", action="store_true")
    ap.add_argument("--out", default="gbs_results")
    args = ap.parse_args(argv)
    spec = importlib.util.spec_from_file_location("mist_b200_experiment_run", os.path.join(BENCH, "experiment", "run.py"))
    run = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(run)
    table = {}
    for gbs in args.global_batch_sizes:
        out = os.path.join(args.out, f"b{gbs}")
        run.main(["--model", args.model, "--experiment", args.experiment, "-n", str(args.nnodes), "-m",
                  str(args.nproc_per_node), "--global-batch-size", str(gbs), "--seq-len", str(args.seq_len), "--spaces",
                  *args.spaces, "--out", out] + (["--skip-exec"] if args.skip_exec else []))
        with open(os.path.join(out, "summary.json")) as f:
            table[gbs] = json.load(f)
    with open(os.path.join(args.out, "summary.json"), "w") as f:
        json.dump(table, f, indent=2)
    tokens = lambda g: g * args.seq_len          # noqa: E731
    for gbs, spaces in table.items():
        for space, s in spaces.items():
            t = s.get("analyzed_total_cost")
            thr = f"{tokens(gbs) / float(t):.0f} tokens/s predicted" if t else "-"
            print(f"gbs {gbs:>5} {space:>12}: tuned {s.get('tuning_best_cost', '-')} s ({thr}), measured "
                  f"{s.get('exec_total_cost', '-')} s")
    return table


if __name__ == "__main__":
    main(sys.argv[1:])
