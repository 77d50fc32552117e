"""Experiment orchestration: tune -> analyze -> exec for a set of search-space ablations
and collect everything into one ``summary.json`` per run directory.

    python benchmark/mist_b200/experiment/run.py --model gpt2/2.7b -n 1 -m 8 --global-batch-size 64 \
        --spaces mist no-offload zero1-only

Each space is a set of configuration overrides; identical best solutions are executed once
(reference: benchmark/mist/experiment/run.py:92-115 choices, :147-179 command lines,
:255-278 multi-node pdsh launch, :309-335 CLI).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BENCH = os.path.dirname(HERE)

SPACES = {
    "mist": [],
    "no-offload": ["tuning.state_offloading_enabled=false", "tuning.activation_offloading_enabled=false"],
    "no-act-offload": ["tuning.activation_offloading_enabled=false"],
    "zero1-only": ["tuning.zero_2_and_3_enabled=false"],
    "no-ckpt-tuning": ["tuning.activation_checkpointing_tuning_enabled=false"],
    "no-pp": ["tuning.tuning_granularity=no-pp"],
    "uniform-pp": ["tuning.tuning_granularity=uniform-pp"],
    "tp-tuning": ["disable_tp_tuning=false"],
}


def sh(cmd, **kw):
    print("$", " ".join(cmd), flush=True)
    return subprocess.run(cmd, **kw)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt2/2.7b")
    ap.add_argument("--experiment", default="template-b200")
    ap.add_argument("-n", "--nnodes", type=int, default=1)
    ap.add_argument("-m", "--nproc-per-node", type=int, default=8)
    ap.add_argument("--global-batch-size", type=int, default=64)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--spaces", nargs="*", default=["mist"])
    ap.add_argument("--out", default="experiment_results")
    ap.add_argument("--skip-exec", action="store_true", help="tune + analyze only (no GPUs needed)")
    ap.add_argument("--skip-tune", action="store_true",
                    help="reuse the best_config.yaml an earlier run left in the output directory (exec only)")
    ap.add_argument("--disable-flash-attn", action="store_true", help="materialised attention scores instead of flash attention")
    ap.add_argument("--hosts", default=None, help="comma separated worker hosts for multi-node exec (pdsh)")
    ap.add_argument("--master-addr", default=None, help="rendezvous address (default: the first host, or 127.0.0.1)")
    ap.add_argument("--master-port", type=int, default=29533)
    args = ap.parse_args(argv)
    base = [f"experiment={args.experiment}", f"model={args.model}", f"hardware.num_nodes={args.nnodes}",
            f"hardware.num_gpus_per_node={args.nproc_per_node}", f"training.global_batch_size={args.global_batch_size}",
            f"training.max_sequence_length={args.seq_len}", "strategy.enabled=false",
            f"model.use_flash_attn={'false' if args.disable_flash_attn else 'true'}"]
    seen = {}
    for space in args.spaces:
        out = os.path.abspath(os.path.join(args.out, space))
        os.makedirs(out, exist_ok=True)
        best = os.path.join(out, "best_config.yaml")
        if not args.skip_tune:
            r = sh([sys.executable, os.path.join(BENCH, "tune", "tune_one_case.py"), *base, *SPACES[space],
                    f"output_dir={out}", f"+output_path={best}"])
            if r.returncode != 0:
                continue
            sh([sys.executable, os.path.join(BENCH, "analysis", "run.py"), "--config-name", "best_config", "-cd", out,
                f"output_dir={out}"])
        if not os.path.exists(best):
            print(f"[{space}] no tuned configuration at {best}")
            continue
        with open(os.path.join(out, "summary.json")) as f:
            sol = json.load(f).get("tuning_best_solution")
        if sol in seen:
            print(f"[{space}] same solution as [{seen[sol]}], not executed again")
            continue
        seen[sol] = space
        if args.skip_exec:
            continue
        multi = args.nnodes > 1 and args.hosts
        master = args.master_addr or (args.hosts.split(",")[0] if multi else "127.0.0.1")
        launcher = [sys.executable, "-m", "torch.distributed.run", f"--nnodes={args.nnodes}",
                    f"--nproc-per-node={args.nproc_per_node}", "--master-addr", master,
                    "--master-port", str(args.master_port)]
        if multi:
            launcher.append("--node-rank=%n")      # pdsh replaces %n by the host's position in the list
        cmd = launcher + [os.path.join(BENCH, "exec", "benchmark_one_case.py"), "--config-name", "best_config", "-cd", out,
                          f"output_dir={out}"]
        if multi:
            # the output directory must be on storage every host sees (the tuned configuration is read
            # there); one ssh fan-out runs the same launcher on every host
            sh(["pdsh", "-S", "-R", "ssh", "-w", args.hosts, f"cd {os.getcwd()} && NCCL_ASYNC_ERROR_HANDLING=1 " + " ".join(cmd)])
        else:
            sh(cmd)
    merged = {}
    for space in args.spaces:
        p = os.path.join(args.out, space, "summary.json")
        if os.path.exists(p):
            with open(p) as f:
                merged[space] = json.load(f)
    with open(os.path.join(args.out, "summary.json"), "w") as f:
        json.dump(merged, f, indent=2)
    print(json.dumps(merged, indent=2))


if __name__ == "__main__":
    main()
