"""Measures what the host spends on one transformer block of this engine (Python, autograd, kernel launches)
and writes it into the operator database's meta file.

A training step cannot run faster than its host thread issues it.  With small micro batches on many-way tensor
parallel layouts the kernels of a block take a few milliseconds, of the same order as what the host needs for
the block (about 1 ms for forward + backward, another 1 ms for a recomputed forward pass under activation
checkpointing).  The cost model therefore prices a block with ``max(device time, host time)``; the host time comes
from here, not from a fit to step times: a model whose kernels are negligible (hidden 256, sequence 128, one
sequence) is stepped with 8 and with 24 blocks, with and without recomputation, and the differences give the
host seconds per block for forward + backward and for a recomputed forward pass.  They are stored with the
number of operators of the block's trace, so layouts with more operators per block (tensor-parallel collectives)
are charged more.

    python -m mist_b200.tools.profile_host_dispatch [--meta <_meta.json>] [--steps 20]

Counterpart in the reference: none (its operator timings include the dispatch of each operator,
mist/node_database/node_spec.py:249-320, and it has no host term for a whole block).
"""
from __future__ import annotations

import argparse
import json
import time
from pathlib import Path


def _overrides(layers: int, ckpt: int):
    return ["experiment=gpt2-1.3b", f"model.num_hidden_layers={layers}", "model.hidden_size=256",
            "model.intermediate_size=1024", "model.num_attention_heads=4", "training.max_sequence_length=128",
            "model.vocab_size=1024", f"strategy.layer_partitions=[{layers}]", "hardware.num_gpus_per_node=1",
            "hardware.num_nodes=1", "training.global_batch_size=1", "strategy.device_assignment=[[1,1]]",
            f"strategy.gradient_checkpointing=[{ckpt}]", "strategy.gradient_accumulation_steps=1",
            "strategy.stage_strategies=[[1,1,1,0,0,0,0,0,0,0]]", "strategy.pre_post_strategy_array=[1,1,1,0,0,0,0,0,0,0]"]


def _step_seconds(layers: int, ckpt: int, steps: int) -> float:
    import torch
    from mist_b200.api import build_training
    session = build_training("config", _overrides(layers, ckpt), seed=0)
    cuda = torch.cuda.is_available()
    ids = torch.randint(0, 1024, (1, 128), device="cuda" if cuda else "cpu")
    sync = torch.cuda.synchronize if cuda else (lambda: None)
    for _ in range(5):
        session.step_on_device(ids, ids)
    session.finish()
    sync()
    best = float("inf")
    for _ in range(3):                       # best of three: the host thread shares its core with other work
        t0 = time.perf_counter()
        for _ in range(steps):
            session.step_on_device(ids, ids)
        session.finish()
        sync()
        best = min(best, (time.perf_counter() - t0) / steps)
    del session
    return best


def measure(steps: int = 20):
    from mist_b200.analyzer.stage_evaluator import StageEvaluator
    from mist_b200.config import load_config
    t8 = _step_seconds(8, 0, steps)
    t24 = _step_seconds(24, 0, steps)
    t24c = _step_seconds(24, 24, steps)
    both = (t24 - t8) / 16.0                 # forward + backward of one block
    rec = max((t24c - t24) / 24.0, 0.0)      # the recomputed forward pass of one block (activation checkpointing)
    cfg, _ = load_config("config", _overrides(8, 0), check_world_size=False)
    nodes = len(StageEvaluator(cfg).analysis(1).layer("block_layer").nodes)
    return {"block_fwd_bwd_s": both, "block_recompute_s": rec, "ops_per_block": nodes,
            "step_s": {"8 blocks": t8, "24 blocks": t24, "24 blocks recomputed": t24c}}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--meta", default=None, help="meta file of the operator database to update")
    ap.add_argument("--steps", type=int, default=20)
    args = ap.parse_args(argv)
    res = measure(args.steps)
    print(json.dumps(res, indent=1))
    if args.meta:
        p = Path(args.meta)
        meta = json.load(open(p)) if p.exists() else {}
        meta["host_dispatch"] = res
        with open(p, "w") as fh:
            json.dump(meta, fh, indent=1)
            fh.write("\n")


if __name__ == "__main__":
    main()
