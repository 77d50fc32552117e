"""Reference arm of bench.py: runs the unmodified reference (Dazz993/Mist, installed under
baseline/_ref by baseline/install_reference.sh) through its own exec entry point,
``benchmark/mist/exec/benchmark_one_case.py::benchmark_multi_devices``, on the benchmark's model and
layout (GPT-3 2.7B, bf16, sequence 2048, micro batch 8 per GPU, DP = N, ZeRO-2, flash attention).

What comes from outside the reference tree (all under baseline/shims, none of it this framework's models,
kernels or engine):

* ``omegaconf`` / ``hydra``: stand-ins on this framework's YAML composer (neither package is in the image);
  the configuration itself is composed from the reference's own YAML tree.
* ``apex`` / ``amp_C``: ``FusedAdam`` and ``multi_tensor_adam`` on torch's fused multi-tensor Adam kernels.
* ``flash_attn_2_cuda``: adapter from flash-attn 2.3.1's call signatures to the flash-attn 2.8 extension
  of this image.
* ``fused_dense_lib`` / ``dropout_layer_norm``: built from the reference's unmodified ``csrc`` for sm_100
  (baseline/build_reference_ext.py).
* ``ref_compat``: names that newer transformers / einops no longer export; and ``mist/overrides/size.py``
  is not executed (its assignment to ``sympy.Basic.__bases__`` crashes CPython 3.12 with sympy 1.14; it
  only serves symbolic analysis, which execution switches off first thing).

The reference's own timing loop (host timers around ``warmup`` + ``number`` iterations, five each) is
replaced by one that runs the requested warm-up and step counts and times them with CUDA events, and the
inputs provider by one that draws token ids uniformly over the vocabulary; ``run_func`` (forward,
backward, gradient reduction, optimizer step inside the next forward) is the reference's own.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
import time
import types
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"


def _first_frame_in_reference(exc) -> str:
    import traceback
    frames = traceback.extract_tb(exc.__traceback__)
    inside = [f for f in frames if str(REF) in f.filename]
    f = inside[-1] if inside else frames[-1]
    name = f.filename.replace(str(REF) + "/", "")
    return f"{name}:{f.lineno} {type(exc).__name__}: {str(exc).splitlines()[0][:200] if str(exc) else ''}"


def unavailable(reason: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": reason}))
    return 0


def setup_paths():
    for p in (str(HERE.parent), str(REF / "ext"), str(REF), str(HERE / "shims")):
        if p in sys.path:
            sys.path.remove(p)
        sys.path.insert(0, p)


def import_reference():
    import torch  # noqa: F401
    import ref_compat
    ref_compat.apply()
    stand_in = types.ModuleType("mist.overrides.size")
    stand_in.__file__ = "<not executed: see baseline/run_reference.py>"
    sys.modules["mist.overrides.size"] = stand_in
    import mist  # noqa: F401
    ref_compat.after_import()
    spec = importlib.util.spec_from_file_location(
        "ref_benchmark_one_case", REF / "benchmark" / "mist" / "exec" / "benchmark_one_case.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def compose_config(world: int, micro_batch: int, layers=None):
    import hydra
    argv = ["--config-name", "config", "experiment=template-a100-sxm4-40gb", "model=gpt2/2.7b",
            "training.params_dtype=bfloat16", "training.exec_dtype=bfloat16",
            f"training.global_batch_size={micro_batch * world}",
            f"hardware.num_gpus_per_node={world}", "hardware.memory_capacity=178.0",
            f"strategy.device_assignment=[[1,{world}]]", "strategy.gradient_checkpointing=[0]",
            "strategy.gradient_accumulation_steps=1",
            f"strategy.stage_strategies=[[{micro_batch},{world},1,0,1,1,0,0,0,0]]",
            f"strategy.pre_post_strategy_array=[{micro_batch},{world},1,0,1,1,0,0,0,0]",
            "model.use_flash_attn=true", "tiny_bench=true", "profile=false", "memory_debug=false",
            "+output_path=null"]
    if layers:
        argv += [f"model.num_hidden_layers={layers}"]
    exec_file = REF / "benchmark" / "mist" / "exec" / "benchmark_one_case.py"
    cfg = hydra.compose_for(str(exec_file), "../configs", "config.yaml", argv)
    cfg.strategy.enabled = True
    cfg.tuning.enabled = False
    return cfg


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=None, help="debug only")
    ap.add_argument("--micro-batch", type=int, default=8)
    args, _ = ap.parse_known_args(argv)

    if not (REF / "mist" / "re_swap_manager" / "manager.py").exists():
        return unavailable("baseline/_ref does not hold the reference: run baseline/install_reference.sh")
    need = ["fused_dense_lib.so", "dropout_layer_norm.so"]
    missing = [n for n in need if not (REF / "ext" / n).exists()]
    if missing:
        return unavailable(f"reference extensions not built ({', '.join(missing)}): run baseline/build_reference_ext.py")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    setup_paths()
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device: the reference's exec path needs one")
        ref = import_reference()
    except BaseException as e:      # noqa: BLE001 - report the first failing statement
        return unavailable("import of the reference failed at " + _first_frame_in_reference(e))

    import torch.distributed as dist
    from mist.config import MistConfig
    mb, seq, vocab = args.micro_batch, 2048, 50304
    record = {}

    # ---- inputs: uniform token ids over the vocabulary, seeded; device-resident for the device-timed
    # region, copied from pinned host memory every step for the end-to-end region
    state = {"mode": "device", "i": 0}
    gen = torch.Generator().manual_seed(1234 + rank)
    n_batches = args.steps + args.warmup
    host = [(torch.randint(0, vocab, (mb, seq), generator=gen).pin_memory(),
             torch.randint(0, vocab, (mb, seq), generator=gen).pin_memory()) for _ in range(n_batches)]
    ondev = []

    def inputs_provider(batch_size, seq_len, device="cuda"):
        # while the reference builds its model on the meta device it also patches the tensor
        # constructors: hand it meta inputs there, as its own provider would
        if torch.empty(1, device=device).is_meta:
            ids = torch.empty(batch_size, seq_len, dtype=torch.long, device="meta")
            return {"input_ids": ids, "labels": torch.empty_like(ids)}
        k = state["i"] % n_batches
        state["i"] += 1
        if state["mode"] == "device":
            if not ondev:
                ondev.extend((a.to(device), b.to(device)) for a, b in host)
            ids, lab = ondev[k]
        else:
            ids, lab = host[k][0].to(device, non_blocking=True), host[k][1].to(device, non_blocking=True)
        return {"input_ids": ids, "labels": lab}

    ref.get_inputs_provider = lambda name: inputs_provider

    # the loss tensor of the last forward pass (the reference's run_func keeps it local)
    from mist.optimizers import grad_scaler as ref_scaler
    orig_scale = ref_scaler.ConstantGradScaler.scale

    def scale(self, loss):
        record["loss"] = loss.detach()
        return orig_scale(self, loss)
    ref_scaler.ConstantGradScaler.scale = scale

    def timed(run_func, warmup, number, prepare_func=None, sync_func=None, num_memory_records=10, enable_tqdm=False):
        def sync():
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
        for _ in range(args.warmup):
            run_func()
        sync()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            run_func()
        t1.record()
        sync()
        record["dev_ms"] = t0.elapsed_time(t1)
        record["alloc"] = torch.cuda.max_memory_allocated() / 2 ** 20
        # end to end: inputs from pinned host memory, loss read back every step
        state["mode"] = "host"
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall = time.perf_counter()
        e0.record()
        for _ in range(args.steps):
            run_func()
            record["last_loss"] = float(record["loss"].item())
        e1.record()
        sync()
        record["e2e_ms"] = max(e0.elapsed_time(e1), (time.perf_counter() - wall) * 1e3)
        import numpy as np
        lat = np.array([record["dev_ms"] / 1e3 / args.steps] * max(args.steps, 1))
        return lat, ([record["alloc"]], [torch.cuda.max_memory_reserved() / 2 ** 20])
    ref.benchmark_func_walltime = timed

    try:
        cfg = compose_config(world, mb, args.layers)
        mist_config = MistConfig.from_dict_config(cfg)
        ref.benchmark_multi_devices(mist_config)
    except BaseException as e:      # noqa: BLE001
        import traceback
        traceback.print_exc()
        return unavailable("the reference's exec path failed at " + _first_frame_in_reference(e))

    times = torch.tensor([record["dev_ms"], record["e2e_ms"]], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = times.tolist()
    if rank == 0:
        tokens = mb * seq * world
        ms = dev_ms / args.steps
        import ref_compat
        print(json.dumps({
            "metric": "tokens/s per iteration (device-timed, max over ranks)", "impl": "reference",
            "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (uniform token ids, seeded; reference's own random init)",
            "config": {"model": "GPT-3 2.7B (32 layers, hidden 2560, 32 heads, FFN 10240, vocab 50304)",
                       "global_batch": mb * world, "seq_len": seq,
                       "parallelism": f"dp{world} ZeRO-2, flash attention", "micro_batch": mb,
                       "layers": args.layers or 32,
                       "substitutions": ["omegaconf/hydra stand-ins", "apex FusedAdam -> torch fused AdamW",
                                         "flash-attn 2.8 behind the 2.3.1 signatures",
                                         "fused_dense_lib + dropout_layer_norm built from the reference csrc for sm_100",
                                         "mist/overrides/size.py not executed"] + ref_compat.APPLIED},
            "e2e": {"value": tokens / (e2e_ms / args.steps / 1e3), "unit": "tokens/s",
                    "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": int(2 * mb * seq * 8) * world,
                    "d2h_bytes_per_step": 4 * world, "last_loss": record.get("last_loss")},
            "peak_allocated_mb": record.get("alloc"),
        }))
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
