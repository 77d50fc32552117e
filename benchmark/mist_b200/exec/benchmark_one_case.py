"""exec: run the strategy of a configuration on real GPUs and report measured latency and
peak memory.

    torchrun --nproc-per-node N benchmark/mist_b200/exec/benchmark_one_case.py --config-name X

Latency is timed on the device (CUDA events around ``number`` iterations after ``warmup``)
and the maximum over ranks is reported; peak allocated / reserved memory is gathered per
stage (reference: benchmark/mist/exec/benchmark_one_case.py:88-621; it times non-pipelined
runs with host timers and reports rank 0's value, summary keys :615-619).
"""
from __future__ import annotations

import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from common import load_from_cli, output_dir  # noqa: E402

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from mist_b200.api import TrainingSession  # noqa: E402
from mist_b200.ops import native  # noqa: E402
from mist_b200.utils.summary import fmt_cost, fmt_memories, update_summary  # noqa: E402


def run(cfg, node, warmup=None, number=None, comm_backend=None, seed=12345):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl" if cuda else "gloo", timeout=datetime.timedelta(seconds=cfg.nccl_timeout),
                                **({"device_id": torch.device("cuda", local)} if cuda else {}))
    tiny = bool(cfg.get("tiny_bench", True))
    warmup = warmup if warmup is not None else (1 if tiny else 5)
    number = number if number is not None else (2 if tiny else 5)
    if cfg.get("memory_debug", False) and cuda:
        torch.cuda.memory._record_memory_history()
    sess = TrainingSession(cfg, comm_backend=comm_backend, seed=seed)
    if world > 1:
        sess.enable_heartbeat()       # every step beats and checks its peers before it launches anything
    ps = sess.ps
    # messages carry rank and stage; only the first data-parallel rank of each (stage, tp) position logs
    from mist_b200.utils.logging import get_logger, log_memory, set_rank_filter
    set_rank_filter(ps.dp_rank, tag=f"rank {rank} stage {ps.stage} tp {ps.tp_rank}")
    log = get_logger()
    log.info("model built: %d parameters on this rank", sess.engine.num_parameters())
    log.info("collectives: data-parallel gradients %s, tensor-parallel linears %s, ZeRO-3 weight gather %s",
             sess.comm_backend, sess.tp_backend, sess.zero3_gather)
    log_memory("after model build:", log)
    mb, G, seq = sess.micro_batch, sess.G, sess.seq_len
    vocab = cfg.model.vocab_size
    gen = torch.Generator().manual_seed(seed + 31 * ps.dp_rank)     # same data on every tp / pp rank of a replica
    dev = sess.device

    from mist_b200.models.provider import family_of, get_inputs_provider
    decoder_only = family_of(cfg.model.name) in ("gpt", "llama", "falcon")
    provider = get_inputs_provider(cfg.model.name)

    def batch():
        if decoder_only:
            ids = torch.randint(0, vocab, (mb * G, seq), generator=gen)
            lab = torch.randint(0, vocab, (mb * G, seq), generator=gen)
            return ids.to(dev), lab.to(dev)
        # encoder-only / encoder-decoder families: the family's own synthetic inputs (token types,
        # decoder ids, sentence-order labels ...), seeded per data-parallel rank
        return (provider(mb * G, seq, vocab, dev, seed=int(torch.randint(0, 2 ** 31 - 1, (1,), generator=gen))),)

    data = [batch() for _ in range(warmup + number)]

    def sync():
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    prof = None
    if cfg.get("profile", False):
        from mist_b200.utils.logging import enable_ranges
        enable_ranges(True)       # label scheduler actions (unshard / grad reduce / optimizer step / swaps)
    if cfg.get("profile", False) and cuda:
        prof = torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA],
                                      on_trace_ready=torch.profiler.tensorboard_trace_handler(
                                          "./logs", worker_name=f"rank{rank}_stage{ps.stage}"))
        prof.start()
    for i in range(warmup):
        (sess.step_on_device if decoder_only else sess.step_on_device_batch)(*data[i])
    sess.finish()
    sync()
    sampler = None
    if cuda and rank == 0:
        from mist_b200.utils.clocks import ClockSampler
        sampler = ClockSampler(dev.index or 0).start()       # SM clock and throttle reasons during the timed region
    if cuda:
        torch.cuda.reset_peak_memory_stats()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
    wall = time.perf_counter()
    loss = None
    for i in range(number):
        loss = (sess.step_on_device if decoder_only else sess.step_on_device_batch)(*data[warmup + i])
    sess.finish()
    if cuda:
        t1.record()
    sync()
    latency = (t0.elapsed_time(t1) / 1e3 if cuda else time.perf_counter() - wall) / number
    clocks = sampler.stop() if sampler is not None else None
    if prof is not None:
        prof.stop()
    native.check_status()
    # buffers of the fused NVLink kernels live in symmetric arenas outside torch's allocator
    from mist_b200.parallel.symm import SymmetricHeap
    alloc = (torch.cuda.max_memory_allocated() + SymmetricHeap.live_bytes) if cuda else 0
    reserved = (torch.cuda.max_memory_reserved() + SymmetricHeap.live_bytes) if cuda else 0
    stats = torch.tensor([latency, float(alloc), float(reserved)], dtype=torch.float64, device=dev)
    S = ps.num_stages
    per_stage = torch.zeros(S, 2, dtype=torch.float64, device=dev)
    per_stage[ps.stage, 0], per_stage[ps.stage, 1] = float(alloc), float(reserved)
    if world > 1:
        lat = stats[:1].clone()
        dist.all_reduce(lat, op=dist.ReduceOp.MAX)
        dist.all_reduce(per_stage, op=dist.ReduceOp.MAX)
        latency = float(lat[0])
    if cfg.get("memory_debug", False) and cuda:
        torch.cuda.memory._dump_snapshot(f"memory_snapshot_rank{rank}.pickle")
    tokens = cfg.training.global_batch_size * seq
    return {"latency": latency, "tokens_per_s": tokens / latency, "loss": float(loss) if loss is not None else None,
            "peak_allocated": per_stage[:, 0].tolist(), "peak_reserved": per_stage[:, 1].tolist(), "rank": rank,
            "backends": {"comm_backend": sess.comm_backend, "tp_backend": sess.tp_backend,
                         "zero3_gather": sess.zero3_gather}, "clocks": clocks}


def main(argv=None):
    cfg, node = load_from_cli(argv)
    try:
        res = run(cfg, node, comm_backend=node.get("comm_backend"))
    except RuntimeError as e:
        # An unrecoverable error on one rank (out of memory, a kernel's bounded wait that ran out, a peer
        # that stopped): mark the job as aborted and end this host's other ranks by their registered
        # process ids, so nobody waits in a collective for a rank that is gone (reference:
        # find_and_kill_other_processes by command-line pattern, benchmark_one_case.py:434-441).
        print(f"[rank {os.environ.get('RANK', '0')}] error: {e}", file=sys.stderr)
        if dist.is_initialized() and dist.get_world_size() > 1:
            from mist_b200.utils.watchdog import Heartbeat, terminate_job
            try:
                store = dist.PrefixStore("mist_b200_hb", dist.distributed_c10d._get_default_store())
                terminate_job(Heartbeat(store, dist.get_rank(), dist.get_world_size()))
            except Exception:       # noqa: BLE001 - the store itself may be gone
                pass
        raise
    if res["rank"] == 0:
        print(f"Total Latency: {res['latency']:.4f}")
        print(f"Throughput: {res['tokens_per_s']:.1f} tokens/s")
        print(f"Collective back ends: {res['backends']}")
        if res.get("loss") is not None:
            print(f"Loss of the last iteration (this rank's stage): {res['loss']:.4f}")
        if res.get("clocks"):
            c = res["clocks"]
            print(f"SM clock under load: {c.get('sm_mhz')} MHz of {c.get('sm_max_mhz')} ({', '.join(c.get('reasons', [])) or 'no throttle reason'})")
        print(f"Peak allocated memory per stage: {fmt_memories(res['peak_allocated'])}")
        print(f"Peak reserved memory per stage: {fmt_memories(res['peak_reserved'])}")
        update_summary(os.path.join(output_dir(node), "summary.json"), {
            "exec_total_cost": fmt_cost(res["latency"]),
            "exec_throughput": f"{res['tokens_per_s']:.1f}",
            "exec_backends": res["backends"],
            "exec_clocks": res.get("clocks"),
            "exec_stage_peak_allocated_memories": fmt_memories(res["peak_allocated"]),
            "exec_stage_peak_reserved_memories": fmt_memories(res["peak_reserved"]),
        })
    if dist.is_initialized():
        dist.destroy_process_group()
    return res


if __name__ == "__main__":
    main()
