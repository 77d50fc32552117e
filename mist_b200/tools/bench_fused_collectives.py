"""Times every fused compute + collective kernel against its library sequence on real peers and
prints each one's fraction of its roofline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m mist_b200.tools.bench_fused_collectives [--only ag,rs,zero3,dp] [--json out.json]

Roofline of a kernel = the slower of (FLOPs / measured bf16 GEMM burst rate) and (bytes that must cross
NVLink per rank and direction / measured peer-copy rate); the two rates default to 1601.6 TFLOP/s and
770 GB/s and can be overridden (``--tflops``, ``--link-gbs``).  Times are medians of CUDA-event timings,
L2 flushed and ranks aligned by a barrier before each repetition, maximum over ranks.

Kernels: all-gather -> GEMM and GEMM -> reduce-scatter of the sequence-parallel linears (Llama-7B
shapes for 2 ranks, GPT-3 13B shapes for 4), the ZeRO-3 weight all-gather fused into a block's first
GEMM, and the data-parallel gradient reduce-scatter + Adam + weight write-back.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="p2p,ag,rs,zero3,dp")
    ap.add_argument("--tflops", type=float, default=1601.6)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--hbm-gbs", type=float, default=6544.0)
    ap.add_argument("--iters", type=int, default=9)
    ap.add_argument("--json", default=None)
    args = ap.parse_args(argv)
    only = set(args.only.split(","))
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from mist_b200.ops import functional as F
    from mist_b200.ops import native
    from mist_b200.ops.native import call, ptr
    from mist_b200.parallel import fused_tp
    from mist_b200.parallel.symm import SymmetricHeap, ptr_table

    g = dist.new_group(list(range(world)))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    PEAK, LINK, HBM = args.tflops * 1e12, args.link_gbs * 1e9, args.hbm_gbs * 1e9

    def timeit(fn, warm=3):
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    rows_out = []

    def report(kind, shape, t_fused, t_lib, flops, link_bytes, extra="", parts=None):
        """``parts``: (GEMM alone, collective alone) in ms -- what the cost model's overlap terms are fitted to."""
        roof = max(flops / PEAK, link_bytes / LINK) * 1e3
        row = dict(kernel=kind, shape=shape, ranks=world, fused_ms=round(t_fused, 4), library_ms=round(t_lib, 4),
                   roofline_ms=round(roof, 4), fraction=round(roof / t_fused, 3), note=extra)
        if parts is not None:
            row["gemm_ms"], row["collective_ms"] = round(parts[0], 4), round(parts[1], 4)
        rows_out.append(row)
        if rank == 0:
            print(f"{kind:34s} R{world} {shape:34s} fused {t_fused:7.3f} ms  library {t_lib:7.3f} ms  "
                  f"roofline {roof:6.3f} ms -> {roof / t_fused:4.2f} {extra}", flush=True)

    if "p2p" in only and world > 1:
        # what SM-issued peer loads reach on this box, per grid size, beside NCCL's all-gather: the link rate
        # that the kernels below can hope for (the roofline's 770 GB/s is a copy-engine figure)
        shard = 64 << 20
        heap = SymmetricHeap(shard + (4 << 20), g)
        src, soff = heap.alloc(shard // 2, torch.bfloat16)
        flags, foff = heap.alloc(32, torch.int32)
        dst = torch.empty(world * shard // 2, dtype=torch.bfloat16, device="cuda")
        st, ft = ptr_table(heap.peer_ptrs(soff)), ptr_table(heap.peer_ptrs(foff))
        ep = [0]
        torch.cuda.synchronize()
        dist.barrier()
        t_nccl = timeit(lambda: dist.all_gather_into_tensor(dst, src, group=g))
        inbound = shard * (world - 1)
        for ctas in (32, 64, 128, 148):
            def gather():
                ep[0] += 1
                call("mb_p2p_all_gather", st, ptr(dst), ft, shard, world, rank, ep[0], ctas, native.stream())
            t = timeit(gather)
            rows_out.append(dict(kernel="peer all-gather (SM loads)", ranks=world, ctas=ctas, fused_ms=round(t, 4),
                                 library_ms=round(t_nccl, 4), inbound_gbs=round(inbound / t / 1e6, 1),
                                 nccl_inbound_gbs=round(inbound / t_nccl / 1e6, 1)))
            if rank == 0:
                print(f"peer all-gather, 64 MiB per rank, R{world} ctas {ctas:3d}: {t:6.3f} ms = {inbound / t / 1e6:5.0f} GB/s inbound"
                      f"   (NCCL all-gather {t_nccl:6.3f} ms = {inbound / t_nccl / 1e6:5.0f} GB/s)", flush=True)
        del heap

    # shapes: tokens per micro batch T, model width h, per-rank widths of the four sequence-parallel linears
    if world <= 2:
        T, h, ffn_gate, ffn, tag = 16384, 4096, 2 * 11008 // world, 11008 // world, "llama-7b"
    else:
        T, h, ffn_gate, ffn, tag = 4096, 5120, 20480 // world, 20480 // world, "gpt3-13b"
    qkv = 3 * h // world
    tp = None
    if only & {"ag", "rs"}:
        tp = fused_tp.FusedTPContext(g, 6 << 30)
    if "ag" in only:
        for N, name in ((qkv, "qkv"), (ffn_gate, "fc1")):
            x = torch.randn(T // world, h, device="cuda", dtype=torch.bfloat16)
            w = torch.randn(N, h, device="cuda", dtype=torch.bfloat16) * 0.02
            t_f = timeit(lambda: fused_tp._ag_gemm(tp, x, w, None, False, "b"))

            def lib():
                xf = torch.empty(T, h, device="cuda", dtype=torch.bfloat16)
                dist.all_gather_into_tensor(xf, x, group=g)
                return xf @ w.t()
            xf0 = torch.empty(T, h, device="cuda", dtype=torch.bfloat16)
            parts = (timeit(lambda: F.gemm(xf0, w)), timeit(lambda: dist.all_gather_into_tensor(xf0, x, group=g)))
            report("AG->GEMM " + name, f"{tag} T{T} K{h} N{N}", t_f, timeit(lib), 2.0 * T * h * N,
                   T * h * 2 * (world - 1) / world, parts=parts)
    if "rs" in only:
        for K, name in ((h // world, "out_proj"), (ffn, "fc2")):
            x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
            w = torch.randn(h, K, device="cuda", dtype=torch.bfloat16) * 0.02
            res = torch.randn(T // world, h, device="cuda", dtype=torch.bfloat16)

            def lib():
                y = x @ w.t()
                o = torch.empty(T // world, h, device="cuda", dtype=torch.bfloat16)
                dist.reduce_scatter_tensor(o, y, group=g)
                return o + res
            link = T * h * 2 * (world - 1) / world
            t_lib = timeit(lib)
            y0 = torch.empty(T, h, device="cuda", dtype=torch.bfloat16)
            o0 = torch.empty(T // world, h, device="cuda", dtype=torch.bfloat16)
            parts = (timeit(lambda: F.gemm(x, w, out=y0)), timeit(lambda: dist.reduce_scatter_tensor(o0, y0, group=g)))
            for form in ("store", "add"):
                fused_tp.RS_FORM = form
                t_f = timeit(lambda: fused_tp._gemm_rs(tp, x, w, False, residual=res))
                report(f"GEMM->RS {name} ({form})", f"{tag} T{T} K{K} N{h}", t_f, t_lib, 2.0 * T * K * h,
                       link * (2 if (form == "add" and world > 2) else 1), "+residual", parts=parts)
            fused_tp.RS_FORM = "store"
    if "zero3" in only and world > 1:
        from mist_b200.parallel.fused_zero3 import ParamGatherContext
        for hh, M, name in ((2560, 16384, "2.7b block"), (6144, 4096, "22b block")):
            numel = 12 * hh * hh + 13 * hh
            padded = (numel + 128 * world - 1) // (128 * world) * (128 * world)
            ctx = ParamGatherContext(g, padded, n_slots=1)
            shard = torch.randn(padded // world, device="cuda", dtype=torch.bfloat16) * 0.02
            x = torch.randn(M, hh, device="cuda", dtype=torch.bfloat16)
            b_off = 2 * hh // 128 * 128 + 128

            def fused():
                ctx.stage_shard(0, shard)
                return ctx.gather_linear(0, x, b_off, 3 * hh, hh)
            full = torch.empty(padded, device="cuda", dtype=torch.bfloat16)

            def lib():
                dist.all_gather_into_tensor(full, shard, group=g)
                return x @ full[b_off:b_off + 3 * hh * hh].view(3 * hh, hh).t()
            wq = full[b_off:b_off + 3 * hh * hh].view(3 * hh, hh)
            parts = (timeit(lambda: F.gemm(x, wq)), timeit(lambda: dist.all_gather_into_tensor(full, shard, group=g)))
            report("ZeRO-3 weight-AG->GEMM", f"{name} M{M} N{3 * hh} K{hh}", timeit(fused), timeit(lib),
                   2.0 * M * 3 * hh * hh, padded * 2 * (world - 1) / world, parts=parts)
            del ctx
    if "dp" in only and world > 1:
        # gradient reduce-scatter + Adam + weight write-back of one GPT-3 2.7B block (78.7 M parameters)
        numel = 12 * 2560 * 2560 + 13 * 2560
        padded = (numel + 128 * world - 1) // (128 * world) * (128 * world)
        shard = padded // world
        heap = SymmetricHeap(padded * 4 + (4 << 20), g)
        grads, goff = heap.alloc(padded, torch.bfloat16)
        params, poff = heap.alloc(padded, torch.bfloat16)
        flags, foff = heap.alloc(32, torch.int32)
        grads.copy_((torch.randn(padded, device="cuda") * 0.01).to(torch.bfloat16))
        master = torch.randn(shard, device="cuda")
        m, v = torch.zeros_like(master), torch.zeros_like(master)
        torch.cuda.synchronize()
        dist.barrier()
        gt, pt, ft = ptr_table(heap.peer_ptrs(goff)), ptr_table(heap.peer_ptrs(poff)), ptr_table(heap.peer_ptrs(foff))
        epoch = [0]
        link = shard * 2 * (world - 1)                    # in: peers' slices of the bucket; out: new weights (same size)
        hbm = shard * (2 + 12 + 12 + 2) + link * 0
        out_shard = torch.empty(shard, dtype=torch.bfloat16, device="cuda")
        full_w = torch.empty(padded, dtype=torch.bfloat16, device="cuda")

        def lib():
            dist.reduce_scatter_tensor(out_shard, grads, group=g)
            F.adam_step(master, m, v, out_shard, full_w[rank * shard:(rank + 1) * shard], lr=1e-4, beta1=0.9, beta2=0.95,
                        eps=1e-8, weight_decay=0.1, step=1, inv_scale=1.0 / world, adamw=True)
            dist.all_gather_into_tensor(full_w, full_w[rank * shard:(rank + 1) * shard].clone(), group=g)
        t_lib = timeit(lib)
        for ctas in (0, 48, 128, 148):
            def fused():
                epoch[0] += 1
                call("mb_fused_grad_reduce_adam", gt, pt, ft, ptr(master), ptr(m), ptr(v), None, shard, world, rank,
                     epoch[0], 0, 1, 1e-4, 0.9, 0.95, 1e-8, 0.1, 1, 1.0 / world, 1, ctas, native.stream())
            t_f = timeit(fused)
            roof = max(link / LINK, hbm / HBM) * 1e3
            gbs = link / (t_f * 1e-3) / 1e9
            rows_out.append(dict(kernel="grad RS + Adam + weight write-back", shape=f"2.7b block {padded} elems", ranks=world,
                                 ctas=ctas, fused_ms=round(t_f, 4), library_ms=round(t_lib, 4), roofline_ms=round(roof, 4),
                                 fraction=round(roof / t_f, 3), nvlink_gbs_per_direction=round(gbs, 1)))
            if rank == 0:
                print(f"grad RS+Adam+write-back R{world} ctas {ctas or 'auto':>4}: fused {t_f:7.3f} ms  "
                      f"NCCL RS + Adam + NCCL AG {t_lib:7.3f} ms  roofline {roof:6.3f} ms -> {roof / t_f:4.2f}  "
                      f"({gbs:5.0f} GB/s in and out per rank)", flush=True)
    torch.cuda.synchronize()
    native.check_status()
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump(rows_out, f, indent=1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
