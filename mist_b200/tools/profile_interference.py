"""Hardware calibration: measures how compute, GPU<->GPU collectives and host<->GPU copies
slow each other down when they run at the same time, and the raw bandwidths.

    torchrun --nproc-per-node 8 -m mist_b200.tools.profile_interference --out calib.json
    python -m mist_b200.tools.comm_model calib.json        # -> the four parameter lists

For every combination of {GEMM, all-gather, host->device copy, device->host copy} each
sized to take roughly 0 / 3 / 6 / 9 ms alone on this machine, the four activities are
launched on four streams at once and the wall time of the group is measured on the device
(CUDA events, max over ranks).  Collective-only sweeps over message sizes and group sizes
give the bandwidth table.  Records: ``{"C", "G2G", "C2G", "G2C"}`` standalone seconds,
``latency`` concurrent seconds, ``g2g_gbytes / c2g_gbytes / g2c_gbytes``, ``intra``,
``inter``.

(reference: mist/tools/profile_interference.py:109-417 and
mist/tools/scripts/profile_interference_single_node.sh; target durations there are
0/3/6/9/12 ms scaled from reference TFLOPS / bandwidth tables, here they are found by a
short search on the device itself.)
"""
from __future__ import annotations

import argparse
import itertools
import json
import os
from typing import Dict, List

import torch
import torch.distributed as dist

TARGETS_MS = (0.0, 3.0, 6.0, 9.0)


def _time(fn, warmup=3, repeat=5, group=None) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(repeat):
        if group is not None:
            dist.barrier(group=group)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e-3)
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda", dtype=torch.float64)
    if group is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t[0])


class Activities:
    def __init__(self, group, max_mb: int = 1024):
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.s_c, self.s_g, self.s_h, self.s_d = (torch.cuda.Stream() for _ in range(4))
        self.gemm_a = torch.randn(8192, 4096, device="cuda", dtype=torch.bfloat16)
        self.gemm_b = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
        n = max_mb << 20
        self.ag_in = torch.empty(n // max(self.world, 1), dtype=torch.uint8, device="cuda")
        self.ag_out = torch.empty(n, dtype=torch.uint8, device="cuda")
        self.host = torch.empty(n, dtype=torch.uint8).pin_memory()
        self.dev_in = torch.empty(n, dtype=torch.uint8, device="cuda")
        self.dev_out = torch.empty(n, dtype=torch.uint8, device="cuda")
        self.host_out = torch.empty(n, dtype=torch.uint8).pin_memory()

    # each activity: amount -> launches on its stream
    def compute(self, reps: int):
        for _ in range(reps):
            torch.matmul(self.gemm_a, self.gemm_b)

    def collective(self, nbytes: int):
        if nbytes and self.world > 1:
            per = nbytes // self.world
            dist.all_gather_into_tensor(self.ag_out[: per * self.world], self.ag_in[:per], group=self.group)

    def h2d(self, nbytes: int):
        if nbytes:
            self.dev_in[:nbytes].copy_(self.host[:nbytes], non_blocking=True)

    def d2h(self, nbytes: int):
        if nbytes:
            self.host_out[:nbytes].copy_(self.dev_out[:nbytes], non_blocking=True)

    def run(self, reps: int, g_bytes: int, h_bytes: int, d_bytes: int):
        cur = torch.cuda.current_stream()
        for s in (self.s_c, self.s_g, self.s_h, self.s_d):
            s.wait_stream(cur)
        with torch.cuda.stream(self.s_c):
            self.compute(reps)
        with torch.cuda.stream(self.s_g):
            self.collective(g_bytes)
        with torch.cuda.stream(self.s_h):
            self.h2d(h_bytes)
        with torch.cuda.stream(self.s_d):
            self.d2h(d_bytes)
        for s in (self.s_c, self.s_g, self.s_h, self.s_d):
            cur.wait_stream(s)


def _size_for(target_s: float, unit_time: float, unit: int, cap: int) -> int:
    if target_s <= 0:
        return 0
    return int(min(cap, max(1, round(target_s / unit_time)) * unit))


def profile(group, intra: int, inter: int, max_mb: int = 512, quick: bool = False) -> List[Dict]:
    act = Activities(group, max_mb)
    cap = max_mb << 20
    unit = 16 << 20
    t_gemm = _time(lambda: act.run(1, 0, 0, 0), group=group)
    t_ag = _time(lambda: act.run(0, unit * 4, 0, 0), group=group) / 4 if act.world > 1 else 0.0
    t_h = _time(lambda: act.run(0, 0, unit * 4, 0), group=group) / 4
    t_d = _time(lambda: act.run(0, 0, 0, unit * 4), group=group) / 4
    targets = (0.0, 3e-3, 9e-3) if quick else tuple(t * 1e-3 for t in TARGETS_MS)
    records: List[Dict] = []
    standalone: Dict = {}

    def alone(kind, amount):
        key = (kind, amount)
        if key not in standalone:
            args = {"c": (amount, 0, 0, 0), "g": (0, amount, 0, 0), "h": (0, 0, amount, 0), "d": (0, 0, 0, amount)}[kind]
            standalone[key] = _time(lambda: act.run(*args), group=group) if amount else 0.0
        return standalone[key]

    for tc, tg, th, td in itertools.product(targets, repeat=4):
        if sum(x > 0 for x in (tc, tg, th, td)) < 1:
            continue
        reps = int(round(tc / t_gemm)) if tc > 0 else 0
        gb = _size_for(tg, t_ag, unit, cap) if act.world > 1 else 0
        hb = _size_for(th, t_h, unit, cap)
        db = _size_for(td, t_d, unit, cap)
        if not (reps or gb or hb or db):
            continue
        lat = _time(lambda: act.run(reps, gb, hb, db), group=group)
        records.append({"C": alone("c", reps), "G2G": alone("g", gb), "C2G": alone("h", hb), "G2C": alone("d", db),
                        "latency": lat, "g2g_gbytes": gb / 1e9, "c2g_gbytes": hb / 1e9, "g2c_gbytes": db / 1e9,
                        "intra": intra, "inter": inter})
    # bandwidth sweeps (one activity at a time)
    for mb in (16, 64, 128, 256, 512):
        nb = min(mb << 20, cap)
        if act.world > 1:
            records.append({"C": 0.0, "G2G": alone("g", nb), "C2G": 0.0, "G2C": 0.0, "latency": alone("g", nb),
                            "g2g_gbytes": nb / 1e9, "c2g_gbytes": 0.0, "g2c_gbytes": 0.0, "intra": intra, "inter": inter})
        records.append({"C": 0.0, "G2G": 0.0, "C2G": alone("h", nb), "G2C": 0.0, "latency": alone("h", nb),
                        "g2g_gbytes": 0.0, "c2g_gbytes": nb / 1e9, "g2c_gbytes": 0.0, "intra": intra, "inter": inter})
        records.append({"C": 0.0, "G2G": 0.0, "C2G": 0.0, "G2C": alone("d", nb), "latency": alone("d", nb),
                        "g2g_gbytes": 0.0, "c2g_gbytes": 0.0, "g2c_gbytes": nb / 1e9, "intra": intra, "inter": inter})
    return records


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="bandwidth.json")
    ap.add_argument("--group-sizes", default="2,4,8")
    ap.add_argument("--max-mb", type=int, default=512)
    ap.add_argument("--quick", action="store_true")
    args = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    records: List[Dict] = []
    sizes = [int(s) for s in args.group_sizes.split(",") if int(s) <= world] or [1]
    for gs in sizes:
        groups = [dist.new_group(list(range(i, i + gs))) for i in range(0, world, gs)] if world > 1 else [None]
        mine = groups[rank // gs] if world > 1 else None
        recs = profile(mine, intra=gs, inter=1, max_mb=args.max_mb, quick=args.quick)
        if rank == 0:
            records.extend(recs)
    if world == 1:
        records = profile(None, 1, 1, args.max_mb, args.quick)
    if rank == 0:
        with open(args.out, "w") as f:
            json.dump(records, f)
        print(f"wrote {len(records)} records to {args.out}")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
