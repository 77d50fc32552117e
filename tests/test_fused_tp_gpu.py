"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels: single-GPU emulation (peers are
local buffers) and a 2-GPU comparison with the NCCL + GEMM path."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mist_b200.utils.device import free_port

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("b_mn", [False, True])
def test_emulated_two_ranks_one_gpu(b_mn):
    """Both "ranks'" buffers live on this GPU and the peer flags are pre-set, so one launch
    covers the gather CTAs, the per-chunk flag waits and the reduce-add epilogue."""
    from mist_b200.ops import native
    from mist_b200.parallel import fused_tp
    torch.manual_seed(0)
    ctx = fused_tp.FusedTPContext(None, 0, emulate_ranks=2)
    rows, K, N = 512, 384, 640
    x_shard = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16)
    peer_rows = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(K, N, device="cuda", dtype=torch.bfloat16) if b_mn
         else torch.randn(N, K, device="cuda", dtype=torch.bfloat16)) * 0.05
    # plant the "peer's" rows in its buffer
    a_full, _ = ctx.gathered(2 * rows, K, "t")
    ctx._keep[-1].view(2 * rows, K)[rows:].copy_(peer_rows)
    y, gathered = fused_tp._ag_gemm(ctx, x_shard, w, None, b_mn, "t")
    torch.cuda.synchronize()
    native.check_status()
    full = torch.cat([x_shard, peer_rows])
    ref = full.float() @ (w.float() if b_mn else w.float().t())
    assert _rel(gathered, full) == 0.0
    assert _rel(y, ref) < 1e-2
    # GEMM -> RS: rank 0 keeps rows [0, rows) of its own partial product (the emulated peer adds nothing)
    x = torch.randn(2 * rows, K, device="cuda", dtype=torch.bfloat16)
    out = fused_tp._gemm_rs(ctx, x, w, b_mn)
    torch.cuda.synchronize()
    native.check_status()
    ref = x.float() @ (w.float() if b_mn else w.float().t())
    assert _rel(out, ref[:rows]) < 1e-2


@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("pair", [1, 0])
def test_emulated_two_ranks_large_tiles(b_mn, pair):
    """Shapes big enough for the CTA-pair variant (256 x 256 tiles, two CTAs per tile); with
    ``pair = 0`` the same shapes run on single CTAs."""
    from mist_b200.ops import native
    from mist_b200.parallel import fused_tp
    lib = native.kernels()
    lib.mb_gemm_comm_set_pair(pair)
    try:
        torch.manual_seed(1)
        ctx = fused_tp.FusedTPContext(None, 0, emulate_ranks=2)
        rows, K, N = 2048, 320, 1280
        x_shard = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16)
        peer_rows = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16)
        w = (torch.randn(K, N, device="cuda", dtype=torch.bfloat16) if b_mn
             else torch.randn(N, K, device="cuda", dtype=torch.bfloat16)) * 0.05
        bias = None if b_mn else torch.randn(N, device="cuda", dtype=torch.bfloat16)
        ctx.gathered(2 * rows, K, "p")
        ctx._keep[-1].view(2 * rows, K)[rows:].copy_(peer_rows)
        for _ in range(2):                      # second launch: epochs advance
            y, gathered = fused_tp._ag_gemm(ctx, x_shard, w, bias, b_mn, "p")
            torch.cuda.synchronize()
            native.check_status()
            assert lib.mb_gemm_comm_last_pair() == pair
            full = torch.cat([x_shard, peer_rows])
            ref = full.float() @ (w.float() if b_mn else w.float().t())
            if bias is not None:
                ref = ref + bias.float()
            assert _rel(gathered, full) == 0.0
            assert _rel(y, ref) < 1e-2
        x = torch.randn(2 * rows, K, device="cuda", dtype=torch.bfloat16)
        out = fused_tp._gemm_rs(ctx, x, w, b_mn)
        torch.cuda.synchronize()
        native.check_status()
        assert lib.mb_gemm_comm_last_pair() == pair
        ref = x.float() @ (w.float() if b_mn else w.float().t())
        assert _rel(out, ref[:rows]) < 1e-2
    finally:
        lib.mb_gemm_comm_set_pair(1)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from mist_b200.ops import functional as F
        from mist_b200.ops import native
        from mist_b200.parallel import dist_ops, fused_tp
        g = dist.new_group(list(range(world)))
        tp = fused_tp.FusedTPContext(g, 512 << 20)
        torch.manual_seed(rank)
        T, K, N = 1024, 512, 768
        x_shard = torch.randn(T // world, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        w1 = (torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_(True)
        w2 = (torch.randn(K, N, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_(True)
        errs = {}
        for it in range(2):
            # fused: column-parallel then row-parallel, as in an MLP
            h = fused_tp.ag_linear(x_shard, w1, None, tp)
            y = fused_tp.linear_rs(h, w2, None, tp)
            gy = torch.ones_like(y) * 0.01
            gx, gw1, gw2 = torch.autograd.grad(y, (x_shard, w1, w2), gy)
            # reference: NCCL collectives + plain linears
            xr = dist_ops.all_gather(x_shard, g)
            hr = F.linear(xr, w1)
            yr = dist_ops.reduce_scatter(F.linear(hr, w2), g)
            gxr, gw1r, gw2r = torch.autograd.grad(yr, (x_shard, w1, w2), gy)
            torch.cuda.synchronize()
            native.check_status()
            errs = {"y": _rel(y, yr), "gx": _rel(gx, gxr), "gw1": _rel(gw1, gw1r), "gw2": _rel(gw2, gw2r)}
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


def test_two_gpus_match_nccl_path():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    for r in range(2):
        for k, v in ret[r].items():
            assert v < 2e-2, (r, k, v)
