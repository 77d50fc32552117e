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
    for form in ("store", "store", "add"):        # two launches of the default form: the slot sets alternate
        fused_tp.RS_FORM = form
        try:
            out = fused_tp._gemm_rs(ctx, x, w, b_mn)
        finally:
            fused_tp.RS_FORM = "store"
        torch.cuda.synchronize()
        native.check_status()
        ref = x.float() @ (w.float() if b_mn else w.float().t())
        assert _rel(out, ref[:rows]) < 1e-2
        assert (out.float() - ref[:rows]).abs().max().item() < 0.05 * ref.abs().max().item()
    # bias and residual are added where the per-rank partial products are summed
    bias = torch.randn(N if not b_mn else w.shape[1], device="cuda", dtype=torch.bfloat16)
    res = torch.randn(rows, bias.numel(), device="cuda", dtype=torch.bfloat16)
    out = fused_tp._gemm_rs(ctx, x, w, b_mn, bias=bias, residual=res)
    torch.cuda.synchronize()
    native.check_status()
    assert _rel(out, ref[:rows] + bias.float() + res.float()) < 1e-2


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
        # the row-parallel bias lives on the first rank only; the residual is this rank's token shard
        b2 = (torch.randn(K, device="cuda", dtype=torch.bfloat16) * 0.5).requires_grad_(True) if rank == 0 else None
        res = torch.randn(T // world, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        errs = {}
        firsts = None
        for it in range(3):
            # fused: column-parallel then row-parallel, as in an MLP
            h = fused_tp.ag_linear(x_shard, w1, None, tp)
            y = fused_tp.linear_rs(h, w2, b2, tp, residual=res)
            gy = torch.ones_like(y) * 0.01
            gx, gw1, gw2, gres = torch.autograd.grad(y, (x_shard, w1, w2, res), gy)
            # reference: NCCL collectives + plain linears
            xr = dist_ops.all_gather(x_shard, g)
            hr = F.linear(xr, w1)
            yr = dist_ops.reduce_scatter(F.linear(hr, w2, b2), g) + res
            gxr, gw1r, gw2r = torch.autograd.grad(yr, (x_shard, w1, w2), gy)
            torch.cuda.synchronize()
            native.check_status()
            errs = {"y": _rel(y, yr), "gx": _rel(gx, gxr), "gw1": _rel(gw1, gw1r), "gw2": _rel(gw2, gw2r),
                    "gres": _rel(gres, gy), "max_y": ((y.float() - yr.float()).abs().max() / yr.float().abs().max()).item()}
            # the same inputs give the same bits on every launch, whatever order the peers' tiles arrive in
            if firsts is None:
                firsts = (y.clone(), gx.clone())
            else:
                errs["repeat"] = float(not (torch.equal(y, firsts[0]) and torch.equal(gx, firsts[1])))
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_multi_gpu_matches_nccl_path(world):
    """Column-parallel + row-parallel linear (bias on the first rank, residual) forward and backward
    on 2 and on 4 GPUs against the NCCL collectives around plain linears, three launches in a row
    (the slot sets alternate), with bit-equal results from launch to launch."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    for r in range(world):
        assert ret[r]["repeat"] == 0.0, (r, "results differ between launches")
        for k, v in ret[r].items():
            if k == "max_y":
                # worst element against the largest output: each source's partial product is rounded to bf16
                # before the sum (as NCCL's bf16 reduce-scatter does), so the error of an element follows the size
                # of the partials, which cancel, not the size of the element
                assert v < 0.02, (r, k, v)
            else:
                assert v < 2e-2, (r, k, v)
