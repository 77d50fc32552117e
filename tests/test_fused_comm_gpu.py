"""NVLink peer-memory kernels: fused gradient reduce + Adam + weight write-back, all-gather,
reduce-scatter (2+ GPUs, compared with the NCCL path), and the bounded flag wait (1 GPU)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mist_b200.utils.device import free_port

pytestmark = pytest.mark.gpu


def test_flag_wait_gives_up_with_status():
    """A wait that nothing satisfies returns after its time limit and reports a status;
    the context stays usable."""
    from mist_b200.ops import native
    from mist_b200.parallel import symm  # noqa: F401  (registers the signatures)
    lib = native.kernels()
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    assert lib.mb_set_peer_wait_ms(100) == 0
    try:
        native.call("mb_wait_on_flags", flags.data_ptr(), 4, 1, native.stream())
        torch.cuda.synchronize()
        assert lib.mb_status_read_and_clear() == 4          # MB_ERR_TIMEOUT_PEER
        # flags already at the epoch: returns at once, no status
        flags.fill_(1)
        native.call("mb_wait_on_flags", flags.data_ptr(), 4, 1, native.stream())
        torch.cuda.synchronize()
        assert lib.mb_status_read_and_clear() == 0
        x = torch.ones(16, device="cuda")
        assert float(x.sum()) == 16.0
    finally:
        lib.mb_set_peer_wait_ms(2000)


def _worker(rank, world, port, zero_flags, G, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from mist_b200.config import StageStrategy, load_config
        from mist_b200.models.provider import base_model_provider, get_inputs_provider
        from mist_b200.ops import native
        from mist_b200.parallel.engine import TrainEngine
        from mist_b200.parallel.state import ParallelState, build_plan
        cfg, _ = load_config("config", ["experiment=gpt2-1.3b", "model.num_hidden_layers=2", "model.hidden_size=256",
                                        "model.intermediate_size=1024", "model.num_attention_heads=4",
                                        "training.max_sequence_length=128", "model.vocab_size=1024",
                                        "strategy.layer_partitions=[2]"], check_world_size=False)
        plan = build_plan([(1, world)], [(2, world, 1)], (1, world))
        ps = ParallelState(plan, rank)
        strat = StageStrategy(2, world, 1, *zero_flags, 0, 0, 0, 0)
        finals = {}
        for backend in ("nccl", "fused"):
            torch.manual_seed(0)
            model = base_model_provider(cfg.model, device="cuda", dtype=torch.bfloat16)
            eng = TrainEngine(model, ps, strat, grad_accum_steps=G, hp=dict(lr=1e-3), comm_backend=backend)
            prov = get_inputs_provider(cfg.model.name)
            for it in range(3):
                batches = [prov(2, 128, 1024, "cuda", seed=1000 * it + 10 * k + rank) for k in range(G)]
                eng.train_step(batches)
            eng.finish()
            torch.cuda.synchronize()
            native.check_status()
            finals[backend] = torch.cat([u.master.clone() for u in eng.units])
        diff = (finals["nccl"] - finals["fused"]).abs().max().item()
        scale = finals["nccl"].abs().max().item()
        ret[rank] = (diff, scale)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("zero_flags,G", [((False, False, True), 1), ((False, True, True), 1), ((False, True, True), 2)])
def test_fused_matches_nccl(zero_flags, G):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_worker, args=(world, port, zero_flags, G, ret), nprocs=world, join=True)
    for r in range(world):
        diff, scale = ret[r]
        # identical math up to bf16 rounding of the reduced gradient: Adam steps differ by
        # at most a few lr in rare sign flips
        assert diff < 5e-3, (diff, scale)
