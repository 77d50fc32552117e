"""The training engine against plain PyTorch on CPU: single rank and gloo data-parallel ranks
for every ZeRO level (losses and final weights must agree with an unsharded AdamW run)."""
import copy
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mist_b200.config import StageStrategy, load_config
from mist_b200.models.provider import base_model_provider, get_inputs_provider
from mist_b200.parallel.engine import TrainEngine
from mist_b200.parallel.state import ParallelState, build_plan

TINY = ["model.num_hidden_layers=3", "model.hidden_size=64", "model.intermediate_size=128",
        "model.num_attention_heads=4", "training.max_sequence_length=32", "model.vocab_size=256",
        "strategy.layer_partitions=[3]", "training.params_dtype=float32"]


def _tiny_model(exp="gpt2-1.3b", seed=0):
    cfg, _ = load_config("config", [f"experiment={exp}"] + TINY, check_world_size=False)
    torch.manual_seed(seed)
    return cfg, base_model_provider(cfg.model, device="cpu", dtype=torch.float32)


@pytest.mark.parametrize("exp", ["gpt2-1.3b", "llama-350m"])
@pytest.mark.parametrize("G,ckpt", [(1, 0), (2, 2)])
def test_single_rank_matches_adamw(exp, G, ckpt):
    cfg, model = _tiny_model(exp)
    ref = copy.deepcopy(model)
    eng = TrainEngine(model, grad_accum_steps=G, ckpt_layers=ckpt, hp=dict(lr=1e-3))
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    prov = get_inputs_provider(cfg.model.name)
    for it in range(3):
        batches = [prov(2, 32, 256, "cpu", seed=10 * it + k) for k in range(G)]
        loss = eng.train_step(batches)
        opt.zero_grad()
        ref_loss = 0.0
        for b in batches:
            l = ref(**b) / G
            l.backward()
            ref_loss += l.item()
        opt.step()
        assert abs(loss.item() - ref_loss) < 1e-4
    diff = max((a - b).abs().max().item() for a, b in zip(model.parameters(), ref.parameters()))
    assert diff < 1e-4


def _dp_worker(rank, world, port, zero_flags, G, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg, model = _tiny_model()
        plan = build_plan([(1, world)], [(2, world, 1)], (1, world))
        ps = ParallelState(plan, rank)
        strat = StageStrategy(2, world, 1, *zero_flags, 0, 0, 0, 0)
        eng = TrainEngine(model, ps, strat, grad_accum_steps=G, hp=dict(lr=1e-3))
        prov = get_inputs_provider(cfg.model.name)
        losses = []
        for it in range(3):
            batches = [prov(2, 32, 256, "cpu", seed=1000 * it + 10 * k + rank) for k in range(G)]
            losses.append(eng.train_step(batches).item())
        if eng.zero3:
            for u in eng.units:
                if u.param_shard is not None and u.flat_param is None:
                    u.unshard(torch.empty(u.padded), ps.dp_ag_group)
        flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
        if rank == 0:
            ret["flat"] = flat.clone()
            ret["losses"] = losses
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("zero_flags", [(False, False, False), (False, False, True), (False, True, True),
                                        (True, True, True)])
@pytest.mark.parametrize("G", [1, 2])
def test_data_parallel_gloo_matches_single_process(zero_flags, G):
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() + hash((zero_flags, G))) % 2000
    mp.spawn(_dp_worker, args=(world, port, zero_flags, G, ret), nprocs=world, join=True)
    # reference: one process sees both ranks' micro batches
    cfg, ref = _tiny_model()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    prov = get_inputs_provider(cfg.model.name)
    for it in range(3):
        opt.zero_grad()
        for k in range(G):
            for r in range(world):
                (ref(**prov(2, 32, 256, "cpu", seed=1000 * it + 10 * k + r)) / (G * world)).backward()
        opt.step()
    flat_ref = torch.cat([p.detach().reshape(-1) for p in ref.parameters()])
    assert (ret["flat"] - flat_ref).abs().max().item() < 2e-4
