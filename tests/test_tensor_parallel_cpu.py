"""Tensor parallelism (with and without sequence parallelism) on two gloo ranks against a
single-process model with the same weights: losses of two training steps and the updated
weights must agree.  The single-process weights are cut into each rank's slices the way the
modules shard them (heads for the fused QKV projection, matching gate / up halves for the gated
MLP, rows or columns for the other linears, vocabulary rows for embedding and head)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mist_b200.utils.device import free_port
from mist_b200.config import load_config
from mist_b200.models.provider import base_model_provider, get_inputs_provider

TINY = ["model.num_hidden_layers=2", "model.hidden_size=64", "model.intermediate_size=128",
        "model.num_attention_heads=4", "training.max_sequence_length=32", "model.vocab_size=256",
        "strategy.layer_partitions=[2]", "training.params_dtype=float32", "hardware.num_gpus_per_node=2",
        "training.global_batch_size=4", "strategy.device_assignment=[[1,2]]", "strategy.gradient_checkpointing=[1]",
        "strategy.gradient_accumulation_steps=2", "strategy.stage_strategies=[[2,1,2,0,0,0,0,0,0,0]]",
        "strategy.pre_post_strategy_array=[2,1,2,0,0,0,0,0,0,0]"]


def shard_like(name: str, full: torch.Tensor, rank: int, world: int, heads: int) -> torch.Tensor:
    """The slice of a single-process parameter that tensor-parallel rank ``rank`` holds."""
    if "cross_attn.Wkv" in name:                               # [k | v], each split by heads
        d = full.shape[0] // (2 * heads)
        lh = heads // world
        return full.view(2, heads, d, *full.shape[1:])[:, rank * lh:(rank + 1) * lh].reshape(2 * lh * d, *full.shape[1:])
    if "cross_attn.Wq" in name or name == "lm_head.bias":     # heads / vocabulary rows are contiguous
        return full.chunk(world, dim=0)[rank]
    if "Wqkv" in name:
        d = full.shape[0] // (3 * heads)
        lh = heads // world
        v = full.view(3, heads, d, *full.shape[1:])[:, rank * lh:(rank + 1) * lh]
        return v.reshape(3 * lh * d, *full.shape[1:])
    if "mlp.fc1" in name and full.shape[0] == 256:            # gated MLP: [gate | up]
        f = full.shape[0] // 2
        lf = f // world
        return full.view(2, f, *full.shape[1:])[:, rank * lf:(rank + 1) * lf].reshape(2 * lf, *full.shape[1:])
    if any(k in name for k in ("mlp.fc1", "word_embeddings", "lm_head.proj")):
        return full.chunk(world, dim=0)[rank]
    if any(k in name for k in ("out_proj.weight", "mlp.fc2.weight")):
        return full.chunk(world, dim=1)[rank]
    return full                                                # norms, position embeddings, row-parallel biases


def _worker(rank, world, port, exp, sp, ref_state, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mist_b200.api import TrainingSession
        cfg, _ = load_config("config", [f"experiment={exp}"] + TINY + [f"sequence_parallel={'true' if sp else 'false'}"],
                             check_world_size=False)
        sess = TrainingSession(cfg, seed=0, device=torch.device("cpu"), hp=dict(lr=1e-3))
        assert sess.ps.tp_size == 2
        with torch.no_grad():
            for n, p in sess.model.named_parameters():
                p.copy_(shard_like(n, ref_state[n], rank, world, 4))
        for u in sess.engine.units:                             # optimizer state follows the new weights
            u.master.copy_(u.flat_param.float())
        prov = get_inputs_provider(cfg.model.name)
        losses = []
        for it in range(2):
            b = prov(4, 32, 256, "cpu", seed=50 + it)
            losses.append(float(sess.step_on_device(b["input_ids"], b["labels"])))
        sess.finish()
        ret[rank] = (losses, {n: p.detach().clone() for n, p in sess.model.named_parameters()})
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exp", ["gpt2-1.3b", "llama-350m"])
@pytest.mark.parametrize("sp", [False, True])
def test_tp2_matches_single_process(exp, sp):
    cfg, _ = load_config("config", [f"experiment={exp}"] + TINY[:8], check_world_size=False)
    torch.manual_seed(3)
    ref = base_model_provider(cfg.model, device="cpu", dtype=torch.float32)
    ref_state = {n: p.detach().clone() for n, p in ref.named_parameters()}
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_worker, args=(2, port, exp, sp, ref_state, ret), nprocs=2, join=True)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    prov = get_inputs_provider(cfg.model.name)
    for it in range(2):
        b = prov(4, 32, 256, "cpu", seed=50 + it)
        opt.zero_grad()
        tot = 0.0
        for k in range(2):                                       # two micro batches of two sequences
            mbatch = {key: v[2 * k: 2 * k + 2] for key, v in b.items()}
            l = ref(**mbatch) / 2
            l.backward()
            tot += l.item()
        opt.step()
        for r in range(2):
            assert abs(ret[r][0][it] - tot) < 2e-4, (r, it, ret[r][0], tot)
    new_state = dict(ref.named_parameters())
    for r in range(2):
        for n, p in ret[r][1].items():
            want = shard_like(n, new_state[n].detach(), r, 2, 4)
            assert (p - want).abs().max().item() < 2e-4, (r, n)


def _hetero_worker(rank, world, port, ref_state, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mist_b200.api import TrainingSession
        cfg, _ = load_config("config", ["experiment=gpt2-1.3b"] + TINY[:8] + [
            "hardware.num_gpus_per_node=4", "training.global_batch_size=4", "strategy.layer_partitions=[1,1]",
            "strategy.device_assignment=[[1,2],[1,2]]", "strategy.gradient_checkpointing=[0,1]",
            "strategy.gradient_accumulation_steps=2",
            "strategy.stage_strategies=[[1,2,1,0,0,1,0,0,0,0],[2,1,2,0,0,0,0,0,0,0]]",
            "strategy.pre_post_strategy_array=[1,2,1,0,0,1,0,0,0,0]"], check_world_size=False)
        sess = TrainingSession(cfg, seed=0, device=torch.device("cpu"), hp=dict(lr=1e-3))
        ps = sess.ps
        with torch.no_grad():
            for n, p in sess.model.named_parameters():
                gname = n.replace("layers.0.", f"layers.{ps.stage}.")
                p.copy_(shard_like(n, ref_state[gname], ps.tp_rank, ps.tp_size, 4))
        for u in sess.engine.units:
            src = u.flat_param[u.shard_range()] if u.sharded_state else u.flat_param
            u.master.copy_(src.float())
        prov = get_inputs_provider(cfg.model.name)
        losses = []
        for it in range(2):
            # stage 0 is data parallel over two ranks with micro batch 1: rank r of the stage feeds
            # sequences r, 2 + r (micro step k takes sequence 2 k + r); stage 1 sees both per micro step
            b = prov(4, 32, 256, "cpu", seed=70 + it)
            if ps.stage == 0:
                idx = torch.tensor([ps.dp_rank, 2 + ps.dp_rank])
            else:
                idx = torch.arange(4)
            losses.append(float(sess.step_on_device(b["input_ids"][idx], b["labels"][idx])))
        sess.finish()
        ret[rank] = (ps.stage, ps.tp_rank, ps.tp_size, losses,
                     {n.replace("layers.0.", f"layers.{ps.stage}."): p.detach().clone()
                      for n, p in sess.model.named_parameters()})
    finally:
        dist.destroy_process_group()


def test_heterogeneous_pipeline_dp2_then_tp2_matches_single_process():
    """Two pipeline stages with different layouts on four ranks: stage 0 is data parallel (two
    ranks, micro batch 1, ZeRO-1), stage 1 tensor parallel (two ranks, micro batch 2); the
    activations are re-sharded along the batch between them."""
    cfg, _ = load_config("config", ["experiment=gpt2-1.3b"] + TINY[:8], check_world_size=False)
    torch.manual_seed(4)
    ref = base_model_provider(cfg.model, device="cpu", dtype=torch.float32)
    ref_state = {n: p.detach().clone() for n, p in ref.named_parameters()}
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_hetero_worker, args=(4, port, ref_state, ret), nprocs=4, join=True)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    prov = get_inputs_provider(cfg.model.name)
    for it in range(2):
        b = prov(4, 32, 256, "cpu", seed=70 + it)
        opt.zero_grad()
        tot = 0.0
        for k in range(2):
            mbatch = {key: v[2 * k: 2 * k + 2] for key, v in b.items()}
            l = ref(**mbatch) / 2
            l.backward()
            tot += l.item()
        opt.step()
        for r in range(4):
            stage, _, _, losses, _ = ret[r]
            if stage == 1:
                assert abs(losses[it] - tot) < 2e-4, (r, it, losses, tot)
    new_state = dict(ref.named_parameters())
    for r in range(4):
        stage, tpr, tps, _, params = ret[r]
        for n, p in params.items():
            want = shard_like(n, new_state[n].detach(), tpr, tps, 4)
            assert (p - want).abs().max().item() < 2e-4, (r, n)


def _pptp_worker(rank, world, port, sp, ref_state, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mist_b200.api import TrainingSession
        cfg, _ = load_config("config", ["experiment=llama-350m"] + TINY[:8] + [
            "hardware.num_gpus_per_node=4", "training.global_batch_size=4", "strategy.layer_partitions=[1,1]",
            "strategy.device_assignment=[[1,2],[1,2]]", "strategy.gradient_checkpointing=[1,0]",
            "strategy.gradient_accumulation_steps=2",
            "strategy.stage_strategies=[[2,1,2,0,0,0,0,0,0,0],[2,1,2,0,0,0,0,0,0,0]]",
            "strategy.pre_post_strategy_array=[2,1,2,0,0,0,0,0,0,0]",
            f"sequence_parallel={'true' if sp else 'false'}"], check_world_size=False)
        sess = TrainingSession(cfg, seed=0, device=torch.device("cpu"), hp=dict(lr=1e-3))
        ps = sess.ps
        with torch.no_grad():
            for n, p in sess.model.named_parameters():
                gname = n.replace("layers.0.", f"layers.{ps.stage}.")
                p.copy_(shard_like(n, ref_state[gname], ps.tp_rank, ps.tp_size, 4))
        for u in sess.engine.units:
            u.master.copy_(u.flat_param.float())
        prov = get_inputs_provider(cfg.model.name)
        losses = []
        for it in range(2):
            b = prov(4, 32, 256, "cpu", seed=90 + it)
            losses.append(float(sess.step_on_device(b["input_ids"], b["labels"])))
        sess.finish()
        ret[rank] = (ps.stage, ps.tp_rank, ps.tp_size, losses,
                     {n.replace("layers.0.", f"layers.{ps.stage}."): p.detach().clone()
                      for n, p in sess.model.named_parameters()})
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("sp", [False, True])
def test_pipeline_of_tensor_parallel_stages_matches_single_process(sp):
    cfg, _ = load_config("config", ["experiment=llama-350m"] + TINY[:8], check_world_size=False)
    torch.manual_seed(5)
    ref = base_model_provider(cfg.model, device="cpu", dtype=torch.float32)
    ref_state = {n: p.detach().clone() for n, p in ref.named_parameters()}
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_pptp_worker, args=(4, port, sp, ref_state, ret), nprocs=4, join=True)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    prov = get_inputs_provider(cfg.model.name)
    for it in range(2):
        b = prov(4, 32, 256, "cpu", seed=90 + it)
        opt.zero_grad()
        tot = 0.0
        for k in range(2):
            mbatch = {key: v[2 * k: 2 * k + 2] for key, v in b.items()}
            l = ref(**mbatch) / 2
            l.backward()
            tot += l.item()
        opt.step()
        for r in range(4):
            if ret[r][0] == 1:
                assert abs(ret[r][3][it] - tot) < 2e-4, (r, it, ret[r][3], tot)
    new_state = dict(ref.named_parameters())
    for r in range(4):
        _, tpr, tps, _, params = ret[r]
        for n, p in params.items():
            want = shard_like(n, new_state[n].detach(), tpr, tps, 4)
            assert (p - want).abs().max().item() < 2e-4, (r, n)


def _dptp_worker(rank, world, port, zero, ref_state, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mist_b200.api import TrainingSession
        vec = f"[1,2,2,{zero[0]},{zero[1]},{zero[2]},0,0,0,0]"
        cfg, _ = load_config("config", ["experiment=gpt2-1.3b"] + TINY[:8] + [
            "hardware.num_gpus_per_node=4", "training.global_batch_size=4", "strategy.layer_partitions=[2]",
            "strategy.device_assignment=[[1,4]]", "strategy.gradient_checkpointing=[0]",
            "strategy.gradient_accumulation_steps=2", f"strategy.stage_strategies=[{vec}]",
            f"strategy.pre_post_strategy_array={vec}", "sequence_parallel=true"], check_world_size=False)
        sess = TrainingSession(cfg, seed=0, device=torch.device("cpu"), hp=dict(lr=1e-3))
        ps = sess.ps
        with torch.no_grad():
            for u in sess.engine.units:          # ZeRO-3 units: fill the persistent shard from the full weights
                full = torch.zeros(u.padded)
                for p, o, n in zip(u.params, u.offsets, u.param_names):
                    name = n if u.name in ("pre", "post") else f"language_model.encoder.layers.{u.name[5:]}.{n}"
                    name = name.replace("embedding.", "language_model.embedding.") if u.name == "pre" else name
                    full[o:o + p.numel()] = shard_like(name, ref_state[name], ps.tp_rank, 2, 4).reshape(-1)
                if u.param_shard is not None:
                    u.param_shard.copy_(full[u.shard_range()])
                    if u.flat_param is not None:
                        u.flat_param.copy_(full)
                else:
                    u.flat_param.copy_(full)
                u.master.copy_(full[u.shard_range()] if u.sharded_state else full)
        prov = get_inputs_provider(cfg.model.name)
        losses = []
        for it in range(2):
            b = prov(4, 32, 256, "cpu", seed=110 + it)
            idx = torch.tensor([ps.dp_rank, 2 + ps.dp_rank])       # micro step k of dp rank d: sequence 2 k + d
            losses.append(float(sess.step_on_device(b["input_ids"][idx], b["labels"][idx])))
        sess.finish()
        out = {}
        for u in sess.engine.units:
            if u.ring_resident and u.flat_param is None:
                u.unshard(torch.empty(u.padded), ps.dp_ag_group)
            for p, o, n in zip(u.params, u.offsets, u.param_names):
                name = n if u.name in ("pre", "post") else f"language_model.encoder.layers.{u.name[5:]}.{n}"
                name = name.replace("embedding.", "language_model.embedding.") if u.name == "pre" else name
                out[name] = u.flat_param[o:o + p.numel()].detach().clone().view(p.shape)
        ret[rank] = (ps.tp_rank, ps.dp_rank, losses, out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("zero", [(0, 0, 1), (0, 1, 1), (1, 1, 1)])
def test_dp2_x_tp2_sequence_parallel_with_zero_matches_single_process(zero):
    cfg, _ = load_config("config", ["experiment=gpt2-1.3b"] + TINY[:8], check_world_size=False)
    torch.manual_seed(6)
    ref = base_model_provider(cfg.model, device="cpu", dtype=torch.float32)
    ref_state = {n: p.detach().clone() for n, p in ref.named_parameters()}
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_dptp_worker, args=(4, port, zero, ref_state, ret), nprocs=4, join=True)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    prov = get_inputs_provider(cfg.model.name)
    for it in range(2):
        b = prov(4, 32, 256, "cpu", seed=110 + it)
        opt.zero_grad()
        per_rank = {0: 0.0, 1: 0.0}
        for s in range(4):
            l = ref(**{k: v[s:s + 1] for k, v in b.items()}) / 4
            l.backward()
            per_rank[s % 2] += l.item() * 2                       # a dp rank reports the mean over its own two
        opt.step()
        for r in range(4):
            assert abs(ret[r][2][it] - per_rank[ret[r][1]]) < 2e-4, (r, it, ret[r][2], per_rank)
    new_state = dict(ref.named_parameters())
    for r in range(4):
        tpr = ret[r][0]
        for n, p in ret[r][3].items():
            want = shard_like(n, new_state[n].detach(), tpr, 2, 4)
            assert (p - want).abs().max().item() < 2e-4, (r, n)


def _family_worker(rank, world, port, fam, sp, ref_state, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mist_b200.api import TrainingSession
        cfg, _ = load_config("config", ["experiment=gpt2-1.3b", f"model={fam}"] + TINY +
                             [f"sequence_parallel={'true' if sp else 'false'}"], check_world_size=False)
        sess = TrainingSession(cfg, seed=0, device=torch.device("cpu"), hp=dict(lr=1e-3))
        with torch.no_grad():
            for n, p in sess.model.named_parameters():
                p.copy_(shard_like(n, ref_state[n], rank, world, 4))
        for u in sess.engine.units:
            u.master.copy_(u.flat_param.float())
        prov = get_inputs_provider(cfg.model.name)
        losses = []
        for it in range(2):
            losses.append(float(sess.step_on_device_batch(prov(4, 32, 256, "cpu", seed=130 + it))))
        sess.finish()
        ret[rank] = (losses, {n: p.detach().clone() for n, p in sess.model.named_parameters()})
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fam", ["bert/1.3b", "t5/1.7b", "falcon/1.3b"])
@pytest.mark.parametrize("sp", [False, True])
def test_tp2_other_families_match_single_process(fam, sp):
    cfg, _ = load_config("config", ["experiment=gpt2-1.3b", f"model={fam}"] + TINY[:8], check_world_size=False)
    torch.manual_seed(7)
    ref = base_model_provider(cfg.model, device="cpu", dtype=torch.float32)
    ref_state = {n: p.detach().clone() for n, p in ref.named_parameters()}
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_family_worker, args=(2, port, fam, sp, ref_state, ret), nprocs=2, join=True)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    prov = get_inputs_provider(cfg.model.name)
    for it in range(2):
        b = prov(4, 32, 256, "cpu", seed=130 + it)
        opt.zero_grad()
        tot = 0.0
        for k in range(2):
            l = ref(**{key: v[2 * k: 2 * k + 2] for key, v in b.items()}) / 2
            l.backward()
            tot += l.item()
        opt.step()
        for r in range(2):
            assert abs(ret[r][0][it] - tot) < 2e-4, (r, it, ret[r][0], tot)
    new_state = dict(ref.named_parameters())
    for r in range(2):
        for n, p in ret[r][1].items():
            want = shard_like(n, new_state[n].detach(), r, 2, 4)
            assert (p - want).abs().max().item() < 2e-4, (r, n)


def _gen_worker(rank, world, port, ref_state, prompt, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mist_b200.inference import generate
        cfg, _ = load_config("config", ["experiment=llama-350m"] + TINY[:8] + ["model.rotary_emb_fraction=1.0"],
                             check_world_size=False)
        group = dist.new_group([0, 1])
        torch.manual_seed(0)
        model = base_model_provider(cfg.model, process_groups=group, pre_post_process_group=group, device="cpu",
                                    dtype=torch.float32)
        with torch.no_grad():
            for n, p in model.named_parameters():
                p.copy_(shard_like(n, ref_state[n], rank, world, 4))
        ret[rank] = generate(model, prompt, max_new_tokens=5, tp_group=group)
    finally:
        dist.destroy_process_group()


def test_tp2_cached_generation_matches_single_process():
    from mist_b200.inference import generate
    cfg, _ = load_config("config", ["experiment=llama-350m"] + TINY[:8] + ["model.rotary_emb_fraction=1.0"],
                         check_world_size=False)
    torch.manual_seed(8)
    ref = base_model_provider(cfg.model, device="cpu", dtype=torch.float32).eval()
    ref_state = {n: p.detach().clone() for n, p in ref.named_parameters()}
    prompt = torch.randint(0, 256, (2, 6))
    want = generate(ref, prompt, max_new_tokens=5)
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_gen_worker, args=(2, port, ref_state, prompt, ret), nprocs=2, join=True)
    assert torch.equal(ret[0], want) and torch.equal(ret[1], want)


def _hetero2_worker(rank, world, port, ref_state, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mist_b200.api import TrainingSession
        cfg, _ = load_config("config", ["experiment=gpt2-1.3b"] + TINY[:8] + [
            "hardware.num_gpus_per_node=3", "training.global_batch_size=4", "strategy.layer_partitions=[1,1]",
            "strategy.device_assignment=[[1,1],[1,2]]", "strategy.gradient_checkpointing=[0,0]",
            "strategy.gradient_accumulation_steps=2",
            "strategy.stage_strategies=[[2,1,1,0,0,0,0,0,0,0],[1,2,1,0,1,1,0,0,0,0]]",
            "strategy.pre_post_strategy=heuristic"], check_world_size=False)   # first and last stage differ in size
        sess = TrainingSession(cfg, seed=0, device=torch.device("cpu"), hp=dict(lr=1e-3))
        ps = sess.ps
        with torch.no_grad():
            for n, p in sess.model.named_parameters():
                p.copy_(ref_state[n.replace("layers.0.", f"layers.{ps.stage}.")])
        for u in sess.engine.units:
            src = u.flat_param[u.shard_range()] if u.sharded_state else u.flat_param
            u.master.copy_(src.float())
        prov = get_inputs_provider(cfg.model.name)
        losses = []
        for it in range(2):
            b = prov(4, 32, 256, "cpu", seed=170 + it)
            idx = torch.arange(4) if ps.stage == 0 else torch.tensor([ps.dp_rank, 2 + ps.dp_rank])
            losses.append(float(sess.step_on_device(b["input_ids"][idx], b["labels"][idx])))
        sess.finish()
        ret[rank] = (ps.stage, ps.dp_rank, losses,
                     {n.replace("layers.0.", f"layers.{ps.stage}."): p.detach().clone()
                      for n, p in sess.model.named_parameters()})
    finally:
        dist.destroy_process_group()


def test_heterogeneous_pipeline_wide_stage_feeds_two_data_parallel_ranks():
    """Stage 0 runs micro batches of two sequences on one rank and splits each between the two
    data-parallel ranks of stage 1 (micro batch 1, ZeRO-2); gradients come back as two halves."""
    cfg, _ = load_config("config", ["experiment=gpt2-1.3b"] + TINY[:8], check_world_size=False)
    torch.manual_seed(9)
    ref = base_model_provider(cfg.model, device="cpu", dtype=torch.float32)
    ref_state = {n: p.detach().clone() for n, p in ref.named_parameters()}
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_hetero2_worker, args=(3, port, ref_state, ret), nprocs=3, join=True)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    prov = get_inputs_provider(cfg.model.name)
    for it in range(2):
        b = prov(4, 32, 256, "cpu", seed=170 + it)
        opt.zero_grad()
        per_dp = {0: 0.0, 1: 0.0}
        for s in range(4):
            l = ref(**{k: v[s:s + 1] for k, v in b.items()}) / 4
            l.backward()
            per_dp[s % 2] += 2 * l.item()
        opt.step()
        for r in range(3):
            stage, d, losses, _ = ret[r]
            if stage == 1:
                assert abs(losses[it] - per_dp[d]) < 2e-4, (r, it, losses, per_dp)
    new_state = dict(ref.named_parameters())
    for r in range(3):
        for n, p in ret[r][3].items():
            assert (p - new_state[n].detach()).abs().max().item() < 2e-4, (r, n)


def _smooth_worker(rank, world, port, logits, labels, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mist_b200.modules.layers import vocab_parallel_cross_entropy
        group = dist.new_group([0, 1])
        per = logits.shape[1] // world
        local = logits[:, rank * per:(rank + 1) * per].clone().requires_grad_(True)
        loss = vocab_parallel_cross_entropy(local, labels, group, label_smoothing=0.2)
        loss.sum().backward()
        ret[rank] = (loss.detach().clone(), local.grad.clone())
    finally:
        dist.destroy_process_group()


def test_label_smoothing_over_vocabulary_shards():
    from mist_b200.modules.layers import vocab_parallel_cross_entropy
    torch.manual_seed(0)
    logits = torch.randn(6, 32)
    labels = torch.randint(0, 32, (6,))
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_smooth_worker, args=(2, free_port(), logits, labels, ret), nprocs=2, join=True)
    full = logits.clone().requires_grad_(True)
    want = vocab_parallel_cross_entropy(full, labels, label_smoothing=0.2)
    want.sum().backward()
    for r in range(2):
        assert torch.allclose(ret[r][0], want.detach(), atol=1e-5)
        assert torch.allclose(ret[r][1], full.grad[:, r * 16:(r + 1) * 16], atol=1e-5)
