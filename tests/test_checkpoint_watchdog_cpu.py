"""Checkpoint save / resume (with a change of ZeRO level in between) and host-side failure
detection, on CPU with gloo ranks.  No GPU is involved: a "failed" rank is one that stops
beating or exits between steps."""
import os
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mist_b200.utils.device import free_port
from mist_b200.config import load_config
from mist_b200.models.provider import get_inputs_provider

TINY = ["model.num_hidden_layers=3", "model.hidden_size=64", "model.intermediate_size=128",
        "model.num_attention_heads=4", "training.max_sequence_length=32", "model.vocab_size=256",
        "strategy.layer_partitions=[3]", "training.params_dtype=float32", "hardware.num_gpus_per_node=2",
        "training.global_batch_size=8", "strategy.device_assignment=[[1,2]]", "strategy.gradient_checkpointing=[0]",
        "strategy.gradient_accumulation_steps=2"]


def _cfg(zero, offload=(0, 0, 0)):
    vec = f"[2,2,1,{zero[0]},{zero[1]},{zero[2]},{offload[0]},{offload[1]},{offload[2]},0]"
    cfg, _ = load_config("config", ["experiment=gpt2-1.3b"] + TINY + [
        f"strategy.stage_strategies=[{vec}]", f"strategy.pre_post_strategy_array={vec}"], check_world_size=False)
    return cfg


def _ckpt_worker(rank, world, port, path, ret, first=((0, 1, 1), (0, 0, 0)), second=((1, 1, 1), (0, 0, 0))):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mist_b200.api import TrainingSession
        from mist_b200.utils import checkpoint
        prov = get_inputs_provider("gpt2")

        def batch(it):
            b = prov(4, 32, 256, "cpu", seed=1000 * it + rank)
            return b["input_ids"], b["labels"]

        # run A: ZeRO-2 for two steps, save, one more step
        a = TrainingSession(_cfg(*first), seed=0, device=torch.device("cpu"), hp=dict(lr=1e-3))
        for it in range(2):
            a.step_on_device(*batch(it))
        a.finish()
        checkpoint.save(a, path, step=2)
        loss_a = float(a.step_on_device(*batch(2)))
        a.finish()
        # run B: ZeRO-3 from another seed, resume, same third step
        b = TrainingSession(_cfg(*second), seed=123, device=torch.device("cpu"), hp=dict(lr=1e-3))
        step = checkpoint.load(b, path)
        loss_b = float(b.step_on_device(*batch(2)))
        b.finish()

        def full_weights(sess):
            out = []
            for u in sess.engine.units:
                if u.ring_resident and u.flat_param is None:
                    u.unshard(torch.empty(u.padded), sess.ps.dp_ag_group if u.is_zero3 else None,
                              streams=sess.engine.swap_streams)
                out.append(u.flat_param[: u.numel].detach().clone())
            return torch.cat(out)

        wa, wb = full_weights(a), full_weights(b)
        if rank == 0:
            ret["step"] = step
            ret["losses"] = (loss_a, loss_b)
            ret["diff"] = (wa - wb).abs().max().item()
            ret["files"] = sorted(os.listdir(path))
    finally:
        dist.destroy_process_group()


def test_checkpoint_resume_under_another_zero_level(tmp_path):
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_ckpt_worker, args=(world, port, str(tmp_path / "ckpt"), ret), nprocs=world, join=True)
    assert ret["step"] == 2
    assert "meta.json" in ret["files"] and "strategy.yaml" in ret["files"]
    assert any(f.startswith("model_stage0") for f in ret["files"])
    assert abs(ret["losses"][0] - ret["losses"][1]) < 1e-5
    assert ret["diff"] < 1e-5
    # one optimizer file per data-parallel rank (each holds that rank's shard and RNG state)
    assert "optim_stage0_tp0_dp0.pt" in ret["files"] and "optim_stage0_tp0_dp1.pt" in ret["files"]


@pytest.mark.parametrize("first,second", [
    # ZeRO-3 with half of the weights, gradients and optimizer state on the host -> plain ZeRO-1
    (((1, 1, 1), (0.5, 0.5, 0.5)), ((0, 0, 1), (0, 0, 0))),
    # ZeRO-2 -> ZeRO-3 with offloaded weights and optimizer state (load writes through the host split)
    (((0, 1, 1), (0, 0, 0)), ((1, 1, 1), (0.5, 0.5, 0.5))),
    # ZeRO-2 with offloaded weights -> the same
    (((0, 1, 1), (0.5, 0.5, 0)), ((0, 1, 1), (0.5, 0.5, 0))),
])
def test_checkpoint_roundtrip_with_offloaded_state(tmp_path, first, second):
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_ckpt_worker, args=(world, port, str(tmp_path / "ckpt"), ret, first, second), nprocs=world, join=True)
    assert ret["step"] == 2
    assert abs(ret["losses"][0] - ret["losses"][1]) < 1e-5
    assert ret["diff"] < 1e-5


def test_checkpoint_restores_rng_per_rank(tmp_path):
    """Each rank's optimizer file carries its own CPU generator state; loading puts it back."""
    from mist_b200.api import TrainingSession
    from mist_b200.utils import checkpoint
    cfg, _ = load_config("config", ["experiment=gpt2-1.3b"] + TINY + [
        "hardware.num_gpus_per_node=1", "strategy.device_assignment=[[1,1]]", "training.global_batch_size=4",
        "strategy.stage_strategies=[[2,1,1,0,0,0,0,0,0,0]]", "strategy.pre_post_strategy_array=[2,1,1,0,0,0,0,0,0,0]"],
        check_world_size=False)
    a = TrainingSession(cfg, seed=0, device=torch.device("cpu"))
    torch.manual_seed(4242)
    checkpoint.save(a, str(tmp_path / "c"), step=5)
    expect = torch.rand(3)
    torch.manual_seed(1)
    assert checkpoint.load(a, str(tmp_path / "c")) == 5
    assert torch.equal(torch.rand(3), expect)


def _hb_worker(rank, world, port, ret):
    from mist_b200.utils.watchdog import Heartbeat
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=30))
    hb = Heartbeat(store, rank, world)
    store.set(f"ready/{rank}", "1")
    for r in range(world):
        store.wait([f"ready/{r}"])
    if rank == 1:
        # this rank "fails" between steps: it stops beating and leaves
        store.set("left/1", "1")
        store.wait(["done/0"])
        return
    store.wait(["left/1"])
    for _ in range(3):
        hb.beat()
        time.sleep(0.3)
    stale = hb.stale_ranks(max_age_s=0.5)
    raised = False
    try:
        hb.check(max_age_s=0.5)
    except RuntimeError:
        raised = True
    ret["stale"] = stale
    ret["raised"] = raised
    ret["pids"] = hb.pids()
    store.set("done/0", "1")


def test_heartbeat_reports_a_rank_that_stopped():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_hb_worker, args=(world, port, ret), nprocs=world, join=True)
    assert ret["stale"] == [1]
    assert ret["raised"]
    assert set(ret["pids"].keys()) == {0, 1}


def test_bounded_wait_status_names():
    """The host side of the device status word: codes map to messages (the device side is
    covered by the GPU tests, where every wait has a time limit)."""
    from mist_b200.ops import native
    assert native._STATUS_NAMES[4].startswith("peer flag")
    assert set(native._STATUS_NAMES) == {1, 2, 3, 4, 5}


def test_p2p_metadata_roundtrip_and_limits():
    from mist_b200.parallel.pipeline import META_LEN, decode_meta, encode_meta
    t = torch.zeros(2, 3, 5, dtype=torch.bfloat16, requires_grad=True)
    vec = encode_meta(t)
    assert len(vec) == META_LEN
    shape, dtype, rg = decode_meta(vec)
    assert shape == (2, 3, 5) and dtype == torch.bfloat16 and rg
    with pytest.raises(AssertionError):
        encode_meta(torch.zeros(1, 1, 1, 1, 1, 1, 1))         # more than 6 dimensions
    with pytest.raises(KeyError):
        encode_meta(torch.zeros(2, dtype=torch.float64))      # dtype without a wire code


def _leaver_worker(rank, world, port, ret):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    x = torch.ones(4)
    dist.all_reduce(x)              # step 1: everybody is there
    if rank == 1:
        os._exit(0)                 # leaves between steps, nothing in flight
    t0 = time.time()
    try:
        dist.all_reduce(x)          # step 2: the peer is gone
        ret["outcome"] = "completed"
    except Exception as e:          # noqa: BLE001 - the point is that it raises instead of hanging
        ret["outcome"] = type(e).__name__
    ret["seconds"] = time.time() - t0
    os._exit(0)


def test_collective_after_a_rank_left_raises_within_the_timeout():
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_leaver_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive()
    assert ret["outcome"] != "completed"
    assert ret["seconds"] < 30


def _ckpt_pptp_worker(rank, world, port, path, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mist_b200.api import TrainingSession
        from mist_b200.utils import checkpoint
        cfg, _ = load_config("config", ["experiment=gpt2-1.3b"] + TINY[:8] + [
            "model.num_hidden_layers=2", "hardware.num_gpus_per_node=4", "training.global_batch_size=4",
            "strategy.layer_partitions=[1,1]", "strategy.device_assignment=[[1,2],[1,2]]",
            "strategy.gradient_checkpointing=[0,0]", "strategy.gradient_accumulation_steps=2",
            "strategy.stage_strategies=[[2,1,2,0,0,0,0,0,0,0],[2,1,2,0,0,0,0,0,0,0]]",
            "strategy.pre_post_strategy_array=[2,1,2,0,0,0,0,0,0,0]"], check_world_size=False)
        prov = get_inputs_provider("gpt2")

        def batch(it):
            b = prov(4, 32, 256, "cpu", seed=500 + it)
            return b["input_ids"], b["labels"]

        a = TrainingSession(cfg, seed=0, device=torch.device("cpu"), hp=dict(lr=1e-3))
        a.step_on_device(*batch(0))
        a.finish()
        checkpoint.save(a, path, step=1)
        loss_a = float(a.step_on_device(*batch(1)))
        b = TrainingSession(cfg, seed=99, device=torch.device("cpu"), hp=dict(lr=1e-3))
        step = checkpoint.load(b, path)
        loss_b = float(b.step_on_device(*batch(1)))
        ret[rank] = (step, loss_a, loss_b, a.ps.stage)
        if rank == 0:
            ret["files"] = sorted(os.listdir(path))
    finally:
        dist.destroy_process_group()


def test_checkpoint_roundtrip_pipeline_of_tensor_parallel_stages(tmp_path):
    """Two pipeline stages of two tensor-parallel ranks: one model / optimizer file per (stage, tp
    rank), and a fresh session resumed from them continues with the same loss."""
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_ckpt_pptp_worker, args=(4, port, str(tmp_path / "ck"), ret), nprocs=4, join=True)
    for s in range(2):
        for t in range(2):
            assert f"model_stage{s}_tp{t}.pt" in ret["files"] and f"optim_stage{s}_tp{t}_dp0.pt" in ret["files"]
    for r in range(4):
        step, la, lb, stage = ret[r]
        assert step == 1
        if stage == 1:
            assert abs(la - lb) < 1e-5, (r, la, lb)


class _DictStore:
    """In-memory stand-in for the job's key-value store."""

    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_terminate_job_signals_only_this_hosts_live_ranks(monkeypatch):
    """Ranks registered from another host, and PIDs that now belong to another process, are left
    alone; the abort key tells the other hosts' ranks to stop at their next check."""
    from mist_b200.utils import watchdog
    store = _DictStore()
    me = watchdog.Heartbeat(store, 0, 4, host="node-a")
    watchdog.Heartbeat(store, 1, 4, host="node-a")
    other = watchdog.Heartbeat(store, 2, 4, host="node-b")
    watchdog.Heartbeat(store, 3, 4, host="node-a")
    # rank 3's PID was recycled: its recorded start time no longer matches
    pid3, host3, _ = store.get("hb/pid/3").decode().split("|")
    store.set("hb/pid/3", f"{pid3}|{host3}|1")
    sent = []
    monkeypatch.setattr(watchdog.os, "kill", lambda pid, sig: sent.append((pid, sig)))
    signalled = watchdog.terminate_job(me)
    assert signalled == [1]
    assert len(sent) == 1
    assert other.aborted()
    with pytest.raises(RuntimeError, match="asked the job to stop"):
        other.check(max_age_s=1e9)
