"""1F1B pipeline over NCCL p2p on 2 GPUs: completes (no ordering deadlock) and trains."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mist_b200.utils.device import free_port

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=60))
    try:
        from mist_b200.api import TrainingSession
        from mist_b200.config import load_config
        from mist_b200.ops import native
        cfg, _ = load_config("config", ["experiment=gpt2-1.3b", "model.num_hidden_layers=4", "model.hidden_size=256",
                                        "model.intermediate_size=1024", "model.num_attention_heads=4",
                                        "training.max_sequence_length=128", "model.vocab_size=1024",
                                        "hardware.num_gpus_per_node=2", "training.global_batch_size=16",
                                        "strategy.layer_partitions=[2,2]", "strategy.device_assignment=[[1,1],[1,1]]",
                                        "strategy.gradient_checkpointing=[1,0]", "strategy.gradient_accumulation_steps=8",
                                        "strategy.stage_strategies=[[2,1,1,0,0,1,0,0,0,0],[2,1,1,0,0,1,0,0,0,0]]",
                                        "strategy.pre_post_strategy_array=[2,1,1,0,0,1,0,0,0,0]"])
        sess = TrainingSession(cfg, seed=0, hp=dict(lr=1e-3))
        g = torch.Generator().manual_seed(5)
        ids = torch.randint(0, 1024, (16, 128), generator=g).cuda()
        lab = torch.randint(0, 1024, (16, 128), generator=g).cuda()
        losses = [float(sess.step_on_device(ids, lab)) for _ in range(4)]
        sess.finish()
        torch.cuda.synchronize()
        native.check_status()
        ret[rank] = losses
    finally:
        dist.destroy_process_group()


def test_two_stage_pipeline_trains():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    port = free_port()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    losses = ret[1]                       # the last stage owns the loss
    assert all(l == l for l in losses) and losses[-1] < losses[0]
