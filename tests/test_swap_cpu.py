"""Host-offload building blocks on CPU (where "host" and "device" are both ordinary memory, so
only the bookkeeping is exercised): split tensors, the activation swapper and an
engine run with activation offloading."""
import copy

import pytest
import torch

from mist_b200.parallel.swap import ActivationSwapper, SplitTensor, SwapStreams


def test_split_tensor_roundtrip():
    streams = SwapStreams("cpu")
    full = torch.arange(4096, dtype=torch.float32)
    sp = SplitTensor(full, 0.5)
    assert sp.host_numel == 2048 and sp.dev_numel == 2048 and sp.device_part.numel() == 2048
    assert torch.equal(sp.full(), full)
    staging = torch.empty(2048)
    got = sp.load(staging, streams)
    assert torch.equal(got, full[2048:])
    got.mul_(2)
    sp.store(got, streams)
    assert torch.equal(sp.full()[2048:], full[2048:] * 2)
    whole = torch.empty(4096)
    sp.load_into(whole, streams)
    assert torch.equal(whole[:2048], full[:2048]) and torch.equal(whole[2048:], full[2048:] * 2)
    sp.store_from(whole + 1, streams)
    assert torch.equal(sp.full(), whole + 1)
    # ratios that round to nothing keep everything on the device
    tiny = SplitTensor(torch.zeros(100), 0.5)
    assert tiny.host_numel == 0 and tiny.load(staging, streams) is None


def test_activation_swapper_restores_values_and_respects_the_ratio():
    streams = SwapStreams("cpu")
    sw = ActivationSwapper(0.5, streams, min_numel=16)
    sw.set_scope("s")
    x = torch.randn(8, 64, requires_grad=True)
    w1 = torch.randn(64, 64, requires_grad=True)
    w2 = torch.randn(64, 64, requires_grad=True)
    with sw.hooks():
        y = torch.tanh(torch.tanh(x @ w1) @ w2).sum()
    assert 0 < sw.bytes_out <= 0.5 * sw._seen["s"] + 1
    sw.prefetch("s")
    y.backward()
    gx, g1, g2 = x.grad.clone(), w1.grad.clone(), w2.grad.clone()
    sw.release("s")
    assert sw.bytes_in == sw.bytes_out
    for t in (x, w1, w2):
        t.grad = None
    torch.tanh(torch.tanh(x @ w1) @ w2).sum().backward()
    assert torch.equal(gx, x.grad) and torch.equal(g1, w1.grad) and torch.equal(g2, w2.grad)


def test_engine_with_activation_offload_matches_adamw():
    from mist_b200.config import StageStrategy, load_config
    from mist_b200.models.provider import base_model_provider, get_inputs_provider
    from mist_b200.parallel.engine import TrainEngine
    from mist_b200.parallel import swap
    tiny = ["model.num_hidden_layers=3", "model.hidden_size=64", "model.intermediate_size=128",
            "model.num_attention_heads=4", "training.max_sequence_length=32", "model.vocab_size=256",
            "strategy.layer_partitions=[3]", "training.params_dtype=float32"]
    cfg, _ = load_config("config", ["experiment=gpt2-1.3b"] + tiny, check_world_size=False)
    torch.manual_seed(0)
    model = base_model_provider(cfg.model, device="cpu", dtype=torch.float32)
    ref = copy.deepcopy(model)
    old = swap.ACTIVATION_SWAP_MIN_NUMEL
    swap.ACTIVATION_SWAP_MIN_NUMEL = 64          # the tiny model's activations are below the default threshold
    try:
        eng = TrainEngine(model, strategy=StageStrategy(2, 1, 1, False, False, False, 0, 0, 0, 0.5),
                          grad_accum_steps=2, hp=dict(lr=1e-3))
        eng.act_swapper.min_numel = 64
        opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
        prov = get_inputs_provider(cfg.model.name)
        for it in range(2):
            batches = [prov(2, 32, 256, "cpu", seed=5 * it + k) for k in range(2)]
            loss = eng.train_step(batches)
            opt.zero_grad()
            tot = 0.0
            for b in batches:
                l = ref(**b) / 2
                l.backward()
                tot += l.item()
            opt.step()
            assert abs(loss.item() - tot) < 1e-4
        assert eng.act_swapper.bytes_out > 0 and eng.act_swapper.bytes_in == eng.act_swapper.bytes_out
        diff = max((a - b).abs().max().item() for a, b in zip(model.parameters(), ref.parameters()))
        assert diff < 1e-4
    finally:
        swap.ACTIVATION_SWAP_MIN_NUMEL = old
