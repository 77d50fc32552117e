"""Timing, materialisation and device helpers (CPU)."""
import time

import numpy as np
import torch
import torch.nn as nn

from mist_b200.config import ModelConfig
from mist_b200.models.provider import base_model_provider, get_inputs_provider
from mist_b200.utils import benchmark, device, materialize


def test_timers_and_summary():
    calls = []

    def work(n, scale=1):
        calls.append(n * scale)
        time.sleep(0.002)

    costs, (alloc, reserved) = benchmark.time_host(work, warmup=1, number=3, prepare=lambda: ((2,), {"scale": 3}))
    assert len(costs) == 3 and all(c >= 0.002 for c in costs) and calls == [6] * 4
    costs2, _ = benchmark.time_device(lambda: time.sleep(0.001), warmup=0, number=2)     # host fallback without a GPU
    assert len(costs2) == 2 and costs2.min() >= 0.001
    lines = []
    mean, median, std = benchmark.summarize(np.array([1e-3, 3e-3, 2e-3]), "step", lines.append)
    assert abs(mean - 2e-3) < 1e-12 and abs(median - 2e-3) < 1e-12 and std > 0
    assert lines[0].startswith("[step]") and "Median: 2.0000 ms" in lines[0]
    assert benchmark.format_time(2.5) == "2.5000 s" and benchmark.format_time(3e-7) == "300.0000 ns"
    assert benchmark.format_size(3 << 20) == "3.00 MB"


def test_model_built_empty_then_materialised_trains():
    cfg = ModelConfig(name="gpt2-t", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      max_position_embeddings=32, vocab_size=256, params_dtype="float32", add_encoder=True,
                      add_decoder=False, use_flash_attn=True, encoder_attn_mask_type="causal")
    with materialize.empty_init():
        m = base_model_provider(cfg, device=None, dtype=torch.float32)
    assert all(p.is_meta for p in m.parameters())
    torch.manual_seed(0)
    materialize.materialize_module(m, "cpu")
    assert not any(p.is_meta for p in m.parameters())
    norm_w = m.language_model.encoder.layers[0].norm1.weight
    assert torch.all(norm_w == 1)                                  # the layer's own initialiser ran
    w = m.language_model.encoder.layers[0].attn.Wqkv.weight
    assert 0.005 < w.std().item() < 0.05
    loss = m(**get_inputs_provider("gpt")(2, 32, 256, "cpu", seed=1))
    loss.backward()
    assert torch.isfinite(loss) and abs(loss.item() - 5.545) < 1.0


def test_materialise_keeps_shared_parameters_shared_and_handles_foreign_modules():
    with materialize.empty_init():
        a = nn.Linear(8, 8)
        b = nn.Linear(8, 8)
        b.weight = a.weight
        net = nn.Sequential(a, nn.LayerNorm(8), b, nn.Embedding(5, 8))
    materialize.materialize_module(net, "cpu")
    assert net[0].weight is net[2].weight and not net[0].weight.is_meta
    assert torch.all(net[1].weight == 1) and torch.all(net[1].bias == 0)
    t = materialize.materialize_tensor(torch.empty(3, 4, device="meta", dtype=torch.bfloat16, requires_grad=True), "cpu")
    assert t.shape == (3, 4) and t.dtype == torch.bfloat16 and t.requires_grad and t.abs().max() < 0.1
    idx = materialize.materialize_tensor(torch.empty(5, device="meta", dtype=torch.long), "cpu")
    assert idx.dtype == torch.long and idx.max() <= 1
    assert materialize.materialize_tensor("not a tensor") == "not a tensor"


def test_device_name_follows_the_override(monkeypatch):
    monkeypatch.setenv("FAKE_DEVICE_NAME", "NVIDIA_B200")
    assert device.device_name() == "NVIDIA_B200"
    monkeypatch.delenv("FAKE_DEVICE_NAME")
    assert device.device_name() == ("cpu" if not torch.cuda.is_available() else device.device_name())
    device.join_streams(None, None)      # no GPU: nothing to do
    assert device.current_device().type in ("cpu", "cuda")


def test_cpu_binding_plan_with_a_fake_nvml():
    """Ranks are bound to the cores NVML names for their GPU: shared per NUMA node (`node`), or split into
    disjoint slices among the ranks of a node (`exclusive`); never outside the cores the process may use."""
    from mist_b200.utils import affinity

    class FakeNvml:
        # GPUs 0-3 hang off cores 0-31, GPUs 4-7 off cores 32-63
        def nvmlDeviceGetHandleByIndex(self, i):
            return i

        def nvmlDeviceGetCpuAffinity(self, handle, words):
            return [0xFFFFFFFF if handle < 4 else 0xFFFFFFFF << 32] + [0] * (words - 1)

    nv = FakeNvml()
    assert affinity.gpu_cpu_set(1, nv) == set(range(32)) and affinity.gpu_cpu_set(6, nv) == set(range(32, 64))
    sets = [affinity.gpu_cpu_set(r, nv) for r in range(8)]
    assert affinity.plan(sets, 5, "node") == set(range(32, 64))
    slices = [affinity.plan(sets, r, "exclusive") for r in range(8)]
    assert all(len(s) == 8 for s in slices)
    assert set().union(*slices[:4]) == set(range(32)) and set().union(*slices[4:]) == set(range(32, 64))
    assert sum(len(s) for s in slices) == 64                       # disjoint
    assert affinity.plan(sets, 2, "off") == set()
    # a container that may only use cores 0-3: stay inside, share when there are fewer cores than ranks
    assert affinity.plan(sets, 1, "node", allowed={0, 1, 2, 3}) == {0, 1, 2, 3}
    assert affinity.plan(sets, 1, "exclusive", allowed={0, 1, 2}) == {0, 1, 2}
    assert affinity.plan(sets, 5, "node", allowed={0, 1, 2, 3}) == set()      # nothing near that GPU: unbound
    # no NVML at all: unbound
    assert affinity.bind_to_gpu(0, 8, "node", nvml=object(), apply=False) == set()
    assert affinity.bind_to_gpu(3, 8, "exclusive", nvml=nv, apply=False) <= set(range(32))


def test_clock_sampler_with_a_stand_in_for_nvidia_smi(tmp_path):
    """The sampler runs the query tool in a helper process and summarises its CSV lines; a missing tool gives
    an empty summary instead of an error."""
    import os
    import stat
    import time
    from mist_b200.utils.clocks import ClockSampler, summarise
    fake = tmp_path / "fake-smi"
    fake.write_text("#!/bin/bash\nwhile true; do echo '0, 1530, 1965, 987.5, 0x4, Not Active, Not Active, Not Active, Active'; "
                    "echo '0, 1560, 1965, 990.1, 0x4, Not Active, Not Active, Not Active, Active'; sleep 0.05; done\n")
    os.chmod(fake, os.stat(fake).st_mode | stat.S_IEXEC)
    s = ClockSampler(0, executable=str(fake)).start()
    time.sleep(0.5)
    out = s.stop()
    assert out["samples"] >= 2 and out["sm_mhz"] in (1530.0, 1545.0, 1560.0) and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"] and out["power_w_max"] == 990.1
    assert ClockSampler(0, executable=str(tmp_path / "missing")).start().stop()["sm_mhz"] is None
    bad = summarise(["garbage", "0, [N/A], 1965, 1, x, Active, Not Active, Not Active, Not Active"])
    assert bad["samples"] == 0 and bad["reasons"] == []
