"""Model zoo on CPU: every family trains a step; checkpoint layout round-trips."""
import os

import pytest
import torch

from mist_b200.config import ModelConfig
from mist_b200.models.provider import base_model_provider, family_of, get_inputs_provider

BASE = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
            max_position_embeddings=32, vocab_size=256, params_dtype="float32", add_encoder=True,
            add_decoder=False, use_flash_attn=True)


def _cfg(family):
    if family == "gpt":
        return ModelConfig(name="gpt2-t", encoder_attn_mask_type="causal", **BASE)
    if family == "llama":
        return ModelConfig(name="llama-t", encoder_attn_mask_type="causal", mlp_type="gated_mlp",
                           normalization="rmsnorm", position_embedding_type="rotary", rotary_emb_fraction=1.0, **BASE)
    if family == "falcon":
        return ModelConfig(name="falcon-t", encoder_attn_mask_type="causal", parallel_block=True,
                           position_embedding_type="rotary", rotary_emb_fraction=1.0, **BASE)
    if family == "bert":
        return ModelConfig(name="bert-t", encoder_attn_mask_type="padding", add_pooler=True, num_tokentypes=2, **BASE)
    b = dict(BASE, add_decoder=True)
    return ModelConfig(name="t5-t", encoder_attn_mask_type="padding", decoder_attn_mask_type="causal", **b)


def test_every_family_trains_one_step():
    for fam in ("gpt", "llama", "falcon", "bert", "t5"):
        cfg = _cfg(fam)
        assert family_of(cfg.name) == fam
        torch.manual_seed(0)
        m = base_model_provider(cfg, device="cpu", dtype=torch.float32)
        batch = get_inputs_provider(cfg.name)(2, 32, 256, "cpu", seed=1)
        loss = m(**batch)
        loss.backward()
        assert torch.isfinite(loss) and abs(loss.item() - 5.545) < 1.6   # ~ln(256) at init
        assert all(p.grad is not None for p in m.parameters() if p.requires_grad)


def test_flash_and_materialised_attention_agree():
    torch.manual_seed(0)
    a = base_model_provider(_cfg("llama"), device="cpu", dtype=torch.float32)
    cfg2 = _cfg("llama")
    cfg2.use_flash_attn = False
    b = base_model_provider(cfg2, device="cpu", dtype=torch.float32)
    b.load_state_dict(a.state_dict())
    batch = get_inputs_provider("llama")(2, 32, 256, "cpu", seed=3)
    assert abs(a(**batch).item() - b(**batch).item()) < 1e-4


def test_nested_checkpoint_layout_roundtrip():
    torch.manual_seed(0)
    m = base_model_provider(_cfg("gpt"), device="cpu", dtype=torch.float32)
    sd = m.state_dict_for_save_checkpoint()
    assert set(sd) == {"language_model", "lm_head"}
    assert {"embedding", "encoder"} <= set(sd["language_model"])
    assert {"word_embeddings", "position_embeddings"} <= set(sd["language_model"]["embedding"])
    torch.manual_seed(1)
    m2 = base_model_provider(_cfg("gpt"), device="cpu", dtype=torch.float32)
    m2.load_state_dict_from_checkpoint(sd)
    batch = get_inputs_provider("gpt")(2, 32, 256, "cpu", seed=3)
    assert abs(m(**batch).item() - m2(**batch).item()) < 1e-6
    # legacy key names are accepted
    legacy = {k.replace("norm1", "input_layernorm").replace("norm2", "post_attention_layernorm")
               .replace("final_norm", "final_layernorm"): v for k, v in sd["language_model"]["encoder"].items()}
    m2.language_model.encoder.load_state_dict(legacy)


def test_gradient_checkpointing_same_grads():
    torch.manual_seed(0)
    m = base_model_provider(_cfg("gpt"), device="cpu", dtype=torch.float32)
    batch = get_inputs_provider("gpt")(2, 32, 256, "cpu", seed=5)
    m(**batch).backward()
    g0 = [p.grad.clone() for p in m.parameters()]
    m.zero_grad()
    m.language_model.encoder.gradient_checkpointing = 2
    m(**batch).backward()
    assert all(torch.allclose(a, p.grad, atol=1e-6) for a, p in zip(g0, m.parameters()))


@pytest.mark.parametrize("fam", ["bert/1.3b", "t5/1.7b", "falcon/1.3b", "gpt2/1.3b"])
def test_exec_entry_point_runs_every_family_on_cpu(fam, tmp_path):
    """The exec driver end to end (session, family input provider, timing, summary) on one CPU rank."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, os.path.join(root, "benchmark/mist_b200/exec/benchmark_one_case.py"), "experiment=gpt2-1.3b",
           f"model={fam}", "model.num_hidden_layers=2", "model.hidden_size=64", "model.intermediate_size=128",
           "model.num_attention_heads=4", "training.max_sequence_length=32", "model.vocab_size=256",
           "strategy.layer_partitions=[2]", "training.params_dtype=float32", "hardware.num_gpus_per_node=1",
           "training.global_batch_size=4", "strategy.device_assignment=[[1,1]]", "strategy.gradient_checkpointing=[1]",
           "strategy.gradient_accumulation_steps=2", "strategy.stage_strategies=[[2,1,1,0,0,0,0,0,0,0]]",
           "strategy.pre_post_strategy_array=[2,1,1,0,0,0,0,0,0,0]", f"output_dir={tmp_path}"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    assert "Throughput:" in r.stdout
    s = json.load(open(tmp_path / "summary.json"))
    assert float(s["exec_total_cost"]) > 0


# ------------------------------------------------------------------------------ padding masks
def _masks(b, s):
    """One right-padded sample, one sample with holes, one without padding."""
    m = torch.ones(b, s, dtype=torch.bool)
    m[0, s - 5:] = False
    m[1, 3] = m[1, 10] = m[1, s - 1] = False
    return m


@pytest.mark.parametrize("flash", [True, False])
@pytest.mark.parametrize("causal", [False, True])
def test_attention_with_padding_mask_equals_attention_over_the_real_tokens(flash, causal):
    from mist_b200.modules.layers import PaddingMask, ParallelMHA
    torch.manual_seed(0)
    b, s, h = 3, 16, 32
    mha = ParallelMHA(h, 4, causal=causal, use_flash_attn=flash, device="cpu", dtype=torch.float32)
    x = torch.randn(b, s, h, requires_grad=True)
    mask = _masks(b, s)
    out = mha(x, attention_mask=PaddingMask.prepare(mask))
    g = torch.randn_like(out) * mask[..., None]
    out.backward(g)
    bias = mha.out_proj.bias.detach()
    for i in range(b):
        xi = x.detach()[i:i + 1, mask[i]].clone().requires_grad_(True)
        oi = mha(xi)
        assert torch.allclose(out[i, mask[i]], oi[0], atol=1e-5)
        assert torch.allclose(out[i, ~mask[i]], bias.expand(int((~mask[i]).sum()), h), atol=1e-6)   # zero context
        oi.backward(g[i:i + 1, mask[i]])
        assert torch.allclose(x.grad[i, mask[i]], xi.grad[0], atol=1e-5)
        assert x.grad[i, ~mask[i]].abs().max() == 0 if (~mask[i]).any() else True
    assert PaddingMask.prepare(torch.ones(b, s)) is None      # no padding: the plain path is taken


def test_bert_with_padding_mask_matches_the_unpadded_sample():
    torch.manual_seed(0)
    cfg = _cfg("bert")
    m = base_model_provider(cfg, device="cpu", dtype=torch.float32)
    m.language_model.encoder.gradient_checkpointing = 1
    b, s = 2, 32
    batch = get_inputs_provider("bert")(b, s, 256, "cpu", seed=3)
    mask = torch.ones(b, s, dtype=torch.bool)
    mask[0, 20:] = False
    logits, _ = m(batch["input_ids"], attention_mask=mask, tokentype_ids=batch["tokentype_ids"])
    alone, _ = m(batch["input_ids"][:1, :20], tokentype_ids=batch["tokentype_ids"][:1, :20])
    assert torch.allclose(logits[0, :20], alone[0], atol=1e-4)
    full, _ = m(batch["input_ids"][1:], tokentype_ids=batch["tokentype_ids"][1:])
    assert torch.allclose(logits[1], full[0], atol=1e-4)
    # the loss is differentiable through the masked path with recomputation
    loss = m(batch["input_ids"], attention_mask=mask, tokentype_ids=batch["tokentype_ids"], lm_labels=batch["lm_labels"])
    loss.backward()
    enc_params = list(m.language_model.encoder.parameters())
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in enc_params)


def test_t5_cross_attention_ignores_padded_encoder_tokens():
    torch.manual_seed(0)
    cfg = _cfg("t5")
    m = base_model_provider(cfg, device="cpu", dtype=torch.float32)
    batch = get_inputs_provider("t5")(2, 32, 256, "cpu", seed=4)
    enc, dec = batch["encoder_input_ids"], batch["decoder_input_ids"]
    mask = torch.ones_like(enc, dtype=torch.bool)
    mask[0, 24:] = False
    logits = m(enc, dec, encoder_attn_mask=mask)
    alone = m(enc[:1, :24], dec[:1])
    assert torch.allclose(logits[0], alone[0], atol=1e-4)
    other = m(enc[1:], dec[1:])
    assert torch.allclose(logits[1], other[0], atol=1e-4)
    # changing a padded encoder token changes nothing
    enc2 = enc.clone()
    enc2[0, 30] = (enc2[0, 30] + 7) % 256
    assert torch.allclose(m(enc2, dec, encoder_attn_mask=mask), logits, atol=1e-6)


def test_residual_from_the_normalised_stream_when_prenorm_is_off():
    """prenorm = False: x1 = LN1(h); a = x1 + attn(x1); x2 = LN2(a); out = x2 + mlp(x2)."""
    import torch.nn.functional as TF
    from mist_b200.models.transformer import ParallelTransformerLayer
    torch.manual_seed(0)
    cfg = ModelConfig(name="gpt2-t", encoder_attn_mask_type="causal", prenorm=False, **BASE)
    layer = ParallelTransformerLayer(cfg, 0, device="cpu", dtype=torch.float32)
    for n in (layer.norm1, layer.norm2):           # make the norms non-trivial
        with torch.no_grad():
            n.weight.uniform_(0.5, 1.5)
            n.bias.uniform_(-0.2, 0.2)
    h = torch.randn(2, 16, 64)
    hidden, residual = layer(h, None)
    x1 = TF.layer_norm(h, (64,), layer.norm1.weight, layer.norm1.bias, cfg.normalization_eps)
    a = x1 + layer.attn(x1)
    x2 = TF.layer_norm(a, (64,), layer.norm2.weight, layer.norm2.bias, cfg.normalization_eps)
    want = x2 + layer.mlp(x2)
    assert torch.allclose(hidden + residual, want, atol=1e-5)
    # and the whole model still trains
    m = base_model_provider(cfg, device="cpu", dtype=torch.float32)
    loss = m(**get_inputs_provider("gpt")(2, 32, 256, "cpu", seed=2))
    loss.backward()
    assert torch.isfinite(loss)


def test_activation_and_softmax_scale_flags_are_honoured():
    import torch.nn.functional as TF
    from mist_b200.modules.layers import ParallelGatedMlp, ParallelMLP
    torch.manual_seed(0)
    x = torch.randn(3, 5, 16)
    for name, ref in (("relu", TF.relu), ("gelu", TF.gelu), ("sqrelu", lambda t: TF.relu(t) ** 2),
                      ("gelu_fast", lambda t: TF.gelu(t, approximate="tanh"))):
        mlp = ParallelMLP(16, 32, activation=name, device="cpu", dtype=torch.float32)
        want = TF.linear(ref(TF.linear(x, mlp.fc1.weight, mlp.fc1.bias)), mlp.fc2.weight, mlp.fc2.bias)
        assert torch.allclose(mlp(x), want, atol=1e-5), name
    for name, ref in (("swiglu", TF.silu), ("geglu", TF.gelu), ("glu", torch.sigmoid)):
        g = ParallelGatedMlp(16, 32, activation=name, device="cpu", dtype=torch.float32)
        gate, up = TF.linear(x, g.fc1.weight).chunk(2, -1)
        assert torch.allclose(g(x), TF.linear(ref(gate) * up, g.fc2.weight), atol=1e-5), name
    cfg = ModelConfig(name="gpt2-t", encoder_attn_mask_type="causal", scale_attn_weights=True,
                      scale_attn_by_inverse_layer_idx=True, **BASE)
    m = base_model_provider(cfg, device="cpu", dtype=torch.float32)
    scales = [l.attn.softmax_scale for l in m.language_model.encoder.layers]
    assert scales == pytest.approx([16 ** -0.5, 16 ** -0.5 / 2])
    cfg2 = ModelConfig(name="gpt2-t", encoder_attn_mask_type="causal", scale_attn_weights=False, **BASE)
    m2 = base_model_provider(cfg2, device="cpu", dtype=torch.float32)
    assert m2.language_model.encoder.layers[0].attn.softmax_scale == 1.0


@pytest.mark.parametrize("interleaved,scale_base", [(True, None), (False, 512.0), (True, 64.0)])
@pytest.mark.parametrize("heads_kv", [4, 2])
def test_interleaved_and_position_scaled_rotary(interleaved, scale_base, heads_kv):
    from mist_b200.modules.layers import ParallelMHA
    from mist_b200.ops import functional as F
    torch.manual_seed(0)
    b, s, hdim, nh, rot = 2, 12, 64, 4, 8
    d = hdim // nh
    mha = ParallelMHA(hdim, nh, heads_kv, causal=True, rotary_emb_dim=rot, rotary_emb_interleaved=interleaved,
                      rotary_emb_scale_base=scale_base, device="cpu", dtype=torch.float32)
    x = torch.randn(b, s, hdim)
    out = mha(x)
    # direct formula
    qkv = torch.nn.functional.linear(x, mha.Wqkv.weight, mha.Wqkv.bias)
    if heads_kv == nh:
        qkv = qkv.view(b, s, 3, nh, d)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    else:
        q = qkv[..., : nh * d].reshape(b, s, nh, d)
        k = qkv[..., nh * d: (nh + heads_kv) * d].reshape(b, s, heads_kv, d)
        v = qkv[..., (nh + heads_kv) * d:].reshape(b, s, heads_kv, d)
    inv = 1.0 / (10000.0 ** (torch.arange(0, rot, 2).float() / rot))
    ang = torch.outer(torch.arange(s).float(), inv)                      # [s, rot/2]
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    sc = torch.ones(s, rot // 2)
    if scale_base is not None:
        base = (torch.arange(0, rot, 2).float() + 0.4 * rot) / (1.4 * rot)
        sc = base[None, :] ** ((torch.arange(s).float() - s // 2) / scale_base)[:, None]
    sc = sc[None, :, None, :]

    def rope(t, scale):
        t = t.clone()
        if interleaved:
            a, c = t[..., 0:rot:2], t[..., 1:rot:2]
            t[..., 0:rot:2], t[..., 1:rot:2] = (a * cos - c * sin) * scale, (a * sin + c * cos) * scale
        else:
            a, c = t[..., : rot // 2], t[..., rot // 2: rot]
            t[..., : rot // 2], t[..., rot // 2: rot] = (a * cos - c * sin) * scale, (a * sin + c * cos) * scale
        return t
    o, _ = F._ref_attention(rope(q, sc), rope(k, 1.0 / sc), v, mha.softmax_scale, True)
    want = torch.nn.functional.linear(o.reshape(b, s, hdim), mha.out_proj.weight, mha.out_proj.bias)
    assert torch.allclose(out, want, atol=1e-5)


def test_label_smoothing_spreads_the_mass_over_the_other_classes():
    """loss = (1 - s) * nll - s * mean_j log p_j with s = a K / (K - 1): the label keeps 1 - a and each of
    the other K - 1 classes gets a / (K - 1) (torch's own label_smoothing spreads a over all K classes)."""
    from mist_b200.modules.layers import vocab_parallel_cross_entropy
    torch.manual_seed(0)
    K, a = 50, 0.1
    logits = torch.randn(7, K, requires_grad=True)
    labels = torch.randint(0, K, (7,))
    labels[3] = -100
    ours = vocab_parallel_cross_entropy(logits, labels, label_smoothing=a)
    ref_in = logits.detach().clone().requires_grad_(True)
    target = torch.full((7, K), a / (K - 1))
    keep = labels != -100
    target[torch.arange(7)[keep], labels[keep]] = 1 - a
    want = -(target * torch.log_softmax(ref_in, -1)).sum(-1) * keep
    assert torch.allclose(ours, want, atol=1e-5)
    ours.sum().backward()
    want.sum().backward()
    assert torch.allclose(logits.grad, ref_in.grad, atol=1e-5)


def test_varlen_attention_equals_per_sequence_attention():
    from mist_b200.ops import functional as F
    torch.manual_seed(0)
    lens = [5, 1, 9, 3]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)))
    q = torch.randn(sum(lens), 4, 16, requires_grad=True)
    k = torch.randn(sum(lens), 2, 16, requires_grad=True)
    v = torch.randn(sum(lens), 2, 16, requires_grad=True)
    out = F.attention_varlen(q, k, v, cu, causal=True)
    out.square().sum().backward()
    grads = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    start = 0
    ref = []
    for n in lens:
        o, _ = F._ref_attention(q[None, start:start + n], k[None, start:start + n], v[None, start:start + n],
                                16 ** -0.5, True)
        ref.append(o[0])
        start += n
    ref = torch.cat(ref)
    assert torch.allclose(out, ref, atol=1e-5)
    ref.square().sum().backward()
    for g, t in zip(grads, (q, k, v)):
        assert torch.allclose(g, t.grad, atol=1e-4)
