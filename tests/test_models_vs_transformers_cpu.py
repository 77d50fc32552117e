"""The GPT and Llama definitions against the `transformers` implementations of the same
architectures: same weights in, same logits and loss out (fp32, CPU)."""
import pytest
import torch

from mist_b200.config import load_config
from mist_b200.models.provider import base_model_provider

transformers = pytest.importorskip("transformers")

TINY = ["model.num_hidden_layers=2", "model.hidden_size=64", "model.intermediate_size=128",
        "model.num_attention_heads=4", "training.max_sequence_length=32", "model.vocab_size=256",
        "strategy.layer_partitions=[2]", "training.params_dtype=float32"]


def _ours(exp, extra=()):
    cfg, _ = load_config("config", [f"experiment={exp}"] + TINY + list(extra), check_world_size=False)
    torch.manual_seed(0)
    return cfg, base_model_provider(cfg.model, device="cpu", dtype=torch.float32).eval()


def test_gpt_matches_hf_gpt2():
    cfg, ours = _ours("gpt2-1.3b")
    hf_cfg = transformers.GPT2Config(vocab_size=256, n_positions=32, n_embd=64, n_layer=2, n_head=4, n_inner=128,
                                     activation_function="gelu_new", resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0,
                                     layer_norm_epsilon=cfg.model.normalization_eps, tie_word_embeddings=False)
    hf = transformers.GPT2LMHeadModel(hf_cfg).eval()
    sd = dict(ours.named_parameters())
    with torch.no_grad():
        hf.transformer.wte.weight.copy_(sd["language_model.embedding.word_embeddings.weight"])
        hf.transformer.wpe.weight.copy_(sd["language_model.embedding.position_embeddings.weight"])
        for i, blk in enumerate(hf.transformer.h):
            pre = f"language_model.encoder.layers.{i}."
            blk.ln_1.weight.copy_(sd[pre + "norm1.weight"]); blk.ln_1.bias.copy_(sd[pre + "norm1.bias"])
            blk.ln_2.weight.copy_(sd[pre + "norm2.weight"]); blk.ln_2.bias.copy_(sd[pre + "norm2.bias"])
            blk.attn.c_attn.weight.copy_(sd[pre + "attn.Wqkv.weight"].t()); blk.attn.c_attn.bias.zero_()
            blk.attn.c_proj.weight.copy_(sd[pre + "attn.out_proj.weight"].t()); blk.attn.c_proj.bias.zero_()
            blk.mlp.c_fc.weight.copy_(sd[pre + "mlp.fc1.weight"].t()); blk.mlp.c_fc.bias.zero_()
            blk.mlp.c_proj.weight.copy_(sd[pre + "mlp.fc2.weight"].t()); blk.mlp.c_proj.bias.zero_()
        hf.transformer.ln_f.weight.copy_(sd["language_model.encoder.final_norm.weight"])
        hf.transformer.ln_f.bias.copy_(sd["language_model.encoder.final_norm.bias"])
        hf.lm_head.weight.copy_(sd["lm_head.proj.weight"])
    ids = torch.randint(0, 256, (2, 32))
    labels = torch.randint(0, 256, (2, 32))
    with torch.no_grad():
        logits = ours(ids).reshape(2, 32, -1)
        ref = hf(ids).logits
        loss = ours(ids, labels=labels)
        ref_loss = torch.nn.functional.cross_entropy(ref.reshape(-1, 256), labels.reshape(-1))
    assert (logits - ref).abs().max().item() < 2e-4
    assert abs(loss.item() - ref_loss.item()) < 1e-4          # our labels are already aligned with the logits


def test_llama_matches_hf_llama():
    # the packaged Llama configurations rotate a quarter of each head (as the reference's do); the
    # published architecture rotates the whole head
    cfg, ours = _ours("llama-350m", ["model.rotary_emb_fraction=1.0"])
    hf_cfg = transformers.LlamaConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=32,
                                      rms_norm_eps=cfg.model.normalization_eps, rope_theta=10000.0,
                                      attention_bias=False, mlp_bias=False, tie_word_embeddings=False,
                                      hidden_act="silu", attention_dropout=0.0)
    hf = transformers.LlamaForCausalLM(hf_cfg).eval()
    sd = dict(ours.named_parameters())
    with torch.no_grad():
        hf.model.embed_tokens.weight.copy_(sd["language_model.embedding.word_embeddings.weight"])
        for i, blk in enumerate(hf.model.layers):
            pre = f"language_model.encoder.layers.{i}."
            q, k, v = sd[pre + "attn.Wqkv.weight"].chunk(3, dim=0)
            blk.self_attn.q_proj.weight.copy_(q); blk.self_attn.k_proj.weight.copy_(k); blk.self_attn.v_proj.weight.copy_(v)
            blk.self_attn.o_proj.weight.copy_(sd[pre + "attn.out_proj.weight"])
            gate, up = sd[pre + "mlp.fc1.weight"].chunk(2, dim=0)
            blk.mlp.gate_proj.weight.copy_(gate); blk.mlp.up_proj.weight.copy_(up)
            blk.mlp.down_proj.weight.copy_(sd[pre + "mlp.fc2.weight"])
            blk.input_layernorm.weight.copy_(sd[pre + "norm1.weight"])
            blk.post_attention_layernorm.weight.copy_(sd[pre + "norm2.weight"])
        hf.model.norm.weight.copy_(sd["language_model.encoder.final_norm.weight"])
        hf.lm_head.weight.copy_(sd["lm_head.proj.weight"])
    ids = torch.randint(0, 256, (2, 32))
    with torch.no_grad():
        logits = ours(ids).reshape(2, 32, -1)
        ref = hf(ids).logits
    assert (logits - ref).abs().max().item() < 2e-4
