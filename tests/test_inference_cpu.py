"""Generation with a key/value cache must produce the tokens a cache-free model would:
after every new token, re-running the whole sequence through the ordinary (training) forward
pass gives the same next-token choice."""
import pytest
import torch

from mist_b200.config import load_config
from mist_b200.inference import generate, kv_cache
from mist_b200.models.provider import base_model_provider

TINY = ["model.num_hidden_layers=2", "model.hidden_size=64", "model.intermediate_size=128",
        "model.num_attention_heads=4", "training.max_sequence_length=64", "model.vocab_size=128",
        "strategy.layer_partitions=[2]", "training.params_dtype=float32"]


@pytest.mark.parametrize("exp,extra", [("gpt2-1.3b", []), ("llama-350m", []),
                                       ("llama-350m", ["+model.num_heads_kv=2"])])     # grouped-query + rotary
def test_cached_generation_matches_full_recompute(exp, extra):
    cfg, _ = load_config("config", [f"experiment={exp}"] + TINY + extra, check_world_size=False)
    if extra:
        assert cfg.model.num_heads_kv == 2
    torch.manual_seed(0)
    model = base_model_provider(cfg.model, device="cpu", dtype=torch.float32).eval()
    prompt = torch.randint(0, 128, (2, 7))
    out = generate(model, prompt, max_new_tokens=6)
    assert out.shape == (2, 13) and torch.equal(out[:, :7], prompt)
    # cache-free oracle
    seq = prompt
    with torch.no_grad():
        for _ in range(6):
            logits = model(seq).reshape(2, seq.shape[1], -1)
            seq = torch.cat([seq, logits[:, -1].argmax(-1, keepdim=True)], dim=1)
    assert torch.equal(out, seq)
    # the cache hooks are removed afterwards: a training-style forward still works
    assert all(getattr(m, "inference_params", None) is None for m in model.modules())


def test_single_token_logits_match_full_forward():
    cfg, _ = load_config("config", ["experiment=llama-350m"] + TINY, check_world_size=False)
    torch.manual_seed(1)
    model = base_model_provider(cfg.model, device="cpu", dtype=torch.float32).eval()
    ids = torch.randint(0, 128, (3, 9))
    with torch.no_grad():
        full = model(ids).reshape(3, 9, -1)
        with kv_cache(model, 3, 16) as ip:
            model(ids[:, :8], position_ids=torch.arange(8).expand(3, -1))
            ip.seqlen_offset = 8
            step = model(ids[:, 8:9], position_ids=torch.full((3, 1), 8)).reshape(3, 1, -1)
    assert (step[:, 0] - full[:, 8]).abs().max().item() < 1e-4


def test_eos_stops_sequences():
    cfg, _ = load_config("config", ["experiment=gpt2-1.3b"] + TINY, check_world_size=False)
    torch.manual_seed(2)
    model = base_model_provider(cfg.model, device="cpu", dtype=torch.float32).eval()
    prompt = torch.randint(0, 128, (2, 4))
    first = generate(model, prompt, max_new_tokens=1)[:, -1]
    out = generate(model, prompt, max_new_tokens=5, eos_token_id=int(first[0]))
    assert (out[0, 4:] == int(first[0])).all()


def test_nucleus_sampling_only_draws_from_the_smallest_set_that_reaches_p():
    cfg, _ = load_config("config", ["experiment=gpt2-1.3b"] + TINY, check_world_size=False)
    torch.manual_seed(0)
    model = base_model_provider(cfg.model, device="cpu", dtype=torch.float32).eval()
    prompt = torch.randint(0, 128, (3, 5))
    with torch.no_grad():
        probs = torch.softmax(model(prompt).reshape(3, 5, -1)[:, -1].float(), -1)
    srt, idx = probs.sort(-1, descending=True)
    allowed = []
    for b in range(3):
        n = int((srt[b].cumsum(0) < 0.6).sum()) + 1          # smallest prefix whose mass reaches 0.6
        allowed.append(set(idx[b, :n].tolist()))
    gen = torch.Generator().manual_seed(3)
    seen = [set() for _ in range(3)]
    for _ in range(40):
        out = generate(model, prompt, max_new_tokens=1, temperature=1.0, top_p=0.6, generator=gen)
        for b in range(3):
            seen[b].add(int(out[b, -1]))
    for b in range(3):
        assert seen[b] <= allowed[b], (b, seen[b] - allowed[b])
    # a very small p is greedy decoding
    greedy = generate(model, prompt, max_new_tokens=3)
    assert torch.equal(generate(model, prompt, max_new_tokens=3, temperature=1.0, top_p=1e-6, generator=gen), greedy)
