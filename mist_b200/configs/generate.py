"""Writes the packaged YAML tree (``python -m mist_b200.configs.generate``).

The tree has the layout the entry points expect: ``config.yaml`` at the root with a
``defaults`` list, hardware/training/strategy/tuning presets under ``experiment/`` and
model shapes under ``model/<family>/<size>.yaml`` (reference layout:
benchmark/mist/configs/config.yaml:3-33, experiment/template-*.yaml, model/*/common.yaml).
Generating the files from tables keeps the model zoo and the B200 presets in one place.
"""
from __future__ import annotations

from pathlib import Path

import yaml

HERE = Path(__file__).resolve().parent

# (hidden, intermediate, layers, heads)
GPT_SIZES = {
    "1.3b": (2048, 8192, 24, 16), "2.7b": (2560, 10240, 32, 32), "7b": (4096, 16384, 32, 32),
    "8b": (4096, 16384, 40, 32), "13b": (5120, 20480, 40, 40), "20b": (6144, 24576, 44, 64),
    "22b": (6144, 24576, 48, 64), "40b": (8192, 32768, 48, 64),
}
LLAMA_SIZES = {
    "350m": (1024, 2816, 24, 16), "1.3b": (2048, 5632, 24, 16), "2.7b": (2560, 6912, 32, 32),
    "7b": (4096, 11008, 32, 32), "13b": (5120, 13824, 40, 40), "20b": (6144, 16384, 44, 64),
    "22b": (6144, 16384, 48, 64), "40b": (8192, 22016, 48, 64), "70b": (8192, 28672, 80, 64),
}
T5_SIZES = {
    "1.7b": (2048, 8192, 16, 16), "3b": (2048, 8192, 24, 32), "7b": (3072, 8192, 32, 32),
    "11b": (4096, 16384, 24, 64), "20b": (6144, 24576, 20, 64), "40b": (8192, 32768, 24, 64),
}
# depth sweeps used by the scaling experiments: (hidden, heads) -> layer counts
GPT_SWEEPS = {
    (2048, 32): (24, 48, 72, 96, 120, 144, 168), (4096, 32): (48, 64, 80, 96, 112, 128),
    (5120, 40): (32, 48, 64, 80), (6144, 64): (48, 64, 80, 96),
}


def _common(family: str) -> dict:
    m = dict(
        fp32_residual_connection=False, fp16_lm_cross_entropy=True, vocab_size=50304, num_tokentypes=0,
        position_embedding_type="absolute", padding_idx=None, rotary_emb_fraction=0.0,
        rotary_emb_base=10000.0, rotary_emb_scale_base=None, rotary_emb_interleaved=False,
        tie_word_embeddings=False, add_encoder=True, add_decoder=False, encoder_attn_mask_type="causal",
        add_pooler=False, num_experts=None, parallel_block=False, parallel_block_tied_norm=False,
        prenorm=True, normalization="layernorm", activation_function="gelu_fast", mlp_type="mlp",
        qkv_proj_bias=False, out_proj_bias=False, mlp_fc1_bias=False, mlp_fc2_bias=False,
        hidden_dropout=0.0, attention_dropout=0.0, scale_attn_weights=True, use_flash_attn=True,
        bias_dropout_fusion=False,
    )
    if family == "llama":
        m.update(position_embedding_type="rotary", rotary_emb_fraction=0.25, normalization="rmsnorm",
                 activation_function="swiglu", mlp_type="gated_mlp")
    elif family == "falcon":
        m.update(position_embedding_type="rotary", rotary_emb_fraction=0.25, parallel_block=True)
    elif family == "bert":
        m.update(num_tokentypes=2, encoder_attn_mask_type="padding", add_pooler=True)
    elif family == "t5":
        m.update(num_tokentypes=2, add_decoder=True, encoder_attn_mask_type="padding",
                 decoder_attn_mask_type="causal")
    return {"model": m}


def _write(path: Path, body: dict, defaults=None, header="# @package _global_\n\n"):
    path.parent.mkdir(parents=True, exist_ok=True)
    out = {}
    if defaults is not None:
        out["defaults"] = defaults
    out.update(body)
    with open(path, "w") as f:
        f.write(header)
        yaml.safe_dump(out, f, sort_keys=False, default_flow_style=None, width=120)


# ------------------------------------------------------------------------ hardware presets
# GPU<->GPU table: 4x4 cells over (inter-node group size, intra-node group size) in
# {1,2,4,8}, each (bandwidth GB/s, bias s).  Single NVSwitch box: only the intra row is real.
def _g2g(intra):
    cells = [[(4.5, 0.0)] * 4 for _ in range(4)]
    cells[0] = [(4.5, 0.0)] + list(intra)
    return [x for row in cells for c in row for x in c]


HARDWARE = {
    # All-gather cells and the 28 interference factors: fitted by mist_b200.tools.comm_model from the full grids of
    # mist_b200.tools.profile_interference on this pool (groups of 2 and 4 on a 4-GPU box, 8 on an 8-GPU box; 810
    # records).  The factors are fitted with an upper bound of 2.5: without it four of them run to 5-17 (they
    # multiply channel times that are tiny in the records that determine them) while the mean error on the
    # records stays the same (9.1 % unbounded, 9.3 % bounded; the earlier hand-set factors: 18.9 %).
    # Host copies depend on how many ranks copy at the same instant: 52 / 54 GB/s to / from the device with 2
    # ranks, 54 / 27 with 4, 23 / 12 with all 8; training runs sit in between (the ranks' copies only partly
    # coincide), and the schema has one pair per direction: 35 / 21 GB/s.
    "b200": dict(gpu_type="NVIDIA B200", num_nodes=1, num_gpus_per_node=8,
                 gpu_gpu_comm_params=_g2g([(445.5, 8.3e-5), (588.2, 9.5e-5), (550.4, 8.4e-5)]),
                 cpu_gpu_comm_params=[35.0, 1.0e-4], gpu_cpu_comm_params=[21.0, 1.5e-4],
                 interference_model_params=[2.38, 1.64, 1.78, 2.5, 1.01, 1.02, 1.12, 1.88, 1.53, 1.38,
                                            1.22, 1.47, 2.5, 2.5, 1.92, 2.5, 1.04, 1.29, 1.0, 1.0,
                                            1.04, 1.16, 1.0, 1.02, 1.97, 1.16, 1.76, 2.01],
                 nvlink=True, memory_capacity=178.0),
    "l4": dict(gpu_type=None, num_nodes=1, num_gpus_per_node=8,
               gpu_gpu_comm_params=[4.5, 0.0, 2.964, 0.0001, 4.1635, 0.0004, 4.6832, 0.0003, 0.4895, 0.0045,
                                    0.9791, 0.0076, 1.7183, 0.0, 3.3215, 0.0013, 0.4609, 0.0102, 0.9195,
                                    0.0008, 1.6759, 0.0045, 2.9659, 0.003, 4.5, 0.0, 4.5, 0.0, 4.5, 0.0, 4.5, 0.0],
               cpu_gpu_comm_params=[5.7546, 0.0004], gpu_cpu_comm_params=[6.1252, 0.0004],
               interference_model_params=[18.9356, 1.2639, 50.0, 1.6046, 2.0865, 1.0009, 2.393, 2.4146, 1.0869,
                                          2.6637, 1.9381, 3.2653, 1.0, 1.234, 50.0, 1.6883, 1.1676, 1.0, 1.0152,
                                          1.0005, 1.0179, 1.0022, 1.0, 2.1383, 1.078, 2.438, 2.4327, 1.0974],
               nvlink=False, memory_capacity=22.488),
    "a100-sxm4-40gb": dict(gpu_type="NVIDIA A100-SXM4-40GB", num_nodes=1, num_gpus_per_node=8,
                           gpu_gpu_comm_params=_g2g([(139.0, 1e-4), (192.6, 1e-4), (210.3, 1e-4)]),
                           cpu_gpu_comm_params=[5.36, 0.0004], gpu_cpu_comm_params=[5.85, 0.0004],
                           interference_model_params=[1.2] * 28, nvlink=True, memory_capacity=39.5),
}

TOP_LEVEL = dict(overlap=True, use_memory_buffer=True, nccl_timeout=120, profile=False, tiny_bench=True,
                 memory_debug=False, enable_advanced_opt_in_first_block=True, disable_tp_tuning=True)


def _training(gbs, seq=2048, vocab=50304, dtype="bfloat16"):
    return dict(max_sequence_length=seq, vocab_size=vocab, global_batch_size=gbs, params_dtype=dtype,
                exec_dtype=dtype, optimizer_dtype="float32", autocast_enabled=False, optimizer_name="adamw")


def _tuning(**kw):
    t = dict(enabled=True, zero_2_and_3_enabled=True, activation_checkpointing_tuning_enabled=True,
             state_offloading_enabled=True, activation_offloading_enabled=True,
             tuning_granularity="uniform-device-pp-mip", sample_size=30, pre_post_strategy="dp",
             pre_post_strategy_array=None)
    t.update(kw)
    return t


def _strategy(stages, G, pre_post=None):
    """stages: list of (layers, (nodes, gpus), ckpt, vector10)"""
    pre_post = list(pre_post if pre_post is not None else stages[0][3])
    pre_post = pre_post[:6] + [0, 0, 0, 0]
    return dict(enabled=True, layer_partitions=[s[0] for s in stages],
                device_assignment=[list(s[1]) for s in stages], gradient_checkpointing=[s[2] for s in stages],
                gradient_accumulation_steps=G, stage_strategies=[list(s[3]) for s in stages],
                pre_post_strategy="preset", pre_post_strategy_array=pre_post)


def _experiment(path, model_ref, hardware, training, strategy, tuning=None, extra=None):
    body = dict(training=training, hardware=dict(hardware), strategy=strategy, tuning=tuning or _tuning())
    body.update(TOP_LEVEL)
    if extra:
        body.update(extra)
    _write(path, body, defaults=[f"/model/{model_ref}", "_self_"] if model_ref else None)


def generate(root: Path = HERE):
    # ---- root config
    _write(root / "config.yaml", dict(work_dir="${hydra:runtime.cwd}", data_dir="${work_dir}/data/",
                                      print_config=True, ignore_warnings=True, seed=None, name=None,
                                      output_path="${hydra:runtime.cwd}/best_config.yaml"),
           defaults=["_self_", {"experiment": "b200-gpt3-2.7b-dp8-zero2"}, {"model": None}])
    # ---- models
    for fam, sizes in (("gpt2", GPT_SIZES), ("falcon", {k: v for k, v in GPT_SIZES.items() if k != "8b"}),
                       ("bert", {k: v for k, v in GPT_SIZES.items() if k not in ("8b", "22b")}),
                       ("llama", LLAMA_SIZES), ("t5", T5_SIZES)):
        _write(root / "model" / fam / "common.yaml", _common("gpt2" if fam == "gpt2" else fam))
        for size, (h, f, L, a) in sizes.items():
            _write(root / "model" / fam / f"{size}.yaml",
                   dict(model=dict(name=f"{fam}-{size}", hidden_size=h, intermediate_size=f,
                                   num_hidden_layers=L, num_attention_heads=a, num_heads_kv=None)),
                   defaults=[f"/model/{fam}/common", "_self_"])
    for (h, a), depths in GPT_SWEEPS.items():
        for L in depths:
            _write(root / "model" / "gpt2" / f"_H{h}_L{L}.yaml",
                   dict(model=dict(name=f"gpt2-h{h}-l{L}", hidden_size=h, intermediate_size=4 * h,
                                   num_hidden_layers=L, num_attention_heads=a, num_heads_kv=None)),
                   defaults=["/model/gpt2/common", "_self_"])
    # ---- hardware templates (no model attached)
    for hw_name, hw in HARDWARE.items():
        n = hw["num_gpus_per_node"]
        _experiment(root / "experiment" / f"template-{hw_name}.yaml", None, hw,
                    _training(64, dtype="bfloat16" if hw_name == "b200" else "float16"),
                    _strategy([("${model.num_hidden_layers}", (1, n), 0, [64 // n // 2, n, 1, 0, 0, 1, 0, 0, 0, 0])], 2),
                    _tuning(zero_2_and_3_enabled=False, activation_checkpointing_tuning_enabled=False))
    b200 = HARDWARE["b200"]
    # ---- the four execution workloads on 8 x B200
    _experiment(root / "experiment" / "b200-gpt3-2.7b-dp8-zero2.yaml", "gpt2/2.7b", b200, _training(64),
                _strategy([(32, (1, 8), 0, [8, 8, 1, 0, 1, 1, 0, 0, 0, 0])], 1))
    _experiment(root / "experiment" / "b200-llama-7b-tp2sp-dp4.yaml", "llama/7b", b200,
                _training(32, seq=4096, vocab=32000),
                _strategy([(32, (1, 8), 8, [4, 4, 2, 0, 1, 1, 0, 0, 0, 0])], 2),
                extra=dict(sequence_parallel=True, model=dict(vocab_size=32000, rotary_emb_fraction=1.0)))
    _experiment(root / "experiment" / "b200-gpt3-13b-pp2-tp4.yaml", "gpt2/13b", b200, _training(128),
                _strategy([(20, (1, 4), 20, [2, 1, 4, 0, 0, 0, 0, 0, 1.0, 0]),
                           (20, (1, 4), 20, [2, 1, 4, 0, 0, 0, 0, 0, 1.0, 0])], 64),
                # sequence-sharded activations between the tensor-parallel linears: the all-reduce of plain tensor
                # parallelism becomes all-gather + reduce-scatter, which the fused GEMM + collective kernels run
                extra=dict(sequence_parallel=True))
    _experiment(root / "experiment" / "b200-gpt3-22b-zero3.yaml", "gpt2/22b", b200, _training(64),
                _strategy([(48, (1, 8), 0, [8, 8, 1, 1, 1, 1, 0, 0, 0, 0.5])], 1),
                extra=dict(model=dict(num_attention_heads=48)))
    # ---- smaller single-box experiments per model size (dp over all GPUs, ZeRO-1)
    for fam, sizes, gbs in (("gpt2", ("1.3b", "2.7b", "7b", "13b", "20b", "22b", "40b"), 64),
                            ("llama", ("350m", "1.3b", "2.7b", "7b", "13b"), 64)):
        for size in sizes:
            _experiment(root / "experiment" / f"{fam}-{size}.yaml", f"{fam}/{size}", b200, _training(gbs),
                        _strategy([("${model.num_hidden_layers}", (1, 8), 0, [4, 8, 1, 0, 0, 1, 0, 0, 0, 0])], 2))
    # ---- the two-GPU kick-the-tires case on the L4 calibration (CPU analyze / tune golden)
    l4 = dict(HARDWARE["l4"], num_gpus_per_node=2)
    small = dict(training=_training(32, dtype="float16"), hardware=l4,
                 strategy=_strategy([(24, (1, 2), 24, [8, 2, 1, 0, 0, 1, 0.0, 0.0, 0.0, 0.0])], 2),
                 tuning=_tuning())
    small.update(TOP_LEVEL)
    m = _common("gpt2")["model"]
    m.update(use_flash_attn=False, name="gpt2-1.3b", hidden_size=2048, intermediate_size=8192,
             num_hidden_layers=24, num_attention_heads=16, num_heads_kv=None)
    small["model"] = m
    _write(root / "test-small-base.yaml", small, header="")
    tuned = dict(small)
    tuned["strategy"] = _strategy([(12, (1, 1), 5, [2, 1, 1, 0, 0, 1, 0, 0, 0, 0]),
                                   (12, (1, 1), 0, [2, 1, 1, 0, 0, 1, 0, 0, 0, 0])], 16)
    _write(root / "test-small.yaml", tuned, header="")
    # same model on two B200s
    b2 = dict(small)
    b2["hardware"] = dict(b200, num_gpus_per_node=2)
    b2["training"] = _training(32)
    _write(root / "test-small-b200.yaml", b2, header="")


if __name__ == "__main__":
    generate()
    print("wrote", HERE)
