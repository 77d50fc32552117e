"""Typed view of an experiment configuration.

A resolved YAML tree (see :mod:`mist_b200.utils.yamlconf`) is split into five objects:
model, training, hardware, tuning and strategy.  The schema, key names, units and
validation rules follow the reference so that its experiment files load unchanged
(reference: mist/config.py:91-270 ModelConfig, :273-315 HardwareConfig, :318-355
TrainingConfig, :358-422 TuningConfig, :425-584 StrategyConfig, :587-641 MistConfig).

Deliberate differences from the reference:
* ``nccl_timeout`` from the file is honoured (the reference overwrites it with 60 s).
* error messages describe the 10-element strategy vector correctly.
"""
from __future__ import annotations

import enum
import os
from dataclasses import dataclass, fields
from typing import Any, List, Optional, Sequence, Tuple

import torch

from .utils import yamlconf

MB = 1 << 20
GB = 1 << 30

#: fraction of the device memory the tuner is allowed to plan with
MEMORY_SAFETY_MARGIN = 0.88

_DTYPES = {
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
}


def to_torch_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _DTYPES[str(name).lower().replace("torch.", "")]
    except KeyError as e:
        raise ValueError(f"unknown dtype '{name}'") from e


class MLPType(enum.Enum):
    mlp = "mlp"
    gated_mlp = "gated_mlp"


class PositionEmbeddingType(enum.Enum):
    absolute = "absolute"
    rotary = "rotary"
    relative = "relative"
    none = "none"


class AttnMaskType(enum.Enum):
    padding = "padding"
    causal = "causal"


class ZeroLevel(enum.IntEnum):
    """Sharding level implied by the (wre, gre, ore) flags of a strategy vector."""
    NONE = 0
    OPT = 1          # ZeRO-1: optimizer states sharded
    OPT_GRAD = 2     # ZeRO-2: + gradients
    FULL = 3         # ZeRO-3: + weights

    @staticmethod
    def from_flags(wre: bool, gre: bool, ore: bool) -> "ZeroLevel":
        if wre:
            return ZeroLevel.FULL
        if gre:
            return ZeroLevel.OPT_GRAD
        if ore:
            return ZeroLevel.OPT
        return ZeroLevel.NONE


@dataclass
class ModelConfig:
    name: str
    hidden_size: int = None
    intermediate_size: Optional[int] = None
    num_hidden_layers: int = None
    num_attention_heads: int = None
    num_heads_kv: Optional[int] = None
    params_dtype: Any = "float16"
    fp32_residual_connection: bool = False
    fp16_lm_cross_entropy: bool = True
    max_position_embeddings: int = None
    vocab_size: int = None
    num_tokentypes: int = 0
    position_embedding_type: Any = "absolute"
    padding_idx: Optional[int] = None
    rotary_emb_base: float = 10000.0
    rotary_emb_scale_base: Any = None
    rotary_emb_fraction: float = 0.0
    rotary_emb_interleaved: bool = False
    tie_word_embeddings: bool = False
    add_encoder: bool = None
    add_decoder: bool = None
    encoder_attn_mask_type: Any = "padding"
    decoder_attn_mask_type: Any = "padding"
    add_pooler: bool = False
    num_experts: Optional[int] = None
    parallel_block: bool = False
    parallel_block_tied_norm: bool = False
    prenorm: bool = True
    normalization: str = "LayerNorm"
    activation_function: str = "gelu_new"
    mlp_type: Any = "mlp"
    multiple_of: int = 256
    qkv_proj_bias: bool = False
    out_proj_bias: bool = False
    mlp_fc1_bias: bool = False
    mlp_fc2_bias: bool = False
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0
    normalization_eps: float = 1e-6
    scale_attn_weights: bool = False
    scale_attn_by_inverse_layer_idx: bool = False
    use_flash_attn: bool = False
    bias_dropout_fusion: bool = True
    tensor_parallel: Optional[bool] = None
    sequence_parallel: Optional[bool] = None

    def __post_init__(self):
        assert self.name is not None, "model.name is required"
        self.name = str(self.name).lower()
        assert self.hidden_size is not None, "model.hidden_size is required"
        self.params_dtype = to_torch_dtype(self.params_dtype)
        if not isinstance(self.mlp_type, MLPType):
            assert self.mlp_type in MLPType.__members__, \
                f"mlp_type must be one of {list(MLPType.__members__)}, got {self.mlp_type}"
            self.mlp_type = MLPType[self.mlp_type]
        if self.intermediate_size is None:
            if self.mlp_type is MLPType.mlp:
                self.intermediate_size = 4 * self.hidden_size
            else:
                f = int(self.hidden_size * 8 / 3)
                self.intermediate_size = (f + self.multiple_of - 1) // self.multiple_of * self.multiple_of
        assert self.num_hidden_layers is not None and self.num_attention_heads is not None
        self.num_heads_kv = self.num_heads_kv or self.num_attention_heads
        assert self.max_position_embeddings is not None and self.vocab_size is not None
        if not isinstance(self.position_embedding_type, PositionEmbeddingType):
            assert self.position_embedding_type in PositionEmbeddingType.__members__, \
                f"unknown position_embedding_type {self.position_embedding_type}"
            self.position_embedding_type = PositionEmbeddingType[self.position_embedding_type]
        if self.position_embedding_type is PositionEmbeddingType.rotary:
            assert self.rotary_emb_fraction is not None
        if isinstance(self.rotary_emb_scale_base, str) and self.rotary_emb_scale_base.lower() == "none":
            self.rotary_emb_scale_base = None
        assert self.add_encoder is not None and self.add_decoder is not None
        for attr, on in (("encoder_attn_mask_type", self.add_encoder), ("decoder_attn_mask_type", self.add_decoder)):
            val = getattr(self, attr)
            if on and not isinstance(val, AttnMaskType):
                assert val in AttnMaskType.__members__, f"unknown {attr} {val}"
                setattr(self, attr, AttnMaskType[val])
        assert self.normalization.lower() in ("layernorm", "rmsnorm")
        if self.sequence_parallel:
            assert self.tensor_parallel, "sequence_parallel needs tensor_parallel"

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def gated(self) -> bool:
        return self.mlp_type is MLPType.gated_mlp

    def params_per_block(self) -> int:
        """Weights of one transformer block (biases and norms included)."""
        h, f = self.hidden_size, self.intermediate_size
        kv = self.num_heads_kv * self.head_dim
        n = h * (h + 2 * kv) + h * h + (3 if self.gated else 2) * h * f
        n += (h + 2 * kv) * self.qkv_proj_bias + h * self.out_proj_bias
        n += (2 * f if self.gated else f) * self.mlp_fc1_bias + h * self.mlp_fc2_bias
        norms = 1 if (self.parallel_block and self.parallel_block_tied_norm) else 2
        n += norms * h * (1 if self.normalization.lower() == "rmsnorm" else 2)
        return n


@dataclass
class HardwareConfig:
    gpu_type: Optional[str] = None
    num_nodes: int = 1
    num_gpus_per_node: int = 1
    gpu_gpu_comm_params: Sequence[float] = ()
    cpu_gpu_comm_params: Sequence[float] = ()
    gpu_cpu_comm_params: Sequence[float] = ()
    interference_model_params: Sequence[float] = ()
    nvlink: Optional[bool] = None
    memory_capacity: float = 0.0      # GB as written in the file
    check_world_size: bool = True

    def __post_init__(self):
        self.gpu_gpu_comm_params = tuple(float(x) for x in self.gpu_gpu_comm_params)
        self.cpu_gpu_comm_params = tuple(float(x) for x in self.cpu_gpu_comm_params)
        self.gpu_cpu_comm_params = tuple(float(x) for x in self.gpu_cpu_comm_params)
        self.interference_model_params = tuple(float(x) for x in self.interference_model_params)
        self.raw_memory_capacity = float(self.memory_capacity)
        #: usable capacity in GB after the planner's safety margin
        self.memory_capacity = self.raw_memory_capacity * MEMORY_SAFETY_MARGIN
        if self.check_world_size and "WORLD_SIZE" in os.environ:
            ws = int(os.environ["WORLD_SIZE"])
            assert self.num_nodes * self.num_gpus_per_node == ws, \
                f"hardware describes {self.num_nodes * self.num_gpus_per_node} devices but WORLD_SIZE={ws}"
        assert len(self.gpu_gpu_comm_params) in (0, 32), "gpu_gpu_comm_params: 4x4 table of (GB/s, s)"
        assert len(self.cpu_gpu_comm_params) in (0, 2) and len(self.gpu_cpu_comm_params) in (0, 2)
        assert len(self.interference_model_params) in (0, 28), "interference_model_params: 28 factors"

    @property
    def num_devices(self) -> int:
        return self.num_nodes * self.num_gpus_per_node


@dataclass
class TrainingConfig:
    global_batch_size: int
    max_sequence_length: int
    params_dtype: Any = "float16"
    exec_dtype: Any = "float16"
    optimizer_dtype: Any = "float32"
    autocast_enabled: bool = False
    optimizer_name: str = "adamw"
    vocab_size: Optional[int] = None
    deallocate_pipeline_outputs: bool = False

    def __post_init__(self):
        self.params_dtype = to_torch_dtype(self.params_dtype)
        self.exec_dtype = to_torch_dtype(self.exec_dtype)
        self.optimizer_dtype = to_torch_dtype(self.optimizer_dtype)


TUNING_GRANULARITIES = (
    "no-pp", "uniform-pp", "uniform-device-pp", "uniform-device-pp-mip", "inter-stage",
    "uniform-pp-simple-heuristic-mem-opt",
)
PRE_POST_STRATEGIES = ("preset", "dp", "intra-node-tp-with-ore", "intra-node-tp-without-ore")

_VECTOR_HELP = ("a strategy vector has 10 elements: [0] micro batch size, [1] dp, [2] tp, "
                "[3] shard weights, [4] shard grads, [5] shard optimizer states, "
                "[6] weight offload ratio, [7] grad offload ratio, [8] optimizer offload ratio, "
                "[9] activation offload ratio")


def normalize_strategy_vector(vec) -> Tuple:
    assert len(vec) == 10, f"{_VECTOR_HELP}; got {list(vec)}"
    return (int(vec[0]), int(vec[1]), int(vec[2]), bool(vec[3]), bool(vec[4]), bool(vec[5]),
            float(vec[6]), float(vec[7]), float(vec[8]), float(vec[9]))


@dataclass
class StageStrategy:
    """Named view of one 10-element strategy vector."""
    micro_batch_size: int
    dp: int
    tp: int
    shard_weights: bool
    shard_grads: bool
    shard_opt: bool
    weight_offload: float
    grad_offload: float
    opt_offload: float
    act_offload: float

    @classmethod
    def from_vector(cls, vec) -> "StageStrategy":
        return cls(*normalize_strategy_vector(vec))

    def to_vector(self) -> Tuple:
        return (self.micro_batch_size, self.dp, self.tp, int(self.shard_weights), int(self.shard_grads),
                int(self.shard_opt), self.weight_offload, self.grad_offload, self.opt_offload,
                self.act_offload)

    @property
    def zero(self) -> ZeroLevel:
        return ZeroLevel.from_flags(self.shard_weights, self.shard_grads, self.shard_opt)


@dataclass
class TuningConfig:
    tuning_granularity: str
    sample_size: int
    pre_post_strategy: Optional[str] = None
    pre_post_strategy_array: Optional[List] = None
    zero_2_and_3_enabled: Optional[bool] = None
    activation_checkpointing_tuning_enabled: Optional[bool] = None
    state_offloading_enabled: Optional[bool] = None
    activation_offloading_enabled: Optional[bool] = None
    layers_offset: int = 2

    def __post_init__(self):
        self.sample_size = int(self.sample_size)
        assert self.tuning_granularity in TUNING_GRANULARITIES, \
            f"tuning_granularity must be one of {TUNING_GRANULARITIES}"
        assert self.pre_post_strategy in PRE_POST_STRATEGIES, \
            f"pre_post_strategy must be one of {PRE_POST_STRATEGIES}"
        self.pre_post_strategy_array = list(self.pre_post_strategy_array or [])
        if self.pre_post_strategy == "preset":
            self.pre_post_strategy_array = list(normalize_strategy_vector(self.pre_post_strategy_array))
        # YAML typos such as "ftrue" must not silently enable a feature
        for name in ("zero_2_and_3_enabled", "activation_checkpointing_tuning_enabled",
                     "state_offloading_enabled", "activation_offloading_enabled"):
            v = getattr(self, name)
            if isinstance(v, str):
                setattr(self, name, v.strip().lower() == "true")


@dataclass
class StrategyConfig:
    layer_partitions: List[int]
    device_assignment: List[Tuple[int, int]]
    gradient_checkpointing: List[int]
    gradient_accumulation_steps: int
    stage_strategies: List[Tuple]
    pre_post_strategy: Any = "heuristic"
    pre_post_strategy_array: Optional[List] = None

    def __post_init__(self):
        self.layer_partitions = [int(x) for x in self.layer_partitions]
        self.gradient_checkpointing = [int(x) for x in self.gradient_checkpointing]
        self.gradient_accumulation_steps = int(self.gradient_accumulation_steps)
        n = len(self.layer_partitions)
        assert n == len(self.device_assignment) == len(self.stage_strategies) == len(self.gradient_checkpointing), (
            "layer_partitions, device_assignment, stage_strategies and gradient_checkpointing need one "
            f"entry per stage; got {n}, {len(self.device_assignment)}, {len(self.stage_strategies)}, "
            f"{len(self.gradient_checkpointing)}")
        self.num_stages = n
        for d in self.device_assignment:
            assert len(d) == 2, f"device_assignment entries are (num_nodes, gpus_per_node); got {list(d)}"
        self.device_assignment = [(int(a), int(b)) for a, b in self.device_assignment]
        self.stage_strategies = [normalize_strategy_vector(s) for s in self.stage_strategies]
        if self.pre_post_strategy == "preset":
            assert self.pre_post_strategy_array is not None, "pre_post_strategy 'preset' needs pre_post_strategy_array"
            self.pre_post_strategy_array = list(normalize_strategy_vector(self.pre_post_strategy_array))

    def stage(self, idx: int) -> StageStrategy:
        return StageStrategy.from_vector(self.stage_strategies[idx])

    def pre_post_vector(self, idx: int) -> Optional[Tuple]:
        """Strategy vector of the embedding / head units of stage ``idx``, or ``None`` when they follow the
        stage's own vector (``heuristic``).  The named choices set the redundancy flags as the reference does
        (mist/analyzer/batched_module_analyzer.py:799-839): ``dp`` shards the optimizer states only,
        ``intra-node-tp-with-ore`` gradients and optimizer states, ``intra-node-tp-without-ore`` gradients only.
        The reference also gives the pre / post layers a mesh of their own under the named choices (all GPUs as
        data parallel, or a node as tensor parallel); here the embedding and the head always run on their
        stage's mesh, so micro batch, dp and tp are the stage's."""
        if self.pre_post_strategy == "preset":
            return tuple(self.pre_post_strategy_array)
        flags = {"dp": (0, 0, 1), "intra-node-tp-with-ore": (0, 1, 1), "intra-node-tp-without-ore": (0, 1, 0)}
        if self.pre_post_strategy in flags:
            v = self.stage_strategies[idx]
            return normalize_strategy_vector([v[0], v[1], v[2], *flags[self.pre_post_strategy], 0, 0, 0, 0])
        return None

    def verify_with_other_config(self, model: ModelConfig, training: TrainingConfig, hardware: HardwareConfig):
        gbs = training.global_batch_size
        G = self.gradient_accumulation_steps
        L = model.num_hidden_layers
        if model.add_decoder and self.num_stages > 1:
            # encoder-decoder models over pipeline stages: the encoder blocks are split over all stages but
            # the last, which holds the whole decoder
            assert self.layer_partitions[-1] == L and sum(self.layer_partitions[:-1]) == L, (
                f"encoder-decoder pipeline: layer_partitions {self.layer_partitions} must split the {L} encoder "
                f"blocks over the first stages and give the last stage the {L} decoder blocks")
        else:
            assert sum(self.layer_partitions) == L, \
                f"layer_partitions sum to {sum(self.layer_partitions)}, model has {L} layers"
        used = sum(n * m for n, m in self.device_assignment)
        assert used == hardware.num_devices, f"device_assignment uses {used} devices, hardware has {hardware.num_devices}"
        for ck, nl in zip(self.gradient_checkpointing, self.layer_partitions):
            assert ck <= nl, f"gradient_checkpointing {self.gradient_checkpointing} exceeds layer_partitions {self.layer_partitions}"
        for idx, s in enumerate(self.stage_strategies):
            assert s[0] * s[1] * G == gbs, (
                f"stage {idx}: micro batch {s[0]} x dp {s[1]} x grad-accum {G} = {s[0] * s[1] * G}, "
                f"global batch is {gbs}")
            n, m = self.device_assignment[idx]
            assert s[1] * s[2] == n * m, f"stage {idx}: dp {s[1]} x tp {s[2]} != {n * m} devices"
        if self.pre_post_strategy == "preset":
            a = self.pre_post_strategy_array
            assert a[0] * a[1] * G == gbs, f"pre/post strategy: {a[0]} x {a[1]} x {G} != global batch {gbs}"
            for d in (self.device_assignment[0], self.device_assignment[-1]):
                assert a[1] * a[2] == d[0] * d[1], f"pre/post strategy: dp {a[1]} x tp {a[2]} != {d[0] * d[1]} devices"


def _pick(cfg_section, cls, extra=None):
    names = {f.name for f in fields(cls)}
    kw = {k: v for k, v in dict(cfg_section).items() if k in names}
    unknown = [k for k in dict(cfg_section) if k not in names]
    if extra:
        kw.update(extra)
    return kw, unknown


class MistConfig:
    """Bundle of the five config objects; unknown attributes fall through to the raw tree
    (``overlap``, ``tiny_bench``, ``profile``, ``disable_tp_tuning``, ...)."""

    def __init__(self, model, training, hardware, tuning, strategy, original=None):
        self.model: ModelConfig = model
        self.training: TrainingConfig = training
        self.hardware: HardwareConfig = hardware
        self.tuning: Optional[TuningConfig] = tuning
        self.strategy: Optional[StrategyConfig] = strategy
        self._original = original
        self.nccl_timeout = int((original or {}).get("nccl_timeout", 120) or 120)

    def __getattr__(self, name):
        orig = self.__dict__.get("_original")
        if orig is not None and name in orig:
            return orig[name]
        raise AttributeError(name)

    def get(self, name, default=None):
        try:
            return getattr(self, name)
        except AttributeError:
            return default

    @property
    def raw(self):
        return self._original

    @classmethod
    def from_dict_config(cls, cfg, check_world_size: bool = True) -> "MistConfig":
        cfg = yamlconf._to_node(yamlconf.resolve(yamlconf._to_plain(cfg)))
        mkw, _ = _pick(cfg.model, ModelConfig, {
            "max_position_embeddings": cfg.training.max_sequence_length,
            "params_dtype": cfg.training.params_dtype,
        })
        model = ModelConfig(**mkw)
        hw = dict(cfg.hardware)
        # older experiment files give per-scope tables; expand them into the 4x4 layout
        if "gpu_gpu_comm_params" not in hw and "intra_node_gpu_gpu_comm_params" in hw:
            hw["gpu_gpu_comm_params"] = expand_comm_table(hw.get("intra_node_gpu_gpu_comm_params"),
                                                          hw.get("inter_node_gpu_gpu_comm_params"))
        hkw, _ = _pick(hw, HardwareConfig, {"check_world_size": check_world_size})
        hardware = HardwareConfig(**hkw)
        tkw, _ = _pick(cfg.training, TrainingConfig)
        training = TrainingConfig(**tkw)
        tuning = None
        if cfg.get("tuning") is not None and cfg.tuning.get("enabled", False):
            ukw, _ = _pick(cfg.tuning, TuningConfig)
            if "layers_offset" not in ukw and cfg.tuning.get("layers_offset") is not None:
                ukw["layers_offset"] = cfg.tuning.layers_offset
            tuning = TuningConfig(**ukw)
        strategy = None
        if cfg.get("strategy") is not None and cfg.strategy.get("enabled", False):
            skw, _ = _pick(cfg.strategy, StrategyConfig)
            strategy = StrategyConfig(**skw)
            strategy.verify_with_other_config(model, training, hardware)
        return cls(model, training, hardware, tuning, strategy, original=cfg)


def expand_comm_table(intra, inter=None) -> List[float]:
    """Builds the 32-number ``(inter, intra) -> (GB/s, bias)`` table from a 3-entry intra-node
    list (group sizes 2, 4, 8) and an optional inter-node list; unmeasured cells get the
    placeholder ``(4.5, 0.0)`` used by the shipped templates."""
    table = [[(4.5, 0.0) for _ in range(4)] for _ in range(4)]
    intra = list(intra or [])
    for i in range(min(3, len(intra) // 2)):
        table[0][i + 1] = (float(intra[2 * i]), float(intra[2 * i + 1]))
    inter = list(inter or [])
    for i in range(min(3, len(inter) // 2)):
        table[i + 1][0] = (float(inter[2 * i]), float(inter[2 * i + 1]))
    return [x for row in table for cell in row for x in cell]


CONFIG_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "configs")


def load_config(config_name: str = "config", overrides: Optional[List[str]] = None,
                config_dirs: Sequence[os.PathLike] = (), check_world_size: bool = True):
    """Composes a YAML by name (searching ``config_dirs`` then the packaged tree) and returns
    ``(MistConfig, raw_node)``."""
    dirs = list(config_dirs) + [CONFIG_DIR]
    node = yamlconf.compose(config_name, dirs, overrides)
    return MistConfig.from_dict_config(node, check_world_size=check_world_size), node
