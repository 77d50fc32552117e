"""Public training API: configuration name -> a session that runs training iterations.

    session = build_training("config", ["experiment=b200-gpt3-2.7b-dp8-zero2"])
    loss = session.step(input_ids_on_host, labels_on_host)

The session hides the strategy: data/tensor/pipeline layout, ZeRO level, activation
checkpointing, offloading and the overlap schedule all come from the ``strategy`` block
of the configuration (the file the tuner writes).  The exec entry point
(``benchmark/mist_b200/exec/benchmark_one_case.py``) and ``bench.py`` are thin wrappers
around it.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .config import MistConfig, StageStrategy, load_config
from .models.provider import base_model_provider, family_of
from .parallel.engine import TrainEngine
from .parallel.state import ParallelState


def _stage_layer_range(cfg: MistConfig, stage: int):
    parts = cfg.strategy.layer_partitions
    if cfg.model.add_decoder and len(parts) > 1 and stage == len(parts) - 1:
        return 0, parts[stage]          # the last stage of an encoder-decoder pipeline: the whole decoder
    start = sum(parts[:stage])
    return start, start + parts[stage]


class TrainingSession:
    def __init__(self, cfg: MistConfig, comm_backend: Optional[str] = None, seed: int = 1234,
                 device: Optional[torch.device] = None, hp: Optional[Dict] = None):
        self.cfg = cfg
        world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        assert world == cfg.hardware.num_devices or world == 1, \
            f"configuration describes {cfg.hardware.num_devices} devices, job has {world}"
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = device
        if device.type == "cuda":
            # optional: restrict this rank to the cores next to its GPU (MIST_B200_BIND_CPU=node|exclusive)
            from .utils.affinity import bind_to_gpu
            self.cpu_cores = bind_to_gpu(device.index or 0, int(os.environ.get("LOCAL_WORLD_SIZE", "1")))
        self.ps = ParallelState.from_config(cfg) if world > 1 else ParallelState.from_config(cfg, rank=0, create_groups=False)
        st = cfg.strategy
        stage = self.ps.stage
        self.strategy = st.stage(stage)
        self.G = st.gradient_accumulation_steps
        self.micro_batch = self.strategy.micro_batch_size
        self.seq_len = cfg.training.max_sequence_length
        self.sequence_parallel = bool(cfg.get("sequence_parallel", False)) and self.ps.tp_size > 1
        from .ops import functional as _F
        # Collective back ends.  "auto" (the default) selects the hand-written NVLink kernels wherever
        # they apply: CUDA, the tcgen05 GEMM back end, and every rank of the group on this node (peer
        # memory); groups that span nodes, CPU runs and the library GEMM back end use NCCL / gloo.
        on_gpu = device.type == "cuda" and world > 1 and _F.Settings.gemm_backend == "tcgen05"

        def _one_node(group):
            from .parallel.symm import group_on_one_node
            return group_on_one_node(group)

        want = comm_backend or str(cfg.get("comm_backend", "auto"))
        if want == "auto":
            want = "fused" if (on_gpu and self.ps.dp_size > 1 and _one_node(self.ps.dp_group)) else "nccl"
        self.comm_backend = want
        tpb = str(cfg.get("tp_backend", "auto"))
        if tpb == "auto":
            tpb = "fused" if (on_gpu and self.ps.tp_size > 1 and self.sequence_parallel
                              and _one_node(self.ps.tp_group)) else "nccl"
        _F.Settings.tp_backend = self.tp_backend = tpb
        z3 = str(cfg.get("zero3_gather", "auto"))
        if z3 == "auto":
            z3 = "fused" if (on_gpu and self.ps.dp_size > 1) else "nccl"
        self.zero3_gather = z3
        dtype = cfg.training.params_dtype
        # same seed on every data-parallel replica; tensor-parallel ranks draw different slices
        torch.manual_seed(seed + 1000 * self.ps.tp_rank + 17 * stage)
        lr = _stage_layer_range(cfg, stage)
        multi_stage = st.num_stages > 1
        self.model = base_model_provider(
            cfg.model, process_groups=self.ps.tp_group, pre_post_process_group=self.ps.tp_group,
            pre_process=self.ps.is_first_stage, post_process=self.ps.is_last_stage,
            layer_range=lr if multi_stage else None, sequence_parallel=self.sequence_parallel,
            device=device, dtype=dtype)
        # Parameters that every tensor-parallel rank holds in full (norms, position tables, BERT's head
        # transform, pooler ...) were drawn from a rank-dependent stream above: make them equal to the
        # first rank's, as the gradient handling of replicated parameters assumes.
        if self.ps.tp_size > 1 and world > 1:
            src = dist.get_global_rank(self.ps.tp_group, 0)
            for p in self.model.parameters():
                if not getattr(p, "_tp_sharded", False):
                    dist.broadcast(p.data, src=src, group=self.ps.tp_group)
        # dropout masks of replicated activations must agree over the tensor-parallel group; where the
        # tokens are sharded (sequence parallelism) every rank adds its own offset to the drawn seeds
        # (the seeds of dropout calls come from torch's CPU generator: from here on it is the same on every
        # rank of a tensor-parallel group and differs between data-parallel replicas)
        torch.manual_seed(seed + 17 * stage + 7919 * self.ps.dp_rank)
        _F.Settings.dropout_seed_offset = 104729 * self.ps.tp_rank if self.sequence_parallel else 0
        # a table tied across the first and the last stage: pair the ranks and copy it over once
        tied_group = None
        ties = bool(getattr(cfg.model, "tie_word_embeddings", False)) or family_of(cfg.model.name) in ("bert", "t5")
        if ties and multi_stage and world > 1:
            tied_group = self.ps.create_embedding_group(getattr(cfg, "nccl_timeout", 120))
            if hasattr(self.model, "tied_parameters"):
                tied = self.model.tied_parameters()
            else:
                one = self.model.tied_parameter() if hasattr(self.model, "tied_parameter") else None
                tied = [] if one is None else [one]
            for t in tied:
                dist.broadcast(t.data, src=self.ps.embedding_src, group=tied_group)
        ppv = st.pre_post_vector(stage)
        pre_post = StageStrategy.from_vector(ppv) if ppv is not None else None
        self.engine = TrainEngine(self.model, self.ps, self.strategy, self.G, st.gradient_checkpointing[stage],
                                  hp=hp, comm_backend=self.comm_backend, overlap=bool(cfg.get("overlap", True)),
                                  zero3_gather=self.zero3_gather,
                                  use_grad_ring=bool(cfg.get("use_memory_buffer", True)),
                                  pre_post_strategy=pre_post, tied_group=tied_group)
        # what the engine settled on (it falls back to the library collectives where a fused path does
        # not apply: offloaded weights or gradients, units with tied tables, groups across nodes)
        self.comm_backend = "fused" if self.engine.fused is not None else "nccl"
        self.zero3_gather = "fused" if self.engine.param_gather is not None else "nccl"
        self.pipeline = None
        if multi_stage:
            from .parallel.pipeline import PipelineSchedule
            self.pipeline = PipelineSchedule(self)
        self._h2d_stream = torch.cuda.Stream() if device.type == "cuda" else None
        # host-side failure detection between steps (see utils/watchdog.py); off unless asked for
        self.heartbeat = None
        self.heartbeat_max_age_s = float(cfg.get("heartbeat_max_age_s", 120.0))
        if bool(cfg.get("heartbeat", False)) and world > 1:
            self.enable_heartbeat()

    def enable_heartbeat(self, store=None, max_age_s: Optional[float] = None):
        """Registers this rank in the job's key-value store; from then on every :meth:`step` beats
        and, before it launches anything, raises if a peer stopped beating or asked to abort."""
        from .utils.watchdog import Heartbeat
        if store is None:
            store = dist.PrefixStore("mist_b200_hb", dist.distributed_c10d._get_default_store())
        if max_age_s is not None:
            self.heartbeat_max_age_s = float(max_age_s)
        self.heartbeat = Heartbeat(store, dist.get_rank(), dist.get_world_size())
        return self.heartbeat

    def _beat(self):
        if self.heartbeat is not None:
            self.heartbeat.beat()
            self.heartbeat.check(self.heartbeat_max_age_s)

    # ------------------------------------------------------------------------------ steps
    def _split_micro(self, ids, labels):
        if self.G == 1:
            return [{"input_ids": ids, "labels": labels}]
        return [{"input_ids": a, "labels": b} for a, b in zip(ids.chunk(self.G), labels.chunk(self.G))]

    def step_on_device(self, input_ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """One iteration on tensors already on the device; returns the loss tensor (device)."""
        self._beat()
        batches = self._split_micro(input_ids, labels)
        if self.pipeline is not None:
            return self.pipeline.train_step(batches)
        return self.engine.train_step(batches)

    def step_on_device_batch(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        """One iteration on a dictionary of model inputs (what the family's inputs provider
        returns: token ids, token types, decoder ids, labels ...), each with this rank's
        ``micro_batch * G`` samples along dimension 0; used for the encoder-only and
        encoder-decoder families whose forward takes more than ids and labels."""
        self._beat()
        if self.G == 1:
            batches = [dict(batch)]
        else:
            parts = {k: v.chunk(self.G) for k, v in batch.items()}
            batches = [{k: parts[k][i] for k in batch} for i in range(self.G)]
        if self.pipeline is not None:
            return self.pipeline.train_step(batches)
        return self.engine.train_step(batches)

    def step(self, input_ids: torch.Tensor, labels: torch.Tensor) -> float:
        """One iteration from host tensors (pinned memory recommended): copies the inputs to
        the device, trains, and returns the loss as a Python float."""
        if self.device.type == "cuda":
            ids = input_ids.to(self.device, non_blocking=True)
            lab = labels.to(self.device, non_blocking=True)
        else:
            ids, lab = input_ids, labels
        loss = self.step_on_device(ids, lab)
        value = float(loss.item())
        self.check_device_status()
        return value

    def check_device_status(self, collective: bool = True):
        """Raises if a kernel's bounded wait ran out since the last check (the kernel then stopped
        issuing work, so this step's results are not to be trusted).  With ``collective`` the status
        is combined over all ranks first, so that every replica stops at the same step.  Call it
        where the device is already synchronised: :meth:`step` does after reading the loss,
        :meth:`finish` does once the outstanding optimizer steps are waited for; callers of
        :meth:`step_on_device` (no host synchronisation per step) get the check in :meth:`finish`
        or can call it themselves every few steps."""
        if self.device.type != "cuda":
            return
        from .ops import native
        code = native.read_and_clear_status()
        world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        if collective and world > 1:
            t = torch.tensor([code], dtype=torch.int32, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            worst = int(t.item())
            if worst and not code:
                raise RuntimeError(f"another rank reported device status {worst} (a bounded wait ran out); "
                                   "this replica stops at the same step")
        if code:
            raise RuntimeError(native.status_message(code))

    def finish(self):
        self.engine.finish()
        if self.device.type == "cuda":
            torch.cuda.synchronize()
            self.check_device_status()

    # -------------------------------------------------------------------------- accounting
    def flops_per_step(self) -> float:
        """Model FLOPs (forward + backward) of this rank's share of one iteration."""
        c = self.cfg.model
        b, s = self.micro_batch * self.G, self.seq_len
        tokens = b * s
        per_layer = 2 * tokens * (c.params_per_block()) + 2 * 2 * b * s * s * c.hidden_size * 0.5
        total = c.num_hidden_layers * per_layer + 2 * tokens * c.hidden_size * c.vocab_size
        return 3.0 * total / max(self.ps.tp_size * self.ps.num_stages, 1)


def build_training(config_name: str = "config", overrides: Optional[List[str]] = None,
                   comm_backend: Optional[str] = None, seed: int = 1234, config_dirs=(), hp=None) -> TrainingSession:
    cfg, _ = load_config(config_name, overrides, config_dirs=config_dirs)
    return TrainingSession(cfg, comm_backend=comm_backend, seed=seed, hp=hp)
