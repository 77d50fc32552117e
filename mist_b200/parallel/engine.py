"""Overlap-centric training engine for one pipeline stage.

The model is cut into *units* (embedding, each transformer block, head).  Each unit owns
a :class:`~mist_b200.parallel.flat_unit.FlatUnit`.  Instead of module hooks scattered over
the model, two autograd markers per block tell the engine where the backward pass is:

* the marker placed after a block runs its backward *before* the block's backward
  (-> ZeRO-3: make the block's weights resident, prefetch the previous block);
* the marker placed before a block runs its backward *after* the block's backward
  (-> the block's gradient bucket is complete: reduce it, step the optimizer on the
  shard and refresh the weights, all on the communication stream while the compute
  stream continues with the previous block).

The weights of a unit are only touched again by the next iteration's forward, which
waits on the unit's ``param_ready`` event; so the optimizer step is overlapped with the
rest of the backward pass instead of being deferred into the next forward.

Parity: reference mist/re_swap_manager/manager.py:796-1338 (ModelReSwapManager),
:1339-1790 (the four hooks), streams :944-964; mist/re_swap_manager/optimizer.py:126-602.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..config import StageStrategy, ZeroLevel
from ..ops import functional as F
from ..utils.logging import record
from .flat_unit import FlatUnit
from .state import ParallelState

DEFAULT_HP = dict(lr=1e-5, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, adamw=True, loss_scale=1.0)


class _Marker(torch.autograd.Function):
    """Identity on (hidden, residual); calls ``fn()`` when the backward pass reaches it."""

    @staticmethod
    def forward(ctx, fn, hidden, residual):
        ctx.fn = fn
        ctx.has_res = residual is not None
        if residual is None:
            return hidden.view_as(hidden)
        return hidden.view_as(hidden), residual.view_as(residual)

    @staticmethod
    def backward(ctx, *grads):
        ctx.fn()
        if ctx.has_res:
            return None, grads[0], grads[1]
        return None, grads[0], None


def _mark(fn, hidden, residual):
    if not torch.is_grad_enabled() or not hidden.requires_grad:
        return hidden, residual
    out = _Marker.apply(fn, hidden, residual)
    if residual is None:
        return out, None
    return out


def _round_up_to(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def _first_matrix(unit: FlatUnit):
    """(weight, element offset, bias offset or None) of the first 2-D parameter in a unit's flat
    layout -- the weight of the block's first GEMM -- when it is a plain ``[N, K]`` matrix."""
    for k, p in enumerate(unit.params):
        if p.dim() == 2:
            if p.shape[1] % 8:
                return None
            bias_off = None
            if k + 1 < len(unit.params) and unit.params[k + 1].dim() == 1 and \
                    unit.params[k + 1].numel() == p.shape[0] and unit.param_names[k + 1].endswith("bias") and \
                    unit.param_names[k + 1].rsplit(".", 1)[0] == unit.param_names[k].rsplit(".", 1)[0]:
                bias_off = unit.offsets[k + 1]
            return p, unit.offsets[k], bias_off
        if p.dim() > 2:
            return None
    return None


class TrainEngine:
    def __init__(self, model: nn.Module, pstate: Optional[ParallelState] = None,
                 strategy: Optional[StageStrategy] = None, grad_accum_steps: int = 1,
                 ckpt_layers: int = 0, hp: Optional[Dict] = None, comm_backend: str = "nccl",
                 grad_dtype: Optional[torch.dtype] = None, overlap: bool = True,
                 pre_post_strategy: Optional[StageStrategy] = None, use_grad_ring: bool = True, tied_group=None,
                 zero3_gather: str = "nccl"):
        self.model = model
        self.ps = pstate or ParallelState.single()
        self.strategy = strategy or StageStrategy(1, 1, 1, False, False, False, 0, 0, 0, 0)
        self.G = int(grad_accum_steps)
        self.hp = dict(DEFAULT_HP, **(hp or {}))
        from ..utils.grad_scaler import ConstantGradScaler
        # constant loss scale (fp16 runs): the loss is multiplied before the backward pass and the
        # optimizer kernels divide by it together with the data-parallel / micro-step average
        self.scaler = ConstantGradScaler(float(self.hp.get("loss_scale", 1.0)))
        self.comm_backend = comm_backend
        self.overlap = overlap
        zero = self.strategy.zero
        pp_zero = (pre_post_strategy or self.strategy).zero
        dp, dpr = self.ps.dp_size, self.ps.dp_rank
        self.device = next(model.parameters()).device
        self.cuda = self.device.type == "cuda"
        if grad_dtype is None:
            # bf16 buckets are enough when nothing is accumulated in them across micro steps
            pdt = next(model.parameters()).dtype
            grad_dtype = pdt if (self.G == 1 or zero >= ZeroLevel.OPT_GRAD) else torch.float32
        self.grad_dtype = grad_dtype

        # ----------------------------------------------------------------------- units
        lm = getattr(model, "language_model", model)
        self.stacks = [s for s in (getattr(lm, "encoder", None), getattr(lm, "decoder", None)) if s is not None]
        layer_params = set()
        self.units: List[FlatUnit] = []
        self.layer_units: Dict[int, List[FlatUnit]] = {}
        mk = dict(dp_size=dp, dp_rank=dpr, device=self.device, dtype=next(model.parameters()).dtype)
        pre_params = []
        if getattr(lm, "embedding", None) is not None:
            pre_params = [(f"embedding.{n}", p) for n, p in lm.embedding.named_parameters()]
        pre_ids = {id(p) for _, p in pre_params}
        for stack in self.stacks:
            stack.hooks = self
            us = []
            # unit names key the events, ring slots and checkpoint entries: the blocks of a second
            # stack (decoder of an encoder-decoder model) restart at index 0, so they get a prefix
            prefix = "layer" if stack is self.stacks[0] else f"stack{self.stacks.index(stack)}_layer"
            for i, layer in enumerate(stack.layers):
                u = FlatUnit(f"{prefix}{layer.layer_idx}", layer, zero=zero, **mk)
                u.ring_index = i          # position in its stack: decides the weight ring slot
                us.append(u)
                layer_params.update(id(p) for p in u.params)
            self.layer_units[id(stack)] = us
        # A stack that is not the last one (the encoder of an encoder-decoder model) finishes its
        # backward pass after every block of the later stacks: its own non-block parameters (the
        # final norm) get their gradient late, so they go with the embedding unit, which is reduced
        # at the very end of the backward pass, not with the head unit, which is reduced first.
        for stack in self.stacks[:-1]:
            for n, p in stack.named_parameters():
                if id(p) not in layer_params and id(p) not in pre_ids:
                    pre_params.append((f"stack{self.stacks.index(stack)}.{n}", p))
                    pre_ids.add(id(p))
        post_params = [(n, p) for n, p in model.named_parameters()
                       if id(p) not in layer_params and id(p) not in pre_ids]
        # A table tied across pipeline stages (the embedding here, the output projection on the last
        # stage, or the other way round): its gradient is summed with the other stage's once per
        # iteration, on the full gradient, so the unit that holds it keeps unsharded gradients and
        # reduces them after the last micro step only (at most ZeRO-1).
        self.tied_group = tied_group
        self._deferred_tied: List[FlatUnit] = []
        has_tied = tied_group is not None and any(getattr(p, "_tied_across_stages", False) for p in model.parameters())
        pp_cap = ZeroLevel.OPT if has_tied else ZeroLevel.OPT_GRAD
        self.pre_unit = FlatUnit("pre", pre_params, zero=min(pp_zero, pp_cap), **mk) if pre_params else None
        self.post_unit = FlatUnit("post", post_params, zero=min(pp_zero, pp_cap), **mk) if post_params else None
        for stack in self.stacks:
            self.units.extend(self.layer_units[id(stack)])
        for u in (self.pre_unit, self.post_unit):
            if u is not None:
                self.units.append(u)
        for stack in self.stacks:
            stack.gradient_checkpointing = min(int(ckpt_layers), len(stack.layers))
        # Parameters that are replicated over the tensor-parallel group but whose gradient each rank
        # only computes in part: norm weights inside the sequence-sharded region (a rank sees its
        # tokens only) and the position / token-type tables (only the first rank adds them).  Their
        # bucket slices are summed over the group before the data-parallel reduction
        # (reference: allreduce_sequence_parallel_grad, mist/distributed/op.py:162-172).
        sp_on = bool(getattr(lm, "sequence_parallel", False))
        for u in self.units:
            u.tp_sum_slices = []
            if self.ps.tp_size > 1:
                for p, o in zip(u.params, u.offsets):
                    if getattr(p, "_tp_partial_grad", False) or (sp_on and getattr(p, "_sequence_parallel", False)):
                        u.tp_sum_slices.append((o, p.numel()))
            u.tied_slices = [(o, p.numel()) for p, o in zip(u.params, u.offsets)
                             if has_tied and getattr(p, "_tied_across_stages", False)]

        # -------------------------------------------------------- buckets, state, streams
        from .swap import ActivationSwapper, SwapStreams
        self.swap_streams = SwapStreams(self.device)
        oo, ao = float(self.strategy.opt_offload), float(self.strategy.act_offload)
        wo, go = float(self.strategy.weight_offload), float(self.strategy.grad_offload)
        # Gradient buckets.  With sharded gradients (ZeRO-2/3) a block's full-size bucket is only
        # needed from its backward pass until its reduction, so the blocks share a ring of two
        # buckets; otherwise every unit keeps its own (it accumulates over micro steps).
        layer_units = self._all_layer_units()
        self.use_grad_ring = bool(use_grad_ring) and zero >= ZeroLevel.OPT_GRAD and dp > 1 and len(layer_units) > 2
        self.grad_ring, self._ring_free, self._ring_next = [], [], 0
        if self.use_grad_ring:
            biggest = max(u.padded for u in layer_units)
            self.grad_ring = [torch.zeros(biggest, dtype=self.grad_dtype, device=self.device) for _ in range(2)]
            self._ring_free = [None, None]
        for u in self.units:
            if self.use_grad_ring and u in layer_units:
                u.ring_slot = None
            else:
                # a unit that accumulates over micro steps although the stage shards its gradients
                # (the tied table's unit) accumulates in fp32 like every other accumulating bucket
                gdt = torch.float32 if (u.tied_slices and self.G > 1) else self.grad_dtype
                u.bind_grad_bucket(torch.zeros(u.padded, dtype=gdt, device=self.device))
            u.init_optimizer_state(offload_ratio=oo if u in layer_units else 0.0)
            if u in layer_units:      # like the optimizer state, only the blocks' tensors are offloaded
                u.enable_weight_offload(wo)
                u.enable_grad_offload(go)
        host_n = max((u.opt_host_numel for u in self.units), default=0)
        self.opt_staging = [torch.empty(host_n, dtype=torch.float32, device=self.device) for _ in range(3)] if host_n else None
        self.act_swapper = ActivationSwapper(ao, self.swap_streams) if ao > 0 else None
        self.compute_stream = torch.cuda.current_stream() if self.cuda else None
        self.comm_stream = torch.cuda.Stream() if (self.cuda and overlap) else self.compute_stream
        self.param_ready: Dict[str, "torch.cuda.Event"] = {}
        #: recorded on the comm stream once a bucket has been read by a mid-iteration reduction
        self.bucket_free: Dict[str, "torch.cuda.Event"] = {}
        self._micro = 0
        self._pending_post = False
        # Ring of full-weight slots (two: current block + the prefetched one) for blocks whose
        # full weights are not persistent on the device: ZeRO-3 shards and host-offloaded weights.
        self.zero3 = any(u.ring_resident for u in layer_units)
        self._step_scratch = None
        if self.zero3:
            biggest = max(u.padded for us in self.layer_units.values() for u in us)
            self._slots = [torch.empty(biggest, dtype=mk["dtype"], device=self.device) for _ in range(2)]
            self._slot_of: Dict[str, int] = {}
            self._gather_done: Dict[str, "torch.cuda.Event"] = {}
            if any(u.weight_split is not None for u in layer_units):
                self._step_scratch = torch.empty(biggest, dtype=mk["dtype"], device=self.device)
                for u in layer_units:      # drop the start-up copies of the full weights
                    if u.weight_split is not None:
                        u._use_views(self._slots[0][: u.padded])
                        u._boot_full = None
        # "fused": in the forward pass a block's remote weight shards are pulled in by the block's
        # first GEMM itself (one kernel) instead of a prefetched all-gather; the backward pass keeps
        # the prefetch.  Needs plain ZeRO-3 shards (no host-offloaded weights) on CUDA.
        self.param_gather = None
        if (comm_backend == "fused" or zero3_gather == "fused") and dp > 1 and self.cuda:
            from .symm import group_on_one_node
            if not group_on_one_node(self.ps.dp_group):
                # peer-memory kernels need every data-parallel rank on this node
                comm_backend = self.comm_backend = "nccl"
                zero3_gather = "nccl"
        if (zero3_gather == "fused" and self.zero3 and self.cuda and dp > 1
                and F.Settings.gemm_backend == "tcgen05" and not (F.Settings.tp_backend == "fused" and self.ps.tp_size > 1)
                and all(u.param_shard is not None for u in layer_units)):
            from .fused_zero3 import ParamGatherContext
            biggest = max(u.padded for u in layer_units)
            self.param_gather = ParamGatherContext(self.ps.dp_group, _round_up_to(biggest, 128 * dp), self.device)
            self._slots = [self.param_gather.slot_tensor(0), self.param_gather.slot_tensor(1)]
            self._dp_root = dist.get_global_rank(self.ps.dp_group, 0)
            for u in layer_units:
                u.first_weight = _first_matrix(u)
        self.fused = None
        if comm_backend == "fused" and dp > 1 and (wo > 0 or go > 0):
            comm_backend = self.comm_backend = "nccl"     # offloaded weights / gradients use the library path
        if comm_backend == "fused" and dp > 1:
            from .fused_comm import FusedDPComm
            self.fused = FusedDPComm(self)

    def _all_layer_units(self):
        return [u for us in self.layer_units.values() for u in us]

    def layer_context(self, stack, i):
        """Context the stack wraps around block ``i``'s forward (activation swapping)."""
        import contextlib
        if self.act_swapper is None or not torch.is_grad_enabled():
            return contextlib.nullcontext()
        self.act_swapper.set_scope((self._micro, id(stack), i))
        return self.act_swapper.hooks()

    # -------------------------------------------------------------------- stream helpers
    def _on_comm(self):
        if self.cuda and self.comm_stream is not self.compute_stream:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            return torch.cuda.stream(self.comm_stream)
        import contextlib
        return contextlib.nullcontext()

    def _wait_params(self, unit: FlatUnit):
        ev = self.param_ready.pop(unit.name, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def _wait_bucket(self, unit: Optional[FlatUnit]):
        if unit is None:
            return
        ev = self.bucket_free.pop(unit.name, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    # ----------------------------------------------------------------- ZeRO-3 residency
    def _slot_for(self, unit: FlatUnit) -> int:
        """Blocks alternate between the two weight slots by their position in the stack, always the
        same slot for the same block: tensors that autograd saved in a forward pass are views into
        the slot, so the block must come back to the same memory for its backward pass, also when
        several forward passes are in flight (pipeline warm-up) before the first backward."""
        slot = unit.ring_index & 1
        self._slot_of[unit.name] = slot
        return slot

    def _gather(self, unit: FlatUnit):
        """Starts the all-gather of ``unit``'s weights into the next ring slot (comm stream)."""
        if not self.zero3 or unit.flat_param is not None or not unit.ring_resident:
            return
        slot = self._slot_for(unit)
        with self._on_comm(), record(f"{unit.name}.unshard"):
            unit.unshard(self._slots[slot], self.ps.dp_ag_group if unit.is_zero3 else None,
                         streams=self.swap_streams)
            if self.cuda:
                ev = torch.cuda.Event()
                ev.record()
                self._gather_done[unit.name] = ev

    def _gather_in_first_gemm(self, unit: FlatUnit) -> bool:
        """Forward pass of a block whose weights are not resident: stages this rank's shard in a
        symmetric slot, fetches the few parameters used before the first GEMM (the input norm)
        with a small broadcast, and arms the first linear layer to run the weight-gathering GEMM.
        Returns False when the block has to take the all-gather path."""
        pg, fw = self.param_gather, getattr(unit, "first_weight", None)
        if pg is None or fw is None or unit.flat_param is not None or unit.padded != pg.padded:
            return False
        weight, b_off, bias_off = fw
        if b_off > unit.shard_numel:
            return False
        slot = self._slot_for(unit)
        full = self._slots[slot][: unit.padded]
        with record(f"{unit.name}.unshard_in_first_gemm"):
            pg.stage_shard(slot, unit.param_shard)
        if b_off:
            dist.broadcast(full[:b_off], src=self._dp_root, group=self.ps.dp_ag_group)
        unit.flat_param = full
        unit._use_views(full)
        unit._boot_full = None
        N, K = weight.shape
        weight.param_gather = lambda x2: pg.gather_linear(slot, x2, b_off, N, K, bias_off)
        return True

    def _ensure_resident(self, unit: FlatUnit):
        if not self.zero3:
            return
        self._gather(unit)
        ev = self._gather_done.pop(unit.name, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def _release(self, unit: FlatUnit):
        if self.zero3:
            with record(f"{unit.name}.reshard"):
                unit.reshard()

    # ----------------------------------------------------------- callbacks from the stack
    def before_layer(self, stack, i, hidden, residual):
        units = self.layer_units[id(stack)]
        u = units[i]
        self._wait_params(u)
        if self._gather_in_first_gemm(u):
            pass                                  # the next block gathers inside its own first GEMM
        else:
            self._ensure_resident(u)
            if i + 1 < len(units) and self.param_gather is None:
                self._gather(units[i + 1])          # one-block look-ahead
        return _mark(lambda: self._layer_backward_done(stack, i), hidden, residual)

    def after_layer(self, stack, i, hidden, residual):
        units = self.layer_units[id(stack)]
        if torch.is_grad_enabled():
            hidden, residual = _mark(lambda: self._layer_backward_start(stack, i), hidden, residual)
        # (not under pipeline parallelism: there further forward passes may come before the
        # backward pass and would reuse the slot)
        keep = (i + 1 == len(units) and stack is self.stacks[-1] and torch.is_grad_enabled()
                and self.ps.num_stages == 1)
        if self.zero3 and not keep:
            # block i's slot is reused by block i+2; only the very last block (of the last stack) stays
            # resident, because the backward pass starts with it
            self._release(units[i])
        if i + 1 == len(units) and self.post_unit is not None:
            self._wait_params(self.post_unit)
        return hidden, residual

    def _acquire_ring_slot(self, unit: FlatUnit):
        slot = self._ring_next
        self._ring_next ^= 1
        ev = self._ring_free[slot]
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)     # the previous user's reduction has read it
            self._ring_free[slot] = None
        unit.ring_slot = slot
        if self.fused is not None and self.fused.handles(unit):
            self.fused.bind_ring_slot(unit, slot)
        else:
            unit.bind_grad_bucket(self.grad_ring[slot], fresh=True)

    def _layer_backward_start(self, stack, i):
        units = self.layer_units[id(stack)]
        self._wait_bucket(units[i])
        if self.use_grad_ring:
            self._acquire_ring_slot(units[i])
        if self.act_swapper is not None and i > 0:
            self.act_swapper.prefetch((self._micro, id(stack), i - 1))   # one block ahead of its backward
        if i + 1 == len(units) and self.post_unit is not None and stack is self.stacks[-1]:
            self._unit_backward_done(self.post_unit)   # head + final norm finished before the last block
        if self.zero3:
            u = units[i]
            if u.flat_param is None:
                self._ensure_resident(u)
            if i > 0:
                self._gather(units[i - 1])

    def _layer_backward_done(self, stack, i):
        if self.act_swapper is not None:
            self.act_swapper.release((self._micro, id(stack), i))
        u = self.layer_units[id(stack)][i]
        self._unit_backward_done(u)
        if self.zero3:
            self._release(u)

    # --------------------------------------------------------------------- gradient path
    def _release_ring_slot(self, unit: FlatUnit):
        slot = getattr(unit, "ring_slot", None)
        if slot is None:
            return
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record()                       # recorded on the stream that ran the reduction
            self._ring_free[slot] = ev
        unit.ring_slot = None

    def _tp_sum_partial_grads(self, unit: FlatUnit):
        """Sums the bucket slices of tensor-parallel-replicated parameters with partial gradients."""
        g = unit.flat_grad
        parts = [g[o:o + n] for o, n in unit.tp_sum_slices]
        flat = torch.cat([t.float() for t in parts]) if len(parts) > 1 else parts[0].float()
        dist.all_reduce(flat, group=self.ps.tp_group)
        off = 0
        for t in parts:
            t.copy_(flat[off:off + t.numel()])
            off += t.numel()

    def _sum_tied_grads(self, unit: FlatUnit):
        """Sums the gradient of the table tied across pipeline stages with the other stage's copy."""
        for o, n in unit.tied_slices:
            dist.all_reduce(unit.flat_grad[o:o + n], group=self.tied_group)

    def flush_tied(self):
        """End of the pipeline schedule: the units that hold a table tied across stages sum its
        gradient with the other stage's copy, reduce and step.  This cannot happen where the unit's
        backward pass ends: the last stage reaches that point at the start of its last backward pass,
        the first stage at the very end of the iteration, and the first stage needs the last stage to
        keep going in between."""
        units, self._deferred_tied = self._deferred_tied, []
        for unit in units:
            with self._on_comm():
                self._sum_tied_grads(unit)
            self._reduce_and_step(unit, True)

    def _unit_backward_done(self, unit: FlatUnit):
        last = self._micro == self.G - 1
        unit.collect_autograd_grads()
        if unit.tp_sum_slices and (last or unit.zero >= ZeroLevel.OPT_GRAD):
            with self._on_comm():
                self._tp_sum_partial_grads(unit)
        if unit.tied_slices:
            if last:
                self._deferred_tied.append(unit)
            return          # gradients accumulate in the unit's bucket until the end of the iteration
        self._reduce_and_step(unit, last)

    def _reduce_and_step(self, unit: FlatUnit, last: bool):
        if self.fused is not None and self.fused.handles(unit) and not unit.opt_host_numel:
            self.fused.reduce_and_step(unit, last)
            return
        with self._on_comm():
            with record(f"{unit.name}.post_backward_grad_reduce"):
                grad = unit.reduce_grads(self.ps.dp_rs_group, last, streams=self.swap_streams)
            if grad is not None:
                swap = ((self.swap_streams, self.opt_staging)
                        if (unit.opt_host_numel or unit.weight_split is not None) else None)
                with record(f"OPT-{unit.name}.step"):
                    unit.optimizer_step(grad, self.hp, self.ps.dp_ag_group,
                                        grad_divisor=float(self.ps.dp_size * self.G) * self.scaler.loss_scale, swap=swap,
                                        step_scratch=self._step_scratch)
                if self.cuda:
                    ev = torch.cuda.Event()
                    ev.record()
                    self.param_ready[unit.name] = ev
            elif self.cuda and self.comm_stream is not self.compute_stream:
                ev = torch.cuda.Event()
                ev.record()
                self.bucket_free[unit.name] = ev
            self._release_ring_slot(unit)

    # ------------------------------------------------------------------------- stepping
    def forward_backward(self, batch: Dict, micro_index: int = 0):
        """One micro step: forward, loss, backward.  Returns the detached loss."""
        self._micro = micro_index
        if self.pre_unit is not None:
            self._wait_params(self.pre_unit)
        loss = self.model(**batch)
        self._wait_bucket(self.pre_unit)
        self._wait_bucket(self.post_unit)
        self.scaler.scale(loss).backward()
        if self.pre_unit is not None:
            self._unit_backward_done(self.pre_unit)
        return loss.detach()

    def train_step(self, batches: List[Dict]):
        """One iteration over ``G`` micro batches; optimizer steps are issued per unit as
        soon as the unit's last gradient is reduced."""
        assert len(batches) == self.G, f"expected {self.G} micro batches, got {len(batches)}"
        losses = [self.forward_backward(b, k) for k, b in enumerate(batches)]
        return torch.stack(losses).mean()

    def finish(self):
        """Blocks the compute stream on every outstanding optimizer step."""
        if self.cuda:
            for ev in self.param_ready.values():
                torch.cuda.current_stream().wait_event(ev)
            self.param_ready.clear()
            if self.comm_stream is not self.compute_stream:
                torch.cuda.current_stream().wait_stream(self.comm_stream)

    # ----------------------------------------------------------------------- accounting
    def num_parameters(self) -> int:
        return sum(u.numel for u in self.units)

    def state_bytes(self) -> Dict[str, int]:
        def persistent(u):
            if u.weight_split is not None:
                return u.weight_split.dev_numel
            return u.param_shard.numel() if u.param_shard is not None else u.flat_param.numel()
        w = sum(persistent(u) * 2 for u in self.units)
        g = sum(u.flat_grad.numel() * u.flat_grad.element_size() for u in self.units)
        o = sum(u.master.numel() * 12 for u in self.units)
        return {"weights": w, "grads": g, "optimizer": o}
