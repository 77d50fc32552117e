"""Flat parameter / gradient / optimizer-state storage of one schedulable unit
(the embedding stage, one transformer block, or the head).

All parameters of the unit are views into one contiguous bf16 buffer and all gradients
into one contiguous bucket, so the data-parallel collectives and the optimizer run once
per unit on flat memory.  Sharding level:

==========  ======================  ==================  =========================
level       weights                 gradients           fp32 master + Adam moments
==========  ======================  ==================  =========================
none        full                    all-reduce          full
ZeRO-1      full                    reduce-scatter at   1/dp shard
                                    the last micro step
ZeRO-2      full                    reduce-scatter      1/dp shard
                                    every micro step
ZeRO-3      1/dp shard; gathered    as ZeRO-2           1/dp shard
            into a ring slot
==========  ======================  ==================  =========================

Host offloading (fractions of the strategy vector): the trailing ``weight_offload`` of the
persistent weights (the full buffer, or the ZeRO-3 shard) and the trailing ``grad_offload``
of the fp32 accumulator of reduced gradients live in pinned host memory.  Offloaded weights
are assembled in a ring slot one block ahead of their use, exactly like ZeRO-3 gathered
weights, and written back after the optimizer step (reference: mist/re_swap_manager/
flat_param.py:1124-1250 swap-in/out of weights and gradients).

Parity: reference mist/re_swap_manager/flat_param.py:91-108 (levels), :315-420 (handle),
:986-1121 (ring-buffer allocation), :1283-1370 (unshard), :1459-1529 (gradient reduction).
Unlike the reference, reduced gradients are averaged over data-parallel ranks and
micro steps (there the division is commented out and gradients are summed).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..config import ZeroLevel
from ..ops import functional as F

ALIGN = 128  # elements: every parameter view starts 256-byte aligned (TMA needs 16)


def _round_up(n, m):
    return (n + m - 1) // m * m


class FlatUnit:
    def __init__(self, name: str, module: nn.Module, *, dp_size: int = 1, dp_rank: int = 0,
                 zero: ZeroLevel = ZeroLevel.NONE, device=None, dtype=torch.bfloat16,
                 allocator=None, init_params: bool = True):
        self.name, self.module = name, module
        self.dp_size, self.dp_rank, self.zero = dp_size, dp_rank, ZeroLevel(zero)
        self.dtype = dtype
        if isinstance(module, nn.Module):
            params = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        else:   # an explicit list of (name, parameter)
            params = [(n, p) for n, p in module if p.requires_grad]
        # de-duplicate tied parameters
        seen, self.params, self.param_names = set(), [], []
        for n, p in params:
            if id(p) not in seen:
                seen.add(id(p))
                self.params.append(p)
                self.param_names.append(n)
        self.device = device if device is not None else (self.params[0].device if self.params else "cpu")
        self.offsets, off = [], 0
        for p in self.params:
            self.offsets.append(off)
            off += _round_up(p.numel(), ALIGN)
        self.numel = off
        self.padded = _round_up(max(off, 1), ALIGN * max(dp_size, 1))
        self.shard_numel = self.padded // dp_size
        alloc = allocator or (lambda n, dt: torch.zeros(n, dtype=dt, device=self.device))
        self._alloc = alloc
        # ---- weights
        self.flat_param: Optional[torch.Tensor] = None     # full weights (None while resharded, ZeRO-3)
        self.param_shard: Optional[torch.Tensor] = None    # persistent 1/dp shard (ZeRO-3 only)
        full = alloc(self.padded, dtype)
        if init_params:
            for p, o in zip(self.params, self.offsets):
                if p.device.type != "meta":
                    full[o:o + p.numel()].copy_(p.detach().reshape(-1).to(dtype))
        if self.zero >= ZeroLevel.FULL and dp_size > 1:
            self.param_shard = full[self.shard_range()].clone()
            self._use_views(full)     # keep shapes/devices sane until the first unshard
            self._boot_full = full
        else:
            self.flat_param = full
            self._use_views(full)
        # ---- gradients
        self.flat_grad: Optional[torch.Tensor] = None      # bound by the engine (own bucket or ring slot)
        self.grad_shard_acc: Optional[torch.Tensor] = None  # fp32 accumulator of the reduced shard
        self.micro_steps_accumulated = 0
        # ---- optimizer state (created by init_optimizer_state)
        self.master = self.exp_avg = self.exp_avg_sq = None
        self.step_count = 0
        # ---- host offloading (enable_weight_offload / enable_grad_offload)
        self.weight_split = None       # SplitTensor of the persistent weights
        self.grad_split = None         # SplitTensor of the fp32 accumulator of the reduced shard

    # ------------------------------------------------------------------------- layout
    def shard_range(self, rank: Optional[int] = None) -> slice:
        r = self.dp_rank if rank is None else rank
        return slice(r * self.shard_numel, (r + 1) * self.shard_numel)

    @property
    def sharded_state(self) -> bool:
        return self.zero >= ZeroLevel.OPT and self.dp_size > 1

    @property
    def state_numel(self) -> int:
        return self.shard_numel if self.sharded_state else self.padded

    @property
    def is_zero3(self) -> bool:
        return self.zero >= ZeroLevel.FULL and self.dp_size > 1

    @property
    def ring_resident(self) -> bool:
        """True when the full weights only exist while the block is in use (ring slot)."""
        return self.param_shard is not None or self.weight_split is not None

    @property
    def persistent_numel(self) -> int:
        return self.shard_numel if self.is_zero3 else self.padded

    def persistent_region(self, full: torch.Tensor) -> torch.Tensor:
        """The part of a full-size buffer that this rank stores persistently."""
        return full[self.shard_range()] if self.is_zero3 else full[: self.padded]

    def enable_weight_offload(self, ratio: float):
        """Moves the trailing ``ratio`` of the persistent weights to pinned host memory.  Call
        after ``init_optimizer_state`` (the master weights are cut from the device copy)."""
        from .swap import SplitTensor
        if ratio <= 0:
            return
        src = self.param_shard if self.param_shard is not None else self.flat_param
        split = SplitTensor(src, ratio)
        if not split.host_numel:
            return
        self.weight_split = split
        self.param_shard = None
        self.flat_param = None

    def enable_grad_offload(self, ratio: float):
        """Keeps the trailing ``ratio`` of the reduced-gradient accumulator on the host between
        micro steps.  Only sharded gradients (ZeRO-2/3) accumulate outside the bucket."""
        from .swap import SplitTensor
        if ratio <= 0 or not (self.zero >= ZeroLevel.OPT_GRAD and self.dp_size > 1):
            return
        acc = torch.zeros(self.shard_numel, dtype=torch.float32, device=self.device)
        split = SplitTensor(acc, ratio)
        if split.host_numel:
            self.grad_split = split

    def _use_views(self, flat: torch.Tensor):
        for p, o in zip(self.params, self.offsets):
            p.data = flat[o:o + p.numel()].view(p.shape)

    def bind_grad_bucket(self, bucket: torch.Tensor, fresh: bool = True):
        """Points every parameter's gradient view into ``bucket`` (a full-size flat tensor)."""
        assert bucket.numel() >= self.padded
        self.flat_grad = bucket[: self.padded]
        for p, o in zip(self.params, self.offsets):
            p.grad_bucket = self.flat_grad[o:o + p.numel()].view(p.shape)
            if fresh:
                p.grad_accumulate = False

    def collect_autograd_grads(self):
        """Moves ``.grad`` tensors produced by autograd (norm weights, biases, embeddings)
        into the bucket; linear weights were written there directly by the wgrad GEMM."""
        for p in self.params:
            g = p.grad
            if g is None:
                if not getattr(p, "grad_accumulate", False):
                    p.grad_bucket.zero_()      # parameter did not take part in this micro step
                    p.grad_accumulate = True
                continue
            if getattr(p, "grad_accumulate", False):
                p.grad_bucket.add_(g.to(p.grad_bucket.dtype))
            else:
                p.grad_bucket.copy_(g)
                p.grad_accumulate = True
            p.grad = None

    # ------------------------------------------------------------------ optimizer state
    def init_optimizer_state(self, state_dtype=torch.float32, offload_ratio: float = 0.0):
        """Creates fp32 master weights and Adam moments; the trailing ``offload_ratio`` of each
        lives in pinned host memory and is staged through device buffers around the step."""
        src = self.param_shard if self.param_shard is not None else (
            self.flat_param[self.shard_range()] if self.sharded_state else self.flat_param)
        self.master = src.detach().to(state_dtype).clone()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.opt_split = None
        if offload_ratio > 0:
            from .swap import SplitTensor
            self.opt_split = [SplitTensor(t, offload_ratio) for t in (self.master, self.exp_avg, self.exp_avg_sq)]
            self.master, self.exp_avg, self.exp_avg_sq = (s.device_part for s in self.opt_split)

    @property
    def opt_host_numel(self) -> int:
        return self.opt_split[0].host_numel if getattr(self, "opt_split", None) else 0

    # --------------------------------------------------------------------------- ZeRO-3
    def unshard(self, slot: torch.Tensor, group, async_op=False, streams=None):
        """Builds the full weights in ``slot`` and points the parameters at it: offloaded
        weights are assembled from their device and host parts, ZeRO-3 shards all-gathered
        (in place when the shard was assembled inside the slot)."""
        assert self.ring_resident
        full = slot[: self.padded]
        handle = None
        if self.weight_split is not None:
            mine = self.persistent_region(full)
            self.weight_split.load_into(mine, streams)
            if self.is_zero3 and group is not None:
                handle = dist.all_gather_into_tensor(full, mine, group=group, async_op=async_op)
        elif group is not None:
            handle = dist.all_gather_into_tensor(full, self.param_shard, group=group, async_op=async_op)
        else:
            full[self.shard_range()].copy_(self.param_shard)
        self.flat_param = full
        self._use_views(full)
        self._boot_full = None
        return handle

    def reshard(self):
        if self.ring_resident:
            self.flat_param = None

    # ---------------------------------------------------------------- gradient reduction
    def _accumulate_offloaded(self, out: torch.Tensor, last_micro_step: bool, streams):
        """Adds one micro step's reduced shard to the accumulator whose tail lives on the host.
        The first micro step writes (nothing to load), the others load-add-store; on the last
        one the full sum is returned in a temporary for the optimizer."""
        sp = self.grad_split
        first = self.micro_steps_accumulated == 1
        full = torch.empty(self.shard_numel, dtype=torch.float32, device=out.device)
        if first:
            F.accumulate_grad(out, full, 1.0, False)
        else:
            sp.load_into(full, streams)
            F.accumulate_grad(out, full, 1.0, True)
        if last_micro_step:
            return full
        sp.store_from(full, streams)
        if streams.cuda:
            full.record_stream(streams.d2h)
        return None

    def reduce_grads(self, group, last_micro_step: bool, streams=None):
        """Reference (NCCL) path.  Returns the tensor the optimizer should consume, or None
        when nothing is due yet."""
        self.micro_steps_accumulated += 1
        if self.dp_size == 1 or group is None:
            return self.flat_grad if last_micro_step else None
        if self.zero >= ZeroLevel.OPT_GRAD:
            out = torch.empty(self.shard_numel, dtype=self.flat_grad.dtype, device=self.flat_grad.device)
            dist.reduce_scatter_tensor(out, self.flat_grad, group=group)
            if self.grad_shard_acc is None and last_micro_step and self.micro_steps_accumulated == 1:
                return out
            for p in self.params:
                p.grad_accumulate = False      # the bucket restarts for the next micro step
            if self.grad_split is not None:
                return self._accumulate_offloaded(out, last_micro_step, streams)
            if self.grad_shard_acc is None:
                self.grad_shard_acc = torch.zeros(self.shard_numel, dtype=torch.float32, device=out.device)
            F.accumulate_grad(out, self.grad_shard_acc, 1.0, True)
            return self.grad_shard_acc if last_micro_step else None
        if not last_micro_step:
            return None
        if self.zero == ZeroLevel.OPT:
            out = torch.empty(self.shard_numel, dtype=self.flat_grad.dtype, device=self.flat_grad.device)
            dist.reduce_scatter_tensor(out, self.flat_grad, group=group)
            return out
        dist.all_reduce(self.flat_grad, group=group)
        return self.flat_grad

    def optimizer_step(self, grad: torch.Tensor, hp: Dict, group, grad_divisor: float, swap=None,
                       step_scratch: Optional[torch.Tensor] = None):
        """Fused Adam on this rank's state, writing the bf16 weights, then (ZeRO-1/2) the
        all-gather that refreshes the other ranks' slices.  ``swap`` = (streams, staging
        buffers) when part of the state lives on the host."""
        self.step_count += 1
        if self.weight_split is not None:
            # offloaded weights: the step writes into a scratch copy that is then split again
            streams = swap[0]
            if streams.cuda:
                torch.cuda.current_stream().wait_stream(streams.d2h)   # scratch free again
            scratch = step_scratch[: self.padded]
            model_out = scratch[self.shard_range()] if self.sharded_state else scratch
        elif self.param_shard is not None:
            model_out = self.param_shard
        elif self.sharded_state:
            model_out = self.flat_param[self.shard_range()]
        else:
            model_out = self.flat_param
        n_state = self.state_numel
        g = grad if grad.numel() == n_state else grad[self.shard_range()]
        kw = dict(lr=hp["lr"], beta1=hp["beta1"], beta2=hp["beta2"], eps=hp["eps"], weight_decay=hp["weight_decay"],
                  step=self.step_count, inv_scale=1.0 / grad_divisor, adamw=hp.get("adamw", True))
        split = getattr(self, "opt_split", None)
        if split is None:
            F.adam_step(self.master, self.exp_avg, self.exp_avg_sq, g, model_out, **kw)
        else:
            streams, staging = swap
            nd = split[0].dev_numel
            cuda = streams.cuda
            if cuda:
                cur = torch.cuda.current_stream()
                streams.h2d.wait_stream(streams.d2h)      # staging buffers free (previous unit stored back)
            staged = [sp_.load(buf, streams) for sp_, buf in zip(split, staging)]
            if nd:
                F.adam_step(self.master, self.exp_avg, self.exp_avg_sq, g[:nd], model_out[:nd], **kw)
            if cuda:
                cur.wait_stream(streams.h2d)
            F.adam_step(staged[0], staged[1], staged[2], g[nd:], model_out[nd:], **kw)
            if cuda:
                streams.d2h.wait_stream(cur)
            for sp_, st in zip(split, staged):
                sp_.store(st, streams)
        if self.weight_split is not None:
            if self.sharded_state and not self.is_zero3 and group is not None:
                dist.all_gather_into_tensor(scratch, model_out, group=group)
            self.weight_split.store_from(self.persistent_region(scratch), swap[0])
        elif self.sharded_state and self.param_shard is None and group is not None:
            dist.all_gather_into_tensor(self.flat_param, model_out, group=group)
        self.micro_steps_accumulated = 0
        if self.grad_shard_acc is not None:
            self.grad_shard_acc.zero_()
        for p in self.params:
            p.grad_accumulate = False
