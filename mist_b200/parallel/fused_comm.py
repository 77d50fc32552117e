"""Data-parallel gradient path on hand-written NVLink kernels.

With ``comm_backend="fused"`` every unit's weight buffer and gradient bucket live in
symmetric memory, and one kernel launch per unit replaces the library sequence
``reduce_scatter -> cast -> Adam -> cast -> all_gather``: each rank pulls its slice of
every peer's bucket over NVLink, reduces in fp32 in a fixed rank order (bit-identical
replicas), applies Adam to its fp32 master shard and stores the new bf16 weights into
every peer's weight buffer.  The launch runs on the communication stream while the
compute stream continues with the backward pass of the previous block.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config import ZeroLevel
from ..ops import native
from ..ops.native import call, ptr
from .flat_unit import FlatUnit
from .symm import SymmetricHeap, ptr_table

FLAG_SLOT_INTS = 32   # ready[R] + done[R] + counter, padded


class FusedDPComm:
    def __init__(self, engine, num_ctas: int = 0):
        self.engine = engine
        ps = engine.ps
        self.group = ps.dp_group
        self.R, self.me = ps.dp_size, ps.dp_rank
        self.num_ctas = num_ctas
        units = [u for u in engine.units if self._eligible(u)]
        gsz = torch.empty(0, dtype=engine.grad_dtype).element_size()
        ring_units = set(id(u) for u in engine._all_layer_units()) if engine.use_grad_ring else set()
        ring_elems = max((u.padded for u in units if id(u) in ring_units), default=0)
        total = (sum(u.padded * (2 + (0 if id(u) in ring_units else gsz)) + 4096 for u in units)
                 + 2 * (ring_elems * gsz + 4096) + FLAG_SLOT_INTS * 4 * (len(units) + 1) + (1 << 20))
        self.heap = SymmetricHeap(total, self.group, engine.device)
        self.tables: Dict[str, Dict] = {}
        flags, flag_off = self.heap.alloc(FLAG_SLOT_INTS * len(units), torch.int32)
        self.ring = []
        if ring_elems:
            for _ in range(2):
                buf, off = self.heap.alloc(ring_elems, engine.grad_dtype)
                self.ring.append((buf, ptr_table(self.heap.peer_ptrs(off))))
        for k, u in enumerate(units):
            t = {}
            if u.param_shard is None:
                new_p, off_p = self.heap.alloc(u.padded, u.dtype)
                new_p.copy_(u.flat_param)
                u.flat_param = new_p
                u._use_views(new_p)
                t["params"] = ptr_table(self.heap.peer_ptrs(off_p))
            else:
                # ZeRO-3: the new weights go to this rank's persistent shard only
                base_bytes = self.me * u.shard_numel * 2
                t["params"] = ptr_table([(ptr(u.param_shard) - base_bytes) if r == self.me else 0
                                         for r in range(self.R)])
            if id(u) in ring_units:
                t["grads"] = None             # bound per backward pass to a ring slot
            else:
                new_g, off_g = self.heap.alloc(u.padded, engine.grad_dtype)
                u.bind_grad_bucket(new_g)
                t["grads"] = ptr_table(self.heap.peer_ptrs(off_g))
            t["flags"] = ptr_table([b + flag_off + 4 * FLAG_SLOT_INTS * k for b in self.heap.peer_base])
            t["epoch"] = 0
            self.tables[u.name] = t
        torch.cuda.synchronize()
        torch.distributed.barrier(group=self.group)

    def _eligible(self, u: FlatUnit) -> bool:
        # a unit whose gradient is first summed with another pipeline stage's copy (tied table)
        # stays on the library path: that sum sits between the backward pass and this reduction
        return u.zero >= ZeroLevel.OPT and u.dp_size > 1 and not getattr(u, "tied_slices", None)

    def handles(self, u: FlatUnit) -> bool:
        return u.name in self.tables

    def bind_ring_slot(self, u: FlatUnit, slot: int):
        buf, table = self.ring[slot]
        u.bind_grad_bucket(buf, fresh=True)
        self.tables[u.name]["grads"] = table

    def reduce_and_step(self, u: FlatUnit, last_micro_step: bool):
        eng = self.engine
        t = self.tables[u.name]
        every_step = u.zero >= ZeroLevel.OPT_GRAD
        if not last_micro_step and not every_step:
            return                                   # ZeRO-1: the bucket keeps accumulating locally
        u.micro_steps_accumulated += 1
        acc = None
        if every_step and eng.G > 1:
            if u.grad_shard_acc is None:
                u.grad_shard_acc = torch.zeros(u.shard_numel, dtype=torch.float32, device=eng.device)
            acc = u.grad_shard_acc
        hp = eng.hp
        t["epoch"] += 1
        if last_micro_step:
            u.step_count += 1
        with eng._on_comm():
            call("mb_fused_grad_reduce_adam", t["grads"], t["params"], t["flags"], ptr(u.master), ptr(u.exp_avg),
                 ptr(u.exp_avg_sq), ptr(acc), u.shard_numel, self.R, self.me, t["epoch"],
                 int(u.flat_grad.dtype == torch.float32), int(last_micro_step), float(hp["lr"]), float(hp["beta1"]),
                 float(hp["beta2"]), float(hp["eps"]), float(hp["weight_decay"]), max(u.step_count, 1),
                 1.0 / (float(self.R * eng.G) * eng.scaler.loss_scale), int(hp.get("adamw", True)), self.num_ctas, native.stream())
            ev = torch.cuda.Event()
            ev.record()
            if last_micro_step:
                eng.param_ready[u.name] = ev
                u.micro_steps_accumulated = 0
            else:
                eng.bucket_free[u.name] = ev
            eng._release_ring_slot(u)
        for p in u.params:
            p.grad_accumulate = False
