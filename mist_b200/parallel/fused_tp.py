"""Sequence-parallel tensor-parallel linears on the fused GEMM + collective kernels.

``ag_linear``  : y = allgather(x_shard) @ W^T (+ bias)      -- column-parallel forward
``linear_rs``  : y_shard = reduce_scatter(x @ W^T) (+ bias) -- row-parallel forward

and their backward passes, which use the same two kernels with the roles swapped:

* column-parallel: ``dx_shard = reduce_scatter(dy @ W)`` is the GEMM->RS kernel with W read
  MN-major; the weight gradient needs the gathered input again, which a peer-memory
  all-gather kernel brings in on the communication stream while the dgrad GEMM runs;
* row-parallel: ``dx = allgather(dy_shard) @ W`` is the AG->GEMM kernel with W read
  MN-major, and it leaves the gathered ``dy`` in local memory for the weight-gradient GEMM.

All buffers that peers touch live in one symmetric heap per tensor-parallel group; flag
blocks are per (kernel mode, shape) call site with a launch counter as epoch.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Tuple

import torch
import torch.distributed as dist

from ..ops import functional as F
from ..ops import native
from ..ops.native import call, ptr
from .symm import SymmetricHeap, ptr_table

native.register_signature(
    "mb_gemm_comm",
    [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
     C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p])

native.register_signature(
    "mb_rs_sum", [C.c_void_p, C.c_size_t, C.c_int, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p])
native.register_signature("mb_gemm_comm_set_pair", [C.c_int], None)
native.register_signature("mb_gemm_comm_last_pair", [], C.c_int)

MODE_AG, MODE_RS = 1, 2
FLAG_INTS = 32


class FusedTPContext:
    """Symmetric buffers and flag blocks of one tensor-parallel group."""

    def __init__(self, group, heap_bytes: int, device=None, n_gather: int = 0, emulate_ranks: int = 0):
        self.group = group
        self.n_gather = n_gather
        if emulate_ranks:
            # single-process stand-in used by profiling runs: "peers" are further local buffers
            self.R, self.me, self.heap = emulate_ranks, 0, None
            self.device = device or torch.device("cuda", torch.cuda.current_device())
        else:
            self.R, self.me = dist.get_world_size(group), dist.get_rank(group)
            self.heap = SymmetricHeap(heap_bytes, group, device)
            self.device = self.heap.device
        self._bufs: Dict[Tuple, Tuple[torch.Tensor, object]] = {}
        self._sites: Dict[Tuple, Dict] = {}

    def _alloc(self, key, numel, dtype):
        if key not in self._bufs:
            if self.heap is not None:
                t, off = self.heap.alloc(numel, dtype)
                table = ptr_table(self.heap.peer_ptrs(off))
            else:
                ts = [torch.zeros(numel, dtype=dtype, device=self.device) for _ in range(self.R)]
                t, table = ts[0], ptr_table([x.data_ptr() for x in ts])
                self._keep = getattr(self, "_keep", []) + ts
            self._bufs[key] = (t, table)
        return self._bufs[key]

    def site(self, key) -> Dict:
        if key not in self._sites:
            flags, table = self._alloc(("flags",) + key, FLAG_INTS, torch.int32)
            chunk = torch.zeros(4096, dtype=torch.int32, device=self.device)
            if self.heap is None:
                flags[: 2 * self.R].fill_(1 << 30)     # emulated peers are always "ready" and "done"
            self._sites[key] = {"flags": table, "flags_t": flags, "chunk": chunk, "epoch": 0}
        return self._sites[key]

    def gathered(self, M, K, tag=""):
        return self._alloc(("A", M, K, tag), M * K, torch.bfloat16)

    def accumulator(self, rows, N, dtype=torch.float32):
        return self._alloc(("acc", rows, N, dtype), rows * N, dtype)

    def rs_slots(self, rows, N):
        """Slots of the store form of GEMM -> reduce-scatter: two sets (used alternately, launch by
        launch) of one ``[rows, N]`` bf16 slot per source rank, in every rank's memory.  Returns
        ``(local tensor [2, R, rows * N], per-set pointer tables)`` where table ``s`` holds, for every
        owner rank, the address of the slot it keeps for tiles from this rank in set ``s``."""
        key = ("rs_slots", rows, N)
        if key not in self._bufs:
            n = rows * N
            if self.heap is not None:
                t, off = self.heap.alloc(2 * self.R * n, torch.bfloat16)
                bases = self.heap.peer_ptrs(off)
            else:
                ts = [torch.zeros(2 * self.R * n, dtype=torch.bfloat16, device=self.device) for _ in range(self.R)]
                t, bases = ts[0], [x.data_ptr() for x in ts]
                self._keep = getattr(self, "_keep", []) + ts
            tables = [ptr_table([b + 2 * ((s * self.R + self.me) * n) for b in bases]) for s in range(2)]
            self._bufs[key] = (t.view(2, self.R, n), tables)
            self._rs_seq = getattr(self, "_rs_seq", {})
            self._rs_seq[key] = 0
        return self._bufs[key]


def _ag_gemm(ctx: FusedTPContext, x_shard: torch.Tensor, w: torch.Tensor, bias, b_mn: bool, tag: str):
    """C[M, N] = allgather(x_shard)[M, K] * B^T; returns (C, gathered A view)."""
    rows, K = x_shard.shape
    M = rows * ctx.R
    N = w.shape[1] if b_mn else w.shape[0]
    a_full, a_table = ctx.gathered(M, K, tag)
    a2 = a_full.view(M, K)
    a2[ctx.me * rows:(ctx.me + 1) * rows].copy_(x_shard)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x_shard.device)
    s = ctx.site((MODE_AG, M, N, K, b_mn, tag))
    s["epoch"] += 1
    call("mb_gemm_comm", MODE_AG, a_table, None, ptr(w), ptr(out), None, s["flags"], ptr(s["chunk"]), M, N, K,
         w.stride(0), out.stride(0), int(b_mn), ptr(bias), ctx.R, ctx.me, s["epoch"], ctx.n_gather, 0, 0, native.stream())
    return out, a2


#: "store" (default): tiles go into per-source slots and are summed in rank order afterwards;
#: "add": the earlier form with TMA reduce-add into one zeroed accumulator (kept for A/B timing)
RS_FORM = "store"


def _gemm_rs(ctx: FusedTPContext, x: torch.Tensor, w: torch.Tensor, b_mn: bool, bias=None, residual=None):
    """``reduce_scatter(x[M, K] * B^T) (+ bias) (+ residual)`` -> this rank's rows, bf16 ``[M/R, N]``.

    Every rank must make the same sequence of calls (the slot set alternates per call)."""
    M, K = x.shape
    N = w.shape[1] if b_mn else w.shape[0]
    rows = M // ctx.R
    if RS_FORM == "store":
        slots, tables = ctx.rs_slots(rows, N)
        key = ("rs_slots", rows, N)
        parity = ctx._rs_seq[key] & 1
        ctx._rs_seq[key] += 1
        s = ctx.site((MODE_RS, M, N, K, b_mn))
        s["epoch"] += 1
        # a bias is added to this rank's partial product inside the kernel: the rank that holds the
        # row-parallel bias (the first) passes it, the others pass none, so every token gets it once
        call("mb_gemm_comm", MODE_RS, None, ptr(x), ptr(w), None, tables[parity], s["flags"], None, M, N, K,
             w.stride(0), N, int(b_mn), ptr(bias), ctx.R, ctx.me, s["epoch"], 0, 0, 2, native.stream())
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=x.device)
        res = residual.contiguous() if residual is not None else None
        call("mb_rs_sum", ptr(slots[parity]), rows * N, ctx.R, rows * N, N, None, ptr(res), ptr(out), native.stream())
        return out
    out = _gemm_rs_add(ctx, x, w, b_mn, bias)
    if residual is not None:
        out = out + residual.reshape(out.shape)
    return out


def _gemm_rs_add(ctx: FusedTPContext, x: torch.Tensor, w: torch.Tensor, b_mn: bool, bias=None):
    """The reduce-add form: fp32 accumulator rows of this rank, as bf16 [M/R, N]."""
    M, K = x.shape
    N = w.shape[1] if b_mn else w.shape[0]
    rows = M // ctx.R
    # two ranks: a + b is order independent, so the sum can be formed in bf16 directly (half the
    # NVLink bytes, no conversion pass); more ranks accumulate in fp32 to stay order independent
    # up to fp32 rounding
    bf16_acc = ctx.R <= 2
    acc, acc_table = ctx.accumulator(rows, N, torch.bfloat16 if bf16_acc else torch.float32)
    acc.zero_()
    s = ctx.site((MODE_RS, M, N, K, b_mn))
    s["epoch"] += 1
    call("mb_gemm_comm", MODE_RS, None, ptr(x), ptr(w), None, acc_table, s["flags"], None, M, N, K, w.stride(0), N,
         int(b_mn), ptr(bias), ctx.R, ctx.me, s["epoch"], 0, 0, int(bf16_acc), native.stream())
    if bf16_acc:
        return acc.view(rows, N).clone()
    out = torch.empty(rows, N, dtype=torch.bfloat16, device=x.device)
    F.cast_to_bf16(acc, out.view(-1))
    return out


class _AGLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, weight, bias, tp):
        y, _ = _ag_gemm(tp, x_shard.contiguous(), weight, bias, False, "fwd")
        ctx.tp = tp
        ctx.save_for_backward(x_shard, weight)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x_shard, weight = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        dx_shard = _gemm_rs(tp, dy, weight, True)                 # dy [M, N] * W [N, K] -> rows of this rank
        # weight gradient needs the gathered input again
        rows, K = x_shard.shape
        x_full, _ = tp.gathered(rows * tp.R, K, "wgrad")
        xf = x_full.view(rows * tp.R, K)
        if tp.heap is not None:
            dist.all_gather_into_tensor(xf, x_shard.contiguous(), group=tp.group)
        else:
            xf.copy_(x_shard.repeat(tp.R, 1))
        bucket = getattr(weight, "grad_bucket", None)
        if bucket is not None:
            F.gemm(dy, xf, a_mn=True, b_mn=True, out=bucket, flags=F.EPI_ACCUM if getattr(weight, "grad_accumulate", False) else 0)
            weight.grad_accumulate = True
            dw = None
        else:
            dw = F.gemm(dy, xf, a_mn=True, b_mn=True)
        db = F.colsum(dy) if ctx.has_bias else None
        return dx_shard, dw, db, None


class _LinearRS(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, tp, residual=None):
        x2 = x.contiguous()
        y = _gemm_rs(tp, x2, weight, False, bias=bias, residual=residual)
        ctx.tp = tp
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        x2, weight = ctx.saved_tensors
        tp = ctx.tp
        # dx = allgather(dy) * W ; W is [N, K_local]: reduction over N -> MN-major B
        dx, dy_full = _ag_gemm(tp, dy_shard.contiguous(), weight, None, True, "bwd")
        bucket = getattr(weight, "grad_bucket", None)
        if bucket is not None:
            F.gemm(dy_full, x2, a_mn=True, b_mn=True, out=bucket,
                   flags=F.EPI_ACCUM if getattr(weight, "grad_accumulate", False) else 0)
            weight.grad_accumulate = True
            dw = None
        else:
            dw = F.gemm(dy_full, x2, a_mn=True, b_mn=True)
        db = F.colsum(dy_shard.contiguous()) if ctx.has_bias else None
        return dx, dw, db, None, (dy_shard if ctx.has_res else None)


def ag_linear(x_shard, weight, bias, tp: FusedTPContext):
    """Column-parallel linear on a ``[tokens / tp, K]`` shard -> ``[tokens, N_local]``."""
    return _AGLinear.apply(x_shard, weight, bias, tp)


def linear_rs(x, weight, bias, tp: FusedTPContext, residual=None):
    """Row-parallel linear ``[tokens, K_local]`` -> this rank's ``[tokens / tp, N]`` rows of the sum
    (+ bias, + ``residual`` of that shape; both are added while the per-rank partial sums are added)."""
    return _LinearRS.apply(x, weight, bias, tp, residual)


_CONTEXTS: Dict[int, FusedTPContext] = {}


def context_for(group, heap_bytes: int = 2 << 30) -> FusedTPContext:
    key = id(group)
    if key not in _CONTEXTS:
        from .symm import group_on_one_node
        if not group_on_one_node(group):
            raise RuntimeError("tp_backend=fused needs the tensor-parallel group on one node (peer memory); "
                               "use tp_backend=nccl for groups that span nodes")
        _CONTEXTS[key] = FusedTPContext(group, heap_bytes)
    return _CONTEXTS[key]
