"""ZeRO-3 weight all-gather fused into the first GEMM of a block.

Under ZeRO-3 each data-parallel rank keeps ``1/R`` of a block's flat bf16 parameters.  The
library path gathers the block with ``all_gather_into_tensor`` and only then starts the
block's first GEMM.  Here one kernel does both: a few CTAs of the persistent GEMM grid
pull the peers' shards over NVLink piece by piece -- the pieces under the GEMM's weight
matrix first -- while the other CTAs start multiplying as soon as the pieces under their
tile have landed; when the kernel ends the whole block is local for its remaining
operators (reference: the all-gather in mist/re_swap_manager/flat_param.py:1283-1370
followed by the QKV ``F.linear`` of mist/modules/fused_dense.py:75).

The full-size weight buffers ("slots", two for the usual one-block look-ahead ring) live in
a symmetric heap of the data-parallel group so peers can read each other's shard in place.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import native
from ..ops.native import call, ptr
from .symm import SymmetricHeap, ptr_table

native.register_signature(
    "mb_gemm_param_gather",
    [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_longlong,
     C.c_longlong, C.c_longlong, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p])

FLAG_INTS = 32


class ParamGatherContext:
    """Symmetric weight slots, flag blocks and chunk flags of one data-parallel group.
    ``n_gather = 0`` lets the kernel wrapper choose the number of gather CTAs (8 to 64, by the bytes to fetch and the size of the GEMM)."""

    def __init__(self, group, padded_numel: int, device=None, n_slots: int = 2, n_gather: int = 0,
                 chunk_bytes: int = 1 << 20, emulate_ranks: int = 0, max_sites: int = 64):
        self.group, self.n_gather, self.chunk_bytes = group, int(n_gather), int(chunk_bytes)
        self.padded = int(padded_numel)
        if emulate_ranks:
            # single-process stand-in (tests, profiling): the "peers" are further local buffers
            # and their flags are pre-set, so one launch never waits for another launch
            self.R, self.me, self.heap = int(emulate_ranks), 0, None
            self.device = device or torch.device("cuda", torch.cuda.current_device())
        else:
            self.R, self.me = dist.get_world_size(group), dist.get_rank(group)
            nbytes = n_slots * (self.padded * 2 + 4096) + max_sites * (FLAG_INTS * 4 + 256) + (1 << 20)
            self.heap = SymmetricHeap(nbytes, group, device)
            self.device = self.heap.device
        assert self.padded % (8 * self.R) == 0
        self.shard_numel = self.padded // self.R
        self.chunks_per_rank = -(-self.shard_numel * 2 // self.chunk_bytes)
        self.slots = []          # (local tensor, pointer table, [all local "peer" tensors] when emulating)
        for _ in range(n_slots):
            if self.heap is not None:
                t, off = self.heap.alloc(self.padded, torch.bfloat16)
                self.slots.append((t, ptr_table(self.heap.peer_ptrs(off)), None))
            else:
                ts = [torch.zeros(self.padded, dtype=torch.bfloat16, device=self.device) for _ in range(self.R)]
                self.slots.append((ts[0], ptr_table([x.data_ptr() for x in ts]), ts))
        self._sites: Dict[Tuple, Dict] = {}

    def slot_tensor(self, i: int) -> torch.Tensor:
        return self.slots[i][0]

    def stage_shard(self, i: int, shard: torch.Tensor):
        """Puts this rank's shard at its place in slot ``i`` (stream ordered before the gather)."""
        lo = self.me * self.shard_numel
        self.slots[i][0][lo:lo + shard.numel()].copy_(shard)

    def _site(self, key) -> Dict:
        if key not in self._sites:
            if self.heap is not None:
                flags, off = self.heap.alloc(FLAG_INTS, torch.int32)
                table = ptr_table(self.heap.peer_ptrs(off))
                flags.zero_()
                torch.cuda.synchronize()
                dist.barrier(group=self.group)       # every rank's flag block exists and is zero
            else:
                fl = [torch.zeros(FLAG_INTS, dtype=torch.int32, device=self.device) for _ in range(self.R)]
                fl[0][: 2 * self.R].fill_(1 << 30)   # emulated peers are always "ready" and "done"
                flags, table = fl[0], ptr_table([x.data_ptr() for x in fl])
                self._keep = getattr(self, "_keep", []) + fl
            chunk = torch.zeros(2 * self.R * self.chunks_per_rank, dtype=torch.int32, device=self.device)   # flags, counters
            self._sites[key] = {"flags": table, "flags_t": flags, "chunk": chunk, "epoch": 0}
        return self._sites[key]

    def gather_linear(self, i: int, x: torch.Tensor, b_off: int, N: int, K: int,
                      bias_off: Optional[int] = None) -> torch.Tensor:
        """``x[M, K] @ W^T (+ bias)`` with ``W = slot[b_off : b_off + N * K].view(N, K)`` while the
        remote shards of slot ``i`` are gathered.  The caller has staged this rank's shard."""
        assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] == K and x.is_contiguous()
        M = x.shape[0]
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        s = self._site((i, M, N, K, b_off))
        s["epoch"] += 1
        call("mb_gemm_param_gather", self.slots[i][1], ptr(x), ptr(out), s["flags"], ptr(s["chunk"]), M, N, K,
             out.stride(0), int(b_off), -1 if bias_off is None else int(bias_off), self.shard_numel, self.chunk_bytes,
             self.R, self.me, s["epoch"], self.n_gather, 0, native.stream())
        return out
