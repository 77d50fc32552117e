"""Symmetric memory: one device arena per rank that every rank of a group maps.

Each rank allocates an arena with the CUDA runtime, exports it as a CUDA IPC handle,
and opens its peers' handles, so kernels can dereference ``peer_ptr(rank, offset)``
directly over NVLink.  Allocation inside the arena is a bump pointer that every rank
advances identically, so one offset names the same object on every rank.

``torch.distributed`` is used only to exchange the 64-byte handles (plumbing); no
collective library touches the data path built on top of this.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import native

_DT = {torch.bfloat16: ("<i2", 2), torch.float16: ("<f2", 2), torch.float32: ("<f4", 4),
       torch.int32: ("<i4", 4), torch.uint8: ("|u1", 1), torch.int64: ("<i8", 8)}

native.register_signature("mb_symm_alloc", [C.c_size_t, C.POINTER(C.c_void_p)])
native.register_signature("mb_symm_free", [C.c_void_p])
native.register_signature("mb_symm_memset", [C.c_void_p, C.c_int, C.c_size_t, C.c_void_p])
native.register_signature("mb_ipc_handle_size", [])
native.register_signature("mb_ipc_get_handle", [C.c_void_p, C.c_void_p])
native.register_signature("mb_ipc_open_handle", [C.c_void_p, C.POINTER(C.c_void_p)])
native.register_signature("mb_ipc_close_handle", [C.c_void_p])
native.register_signature("mb_set_peer_wait_ms", [C.c_int])
native.register_signature("mb_set_fused_grad_ctas", [C.c_int], None)
native.register_signature("mb_wait_on_flags", [C.c_void_p, C.c_int, C.c_int, C.c_void_p])
native.register_signature(
    "mb_fused_grad_reduce_adam",
    [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
     C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float,
     C.c_int, C.c_float, C.c_int, C.c_int, C.c_void_p])
native.register_signature(
    "mb_p2p_all_gather", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p])
native.register_signature(
    "mb_p2p_reduce_scatter", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int,
                              C.c_int, C.c_int, C.c_void_p])


class _RawCuda:
    """Adapter exposing a raw device pointer through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def tensor_from_ptr(ptr: int, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
    nbytes = numel * _DT[dtype][1]
    raw = torch.as_tensor(_RawCuda(ptr, nbytes), device=device)
    return raw.view(dtype)


def ptr_table(ptrs: List[int]):
    """ctypes array of device pointers, passed by address to the launch wrappers."""
    arr = (C.c_void_p * len(ptrs))(*[C.c_void_p(p) for p in ptrs])
    return arr


def group_on_one_node(group) -> bool:
    """True when every rank of ``group`` runs on this host (peer memory over NVLink / CUDA IPC
    needs that; groups that span nodes stay on the NCCL paths)."""
    import os
    import socket
    if group is None or not dist.is_initialized():
        return True
    # a launcher that reports as many local ranks as ranks in the job runs on one node: no
    # collective is needed to know it (the same answer on every rank)
    lw, w = os.environ.get("LOCAL_WORLD_SIZE"), os.environ.get("WORLD_SIZE")
    if lw is not None and w is not None and lw == w:
        return True
    names: List[Optional[str]] = [None] * dist.get_world_size(group)
    dist.all_gather_object(names, socket.gethostname(), group=group)
    return len(set(names)) == 1


class SymmetricHeap:
    ALIGN = 1024
    #: bytes of all live arenas of this process: they come from the driver, not from torch's caching allocator,
    #: so ``torch.cuda.max_memory_allocated`` does not see them (memory reports add this figure)
    live_bytes = 0

    def __init__(self, nbytes: int, group, device=None):
        lib = native.kernels()
        assert lib is not None, "symmetric memory needs a GPU"
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        base = C.c_void_p()
        rc = lib.mb_symm_alloc(self.nbytes, C.byref(base))
        if rc != 0:
            raise RuntimeError(f"could not allocate a {self.nbytes >> 20} MiB symmetric arena")
        self.base = base.value
        SymmetricHeap.live_bytes += self.nbytes
        lib.mb_symm_memset(self.base, 0, self.nbytes, None)
        torch.cuda.synchronize()
        hsize = lib.mb_ipc_handle_size()
        handle = (C.c_ubyte * hsize)()
        if lib.mb_ipc_get_handle(self.base, handle) != 0:
            raise RuntimeError("cudaIpcGetMemHandle failed")
        mine = bytes(handle)
        gathered: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(gathered, mine, group=group)
        self.peer_base: List[int] = []
        for r, h in enumerate(gathered):
            if r == self.rank:
                self.peer_base.append(self.base)
                continue
            buf = (C.c_ubyte * hsize).from_buffer_copy(h)
            out = C.c_void_p()
            rc = lib.mb_ipc_open_handle(buf, C.byref(out))
            if rc != 0:
                raise RuntimeError(f"cudaIpcOpenMemHandle failed for rank {r} (code {rc})")
            self.peer_base.append(out.value)
        self.offset = 0
        dist.barrier(group=group)

    def alloc(self, numel: int, dtype: torch.dtype) -> Tuple[torch.Tensor, int]:
        """Returns (local tensor view, offset).  Every rank must call with the same sizes in
        the same order."""
        nbytes = numel * _DT[dtype][1]
        off = self.offset
        self.offset = (off + nbytes + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        if self.offset > self.nbytes:
            raise MemoryError("symmetric arena exhausted")
        return tensor_from_ptr(self.base + off, numel, dtype, self.device), off

    def peer_ptrs(self, offset: int) -> List[int]:
        return [b + offset for b in self.peer_base]

    def close(self):
        lib = native.kernels()
        for r, b in enumerate(self.peer_base):
            if r != self.rank:
                lib.mb_ipc_close_handle(b)
        lib.mb_symm_free(self.base)
        SymmetricHeap.live_bytes -= self.nbytes
