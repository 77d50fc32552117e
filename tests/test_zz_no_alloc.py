"""The allocation-free column-sum entry point, called through its exported C symbol.

Some hosts of the kernel library may not allocate device memory at all (a plugin inside an
application whose memory manager owns the GPU, a service with a frozen memory layout).  For
them ``mb_colsum_static`` keeps its scratch inside the library.  This test checks that it
gives the same result as the regular ``mb_colsum`` (which takes a caller-allocated scratch
buffer) on two consecutive calls -- the second call finds the first call's leftovers in the
shared scratch -- and that an oversized problem is refused.  The file name sorts last so a
run that stops at the first failure has already executed every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from mist_b200.ops import native
    lib = C.CDLL(str(native.kernels_path()))
    lib.mb_colsum_static.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.mb_colsum_static.restype = C.c_int
    lib.mb_colsum_static_capacity.restype = C.c_long
    lib.mb_colsum.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.mb_colsum.restype = C.c_int
    return lib


def test_static_scratch_colsum_matches_regular_entry_point_twice():
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(0)
    cap = lib.mb_colsum_static_capacity()
    assert cap == 1 << 20
    for call, (rows, cols, fp32) in enumerate([(4096, 2560, False), (1000, 10240, True)]):
        x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
        dt = torch.float32 if fp32 else torch.bfloat16
        out_new = torch.zeros(cols, device="cuda", dtype=dt)
        out_ref = torch.zeros(cols, device="cuda", dtype=dt)
        scratch = torch.empty(((rows + 255) // 256) * cols, device="cuda", dtype=torch.float32)
        torch.cuda.synchronize()
        assert lib.mb_colsum_static(x.data_ptr(), out_new.data_ptr(), rows, cols, int(fp32), 0, stream) == 0
        assert lib.mb_colsum(x.data_ptr(), out_ref.data_ptr(), scratch.data_ptr(), rows, cols, int(fp32), 0, stream) == 0
        torch.cuda.synchronize()
        oracle = x.float().sum(0)
        rel = ((out_new.float() - out_ref.float()).norm() / (out_ref.float().norm() + 1e-12)).item()
        assert rel < 1e-6, (call, rel)                      # same kernels, same order of additions
        rel_o = ((out_new.float() - oracle).norm() / (oracle.norm() + 1e-12)).item()
        assert rel_o < (1e-5 if fp32 else 2e-2), (call, rel_o)


def test_static_scratch_colsum_refuses_oversized_problem():
    lib = _lib()
    rows, cols = 256 * 200, 8192                             # 200 * 8192 floats > 1 Mi
    x = torch.empty(8, device="cuda", dtype=torch.bfloat16)  # never read: the call must be refused first
    out = torch.empty(cols, device="cuda", dtype=torch.float32)
    assert lib.mb_colsum_static(x.data_ptr(), out.data_ptr(), rows, cols, 1, 0, None) == -22
