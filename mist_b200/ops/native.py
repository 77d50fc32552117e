"""ctypes bindings of the in-tree native libraries.

The kernels library exports plain C symbols taking device pointers and a stream, so
no framework-specific extension build is needed: tensors are passed as
``tensor.data_ptr()`` and the current stream as ``torch.cuda.current_stream().cuda_stream``.

On a machine with a GPU a missing library is an error (no silent eager fallback);
on a CPU-only machine ``kernels()`` returns ``None`` and callers use their reference
PyTorch implementation, which is also the oracle of the numerics tests.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

_NATIVE = Path(__file__).resolve().parent.parent / "_native"
_KERNELS = None
_RUNTIME = None

# number of kernels launched through this module (reported by bench.py)
launch_count = 0

_p = C.c_void_p
_i = C.c_int
_l = C.c_long
_f = C.c_float
_z = C.c_size_t
_u64 = C.c_uint64

_SIGNATURES = {
    "mb_status_read_and_clear": ([], _i),
    "mb_status_device_ptr": ([], _p),
    "mb_gemm_bf16": ([_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p, _p, _f, _i, _i, _p], _i),
    "mb_gemm_pair_bf16": ([_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p, _p, _f, _i, _p], _i),
    "mb_decode_attn": ([_p, _p, _p, _p, _i, _i, _i, _i, _i, _l, _l, _l, _l, _l, _l, _f, _p], _i),
    "mb_norm_bwd_scratch_rows": ([_i, _i], _i),
    "mb_norm_fwd": ([_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _f, _i, _p], _i),
    "mb_norm_bwd": ([_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p], _i),
    "mb_norm_pipe_parts": ([_i, _i, _i, _i, _i, _i], _i),
    "mb_norm_fwd_pipe": ([_p] * 12 + [_i, _i, _f, _i, _i, _f, _u64, _p], _i),
    "mb_norm_bwd_pipe": ([_p] * 15 + [_i, _i, _i, _i, _f, _u64, _p], _i),
    "mb_norm_bwd_finalize": ([_p, _p, _p, _p, _i, _i, _p], _i),
    "mb_gelu_fwd": ([_p, _p, _p, _z, _i, _p], _i),
    "mb_gelu_bwd": ([_p, _p, _p, _p, _z, _i, _p], _i),
    "mb_swiglu_fwd": ([_p, _p, _z, _i, _p], _i),
    "mb_swiglu_bwd": ([_p, _p, _p, _z, _i, _p], _i),
    "mb_bias_dropout_add": ([_p, _p, _p, _p, _z, _i, _f, _u64, _p], _i),
    "mb_dropout_bwd": ([_p, _p, _z, _f, _u64, _p], _i),
    "mb_rope": ([_p, _p, _p, _z, _i, _i, _i, _i, _i, _i, _i, _p], _i),
    "mb_embedding_fwd": ([_p, _p, _p, _p, _z, _i, _i, _i, _i, _p], _i),
    "mb_embedding_bwd": ([_p, _p, _p, _p, _i, _i, _i, _i, _i, _p], _i),
    "mb_colsum": ([_p, _p, _p, _i, _i, _i, _i, _p], _i),
    "mb_cast_f32_to_bf16": ([_p, _p, _z, _f, _p], _i),
    "mb_axpy_bf16_to_f32": ([_p, _p, _z, _f, _i, _p], _i),
    "mb_add_bf16": ([_p, _p, _z, _p], _i),
    "mb_xent_stats": ([_p, _p, _p, _i, _i, _i, _i, _p], _i),
    "mb_xent_loss": ([_p, _p, _p, _p, _i, _i, _p], _i),
    "mb_xent_bwd": ([_p, _p, _p, _p, _f, _i, _i, _i, _i, _i, _i, _p], _i),
    "mb_causal_softmax_fwd": ([_p, _p, _z, _i, _i, _f, _i, _p], _i),
    "mb_causal_softmax_bwd": ([_p, _p, _p, _z, _i, _f, _p], _i),
    "mb_adam_step": ([_p, _p, _p, _p, _i, _p, _z, _f, _f, _f, _f, _f, _i, _f, _i, _p], _i),
    "mb_attn_bwd": ([_p] * 11 + [_i] * 5 + [_l] * 18 + [_f, _i, _p, _p, _p], _i),
    "mb_attn_fwd": ([_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i] + [_l] * 12 + [_f, _i, _i, _p, _p, _p], _i),
}

_OPTIONAL = {}


def register_signature(name, argtypes, restype=_i):
    """Lets later-loaded modules declare further exported symbols."""
    _OPTIONAL[name] = (argtypes, restype)
    if _KERNELS is not None and hasattr(_KERNELS, name):
        fn = getattr(_KERNELS, name)
        fn.argtypes, fn.restype = argtypes, restype


def kernels_path() -> Path:
    return _NATIVE / "libmist_b200_kernels.so"


def runtime_path() -> Path:
    return _NATIVE / "libmist_b200_runtime.so"


def kernels():
    """The kernels library, or None on a machine without a GPU."""
    global _KERNELS
    if _KERNELS is not None:
        return _KERNELS
    if not torch.cuda.is_available():
        return None
    path = kernels_path()
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing on a machine with a GPU; run `python -m mist_b200.ops.build` "
            "(the framework does not fall back to eager PyTorch on CUDA tensors)")
    lib = C.CDLL(str(path))
    for name, (argtypes, restype) in list(_SIGNATURES.items()) + list(_OPTIONAL.items()):
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = argtypes, restype
    _KERNELS = lib
    return lib


def runtime():
    """The host-side C++ runtime (CPU code; available with or without a GPU)."""
    global _RUNTIME
    if _RUNTIME is not None:
        return _RUNTIME
    path = runtime_path()
    if not path.exists():
        from . import build
        build.build_runtime()
    _RUNTIME = C.CDLL(str(path))
    return _RUNTIME


def use_native(*tensors) -> bool:
    """True when the op should run on the CUDA kernels (any tensor lives on a GPU)."""
    for t in tensors:
        if t is not None and t.is_cuda:
            if kernels() is None:
                raise RuntimeError("CUDA tensor but no kernels library")
            return True
    return False


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def call(name: str, *args):
    """Launches an exported kernel wrapper and raises on a non-zero return code."""
    global launch_count
    fn = getattr(kernels(), name)
    rc = fn(*args)
    launch_count += 1
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")
    return rc


_STATUS_NAMES = {1: "TMA stage wait timed out", 2: "free-stage wait timed out",
                 3: "accumulator wait timed out", 4: "peer flag wait timed out", 5: "bad argument"}


def read_and_clear_status() -> int:
    """The device status word set by bounded waits that gave up (0 = none); clears it."""
    lib = kernels()
    return 0 if lib is None else int(lib.mb_status_read_and_clear())


def status_message(code: int) -> str:
    return f"a kernel reported status {code}: {_STATUS_NAMES.get(code, 'unknown')}"


def check_status():
    """Reads (and clears) the device status word and raises if a bounded wait gave up."""
    code = read_and_clear_status()
    if code != 0:
        raise RuntimeError(status_message(code))
    return 0
