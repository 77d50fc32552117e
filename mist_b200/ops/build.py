"""Builds the native libraries in-tree with nvcc / g++ (no framework headers needed).

Two shared objects are produced under ``mist_b200/_native``:

* ``libmist_b200_kernels.so`` -- every ``.cu`` file under ``mist_b200/csrc`` compiled
  for sm_100a only.
* ``libmist_b200_runtime.so`` -- the host-side C++ runtime under ``mist_b200/runtime``
  (solver, Pareto sampler, schedule simulator, copy-engine planner).

Run ``python -m mist_b200.ops.build`` to (re)build; both libraries are rebuilt only
when a source is newer than the library.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "csrc"
RUNTIME = PKG / "runtime"
OUT = PKG / "_native"
KERNELS_SO = OUT / "libmist_b200_kernels.so"
RUNTIME_SO = OUT / "libmist_b200_runtime.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")
    return cand


def _newer(srcs, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in srcs)


def _run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("build failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), res.stdout, res.stderr))
    return res.stdout + res.stderr


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    OUT.mkdir(exist_ok=True)
    cus = sorted(CSRC.glob("*.cu"))
    hdrs = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    if not force and not _newer(cus + hdrs, KERNELS_SO):
        return KERNELS_SO
    objdir = OUT / "obj"
    objdir.mkdir(exist_ok=True)
    nvcc = _nvcc()

    def compile_one(cu: Path) -> Path:
        obj = objdir / (cu.stem + ".o")
        if force or _newer([cu] + hdrs, obj):
            extra = ["-Xptxas", "-v"] if verbose else []
            out = _run([nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(cu), "-o", str(obj)])
            if verbose:
                print(out)
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, len(cus))) as ex:
        objs = list(ex.map(compile_one, cus))
    _run([nvcc, "-shared", "-o", str(KERNELS_SO), *map(str, objs), "-Xcompiler", "-fPIC"])
    return KERNELS_SO


def build_runtime(force: bool = False) -> Path:
    OUT.mkdir(exist_ok=True)
    srcs = sorted(RUNTIME.glob("*.cpp"))
    hdrs = sorted(RUNTIME.glob("*.h")) + sorted(RUNTIME.glob("*.hpp"))
    if not srcs:
        return RUNTIME_SO
    if not force and not _newer(srcs + hdrs, RUNTIME_SO):
        return RUNTIME_SO
    gxx = shutil.which("g++") or "g++"
    _run([gxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-pthread",
          "-I", str(RUNTIME), "-o", str(RUNTIME_SO), *map(str, srcs)])
    return RUNTIME_SO


def build_all(force: bool = False, verbose: bool = False):
    return build_kernels(force, verbose), build_runtime(force)


if __name__ == "__main__":
    k, r = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", k, r)
