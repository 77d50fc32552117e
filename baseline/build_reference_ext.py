"""Builds the two native extensions the reference's Dockerfile builds (csrc/fused_dense_lib and
csrc/layer_norm, Dockerfile:45-48) from the unmodified sources under baseline/_ref/csrc, for sm_100
only, into baseline/_ref/ext.  The reference's own setup.py files pin arch lists that stop at sm_90, so
the sources are handed to torch's extension builder directly with the same defines.

    python baseline/build_reference_ext.py [fused_dense_lib] [dropout_layer_norm] [--sizes 2560,4096]

``--sizes`` limits the layer-norm build to the instantiation files of those hidden sizes (each file
registers its own launchers, so the others are simply not available at run time).  The default is the
benchmark model's 2560 alone: all 14 sizes give a 300 MB library that every GPU call would carry.
"""
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "_ref" / "csrc"
OUT = HERE / "_ref" / "ext"


def main():
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 8))
    import torch
    from torch.utils.cpp_extension import load

    OUT.mkdir(exist_ok=True)
    gen = []
    if (Path(torch.__path__[0]) / "include" / "ATen" / "CUDAGeneratorImpl.h").exists():
        gen = ["-DOLD_GENERATOR_PATH"]
    nvcc = ["-O3", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
            "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
            "-U__CUDA_NO_BFLOAT162_OPERATORS__", "-U__CUDA_NO_BFLOAT162_CONVERSIONS__",
            "--expt-relaxed-constexpr", "--expt-extended-lambda", "--use_fast_math"] + gen
    argv = sys.argv[1:]
    sizes = ["2560"]
    if "--sizes" in argv:
        i = argv.index("--sizes")
        sizes = argv[i + 1].split(",")
        del argv[i:i + 2]
    which = argv or ["fused_dense_lib", "dropout_layer_norm"]
    if "fused_dense_lib" in which:
        d = CSRC / "fused_dense_lib"
        load(name="fused_dense_lib", sources=[str(d / "fused_dense.cpp"), str(d / "fused_dense_cuda.cu")],
             extra_cflags=["-O3"], extra_cuda_cflags=["-O3"], build_directory=_bd("fused_dense_lib"),
             is_python_module=False, verbose=True)
    if "dropout_layer_norm" in which:
        d = CSRC / "layer_norm"
        srcs = [str(d / "ln_api.cpp")] + sorted(str(p) for p in d.glob("ln_*.cu")
                                               if sizes == ["all"] or p.stem.rsplit("_", 1)[1] in sizes)
        load(name="dropout_layer_norm", sources=srcs, extra_cflags=["-O3"] + gen, extra_cuda_cflags=nvcc,
             extra_include_paths=[str(d)], build_directory=_bd("dropout_layer_norm"),
             is_python_module=False, verbose=True)
    for so in OUT.glob("*/*.so"):
        target = OUT / so.name
        if not target.exists() or target.stat().st_mtime < so.stat().st_mtime:
            target.write_bytes(so.read_bytes())
    print("built:", sorted(p.name for p in OUT.glob("*.so")))


def _bd(name):
    p = OUT / name
    p.mkdir(exist_ok=True)
    return str(p)


if __name__ == "__main__":
    main()
