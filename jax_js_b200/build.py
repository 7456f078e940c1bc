"""Builds jax_js_b200/libjaxcuda.so in-tree with nvcc for sm_100a.

    python -m jax_js_b200.build [--force]

The host sources are plain C++17; sort.cu holds the only ahead-of-time device code (the
Kernel skeletons are CUDA C text compiled by NVRTC at prepare time).  The runtime is
linked statically against cudart and dynamically against NVRTC; the CUDA driver and NCCL
are resolved at run time, so the library loads on a machine without a GPU.
"""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libjaxcuda.so"
CUDA_HOME = Path("/usr/local/cuda")

SOURCES = ["runtime.cpp", "ir.cpp", "emit.cpp", "gemm_tc.cpp", "sort.cu", "scatter.cu", "linalg.cu", "fft.cu"]


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*")) + list((HERE.parent / "include").glob("*.h"))
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB
    cmd = [str(CUDA_HOME / "bin" / "nvcc"),
           "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "-shared",
           "-cudart", "static", "-o", str(LIB)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(CSRC / s) for s in SOURCES]
    cmd += ["-lnvrtc", "-ldl", "-Xlinker", f"-rpath={CUDA_HOME}/lib64"]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
