"""Compile libnvfp4_b200.so (sm_100a only) in-tree with nvcc.

  python -m nvfp4quant_test_b200.build [--force]
"""
from __future__ import annotations

import os
import pathlib
import shutil
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB = PKG / "libnvfp4_b200.so"

SOURCES = ["quant.cu", "global_scale.cu", "global_scale_static.cu", "importance.cu", "gemm.cu", "status.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false",  # every fused multiply-add in the kernels is written explicitly
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not pathlib.Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.inc")) + list(INCLUDE.glob("*.h"))
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Build the shared library if it is missing or older than its sources."""
    if not force and not _stale():
        return LIB
    srcs = [str(CSRC / s) for s in SOURCES if (CSRC / s).exists()]
    extra = os.environ.get("NVFP4_EXTRA_NVCC_FLAGS", "").split()   # e.g. -DNVFP4_QUANT_MIN_BLOCKS=6 for experiments
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, f"-I{INCLUDE}", f"-I{CSRC}", "-shared", "-o", str(LIB), *srcs]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    env = dict(os.environ)
    # nvcc picks its host compiler itself; a CC/CXX meant for another toolchain would only mislead it
    env.pop("CC", None)
    env.pop("CXX", None)
    res = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
