import pathlib
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]
for p in (ROOT, ROOT / "tests" / "golden"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O

    O.build()
    O.lib()
    return O


@pytest.fixture(scope="session")
def golden():
    """Reference outputs captured on a B200 (tests/golden/make_reference_golden.py)."""
    import json

    import numpy as np

    g = ROOT / "tests" / "golden"
    if not (g / "reference_golden.npz").exists():
        pytest.skip("reference_golden.npz not present")
    return json.loads((g / "reference_golden.json").read_text()), np.load(g / "reference_golden.npz")


def build_probe_lib(force: bool = False) -> pathlib.Path:
    """Compile tests/csrc/probe_kernels.cu (two diagnostic kernels used only by the tests) for sm_100a."""
    import os
    import shutil
    import subprocess

    src = ROOT / "tests" / "csrc" / "probe_kernels.cu"
    out = ROOT / "tests" / "_build" / "libnvfp4_test_probes.so"
    if not force and out.exists() and out.stat().st_mtime >= src.stat().st_mtime:
        return out
    out.parent.mkdir(parents=True, exist_ok=True)
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
           f"-I{ROOT / 'include'}", f"-I{ROOT / 'nvfp4quant_test_b200' / 'csrc'}", "-shared", "-o", str(out), str(src)]
    res = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    return out


@pytest.fixture(scope="session")
def probe_lib():
    """Test-only library with the div.full / rcp.approx table probes (not part of the product library)."""
    import ctypes

    L = ctypes.CDLL(str(build_probe_lib()))
    vp = ctypes.c_void_p
    L.nvfp4_probe_div_full_table.restype = ctypes.c_int
    L.nvfp4_probe_div_full_table.argtypes = [vp, vp]
    L.nvfp4_probe_amax_out_scale_table.restype = ctypes.c_int
    L.nvfp4_probe_amax_out_scale_table.argtypes = [vp, vp, vp]
    return L


@pytest.fixture(scope="session")
def cuda_lib():
    """The product library on a CUDA device; fails (does not skip) when it is missing."""
    import torch

    assert torch.cuda.is_available(), "gpu-marked tests need a CUDA device"
    from nvfp4quant_test_b200 import _lib

    return _lib.lib()
