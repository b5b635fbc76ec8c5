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


@pytest.fixture(scope="session")
def cuda_lib():
    """The product library on a CUDA device; fails (does not skip) when it is missing."""
    import torch

    assert torch.cuda.is_available(), "gpu-marked tests need a CUDA device"
    from nvfp4quant_test_b200 import _lib

    return _lib.lib()
