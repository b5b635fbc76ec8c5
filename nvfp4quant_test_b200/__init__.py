"""B200-native (sm_100a) NVFP4 ScaleSweep quantization and block-scaled FP4 GEMM.

Host-side mirror of the `kernels/` entry points of efsotr/nvfp4quant_test; the
arithmetic runs in hand-written CUDA behind the C ABI of include/nvfp4_b200.h.
"""
from . import _lib  # noqa: F401

__all__ = ["kernels", "helper", "sharding"]
__version__ = "0.1.0"
