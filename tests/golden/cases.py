"""Seeded input cases shared by the golden-fixture generator and the parity tests.

Inputs come from torch's CPU generator, so the same bits are produced on any host; each
fixture also stores a sha256 of its input bytes and the tests check it before use.
"""
from __future__ import annotations

import hashlib

import numpy as np
import torch


def _gauss(shape, seed, dtype=torch.bfloat16, scale=1.0):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * scale).to(dtype)


def _laplace(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    u = torch.rand(shape, generator=g, dtype=torch.float64) - 0.5
    return (-torch.sign(u) * torch.log1p(-2 * u.abs())).to(torch.float32).to(dtype)


def _importance(kind, dim, seed=123):
    if kind == "ones":
        return torch.ones((1, dim), dtype=torch.float32)
    if kind == "ramp":
        return torch.linspace(0.25, 2.0, dim, dtype=torch.float32).view(1, dim)
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return 0.25 + 1.75 * torch.rand((1, dim), dtype=torch.float32, generator=g)


def _edge_rows(dtype):
    """[16, 64]: blocks of zeros, negative zeros, tiny, huge, inf, NaN, ties and saturating values."""
    x = torch.zeros((16, 64), dtype=torch.float32)
    g = torch.Generator(device="cpu")
    g.manual_seed(7)
    x[0, 16:32] = -0.0
    x[1, 0:16] = 1e-30
    x[1, 16:32] = torch.randn(16, generator=g) * 1e-6
    x[2, 0:16] = torch.randn(16, generator=g) * 3e4
    x[2, 16:32] = 6.0
    x[3, 0:16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    x[4, 0:16] = torch.randn(16, generator=g)
    x[4, 3] = float("inf")
    x[5, 0:16] = torch.randn(16, generator=g)
    x[5, 5] = float("nan")
    x[6, 0:16] = float("nan")
    x[7, 0:16] = torch.randn(16, generator=g) * 50.0   # with gs_inv large: base scale saturates at 448
    x[8] = torch.randn(64, generator=g) * 1e-3
    x[9, 0:16] = torch.tensor([1.0] + [0.0] * 15)
    x[10, 0:16] = -torch.arange(16, dtype=torch.float32)
    x[11:] = torch.randn((5, 64), generator=g)
    if dtype != torch.float32:
        x[1, 0:16] = 1e-30 if dtype == torch.bfloat16 else 6e-8
    return x.to(dtype)


# name -> dict(x, fp8_max or gs_inv, variant, importance, swizzled, padded_n, lower, upper)
def build_cases():
    cases = {}

    def add(name, x, variant, fp8_max=256.0, gs_inv=None, imp=None, swizzled=True, padded_n=None,
            lower=None, upper=None):
        cases[name] = dict(x=x, variant=variant, fp8_max=fp8_max, gs_inv=gs_inv, importance=imp,
                           swizzled=swizzled, padded_n=padded_n, lower=lower, upper=upper)

    add("mse_128x8192_seed0_fp8max448", _gauss((128, 8192), 0), "mse", fp8_max=448.0)
    add("mse_128x8192_seed0_fp8max256", _gauss((128, 8192), 0), "mse", fp8_max=256.0)
    add("mse_130x208_pad256", _gauss((130, 208), 1), "mse", padded_n=256)
    add("mse_7x48_linear", _gauss((7, 48), 2), "mse", swizzled=False)
    add("mse_257x1024_linear", _gauss((257, 1024), 3), "mse", swizzled=False)
    add("mse_33x64_f16", _gauss((33, 64), 4, torch.float16), "mse")
    add("mse_16x128_f32", _gauss((16, 128), 5, torch.float32), "mse")
    add("mse_1x8192", _gauss((1, 8192), 6), "mse")
    add("mse_laplace_300x512", _laplace((300, 512), 8), "mse")
    add("mse_edge_bf16", _edge_rows(torch.bfloat16), "mse", gs_inv=1.0)
    add("mse_edge_f32", _edge_rows(torch.float32), "mse", gs_inv=1.0)
    add("mse_edge_bf16_gs100", _edge_rows(torch.bfloat16), "mse", gs_inv=100.0)
    add("weighted_128x1024_ones", _gauss((128, 1024), 10), "weighted", imp=_importance("ones", 1024))
    add("weighted_128x1024_ramp", _gauss((128, 1024), 10), "weighted", imp=_importance("ramp", 1024))
    add("weighted_200x512_random", _laplace((200, 512), 11), "weighted", imp=_importance("random", 512))
    add("weighted_64x256_window_m2_p3", _gauss((64, 256), 12), "weighted", imp=_importance("random", 256),
        lower=-2, upper=3)
    add("weighted_130x208_pad256", _gauss((130, 208), 13), "weighted", imp=_importance("ramp", 208), padded_n=256)
    add("weighted_edge_bf16", _edge_rows(torch.bfloat16), "weighted", gs_inv=1.0, imp=_importance("random", 64))
    add("weighted_laplace_sqnorm_256x2048", _laplace((256, 2048), 14), "weighted",
        imp=(_laplace((512, 2048), 15).float() ** 2).sum(0, keepdim=True))
    add("amax_128x1024", _gauss((128, 1024), 20), "amax", fp8_max=448.0)
    add("amax_130x208", _gauss((130, 208), 21), "amax", fp8_max=448.0)
    add("amax_33x64_f16", _gauss((33, 64), 22, torch.float16), "amax", fp8_max=448.0)
    add("amax_laplace_300x512", _laplace((300, 512), 23), "amax", fp8_max=448.0)
    return cases


def gemm_cases():
    """name -> (M, N, K, seed).  cutlass_scaled_fp4_mm needs N % 32 == 0, so the fixture shapes respect that;
    the tests against the fp64 oracle also cover other N."""
    return {
        "gemm_128x256x256": (128, 256, 256, 30),
        "gemm_130x288x512": (130, 288, 512, 31),
        "gemm_1x512x1024": (1, 512, 1024, 32),
        "gemm_16x128x64": (16, 128, 64, 33),
        "gemm_300x544x320": (300, 544, 320, 34),
    }


def gemm_operands(M, N, K, seed):
    return _laplace((M, K), seed), _laplace((N, K), seed + 1000)


def tensor_bytes(t: torch.Tensor) -> bytes:
    t = t.contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    return t.numpy().tobytes()


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(tensor_bytes(t)).hexdigest()


def global_scale_cpu(x: torch.Tensor, fp8_max: float):
    """amax/(6*fp8_max) the way torch evaluates helper.py:96-100 on a CUDA tensor:
    division by a host scalar multiplies by its fp32 reciprocal; reciprocal() is an IEEE division."""
    amax = np.float32(x.float().abs().max().item())
    inv_den = np.float32(1.0) / np.float32(6.0 * fp8_max)
    gs = np.float32(amax * inv_den)
    with np.errstate(divide="ignore"):
        gs_inv = np.float32(1.0) / gs
    return float(gs), float(gs_inv)
