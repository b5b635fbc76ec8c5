"""amax ("vllm") NVFP4 baseline quantizer.

Counterpart of `vllm._custom_ops.scaled_fp4_quant` (vllm 0.22.0,
vllm/_custom_ops.py:1600-1665), the baseline the reference times at bench.py:118-125:
per block scale = E4M3(input_global_scale * amax/6), codes = RNE_E2M1(x / (scale / input_global_scale)).
"""
from __future__ import annotations

import torch

from .. import _lib
from ._launch import BLOCK_SIZE, quant_out  # noqa: F401
from .kernel_vllm import create_fp4_output_tensors


def amax_nvfp4_quant_out(input, input_scale, is_sf_swizzled_layout: bool = True, *, output, output_scale) -> None:
    quant_out(_lib.VARIANT_AMAX, input, None, input_scale, is_sf_swizzled_layout, output, output_scale, 0, 0)


def amax_nvfp4_quant_impl(input: torch.Tensor, input_scale: torch.Tensor, is_sf_swizzled_layout: bool = True,
                          padded_n: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    if input.ndim != 2:
        raise ValueError(f"input must be 2D [num_row, dim], got {tuple(input.shape)}")
    m, n = input.shape
    if padded_n is not None and (padded_n < n or padded_n % BLOCK_SIZE):
        raise ValueError(f"padded_n must be a multiple of {BLOCK_SIZE} that is >= n, got padded_n={padded_n}, n={n}")
    output, output_scale = create_fp4_output_tensors(m, n, input.device, is_sf_swizzled_layout, padded_n=padded_n)
    amax_nvfp4_quant_out(input, input_scale, is_sf_swizzled_layout, output=output, output_scale=output_scale)
    return output, output_scale.view(torch.float8_e4m3fn)


def scaled_fp4_quant(input: torch.Tensor, input_global_scale: torch.Tensor, is_sf_swizzled_layout: bool = True,
                     backend: str = "none", padded_n: int | None = None):
    """Same signature as the vllm op; leading dimensions are flattened like it does."""
    if input.ndim < 1:
        raise ValueError(f"input.ndim needs to be >= 1, but got {input.ndim}.")
    x2 = input.reshape(1 if input.ndim == 1 else -1, input.shape[-1])
    return amax_nvfp4_quant_impl(x2, input_global_scale, is_sf_swizzled_layout, padded_n)
