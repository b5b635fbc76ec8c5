"""Unweighted ScaleSweep NVFP4 quantization (ScaleSweep_MSE and ScaleSweep_MSE_round).

Same call signatures and results as kernels/kernel_ScaleSweep_MSE.py:380-437 of
efsotr/nvfp4quant_test.  Per 16-element block the raw E4M3 scale codes
base-3 .. base+7 around base = RNE_E4M3(amax/6) are tried in ascending order and the
one with the least fp32 squared error wins (lowest code on ties).

`ScaleSweep_MSE_round` is listed in the reference's result tables (README.md:50,61,74)
but its source is not published; there it matches ScaleSweep_MSE in every printed
digit.  It is exported here with the only definition the published material gives
(round-to-nearest base, window -3..+7), i.e. as an alias.
"""
from __future__ import annotations

import torch

from .. import _lib
from ._launch import BLOCK_SIZE, quant_out  # noqa: F401
from .kernel_vllm import create_fp4_output_tensors

LOWER_BOUND = -3
UPPER_BOUND = 7


def scalesweep_mse_nvfp4_quant_out(
    input: torch.Tensor,
    input_scale: torch.Tensor,
    is_sf_swizzled_layout: bool = True,
    *,
    output: torch.Tensor,
    output_scale: torch.Tensor,
) -> None:
    """Quantize into caller-owned `output` (uint8 [m, P/2]) and `output_scale`
    (any 1- or 4-byte dtype, viewed as bytes).  P = output.shape[-1] * 2 may exceed
    input.shape[-1]; the extra columns quantize as zeros."""
    quant_out(_lib.VARIANT_MSE, input, None, input_scale, is_sf_swizzled_layout, output, output_scale,
              LOWER_BOUND, UPPER_BOUND)


def scalesweep_mse_nvfp4_quant_impl(
    input: torch.Tensor,
    input_scale: torch.Tensor,
    is_sf_swizzled_layout: bool = True,
    padded_n: int | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Returns (codes uint8 [m, P/2], scales float8_e4m3fn) with P = padded_n or n."""
    if input.ndim != 2:
        raise ValueError(f"input must be 2D [num_row, dim], got {tuple(input.shape)}")
    m, n = input.shape
    output, output_scale = create_fp4_output_tensors(m, n, input.device, is_sf_swizzled_layout, padded_n=padded_n)
    scalesweep_mse_nvfp4_quant_out(input, input_scale, is_sf_swizzled_layout, output=output, output_scale=output_scale)
    return output, output_scale.view(torch.float8_e4m3fn)


scalesweep_mse_round_nvfp4_quant_out = scalesweep_mse_nvfp4_quant_out
scalesweep_mse_round_nvfp4_quant_impl = scalesweep_mse_nvfp4_quant_impl
