"""Importance-weighted ScaleSweep NVFP4 quantization.

Same call signatures, checks and results as kernels/kernel_ScaleSweep.py:419-513 of
efsotr/nvfp4quant_test: per-input-column fp32 weights `importance[1, dim]`, base code
rounded DOWN on the E4M3 grid, default window -8..+7, weighted squared errors summed
as a fixed pairwise tree.
"""
from __future__ import annotations

import torch

from .. import _lib
from ._launch import BLOCK_SIZE, check_importance, quant_out  # noqa: F401
from .kernel_vllm import create_fp4_output_tensors

LOWER_BOUND = -8
UPPER_BOUND = 7


def scalesweep_weighted_mse_nvfp4_quant_out(
    input: torch.Tensor,
    importance: torch.Tensor,
    input_scale: torch.Tensor,
    is_sf_swizzled_layout: bool = True,
    *,
    output: torch.Tensor,
    output_scale: torch.Tensor,
    lower_bound: int = LOWER_BOUND,
    upper_bound: int = UPPER_BOUND,
) -> None:
    check_importance(input, importance)
    quant_out(_lib.VARIANT_WEIGHTED, input, importance, input_scale, is_sf_swizzled_layout, output, output_scale,
              lower_bound, upper_bound)


def scalesweep_weighted_mse_nvfp4_quant_impl(
    input: torch.Tensor,
    importance: torch.Tensor,
    input_scale: torch.Tensor,
    is_sf_swizzled_layout: bool = True,
    padded_n: int | None = None,
    *,
    lower_bound: int = LOWER_BOUND,
    upper_bound: int = UPPER_BOUND,
) -> tuple[torch.Tensor, torch.Tensor]:
    check_importance(input, importance)
    m, n = input.shape
    output, output_scale = create_fp4_output_tensors(m, n, input.device, is_sf_swizzled_layout, padded_n=padded_n)
    scalesweep_weighted_mse_nvfp4_quant_out(
        input, importance, input_scale, is_sf_swizzled_layout,
        output=output, output_scale=output_scale, lower_bound=lower_bound, upper_bound=upper_bound)
    return output, output_scale.view(torch.float8_e4m3fn)
