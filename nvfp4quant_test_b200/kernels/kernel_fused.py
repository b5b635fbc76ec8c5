"""Global scale + ScaleSweep quantization as one call.

The reference computes the tensor-wide scale first (`get_nvfp4_global_scale`, helper.py:96-100 of
efsotr/nvfp4quant_test) and hands its reciprocal to the quantizer (bench.py:57-67): two passes over the tensor
and two launches.  For tensors that fit the GPU's resident grid (about 3 M elements on a B200: activations of up
to a few hundred tokens) both happen in one launch here, with the tensor read once; larger tensors take the two
launches.  Bytes and scales are identical either way.
"""
from __future__ import annotations

import torch

from .. import _lib
from .. import helper as _helper
from ._launch import check_importance, quant_fused_out, quant_out
from .kernel_vllm import create_fp4_output_tensors
from . import kernel_ScaleSweep as _weighted
from . import kernel_ScaleSweep_MSE as _mse


def scalesweep_nvfp4_quant_with_global_scale(
    input: torch.Tensor,
    fp8_max: float = _helper.FP8_E4M3_MAX_4OVER6,
    importance: torch.Tensor | None = None,
    is_sf_swizzled_layout: bool = True,
    padded_n: int | None = None,
    *,
    lower_bound: int | None = None,
    upper_bound: int | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(codes, scales, global_scale, global_scale_inv).  Without `importance` this is ScaleSweep_MSE (window
    -3..+7), with it the importance-weighted ScaleSweep (window -8..+7 unless given); the two scale tensors are
    0-dim float32 views, as `get_nvfp4_global_scale` returns them."""
    if input.ndim != 2:
        raise ValueError(f"input must be 2D [num_row, dim], got {tuple(input.shape)}")
    if importance is None:
        variant, mod = _lib.VARIANT_MSE, _mse
    else:
        check_importance(input, importance)
        variant, mod = _lib.VARIANT_WEIGHTED, _weighted
    lower = mod.LOWER_BOUND if lower_bound is None else lower_bound
    upper = mod.UPPER_BOUND if upper_bound is None else upper_bound
    m, n = input.shape
    output, output_scale = create_fp4_output_tensors(m, n, input.device, is_sf_swizzled_layout, padded_n=padded_n)
    gs = quant_fused_out(variant, input, importance, fp8_max, is_sf_swizzled_layout, output, output_scale, lower, upper)
    if gs is None:
        g, g_inv = _helper.get_nvfp4_global_scale(input, fp8_max)
        quant_out(variant, input, importance, g_inv, is_sf_swizzled_layout, output, output_scale, lower, upper)
    else:
        g, g_inv = gs[0], gs[1]
    return output, output_scale.view(torch.float8_e4m3fn), g, g_inv
