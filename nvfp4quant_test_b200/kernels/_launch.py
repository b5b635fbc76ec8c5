"""Argument checking and the one launch path shared by every quantizer entry point."""
from __future__ import annotations

import torch

from .. import _lib

BLOCK_SIZE = 16


def _check_common(input: torch.Tensor, input_scale: torch.Tensor) -> None:
    if not isinstance(input, torch.Tensor) or input.ndim != 2:
        raise ValueError(f"input must be 2D [num_row, dim], got {tuple(getattr(input, 'shape', ()))}")
    if input.shape[-1] % BLOCK_SIZE != 0:
        raise ValueError(f"input.shape[-1] must be divisible by {BLOCK_SIZE}")
    if not input.is_cuda:
        raise ValueError("input must be a CUDA tensor: these kernels have no CPU path")
    if input_scale.device != input.device:
        raise ValueError(f"input and input_scale must be on the same device: {input.device} vs {input_scale.device}")
    if input_scale.dtype != torch.float32 or input_scale.numel() < 1:
        raise ValueError("input_scale must be a float32 tensor holding 1 / global_scale")


def check_importance(input: torch.Tensor, importance: torch.Tensor) -> None:
    # same conditions and wording as the reference's _check_inputs (kernels/kernel_ScaleSweep.py:419-433)
    if input.ndim != 2:
        raise ValueError(f"input must be 2D [num_row, dim], got {tuple(input.shape)}")
    if input.shape[-1] % BLOCK_SIZE != 0:
        raise ValueError(f"input.shape[-1] must be divisible by {BLOCK_SIZE}")
    if importance.shape != (1, input.shape[-1]):
        raise ValueError(
            f"importance must have shape [1, dim], got {tuple(importance.shape)}, "
            f"expected {(1, input.shape[-1])}")
    if input.device != importance.device:
        raise ValueError(
            f"input and importance must be on the same device: {input.device} vs {importance.device}")


def quant_out(variant: int, input: torch.Tensor, importance: torch.Tensor | None, input_scale: torch.Tensor,
              is_sf_swizzled_layout: bool, output: torch.Tensor, output_scale: torch.Tensor,
              lower: int, upper: int, impl: int = 0) -> None:
    """Validate, then launch on the current stream of input.device.  Writes output / output_scale in place."""
    _check_common(input, input_scale)
    if not input.is_contiguous():
        input = input.contiguous()
    m, n = input.shape
    if output.dtype != torch.uint8 or output.ndim != 2 or output.shape[0] != m or not output.is_contiguous():
        raise ValueError(f"output must be a contiguous uint8 tensor [num_row, padded_n/2], got {tuple(output.shape)} {output.dtype}")
    physical_n = output.shape[-1] * 2
    if physical_n % BLOCK_SIZE != 0 or physical_n < n:
        raise ValueError(f"output holds {physical_n} columns; need a multiple of {BLOCK_SIZE} that is >= {n}")
    if output.device != input.device or output_scale.device != input.device:
        raise ValueError("output and output_scale must be on the input's device")
    if not output_scale.is_contiguous():
        raise ValueError("output_scale must be contiguous")
    blocks = physical_n // BLOCK_SIZE
    if is_sf_swizzled_layout:
        need = ((m + 127) // 128 * 128) * ((blocks + 3) // 4 * 4)
    else:
        need = m * blocks
    have = output_scale.numel() * output_scale.element_size()
    if have < need:
        raise ValueError(f"output_scale holds {have} bytes, the scale layout needs {need}")
    imp_ptr = None
    if variant == _lib.VARIANT_WEIGHTED:
        if importance.dtype != torch.float32:
            importance = importance.float()
        if not importance.is_contiguous():
            importance = importance.contiguous()
        imp_ptr = importance.data_ptr()
    if m == 0 or physical_n == 0:
        return
    args = (impl, variant, input.data_ptr(), _lib.dtype_code(input.dtype), imp_ptr, input_scale.data_ptr(),
            output.data_ptr(), output_scale.data_ptr(), m, n, physical_n, lower, upper,
            1 if is_sf_swizzled_layout else 0, _lib.current_stream_ptr(input.device))
    if input.device.index == torch.cuda.current_device():
        st = _lib.lib().nvfp4_quant_launch_impl(*args)
    else:  # launch with the tensor's device current
        with torch.cuda.device(input.device):
            st = _lib.lib().nvfp4_quant_launch_impl(*args)
    if st < 0 and st in (-2, -5):
        raise ValueError(_lib.status_string(st))
    _lib.check(st, "nvfp4_quant_launch")
