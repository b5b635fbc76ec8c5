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


def _check_outputs(input: torch.Tensor, is_sf_swizzled_layout: bool, output: torch.Tensor,
                   output_scale: torch.Tensor) -> tuple[int, int, int]:
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
    return m, n, physical_n


def _importance_ptr(variant: int, importance: torch.Tensor | None):
    """(pointer or None, tensor kept alive until the launch is enqueued)."""
    if variant != _lib.VARIANT_WEIGHTED:
        return None, None
    if importance.dtype != torch.float32:
        importance = importance.float()
    if not importance.is_contiguous():
        importance = importance.contiguous()
    return importance.data_ptr(), importance


def _raise(st: int, what: str) -> None:
    if st < 0 and st in (-2, -5):
        raise ValueError(_lib.status_string(st))
    _lib.check(st, what)


def quant_out(variant: int, input: torch.Tensor, importance: torch.Tensor | None, input_scale: torch.Tensor,
              is_sf_swizzled_layout: bool, output: torch.Tensor, output_scale: torch.Tensor,
              lower: int, upper: int, impl: int = 0) -> None:
    """Validate, then launch on the current stream of input.device.  Writes output / output_scale in place."""
    _check_common(input, input_scale)
    if not input.is_contiguous():
        input = input.contiguous()
    m, n, physical_n = _check_outputs(input, is_sf_swizzled_layout, output, output_scale)
    imp_ptr, _keep = _importance_ptr(variant, importance)
    if m == 0 or physical_n == 0:
        return
    args = (impl, variant, input.data_ptr(), _lib.dtype_code(input.dtype), imp_ptr, input_scale.data_ptr(),
            output.data_ptr(), output_scale.data_ptr(), m, n, physical_n, lower, upper,
            1 if is_sf_swizzled_layout else 0, _lib.current_stream_ptr(input.device))
    with _lib.device_guard(input.device):   # launch with the tensor's device current
        st = _lib.lib().nvfp4_quant_launch_impl(*args)
    _raise(st, "nvfp4_quant_launch")


_fused_scratch = _lib.StreamScratch(4)


def quant_fused_out(variant: int, input: torch.Tensor, importance: torch.Tensor | None, fp8_max: float,
                    is_sf_swizzled_layout: bool, output: torch.Tensor, output_scale: torch.Tensor,
                    lower: int, upper: int) -> torch.Tensor | None:
    """Global scale and sweep in ONE launch (the tensor's blocks stay in registers across a grid-wide wait).
    Returns a float32 [2] CUDA tensor (global_scale, 1 / global_scale), or None when the tensor does not fit the
    resident grid of the device, in which case nothing was launched and the caller uses the two-launch path."""
    if not isinstance(input, torch.Tensor) or input.ndim != 2:
        raise ValueError(f"input must be 2D [num_row, dim], got {tuple(getattr(input, 'shape', ()))}")
    if input.shape[-1] % BLOCK_SIZE != 0:
        raise ValueError(f"input.shape[-1] must be divisible by {BLOCK_SIZE}")
    if not input.is_cuda:
        raise ValueError("input must be a CUDA tensor: these kernels have no CPU path")
    if not input.is_contiguous():
        input = input.contiguous()
    m, n, physical_n = _check_outputs(input, is_sf_swizzled_layout, output, output_scale)
    if m == 0 or n == 0:
        raise ValueError("the global scale of an empty tensor is undefined")
    imp_ptr, _keep = _importance_ptr(variant, importance)
    stream = _lib.current_stream_ptr(input.device)
    scratch = _fused_scratch.get(input.device, stream)
    gs = torch.empty(2, dtype=torch.float32, device=input.device)
    with _lib.device_guard(input.device):
        st = _lib.lib().nvfp4_quant_fused_launch(
            variant, input.data_ptr(), _lib.dtype_code(input.dtype), imp_ptr, float(fp8_max), gs.data_ptr(),
            scratch.data_ptr(), output.data_ptr(), output_scale.data_ptr(), m, n, physical_n,
            lower, upper, 1 if is_sf_swizzled_layout else 0, stream)
    if st == _lib.ERR_TOO_LARGE:
        return None
    _raise(st, "nvfp4_quant_fused_launch")
    return gs
