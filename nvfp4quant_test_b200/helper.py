"""Bench / evaluation helpers with the names of the reference's helper.py.

`get_nvfp4_global_scale` (helper.py:96-100 of efsotr/nvfp4quant_test) runs as a CUDA
reduction kernel here; the dequantizer and error metrics (helper.py:103-147) are
plain torch and work on any device.
"""
from __future__ import annotations

import torch

from . import _lib

FP4_E2M1_MAX = 6.0
FP8_E4M3_MAX_NVFP4 = 448.0
FP8_E4M3_MAX_4OVER6 = 256.0

_scratch = _lib.StreamScratch(2)


def get_nvfp4_global_scale(x: torch.Tensor, FP8_MAX: float = FP8_E4M3_MAX_NVFP4, out: torch.Tensor | None = None):
    """(global_scale, global_scale_inv) as 0-dim float32 CUDA tensors; amax(|x|)/(6*FP8_MAX) and its reciprocal.
    `out` (optional): a contiguous float32 [2] CUDA tensor to write them into instead of a fresh one."""
    if not x.is_cuda:
        raise ValueError("x must be a CUDA tensor")
    if out is not None and (out.dtype != torch.float32 or out.device != x.device or out.shape != (2,)
                            or not out.is_contiguous()):
        raise ValueError("out must be a contiguous float32 [2] tensor on x's device")
    if not x.is_contiguous():
        x = x.contiguous()
    if x.data_ptr() & 15:
        # the kernel reads 16-byte vectors; a view that starts in the middle of one (x.view(-1)[1:], a row slice of a
        # matrix with an odd width) is copied to aligned storage, so that any tensor the reference's
        # x.abs().max() accepts works here too
        x = x.clone()
    stream = _lib.current_stream_ptr(x.device)
    scratch = _scratch.get(x.device, stream)
    if out is None:
        out = torch.empty(2, dtype=torch.float32, device=x.device)
    with _lib.device_guard(x.device):
        st = _lib.lib().nvfp4_global_scale_launch(x.data_ptr(), _lib.dtype_code(x.dtype), x.numel(), float(FP8_MAX),
                                                  out.data_ptr(), scratch.data_ptr(), stream)
    _lib.check(st, "nvfp4_global_scale_launch")
    return out[0], out[1]


def channel_square_norm(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 [1, dim]: squared L2 norm of every input channel (column) of the 2-D batch x - the importance
    vector for the operand x is multiplied with (README.md:11 of the reference).  `out` (optional): a contiguous
    float32 [1, dim] CUDA tensor to write into."""
    if x.ndim != 2 or not x.is_cuda:
        raise ValueError("x must be a 2D CUDA tensor")
    if out is not None and (out.dtype != torch.float32 or out.device != x.device or out.shape != (1, x.shape[1])
                            or not out.is_contiguous()):
        raise ValueError("out must be a contiguous float32 [1, dim] tensor on x's device")
    if x.shape[1] % 4:
        raise ValueError("x.shape[1] must be divisible by 4")
    # a column slice of a wider batch (x_full[:, c0:c1]) is read in place through its row pitch
    in_place = x.shape[0] <= 1 or (x.stride(1) == 1 and x.stride(0) >= x.shape[1] and x.stride(0) % 4 == 0)
    if not in_place or x.data_ptr() & 15:
        x = x.contiguous()
        if x.data_ptr() & 15:
            x = x.clone()
    ld = x.stride(0) if x.shape[0] > 1 else x.shape[1]
    if out is None:
        out = torch.empty((1, x.shape[1]), dtype=torch.float32, device=x.device)
    with _lib.device_guard(x.device):
        st = _lib.lib().nvfp4_channel_sqnorm_launch_strided(x.data_ptr(), _lib.dtype_code(x.dtype), x.shape[0], x.shape[1],
                                                            ld, out.data_ptr(), _lib.current_stream_ptr(x.device))
    _lib.check(st, "nvfp4_channel_sqnorm_launch_strided")
    return out


def error_stats(ref, pred):
    diff = pred.float() - ref.float()
    return torch.mean(diff * diff).item(), torch.max(torch.abs(diff)).item()


def weighted_error_stats(weight, reconstructed, imp):
    err = reconstructed.float() - weight.float()
    return torch.mean(err * err * imp.float()).item(), torch.max(torch.abs(err)).item()


_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def unpack_fp4_e2m1(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [m, k/2] -> float32 [m, k]; low nibble first."""
    assert packed.dtype == torch.uint8
    lut = torch.tensor(_E2M1 + tuple(-v for v in _E2M1), dtype=torch.float32, device=packed.device)
    both = torch.stack((packed & 0x0F, packed >> 4), dim=-1).long()
    return lut[both].reshape(packed.shape[0], packed.shape[1] * 2)


def dequantize_base(q, scale_fp8, global_scale):
    """q uint8 [m, k/2], scale_fp8 float8_e4m3fn [m, k/16] (row-major, i.e. already unswizzled)."""
    scales = scale_fp8.to(torch.float32).repeat_interleave(16, dim=1)
    return unpack_fp4_e2m1(q) * scales * global_scale.float()


def dequantize(kind, *args, **kwargs):
    if kind == "base":
        return dequantize_base(*args, **kwargs)
    raise ValueError(f"unknown dequant kind: {kind}")
