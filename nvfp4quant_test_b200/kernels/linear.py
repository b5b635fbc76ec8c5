"""Preallocated building blocks for a decode loop that is launched eagerly (no CUDA graph).

`nvfp4_scaled_mm_grouped` and the quantizer entry points allocate their outputs, check their arguments and build
their argument arrays on every call; that is tens of microseconds of Python per call, several times what the GPU
needs for a decode-sized launch.  The two classes here do that work once: buffers are allocated and arguments are
checked at construction, a call is one C ABI call.  Outputs are reused from call to call (copy what must be kept), and
an instance serves one stream at a time.  Bits equal the allocating entry points'.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib
from .. import helper as _helper
from . import kernel_ScaleSweep_MSE as _mse
from .kernel_gemm import PreparedWeight, _scale_bytes
from .kernel_vllm import create_fp4_output_tensors


class ActivationQuantizer:
    """global scale -> ScaleSweep_MSE quantization of an activation [tokens, k] with one host call
    (nvfp4_quant_chain_launch: two kernels, the second a programmatic dependent launch of the first)."""

    def __init__(self, tokens: int, k: int, device, fp8_max: float = _helper.FP8_E4M3_MAX_4OVER6,
                 dtype: torch.dtype = torch.bfloat16):
        if tokens < 1 or k < 16 or k % 16:
            raise ValueError("tokens >= 1 and k a positive multiple of 16 are required")
        self.tokens, self.k, self.dtype, self.fp8_max = tokens, k, dtype, float(fp8_max)
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())   # tensors report an explicit index
        self._dtype_code = _lib.dtype_code(dtype)
        self.codes, scales = create_fp4_output_tensors(tokens, k, self.device, True)
        self.scales = scales.view(torch.float8_e4m3fn)
        self.global_scale = torch.zeros(2, dtype=torch.float32, device=self.device)   # (scale, 1 / scale)
        self._scratch = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._args = (self.global_scale.data_ptr(), self._scratch.data_ptr(), self.codes.data_ptr(), scales.data_ptr(),
                      tokens, k, k, _mse.LOWER_BOUND, _mse.UPPER_BOUND, 1)
        self._scales_storage = scales

    def __call__(self, x: torch.Tensor):
        """Returns (codes, scales, global_scale[0:1]); the three tensors are this object's buffers."""
        if x.shape != (self.tokens, self.k) or x.dtype != self.dtype or x.device != self.device or not x.is_contiguous():
            raise ValueError(f"x must be a contiguous {self.dtype} [{self.tokens}, {self.k}] tensor on {self.device}")
        if x.data_ptr() & 15:
            raise ValueError("x must be 16-byte aligned")
        with _lib.device_guard(self.device):
            st = _lib.lib().nvfp4_quant_chain_launch(_lib.VARIANT_MSE, x.data_ptr(), self._dtype_code, None, self.fp8_max,
                                                     *self._args, _lib.current_stream_ptr(self.device))
        _lib.check(st, "nvfp4_quant_chain_launch")
        return self.codes, self.scales, self.global_scale[0:1]


class LinearGroup:
    """y_i = (alpha_a * weight_scale_i) * dq(a) @ dq(weight_i).T for prepared weights that read the same activation
    (q / k / v, gate / up), `tokens` rows at a time, into preallocated bf16 outputs: one nvfp4_gemm_launch_grouped call."""

    def __init__(self, weights: list[PreparedWeight], weight_scales: list[torch.Tensor], tokens: int):
        if not weights or len(weights) != len(weight_scales) or len(weights) > 64:
            raise ValueError("between 1 and 64 weights, one scale tensor per weight")
        self.weights, self.weight_scales, self.tokens = list(weights), list(weight_scales), tokens
        self.device, self.k = weights[0].device, weights[0].k
        for w, s in zip(weights, weight_scales):
            if w.device != self.device or w.k != self.k or not w._handle:
                raise ValueError("the weights of a group share the device and K, and must be open")
            if s.dtype != torch.float32 or s.device != self.device or s.numel() < 1:
                raise ValueError("weight scales must be float32 tensors on the weights' device")
        n = len(weights)
        self.outs = [torch.empty((tokens, w.n), dtype=torch.bfloat16, device=self.device) for w in weights]
        self._handles = (ctypes.c_void_p * n)(*[w._handle.value for w in weights])
        self._alphas = (ctypes.c_void_p * n)(*[s.data_ptr() for s in weight_scales])
        self._outs = (ctypes.c_void_p * n)(*[o.data_ptr() for o in self.outs])
        self._n = n
        self._min_scale_bytes = _scale_bytes(tokens, self.k)

    def __call__(self, codes: torch.Tensor, scales: torch.Tensor, alpha_a: torch.Tensor | None):
        """codes / scales: the quantized activation [tokens, K/2] and its tiled scales; alpha_a: its global scale (one
        float32 on the device) or None.  Returns this object's output tensors."""
        if (codes.shape != (self.tokens, self.k // 2) or codes.dtype != torch.uint8 or codes.device != self.device
                or not codes.is_contiguous()):
            raise ValueError(f"codes must be a contiguous uint8 [{self.tokens}, {self.k // 2}] tensor on {self.device}")
        if scales.numel() * scales.element_size() < self._min_scale_bytes or not scales.is_contiguous():
            raise ValueError("scales are smaller than the tiled layout of the activation needs")
        with _lib.device_guard(self.device):
            st = _lib.lib().nvfp4_gemm_launch_grouped(self._handles, self._n, codes.data_ptr(), scales.data_ptr(),
                                                      None if alpha_a is None else alpha_a.data_ptr(), self._alphas,
                                                      self._outs, self.tokens, _lib.current_stream_ptr(self.device))
        _lib.check(st, "nvfp4_gemm_launch_grouped")
        return self.outs
