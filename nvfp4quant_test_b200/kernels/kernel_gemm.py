"""NVFP4 block-scaled GEMM: out = alpha * dq(a) @ dq(b).T in bf16.

Same signature and operand formats as `vllm._custom_ops.cutlass_scaled_fp4_mm`
(vllm 0.22.0, vllm/_custom_ops.py:741-752), the GEMM the reference feeds with its
quantizers' output (README.md:11,68): `a` uint8 [M, K/2], `b` uint8 [N, K/2], both
K-major packed E2M1; block scales in the 128x4-tiled float8_e4m3fn layout; `alpha` a
one-element float32 CUDA tensor (= global_scale_a * global_scale_b).
"""
from __future__ import annotations

import torch

from .. import _lib


def _scale_bytes(rows: int, k: int) -> int:
    return ((rows + 127) // 128 * 128) * ((k // 16 + 3) // 4 * 4)


def nvfp4_scaled_mm(a: torch.Tensor, b: torch.Tensor, block_scale_a: torch.Tensor, block_scale_b: torch.Tensor,
                    alpha: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    if a.ndim != 2 or b.ndim != 2:
        raise ValueError("a and b must be 2D [rows, K/2] uint8 tensors")
    if a.dtype != torch.uint8 or b.dtype != torch.uint8:
        raise ValueError("a and b must hold packed E2M1 codes as uint8")
    if out_dtype != torch.bfloat16:
        raise ValueError("only bfloat16 output is implemented")
    if not (a.is_cuda and b.device == a.device and block_scale_a.device == a.device
            and block_scale_b.device == a.device and alpha.device == a.device):
        raise ValueError("all operands must be CUDA tensors on one device")
    m, n, k = a.shape[0], b.shape[0], a.shape[1] * 2
    if b.shape[1] * 2 != k:
        raise ValueError(f"a and b disagree on K: {k} vs {b.shape[1] * 2}")
    if k % 64 != 0:
        raise ValueError(f"K must be a multiple of 64 (quantize with padded_n to pad it), got {k}")
    if alpha.dtype != torch.float32 or alpha.numel() < 1:
        raise ValueError("alpha must be a float32 tensor with one element")
    if not a.is_contiguous():
        a = a.contiguous()
    if not b.is_contiguous():
        b = b.contiguous()
    sfa = block_scale_a if block_scale_a.is_contiguous() else block_scale_a.contiguous()
    sfb = block_scale_b if block_scale_b.is_contiguous() else block_scale_b.contiguous()
    for name, sf, rows in (("block_scale_a", sfa, m), ("block_scale_b", sfb, n)):
        have = sf.numel() * sf.element_size()
        if have < _scale_bytes(rows, k):
            raise ValueError(f"{name} holds {have} bytes, the tiled layout for [{rows}, {k}] needs {_scale_bytes(rows, k)}")
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    elif out.shape != (m, n) or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError("out must be a contiguous bfloat16 [M, N] tensor")
    if m == 0 or n == 0:
        return out
    L = _lib.lib()
    stream = _lib.current_stream_ptr(a.device)
    args = (a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), alpha.data_ptr(), out.data_ptr(), m, n, k)
    with _lib.device_guard(a.device):
        st = L.nvfp4_gemm_launch(*args, None, 0, stream)
        if st == _ERR_WORKSPACE:
            # only when K ranges were switched on through the tuning hook: ask for the size, then launch again
            ws_bytes = L.nvfp4_gemm_workspace_bytes(m, n, k)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
            st = L.nvfp4_gemm_launch(*args, ws.data_ptr(), ws_bytes, stream)
    _lib.check(st, "nvfp4_gemm_launch")
    return out


_ERR_WORKSPACE = -6


class PreparedWeight:
    """A quantized weight [N, K] that will be multiplied many times (a model's linear layer).  Its tensor maps are
    encoded once (nvfp4_gemm_prepare); `nvfp4_scaled_mm_prepared` then costs less host time per call than
    `nvfp4_scaled_mm` and gives the same bits.  Keeps references to the two tensors, which must not be resized or
    moved while this object lives (their contents may be overwritten in place)."""

    def __init__(self, b: torch.Tensor, block_scale_b: torch.Tensor):
        import ctypes

        if b.ndim != 2 or b.dtype != torch.uint8 or not b.is_cuda or not b.is_contiguous():
            raise ValueError("b must be a contiguous CUDA uint8 tensor [N, K/2]")
        if block_scale_b.device != b.device or not block_scale_b.is_contiguous():
            raise ValueError("block_scale_b must be a contiguous tensor on b's device")
        self.n, self.k = b.shape[0], b.shape[1] * 2
        if self.k % 64 != 0:
            raise ValueError(f"K must be a multiple of 64, got {self.k}")
        have = block_scale_b.numel() * block_scale_b.element_size()
        if have < _scale_bytes(self.n, self.k):
            raise ValueError(f"block_scale_b holds {have} bytes, the tiled layout needs {_scale_bytes(self.n, self.k)}")
        self.b, self.block_scale_b, self.device = b, block_scale_b, b.device
        self._handle = ctypes.c_void_p()
        with _lib.device_guard(b.device):
            st = _lib.lib().nvfp4_gemm_prepare(b.data_ptr(), block_scale_b.data_ptr(), self.n, self.k, ctypes.byref(self._handle))
        _lib.check(st, "nvfp4_gemm_prepare")

    def close(self) -> None:
        if getattr(self, "_handle", None):
            _lib.lib().nvfp4_gemm_release(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


def nvfp4_scaled_mm_prepared(a: torch.Tensor, block_scale_a: torch.Tensor, alpha: torch.Tensor, weight: PreparedWeight,
                             out: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N] (bf16) = alpha * dq(a) @ dq(weight).T; same bits as nvfp4_scaled_mm(a, weight.b, ...)."""
    if a.ndim != 2 or a.dtype != torch.uint8 or a.device != weight.device:
        raise ValueError("a must be a uint8 [M, K/2] tensor on the weight's device")
    if a.shape[1] * 2 != weight.k:
        raise ValueError(f"a and the weight disagree on K: {a.shape[1] * 2} vs {weight.k}")
    if alpha.dtype != torch.float32 or alpha.device != a.device:
        raise ValueError("alpha must be a float32 tensor on a's device")
    if not a.is_contiguous():
        a = a.contiguous()
    sfa = block_scale_a if block_scale_a.is_contiguous() else block_scale_a.contiguous()
    m = a.shape[0]
    if sfa.numel() * sfa.element_size() < _scale_bytes(m, weight.k):
        raise ValueError("block_scale_a is smaller than the tiled layout of a needs")
    if out is None:
        out = torch.empty((m, weight.n), dtype=torch.bfloat16, device=a.device)
    elif out.shape != (m, weight.n) or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError("out must be a contiguous bfloat16 [M, N] tensor")
    if m == 0:
        return out
    if not weight._handle:
        raise ValueError("the prepared weight has been closed")
    L = _lib.lib()
    stream = _lib.current_stream_ptr(a.device)
    with _lib.device_guard(a.device):
        st = L.nvfp4_gemm_launch_prepared(weight._handle, a.data_ptr(), sfa.data_ptr(), alpha.data_ptr(), out.data_ptr(),
                                          m, None, 0, stream)
        if st == _ERR_WORKSPACE:
            ws_bytes = L.nvfp4_gemm_workspace_bytes(m, weight.n, weight.k)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
            st = L.nvfp4_gemm_launch_prepared(weight._handle, a.data_ptr(), sfa.data_ptr(), alpha.data_ptr(),
                                              out.data_ptr(), m, ws.data_ptr(), ws_bytes, stream)
    _lib.check(st, "nvfp4_gemm_launch_prepared")
    return out


def nvfp4_scaled_mm_grouped(a: torch.Tensor, block_scale_a: torch.Tensor, alpha_a: torch.Tensor | None,
                            weights: list[PreparedWeight], alpha_w: list[torch.Tensor],
                            outs: list[torch.Tensor] | None = None) -> list[torch.Tensor]:
    """[alpha_w[i] * alpha_a * dq(a) @ dq(weights[i]).T for i] as bf16 [M, N_i] tensors: one activation against several
    prepared weights of equal K (a layer's q / k / v, or gate / up).  `alpha_a` (the activation's global scale, or None)
    and each `alpha_w[i]` (the weight's global scale) are one-element float32 CUDA tensors; their product is taken inside
    the kernel.  At decode-sized M the whole group is one launch (nvfp4_gemm_launch_grouped)."""
    import ctypes

    n = len(weights)
    if n == 0:
        return []
    if len(alpha_w) != n or (outs is not None and len(outs) != n):
        raise ValueError("weights, alpha_w and outs must have the same length")
    if n > 64:
        raise ValueError("at most 64 weights per call")
    dev, k = weights[0].device, weights[0].k
    if a.ndim != 2 or a.dtype != torch.uint8 or a.device != dev:
        raise ValueError("a must be a uint8 [M, K/2] tensor on the weights' device")
    if a.shape[1] * 2 != k:
        raise ValueError(f"a and the weights disagree on K: {a.shape[1] * 2} vs {k}")
    if not a.is_contiguous():
        a = a.contiguous()
    sfa = block_scale_a if block_scale_a.is_contiguous() else block_scale_a.contiguous()
    m = a.shape[0]
    if sfa.numel() * sfa.element_size() < _scale_bytes(m, k):
        raise ValueError("block_scale_a is smaller than the tiled layout of a needs")
    if alpha_a is not None and (alpha_a.dtype != torch.float32 or alpha_a.device != dev or alpha_a.numel() < 1):
        raise ValueError("alpha_a must be a float32 tensor on a's device")
    if outs is None:
        outs = [torch.empty((m, w.n), dtype=torch.bfloat16, device=dev) for w in weights]
    for w, al, o in zip(weights, alpha_w, outs):
        if w.device != dev or w.k != k:
            raise ValueError("all weights of a group share the device and K")
        if not w._handle:
            raise ValueError("a prepared weight of the group has been closed")
        if al.dtype != torch.float32 or al.device != dev or al.numel() < 1:
            raise ValueError("alpha_w entries must be float32 tensors on a's device")
        if o.shape != (m, w.n) or o.dtype != torch.bfloat16 or not o.is_contiguous() or o.device != dev:
            raise ValueError("outs[i] must be a contiguous bfloat16 [M, N_i] tensor on a's device")
    if m == 0:
        return outs
    handles = (ctypes.c_void_p * n)(*[w._handle.value for w in weights])
    alphas = (ctypes.c_void_p * n)(*[al.data_ptr() for al in alpha_w])
    out_ptrs = (ctypes.c_void_p * n)(*[o.data_ptr() for o in outs])
    with _lib.device_guard(dev):
        st = _lib.lib().nvfp4_gemm_launch_grouped(handles, n, a.data_ptr(), sfa.data_ptr(),
                                                  None if alpha_a is None else alpha_a.data_ptr(), alphas, out_ptrs, m,
                                                  _lib.current_stream_ptr(dev))
    _lib.check(st, "nvfp4_gemm_launch_grouped")
    return outs


def cutlass_scaled_fp4_mm(a, b, block_scale_a, block_scale_b, alpha, out_dtype):
    """Drop-in name of the vllm op."""
    return nvfp4_scaled_mm(a, b, block_scale_a, block_scale_b, alpha, out_dtype)


def gemm_last_status(device=None) -> int:
    """Synchronise and return the device status word of the last GEMM (0 = ok)."""
    import ctypes

    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    word = ctypes.c_uint32(0)
    with torch.cuda.device(dev):
        st = _lib.lib().nvfp4_gemm_last_status(_lib.current_stream_ptr(dev), ctypes.byref(word))
    _lib.check(st, "nvfp4_gemm_last_status")
    return word.value
