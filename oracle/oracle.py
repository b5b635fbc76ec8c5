"""ctypes front end of the CPU oracle (oracle/nvfp4_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports it.

Arrays are numpy: bf16 / fp16 inputs are passed as uint16 bit patterns
(`torch_tensor.view(torch.int16).numpy().view(np.uint16)`), fp32 as float32.
"""
from __future__ import annotations

import ctypes
import pathlib
import subprocess

import numpy as np

_HERE = pathlib.Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libnvfp4_oracle.so"

VARIANT_MSE, VARIANT_WEIGHTED, VARIANT_AMAX = 0, 1, 2
DT_BF16, DT_F16, DT_F32 = 0, 1, 2

_lib = None


def build(force: bool = False) -> pathlib.Path:
    """Compile the oracle with the Makefile beside it (gcc only)."""
    if force or not _LIB_PATH.exists() or any(
        (_HERE / f).stat().st_mtime > _LIB_PATH.stat().st_mtime
        for f in ("nvfp4_oracle.c", "div_full_table.h", "oracle.py")
    ):
        subprocess.run(["make", "-C", str(_HERE), "-B"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        L = ctypes.CDLL(str(_LIB_PATH))
        i64, f32, vp, ci = ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_int
        L.nvfp4_oracle_quant.restype = ci
        L.nvfp4_oracle_quant.argtypes = [ci, vp, ci, vp, f32, vp, vp, i64, i64, i64, ci, ci, ci, vp, f32, ci]
        L.nvfp4_oracle_dequant.restype = ci
        L.nvfp4_oracle_dequant.argtypes = [vp, vp, f32, vp, i64, i64, ci]
        L.nvfp4_oracle_gemm.restype = ci
        L.nvfp4_oracle_gemm.argtypes = [vp, vp, vp, vp, f32, vp, i64, i64, i64]
        L.nvfp4_oracle_best_raw_exhaustive.restype = ci
        L.nvfp4_oracle_best_raw_exhaustive.argtypes = [vp]
        L.nvfp4_oracle_sweep_block_f32.restype = ci
        L.nvfp4_oracle_sweep_block_f32.argtypes = [ci, vp, vp, ci, ci]
        L.nvfp4_oracle_e4m3_to_f32.restype = f32
        L.nvfp4_oracle_e4m3_to_f32.argtypes = [ctypes.c_uint8]
        L.nvfp4_oracle_f32_to_e4m3.restype = ctypes.c_uint8
        L.nvfp4_oracle_f32_to_e4m3.argtypes = [f32]
        L.nvfp4_oracle_swizzled_offset.restype = i64
        L.nvfp4_oracle_swizzled_offset.argtypes = [i64, i64, i64]
        L.nvfp4_oracle_offset_histogram.restype = None
        L.nvfp4_oracle_offset_histogram.argtypes = [vp, i64, vp, vp]
        L.nvfp4_oracle_prune_study.restype = i64
        L.nvfp4_oracle_prune_study.argtypes = [vp, i64, f32, ci, ci, vp, vp, vp, vp]
        L.nvfp4_oracle_div_full_table_is_measured.restype = ci
        L.nvfp4_oracle_div_full_bits.restype = ctypes.c_uint32
        L.nvfp4_oracle_div_full_bits.argtypes = [ci]
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def round_up(x: int, y: int) -> int:
    return (x + y - 1) // y * y


def _dtype_code(x: np.ndarray, x_dtype: str | None) -> int:
    if x.dtype == np.float32:
        return DT_F32
    if x.dtype == np.float16:
        return DT_F16
    if x.dtype == np.uint16:
        return DT_F16 if x_dtype == "f16" else DT_BF16
    raise TypeError(f"unsupported input dtype {x.dtype}")


def quant(variant: int, x: np.ndarray, gs_inv: float, importance: np.ndarray | None = None, *,
          swizzled: bool = True, padded_n: int | None = None, lower: int = -3, upper: int = 7,
          x_dtype: str | None = None, fill: int = 0, amax_table: np.ndarray | None = None,
          amax_sixth: float = 0.0, nthreads: int = 0):
    """Returns (codes uint8 [m, P/2], scales uint8) with P = padded_n or n.

    scales is [round_up(m,128), round_up(P/16,4)] (swizzled byte order, pre-filled
    with `fill`) or [m, P/16] (linear).
    """
    x = np.ascontiguousarray(x)
    m, n = x.shape
    P = n if padded_n is None else padded_n
    codes = np.full((m, P // 2), fill, dtype=np.uint8)
    if swizzled:
        scales = np.full((round_up(m, 128), round_up(P // 16, 4)), fill, dtype=np.uint8)
    else:
        scales = np.full((m, P // 16), fill, dtype=np.uint8)
    imp = None
    if importance is not None:
        imp = np.ascontiguousarray(importance, dtype=np.float32).reshape(-1)
        assert imp.size == n
    tab = None
    if amax_table is not None:
        tab = np.ascontiguousarray(amax_table, dtype=np.float32)
        assert tab.size >= 127
    rc = lib().nvfp4_oracle_quant(variant, _ptr(x), _dtype_code(x, x_dtype), _ptr(imp), float(gs_inv),
                                  _ptr(codes), _ptr(scales), m, n, P, lower, upper, int(swizzled),
                                  _ptr(tab), float(amax_sixth), nthreads)
    if rc != 0:
        raise ValueError(f"nvfp4_oracle_quant rejected its arguments (rc={rc})")
    return codes, scales


def dequant(codes: np.ndarray, scales: np.ndarray, gs: float, *, swizzled: bool = True) -> np.ndarray:
    codes = np.ascontiguousarray(codes)
    scales = np.ascontiguousarray(scales)
    m, half = codes.shape
    out = np.empty((m, half * 2), dtype=np.float32)
    rc = lib().nvfp4_oracle_dequant(_ptr(codes), _ptr(scales), float(gs), _ptr(out), m, half * 2, int(swizzled))
    assert rc == 0
    return out


def gemm(a, b, sfa, sfb, alpha: float) -> np.ndarray:
    """fp64-accumulated alpha * dq(a) @ dq(b).T, returned as float32 [M, N]."""
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    sfa, sfb = np.ascontiguousarray(sfa), np.ascontiguousarray(sfb)
    M, N, K = a.shape[0], b.shape[0], a.shape[1] * 2
    assert b.shape[1] * 2 == K
    out = np.empty((M, N), dtype=np.float32)
    rc = lib().nvfp4_oracle_gemm(_ptr(a), _ptr(b), _ptr(sfa), _ptr(sfb), float(alpha), _ptr(out), M, N, K)
    assert rc == 0
    return out


def best_raw_exhaustive(v16: np.ndarray) -> int:
    v = np.ascontiguousarray(v16, dtype=np.float32)
    assert v.size == 16
    return lib().nvfp4_oracle_best_raw_exhaustive(_ptr(v))


def sweep_block(variant: int, v16: np.ndarray, w16: np.ndarray | None = None, lower: int = -3, upper: int = 7) -> int:
    v = np.ascontiguousarray(v16, dtype=np.float32)
    w = None if w16 is None else np.ascontiguousarray(w16, dtype=np.float32)
    return lib().nvfp4_oracle_sweep_block_f32(variant, _ptr(v), _ptr(w), lower, upper)


def offset_histogram(blocks: np.ndarray):
    """{offset: count} of (exhaustive optimum raw code - RNE base code) over fp32 blocks [n, 16], and the number of
    blocks skipped (base code outside 16..119: subnormal window or within reach of saturation)."""
    x = np.ascontiguousarray(blocks, dtype=np.float32).reshape(-1, 16)
    hist = np.zeros(128, dtype=np.int64)
    skipped = np.zeros(1, dtype=np.int64)
    lib().nvfp4_oracle_offset_histogram(_ptr(x), x.shape[0], _ptr(hist), _ptr(skipped))
    return {i - 64: int(c) for i, c in enumerate(hist) if c}, int(skipped[0])


def prune_study(blocks: np.ndarray, gs_inv: float = 1.0, lower: int = -3, upper: int = 7) -> dict:
    """Survivor statistics of the saturation-bound pruning rule for the unweighted sweep (see the C source)."""
    x = np.ascontiguousarray(blocks, dtype=np.float32).reshape(-1, 16)
    nc = upper - lower + 1
    surv = np.zeros(nc + 1, np.int64)
    warp = np.zeros(nc + 1, np.int64)
    pruned = np.zeros(nc, np.int64)
    prefix = np.zeros(nc, np.int64)
    wrong = lib().nvfp4_oracle_prune_study(_ptr(x), x.shape[0], float(gs_inv), lower, upper, _ptr(surv), _ptr(warp),
                                           _ptr(pruned), _ptr(prefix))
    return {"blocks": int(x.shape[0]), "changed": int(wrong), "survivors": surv, "warp_max": warp,
            "pruned_by_offset": pruned, "prefix_elements": prefix}


def e4m3_to_f32(raw: int) -> float:
    return lib().nvfp4_oracle_e4m3_to_f32(raw)


def f32_to_e4m3(x: float) -> int:
    return lib().nvfp4_oracle_f32_to_e4m3(x)


def swizzled_offset(row: int, col: int, k_pad: int) -> int:
    return lib().nvfp4_oracle_swizzled_offset(row, col, k_pad)


def div_full_table_is_measured() -> bool:
    return bool(lib().nvfp4_oracle_div_full_table_is_measured())


def bf16_bits(t) -> np.ndarray:
    """torch bf16 / fp16 tensor (CPU) -> numpy uint16 bit patterns."""
    import torch

    assert t.dtype in (torch.bfloat16, torch.float16)
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)
