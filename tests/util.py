"""Helpers shared by the parity tests."""
from __future__ import annotations

import numpy as np
import torch

VARIANT = {"mse": 0, "weighted": 1, "amax": 2}


def window(case):
    lo, up = (-3, 7) if case["variant"] == "mse" else (-8, 7)
    if case["lower"] is not None:
        lo, up = case["lower"], case["upper"]
    return lo, up


def to_numpy_input(x: torch.Tensor):
    """(array, x_dtype hint) in the form oracle.quant accepts."""
    if x.dtype == torch.float32:
        return x.contiguous().numpy(), None
    arr = x.contiguous().view(torch.int16).numpy().view(np.uint16)
    return arr, ("f16" if x.dtype == torch.float16 else None)


def logical_scale_index(m: int, blocks: int, swizzled: bool) -> np.ndarray:
    """Flat byte offsets of the m x blocks logical scales inside the scale buffer."""
    if not swizzled:
        return np.arange(m * blocks, dtype=np.int64)
    k_pad = (blocks + 3) // 4 * 4
    row = np.arange(m, dtype=np.int64)[:, None]
    col = np.arange(blocks, dtype=np.int64)[None, :]
    off = (row // 128) * (k_pad * 128) + (col // 4) * 512 + (row % 32) * 16 + (row % 128) // 32 * 4 + col % 4
    return off.reshape(-1)


def oracle_quant_case(O, case, gs_inv: float, amax_table=None):
    x, hint = to_numpy_input(case["x"])
    lo, up = window(case)
    imp = None if case["importance"] is None else case["importance"].numpy()
    sixth = float(amax_table[127]) if amax_table is not None else 0.0
    codes, scales = O.quant(VARIANT[case["variant"]], x, gs_inv, imp, swizzled=case["swizzled"],
                            padded_n=case["padded_n"], lower=lo, upper=up, x_dtype=hint,
                            amax_table=amax_table, amax_sixth=sixth)
    return codes, scales.reshape(-1)
