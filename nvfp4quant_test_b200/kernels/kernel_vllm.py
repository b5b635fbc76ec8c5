"""NVFP4 scale-factor layout helpers.

Counterpart of kernels/kernel_vllm.py of efsotr/nvfp4quant_test (`round_up`,
`swizzle_vllm_fp4_scale`, `unswizzle_vllm_fp4_scale`) plus the output allocation
contract of vllm's `create_fp4_output_tensors` (vllm/_custom_ops.py:36-86), which
the reference's `_impl` entry points call.

Layout: scales of a [m, n] tensor form a [round_up(m,128), round_up(n/16,4)] byte
matrix stored as 128-row x 4-column tiles of 512 contiguous bytes; inside a tile the
byte of (row, col) sits at (row % 32) * 16 + (row % 128) // 32 * 4 + col % 4.  That is
the operand layout tcgen05 block-scaled MMA reads, so the GEMM consumes it unchanged.
These helpers are pure torch (gather/scatter by a computed index) and work on any device.
"""
from __future__ import annotations

import torch


def round_up(x, y):
    return (x + y - 1) // y * y


def _tile_index(m_pad: int, k_pad: int, device) -> torch.Tensor:
    """index[row, col] = byte offset of block (row, col) in the tiled buffer."""
    row = torch.arange(m_pad, device=device, dtype=torch.int64).unsqueeze(1)
    col = torch.arange(k_pad, device=device, dtype=torch.int64).unsqueeze(0)
    return (row // 128) * (k_pad * 128) + (col // 4) * 512 + (row % 32) * 16 + (row % 128) // 32 * 4 + col % 4


def swizzle_vllm_fp4_scale(scale: torch.Tensor, m: int, n: int, block_size: int = 16) -> torch.Tensor:
    """[m, n/block_size] row-major scales -> flat tiled buffer (padding filled with zeros)."""
    assert n % block_size == 0
    k = n // block_size
    assert tuple(scale.shape) == (m, k)
    m_pad, k_pad = round_up(m, 128), round_up(k, 4)
    raw = scale.view(torch.uint8) if scale.element_size() == 1 else scale
    flat = torch.zeros(m_pad * k_pad, dtype=raw.dtype, device=raw.device)
    idx = _tile_index(m_pad, k_pad, raw.device)[:m, :k]
    flat[idx.reshape(-1)] = raw.reshape(-1)
    return flat.view(scale.dtype) if scale.element_size() == 1 else flat


def unswizzle_vllm_fp4_scale(scale_swizzled: torch.Tensor, m: int, n: int, block_size: int = 16) -> torch.Tensor:
    """Flat (or [m_pad, k_pad]-shaped) tiled buffer -> [m, n/block_size] row-major scales."""
    assert n % block_size == 0
    k = n // block_size
    m_pad, k_pad = round_up(m, 128), round_up(k, 4)
    one_byte = scale_swizzled.element_size() == 1
    raw = scale_swizzled.view(torch.uint8) if one_byte else scale_swizzled
    flat = raw.reshape(-1)
    assert flat.numel() == m_pad * k_pad, (flat.numel(), m_pad, k_pad)
    idx = _tile_index(m_pad, k_pad, raw.device)[:m, :k]
    out = flat[idx.reshape(-1)].reshape(m, k).contiguous()
    return out.view(scale_swizzled.dtype) if one_byte else out


def create_fp4_scale_tensor(m: int, n: int, device, is_sf_swizzled_layout: bool) -> torch.Tensor:
    if is_sf_swizzled_layout:
        return torch.empty((round_up(m, 128), round_up(n // 16, 4) // 4), device=device, dtype=torch.int32)
    return torch.empty((m, n // 16), device=device, dtype=torch.uint8)


def create_fp4_output_tensors(m: int, n: int, device, is_sf_swizzled_layout: bool, padded_n: int | None = None):
    """(codes uint8 [m, P/2], scales) with P = padded_n or n; uninitialised like the original."""
    physical_n = padded_n if padded_n is not None else n
    output = torch.empty((m, physical_n // 2), device=device, dtype=torch.uint8)
    return output, create_fp4_scale_tensor(m, physical_n, device, is_sf_swizzled_layout)
