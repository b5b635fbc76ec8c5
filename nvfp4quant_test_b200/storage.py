"""File format for NVFP4-quantized matrices: what a serving stack loads instead of bf16 weights.

One `.nvfp4` file = a small JSON header + raw little-endian payloads:
    magic "NVFP4Q01", uint32 header length, header JSON, then for every tensor its packed E2M1 codes
    (uint8 [rows, cols/2]), its E4M3 block scales in the 128x4-tiled order the GEMM consumes
    (uint8 [round_up(rows,128) * round_up(cols/16,4)]) and its fp32 global scale.
Scales are stored tiled (ready for nvfp4_scaled_mm); `as_linear_scales` converts to the row-major [rows, cols/16]
view (the reference's unswizzle_vllm_fp4_scale, kernels/kernel_vllm.py:51-70).  Pure torch/numpy, any device.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

from .kernels.kernel_vllm import round_up, swizzle_vllm_fp4_scale, unswizzle_vllm_fp4_scale

MAGIC = b"NVFP4Q01"


def save(path, tensors: dict) -> None:
    """tensors: name -> (codes uint8 [rows, cols/2], scales (tiled, any 1-byte/int32 dtype), global_scale)."""
    header, blobs, offset = {"tensors": {}}, [], 0
    for name, (codes, scales, gs) in tensors.items():
        rows, half = codes.shape
        cols = half * 2
        c = codes.detach().contiguous().cpu().numpy()
        s = scales.detach().contiguous().view(torch.uint8).reshape(-1).cpu().numpy()
        need = round_up(rows, 128) * round_up(cols // 16, 4)
        if s.size != need:
            raise ValueError(f"{name}: scale buffer has {s.size} bytes, the tiled layout needs {need}")
        g = np.array([float(gs)], dtype="<f4")
        entry = {"rows": rows, "cols": cols, "codes": [offset, c.nbytes]}
        offset += c.nbytes
        entry["scales"] = [offset, s.nbytes]
        offset += s.nbytes
        entry["global_scale"] = [offset, 4]
        offset += 4
        header["tensors"][name] = entry
        blobs += [c.tobytes(), s.tobytes(), g.tobytes()]
    raw = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<I", len(raw)) + raw)
        for b in blobs:
            f.write(b)


def load(path, device="cpu") -> dict:
    """name -> (codes uint8 [rows, cols/2], scales float8_e4m3fn [round_up(rows,128), round_up(cols/16,4)] tiled,
    global_scale 0-dim float32)."""
    data = Path(path).read_bytes()
    if data[:8] != MAGIC:
        raise ValueError("not an NVFP4Q01 file")
    (hlen,) = struct.unpack("<I", data[8:12])
    header = json.loads(data[12:12 + hlen])
    base = 12 + hlen
    out = {}
    for name, e in header["tensors"].items():
        rows, cols = e["rows"], e["cols"]
        o, n = e["codes"]
        codes = torch.from_numpy(np.frombuffer(data, dtype=np.uint8, count=n, offset=base + o).copy()).reshape(rows, cols // 2)
        o, n = e["scales"]
        scales = torch.from_numpy(np.frombuffer(data, dtype=np.uint8, count=n, offset=base + o).copy())
        scales = scales.reshape(round_up(rows, 128), round_up(cols // 16, 4)).view(torch.float8_e4m3fn)
        o, _ = e["global_scale"]
        gs = torch.tensor(np.frombuffer(data, dtype="<f4", count=1, offset=base + o)[0], dtype=torch.float32)
        out[name] = (codes.to(device), scales.to(device), gs.to(device))
    return out


def as_linear_scales(scales_tiled: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    return unswizzle_vllm_fp4_scale(scales_tiled, rows, cols)


def as_tiled_scales(scales_linear: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    return swizzle_vllm_fp4_scale(scales_linear, rows, cols)
