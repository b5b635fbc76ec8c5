"""Partitioning of the hot path across the GPUs of one node (one process per GPU).

Every 16-element block is independent once the tensor-wide `global_scale_inv` is known,
so quantization shards by rows and the GEMM by weight rows (the N dimension) with no
collective on the data path.  Shards start at multiples of 128 rows: a 128-row group of
the tiled scale layout is `k_pad * 128` contiguous bytes, so each rank's scales are one
contiguous slab of the global scale buffer and the shards concatenate bit for bit into
what a single GPU would have produced.  The only optional communication is a 4-byte MAX
all-reduce when the global amax has to be taken over sharded data, and a final gather.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

GROUP_ROWS = 128


def round_up(x: int, y: int) -> int:
    return (x + y - 1) // y * y


def row_shards(rows: int, world: int, align: int = GROUP_ROWS) -> list[tuple[int, int]]:
    """Contiguous [start, stop) per rank; starts are multiples of `align`; sizes differ by at most one group."""
    if world < 1:
        raise ValueError("world must be >= 1")
    groups = (rows + align - 1) // align
    base, extra = divmod(groups, world)
    out, g = [], 0
    for r in range(world):
        take = base + (1 if r < extra else 0)
        start = min(g * align, rows)
        stop = min((g + take) * align, rows)
        out.append((start, stop))
        g += take
    return out


def scale_slab(start: int, stop: int, blocks: int) -> tuple[int, int]:
    """Byte range of rows [start, stop) inside the tiled scale buffer of a matrix with `blocks` scale columns."""
    if start % GROUP_ROWS:
        raise ValueError("shards must start at a multiple of 128 rows")
    k_pad = round_up(blocks, 4)
    return start * k_pad, round_up(stop, GROUP_ROWS) * k_pad


def global_amax_scale(local_amax: torch.Tensor, fp8_max: float, group=None) -> tuple[torch.Tensor, torch.Tensor]:
    """Tensor-wide (global_scale, global_scale_inv) from each rank's local amax: one 4-byte MAX all-reduce.
    Arithmetic as helper.get_nvfp4_global_scale (multiply by the fp32 reciprocal of 6*fp8_max, then 1/x)."""
    amax = local_amax.detach().float().reshape(1).clone()
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    inv_den = torch.tensor(1.0, dtype=torch.float32, device=amax.device) / torch.tensor(
        6.0 * fp8_max, dtype=torch.float32, device=amax.device)
    gs = amax * inv_den
    return gs.reshape(()), gs.reciprocal().reshape(())


def quantize_row_shard(quantize: Callable, x_full_rows: int, x_local: torch.Tensor, rank: int, world: int, **kw):
    """Run `quantize(x_local, **kw) -> (codes, scales)` on this rank's rows; returns them with the shard bounds.
    `x_local` must be rows row_shards(x_full_rows, world)[rank] of the full matrix."""
    start, stop = row_shards(x_full_rows, world)[rank]
    if x_local.shape[0] != stop - start:
        raise ValueError(f"rank {rank} expects {stop - start} rows, got {x_local.shape[0]}")
    codes, scales = quantize(x_local, **kw)
    return codes, scales, (start, stop)


def gather_rows(codes: torch.Tensor, scales: torch.Tensor, rows: int, blocks: int, group=None):
    """Optional final gather: every rank ends with the full codes [rows, blocks*8] and the full tiled scale
    buffer (uint8, flat), identical to a single-GPU quantization."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    shards = row_shards(rows, world)
    scales = scales.contiguous().view(torch.uint8).reshape(-1)
    max_rows = max(b - a for a, b in shards)
    max_sc = max(scale_slab(a, b, blocks)[1] - scale_slab(a, b, blocks)[0] for a, b in shards)
    cbuf = torch.zeros((max_rows, blocks * 8), dtype=torch.uint8, device=codes.device)
    sbuf = torch.zeros(max_sc, dtype=torch.uint8, device=codes.device)
    a, b = shards[rank]
    cbuf[: b - a] = codes
    sbuf[: scales.numel()] = scales
    call = [torch.empty_like(cbuf) for _ in range(world)]
    sall = [torch.empty_like(sbuf) for _ in range(world)]
    dist.all_gather(call, cbuf, group=group)
    dist.all_gather(sall, sbuf, group=group)
    full_codes = torch.cat([call[r][: shards[r][1] - shards[r][0]] for r in range(world)], 0)
    full_scales = torch.zeros(round_up(rows, GROUP_ROWS) * round_up(blocks, 4), dtype=torch.uint8, device=codes.device)
    for r, (s0, s1) in enumerate(shards):
        lo, hi = scale_slab(s0, s1, blocks)
        full_scales[lo:hi] = sall[r][: hi - lo]
    return full_codes, full_scales


def column_shards(n: int, world: int, align: int = GROUP_ROWS) -> list[tuple[int, int]]:
    """N-dimension shards for the GEMM: weight rows [start, stop) per rank (same rule as row_shards)."""
    return row_shards(n, world, align)
