"""Partitioning of the hot path across the GPUs of one node (one process per GPU).

Every 16-element block is independent once the tensor-wide `global_scale_inv` is known,
so quantization shards by rows and the GEMM by weight rows (the N dimension) with no
collective on the data path.  Shards start at multiples of 128 rows: a 128-row group of
the tiled scale layout is `k_pad * 128` contiguous bytes, so each rank's scales are one
contiguous slab of the global scale buffer and the shards concatenate bit for bit into
what a single GPU would have produced.  The only optional communication is a 4-byte MAX
all-reduce when the global amax has to be taken over sharded data, and a final gather.
When the importance vector of a weight is itself computed on the fly (channel square norms
of an activation batch), that reduction shards by COLUMNS - columns are independent, so the
slices concatenate to the single-GPU bits - and one small all-gather carries both the slices
and every rank's local scale.
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


IMPORTANCE_ALIGN = 16   # columns per CTA of the channel-square-norm kernel


def importance_shards(n: int, world: int) -> list[tuple[int, int]]:
    """Column ranges [start, stop) of the importance reduction per rank (starts at multiples of 16 columns)."""
    return row_shards(n, world, IMPORTANCE_ALIGN)


def gather_importance_and_scale(imp_part: torch.Tensor, gs_local: torch.Tensor, n: int, group=None):
    """(importance [1, n], global_scale, global_scale_inv) for a row-sharded weight whose importance is reduced on the
    fly: `imp_part` is this rank's slice importance_shards(n, world)[rank] of the channel square norms (fp32), and
    `gs_local` the global scale of this rank's weight rows (amax_local / (6 * fp8_max), as get_nvfp4_global_scale
    returns it).  ONE all-gather moves both; the tensor-wide scale is the maximum of the local ones (multiplying by a
    positive constant is monotone), its reciprocal one fp32 division, as on a single GPU."""
    imp_part = imp_part.reshape(-1).float()
    gs_local = gs_local.detach().float().reshape(1)
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    if world == 1:
        if imp_part.numel() != n:
            raise ValueError(f"expected {n} importance values, got {imp_part.numel()}")
        gs = gs_local.reshape(())
        return imp_part.reshape(1, n), gs, gs.reciprocal()
    rank = dist.get_rank(group)
    shards = importance_shards(n, world)
    a, b = shards[rank]
    if imp_part.numel() != b - a:
        raise ValueError(f"rank {rank} expects {b - a} importance values, got {imp_part.numel()}")
    width = max(d - c for c, d in shards)
    mine = torch.zeros(width + 1, dtype=torch.float32, device=imp_part.device)
    mine[: b - a] = imp_part
    mine[width:] = gs_local
    flat = torch.empty(world * (width + 1), dtype=torch.float32, device=imp_part.device)
    dist.all_gather_into_tensor(flat, mine, group=group)
    everything = flat.view(world, width + 1)
    if all(d - c == width for c, d in shards):
        imp = everything[:, :width].reshape(1, n)
    else:
        imp = torch.cat([everything[r, : d - c] for r, (c, d) in enumerate(shards)]).reshape(1, n)
    gs = everything[:, width].max()
    return imp.contiguous(), gs, gs.reciprocal()
