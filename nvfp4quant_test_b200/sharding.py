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


class ImportanceGather:
    """Send / receive buffers for a row-sharded weight whose importance is reduced on the fly, allocated once.

    Every rank reduces the channel square norms of its column slice `columns` of the activation batch straight into
    `imp_slot` and the global scale of its weight rows, (amax_local / (6 * fp8_max), its reciprocal) as
    get_nvfp4_global_scale computes them, straight into `scale_slot`; `gather()` then moves both with ONE all-gather
    and returns (importance [1, n], global_scale, global_scale_inv) of the whole weight.  The tensor-wide scale is the
    largest local one (multiplying the amax by a positive constant is monotone) and its reciprocal the smallest local
    reciprocal (a correctly rounded division is monotone too), so both are the bits a single GPU computes."""

    def __init__(self, n: int, device, group=None):
        self.n, self.group = n, group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.shards = importance_shards(n, self.world)
        self.columns = self.shards[self.rank]
        self.width = max(b - a for a, b in self.shards)
        self._mine = torch.zeros(self.width + 2, dtype=torch.float32, device=device)
        self._all = torch.empty(self.world * (self.width + 2), dtype=torch.float32, device=device)
        a, b = self.columns
        self.imp_slot = self._mine[: b - a].view(1, b - a)
        self.scale_slot = self._mine[self.width:]
        self._even = all(d - c == self.width for c, d in self.shards)

    def gather(self):
        w = self.width
        if self.world == 1:
            return self.imp_slot, self.scale_slot[0], self.scale_slot[1]
        dist.all_gather_into_tensor(self._all, self._mine, group=self.group)
        table = self._all.view(self.world, w + 2)
        if self._even:
            imp = table[:, :w].reshape(1, self.n)          # one copy: the slices sit w + 2 apart
        else:
            imp = torch.cat([table[r, : d - c] for r, (c, d) in enumerate(self.shards)]).reshape(1, self.n)
        return imp, table[:, w].amax(), table[:, w + 1].amin()


def gather_importance_and_scale(imp_part: torch.Tensor, gs_local: torch.Tensor, n: int, group=None):
    """(importance [1, n], global_scale, global_scale_inv) from this rank's importance slice
    importance_shards(n, world)[rank] and the global scale of its weight rows: ImportanceGather for callers that hold
    the two as separate tensors (it copies them into the send buffer)."""
    g = ImportanceGather(n, imp_part.device, group)
    imp_part = imp_part.reshape(1, -1).float()
    if imp_part.shape[1] != g.imp_slot.shape[1]:
        raise ValueError(f"rank {g.rank} expects {g.imp_slot.shape[1]} importance values, got {imp_part.shape[1]}")
    g.imp_slot.copy_(imp_part)
    gs = gs_local.detach().float().reshape(1)
    g.scale_slot[0:1].copy_(gs)
    g.scale_slot[1:2].copy_(gs.reciprocal())
    imp, gs_all, gs_inv = g.gather()
    return imp.contiguous(), gs_all.reshape(()), gs_inv.reshape(())
