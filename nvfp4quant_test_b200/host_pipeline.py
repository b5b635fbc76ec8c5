"""Quantize a tensor that lives in (pinned) host memory, overlapping PCIe copies with the kernel.

Rows are independent once `global_scale_inv` is known, so the input is cut into row chunks that are a
multiple of 128 rows (one chunk's scales are then a contiguous slab of the tiled scale buffer).  Chunk i is
copied host->device on one stream, quantized on a second, and its codes and scales are copied back on a
third, with events ordering the three; chunk i+1's upload runs while chunk i is quantized and chunk i-1
is downloaded.  The result is byte-identical to quantizing the whole tensor in one launch.
"""
from __future__ import annotations

import torch

from . import _lib
from .kernels import _launch
from .sharding import round_up, scale_slab


def chunk_plan(rows: int, chunk_rows: int) -> list[tuple[int, int]]:
    """[start, stop) row ranges; every start is a multiple of 128."""
    if chunk_rows < 128 or chunk_rows % 128:
        raise ValueError("chunk_rows must be a positive multiple of 128")
    return [(a, min(a + chunk_rows, rows)) for a in range(0, rows, chunk_rows)]


class HostQuantizer:
    """Reusable staging buffers and streams for one (rows, dim, dtype, variant) shape."""

    def __init__(self, rows: int, dim: int, dtype=torch.bfloat16, device="cuda", chunk_rows: int = 1024,
                 variant: int = _lib.VARIANT_MSE, lower: int = -3, upper: int = 7, depth: int = 3):
        if dim % 16:
            raise ValueError("dim must be divisible by 16")
        self.rows, self.dim, self.dtype, self.device = rows, dim, dtype, torch.device(device)
        self.variant, self.lower, self.upper = variant, lower, upper
        self.plan = chunk_plan(rows, chunk_rows)
        self.blocks = dim // 16
        self.k_pad = round_up(self.blocks, 4)
        cr = min(chunk_rows, round_up(rows, 128))
        self.depth = depth
        self.stage_in = [torch.empty((cr, dim), dtype=dtype, device=self.device) for _ in range(depth)]
        self.stage_codes = [torch.empty((cr, dim // 2), dtype=torch.uint8, device=self.device) for _ in range(depth)]
        self.stage_scales = [torch.empty(round_up(cr, 128) * self.k_pad, dtype=torch.uint8, device=self.device)
                             for _ in range(depth)]
        self.s_up, self.s_run, self.s_down = (torch.cuda.Stream(self.device) for _ in range(3))
        self.ev_up = [torch.cuda.Event() for _ in range(depth)]
        self.ev_run = [torch.cuda.Event() for _ in range(depth)]
        self.ev_down = [torch.cuda.Event() for _ in range(depth)]
        self._used = [False] * depth      # slot j's events have been recorded by an earlier chunk (of this or a previous call)

    def __call__(self, x_host: torch.Tensor, gs_inv: torch.Tensor, codes_host: torch.Tensor,
                 scales_host: torch.Tensor, importance: torch.Tensor | None = None) -> None:
        """x_host [rows, dim] (pinned for real overlap); codes_host uint8 [rows, dim/2]; scales_host uint8
        [round_up(rows,128) * round_up(dim/16,4)] (tiled layout).  Returns once everything has been enqueued;
        the caller synchronises (e.g. torch.cuda.synchronize()) before reading the host outputs."""
        if tuple(x_host.shape) != (self.rows, self.dim) or x_host.dtype != self.dtype:
            raise ValueError("input does not match the shape this quantizer was built for")
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_up, self.s_run, self.s_down):
            s.wait_stream(cur)
        flat_scales = scales_host.view(torch.uint8).reshape(-1)
        for i, (a, b) in enumerate(self.plan):
            j = i % self.depth
            n = b - a
            with torch.cuda.stream(self.s_up):
                if self._used[j]:
                    self.s_up.wait_event(self.ev_run[j])      # staging input free once its kernel ran
                self.stage_in[j][:n].copy_(x_host[a:b], non_blocking=True)
                self.ev_up[j].record(self.s_up)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_up[j])
                if self._used[j]:
                    self.s_run.wait_event(self.ev_down[j])    # staging outputs free once downloaded
                _launch.quant_out(self.variant, self.stage_in[j][:n], importance, gs_inv, True,
                                  self.stage_codes[j][:n], self.stage_scales[j], self.lower, self.upper)
                self.ev_run[j].record(self.s_run)
            with torch.cuda.stream(self.s_down):
                self.s_down.wait_event(self.ev_run[j])
                codes_host[a:b].copy_(self.stage_codes[j][:n], non_blocking=True)
                lo, hi = scale_slab(a, b, self.blocks)
                flat_scales[lo:hi].copy_(self.stage_scales[j][: hi - lo], non_blocking=True)
                self.ev_down[j].record(self.s_down)
            self._used[j] = True
        cur.wait_stream(self.s_down)
        cur.wait_stream(self.s_run)
