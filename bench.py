"""Benchmark of the hot path: ScaleSweep_MSE NVFP4 quantization of a bf16 [8192, 8192] tensor per GPU
(the bsz = 8192 row of the reference's latency sweep, bench.py:31,131-150 of efsotr/nvfp4quant_test),
plus the NVFP4 GEMM that consumes such operands.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
         --master-port P bench.py --gpus N --steps K --warmup W

One JSON line is printed by rank 0.  A step = one quantization of this rank's [8192, 8192] shard
(rows are independent, so ranks share nothing: weak scaling, no collective on the data path).
`value` = algorithmic bytes moved per second over all ranks, inputs resident in HBM, timed with CUDA
events (max over ranks).  `e2e` = the same metric through the public host-buffer entry point
(host_pipeline.HostQuantizer: pinned host input, codes + scales copied back to pinned host memory, every step).
Algorithmic bytes per row of 8192 elements: 16384 read + 4096 codes + 512 scales = 20992.
`--impl reference` times the CPU restatement of the reference's algorithm (oracle/) on all host
threads; the reference itself is GPU-only Triton code and has no CPU implementation.
"""
from __future__ import annotations

import argparse
import json
import os
import pathlib
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS, DIM = 8192, 8192
BYTES_PER_ROW = DIM * 2 + DIM // 2 + DIM // 16          # 20992
ALGO_BYTES = ROWS * BYTES_PER_ROW                        # 171 966 464 per launch
METRIC = "ScaleSweep_MSE NVFP4 quantization throughput, bf16 [8192, 8192] per GPU (algorithmic GB/s)"
WORKLOAD = "configs[1] bsz=8192: ScaleSweep_MSE quant of bf16 [8192,8192] N(0,1), FP8_MAX=256, swizzled scales"
NOMINAL_FP4_TFLOPS = 9000.0
# dram__bytes_read.sum + dram__bytes_write.sum of one quant_kernel launch on this workload (ncu capture,
# summarised under profiles/): 135.14 MB read + 21.24 MB written (the rest of the 37.7 MB of
# outputs is still in L2 when the kernel ends).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 156_381_696


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 0.0)), "measured (MEASURED_PEAKS.json)"
    return 6650.0, 1590.0, "fallback (earlier measurement on this pool)"


class ClockSampler(threading.Thread):
    """Reads SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int, period_s: float = 0.002):
        super().__init__(daemon=True)
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
        self.max_mhz = None
        self._stop_evt, self.window = threading.Event(), [None, None]
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake_slowdown",
        }
        while not self._stop_evt.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:  # noqa: BLE001
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, mask))
                for bit, name in names.items():
                    if mask & bit and self._in_window():
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def _in_window(self):
        return self.window[0] is not None and self.window[1] is None

    def stop(self):
        self._stop_evt.set()

    def summary(self):
        t0, t1 = self.window
        inside = [m for (t, m, _) in self.samples if t0 is not None and t1 is not None and t0 <= t <= t1]
        pool = inside or [m for (_, m, _) in self.samples]
        pool.sort()
        med = pool[len(pool) // 2] if pool else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(inside)}


def cpu_baseline(rows: int, threads: int):
    """Time the CPU port of the same algorithm (oracle/) on `rows` rows of the same workload."""
    import numpy as np
    import torch

    from oracle import oracle as O

    O.build()
    g = torch.Generator(device="cpu")
    g.manual_seed(0)
    x = torch.randn((rows, DIM), generator=g, dtype=torch.float32).to(torch.bfloat16)
    amax = float(x.float().abs().max())
    gs_inv = float(np.float32(1.0) / np.float32(np.float32(amax) * (np.float32(1.0) / np.float32(6.0 * 256.0))))
    xb = O.bf16_bits(x)
    O.quant(0, xb[:64], gs_inv, nthreads=threads)  # warm the thread pool
    t0 = time.perf_counter()
    O.quant(0, xb, gs_inv, nthreads=threads)
    dt = time.perf_counter() - t0
    return rows * BYTES_PER_ROW / dt / 1e9, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows = 1024
    for _ in range(max(args.warmup, 1)):
        cpu_baseline(rows, threads)
    t = []
    for _ in range(args.steps):
        _, dt = cpu_baseline(rows, threads)
        t.append(dt)
    per_step = sum(t) / len(t)
    val = rows * BYTES_PER_ROW / per_step / 1e9
    sample = f"{rows} of {ROWS} rows per step (same N(0,1) bf16 rows, all 11 candidates), {threads} OpenMP threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-gemm", action="store_true", help="skip the secondary GEMM measurement")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # keep stdout to the one JSON line: NCCL prints its version banner there at the VERSION debug level
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)

    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- inputs: this rank's [8192, 8192] shard, 4 distinct copies so every step reads data that is
    #      not in the 126 MB L2 (each input is 134 MB; 4 x 134 MB rotate)
    n_rot = 4
    gen = torch.Generator(device=dev)
    gen.manual_seed(1000 + rank)
    xs = [torch.normal(0.0, 1.0, size=(ROWS, DIM), generator=gen, device=dev, dtype=torch.bfloat16)
          for _ in range(n_rot)]
    gs_pairs = [H.get_nvfp4_global_scale(x, 256.0) for x in xs]      # outside the timed region, like the reference
    gs_inv = [p[1].reshape(1).clone() for p in gs_pairs]
    codes, scales = K.create_fp4_output_tensors(ROWS, DIM, dev, True)

    def step(i):
        K.scalesweep_mse_nvfp4_quant_out(xs[i % n_rot], gs_inv[i % n_rot], True, output=codes, output_scale=scales)

    sampler = ClockSampler(local_rank)
    sampler.start()
    for i in range(args.warmup):
        step(i)
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.window[0] = time.perf_counter()
    start.record()
    for i in range(args.steps):
        step(i)
    end.record()
    barrier()
    sampler.window[1] = time.perf_counter()
    ms_total = max_over_ranks(start.elapsed_time(end))
    ms_step = ms_total / args.steps
    value = world * ALGO_BYTES / (ms_step * 1e-3) / 1e9
    kernel_gbs = ALGO_BYTES / (ms_step * 1e-3) / 1e9     # one kernel per step: its average duration is the step

    # ---- end to end through the public host-buffer entry point: pinned host input -> device -> quantize
    #      -> pinned host codes + scales, every step (row chunks pipelined over three streams)
    from nvfp4quant_test_b200.host_pipeline import HostQuantizer

    host_in = torch.empty((ROWS, DIM), dtype=torch.bfloat16, pin_memory=True)
    host_in.copy_(xs[0])
    host_codes = torch.empty((ROWS, DIM // 2), dtype=torch.uint8, pin_memory=True)
    host_scales = torch.empty((ROWS * DIM // 16,), dtype=torch.uint8, pin_memory=True)
    hq = HostQuantizer(ROWS, DIM, torch.bfloat16, dev, chunk_rows=1024)
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_step():
        hq(host_in, gs_inv[0], host_codes, host_scales)

    for _ in range(3):
        e2e_step()
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2.record()
    barrier()
    e2e_ms = max_over_ranks(s2.elapsed_time(e2)) / e2e_steps
    e2e_value = world * ALGO_BYTES / (e2e_ms * 1e-3) / 1e9
    sampler.stop()

    # ---- secondary: the GEMM that consumes the quantized operands (M = K = 8192, N = 8192 per GPU)
    gemm = None
    if not args.no_gemm:
        qa, sa = K.scalesweep_mse_nvfp4_quant_impl(xs[0], gs_inv[0], True)
        qb, sb = K.scalesweep_mse_nvfp4_quant_impl(xs[1], gs_inv[1], True)
        alpha = (gs_pairs[0][0] * gs_pairs[1][0]).reshape(1).float()
        out = torch.empty((ROWS, ROWS), dtype=torch.bfloat16, device=dev)
        for _ in range(3):
            K.nvfp4_scaled_mm(qa, qb, sa, sb, alpha, torch.bfloat16, out=out)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        g0.record()
        for _ in range(reps):
            K.nvfp4_scaled_mm(qa, qb, sa, sb, alpha, torch.bfloat16, out=out)
        g1.record()
        barrier()
        gms = max_over_ranks(g0.elapsed_time(g1)) / reps
        tf = world * 2.0 * ROWS * ROWS * DIM / (gms * 1e-3) / 1e12
        _, bf16_tf, _ = measured_peaks()
        gemm = {"tflops": tf, "ms": gms, "shape_per_gpu": [ROWS, ROWS, DIM],
                "frac_of_nominal_dense_fp4_9000": tf / world / NOMINAL_FP4_TFLOPS,
                "frac_of_4x_measured_bf16": (tf / world / (4 * bf16_tf)) if bf16_tf else None,
                "status": K.kernel_gemm.gemm_last_status(dev)}

        # decode-sized GEMM: 16 tokens against 8192 x 8192 weights that rotate through ~600 MB, so that every launch
        # streams its weights from HBM (one repeated weight would sit in the 126 MB L2); random codes / scale bytes
        # (timing only), launches replayed from a CUDA graph so that the host is not in the way
        try:
            n_w, tokens = 16, 16
            g = torch.Generator(device=dev)
            g.manual_seed(99)
            wq = [torch.randint(0, 256, (ROWS, DIM // 2), dtype=torch.uint8, device=dev, generator=g) for _ in range(n_w)]
            ws = [torch.randint(0x30, 0x40, (ROWS, DIM // 16), dtype=torch.uint8, device=dev, generator=g) for _ in range(n_w)]
            xq = torch.randint(0, 256, (tokens, DIM // 2), dtype=torch.uint8, device=dev, generator=g)
            xs_ = torch.randint(0x30, 0x40, (128, DIM // 16), dtype=torch.uint8, device=dev, generator=g)
            one = torch.ones(1, dtype=torch.float32, device=dev)
            dout = torch.empty((tokens, ROWS), dtype=torch.bfloat16, device=dev)
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for i in range(n_w):
                    K.nvfp4_scaled_mm(xq, wq[i], xs_, ws[i], one, torch.bfloat16, out=dout)
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize(dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(n_w):
                    K.nvfp4_scaled_mm(xq, wq[i], xs_, ws[i], one, torch.bfloat16, out=dout)
            graph.replay()
            barrier()
            d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dreps = 10
            d0.record()
            for _ in range(dreps):
                graph.replay()
            d1.record()
            barrier()
            dus = max_over_ranks(d0.elapsed_time(d1)) / (dreps * n_w) * 1e3
            wbytes = ROWS * DIM // 2 + ROWS * DIM // 16
            hbm_peak_, _, _ = measured_peaks()
            gemm["decode"] = {"shape_per_gpu": [tokens, ROWS, DIM], "us": dus,
                              "weight_stream_gbs": wbytes / (dus * 1e-6) / 1e9,
                              "frac_of_measured_hbm": wbytes / (dus * 1e-6) / 1e9 / hbm_peak_,
                              "note": "16 weight matrices rotate (600 MB > L2); CUDA graph replay",
                              "status": K.kernel_gemm.gemm_last_status(dev)}
            del wq, ws, graph
        except Exception as exc:  # the headline number must not depend on this extra
            gemm["decode"] = {"error": repr(exc)}

    hbm_peak, _, peak_src = measured_peaks()
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "us_per_step": ms_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_gpu": ROWS, "dim": DIM, "window": [-3, 7],
                   "l2": "4 distinct 134 MB inputs rotate, so each step reads data larger than the 126 MB L2",
                   "partitioning": f"rows, {world} independent shard(s), no collective"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": ROWS * DIM * 2, "d2h_bytes_per_step": ROWS * DIM // 2 + ROWS * DIM // 16},
        "gpu_launches": args.steps * world,
        "roofline": {"bound": "hbm", "achieved": kernel_gbs, "peak": hbm_peak, "unit": "GB/s",
                     "frac": kernel_gbs / hbm_peak, "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                     "peak_source": peak_src, "kernel": "nvfp4::quant_kernel<bf16, MSE>",
                     "algorithmic_bytes_per_launch": ALGO_BYTES},
        "clocks": sampler.summary(),
    }
    if gemm is not None:
        line["gemm"] = gemm
    if rank == 0 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        cpu_rows = ROWS
        val, dt = cpu_baseline(cpu_rows, threads)
        line["cpu_baseline"] = {"value": val, "unit": "GB/s", "cores": threads, "kind": "port",
                                "sample": f"all {cpu_rows} rows once ({dt:.2f} s wall) with {threads} OpenMP threads"}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
