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

Further objects on the same line (each measured in this process with the same CUDA-event method):
  sustained       >= 0.5 s of back-to-back launches of the quantizer and of the 8192^3 GEMM with the SM clock sampled
                  every millisecond: microseconds, median MHz, their product
  gemm            8192^3 per GPU with `roofline` (against the tensor-pipe rate measured by the probe kernel in
                  the same run, burst and power-capped), and `decode` (16 tokens over rotating weights)
  third_party     vllm's scaled_fp4_quant / cutlass_scaled_fp4_mm on the same shapes, when vllm loads
  strong_scaling  the three partitioned workloads at --gpus N: one [8192, 8192] weight quantized by rows / N per GPU
                  with importance from a [4096, 8192] batch; the GEMM with N = 28672 weight rows / N per GPU at
                  M = 2048; the Llama-3-8B-shaped stack with 32 layers / N per GPU
`--impl reference` times the CPU restatement of the reference's algorithm (oracle/) on all host
threads over the same 8192 rows per step; the reference itself is GPU-only Triton code and has no CPU implementation.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import pathlib
import sys
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
# summarised under profiles/): 135.14 MB read + 21.00 MB written (the rest of the 37.7 MB of
# outputs is still in L2 when the kernel ends).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 156_140_800


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 0.0)), "measured (MEASURED_PEAKS.json)"
    return 6650.0, 1590.0, "fallback (6650 GB/s copy rate, 1590 TFLOP/s bf16: no MEASURED_PEAKS.json present)"


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
    """CPU arm: the oracle port over all 8192 rows per step (the same work as one step of the GPU arm)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import torch

    from oracle import oracle as O

    O.build()
    threads = os.cpu_count() or 1
    g = torch.Generator(device="cpu")
    g.manual_seed(0)
    x = torch.randn((ROWS, DIM), generator=g, dtype=torch.float32).to(torch.bfloat16)
    amax = float(x.float().abs().max())
    gs_inv = float(np.float32(1.0) / np.float32(np.float32(amax) * (np.float32(1.0) / np.float32(6.0 * 256.0))))
    xb = O.bf16_bits(x)
    for _ in range(max(args.warmup, 1)):
        O.quant(0, xb[:1024], gs_inv, nthreads=threads)      # warm-up on an eighth of the rows: thread pool, page faults
    t = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        O.quant(0, xb, gs_inv, nthreads=threads)
        t.append(time.perf_counter() - t0)
    per_step = sum(t) / len(t)
    val = ALGO_BYTES / per_step / 1e9
    sample = f"all {ROWS} rows per step (same N(0,1) bf16 shape, all 11 candidates), {threads} OpenMP threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_gpu": ROWS, "dim": DIM, "window": [-3, 7], "sample": sample},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def third_party(dev, xs, gs448_inv, torch, B):
    """vllm's own ops on the same shapes, same process, same timing method (context for the numbers above)."""
    try:
        with contextlib.redirect_stdout(sys.stderr):
            import vllm._custom_ops as ops
        ops.scaled_fp4_quant(xs[0][:128], gs448_inv[0])
        torch.cuda.synchronize()
    except Exception as exc:  # noqa: BLE001 - vllm or its compiled ops are not usable here
        return "unavailable: " + repr(exc)[:200]
    import nvfp4quant_test_b200.kernels as K

    out = {}
    ms = B.time_launches(lambda i: ops.scaled_fp4_quant(xs[i % len(xs)], gs448_inv[i % len(xs)]), 30)
    ours = B.time_launches(lambda i: K.scaled_fp4_quant(xs[i % len(xs)], gs448_inv[i % len(xs)]), 30)
    out["scaled_fp4_quant_8192x8192_us"] = {"vllm": ms * 1e3, "ours_amax": ours * 1e3}
    from nvfp4quant_test_b200.sweep import do_bench

    small = {}
    for bsz in (1, 8, 64):
        w = xs[0][:bsz].contiguous()
        small[str(bsz)] = {"vllm": do_bench(lambda: ops.scaled_fp4_quant(w, gs448_inv[0]), 5, 30) * 1e3,
                           "ours_amax": do_bench(lambda: K.scaled_fp4_quant(w, gs448_inv[0]), 5, 30) * 1e3}
    out["scaled_fp4_quant_small_bsz_us"] = dict(small, method="L2 flushed before every call, allocation of the outputs included")
    # GEMMs: random codes / scale bytes (timing only)
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    one = torch.ones(1, dtype=torch.float32, device=dev)

    def operands(m, n, k, copies):
        a = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device=dev, generator=g)
        sa = torch.randint(0x30, 0x40, ((m + 127) // 128 * 128, k // 16), dtype=torch.uint8, device=dev, generator=g)
        bs = [torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev, generator=g) for _ in range(copies)]
        sbs = [torch.randint(0x30, 0x40, (n, k // 16), dtype=torch.uint8, device=dev, generator=g) for _ in range(copies)]
        return a, sa, bs, sbs

    gem = {}
    # the headline shape, a decode batch, and the few-hundred-token cells of the Llama-shaped layers
    shapes = ((8192, 8192, 8192, 1), (16, 8192, 8192, 8), (256, 4096, 4096, 32), (128, 4096, 4096, 32), (128, 1024, 4096, 32),
              (128, 6144, 4096, 20), (256, 14336, 4096, 8), (256, 8192, 8192, 8), (512, 14336, 4096, 8), (2048, 4096, 4096, 32))
    for (m, n, k, copies) in shapes:
        a, sa, bs, sbs = operands(m, n, k, copies)
        f8 = torch.float8_e4m3fn

        def theirs():
            for i in range(copies):
                ops.cutlass_scaled_fp4_mm(a, bs[i], sa.view(f8), sbs[i].view(f8), one, torch.bfloat16)

        o = torch.empty((m, n), dtype=torch.bfloat16, device=dev)

        def mine_raw():
            for i in range(copies):
                K.nvfp4_scaled_mm(a, bs[i], sa, sbs[i], one, torch.bfloat16, out=o)

        pws = [K.PreparedWeight(bs[i], sbs[i]) for i in range(copies)]

        def mine():
            for i in range(copies):
                K.nvfp4_scaled_mm_prepared(a, sa, one, pws[i], out=o)

        gem[f"{m}x{n}x{k}"] = {"cutlass_scaled_fp4_mm": B.time_graph(theirs, copies), "ours": B.time_graph(mine, copies),
                               "ours_raw_pointers": B.time_graph(mine_raw, copies), "weight_copies": copies}
        del a, sa, bs, sbs, pws
    out["gemm_us"] = dict(gem, method="CUDA graph replay over rotating weight copies; `ours` = prepared weights (the "
                                      "GEMM streams them while its predecessor finishes), `ours_raw_pointers` = the "
                                      "drop-in call, which waits for its predecessor before reading either operand")
    return out


def strong_scaling(dev, rank, world, torch, dist, max_over_ranks, barrier):
    """The partitioned workloads (total work fixed, split over the ranks); milliseconds are max over ranks."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import benchtools as B
    from nvfp4quant_test_b200 import gemm_sweep as GS
    from nvfp4quant_test_b200 import helper as H
    from nvfp4quant_test_b200 import llama_stack
    from nvfp4quant_test_b200.sharding import row_shards

    out = {}
    # -- one Laplace(0,1) [8192, 8192] weight, rows / N per GPU; importance = channel square norms of a Laplace
    #    [4096, 8192] batch; the tensor-wide scale needs one 4-byte MAX all-reduce (gs = amax * c is monotone in amax)
    w_full = GS.laplace((ROWS, DIM), 0, dev)
    act = GS.laplace((4096, DIM), 1, dev)
    a, b = row_shards(ROWS, world)[rank]
    w = w_full[a:b].contiguous()
    del w_full
    codes, scales = K.create_fp4_output_tensors(b - a, DIM, dev, True)

    from nvfp4quant_test_b200.sharding import ImportanceGather

    ig = ImportanceGather(DIM, dev)
    c0, c1 = ig.columns

    def step2(_i):
        # the importance reduction shards by columns (each rank reads 1 / world of the batch), the weight by rows; both
        # kernels write into the send buffer of one all-gather that carries the importance slices and the local scales
        H.channel_square_norm(act[:, c0:c1], out=ig.imp_slot)
        H.get_nvfp4_global_scale(w, 256.0, out=ig.scale_slot)
        imp, _gs, gs_inv = ig.gather()
        K.scalesweep_weighted_mse_nvfp4_quant_out(w, imp, gs_inv, True, output=codes, output_scale=scales)

    barrier()
    ms = max_over_ranks(B.time_launches(step2, 20))
    out["config2_weighted_weight_quant"] = {
        "ms": ms, "rows_per_gpu": b - a, "shape": [ROWS, DIM], "gweights_per_s": ROWS * DIM / (ms * 1e-3) / 1e9,
        "includes": "importance reduction over the [4096, 8192] batch (columns / N per GPU) + shard amax + one all-gather "
                    "of the importance slices and local scales + weighted sweep"}
    del w, act, codes, scales
    # -- GEMM: M = 2048 activations against N = 28672 weight rows, N / world rows per GPU, K = 8192
    M, N, Kd = 2048, 28672, 8192
    na, nb = row_shards(N, world)[rank]
    x = GS.laplace((M, Kd), 3, dev)
    wsh = GS.laplace((nb - na, Kd), 100 + rank, dev)
    qa, sa, gsa = GS.quantize_operand("ScaleSweep_MSE", x, wsh)
    qw, sw, gsw = GS.quantize_operand("ScaleSweep_MSE", wsh, x)
    alpha = (gsa * gsw).reshape(1).float()
    o = torch.empty((M, nb - na), dtype=torch.bfloat16, device=dev)
    barrier()
    ms = max_over_ranks(B.time_launches(lambda _i: K.nvfp4_scaled_mm(qa, qw, sa, sw, alpha, torch.bfloat16, out=o), 20))
    out["config3_gemm_m2048_n28672"] = {"ms": ms, "weight_rows_per_gpu": nb - na, "shape": [M, N, Kd],
                                        "tflops": 2.0 * M * N * Kd / (ms * 1e-3) / 1e12}
    del x, wsh, qa, sa, qw, sw, o
    torch.cuda.empty_cache()
    # -- Llama-3-8B-shaped stack, 32 layers / world per GPU
    barrier()
    res = llama_stack.run(32, [1, 32, 256, 4096])
    if rank == 0:
        out["config4_llama_stack"] = {
            "quantize_ms": res["quantize_ms"], "quantize_first_pass_ms": res["quantize_first_pass_ms"],
            "quantize_gweights_per_s": res["quantize_gweights_per_s"],
            "gemm_phase_ms_all_layers": {str(g["tokens"]): g["ms_all_layers"] for g in res["gemm"]},
            "gemm_phase_eager_ms_all_layers": {str(g["tokens"]): g["eager_ms_all_layers"] for g in res["gemm"]},
            "layers_per_gpu": 32 // world if world <= 32 else 0,
            "includes": "per layer: activation global scale + ScaleSweep quantization + 7 GEMMs, one CUDA graph per rank"}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-gemm", action="store_true", help="skip the secondary GEMM measurement")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the sustained passes, the third-party comparison and the strong-scaling workloads")
    ap.add_argument("--deadline", type=float, default=900.0,
                    help="seconds after which a stuck run prints every thread's Python stack to stderr and exits with code 3")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    import faulthandler

    faulthandler.dump_traceback_later(args.deadline, exit=True, file=sys.stderr)
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
    from nvfp4quant_test_b200 import benchtools as B
    from nvfp4quant_test_b200 import helper as H

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    t_start = time.perf_counter()

    def phase(name: str) -> None:
        """Progress note on stderr (stdout carries only the JSON line)."""
        if rank == 0:
            print(f"[bench {time.perf_counter() - t_start:7.2f} s] {name}", file=sys.stderr, flush=True)

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

    phase("timed quantization steps")
    sampler = B.ClockSampler(local_rank)
    sampler.start()
    for i in range(args.warmup):
        step(i)
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.perf_counter()
    start.record()
    for i in range(args.steps):
        step(i)
    end.record()
    barrier()
    t_end = time.perf_counter()
    ms_total = max_over_ranks(start.elapsed_time(end))
    ms_step = ms_total / args.steps
    value = world * ALGO_BYTES / (ms_step * 1e-3) / 1e9
    kernel_gbs = ALGO_BYTES / (ms_step * 1e-3) / 1e9     # one kernel per step: its average duration is the step
    clocks = sampler.window(t_begin, t_end)

    # ---- end to end through the public host-buffer entry point: pinned host input -> device -> quantize
    #      -> pinned host codes + scales, every step (row chunks pipelined over three streams)
    from nvfp4quant_test_b200.host_pipeline import HostQuantizer

    phase("end-to-end steps through the host pipeline")
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

    hbm_peak, bf16_tf, peak_src = measured_peaks()
    extras = not args.no_extras

    # ---- sustained pass of the quantizer: >= 0.5 s back to back, clocks sampled every millisecond
    phase("sustained quantizer pass")
    sustained = {}
    if extras:
        barrier()
        sustained["quant"] = B.time_sustained(step, 0.5, sampler, ms_step)
        sustained["quant"]["frac_of_measured_hbm"] = ALGO_BYTES / (sustained["quant"]["us"] * 1e-6) / 1e9 / hbm_peak

    # ---- secondary: the GEMM that consumes the quantized operands (M = K = 8192, N = 8192 per GPU)
    gemm = None
    if not args.no_gemm:
        phase("GEMM 8192^3")
        qa, sa = K.scalesweep_mse_nvfp4_quant_impl(xs[0], gs_inv[0], True)
        qb, sb = K.scalesweep_mse_nvfp4_quant_impl(xs[1], gs_inv[1], True)
        alpha = (gs_pairs[0][0] * gs_pairs[1][0]).reshape(1).float()
        out = torch.empty((ROWS, ROWS), dtype=torch.bfloat16, device=dev)

        def gstep(_i):
            K.nvfp4_scaled_mm(qa, qb, sa, sb, alpha, torch.bfloat16, out=out)

        barrier()
        gms = max_over_ranks(B.time_launches(gstep, 10))
        flop = 2.0 * ROWS * ROWS * DIM
        tf = world * flop / (gms * 1e-3) / 1e12
        gemm = {"tflops": tf, "ms": gms, "shape_per_gpu": [ROWS, ROWS, DIM],
                "frac_of_nominal_dense_fp4_9000": tf / world / NOMINAL_FP4_TFLOPS,
                "frac_of_4x_measured_bf16": (tf / world / (4 * bf16_tf)) if bf16_tf else None,
                "status": K.kernel_gemm.gemm_last_status(dev)}
        # decode-sized GEMM: 16 tokens against 8192 x 8192 weights that rotate through ~600 MB, so that every launch
        # streams its weights from HBM (one repeated weight would sit in the 126 MB L2); random codes / scale bytes
        # (timing only), launches replayed from a CUDA graph so that the host is not in the way
        try:
            phase("decode-sized GEMM")
            n_w, tokens = 16, 16
            g = torch.Generator(device=dev)
            g.manual_seed(99)
            wq = [torch.randint(0, 256, (ROWS, DIM // 2), dtype=torch.uint8, device=dev, generator=g) for _ in range(n_w)]
            ws = [torch.randint(0x30, 0x40, (ROWS, DIM // 16), dtype=torch.uint8, device=dev, generator=g) for _ in range(n_w)]
            xq = torch.randint(0, 256, (tokens, DIM // 2), dtype=torch.uint8, device=dev, generator=g)
            xs_ = torch.randint(0x30, 0x40, (128, DIM // 16), dtype=torch.uint8, device=dev, generator=g)
            one = torch.ones(1, dtype=torch.float32, device=dev)
            dout = torch.empty((tokens, ROWS), dtype=torch.bfloat16, device=dev)

            pws = [K.PreparedWeight(wq[i], ws[i]) for i in range(n_w)]

            def record():
                for i in range(n_w):
                    K.nvfp4_scaled_mm_prepared(xq, xs_, one, pws[i], out=dout)

            barrier()
            dus = max_over_ranks(B.time_graph(record, n_w))
            wbytes = ROWS * DIM // 2 + ROWS * DIM // 16
            gemm["decode"] = {"shape_per_gpu": [tokens, ROWS, DIM], "us": dus,
                              "weight_stream_gbs": wbytes / (dus * 1e-6) / 1e9,
                              "frac_of_measured_hbm": wbytes / (dus * 1e-6) / 1e9 / hbm_peak,
                              "note": "16 prepared weight matrices rotate (600 MB > L2); CUDA graph replay",
                              "status": K.kernel_gemm.gemm_last_status(dev)}
            del wq, ws, pws
        except Exception as exc:  # the headline number must not depend on this extra
            gemm["decode"] = {"error": repr(exc)}
        if extras:
            barrier()
            phase("FP4 tensor-pipe probe and sustained GEMM pass")
            peak = B.fp4_peak(sampler)       # the tensor pipe's own rate for this instruction, same run
            barrier()
            sus = B.time_sustained(gstep, 0.5, sampler, gms)
            sus_tf = flop / (sus["us"] * 1e-6) / 1e12
            sus["tflops_per_gpu"] = sus_tf
            sus["tflops_at_max_clock"] = (sus_tf * sampler.max_mhz / sus["sm_mhz_median"]) if sus.get("sm_mhz_median") and sampler.max_mhz else None
            sustained["gemm_8192"] = sus
            gemm["roofline"] = {
                "bound": "tensor", "achieved": sus_tf, "peak": peak["sustained_tflops"], "unit": "TFLOP/s",
                "frac": sus_tf / peak["sustained_tflops"],
                "peak_source": "probe kernel of this run: back-to-back tcgen05.mma kind::mxf4nvf4 on shared-memory operands, ~0.4 s under the power cap",
                "burst": {"achieved": tf / world, "peak": peak["burst_tflops"], "frac": tf / world / peak["burst_tflops"]},
                "nominal_dense_fp4": NOMINAL_FP4_TFLOPS, "frac_of_nominal": sus_tf / NOMINAL_FP4_TFLOPS,
                "peak_probe": peak, "kernel": "gemm::pair::gemm_pair_kernel<192>",
                "algorithmic_flop_per_launch": flop}

        del qa, qb, sa, sb, out

    tp = None
    if extras:
        barrier()
        if rank == 0:
            phase("third-party ops")
            gs448_inv = [H.get_nvfp4_global_scale(x, 448.0)[1].reshape(1).clone() for x in xs]
            try:
                tp = third_party(dev, xs, gs448_inv, torch, B)
            except Exception as exc:  # noqa: BLE001
                tp = "unavailable: " + repr(exc)[:200]
        barrier()
    del xs
    torch.cuda.empty_cache()

    strong = None
    if extras:
        try:
            phase("strong-scaling workloads")
            strong = strong_scaling(dev, rank, world, torch, dist, max_over_ranks, barrier)
        except Exception as exc:  # noqa: BLE001
            strong = {"error": repr(exc)[:300]}
    sampler.stop()

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
        "clocks": dict({k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "reasons", "samples")}, source="timed region"),
    }
    if clocks["samples"] < 3 and sustained.get("quant", {}).get("clock_samples"):
        # the timed region is a few milliseconds: too short for the 1 ms sampler; the sustained pass of the same kernel
        # right after it has the record
        q = sustained["quant"]
        line["clocks"] = {"sm_mhz": q["sm_mhz_median"], "sm_max_mhz": sampler.max_mhz, "reasons": q["reasons"],
                          "samples": q["clock_samples"], "source": "sustained pass of the same kernel (timed region too short to sample)"}
    if sustained:
        line["sustained"] = sustained
    if gemm is not None:
        line["gemm"] = gemm
    if extras:
        line["third_party"] = tp if tp is not None else "measured on rank 0 only"
        line["strong_scaling"] = strong
    if rank == 0 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        cpu_rows = ROWS
        phase("CPU baseline")
        val, dt = cpu_baseline(cpu_rows, threads)
        line["cpu_baseline"] = {"value": val, "unit": "GB/s", "cores": threads, "kind": "port",
                                "sample": f"all {cpu_rows} rows once ({dt:.2f} s wall) with {threads} OpenMP threads"}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
