"""Latency / error sweep with the command line and JSON schema of the reference's bench.py
(bench.py:35-49 arguments, :84-114 result rows of efsotr/nvfp4quant_test).

  python -m nvfp4quant_test_b200.sweep [vllm] [ScaleSweep_MSE] [ScaleSweep_MSE_round] [ScaleSweep] \
         [--dim 8192] [--imp ones|ramp|random] [--output FILE | --output-dir result] [--warmup 10] [--rep 100]

For every bsz in {1, 8, 64, 128, 256, 512, 1024, 2048, 4096, 8192} the quantizer is timed the way
triton.testing.do_bench does it (warm-up and repetition budgets in milliseconds, L2 flushed before every timed
call, CUDA events, mean), allocation of the outputs included, then one more call's result is dequantized and
mse / max_abs_error / weighted_mse against the bf16 input are recorded.  Inputs: N(0,1) bf16 from the CUDA
generator with seed 0; global scale amax/(6*448) for the amax baseline and amax/(6*256) for the sweeps.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from . import helper as H
from . import kernels as K

BSZ_LIST = [1, 8, 64, 128, 256, 512, 1024, 2048, 4096, 8192]
BENCHMARKS = ["vllm", "ScaleSweep_MSE", "ScaleSweep_MSE_round", "ScaleSweep"]


def make_w(m: int, k: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return torch.normal(0.0, 1.0, size=(m, k), generator=g, device="cuda", dtype=torch.bfloat16)


def make_imp(kind: str, dim: int) -> torch.Tensor:
    if kind == "ones":
        return torch.ones((1, dim), device="cuda", dtype=torch.float32)
    if kind == "ramp":
        return torch.linspace(0.25, 2.0, dim, device="cuda", dtype=torch.float32).view(1, dim)
    if kind == "random":
        g = torch.Generator(device="cuda")
        g.manual_seed(123)
        return 0.25 + 1.75 * torch.rand((1, dim), device="cuda", dtype=torch.float32, generator=g)
    raise NotImplementedError(f"unsupported --imp {kind}")


def do_bench(fn, warmup: float = 10, rep: float = 100) -> float:
    """Mean milliseconds per call; `warmup` and `rep` are time budgets in ms like triton's do_bench."""
    fn()
    torch.cuda.synchronize()
    cache = torch.empty(256 * 1024 * 1024, dtype=torch.int8, device="cuda")   # larger than the 126 MB L2
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(5):
        cache.zero_()
        fn()
    e.record()
    torch.cuda.synchronize()
    estimate = s.elapsed_time(e) / 5
    n_warmup = max(1, int(warmup / estimate))
    n_repeat = max(1, int(rep / estimate))
    for _ in range(n_warmup):
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    for i in range(n_repeat):
        cache.zero_()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in zip(starts, ends)) / n_repeat


def run_one(name: str, args, bsz_list=None) -> dict:
    props = torch.cuda.get_device_properties("cuda")
    fp8_max = 448.0 if name == "vllm" else 256.0
    result = {
        "name": f"cuda.{name}", "sm_count": props.multi_processor_count, "dim": args.dim, "scale_layout": "swizzled",
        "weight_distribution": "Normal(0, 1)",
        "environment": {"torch": torch.__version__, "gpu": props.name, "sm": props.major * 10 + props.minor},
        "results": [],
    }
    if name == "ScaleSweep":
        result.update(lower_bound=-8, upper_bound=7, imp=args.imp)
    elif name != "vllm":
        result.update(lower_bound=-3, upper_bound=7)
    for bsz in (bsz_list or BSZ_LIST):
        w = make_w(bsz, args.dim)
        gs, gs_inv = H.get_nvfp4_global_scale(w, fp8_max)
        imp = make_imp(args.imp, args.dim)
        if name == "vllm":
            fn = lambda: K.scaled_fp4_quant(w, gs_inv)
        elif name == "ScaleSweep":
            fn = lambda: K.scalesweep_weighted_mse_nvfp4_quant_impl(w, imp, gs_inv, is_sf_swizzled_layout=True)
        elif name == "ScaleSweep_MSE_round":
            fn = lambda: K.scalesweep_mse_round_nvfp4_quant_impl(w, gs_inv, is_sf_swizzled_layout=True)
        else:
            fn = lambda: K.scalesweep_mse_nvfp4_quant_impl(w, gs_inv, is_sf_swizzled_layout=True)
        ms = do_bench(fn, args.warmup, args.rep)
        code, scale = fn()
        rec = H.dequantize("base", code, K.unswizzle_vllm_fp4_scale(scale, bsz, args.dim), gs)
        mse, max_abs = H.error_stats(w, rec)
        wmse, _ = H.weighted_error_stats(w, rec, imp)
        result["results"].append({"bsz": bsz, "dim": args.dim, "latency_ms": ms, "mse": mse,
                                  "max_abs_error": max_abs, "weighted_mse": wmse,
                                  "algorithmic_GBps": bsz * (args.dim * 2 + args.dim // 2 + args.dim // 16) / ms / 1e6})
    return result


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("benchmarks", nargs="*", choices=BENCHMARKS)
    ap.add_argument("--dim", type=int, default=8192)
    ap.add_argument("--imp", choices=["ones", "ramp", "random"], default="ones")
    ap.add_argument("--output", type=Path)
    ap.add_argument("--output-dir", type=Path, default=Path("result"))
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--rep", type=int, default=100)
    args = ap.parse_args()
    if not args.benchmarks:
        args.benchmarks = BENCHMARKS
    if args.output is not None and len(args.benchmarks) != 1:
        ap.error("--output can only be used when running one benchmark")
    if not torch.cuda.is_available() or torch.cuda.get_device_capability()[0] < 10:
        raise RuntimeError("these NVFP4 kernels require an sm_100 GPU")
    for name in args.benchmarks:
        res = run_one(name, args)
        out = args.output or args.output_dir / f"bench_{name}_results.json"
        out.parent.mkdir(parents=True, exist_ok=True)
        out.write_text(json.dumps(res, indent=2) + "\n")
        print(f"saved results to {out}")


if __name__ == "__main__":
    main()
