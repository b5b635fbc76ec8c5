"""NVFP4 GEMM sweep: latency, throughput and output error for operands produced by each quantizer.

The reference's README describes this experiment (README.md:11,66-75 of efsotr/nvfp4quant_test: activation and
weight ~ Laplace(0, 1); the importance of one operand's input channels is the other operand's per-channel squared
norm; `cutlass_scaled_fp4_mm` on the quantized operands; mse / max_abs_error against the unquantized product) but
its driver script is not part of the published sources.  This module is that driver for the kernels of this
package, with the command-line style of the reference's bench.py (bench.py:35-49):

  python -m nvfp4quant_test_b200.gemm_sweep [vllm] [ScaleSweep_MSE] [ScaleSweep_MSE_round] [ScaleSweep] \
         [--k 8192] [--m 1 16 128 2048 8192] [--n 8192 28672] [--output-dir result]

Per (quantizer, M, N): both operands are quantized (ScaleSweep: importance-weighted, each with the other's channel
square norms; the others unweighted / amax), alpha = global_scale_a * global_scale_b, then the GEMM is replayed from
a CUDA graph over copies of the weight that rotate through more memory than the L2 holds, so that small-M rows
measure weight streaming from HBM.  Rows of the JSON: M, N, K, quantizer, us, tflops, weight_gbs, bound
("tensor" | "hbm"), roofline_frac (of the measured FP4 tensor-pipe rate or of the measured HBM copy rate), mse and
max_abs_error against the fp32 product of the unquantized bf16 operands.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from . import benchtools as B
from . import helper as H
from . import kernels as K

QUANTIZERS = ["vllm", "ScaleSweep_MSE", "ScaleSweep_MSE_round", "ScaleSweep"]
M_LIST = [1, 16, 128, 2048, 8192]
N_LIST = [8192, 28672]
L2_BYTES = 126 * 1024 * 1024
HBM_FALLBACK_GBS = 6650.0


def laplace(shape, seed: int, device="cuda") -> torch.Tensor:
    """Laplace(0, 1) bf16 by inverse CDF from a seeded uniform (CUDA generator)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    u = torch.rand(shape, generator=g, device=device, dtype=torch.float32) - 0.5
    # rand() can return exactly 0, i.e. |u| = 0.5 and an infinite sample: keep |u| one fp32 step inside
    mag = torch.clamp(u.abs(), max=0.5 - 2.0 ** -25)
    return (-torch.sign(u) * torch.log1p(-2.0 * mag)).to(torch.bfloat16)


def quantize_operand(name: str, x: torch.Tensor, other: torch.Tensor):
    """(codes, tiled scales, global_scale) of x with quantizer `name`; `other` is the operand x is multiplied with."""
    fp8_max = 448.0 if name == "vllm" else 256.0
    gs, gs_inv = H.get_nvfp4_global_scale(x, fp8_max)
    if name == "vllm":
        q, s = K.scaled_fp4_quant(x, gs_inv)
    elif name == "ScaleSweep":
        q, s = K.scalesweep_weighted_mse_nvfp4_quant_impl(x, H.channel_square_norm(other), gs_inv)
    elif name == "ScaleSweep_MSE_round":
        q, s = K.scalesweep_mse_round_nvfp4_quant_impl(x, gs_inv)
    else:
        q, s = K.scalesweep_mse_nvfp4_quant_impl(x, gs_inv)
    return q, s, gs


def output_error(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, chunk: int = 1024):
    """(mse, max_abs_error) of `out` against a.float() @ w.float().T, evaluated in row chunks."""
    wf = w.float()
    se, mx, n = 0.0, 0.0, 0
    for i in range(0, a.shape[0], chunk):
        ref = a[i:i + chunk].float() @ wf.T
        d = out[i:i + chunk].float() - ref
        se += float((d * d).sum())
        mx = max(mx, float(d.abs().max()))
        n += d.numel()
    return se / n, mx


def measure(name: str, m: int, n: int, k: int, peaks: dict, replays: int = 10) -> dict:
    a = laplace((m, k), 1)
    w = laplace((n, k), 0)
    qa, sa, gsa = quantize_operand(name, a, w)
    qw, sw, gsw = quantize_operand(name, w, a)
    alpha = (gsa * gsw).reshape(1).float()
    wbytes = qw.numel() + sw.numel()
    copies = max(2, -(-2 * L2_BYTES // wbytes))        # the rotation covers at least twice the L2
    qws = [qw] + [qw.clone() for _ in range(copies - 1)]
    sws = [sw] + [sw.clone() for _ in range(copies - 1)]
    out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)

    pws = [K.PreparedWeight(qws[i], sws[i]) for i in range(copies)]   # as a serving stack holds its weights

    def record():
        for i in range(copies):
            K.nvfp4_scaled_mm_prepared(qa, sa, alpha, pws[i], out=out)

    us = B.time_graph(record, copies, replays)
    mse, max_abs = output_error(out, a, w)
    tflops = 2.0 * m * n * k / (us * 1e-6) / 1e12
    gbs = wbytes / (us * 1e-6) / 1e9
    bound = "hbm" if m <= 128 else "tensor"
    frac = gbs / peaks["hbm_gbs"] if bound == "hbm" else tflops / peaks["fp4_tflops"]
    return {"M": m, "N": n, "K": k, "quantizer": name, "us": us, "tflops": tflops, "weight_gbs": gbs, "bound": bound,
            "roofline_frac": frac, "mse": mse, "max_abs_error": max_abs, "weight_copies": copies,
            "status": K.kernel_gemm.gemm_last_status(a.device)}


def measured_peaks() -> dict:
    """FP4 tensor-pipe rate from the probe kernel (sustained figure) and the HBM copy rate from MEASURED_PEAKS.json
    at the repository root when that file exists, else a stated fallback."""
    fp4 = B.fp4_peak()
    hbm, src = HBM_FALLBACK_GBS, "fallback 6650 GB/s"
    p = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if p.exists():
        hbm, src = float(json.loads(p.read_text())["hbm_gbs"]), "MEASURED_PEAKS.json"
    return {"fp4_tflops": fp4["sustained_tflops"], "fp4_burst_tflops": fp4["burst_tflops"], "hbm_gbs": hbm,
            "hbm_source": src}


def run_one(name: str, m_list, n_list, k: int, peaks: dict | None = None) -> dict:
    props = torch.cuda.get_device_properties("cuda")
    peaks = peaks or measured_peaks()
    res = {"name": f"cuda.gemm.{name}", "sm_count": props.multi_processor_count, "K": k,
           "operand_distribution": "Laplace(0, 1)", "peaks": peaks,
           "environment": {"torch": torch.__version__, "gpu": props.name, "sm": props.major * 10 + props.minor},
           "results": []}
    for n in n_list:
        for m in m_list:
            res["results"].append(measure(name, m, n, k, peaks))
            torch.cuda.empty_cache()
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("quantizers", nargs="*", choices=QUANTIZERS)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--m", type=int, nargs="*", default=M_LIST)
    ap.add_argument("--n", type=int, nargs="*", default=N_LIST)
    ap.add_argument("--output-dir", type=Path, default=Path("result"))
    args = ap.parse_args()
    if not torch.cuda.is_available() or torch.cuda.get_device_capability()[0] < 10:
        raise RuntimeError("these NVFP4 kernels require an sm_100 GPU")
    peaks = measured_peaks()
    for name in args.quantizers or QUANTIZERS:
        res = run_one(name, args.m, args.n, args.k, peaks)
        out = args.output_dir / f"gemm_{name}_results.json"
        out.parent.mkdir(parents=True, exist_ok=True)
        out.write_text(json.dumps(res, indent=2) + "\n")
        print(f"saved results to {out}")


if __name__ == "__main__":
    main()
