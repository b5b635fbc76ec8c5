"""Markdown report from the JSON files `sweep.py` and `gemm_sweep.py` write: the quantization latency table
(kernel x bsz) and error table at the largest bsz, then the GEMM latency / throughput / error tables, in the layout
of the tables the reference publishes (README.md:44-75 of efsotr/nvfp4quant_test; its make_markdown.py:193-212
assembles the same sections).

  python -m nvfp4quant_test_b200.report result/ [-o result/benchmark_report.md]
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path


def _fmt(x) -> str:
    return "-" if x is None else f"{x:.6g}"


def build_report(results: list[dict]) -> str:
    if not results:
        raise ValueError("no result files")
    bszs = sorted({r["bsz"] for res in results for r in res["results"]})
    env = results[0].get("environment", {})
    lines = ["# NVFP4 quantization benchmark report", "", "## Environment", "",
             "| " + " | ".join(env) + " | sm_count |", "| " + " | ".join("---" for _ in range(len(env) + 1)) + " |",
             "| " + " | ".join(str(v) for v in env.values()) + f" | {results[0].get('sm_count')} |", "",
             f"## Quantization latency (ms), dim = {results[0]['dim']}", "",
             "| kernel | " + " | ".join(str(b) for b in bszs) + " |", "| --- | " + " | ".join("---" for _ in bszs) + " |"]
    for res in results:
        by = {r["bsz"]: r for r in res["results"]}
        lines.append(f"| {res['name']} | " + " | ".join(_fmt(by[b]["latency_ms"]) if b in by else "-" for b in bszs) + " |")
    top = bszs[-1]
    lines += ["", f"## Quantization error at bsz = {top}", "", "| kernel | mse | weighted_mse | max_abs_error |",
              "| --- | --- | --- | --- |"]
    for res in results:
        r = {x["bsz"]: x for x in res["results"]}.get(top)
        if r:
            lines.append(f"| {res['name']} | {_fmt(r['mse'])} | {_fmt(r.get('weighted_mse'))} | {_fmt(r['max_abs_error'])} |")
    return "\n".join(lines) + "\n"


def build_gemm_report(results: list[dict]) -> str:
    """GEMM sections: microseconds per (M, N) and quantizer, achieved TFLOP/s or weight GB/s with the roofline
    fraction, and the output error table (README.md:66-75 of the reference prints the error table)."""
    if not results:
        return ""
    shapes = sorted({(r["N"], r["M"]) for res in results for r in res["results"]})
    head = " | ".join(f"{m}x{n}" for n, m in shapes)
    sep = " | ".join("---" for _ in shapes)
    peaks = results[0].get("peaks", {})
    lines = ["", f"## NVFP4 GEMM latency (us), K = {results[0]['K']}, M x N", "", f"| quantizer | {head} |", f"| --- | {sep} |"]
    for res in results:
        by = {(r["N"], r["M"]): r for r in res["results"]}
        lines.append(f"| {res['name']} | " + " | ".join(_fmt(by[s]["us"]) if s in by else "-" for s in shapes) + " |")
    lines += ["", "## NVFP4 GEMM throughput (TFLOP/s where the tensor pipe bounds, weight GB/s where HBM does; fraction of the measured peak)",
              "", f"measured peaks: FP4 tensor pipe {_fmt(peaks.get('fp4_tflops'))} TFLOP/s sustained, HBM {_fmt(peaks.get('hbm_gbs'))} GB/s",
              "", f"| quantizer | {head} |", f"| --- | {sep} |"]
    for res in results:
        by = {(r["N"], r["M"]): r for r in res["results"]}
        cells = []
        for s in shapes:
            r = by.get(s)
            if r is None:
                cells.append("-")
            elif r["bound"] == "hbm":
                cells.append(f"{r['weight_gbs']:.0f} GB/s ({100 * r['roofline_frac']:.0f} %)")
            else:
                cells.append(f"{r['tflops']:.0f} TF ({100 * r['roofline_frac']:.0f} %)")
        lines.append(f"| {res['name']} | " + " | ".join(cells) + " |")
    top = max(shapes, key=lambda s: (s[1], s[0]))
    lines += ["", f"## NVFP4 GEMM error at M = {top[1]}, N = {top[0]} (against the fp32 product of the bf16 operands)", "",
              "| quantizer | mse | max_abs_error |", "| --- | --- | --- |"]
    for res in results:
        r = {(x["N"], x["M"]): x for x in res["results"]}.get(top)
        if r:
            lines.append(f"| {res['name']} | {_fmt(r['mse'])} | {_fmt(r['max_abs_error'])} |")
    return "\n".join(lines) + "\n"


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("result_dir", type=Path)
    ap.add_argument("-o", "--output", type=Path)
    args = ap.parse_args()
    results = [json.loads(p.read_text()) for p in sorted(args.result_dir.glob("bench_*_results.json"))]
    gemm = [json.loads(p.read_text()) for p in sorted(args.result_dir.glob("gemm_*_results.json"))]
    text = (build_report(results) if results else "# NVFP4 benchmark report\n") + build_gemm_report(gemm)
    out = args.output or args.result_dir / "benchmark_report.md"
    out.write_text(text)
    print(f"wrote {out}")


if __name__ == "__main__":
    main()
