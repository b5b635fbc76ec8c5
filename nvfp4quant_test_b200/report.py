"""Markdown report from the JSON files `sweep.py` writes: one latency table (kernel x bsz) and one error table at
the largest bsz, in the layout of the tables the reference publishes (README.md:44-63 of efsotr/nvfp4quant_test).

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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("result_dir", type=Path)
    ap.add_argument("-o", "--output", type=Path)
    args = ap.parse_args()
    results = [json.loads(p.read_text()) for p in sorted(args.result_dir.glob("bench_*_results.json"))]
    text = build_report(results)
    out = args.output or args.result_dir / "benchmark_report.md"
    out.write_text(text)
    print(f"wrote {out}")


if __name__ == "__main__":
    main()
