"""GPU: the two sweep drivers (quantization latency / error, GEMM latency / throughput / error) on a small subset,
checking the JSON schema the report generator consumes and the error values against known ranges."""
import argparse

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_quantization_sweep_rows(cuda_lib):
    from nvfp4quant_test_b200 import report, sweep

    args = argparse.Namespace(dim=2048, imp="ramp", warmup=1, rep=3)
    results = []
    for name in sweep.BENCHMARKS:
        res = sweep.run_one(name, args, bsz_list=[8, 256])
        results.append(res)
        assert res["name"] == f"cuda.{name}" and res["dim"] == 2048 and res["scale_layout"] == "swizzled"
        assert [r["bsz"] for r in res["results"]] == [8, 256]
        for r in res["results"]:
            assert set(r) >= {"bsz", "dim", "latency_ms", "mse", "max_abs_error", "weighted_mse", "algorithmic_GBps"}
            assert 0.0 < r["latency_ms"] < 5.0
            # N(0,1) inputs: the sweeps reach ~0.0066, the amax baseline ~0.009 (same bytes as the reference kernels)
            lo, hi = (0.0075, 0.0105) if name == "vllm" else (0.0055, 0.0078)
            assert lo < r["mse"] < hi, (name, r)
    by = {r["name"]: r["results"][1] for r in results}
    assert by["cuda.ScaleSweep_MSE"]["mse"] == by["cuda.ScaleSweep_MSE_round"]["mse"]
    assert by["cuda.ScaleSweep"]["weighted_mse"] <= by["cuda.ScaleSweep_MSE"]["weighted_mse"] * (1 + 1e-6)
    text = report.build_report(results)
    assert "| cuda.ScaleSweep_MSE |" in text and "bsz = 256" in text


def test_gemm_sweep_rows(cuda_lib):
    from nvfp4quant_test_b200 import gemm_sweep, report

    peaks = gemm_sweep.measured_peaks()
    assert 3000.0 < peaks["fp4_tflops"] <= peaks["fp4_burst_tflops"] * 1.05 < 12000.0
    results = [gemm_sweep.run_one(name, [16, 256], [1024], 2048, peaks) for name in gemm_sweep.QUANTIZERS]
    for res in results:
        assert [(r["M"], r["N"]) for r in res["results"]] == [(16, 1024), (256, 1024)]
        for r in res["results"]:
            assert set(r) >= {"M", "N", "K", "quantizer", "us", "tflops", "weight_gbs", "bound", "roofline_frac",
                              "mse", "max_abs_error"}
            assert r["status"] == 0 and 0.0 < r["us"] < 1000.0 and 0.0 < r["roofline_frac"] < 1.2
            assert r["bound"] == ("hbm" if r["M"] <= 128 else "tensor")
            # Laplace(0,1) operands, K = 2048: output variance 4 K = 8192; NVFP4 on both operands leaves ~1-2 % of it
            assert 20.0 < r["mse"] < 400.0 and r["max_abs_error"] < 150.0, r
    by = {res["name"]: res["results"][1]["mse"] for res in results}
    assert by["cuda.gemm.ScaleSweep_MSE"] < by["cuda.gemm.vllm"]        # the sweep beats the amax baseline (README.md:70-75)
    assert by["cuda.gemm.ScaleSweep_MSE"] == by["cuda.gemm.ScaleSweep_MSE_round"]
    text = report.build_gemm_report(results)
    assert "| cuda.gemm.ScaleSweep |" in text and "M = 256, N = 1024" in text
