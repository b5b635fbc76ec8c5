"""CPU: the host-side mirror of the reference's `kernels` package - names, signatures, allocation
contract and error behaviour (no kernel is launched here)."""
import inspect

import pytest
import pathlib

import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]


def test_module_surface_matches_the_reference():
    from nvfp4quant_test_b200.kernels import kernel_ScaleSweep as W
    from nvfp4quant_test_b200.kernels import kernel_ScaleSweep_MSE as M
    from nvfp4quant_test_b200.kernels import kernel_vllm as V

    assert (M.BLOCK_SIZE, M.LOWER_BOUND, M.UPPER_BOUND) == (16, -3, 7)
    assert (W.BLOCK_SIZE, W.LOWER_BOUND, W.UPPER_BOUND) == (16, -8, 7)
    sig = inspect.signature(M.scalesweep_mse_nvfp4_quant_impl)
    assert list(sig.parameters) == ["input", "input_scale", "is_sf_swizzled_layout", "padded_n"]
    sig = inspect.signature(M.scalesweep_mse_nvfp4_quant_out)
    assert list(sig.parameters) == ["input", "input_scale", "is_sf_swizzled_layout", "output", "output_scale"]
    assert sig.parameters["output"].kind is inspect.Parameter.KEYWORD_ONLY
    sig = inspect.signature(W.scalesweep_weighted_mse_nvfp4_quant_impl)
    assert list(sig.parameters) == ["input", "importance", "input_scale", "is_sf_swizzled_layout", "padded_n",
                                    "lower_bound", "upper_bound"]
    assert sig.parameters["lower_bound"].default == -8 and sig.parameters["upper_bound"].default == 7
    sig = inspect.signature(W.scalesweep_weighted_mse_nvfp4_quant_out)
    assert list(sig.parameters) == ["input", "importance", "input_scale", "is_sf_swizzled_layout", "output",
                                    "output_scale", "lower_bound", "upper_bound"]
    assert V.round_up(130, 128) == 256 and V.round_up(128, 128) == 128
    import nvfp4quant_test_b200.kernels as K

    for name in ("scalesweep_mse_round_nvfp4_quant_impl", "amax_nvfp4_quant_impl", "scaled_fp4_quant",
                 "nvfp4_scaled_mm", "cutlass_scaled_fp4_mm", "create_fp4_output_tensors"):
        assert hasattr(K, name)


def test_output_allocation_contract():
    """Shapes and dtypes of vllm's create_fp4_output_tensors (vllm/_custom_ops.py:36-86)."""
    from nvfp4quant_test_b200.kernels import create_fp4_output_tensors

    c, s = create_fp4_output_tensors(130, 208, "cpu", True)
    assert c.shape == (130, 104) and c.dtype == torch.uint8
    assert s.shape == (256, 4) and s.dtype == torch.int32          # round_up(13, 4) / 4 int32 per row
    c, s = create_fp4_output_tensors(130, 208, "cpu", True, padded_n=256)
    assert c.shape == (130, 128) and s.shape == (256, 4)
    c, s = create_fp4_output_tensors(7, 48, "cpu", False)
    assert c.shape == (7, 24) and s.shape == (7, 3) and s.dtype == torch.uint8


def test_weighted_input_checks_raise_value_error():
    """Same conditions as the reference's _check_inputs (kernels/kernel_ScaleSweep.py:419-433)."""
    from nvfp4quant_test_b200.kernels import scalesweep_weighted_mse_nvfp4_quant_impl as q

    gs = torch.ones(1)
    with pytest.raises(ValueError, match="input must be 2D"):
        q(torch.zeros(4, 4, 16), torch.ones(1, 16), gs)
    with pytest.raises(ValueError, match="divisible by 16"):
        q(torch.zeros(4, 24), torch.ones(1, 24), gs)
    with pytest.raises(ValueError, match=r"importance must have shape \[1, dim\]"):
        q(torch.zeros(4, 32), torch.ones(32), gs)
    with pytest.raises(ValueError, match=r"importance must have shape \[1, dim\]"):
        q(torch.zeros(4, 32), torch.ones(1, 16), gs)


def test_no_cpu_fallback():
    """CPU tensors are rejected: the product path has no CPU implementation."""
    import nvfp4quant_test_b200.kernels as K

    x = torch.zeros(4, 32, dtype=torch.bfloat16)
    gs = torch.ones(1)
    with pytest.raises(ValueError, match="CUDA tensor"):
        K.scalesweep_mse_nvfp4_quant_impl(x, gs)
    with pytest.raises(ValueError, match="CUDA tensor"):
        K.amax_nvfp4_quant_impl(x, gs)
    with pytest.raises(ValueError, match="CUDA tensor"):
        K.scalesweep_weighted_mse_nvfp4_quant_impl(x, torch.ones(1, 32), gs)
    with pytest.raises(ValueError, match="CUDA"):
        K.nvfp4_scaled_mm(torch.zeros(4, 32, dtype=torch.uint8), torch.zeros(4, 32, dtype=torch.uint8),
                          torch.zeros(128, 4, dtype=torch.uint8), torch.zeros(128, 4, dtype=torch.uint8),
                          torch.ones(1), torch.bfloat16)
    from nvfp4quant_test_b200 import helper as H

    with pytest.raises(ValueError, match="CUDA"):
        H.get_nvfp4_global_scale(x)


def test_product_package_never_imports_the_oracle():
    import pathlib

    pkg = pathlib.Path(__file__).resolve().parents[1] / "nvfp4quant_test_b200"
    for f in pkg.rglob("*.py"):
        text = f.read_text()
        assert "oracle" not in text.replace("the CPU oracle", ""), f"{f} mentions the oracle"
    for f in pkg.rglob("*.cu*"):
        assert "nvfp4_oracle" not in f.read_text()


def test_host_pipeline_chunk_plan():
    from nvfp4quant_test_b200.host_pipeline import chunk_plan

    assert chunk_plan(8192, 1024) == [(i * 1024, (i + 1) * 1024) for i in range(8)]
    assert chunk_plan(300, 128) == [(0, 128), (128, 256), (256, 300)]
    assert chunk_plan(1, 1024) == [(0, 1)]
    for bad in (0, 100, 129):
        with pytest.raises(ValueError):
            chunk_plan(1024, bad)


def test_llama_stack_layer_partition():
    from nvfp4quant_test_b200.llama_stack import LAYER_SHAPES, layers_for_rank, weights_per_layer

    assert weights_per_layer() == 218_103_808          # 218.1 M weights per layer, 6.98 G for 32 layers
    assert LAYER_SHAPES["down"] == (4096, 14336) and LAYER_SHAPES["k"] == (1024, 4096)
    for n_layers, world in ((32, 8), (32, 1), (32, 3), (2, 4)):
        got = [list(layers_for_rank(n_layers, r, world)) for r in range(world)]
        assert sum(got, []) == list(range(n_layers))
        assert max(map(len, got)) - min(map(len, got)) <= 1
    assert list(layers_for_rank(32, 5, 8)) == [20, 21, 22, 23]


def test_llama_stack_weight_scale_slots():
    """The alphas of a layer come from one multiplication per input width: the global scales of the matrices that
    share an input are stacked in dict order and every matrix knows its slot."""
    from nvfp4quant_test_b200.llama_stack import LAYER_SHAPES, stack_weight_scales

    qlayer = {name: (torch.empty((n, k // 2), dtype=torch.uint8), None, torch.tensor(float(i + 1)))
              for i, (name, (n, k)) in enumerate(LAYER_SHAPES.items())}
    ws = stack_weight_scales(qlayer)
    assert sorted(ws) == [4096, 14336]
    vec, slots = ws[4096]
    assert list(slots) == ["q", "k", "v", "o", "gate", "up"] and vec.tolist() == [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]
    vec, slots = ws[14336]
    assert slots == {"down": 0} and vec.tolist() == [7.0] and vec.dtype == torch.float32


def test_storage_round_trip(tmp_path):
    """codes + tiled scales + global scale survive save/load bit for bit; linear <-> tiled converters invert."""
    from nvfp4quant_test_b200 import storage

    g = torch.Generator().manual_seed(1)
    tensors = {}
    for name, (rows, cols) in {"q": (130, 208), "down": (256, 64)}.items():
        codes = torch.randint(0, 256, (rows, cols // 2), dtype=torch.uint8, generator=g)
        lin = torch.randint(0, 127, (rows, cols // 16), dtype=torch.uint8, generator=g)
        tiled = storage.as_tiled_scales(lin, rows, cols)
        tensors[name] = (codes, tiled, 0.0123 * (1 + len(name)))
    path = tmp_path / "w.nvfp4"
    storage.save(path, tensors)
    back = storage.load(path)
    for name, (codes, tiled, gs) in tensors.items():
        c2, s2, g2 = back[name]
        rows, cols = codes.shape[0], codes.shape[1] * 2
        assert torch.equal(c2, codes) and torch.equal(s2.view(torch.uint8).reshape(-1), tiled)
        assert s2.dtype == torch.float8_e4m3fn and float(g2) == float(torch.tensor(gs, dtype=torch.float32))
        assert torch.equal(storage.as_tiled_scales(storage.as_linear_scales(s2, rows, cols), rows, cols).view(torch.uint8),
                           tiled)
    with pytest.raises(ValueError):
        storage.save(tmp_path / "bad.nvfp4", {"x": (tensors["q"][0], tensors["q"][1][:10], 1.0)})
    (tmp_path / "junk").write_bytes(b"not a file of ours")
    with pytest.raises(ValueError):
        storage.load(tmp_path / "junk")


def test_report_tables():
    from nvfp4quant_test_b200.report import build_report

    def res(name, scale):
        return {"name": name, "sm_count": 148, "dim": 8192, "environment": {"torch": "2.11", "gpu": "B200"},
                "results": [{"bsz": b, "dim": 8192, "latency_ms": scale * b / 1000, "mse": 0.0066, "max_abs_error": 0.586,
                             "weighted_mse": 0.0066} for b in (1, 128, 8192)]}

    text = build_report([res("cuda.ScaleSweep_MSE", 0.0155), res("cuda.vllm", 0.005)])
    assert "| kernel | 1 | 128 | 8192 |" in text
    assert "| cuda.ScaleSweep_MSE | 1.55e-05 | 0.001984 | 0.126976 |" in text
    assert "## Quantization error at bsz = 8192" in text and "| cuda.vllm | 0.0066 | 0.0066 | 0.586 |" in text
    with pytest.raises(ValueError):
        build_report([])


def test_gemm_report_tables():
    from nvfp4quant_test_b200.report import build_gemm_report

    def row(m, n, us, bound):
        return {"M": m, "N": n, "K": 8192, "quantizer": "x", "us": us, "tflops": 2.0 * m * n * 8192 / us / 1e6,
                "weight_gbs": n * 4608 / us / 1e3, "bound": bound, "roofline_frac": 0.5, "mse": 444.2, "max_abs_error": 117.8}

    res = {"name": "cuda.gemm.ScaleSweep", "K": 8192, "peaks": {"fp4_tflops": 6770.0, "hbm_gbs": 6548.8},
           "results": [row(16, 8192, 11.0, "hbm"), row(8192, 8192, 205.0, "tensor"), row(8192, 28672, 710.0, "tensor")]}
    text = build_gemm_report([res])
    assert "| quantizer | 16x8192 | 8192x8192 | 8192x28672 |" in text
    assert "GB/s (50 %)" in text and "TF (50 %)" in text
    assert "M = 8192, N = 28672" in text and "| cuda.gemm.ScaleSweep | 444.2 | 117.8 |" in text
    assert build_gemm_report([]) == ""


def test_stream_scratch_is_bounded():
    from nvfp4quant_test_b200._lib import StreamScratch

    sc = StreamScratch(2, capacity=4)
    dev = torch.device("cpu")
    first = sc.get(dev, 100)
    assert first.dtype == torch.int32 and first.numel() == 2 and int(first.abs().sum()) == 0
    assert sc.get(dev, 100) is first                  # same stream: same buffer
    for s in range(101, 110):
        sc.get(dev, s)
    assert len(sc) == 4                               # older streams were dropped
    assert sc.get(dev, 100) is not first              # ... including the first one, which gets a fresh buffer
    assert sc.get(dev, 109) is sc.get(dev, 109)


def test_bench_reference_arm_prints_one_schema_complete_line():
    """`bench.py --impl reference` (the CPU port on all host threads over the full 8192 rows) prints exactly one JSON
    line with the keys of the benchmark contract."""
    import json
    import subprocess
    import sys

    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "GB/s" and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert d["config"]["rows_per_gpu"] == 8192 and "configs[1]" in d["config"]["workload"]
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0 and d["steps"] == 1 and 0.01 < d["value"] < 50.0


def test_capture_id_is_zero_without_a_capture():
    from nvfp4quant_test_b200 import _lib

    assert _lib.capture_id(0) == 0          # no GPU, or the default stream outside a capture
