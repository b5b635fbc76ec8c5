"""CPU: the oracle against outputs of the reference itself (Triton kernels / vllm ops run on a B200)."""
import numpy as np

import cases as C
import util


def _gs_inv(info):
    return float(np.array([info["gs_inv_bits"]], dtype=np.int32).view(np.float32)[0])


def test_oracle_reproduces_reference_scalesweep_bytes(oracle, golden):
    meta, arrays = golden
    assert oracle.div_full_table_is_measured()
    cs = C.build_cases()
    checked = 0
    for name, info in meta["cases"].items():
        c = cs[name]
        if c["variant"] == "amax":
            continue
        assert C.sha(c["x"]) == info["x_sha256"], f"{name}: seeded input differs from the one the fixture was made with"
        codes, scales = util.oracle_quant_case(oracle, c, _gs_inv(info))
        m, n = c["x"].shape
        blocks = (c["padded_n"] or n) // 16
        idx = util.logical_scale_index(m, blocks, c["swizzled"])
        assert np.array_equal(codes, arrays[name + ".codes"]), name
        assert np.array_equal(scales[idx], arrays[name + ".scales"].reshape(-1)[idx]), name
        checked += 1
    assert checked >= 19


def test_global_scale_formula_matches_reference(golden):
    """helper.py:96-100 evaluated by torch on the GPU == the fp32 formula the CUDA kernel and the tests use."""
    meta, _ = golden
    cs = C.build_cases()
    for name, info in meta["cases"].items():
        c = cs[name]
        if c["gs_inv"] is not None:
            continue
        gs, gs_inv = C.global_scale_cpu(c["x"], c["fp8_max"])
        assert np.float32(gs).view(np.int32) == info["gs_bits"], name
        assert np.float32(gs_inv).view(np.int32) == info["gs_inv_bits"], name


def test_oracle_amax_close_to_vllm_op(oracle, golden):
    """The vllm op uses rcp.approx.ftz for its two reciprocals; with IEEE division on the CPU the scale
    bytes must still agree exactly and codes may differ by one grid step in a handful of elements."""
    meta, arrays = golden
    cs = C.build_cases()
    for name, info in meta["cases"].items():
        c = cs[name]
        if c["variant"] != "amax":
            continue
        codes, scales = util.oracle_quant_case(oracle, c, _gs_inv(info))
        m, n = c["x"].shape
        idx = util.logical_scale_index(m, n // 16, c["swizzled"])
        assert np.array_equal(scales[idx], arrays[name + ".scales"].reshape(-1)[idx]), name
        ref = arrays[name + ".codes"]
        bad = codes != ref
        assert bad.mean() < 2e-3, (name, bad.mean())
        lo = np.abs((codes & 7).astype(int) - (ref & 7).astype(int))
        hi = np.abs(((codes >> 4) & 7).astype(int) - ((ref >> 4) & 7).astype(int))
        assert lo.max() <= 1 and hi.max() <= 1, name


def test_oracle_gemm_close_to_cutlass(oracle, golden):
    """fp64 dot products rounded to bf16 vs cutlass_scaled_fp4_mm (fp32 accumulation): <= 1 bf16 ulp apart."""
    import torch

    meta, arrays = golden
    assert meta["gemm"], "fixture holds no GEMM case"
    for name, info in meta["gemm"].items():
        alpha = float(np.array([info["alpha_bits"]], dtype=np.int32).view(np.float32)[0])
        ref = oracle.gemm(arrays[name + ".qa"], arrays[name + ".qb"], arrays[name + ".sa"].reshape(-1),
                          arrays[name + ".sb"].reshape(-1), alpha)
        got = torch.from_numpy(arrays[name + ".out_bf16_bits"]).view(torch.bfloat16).float().numpy()
        want = torch.from_numpy(ref).to(torch.bfloat16).float().numpy()
        tol = np.maximum(np.abs(ref) * 2.0 ** -7, np.abs(ref).max() * 2.0 ** -16)
        assert (np.abs(got - ref) <= tol).all(), name
        assert (got == want).mean() > 0.97, (name, (got == want).mean())
