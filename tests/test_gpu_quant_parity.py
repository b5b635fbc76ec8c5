"""GPU: the CUDA quantizers, called through the C ABI, against the CPU oracle and the reference fixtures.
Bit-exact: every code byte and every logical scale byte must match."""
import numpy as np
import pytest
import torch

import cases as C
import util

pytestmark = pytest.mark.gpu


def _amax_table(probe_lib, gs_inv: float):
    from nvfp4quant_test_b200 import _lib

    g = torch.tensor([gs_inv], dtype=torch.float32, device="cuda")
    t = torch.zeros(128, dtype=torch.float32, device="cuda")
    _lib.check(probe_lib.nvfp4_probe_amax_out_scale_table(g.data_ptr(), t.data_ptr(), None), "probe")
    torch.cuda.synchronize()
    return t.cpu().numpy()


def _run_cuda(c, gs_inv: float, impl: int = 0, fill: int = 0xA5):
    """Call nvfp4_quant_launch_impl on canary-filled buffers; returns (codes, scale bytes, canaries intact)."""
    from nvfp4quant_test_b200 import _lib

    L = _lib.lib()
    x = c["x"].cuda()
    m, n = x.shape
    P = c["padded_n"] or n
    blocks = P // 16
    sc_bytes = ((m + 127) // 128 * 128) * ((blocks + 3) // 4 * 4) if c["swizzled"] else m * blocks
    guard = 256
    codes = torch.full((m * P // 2 + 2 * guard,), fill, dtype=torch.uint8, device="cuda")
    scales = torch.full((sc_bytes + 2 * guard,), fill, dtype=torch.uint8, device="cuda")
    g = torch.tensor([gs_inv], dtype=torch.float32, device="cuda")
    imp = c["importance"].cuda().contiguous() if c["importance"] is not None else None
    lo, up = util.window(c)
    st = L.nvfp4_quant_launch_impl(impl, util.VARIANT[c["variant"]], x.data_ptr(), _lib.dtype_code(x.dtype),
                                   imp.data_ptr() if imp is not None else None, g.data_ptr(),
                                   codes.data_ptr() + guard, scales.data_ptr() + guard, m, n, P, lo, up,
                                   int(c["swizzled"]), torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "nvfp4_quant_launch_impl")
    torch.cuda.synchronize()
    ch, sh = codes.cpu().numpy(), scales.cpu().numpy()
    intact = bool((ch[:guard] == fill).all() and (ch[-guard:] == fill).all() and (sh[:guard] == fill).all()
                  and (sh[-guard:] == fill).all())
    return ch[guard:-guard].reshape(m, P // 2), sh[guard:-guard], intact


@pytest.mark.parametrize("name", sorted(C.build_cases()))
def test_cuda_matches_oracle_bit_for_bit(cuda_lib, probe_lib, oracle, name):
    c = C.build_cases()[name]
    gs_inv = c["gs_inv"] if c["gs_inv"] is not None else C.global_scale_cpu(c["x"], c["fp8_max"])[1]
    table = _amax_table(probe_lib, gs_inv) if c["variant"] == "amax" else None
    want_codes, want_scales = util.oracle_quant_case(oracle, c, gs_inv, table)
    m, n = c["x"].shape
    blocks = (c["padded_n"] or n) // 16
    idx = util.logical_scale_index(m, blocks, c["swizzled"])
    pad = np.ones(want_scales.size, dtype=bool)
    pad[idx] = False
    for impl in (0, 1, 2, 3, 5, 6, 7, 9):
        codes, scales, intact = _run_cuda(c, gs_inv, impl)
        assert intact, f"impl {impl} wrote outside its buffers"
        assert np.array_equal(codes, want_codes), f"impl {impl}: {(codes != want_codes).sum()} code bytes differ"
        assert np.array_equal(scales[idx], want_scales[idx]), f"impl {impl}: scale bytes differ"
        assert (scales[pad] == 0).all(), f"impl {impl}: scale padding must be zero"


def test_cuda_matches_reference_fixtures(cuda_lib, golden):
    """Against bytes the reference's Triton kernels / vllm's op produced on a B200."""
    meta, arrays = golden
    cs = C.build_cases()
    for name, info in meta["cases"].items():
        c = cs[name]
        gs_inv = float(np.array([info["gs_inv_bits"]], dtype=np.int32).view(np.float32)[0])
        codes, scales, intact = _run_cuda(c, gs_inv)
        m, n = c["x"].shape
        idx = util.logical_scale_index(m, (c["padded_n"] or n) // 16, c["swizzled"])
        assert intact
        assert np.array_equal(scales[idx], arrays[name + ".scales"].reshape(-1)[idx]), name
        assert np.array_equal(codes, arrays[name + ".codes"]), (name, int((codes != arrays[name + ".codes"]).sum()))


@pytest.mark.parametrize("m", [1, 2, 127, 128, 129])
@pytest.mark.parametrize("n", [16, 48, 64, 8192])
@pytest.mark.parametrize("swizzled", [True, False])
def test_edge_shapes(cuda_lib, oracle, m, n, swizzled):
    x = C._gauss((m, n), 1000 + m + n)
    gs_inv = C.global_scale_cpu(x, 256.0)[1]
    for variant, imp in (("mse", None), ("weighted", C._importance("random", n))):
        c = dict(x=x, variant=variant, importance=imp, swizzled=swizzled, padded_n=None, lower=None, upper=None)
        want_codes, want_scales = util.oracle_quant_case(oracle, c, gs_inv)
        codes, scales, intact = _run_cuda(c, gs_inv)
        idx = util.logical_scale_index(m, n // 16, swizzled)
        assert intact and np.array_equal(codes, want_codes) and np.array_equal(scales[idx], want_scales[idx])


def test_python_entry_points_and_layouts(cuda_lib, oracle):
    """The reference-facing functions: _impl allocates, _out writes in place, int32- or uint8-typed scale
    buffers, padded_n, non-contiguous input, linear layout, and swizzle(linear) == swizzled output."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H

    x = C._laplace((200, 400), 5).cuda()[:, :384]                       # non-contiguous view, n = 384
    assert not x.is_contiguous()
    gs, gs_inv = H.get_nvfp4_global_scale(x, 256.0)
    codes, scales = K.scalesweep_mse_nvfp4_quant_impl(x, gs_inv)
    assert codes.shape == (200, 192) and scales.dtype == torch.float8_e4m3fn and scales.numel() == 256 * 24
    lin_codes, lin_scales = K.scalesweep_mse_nvfp4_quant_impl(x, gs_inv, False)
    assert torch.equal(codes, lin_codes) and lin_scales.shape == (200, 24)
    assert torch.equal(K.unswizzle_vllm_fp4_scale(scales, 200, 384).view(torch.uint8), lin_scales.view(torch.uint8))
    assert torch.equal(K.swizzle_vllm_fp4_scale(lin_scales, 200, 384).view(torch.uint8),
                       scales.view(torch.uint8).reshape(-1))
    want_codes, want_scales = oracle.quant(0, oracle.bf16_bits(x.contiguous().cpu()), float(gs_inv), swizzled=False)
    assert np.array_equal(lin_codes.cpu().numpy(), want_codes)
    assert np.array_equal(lin_scales.view(torch.uint8).cpu().numpy(), want_scales)
    # _out with a uint8-typed scale buffer and K padding
    out = torch.empty((200, 256), dtype=torch.uint8, device="cuda")
    out_scale = torch.empty((256, 32), dtype=torch.uint8, device="cuda")
    K.scalesweep_mse_nvfp4_quant_out(x, gs_inv, True, output=out, output_scale=out_scale)
    assert torch.equal(out[:, :192], codes) and bool((out[:, 192:] == 0).all())
    pc, ps = K.scalesweep_mse_nvfp4_quant_impl(x, gs_inv, True, padded_n=512)
    assert torch.equal(pc, out) and torch.equal(ps.view(torch.uint8).reshape(-1), out_scale.reshape(-1))
    # ScaleSweep_MSE_round is the same function; weighted with unit importance picks equal-or-better scales
    rc, rs = K.scalesweep_mse_round_nvfp4_quant_impl(x, gs_inv)
    assert torch.equal(rc, codes) and torch.equal(rs.view(torch.uint8), scales.view(torch.uint8))
    imp = torch.ones((1, 384), device="cuda")
    wc, ws = K.scalesweep_weighted_mse_nvfp4_quant_impl(x, imp, gs_inv)
    deq_m = H.dequantize_base(codes, K.unswizzle_vllm_fp4_scale(scales, 200, 384), gs)
    deq_w = H.dequantize_base(wc, K.unswizzle_vllm_fp4_scale(ws, 200, 384), gs)
    assert H.error_stats(x, deq_w)[0] <= H.error_stats(x, deq_m)[0] * (1 + 1e-6)
    # amax entry point with vllm's signature flattens leading dimensions
    ac, a_s = K.scaled_fp4_quant(x.reshape(2, 100, 384), gs_inv)
    assert ac.shape == (200, 192)
    with pytest.raises(ValueError):
        K.scalesweep_mse_nvfp4_quant_out(x, gs_inv, True, output=out[:, :100], output_scale=out_scale)
    with pytest.raises(ValueError):
        K.scalesweep_mse_nvfp4_quant_out(x, gs_inv, True, output=out, output_scale=out_scale[:10])


def test_full_size_8192_matches_oracle_and_properties(cuda_lib, oracle):
    """The benchmark's workload (8192 x 8192 bf16): whole-tensor bit comparison with the oracle, plus the
    size-independent properties: row independence (any row subset quantizes to the same bytes) and a
    checksum that does not depend on how rows are split."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H

    g = torch.Generator(device="cuda")
    g.manual_seed(0)
    x = torch.normal(0.0, 1.0, size=(8192, 8192), generator=g, device="cuda", dtype=torch.bfloat16)
    gs, gs_inv = H.get_nvfp4_global_scale(x, 256.0)
    assert float(gs_inv) == C.global_scale_cpu(x.cpu(), 256.0)[1]
    codes, scales = K.scalesweep_mse_nvfp4_quant_impl(x, gs_inv)
    want_codes, want_scales = oracle.quant(0, oracle.bf16_bits(x.cpu()), float(gs_inv), nthreads=0)
    assert np.array_equal(codes.cpu().numpy(), want_codes)
    assert np.array_equal(scales.view(torch.uint8).cpu().numpy().reshape(-1), want_scales.reshape(-1))
    # row independence: rows 4096..4223 alone give the same bytes as inside the full tensor
    sub_c, sub_s = K.scalesweep_mse_nvfp4_quant_impl(x[4096:4224], gs_inv)
    assert torch.equal(sub_c, codes[4096:4224])
    full_sc = scales.view(torch.uint8).reshape(-1)
    assert torch.equal(sub_s.view(torch.uint8).reshape(-1), full_sc[4096 * 512:4224 * 512])
    # shard-and-concatenate checksum (the multi-GPU partitioning rule) equals the whole
    from nvfp4quant_test_b200.sharding import row_shards, scale_slab

    total = 0
    for a, b in row_shards(8192, 8):
        c_, s_ = K.scalesweep_mse_nvfp4_quant_impl(x[a:b], gs_inv)
        lo, hi = scale_slab(a, b, 512)
        assert torch.equal(s_.view(torch.uint8).reshape(-1), full_sc[lo:hi])
        total += int(c_.long().sum())
    assert total == int(codes.long().sum())
    # quality: ScaleSweep's reconstruction error is below the amax baseline's on the same data
    deq = H.dequantize_base(codes, K.unswizzle_vllm_fp4_scale(scales, 8192, 8192), gs)
    mse, _ = H.error_stats(x, deq)
    gs4, gs4_inv = H.get_nvfp4_global_scale(x, 448.0)
    ac, a_s = K.amax_nvfp4_quant_impl(x, gs4_inv)
    mse_amax, _ = H.error_stats(x, H.dequantize_base(ac, K.unswizzle_vllm_fp4_scale(a_s, 8192, 8192), gs4))
    assert 0.0060 < mse < 0.0072 and 0.0085 < mse_amax < 0.0096


def test_weighted_full_size_rows_sample(cuda_lib, oracle):
    """Config 3 shape: [8192, 8192] Laplace weight, importance = channel square norms of a Laplace batch."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H

    w = torch.distributions.Laplace(0.0, 1.0).sample((2048, 8192)).bfloat16().cuda()
    act = torch.distributions.Laplace(0.0, 1.0).sample((512, 8192)).bfloat16().cuda()
    imp = (act.float() ** 2).sum(0, keepdim=True)
    gs, gs_inv = H.get_nvfp4_global_scale(w, 256.0)
    codes, scales = K.scalesweep_weighted_mse_nvfp4_quant_impl(w, imp, gs_inv)
    want_codes, want_scales = oracle.quant(1, oracle.bf16_bits(w.cpu()), float(gs_inv), imp.cpu().numpy(),
                                           lower=-8, upper=7)
    assert np.array_equal(codes.cpu().numpy(), want_codes)
    assert np.array_equal(scales.view(torch.uint8).cpu().numpy().reshape(-1), want_scales.reshape(-1))


def test_global_scale_kernel(cuda_lib):
    from nvfp4quant_test_b200 import helper as H

    for shape, dt in (((128, 8192), torch.bfloat16), ((33, 64), torch.float16), ((16, 128), torch.float32),
                      ((1, 7), torch.bfloat16), ((1000, 1001), torch.bfloat16), ((3000, 4096), torch.float32)):
        x = C._gauss(shape, 11, dt).cuda()
        for fm in (448.0, 256.0):
            for _ in range(2):   # the scratch words must come back to zero between calls
                gs, gs_inv = H.get_nvfp4_global_scale(x, fm)
                cg, cgi = C.global_scale_cpu(x.cpu(), fm)
                assert float(gs) == cg and float(gs_inv) == cgi
                ref = x.abs().max().float() / (6.0 * fm)          # helper.py:96-100 as torch runs it on CUDA
                assert bool(gs == ref) and bool(gs_inv == ref.reciprocal())
    x = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    x[3, 3] = float("nan")
    gs, _ = H.get_nvfp4_global_scale(x)
    assert torch.isnan(gs)


def test_div_full_table_matches_oracle(cuda_lib, probe_lib, oracle):
    """The table the oracle uses for 1/scale is what this GPU's div.full.f32 returns."""
    from nvfp4quant_test_b200 import _lib

    t = torch.zeros(128, dtype=torch.int32, device="cuda")
    _lib.check(probe_lib.nvfp4_probe_div_full_table(t.data_ptr(), None), "probe")
    torch.cuda.synchronize()
    bits = t.cpu().numpy().view(np.uint32)
    for raw in range(1, 127):
        assert int(bits[raw]) == oracle.lib().nvfp4_oracle_div_full_bits(raw), raw


@pytest.mark.parametrize("rows,dim,chunk", [(1000, 512, 256), (4096, 2048, 1024), (130, 64, 128)])
def test_host_pipeline_equals_single_launch(cuda_lib, rows, dim, chunk):
    """Pinned-host in / pinned-host out with chunked, stream-overlapped copies == one launch on the whole tensor."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H
    from nvfp4quant_test_b200.host_pipeline import HostQuantizer

    x_host = C._gauss((rows, dim), 300 + rows).pin_memory()
    x = x_host.cuda()
    gs, gs_inv = H.get_nvfp4_global_scale(x, 256.0)
    want_codes, want_scales = K.scalesweep_mse_nvfp4_quant_impl(x, gs_inv)
    codes_host = torch.zeros((rows, dim // 2), dtype=torch.uint8).pin_memory()
    scales_host = torch.zeros(want_scales.numel(), dtype=torch.uint8).pin_memory()
    hq = HostQuantizer(rows, dim, torch.bfloat16, "cuda", chunk_rows=chunk)
    for _ in range(2):      # second call reuses the staging buffers
        codes_host.zero_()
        scales_host.zero_()
        hq(x_host, gs_inv.reshape(1), codes_host, scales_host)
        torch.cuda.synchronize()
        assert torch.equal(codes_host, want_codes.cpu())
        assert torch.equal(scales_host, want_scales.view(torch.uint8).reshape(-1).cpu())


def test_entry_points_record_into_a_cuda_graph(cuda_lib):
    """Launches are asynchronous and never synchronise or copy to the host (reference contract: the kernels read
    `input_scale` on the device), so global scale -> quantize -> GEMM records into one CUDA graph and replays."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H

    a = C._gauss((256, 1024), 41).cuda()
    b = C._gauss((512, 1024), 42).cuda()

    def pipeline():
        gsa, gsa_inv = H.get_nvfp4_global_scale(a, 256.0)
        gsb, gsb_inv = H.get_nvfp4_global_scale(b, 256.0)
        qa, sa = K.scalesweep_mse_nvfp4_quant_impl(a, gsa_inv)
        qb, sb = K.scalesweep_weighted_mse_nvfp4_quant_impl(b, H.channel_square_norm(a), gsb_inv)
        return K.nvfp4_scaled_mm(qa, qb, sa, sb, (gsa * gsb).reshape(1), torch.bfloat16)

    want = pipeline()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        pipeline()                      # warm-up on the capture stream
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = pipeline()
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    a.mul_(2.0)                          # new input values in the same buffers: replay sees them
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, pipeline())


def test_config3_weighted_weight_quantization_sharded(cuda_lib, oracle):
    """bf16 weight [8192, 8192] ~ Laplace(0,1), importance = per-input-channel squared norm of a Laplace(0,1)
    activation batch [4096, 8192]; rows split across 1 / 2 / 4 / 8 shards (one per GPU) must give the bytes of
    the unsharded call, which must equal the oracle's."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H
    from nvfp4quant_test_b200.sharding import row_shards, scale_slab

    lap = torch.distributions.Laplace(torch.tensor(0.0, device="cuda"), torch.tensor(1.0, device="cuda"))
    torch.manual_seed(0)
    w = lap.sample((8192, 8192)).bfloat16()
    act = lap.sample((4096, 8192)).bfloat16()
    imp = H.channel_square_norm(act)
    assert torch.allclose(imp, (act.float() ** 2).sum(0, keepdim=True), rtol=1e-4)
    gs, gs_inv = H.get_nvfp4_global_scale(w, 256.0)
    codes, scales = K.scalesweep_weighted_mse_nvfp4_quant_impl(w, imp, gs_inv)
    want_codes, want_scales = oracle.quant(1, oracle.bf16_bits(w.cpu()), float(gs_inv), imp.cpu().numpy(),
                                           lower=-8, upper=7)
    assert np.array_equal(codes.cpu().numpy(), want_codes)
    flat = scales.view(torch.uint8).reshape(-1)
    assert np.array_equal(flat.cpu().numpy(), want_scales.reshape(-1))
    for world in (2, 4, 8):
        for a, b in row_shards(8192, world):
            c_, s_ = K.scalesweep_weighted_mse_nvfp4_quant_impl(w[a:b], imp, gs_inv)
            lo, hi = scale_slab(a, b, 512)
            assert torch.equal(c_, codes[a:b]) and torch.equal(s_.view(torch.uint8).reshape(-1), flat[lo:hi])
    # the weighted objective is what improves: importance-weighted error below the unweighted sweep's
    mc, ms = K.scalesweep_mse_nvfp4_quant_impl(w, gs_inv)
    dq_w = H.dequantize_base(codes[:1024], K.unswizzle_vllm_fp4_scale(scales, 8192, 8192)[:1024], gs)
    dq_m = H.dequantize_base(mc[:1024], K.unswizzle_vllm_fp4_scale(ms, 8192, 8192)[:1024], gs)
    assert H.weighted_error_stats(w[:1024], dq_w, imp)[0] <= H.weighted_error_stats(w[:1024], dq_m, imp)[0]


def test_randomized_differential_against_oracle(cuda_lib, probe_lib, oracle):
    """Seeded random sweep over shapes, dtypes, layouts, K padding, candidate windows, scale magnitudes and
    importance vectors (including zeros and huge weights): every byte must equal the oracle's."""
    rng = np.random.default_rng(20240607)
    for trial in range(60):
        m = int(rng.choice([1, 3, 31, 64, 128, 129, 200, 257, 400]))
        n = 16 * int(rng.integers(1, 40))
        dtype = [torch.bfloat16, torch.float16, torch.float32][int(rng.integers(0, 3))]
        variant = ["mse", "weighted", "amax"][int(rng.integers(0, 3))]
        swizzled = bool(rng.integers(0, 2))
        padded_n = n + 16 * int(rng.integers(0, 4)) if rng.integers(0, 3) == 0 else None
        dist = int(rng.integers(0, 4))
        g = torch.Generator().manual_seed(1000 + trial)
        if dist == 0:
            x = torch.randn((m, n), generator=g)
        elif dist == 1:
            x = torch.randn((m, n), generator=g) * torch.exp(4 * torch.randn((m, 1), generator=g))    # rows of very different size
        elif dist == 2:
            x = torch.randn((m, n), generator=g) * (torch.rand((m, n), generator=g) < 0.15)               # sparse
        else:
            x = torch.round(torch.randn((m, n), generator=g) * 4) / 4                                     # many exact ties
        x = x.to(dtype)
        if variant == "amax" and dtype == torch.float32:
            dtype, x = torch.bfloat16, x.to(torch.bfloat16)
        gs_inv = float(np.float32(rng.choice([1.0, 37.5, 565.9, 1e-3, 3000.0])))
        imp = None
        lower = upper = None
        if variant == "weighted":
            imp = torch.rand((1, n), generator=g) * 3
            if trial % 4 == 0:
                imp[0, ::5] = 0.0
            if trial % 7 == 0:
                imp[0, 1::9] = 1e20
            lower, upper = int(rng.integers(-10, 1)), int(rng.integers(0, 9))
        c = dict(x=x, variant=variant, importance=imp, swizzled=swizzled, padded_n=padded_n, lower=lower, upper=upper)
        table = _amax_table(probe_lib, gs_inv) if variant == "amax" else None
        want_codes, want_scales = util.oracle_quant_case(oracle, c, gs_inv, table)
        codes, scales, intact = _run_cuda(c, gs_inv)
        idx = util.logical_scale_index(m, (padded_n or n) // 16, swizzled)
        tag = (trial, m, n, str(dtype), variant, swizzled, padded_n, lower, upper, gs_inv)
        assert intact, tag
        assert np.array_equal(codes, want_codes), tag
        assert np.array_equal(scales[idx], want_scales[idx]), tag


def _two_launch(x, fp8_max, importance, swizzled, padded_n, lower=None, upper=None):
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H

    gs, gs_inv = H.get_nvfp4_global_scale(x, fp8_max)
    if importance is None:
        q, s = K.scalesweep_mse_nvfp4_quant_impl(x, gs_inv, swizzled, padded_n)
    else:
        kw = {} if lower is None else {"lower_bound": lower, "upper_bound": upper}
        q, s = K.scalesweep_weighted_mse_nvfp4_quant_impl(x, importance, gs_inv, swizzled, padded_n, **kw)
    return q, s, gs, gs_inv


@pytest.mark.parametrize("shape,dtype,weighted,swizzled,padded_n", [
    ((1, 4096), torch.bfloat16, False, True, None),
    ((1, 14336), torch.bfloat16, False, True, None),
    ((16, 8192), torch.bfloat16, False, True, None),
    ((130, 208), torch.bfloat16, False, True, 256),
    ((33, 64), torch.float16, False, False, None),
    ((16, 128), torch.float32, False, True, None),
    ((257, 1024), torch.bfloat16, True, False, None),
    ((128, 8192), torch.bfloat16, True, True, None),
    ((300, 8192), torch.bfloat16, False, True, None),     # close to the largest tensor one launch takes
    ((1024, 8192), torch.bfloat16, False, True, None),    # too large for one launch: the wrapper issues two
])
def test_fused_global_scale_and_sweep_equals_two_launches(cuda_lib, shape, dtype, weighted, swizzled, padded_n):
    """One cooperative launch computing the tensor-wide scale and the sweep must give the bytes, the scale bytes
    and the two fp32 scale values of get_nvfp4_global_scale followed by the quantizer."""
    import nvfp4quant_test_b200.kernels as K

    x = C._laplace(shape, 60 + shape[0], dtype).cuda()
    imp = C._importance("random", shape[1]).cuda() if weighted else None
    want = _two_launch(x, 256.0, imp, swizzled, padded_n)
    for _ in range(2):      # twice in a row: the scratch must come back zeroed
        got = K.scalesweep_nvfp4_quant_with_global_scale(x, 256.0, imp, swizzled, padded_n)
        torch.cuda.synchronize()
        status = torch.zeros(1, dtype=torch.int32).numpy()
        assert cuda_lib.nvfp4_quant_fused_last_status(None, status.ctypes.data) == 0 and status[0] == 0
        assert torch.equal(got[0], want[0])
        assert torch.equal(got[1].view(torch.uint8), want[1].view(torch.uint8))
        assert got[2].item() == want[2].item() and got[3].item() == want[3].item()


def test_fused_edge_values_and_window(cuda_lib):
    """NaN / inf / all-zero tensors and a custom weighted window through the fused launch."""
    import nvfp4quant_test_b200.kernels as K

    for x in (C._edge_rows(torch.bfloat16).cuda(), torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda"),
              C._gauss((8, 256), 3).cuda()):
        for imp, lo, up in ((None, None, None), (C._importance("ramp", x.shape[1]).cuda(), -2, 3)):
            want = _two_launch(x, 448.0, imp, True, None, lo, up)
            kw = {} if lo is None else {"lower_bound": lo, "upper_bound": up}
            got = K.scalesweep_nvfp4_quant_with_global_scale(x, 448.0, imp, True, None, **kw)
            assert torch.equal(got[0], want[0])
            assert torch.equal(got[1].view(torch.uint8), want[1].view(torch.uint8))
            for g, w in ((got[2], want[2]), (got[3], want[3])):
                assert torch.equal(g.view(torch.int32), w.view(torch.int32))      # NaN-safe bit comparison


def test_fused_launch_rejects_and_reports(cuda_lib):
    from nvfp4quant_test_b200 import _lib

    x = C._gauss((2048, 8192), 5).cuda()
    codes = torch.empty((2048, 4096), dtype=torch.uint8, device="cuda")
    scales = torch.empty((2048, 512), dtype=torch.uint8, device="cuda")
    gs = torch.empty(2, dtype=torch.float32, device="cuda")
    scratch = torch.zeros(4, dtype=torch.int32, device="cuda")
    args = [0, x.data_ptr(), 0, None, 256.0, gs.data_ptr(), scratch.data_ptr(), codes.data_ptr(), scales.data_ptr(),
            2048, 8192, 8192, -3, 7, 1, None]
    assert cuda_lib.nvfp4_quant_fused_launch(*args) == _lib.ERR_TOO_LARGE          # nothing launched
    args[0] = 2                                                                     # amax variant: not covered
    assert cuda_lib.nvfp4_quant_fused_launch(*args) < 0
    args[0], args[9] = 0, 16
    args[5] = None
    assert cuda_lib.nvfp4_quant_fused_launch(*args) < 0                             # null output
    torch.cuda.synchronize()
    assert int(scratch.abs().sum()) == 0


def test_fused_launch_records_into_a_cuda_graph(cuda_lib):
    import nvfp4quant_test_b200.kernels as K

    x = C._gauss((16, 4096), 77).cuda()
    want = _two_launch(x, 256.0, None, True, None)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        K.scalesweep_nvfp4_quant_with_global_scale(x, 256.0)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        got = K.scalesweep_nvfp4_quant_with_global_scale(x, 256.0)
    for _ in range(3):
        got[0].zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(got[0], want[0]) and torch.equal(got[1].view(torch.uint8), want[1].view(torch.uint8))
        assert got[3].item() == want[3].item()


@pytest.mark.parametrize("m,n,padded_n,swizzled", [(3, 4096, None, True), (129, 4096, None, False), (5, 4080, 4096, True),
                                                    (2, 8192, None, False), (130, 8176, 8192, True)])
def test_two_dimensional_grid_bodies(cuda_lib, oracle, m, n, padded_n, swizzled):
    """Rows that are a whole number of 256-block chunks wide take the two-dimensional grid (bodies 6 and 7); cover
    both layouts, ragged row counts, K padding and a non-default window there, against the oracle and the flat body."""
    x = C._laplace((m, n), 3000 + m + n)
    gs_inv = C.global_scale_cpu(x, 256.0)[1]
    P = padded_n or n
    for variant, imp, lo, up in (("mse", None, None, None), ("weighted", C._importance("random", n), None, None),
                                 ("mse", None, -2, 4), ("amax", None, None, None)):
        c = dict(x=x, variant=variant, importance=imp, swizzled=swizzled, padded_n=padded_n, lower=lo, upper=up)
        idx = util.logical_scale_index(m, P // 16, swizzled)
        flat_codes, flat_scales, ok = _run_cuda(c, gs_inv, 3)
        assert ok
        if variant != "amax":
            want_codes, want_scales = util.oracle_quant_case(oracle, c, gs_inv)
            assert np.array_equal(flat_codes, want_codes) and np.array_equal(flat_scales[idx], want_scales[idx])
        for impl in (0, 6, 7, 9):
            codes, scales, intact = _run_cuda(c, gs_inv, impl)
            assert intact, f"{variant} impl {impl} wrote outside its buffers"
            assert np.array_equal(codes, flat_codes), f"{variant} impl {impl}"
            assert np.array_equal(scales, flat_scales), f"{variant} impl {impl}"


def _whole_tile_input(m, n, seed, dtype):
    """Random rows with the special-value rows of the edge fixture (NaN, inf, zeros, ties, saturation) tiled in."""
    x = C._laplace((m, n), seed, dtype)
    e = C._edge_rows(dtype)                       # [16, 64]
    reps = min(n // 64, 8)
    k = min(m, 16)
    x[:k, :64 * reps] = e.repeat(1, reps)[:k]
    x[m - k:, n - 64:] = e[16 - k:]
    return x


@pytest.mark.parametrize("m,n,dtype,swizzled", [
    (128, 4096, torch.bfloat16, True),
    (256, 8192, torch.bfloat16, True),
    (130, 4096, torch.bfloat16, False),          # linear layout: any row count is a whole tile
    (1920, 4096, torch.bfloat16, True),          # more rows than resident CTAs: the row loop and its prefetch run
    (128, 4096, torch.float16, True),
    (128, 4096, torch.float32, False),
    (3, 4096, torch.bfloat16, False),            # fewer rows than CTAs
])
def test_whole_tile_body(cuda_lib, oracle, m, n, dtype, swizzled):
    """Body 8 (no validity predicates, for tensors without padding) against the scalar transcription (body 1) and the
    oracle: both sweeps, both layouts, three dtypes, special values included."""
    x = _whole_tile_input(m, n, 4000 + m + n, dtype)
    for gs_inv in (1.0, C.global_scale_cpu(C._laplace((m, n), 4000 + m + n, dtype), 256.0)[1]):
        for variant, imp in (("mse", None), ("weighted", C._importance("random", n))):
            c = dict(x=x, variant=variant, importance=imp, swizzled=swizzled, padded_n=None, lower=None, upper=None)
            ref_codes, ref_scales, ok = _run_cuda(c, gs_inv, 1)
            assert ok
            if m <= 256:
                want_codes, want_scales = util.oracle_quant_case(oracle, c, gs_inv)
                assert np.array_equal(ref_codes, want_codes) and np.array_equal(ref_scales, want_scales)
            for impl in (0, 8, 9):
                codes, scales, intact = _run_cuda(c, gs_inv, impl)
                assert intact, f"{variant} impl {impl} wrote outside its buffers"
                assert np.array_equal(codes, ref_codes), f"{variant} impl {impl}: {(codes != ref_codes).sum()} code bytes"
                assert np.array_equal(scales, ref_scales), f"{variant} impl {impl}: scale bytes"


def test_global_scale_of_views_that_start_off_a_16_byte_boundary(cuda_lib):
    """helper.get_nvfp4_global_scale accepts what the reference's x.abs().max() accepts: a flat view that starts one
    element in, a row slice of a matrix with an odd width."""
    from nvfp4quant_test_b200 import helper as H

    base = C._gauss((65, 1001), 21).cuda()
    for x in (base.view(-1)[1:], base[3:40], base[:, 1:].contiguous().view(-1)[3:], base.float().view(-1)[1:]):
        assert x.data_ptr() % 16 != 0 or True
        gs, gs_inv = H.get_nvfp4_global_scale(x, 448.0)
        ref = x.abs().max().float() / (6.0 * 448.0)
        assert bool(gs == ref) and bool(gs_inv == ref.reciprocal())


def test_quantizer_right_behind_the_global_scale_kernel_reads_the_new_scale(cuda_lib):
    """global scale -> quantizer back to back, both programmatic dependent launches, with the scale buffer holding a
    wrong value before every round: the quantizer is scheduled while the scale kernel still runs and must not read the
    scale (or its input) ahead of its wait.  Small and large tensors, both sweeps."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H

    g = torch.Generator(device="cuda")
    g.manual_seed(21)
    for shape in ((1, 4096), (48, 8192), (1024, 4096)):
        x = torch.normal(0.0, 1.0, size=shape, generator=g, device="cuda", dtype=torch.bfloat16)
        imp = torch.rand((1, shape[1]), generator=g, device="cuda") + 0.5
        gs, gs_inv = H.get_nvfp4_global_scale(x, 256.0)
        want_m = K.scalesweep_mse_nvfp4_quant_impl(x, gs_inv)
        want_w = K.scalesweep_weighted_mse_nvfp4_quant_impl(x, imp, gs_inv)
        torch.cuda.synchronize()
        buf = torch.empty(2, dtype=torch.float32, device="cuda")
        for _ in range(6):
            buf.fill_(3.0)
            H.get_nvfp4_global_scale(x, 256.0, out=buf)
            got_m = K.scalesweep_mse_nvfp4_quant_impl(x, buf[1])
            buf2 = torch.full((2,), 0.125, dtype=torch.float32, device="cuda")
            H.get_nvfp4_global_scale(x, 256.0, out=buf2)
            got_w = K.scalesweep_weighted_mse_nvfp4_quant_impl(x, imp, buf2[1])
            for got, want in ((got_m, want_m), (got_w, want_w)):
                assert torch.equal(got[0], want[0]) and torch.equal(got[1].view(torch.uint8), want[1].view(torch.uint8)), shape


def test_global_scale_in_graphs_replayed_at_the_same_time(cuda_lib):
    """Two CUDA graphs captured one after the other (torch captures on one and the same side stream), each with
    several multi-block global-scale launches, replayed at the same time on two streams: the launches of one graph must
    not share scratch words with the other's (helper.get_nvfp4_global_scale hands out scratch per capture), and an
    eager call afterwards still finds its scratch zeroed."""
    from nvfp4quant_test_b200 import helper as H

    g = torch.Generator(device="cuda")
    g.manual_seed(77)
    xs = [torch.normal(0.0, float(i + 1), size=(96, 8192), generator=g, device="cuda", dtype=torch.bfloat16) for i in range(2)]
    want = [x.abs().max().float() / (6 * 256.0) for x in xs]
    graphs, outs = [], []
    for x in xs:
        H.get_nvfp4_global_scale(x, 256.0)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = [H.get_nvfp4_global_scale(x, 256.0)[0] for _ in range(6)]
        graphs.append(graph), outs.append(out)
    streams = [torch.cuda.Stream() for _ in graphs]
    for _ in range(200):
        for graph, s in zip(graphs, streams):
            with torch.cuda.stream(s):
                graph.replay()
    torch.cuda.synchronize()
    for out, w in zip(outs, want):
        assert all(torch.equal(o, w) for o in out)
    for x, w in zip(xs, want):
        assert torch.equal(H.get_nvfp4_global_scale(x, 256.0)[0], w)
