"""GPU: the tcgen05 NVFP4 GEMM against the fp64 oracle and against cutlass_scaled_fp4_mm outputs.

Tolerance: fp32 accumulation of exact products, rounded once to bf16.  Every element must be within
2^-7 relative (one bf16 ulp) of the fp64 result, or within 2^-16 of the largest magnitude for values
near cancellation; in practice almost all elements equal the correctly rounded bf16 value."""
import numpy as np
import pytest
import torch

import cases as C

pytestmark = pytest.mark.gpu


def _quantize(x, imp=None):
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H

    gs, gs_inv = H.get_nvfp4_global_scale(x, 256.0)
    if imp is None:
        q, s = K.scalesweep_mse_nvfp4_quant_impl(x, gs_inv)
    else:
        q, s = K.scalesweep_weighted_mse_nvfp4_quant_impl(x, imp, gs_inv)
    return q, s, gs


def _check(out, ref):
    o = out.float().cpu().numpy()
    tol = np.maximum(np.abs(ref) * 2.0 ** -7, np.abs(ref).max() * 2.0 ** -16)
    assert not np.isnan(o).any()
    assert (np.abs(o - ref) <= tol).all(), float(np.abs(o - ref).max())
    want = torch.from_numpy(ref).to(torch.bfloat16).float().numpy()
    assert (o == want).mean() > 0.97


@pytest.mark.parametrize("M,N,K_", [(128, 256, 256), (130, 264, 512), (1, 512, 1024), (16, 128, 64), (300, 520, 320),
                                    (128, 128, 8192), (257, 1000, 192), (129, 8, 64), (256, 1024, 2048)])
def test_gemm_matches_fp64_oracle(cuda_lib, oracle, M, N, K_):
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    a, b = C.gemm_operands(M, N, K_, 40 + M + N)
    a, b = a.cuda(), b.cuda()
    qa, sa, gsa = _quantize(a, (b.float() ** 2).sum(0, keepdim=True))
    qb, sb, gsb = _quantize(b, (a.float() ** 2).sum(0, keepdim=True))
    alpha = (gsa * gsb).reshape(1).float()
    out = K.nvfp4_scaled_mm(qa, qb, sa, sb, alpha, torch.bfloat16)
    assert gemm_last_status() == 0
    ref = oracle.gemm(qa.cpu().numpy(), qb.cpu().numpy(), sa.view(torch.uint8).cpu().numpy().reshape(-1),
                      sb.view(torch.uint8).cpu().numpy().reshape(-1), float(alpha))
    _check(out, ref)
    # drop-in name of the vllm op and exact alpha scaling by a power of two
    out2 = K.cutlass_scaled_fp4_mm(qa, qb, sa, sb, alpha * 4, torch.bfloat16)
    assert torch.equal(out2.float(), out.float() * 4)


@pytest.mark.parametrize("M,N,K_", [(128, 256, 256), (300, 520, 320), (1, 512, 1024), (512, 768, 1024), (257, 1000, 192),
                                    (1024, 2048, 4096)])
def test_gemm_kernel_paths_agree(cuda_lib, oracle, M, N, K_):
    """128x64, 128x128, 128x256 and CTA-pair kernels must give the same bf16 bits (fp32 accumulation in
    the same K order) and each must satisfy the oracle tolerance."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    a, b = C.gemm_operands(M, N, K_, 90 + M)
    qa, sa, gsa = _quantize(a.cuda())
    qb, sb, gsb = _quantize(b.cuda())
    alpha = (gsa * gsb).reshape(1).float()
    outs = []
    try:
        for path in (1, 2, 3, 4, 6, 7):
            assert cuda_lib.nvfp4_gemm_force_path(path) == 0
            out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            K.nvfp4_scaled_mm(qa, qb, sa, sb, alpha, torch.bfloat16, out=out)
            assert gemm_last_status() == 0, f"path {path}"
            outs.append(out)
    finally:
        cuda_lib.nvfp4_gemm_force_path(0)
    ref = oracle.gemm(qa.cpu().numpy(), qb.cpu().numpy(), sa.view(torch.uint8).cpu().numpy().reshape(-1),
                      sb.view(torch.uint8).cpu().numpy().reshape(-1), float(alpha))
    for path, out in zip((1, 2, 3, 4, 6, 7), outs):
        _check(out, ref)
    assert all(torch.equal(outs[0], o) for o in outs[1:])


@pytest.mark.parametrize("M,N,K_,splits,rotate", [(1, 512, 2048, 2, 1), (16, 8192, 8192, 4, 1), (128, 1024, 4096, 2, 0),
                                                  (130, 264, 2304, 2, 0), (130, 264, 2304, 3, 1), (64, 520, 8192, 4, 1),
                                                  (300, 520, 1280, 5, 0)])
def test_gemm_k_ranges_and_rotation(cuda_lib, oracle, M, N, K_, splits, rotate):
    """Optional K ranges (fp32 partial tiles summed by a second kernel) and K-loop rotation of the single-CTA
    kernel, switched on through the tuning hook.  Same tolerance as every other path (the summation order differs, nothing else)."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    a, b = C.gemm_operands(M, N, K_, 70 + M)
    qa, sa, gsa = _quantize(a.cuda())
    qb, sb, gsb = _quantize(b.cuda())
    alpha = (gsa * gsb).reshape(1).float()
    try:
        assert cuda_lib.nvfp4_gemm_tune(splits, rotate) == 0
        assert cuda_lib.nvfp4_gemm_workspace_bytes(M, N, K_) >= 2 * M * N * 4
        out = K.nvfp4_scaled_mm(qa, qb, sa, sb, alpha, torch.bfloat16)
        assert gemm_last_status() == 0
    finally:
        cuda_lib.nvfp4_gemm_tune(0, -1)
    ref = oracle.gemm(qa.cpu().numpy(), qb.cpu().numpy(), sa.view(torch.uint8).cpu().numpy().reshape(-1),
                      sb.view(torch.uint8).cpu().numpy().reshape(-1), float(alpha))
    _check(out, ref)


def test_gemm_matches_cutlass_fixture(cuda_lib, golden):
    """Same quantized operands as the fixture -> compare with what cutlass_scaled_fp4_mm returned on a B200."""
    import nvfp4quant_test_b200.kernels as K

    meta, arrays = golden
    assert meta["gemm"]
    for name, info in meta["gemm"].items():
        qa = torch.from_numpy(arrays[name + ".qa"]).cuda()
        qb = torch.from_numpy(arrays[name + ".qb"]).cuda()
        sa = torch.from_numpy(arrays[name + ".sa"]).cuda()
        sb = torch.from_numpy(arrays[name + ".sb"]).cuda()
        alpha = torch.from_numpy(np.array([info["alpha_bits"]], dtype=np.int32).view(np.float32)).cuda()
        out = K.nvfp4_scaled_mm(qa, qb, sa, sb, alpha, torch.bfloat16)
        want = torch.from_numpy(arrays[name + ".out_bf16_bits"]).view(torch.bfloat16).float()
        got = out.float().cpu()
        # both accumulate exact products in fp32 (different orders): at most one bf16 ulp apart
        tol = torch.maximum(want.abs() * 2.0 ** -7, want.abs().max() * 2.0 ** -16)
        assert bool(((got - want).abs() <= tol).all()), name
        assert float((got == want).float().mean()) > 0.97, name


def test_gemm_full_size_sampled(cuda_lib, oracle):
    """M = N = K = 8192 (the benchmark's GEMM): sampled rows/columns against fp64 dot products, plus
    linearity in alpha and independence from how N is sharded."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    a = torch.randn((8192, 8192), generator=g, device="cuda").bfloat16()
    b = torch.randn((8192, 8192), generator=g, device="cuda").bfloat16()
    qa, sa, gsa = _quantize(a)
    qb, sb, gsb = _quantize(b)
    alpha = (gsa * gsb).reshape(1).float()
    out = K.nvfp4_scaled_mm(qa, qb, sa, sb, alpha, torch.bfloat16)
    assert gemm_last_status() == 0
    rows = [0, 127, 128, 4095, 8191]
    cols = list(range(0, 8192, 97))
    sa_u = K.unswizzle_vllm_fp4_scale(sa, 8192, 8192)
    sb_u = K.unswizzle_vllm_fp4_scale(sb, 8192, 8192)
    from nvfp4quant_test_b200 import helper as H

    da = H.dequantize_base(qa[rows], sa_u[rows], torch.tensor(1.0)).double()
    db = H.dequantize_base(qb[cols], sb_u[cols], torch.tensor(1.0)).double()
    ref = (da @ db.T * float(alpha)).cpu().numpy()
    got = out[rows][:, cols].float().cpu().numpy()
    tol = np.maximum(np.abs(ref) * 2.0 ** -7, np.abs(ref).max() * 2.0 ** -16)
    assert (np.abs(got - ref) <= tol).all()
    # N-sharding (the multi-GPU partitioning): each 1024-row slice of b gives the same output columns
    for n0 in (0, 3072, 7168):
        part = K.nvfp4_scaled_mm(qa, qb[n0:n0 + 1024], sa, sb.view(torch.uint8).reshape(-1)[n0 * 512:(n0 + 1024) * 512],
                                 alpha, torch.bfloat16)
        assert torch.equal(part, out[:, n0:n0 + 1024])


def test_channel_square_norm_kernel(cuda_lib):
    from nvfp4quant_test_b200 import helper as H

    for shape, dt in (((2048, 4096), torch.bfloat16), ((300, 520), torch.float16), ((77, 132), torch.float32),
                      ((1, 8), torch.bfloat16)):
        x = C._laplace(shape, 17, dt if dt != torch.float32 else torch.float32).cuda()
        got = H.channel_square_norm(x)
        want = (x.double() ** 2).sum(0, keepdim=True)
        assert got.shape == (1, shape[1]) and got.dtype == torch.float32
        assert torch.allclose(got.double(), want, rtol=2e-5, atol=0)
        assert torch.equal(got, H.channel_square_norm(x))       # fixed summation order
        # column slices are read in place through the row pitch and concatenate to the same bits (how several GPUs
        # share the reduction); a slice that starts off a 16-byte boundary is copied first, same bits again
        if shape[1] >= 64:
            cuts = [0, 16, 48, shape[1] // 2 // 16 * 16, shape[1]]
            parts = [H.channel_square_norm(x[:, a:b]) for a, b in zip(cuts, cuts[1:]) if b > a]
            assert torch.equal(torch.cat(parts, 1), got)
            assert torch.equal(H.channel_square_norm(x[:, 4:36]), got[:, 4:36])
    L = cuda_lib
    x = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(64, dtype=torch.float32, device="cuda")
    assert L.nvfp4_channel_sqnorm_launch_strided(x.data_ptr(), 0, 8, 32, 16, out.data_ptr(), None) == -2    # ld < n
    assert L.nvfp4_channel_sqnorm_launch_strided(x.data_ptr(), 0, 8, 32, 62, out.data_ptr(), None) == -2    # ld % 4
    assert L.nvfp4_channel_sqnorm_launch_strided(x.data_ptr() + 8, 0, 8, 32, 64, out.data_ptr(), None) == -4


def test_llama_stack_layer_shapes(cuda_lib, oracle):
    """Config-5 shapes: one Llama-3-8B-shaped layer, importance = squared norms of a calibration batch.
    Weight bytes checked against the oracle on the two narrow matrices in full and on row samples of the rest;
    the layer's GEMMs at a token batch of 32 against fp64 dot products on sampled outputs."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H
    from nvfp4quant_test_b200 import llama_stack as LS

    dev = torch.device("cuda")
    calib = LS.make_calibration(dev)
    importance = {k: H.channel_square_norm(x) for k, x in calib.items()}
    weights = LS.make_layer(0, dev)
    q = LS.quantize_layer(weights, importance)
    for name, (codes, scales, gs) in q.items():
        n, k = LS.LAYER_SHAPES[name]
        assert codes.shape == (n, k // 2)
        rows = slice(0, n) if n <= 1024 else slice(n // 2, n // 2 + 256)
        w = weights[name][rows].contiguous()
        _, gs_inv_t = H.get_nvfp4_global_scale(weights[name], 256.0)
        want_codes, want_scales = oracle.quant(1, oracle.bf16_bits(w.cpu()), float(gs_inv_t),
                                               importance[k].cpu().numpy(), swizzled=False, lower=-8, upper=7)
        assert np.array_equal(codes[rows].cpu().numpy(), want_codes), name
        lin = K.unswizzle_vllm_fp4_scale(scales, n, k).view(torch.uint8)[rows]
        assert np.array_equal(lin.cpu().numpy(), want_scales), name
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    acts = {kk: torch.normal(0.0, 1.0, size=(32, kk), generator=gen, device=dev, dtype=torch.bfloat16) for kk in calib}
    outs = LS.layer_gemms(q, acts, {})
    # the same GEMMs dealt out over side streams (forked from / joined into the current stream): same bits
    side = [torch.cuda.Stream() for _ in range(3)]
    outs_side = LS.layer_gemms(q, acts, {}, None, side)
    torch.cuda.synchronize()
    assert all(torch.equal(outs[name], outs_side[name]) for name in outs)
    # and as grouped launches (q+k+v, o, gate+up, down) with the output scales formed inside the kernel: the K ranges
    # per tile are chosen from a group's total tile count, so sums may differ in the last fp32 bit before the bf16 store
    outs_grouped = LS.layer_gemms_grouped(q, acts, LS.stack_weight_scales(q), LS.prepare_layer(q))
    torch.cuda.synchronize()
    for name, want in outs.items():
        tol_g = torch.maximum(want.float().abs() * 2.0 ** -7, want.float().abs().max() * 2.0 ** -16)
        assert bool(((outs_grouped[name].float() - want.float()).abs() <= tol_g).all()), name
    for name in ("k", "down", "gate"):
        n, k = LS.LAYER_SHAPES[name]
        codes, scales, gs_w = q[name]
        gs_x, gs_x_inv = H.get_nvfp4_global_scale(acts[k], 256.0)
        qa, sa = K.scalesweep_mse_nvfp4_quant_impl(acts[k], gs_x_inv)
        cols = list(range(0, n, max(1, n // 61)))
        da = H.dequantize_base(qa, K.unswizzle_vllm_fp4_scale(sa, 32, k), torch.tensor(1.0)).double()
        db = H.dequantize_base(codes[cols], K.unswizzle_vllm_fp4_scale(scales, n, k)[cols], torch.tensor(1.0)).double()
        ref = (da @ db.T * float(gs_x * gs_w)).cpu().numpy()
        got = outs[name][:, cols].float().cpu().numpy()
        tol = np.maximum(np.abs(ref) * 2.0 ** -7, np.abs(ref).max() * 2.0 ** -16)
        assert outs[name].shape == (32, n) and (np.abs(got - ref) <= tol).all(), name


@pytest.mark.parametrize("N", [8192, 28672])
def test_config4_gemm_shapes(cuda_lib, N):
    """Activation [M, 8192] and weight [N, 8192] ~ Laplace(0,1), each quantized with importance from the other
    operand's channel square norms; M in {1, 16, 128, 2048, 8192}.  Sampled outputs against fp64 dot products of
    the dequantized operands."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    lap = torch.distributions.Laplace(torch.tensor(0.0, device="cuda"), torch.tensor(1.0, device="cuda"))
    torch.manual_seed(N)
    w = lap.sample((N, 8192)).bfloat16()
    a_full = lap.sample((8192, 8192)).bfloat16()
    gs_w, gs_w_inv = H.get_nvfp4_global_scale(w, 256.0)
    qw, sw = K.scalesweep_weighted_mse_nvfp4_quant_impl(w, H.channel_square_norm(a_full), gs_w_inv)
    imp_a = H.channel_square_norm(w)
    sw_lin = K.unswizzle_vllm_fp4_scale(sw, N, 8192)
    cols = list(range(0, N, N // 53)) + [N - 1]
    db = H.dequantize_base(qw[cols], sw_lin[cols], torch.tensor(1.0)).double()
    for M in (1, 16, 128, 2048, 8192):
        a = a_full[:M].contiguous()
        gs_a, gs_a_inv = H.get_nvfp4_global_scale(a, 256.0)
        qa, sa = K.scalesweep_weighted_mse_nvfp4_quant_impl(a, imp_a, gs_a_inv)
        alpha = (gs_a * gs_w).reshape(1).float()
        out = K.nvfp4_scaled_mm(qa, qw, sa, sw, alpha, torch.bfloat16)
        assert gemm_last_status() == 0 and out.shape == (M, N)
        rows = sorted(set([0, M - 1, M // 2] + list(range(0, M, max(1, M // 7)))))
        da = H.dequantize_base(qa[rows], K.unswizzle_vllm_fp4_scale(sa, M, 8192)[rows], torch.tensor(1.0)).double()
        ref = (da @ db.T * float(alpha)).cpu().numpy()
        got = out[rows][:, cols].float().cpu().numpy()
        tol = np.maximum(np.abs(ref) * 2.0 ** -7, np.abs(ref).max() * 2.0 ** -16)
        assert (np.abs(got - ref) <= tol).all(), (M, N, float(np.abs(got - ref).max()))
        del out


@pytest.mark.parametrize("M,N,K_,ranks", [(1, 512, 1024, 0), (1, 512, 1024, 2), (2, 130, 64, 0), (5, 1000, 2304, 3),
                                          (16, 8192, 8192, 0), (16, 8192, 8192, 8), (17, 264, 320, 2), (32, 4096, 4096, 0),
                                          (33, 520, 1280, 4), (64, 1024, 8192, 4), (4, 96, 24576, 8), (65, 264, 2304, 2),
                                          (128, 1000, 4096, 3)])
def test_gemm_skinny_kernel(cuda_lib, oracle, M, N, K_, ranks):
    """The decode-sized kernel (weight rows on the MMA's 128 rows, token tile 16..128, K ranges spread over a
    thread-block cluster and reduced in rank 0's shared memory), with the number of ranges chosen by shape
    (0) or forced.  Oracle tolerance; with one range the bits must equal the 128x128 kernel's."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    a, b = C.gemm_operands(M, N, K_, 40 + M)
    qa, sa, gsa = _quantize(a.cuda())
    qb, sb, gsb = _quantize(b.cuda())
    alpha = (gsa * gsb).reshape(1).float()
    outs = {}
    try:
        for path, r in ((1, 0), (5, ranks), (5, 1)):
            assert cuda_lib.nvfp4_gemm_force_path(path) == 0
            assert cuda_lib.nvfp4_gemm_tune(r, -1) == 0
            out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            K.nvfp4_scaled_mm(qa, qb, sa, sb, alpha, torch.bfloat16, out=out)
            assert gemm_last_status() == 0, f"path {path} ranks {r}"
            outs[(path, r)] = out
    finally:
        cuda_lib.nvfp4_gemm_force_path(0)
        cuda_lib.nvfp4_gemm_tune(0, -1)
    ref = oracle.gemm(qa.cpu().numpy(), qb.cpu().numpy(), sa.view(torch.uint8).cpu().numpy().reshape(-1),
                      sb.view(torch.uint8).cpu().numpy().reshape(-1), float(alpha))
    for out in outs.values():
        _check(out, ref)
    assert torch.equal(outs[(1, 0)], outs[(5, 1)])


def test_gemm_skinny_is_default_for_decode_batches(cuda_lib):
    """Shapes with M <= 32 take the skinny kernel when nothing is forced: same bits as forcing it."""
    import nvfp4quant_test_b200.kernels as K

    M, N, K_ = 8, 768, 2048
    a, b = C.gemm_operands(M, N, K_, 77)
    qa, sa, gsa = _quantize(a.cuda())
    qb, sb, gsb = _quantize(b.cuda())
    alpha = (gsa * gsb).reshape(1).float()
    auto = K.nvfp4_scaled_mm(qa, qb, sa, sb, alpha, torch.bfloat16)
    try:
        assert cuda_lib.nvfp4_gemm_force_path(5) == 0
        forced = K.nvfp4_scaled_mm(qa, qb, sa, sb, alpha, torch.bfloat16)
    finally:
        cuda_lib.nvfp4_gemm_force_path(0)
    assert torch.equal(auto, forced)


def test_gemm_randomized_shapes_all_kernels(cuda_lib):
    """Seeded random shapes with random codes and scale bytes: the tile and pair kernels (paths 1, 2, 3, 4, 6) must
    agree bit for bit, the skinny kernel with one K range too; with a random number of K ranges it must stay
    within one bf16 ulp of them (floor: 2^-16 of the largest output, for sums that cancel)."""
    import random

    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    rng = random.Random(20240607)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    try:
        for _ in range(40):
            M = rng.choice([1, 3, 16, 17, 32, 33, 64, 100, 128, 129, 256, 300])
            N = rng.choice([8, 64, 136, 200, 256, 520, 1024, 4096])
            K_ = 64 * rng.choice([1, 2, 3, 5, 8, 16, 33, 64])
            qa = torch.randint(0, 256, (M, K_ // 2), dtype=torch.uint8, device="cuda", generator=gen)
            qb = torch.randint(0, 256, (N, K_ // 2), dtype=torch.uint8, device="cuda", generator=gen)
            kp = (K_ // 16 + 3) // 4 * 4
            sa = torch.randint(0x28, 0x48, ((M + 127) // 128 * 128, kp), dtype=torch.uint8, device="cuda", generator=gen)
            sb = torch.randint(0x28, 0x48, ((N + 127) // 128 * 128, kp), dtype=torch.uint8, device="cuda", generator=gen)
            alpha = torch.rand(1, device="cuda", generator=gen) + 0.5
            runs = [(1, 0), (2, 0), (3, 0), (4, 0), (6, 0), (7, 0), (0, 0)]
            if M <= 128:
                runs += [(5, 1), (5, rng.choice([2, 3, 4, 8]))]
            outs = {}
            for path, ranks in runs:
                assert cuda_lib.nvfp4_gemm_force_path(path) == 0 and cuda_lib.nvfp4_gemm_tune(ranks, -1) == 0
                out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
                K.nvfp4_scaled_mm(qa, qb, sa.view(torch.float8_e4m3fn), sb.view(torch.float8_e4m3fn), alpha,
                                  torch.bfloat16, out=out)
                outs[(path, ranks)] = out
            assert gemm_last_status() == 0
            ref = outs[(1, 0)]
            assert not torch.isnan(ref).any()
            for key in ((2, 0), (3, 0), (4, 0), (6, 0), (7, 0), (5, 1)):
                if key in outs:
                    assert torch.equal(outs[key], ref), (M, N, K_, key)
            tol = torch.maximum(ref.float().abs() * 2.0 ** -7, ref.float().abs().max() * 2.0 ** -16)
            for key, out in outs.items():
                assert bool(((out.float() - ref.float()).abs() <= tol).all()), (M, N, K_, key)
    finally:
        cuda_lib.nvfp4_gemm_force_path(0)
        cuda_lib.nvfp4_gemm_tune(0, -1)


def test_saved_quantized_weights_load_on_the_device_and_give_the_same_gemm_bits(cuda_lib, tmp_path):
    """Serving use of the file format (what llm_test/nvfp4_quant.py:36-50 of the reference does with save_pretrained):
    quantize -> storage.save -> storage.load(device="cuda") -> GEMM must equal the GEMM on the never-saved operands
    bit for bit, also when the scales take the detour through the row-major layout and back."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H
    from nvfp4quant_test_b200 import storage

    x = C._laplace((48, 1024), 70).cuda()
    weights = {"gate": C._laplace((1536, 1024), 71).cuda(), "odd_rows": C._laplace((200, 1024), 72).cuda()}
    imp = H.channel_square_norm(x)
    q = {}
    for name, w in weights.items():
        gs, gs_inv = H.get_nvfp4_global_scale(w, 256.0)
        codes, scales = K.scalesweep_weighted_mse_nvfp4_quant_impl(w, imp, gs_inv)
        q[name] = (codes, scales, gs)
    storage.save(tmp_path / "layer.nvfp4", q)
    loaded = storage.load(tmp_path / "layer.nvfp4", device="cuda")
    gsx, gsx_inv = H.get_nvfp4_global_scale(x, 256.0)
    qx, sx = K.scalesweep_mse_nvfp4_quant_impl(x, gsx_inv)
    for name, (codes, scales, gs) in q.items():
        lc, ls, lg = loaded[name]
        assert lc.is_cuda and torch.equal(lc, codes) and torch.equal(ls.view(torch.uint8).reshape(-1), scales.view(torch.uint8).reshape(-1))
        assert lg.item() == gs.item()
        want = K.nvfp4_scaled_mm(qx, codes, sx, scales, (gsx * gs).reshape(1), torch.bfloat16)
        got = K.nvfp4_scaled_mm(qx, lc, sx, ls, (gsx * lg).reshape(1), torch.bfloat16)
        assert torch.equal(got, want), name
        rows, cols = weights[name].shape
        relaid = storage.as_tiled_scales(storage.as_linear_scales(ls, rows, cols), rows, cols)
        got2 = K.nvfp4_scaled_mm(qx, lc, sx, relaid, (gsx * lg).reshape(1), torch.bfloat16)
        assert torch.equal(got2, want), name
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    assert gemm_last_status() == 0


def test_llama_stack_run_end_to_end(cuda_lib):
    """The stack driver itself on a few layers: quantization phase, then the GEMM phase as one CUDA graph: at a decode
    batch grouped launches chained on one stream, at 256 tokens the GEMMs of a layer on four streams (where tile and
    CTA-pair kernels of different widths run at the same time)."""
    from nvfp4quant_test_b200 import llama_stack as LS

    res = LS.run(4, [16, 256])
    assert res["layers"] == 4 and res["quantize_ms"] > 0 and res["quantize_gweights_per_s"] > 10
    assert [g["tokens"] for g in res["gemm"]] == [16, 256]
    for g in res["gemm"]:
        assert g["cuda_graph"] and g["streams"] == (1 if g["tokens"] <= 64 else 4) and 0.0 < g["ms_all_layers"] < 50.0
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    assert gemm_last_status() == 0


def test_prepared_weight_gives_the_same_bits_on_every_kernel_path(cuda_lib):
    """nvfp4_gemm_prepare + nvfp4_gemm_launch_prepared == nvfp4_gemm_launch, for token counts that take the skinny,
    the tile and the CTA-pair kernels, with one handle reused across all of them and across streams."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    g = torch.Generator(device="cuda")
    g.manual_seed(11)
    n, k = 4096 + 192, 2048
    w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda", generator=g)
    sw = torch.randint(0x28, 0x48, ((n + 127) // 128 * 128, k // 16), dtype=torch.uint8, device="cuda", generator=g)
    alpha = torch.full((1,), 0.37, dtype=torch.float32, device="cuda")
    pw = K.PreparedWeight(w, sw)
    side = torch.cuda.Stream()
    for m in (1, 16, 48, 128, 200, 256, 512, 1024, 2304):
        a = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device="cuda", generator=g)
        sa = torch.randint(0x28, 0x48, ((m + 127) // 128 * 128, k // 16), dtype=torch.uint8, device="cuda", generator=g)
        want = K.nvfp4_scaled_mm(a, w, sa, sw, alpha, torch.bfloat16)
        got = K.nvfp4_scaled_mm_prepared(a, sa, alpha, pw)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            got_side = K.nvfp4_scaled_mm_prepared(a, sa, alpha, pw)
        torch.cuda.current_stream().wait_stream(side)
        assert torch.equal(got, want) and torch.equal(got_side, want), m
    assert gemm_last_status() == 0
    with pytest.raises(ValueError):
        K.nvfp4_scaled_mm_prepared(a[:, :512], sa, alpha, pw)             # K mismatch
    pw.close()
    pw.close()                                                             # idempotent
    with pytest.raises(ValueError):
        K.nvfp4_scaled_mm_prepared(a, sa, alpha, pw)


@pytest.mark.parametrize("M", [1, 16, 33, 100, 256])
def test_grouped_gemm_equals_one_by_one_calls(cuda_lib, M):
    """One activation against a group of prepared weights of different N (ragged last tiles included), alphas
    multiplied inside the kernel: with one K range per tile every output equals the one-by-one prepared call bit for
    bit (decode-sized M: one launch for the group; M = 256: the per-weight fallback), with the default K ranges it
    stays within one bf16 ulp; more than 8 weights are cut into several launches."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    g = torch.Generator(device="cuda")
    g.manual_seed(100 + M)
    k = 1024
    ns = [512, 136, 128, 1000, 8, 256, 384, 64, 192, 2048]          # ten weights: two launches at decode sizes
    ws, sws, pws, alphas = [], [], [], []
    for n in ns:
        w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda", generator=g)
        sw = torch.randint(0x28, 0x48, ((n + 127) // 128 * 128, k // 16), dtype=torch.uint8, device="cuda", generator=g)
        ws.append(w), sws.append(sw), pws.append(K.PreparedWeight(w, sw))
        alphas.append(torch.rand(1, device="cuda", generator=g) + 0.5)
    a = torch.randint(0, 256, (M, k // 2), dtype=torch.uint8, device="cuda", generator=g)
    sa = torch.randint(0x28, 0x48, ((M + 127) // 128 * 128, k // 16), dtype=torch.uint8, device="cuda", generator=g)
    alpha_a = torch.rand(1, device="cuda", generator=g) + 0.25
    try:
        for ranks in (1, 0):
            if M <= 128:
                assert cuda_lib.nvfp4_gemm_force_path(5) == 0 and cuda_lib.nvfp4_gemm_tune(ranks, -1) == 0
            single = [K.nvfp4_scaled_mm_prepared(a, sa, al * alpha_a, pw) for al, pw in zip(alphas, pws)]
            outs = [torch.full((M, n), float("nan"), dtype=torch.bfloat16, device="cuda") for n in ns]
            got = K.nvfp4_scaled_mm_grouped(a, sa, alpha_a, pws, alphas, outs)
            plain = K.nvfp4_scaled_mm_grouped(a, sa, None, pws[:3], [al * alpha_a for al in alphas[:3]])
            assert gemm_last_status() == 0
            for i, (x, y) in enumerate(zip(got, single)):
                assert not torch.isnan(x).any()
                if ranks == 1 or M > 128:
                    assert torch.equal(x, y), (M, ranks, i)
                else:
                    tol = torch.maximum(y.float().abs() * 2.0 ** -7, y.float().abs().max() * 2.0 ** -16)
                    assert bool(((x.float() - y.float()).abs() <= tol).all()), (M, ranks, i)
            for x, y in zip(plain, got[:3]):
                if ranks == 1 or M > 128:
                    assert torch.equal(x, y)
    finally:
        cuda_lib.nvfp4_gemm_force_path(0)
        cuda_lib.nvfp4_gemm_tune(0, -1)
    with pytest.raises(ValueError):
        K.nvfp4_scaled_mm_grouped(a, sa, alpha_a, pws, alphas[:-1])
    assert K.nvfp4_scaled_mm_grouped(a, sa, alpha_a, [], []) == []


def test_quantize_then_grouped_gemm_chain_in_a_cuda_graph(cuda_lib, oracle):
    """global scale -> quantizer -> grouped GEMM -> global scale -> quantizer -> GEMM on one stream, every kernel a
    programmatic dependent launch, recorded into a CUDA graph and replayed on fresh inputs: each replay must equal the
    same chain launched with plain stream order (the switch of nvfp4_gemm_tune_pdl), bit for bit."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    k, tokens = 2048, 8
    pws, gws = [], []
    keep = []
    for n in (2048, 256, 256):
        w = torch.normal(0.0, 0.02, size=(n, k), generator=g, device="cuda", dtype=torch.bfloat16)
        gs, gi = H.get_nvfp4_global_scale(w, H.FP8_E4M3_MAX_4OVER6)
        c, s = K.scalesweep_mse_nvfp4_quant_impl(w, gi)
        keep.append((c, s))
        pws.append(K.PreparedWeight(c, s)), gws.append(gs.reshape(1).float())
    w2 = torch.normal(0.0, 0.02, size=(512, 2048), generator=g, device="cuda", dtype=torch.bfloat16)
    gs2, gi2 = H.get_nvfp4_global_scale(w2, H.FP8_E4M3_MAX_4OVER6)
    c2, s2 = K.scalesweep_mse_nvfp4_quant_impl(w2, gi2)
    pw2, gw2 = K.PreparedWeight(c2, s2), gs2.reshape(1).float()
    x = torch.empty((tokens, k), dtype=torch.bfloat16, device="cuda")

    def chain():
        gx, gxi = H.get_nvfp4_global_scale(x, H.FP8_E4M3_MAX_4OVER6)
        qa, sa = K.scalesweep_mse_nvfp4_quant_impl(x, gxi)
        q, kk, v = K.nvfp4_scaled_mm_grouped(qa, sa, gx.reshape(1), pws, gws)
        gq, gqi = H.get_nvfp4_global_scale(q, H.FP8_E4M3_MAX_4OVER6)
        qq, sq = K.scalesweep_mse_nvfp4_quant_impl(q, gqi)
        (o,) = K.nvfp4_scaled_mm_grouped(qq, sq, gq.reshape(1), [pw2], [gw2])
        return q, kk, v, o

    x.normal_(generator=g)
    chain()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = chain()
    for trial in range(3):
        x.normal_(generator=g)
        graph.replay()
        got = [t.clone() for t in outs]
        try:
            assert cuda_lib.nvfp4_gemm_tune_pdl(0) == 0
            want = chain()
        finally:
            cuda_lib.nvfp4_gemm_tune_pdl(1)
        torch.cuda.synchronize()
        for a_, b_ in zip(got, want):
            assert torch.equal(a_, b_), trial
        assert float(got[3].float().abs().max()) > 0.0
    assert gemm_last_status() == 0


def test_gemm_right_behind_the_quantizer_of_its_weight(cuda_lib):
    """Drop-in use as the reference's benchmark chains it: quantize the weight, then multiply, back to back on one
    stream with raw pointers.  The GEMM is a programmatic dependent launch, so it may be scheduled while the quantizer
    is still running; it must not read the weight before that kernel is done.  The code buffer holds garbage before
    every round, so an early read changes the output."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H

    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    n, k, m = 4096, 4096, 16
    w = torch.normal(0.0, 1.0, size=(n, k), generator=g, device="cuda", dtype=torch.bfloat16)
    x = torch.normal(0.0, 1.0, size=(m, k), generator=g, device="cuda", dtype=torch.bfloat16)
    gw, gwi = H.get_nvfp4_global_scale(w, H.FP8_E4M3_MAX_4OVER6)
    gx, gxi = H.get_nvfp4_global_scale(x, H.FP8_E4M3_MAX_4OVER6)
    qx, sx = K.scalesweep_mse_nvfp4_quant_impl(x, gxi)
    alpha = (gw * gx).reshape(1).float()
    codes, scales = K.create_fp4_output_tensors(n, k, w.device, True)
    K.scalesweep_mse_nvfp4_quant_out(w, gwi, True, output=codes, output_scale=scales)
    torch.cuda.synchronize()
    want = K.nvfp4_scaled_mm(qx, codes, sx, scales.view(torch.float8_e4m3fn), alpha, torch.bfloat16)
    torch.cuda.synchronize()
    for m_tokens in (16, 256):
        xa = x if m_tokens == 16 else x.repeat(16, 1)
        qa, sa = K.scalesweep_mse_nvfp4_quant_impl(xa, gxi)
        for _ in range(10):
            codes.fill_(0x77)
            scales.view(torch.uint8).fill_(0x38)
            K.scalesweep_mse_nvfp4_quant_out(w, gwi, True, output=codes, output_scale=scales)
            got = K.nvfp4_scaled_mm(qa, codes, sa, scales.view(torch.float8_e4m3fn), alpha, torch.bfloat16)
            assert torch.equal(got[:16], want)


def test_preallocated_decode_blocks_equal_the_allocating_entry_points(cuda_lib):
    """kernels.ActivationQuantizer (global scale + sweep from one host call) and kernels.LinearGroup (grouped GEMM into
    preallocated outputs), and llama_stack.DecodeLayer built from them: the same bits as get_nvfp4_global_scale +
    scalesweep_mse_nvfp4_quant_impl + nvfp4_scaled_mm_grouped, call after call on changing inputs."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H
    from nvfp4quant_test_b200 import llama_stack as LS

    dev = torch.device("cuda")
    calib = LS.make_calibration(dev)
    importance = {k: H.channel_square_norm(x) for k, x in calib.items()}
    q = LS.quantize_layer(LS.make_layer(1, dev), importance)
    ws, pw = LS.stack_weight_scales(q), LS.prepare_layer(q)
    gen = torch.Generator(device=dev)
    gen.manual_seed(9)
    for tokens in (1, 24):
        layer = LS.DecodeLayer(q, ws, pw, tokens, dev)
        for _ in range(3):
            acts = {kk: torch.normal(0.0, 1.0, size=(tokens, kk), generator=gen, device=dev, dtype=torch.bfloat16)
                    for kk in calib}
            got = layer(acts)
            want = LS.layer_gemms_grouped(q, acts, ws, pw)
            for name in want:
                assert torch.equal(got[name], want[name]), (tokens, name)
            for kk, quantizer in layer.quantizers.items():
                gs, gi = H.get_nvfp4_global_scale(acts[kk], H.FP8_E4M3_MAX_4OVER6)
                codes, scales = K.scalesweep_mse_nvfp4_quant_impl(acts[kk], gi)
                assert torch.equal(quantizer.codes, codes) and torch.equal(quantizer.scales.view(torch.uint8), scales.view(torch.uint8))
                assert torch.equal(quantizer.global_scale, torch.stack([gs, gi]))
    with pytest.raises(ValueError):
        layer({kk: v[:1] for kk, v in acts.items()})                       # wrong token count
    with pytest.raises(ValueError):
        K.LinearGroup([pw["q"], pw["down"]], [ws[4096][0][:1], ws[14336][0][:1]], 4)   # different K


def test_random_launch_chains_do_not_depend_on_dependent_launch(cuda_lib):
    """Seeded random programs over a small pool of reused buffers - global scale, the three quantizers, GEMMs with raw
    pointers (also on a weight quantized by the launch just before), with prepared weights and grouped, GEMM outputs
    fed back as the next activation, torch kernels in between - run back to back on one stream with every library
    kernel a programmatic dependent launch, eagerly and as a CUDA graph, must leave every buffer with the bits the same
    program leaves under plain stream order (nvfp4_gemm_tune_pdl(0)).  Buffers are reused on purpose, so that the
    programs are full of read-after-write and write-after-read pairs between neighbouring launches."""
    import random

    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    dev = torch.device("cuda")
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234)
    kdim = 512
    const_w = []                                                  # constant, prepared weights [n, kdim]
    for n in (512, 256, 512):
        w = torch.normal(0.0, 0.05, size=(n, kdim), generator=gen, device=dev, dtype=torch.bfloat16)
        gs, gi = H.get_nvfp4_global_scale(w, 256.0)
        c, s = K.scalesweep_mse_nvfp4_quant_impl(w, gi)
        const_w.append((K.PreparedWeight(c, s), gs.reshape(1).clone(), c, s))
    torch.cuda.synchronize()

    def build_state(m):
        st = {"x": torch.normal(0.0, 1.0, size=(m, kdim), generator=gen, device=dev, dtype=torch.bfloat16),
              "src": torch.normal(0.0, 1.0, size=(m, kdim), generator=gen, device=dev, dtype=torch.bfloat16),
              "wsrc": torch.normal(0.0, 0.05, size=(512, kdim), generator=gen, device=dev, dtype=torch.bfloat16),
              "imp": torch.rand((1, kdim), generator=gen, device=dev) + 0.5,
              "gs": torch.ones(2, dtype=torch.float32, device=dev),
              "wgs": torch.ones(2, dtype=torch.float32, device=dev),
              "alpha": torch.ones(1, dtype=torch.float32, device=dev),
              "y": [torch.zeros((m, n), dtype=torch.bfloat16, device=dev) for n in (512, 256, 512)]}
        st["qx"], st["sx"] = K.create_fp4_output_tensors(m, kdim, dev, True)
        st["qw"], st["sw"] = K.create_fp4_output_tensors(512, kdim, dev, True)
        H.get_nvfp4_global_scale(st["x"], 256.0, out=st["gs"])
        K.scalesweep_mse_nvfp4_quant_out(st["x"], st["gs"][1], True, output=st["qx"], output_scale=st["sx"])
        H.get_nvfp4_global_scale(st["wsrc"], 256.0, out=st["wgs"])
        K.scalesweep_mse_nvfp4_quant_out(st["wsrc"], st["wgs"][1], True, output=st["qw"], output_scale=st["sw"])
        return st

    def run_program(prog, st):
        f8 = torch.float8_e4m3fn
        for op, arg in prog:
            if op == "new_x":                       # a torch kernel rewrites the activation
                st["x"].copy_(st["src"]).mul_(arg)
            elif op == "feed_back":                 # a GEMM output becomes the activation (n == kdim for y[0], y[2])
                st["x"].copy_(st["y"][arg])
            elif op == "scale":
                H.get_nvfp4_global_scale(st["x"], 256.0, out=st["gs"])
            elif op == "quant":
                if arg == 0:
                    K.scalesweep_mse_nvfp4_quant_out(st["x"], st["gs"][1], True, output=st["qx"], output_scale=st["sx"])
                elif arg == 1:
                    K.scalesweep_weighted_mse_nvfp4_quant_out(st["x"], st["imp"], st["gs"][1], True, output=st["qx"],
                                                              output_scale=st["sx"])
                else:
                    K.amax_nvfp4_quant_out(st["x"], st["gs"][1], True, output=st["qx"], output_scale=st["sx"])
            elif op == "requant_w":                 # the raw-pointer weight is rewritten right before it is used
                st["wsrc"].mul_(arg)
                H.get_nvfp4_global_scale(st["wsrc"], 256.0, out=st["wgs"])
                K.scalesweep_mse_nvfp4_quant_out(st["wsrc"], st["wgs"][1], True, output=st["qw"], output_scale=st["sw"])
            elif op == "alpha":
                torch.mul(st["gs"][0:1], st["wgs"][0:1], out=st["alpha"])
            elif op == "mm_raw":
                K.nvfp4_scaled_mm(st["qx"], st["qw"], st["sx"].view(f8), st["sw"].view(f8), st["alpha"], torch.bfloat16,
                                  out=st["y"][0])
            elif op == "mm_prepared":
                pw, gw, _, _ = const_w[arg]
                K.nvfp4_scaled_mm_prepared(st["qx"], st["sx"].view(f8), gw, pw, out=st["y"][arg])
            elif op == "mm_grouped":
                K.nvfp4_scaled_mm_grouped(st["qx"], st["sx"].view(f8), st["gs"][0:1], [c[0] for c in const_w],
                                          [c[1] for c in const_w], st["y"])

    def bits(t):                                    # bit patterns: NaNs (programs overflow on purpose) compare equal
        return t.contiguous().view(torch.uint8).clone()

    def snapshot(st):
        return [bits(st[k]) for k in ("x", "gs", "wgs", "alpha", "qx", "qw", "sx", "sw")] + [bits(y) for y in st["y"]]

    rng = random.Random(99)
    ops = ["new_x", "feed_back", "scale", "quant", "requant_w", "alpha", "mm_raw", "mm_prepared", "mm_grouped"]
    try:
        for trial in range(30):
            m = rng.choice([1, 8, 24, 40, 150])
            prog = []
            for _ in range(rng.randint(8, 16)):
                op = rng.choice(ops)
                arg = {"new_x": rng.choice([0.5, 1.5, 3.0]), "feed_back": rng.choice([0, 2]), "quant": rng.choice([0, 1, 2]),
                       "requant_w": rng.choice([0.5, 2.0]), "mm_prepared": rng.randrange(3)}.get(op)
                prog.append((op, arg))
            gen.manual_seed(500 + trial)
            base = build_state(m)
            torch.cuda.synchronize()
            results = []
            for mode in ("plain", "pdl", "pdl_graph"):
                st = {k: ([t.clone() for t in v] if isinstance(v, list) else v.clone()) for k, v in base.items()}
                assert cuda_lib.nvfp4_gemm_tune_pdl(0 if mode == "plain" else 1) == 0
                torch.cuda.synchronize()
                if mode == "pdl_graph":
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(side):
                        warm = {k: ([t.clone() for t in v] if isinstance(v, list) else v.clone()) for k, v in base.items()}
                        run_program(prog, warm)      # first launches of every kernel outside the capture
                    torch.cuda.current_stream().wait_stream(side)
                    torch.cuda.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        run_program(prog, st)
                    graph.replay()
                else:
                    run_program(prog, st)
                torch.cuda.synchronize()
                results.append(snapshot(st))
            for other, name in ((results[1], "eager"), (results[2], "graph")):
                for i, (a_, b_) in enumerate(zip(results[0], other)):
                    assert torch.equal(a_, b_), f"trial {trial} (m = {m}) {name}: buffer {i} differs; program {prog}"
        assert gemm_last_status() == 0
    finally:
        cuda_lib.nvfp4_gemm_tune_pdl(1)


def test_graphs_of_different_token_counts_replayed_at_the_same_time(cuda_lib):
    """Three CUDA graphs of a few Llama-shaped layers (1 token: grouped decode-sized launches; 256 and 1024 tokens: tile
    and CTA-pair kernels on forked streams, global-scale launches that go through scratch words) replayed at the same
    time on three streams: every replay leaves the bits of the plain, eager run, and no bounded wait runs out."""
    from nvfp4quant_test_b200 import helper as H
    from nvfp4quant_test_b200 import llama_stack as LS
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    dev = torch.device("cuda", torch.cuda.current_device())
    calib = LS.make_calibration(dev)
    importance = {k: H.channel_square_norm(x) for k, x in calib.items()}
    qlayers = [LS.quantize_layer(LS.make_layer(i, dev), importance) for i in range(3)]
    wscales = [LS.stack_weight_scales(q) for q in qlayers]
    prepared = [LS.prepare_layer(q) for q in qlayers]
    side = [torch.cuda.Stream(device=dev) for _ in range(4)]
    items = []
    for tokens in (1, 256, 1024):
        gen = torch.Generator(device=dev)
        gen.manual_seed(tokens)
        acts = {k: torch.normal(0.0, 1.0, size=(tokens, k), generator=gen, device=dev, dtype=torch.bfloat16) for k in calib}
        if tokens <= LS.GROUPED_MAX_TOKENS:
            layers = [LS.DecodeLayer(q, ws, pw, tokens, dev) for q, ws, pw in zip(qlayers, wscales, prepared)]

            def fn(layers=layers, acts=acts):
                return [layer(acts) for layer in layers][-1]
        else:
            def fn(acts=acts):
                return [LS.layer_gemms(q, acts, {}, ws, side, pw) for q, ws, pw in zip(qlayers, wscales, prepared)][-1]
        try:
            assert cuda_lib.nvfp4_gemm_tune_pdl(0) == 0
            truth = {k: v.clone() for k, v in fn().items()}
        finally:
            cuda_lib.nvfp4_gemm_tune_pdl(1)
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = fn()
        items.append((graph, out, truth, fn, acts))      # fn / acts own the buffers the graph points into
    streams = [torch.cuda.Stream(device=dev) for _ in items]
    for _ in range(60):
        for (graph, *_rest), s in zip(items, streams):
            with torch.cuda.stream(s):
                graph.replay()
    torch.cuda.synchronize()
    assert gemm_last_status() == 0
    for graph, out, truth, _fn, _acts in items:
        for name, want in truth.items():
            assert torch.equal(out[name].view(torch.int16), want.view(torch.int16)), name
