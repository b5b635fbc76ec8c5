"""GPU: the error paths of the kernels that wait on something, exercised without faulting anything.

Every wait inside these kernels is bounded; when the limit passes, the kernel records a status word and returns.
Here the limit is lowered to a millisecond and a wait is made to run out on purpose by a hook that withholds the
one signal it waits for (a flag that nothing sets): the launch must return, the status must be readable, and the
next ordinary launch must work.  Nothing traps, reads a bad address or spins without a limit."""
import ctypes

import numpy as np
import pytest
import torch

import cases as C

pytestmark = pytest.mark.gpu


def test_fused_quantizer_grid_wait_gives_up_and_recovers(cuda_lib):
    import nvfp4quant_test_b200.kernels as K

    L = cuda_lib
    x = C._gauss((128, 4096), 7).cuda()
    want = K.scalesweep_nvfp4_quant_with_global_scale(x, 256.0)
    codes = torch.empty((128, 2048), dtype=torch.uint8, device="cuda")
    scales = torch.empty((128, 256), dtype=torch.uint8, device="cuda")
    gs = torch.zeros(2, dtype=torch.float32, device="cuda")
    scratch = torch.zeros(4, dtype=torch.int32, device="cuda")
    args = lambda: (0, x.data_ptr(), 0, None, 256.0, gs.data_ptr(), scratch.data_ptr(), codes.data_ptr(),
                    scales.data_ptr(), 128, 4096, 4096, -3, 7, 1, None)
    status = ctypes.c_uint32(7)
    assert L.nvfp4_quant_fused_set_wait_limit_ns(1_000_000) == 0          # 1 ms
    try:
        scratch[3] = 1                                                    # CTA 0 withholds its arrival
        assert L.nvfp4_quant_fused_launch(*args()) == 0
        assert L.nvfp4_quant_fused_last_status(None, ctypes.byref(status)) == 0
        assert status.value == 1                                          # the wait ran out; the kernel returned
        assert L.nvfp4_quant_fused_last_status(None, ctypes.byref(status)) == 0 and status.value == 0   # reading cleared it
    finally:
        assert L.nvfp4_quant_fused_set_wait_limit_ns(0) == 0              # back to the default
    scratch.zero_()                                                       # as the header asks after a failed launch
    assert L.nvfp4_quant_fused_launch(*args()) == 0
    assert L.nvfp4_quant_fused_last_status(None, ctypes.byref(status)) == 0 and status.value == 0
    assert torch.equal(codes, want[0]) and torch.equal(scales.reshape(-1), want[1].view(torch.uint8).reshape(-1))
    assert gs[0].item() == want[2].item() and int(scratch.abs().sum()) == 0
    assert L.nvfp4_quant_fused_set_wait_limit_ns(5) == -5                 # below a microsecond: rejected


def test_gemm_wait_gives_up_and_recovers(cuda_lib):
    """mbar_wait is shared by every GEMM kernel; the probe kernel with its last commit left out is the one place a
    wait can be made to expire without touching a real GEMM's pipeline."""
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    L = cuda_lib
    sms = ctypes.c_int(0)
    assert gemm_last_status() == 0
    assert L.nvfp4_gemm_set_wait_limit_ns(1_000_000) == 0
    try:
        assert L.nvfp4_gemm_peak_probe(64, 2, ctypes.byref(sms), None) == 0
        st = gemm_last_status()
        assert st != 0 and (st >> 24) == 4                                # role 4 = the probe's issuing warp
        assert gemm_last_status() == 0                                    # cleared by the read
    finally:
        assert L.nvfp4_gemm_set_wait_limit_ns(0) == 0
    # TMEM was freed and the device is fine: the ordinary probe and a real GEMM run and report ok
    assert L.nvfp4_gemm_peak_probe(64, 0, ctypes.byref(sms), None) == 0
    assert L.nvfp4_gemm_peak_probe(64, 1, ctypes.byref(sms), None) == 0 and sms.value % 2 == 0
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200 import helper as H

    a, b = C._laplace((256, 512), 1).cuda(), C._laplace((384, 512), 2).cuda()
    gsa, gia = H.get_nvfp4_global_scale(a, 256.0)
    gsb, gib = H.get_nvfp4_global_scale(b, 256.0)
    qa, sa = K.scalesweep_mse_nvfp4_quant_impl(a, gia)
    qb, sb = K.scalesweep_mse_nvfp4_quant_impl(b, gib)
    out = K.nvfp4_scaled_mm(qa, qb, sa, sb, (gsa * gsb).reshape(1), torch.bfloat16)
    assert gemm_last_status() == 0
    ref = (H.dequantize_base(qa, K.unswizzle_vllm_fp4_scale(sa, 256, 512), gsa).double()
           @ H.dequantize_base(qb, K.unswizzle_vllm_fp4_scale(sb, 384, 512), gsb).double().T)
    assert torch.allclose(out.double(), ref, rtol=2 ** -7, atol=float(ref.abs().max()) * 2 ** -16)
    assert L.nvfp4_gemm_peak_probe(0, 0, None, None) == -5 and L.nvfp4_gemm_peak_probe(8, 3, None, None) == -3


def test_concurrent_gemms_of_different_kernels_on_four_streams(cuda_lib):
    """GEMM launches may overlap on the GPU.  Kernels with different tile shapes running at the same time on several
    streams once left a CTA waiting for TMEM for ever (their shared-memory footprints differed; now every kernel that
    takes all TMEM columns also takes a whole SM's shared memory).  A graph of mixed shapes over four streams, replayed
    several times, must finish and give the bits of the same GEMMs run one after the other."""
    import nvfp4quant_test_b200.kernels as K
    from nvfp4quant_test_b200.kernels.kernel_gemm import gemm_last_status

    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    k = 4096
    tokens = 256
    shapes = [4096, 1024, 1024, 4096, 14336, 14336, 6144, 512]      # 128x64 tiles and CTA pairs of two widths at this K
    x = torch.randint(0, 256, (tokens, k // 2), dtype=torch.uint8, device="cuda", generator=g)
    sx = torch.randint(0x30, 0x40, (tokens, k // 16), dtype=torch.uint8, device="cuda", generator=g)
    ws = [torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda", generator=g) for n in shapes]
    sws = [torch.randint(0x30, 0x40, ((n + 127) // 128 * 128, k // 16), dtype=torch.uint8, device="cuda", generator=g) for n in shapes]
    one = torch.ones(1, dtype=torch.float32, device="cuda")
    want = [K.nvfp4_scaled_mm(x, w, sx, s, one, torch.bfloat16) for w, s in zip(ws, sws)]
    outs = [torch.empty_like(o) for o in want]
    streams = [torch.cuda.Stream() for _ in range(4)]

    def launch_all():
        main = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(main)
        for rep in range(4):
            for i, (w, s) in enumerate(zip(ws, sws)):
                st = streams[i % 4]
                st.wait_event(start)
                with torch.cuda.stream(st):
                    K.nvfp4_scaled_mm(x, w, sx, s, one, torch.bfloat16, out=outs[i])
        for st in streams:
            e = torch.cuda.Event()
            e.record(st)
            main.wait_event(e)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launch_all()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launch_all()
    for _ in range(20):
        graph.replay()
    torch.cuda.synchronize()
    assert gemm_last_status() == 0
    for o, w_ in zip(outs, want):
        assert torch.equal(o, w_)
