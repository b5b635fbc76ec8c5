"""GPU: the allocation-free global-scale entry point (nvfp4_global_scale_launch_static).

It exists for hosts that cannot obtain device scratch memory themselves - a plugin that is only
handed raw device pointers, a serving process with a frozen memory pool - and keeps its scratch in
an array inside the library.  Here it is called through the C ABI twice in a row on different inputs
and must return exactly the bits of the ordinary entry point (which uses caller-provided scratch);
the second call also proves that what the first call left in the shared array does no harm.
This file sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bind(L):
    i64, ci, vp, f32 = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_float
    L.nvfp4_global_scale_launch_static.restype = ci
    L.nvfp4_global_scale_launch_static.argtypes = [vp, ci, i64, f32, vp, vp]
    L.nvfp4_global_scale_static_max_bytes.restype = i64
    L.nvfp4_global_scale_static_max_bytes.argtypes = []
    return L


def test_static_scratch_entry_point_matches_regular_one(cuda_lib):
    from nvfp4quant_test_b200 import _lib

    L = _bind(cuda_lib)
    assert L.nvfp4_global_scale_static_max_bytes() == 512 * 1024 * 1024
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    inputs = [
        (torch.randn((8192, 8192), generator=gen, device="cuda") * 3.0).to(torch.bfloat16),   # 128 MiB, 1024 blocks
        torch.randn((1000, 1001), generator=gen, device="cuda").to(torch.bfloat16),            # ragged tail
        torch.randn((33, 64), generator=gen, device="cuda").to(torch.float16),
        torch.randn((3000, 4096), generator=gen, device="cuda"),                                # fp32
        torch.zeros((1, 7), device="cuda", dtype=torch.bfloat16),
    ]
    for fp8_max in (448.0, 256.0):
        for x in inputs:                      # consecutive calls share the library's array
            code = _lib.dtype_code(x.dtype)
            want = torch.empty(2, dtype=torch.float32, device="cuda")
            scratch = torch.zeros(2, dtype=torch.int32, device="cuda")
            _lib.check(L.nvfp4_global_scale_launch(x.data_ptr(), code, x.numel(), fp8_max, want.data_ptr(),
                                                   scratch.data_ptr(), stream), "regular")
            got = torch.full((2,), -1.0, dtype=torch.float32, device="cuda")
            _lib.check(L.nvfp4_global_scale_launch_static(x.data_ptr(), code, x.numel(), fp8_max, got.data_ptr(),
                                                          stream), "static")
            torch.cuda.synchronize()
            assert torch.equal(got.view(torch.int32), want.view(torch.int32)), (tuple(x.shape), x.dtype, fp8_max)
    # NaN propagates the same way
    x = inputs[1].clone()
    x[500, 500] = float("nan")
    got = torch.zeros(2, dtype=torch.float32, device="cuda")
    _lib.check(L.nvfp4_global_scale_launch_static(x.data_ptr(), 0, x.numel(), 448.0, got.data_ptr(), stream), "static")
    torch.cuda.synchronize()
    assert torch.isnan(got).all()


def test_static_scratch_entry_point_rejects_what_it_cannot_serve(cuda_lib):
    from nvfp4quant_test_b200 import _lib

    L = _bind(cuda_lib)
    out = torch.zeros(2, dtype=torch.float32, device="cuda")
    P = out.data_ptr()   # never dereferenced: the size check comes first
    too_many = 512 * 1024 * 1024 // 2 + 1
    assert L.nvfp4_global_scale_launch_static(P, 0, too_many, 448.0, P, None) == -9
    assert "built-in scratch" in _lib.status_string(-9)
    assert L.nvfp4_global_scale_launch_static(P, 2, 512 * 1024 * 1024 // 4 + 1, 448.0, P, None) == -9
    assert L.nvfp4_global_scale_launch_static(P, 7, 16, 448.0, P, None) == -3
    assert L.nvfp4_global_scale_launch_static(None, 0, 16, 448.0, P, None) == -1
    assert L.nvfp4_global_scale_launch_static(P, 0, 16, 448.0, None, None) == -1
    torch.cuda.synchronize()


def test_static_scratch_entry_point_allocates_nothing_and_chains_on_a_stream(cuda_lib):
    """The property the entry point exists for: device memory in use does not change across calls (cudaMemGetInfo
    before and after), and calls issued back to back on one stream - no synchronisation between them, the case the
    header promises is safe because each call re-clears its counter in stream order - all give the right bits."""
    from nvfp4quant_test_b200 import _lib

    L = _bind(cuda_lib)
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device="cuda")
    gen.manual_seed(9)
    xs = [torch.randn((2048, 4096), generator=gen, device="cuda").to(torch.bfloat16) * (i + 1) for i in range(6)]
    xs.append(torch.randn((777, 1001), generator=gen, device="cuda"))                    # fp32, ragged
    outs = torch.full((len(xs), 2), -1.0, dtype=torch.float32, device="cuda")
    want = torch.empty((len(xs), 2), dtype=torch.float32, device="cuda")
    scratch = torch.zeros(2, dtype=torch.int32, device="cuda")
    for i, x in enumerate(xs):
        _lib.check(L.nvfp4_global_scale_launch(x.data_ptr(), _lib.dtype_code(x.dtype), x.numel(), 448.0,
                                               want[i].data_ptr(), scratch.data_ptr(), stream), "regular")
    _lib.check(L.nvfp4_global_scale_launch_static(xs[0].data_ptr(), 0, xs[0].numel(), 448.0, outs[0].data_ptr(), stream),
               "static")            # first call on this device (if no earlier test made it): resolves the symbol address
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for i, x in enumerate(xs):      # back to back, one stream, no synchronisation in between
        st = L.nvfp4_global_scale_launch_static(x.data_ptr(), _lib.dtype_code(x.dtype), x.numel(), 448.0,
                                                outs[i].data_ptr(), stream)
        assert st == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    assert torch.equal(outs.view(torch.int32), want.view(torch.int32))
