// Test-only diagnostic kernels (built into a separate library by tests/conftest.py, not shipped with the product):
// they expose what this GPU's div.full.f32 and rcp.approx.ftz return for the 127 scale values, which pins the CPU
// oracle's tables.
#include "common.cuh"

namespace nvfp4 {
namespace {

__global__ void div_full_table_kernel(uint32_t* out) {
    const uint32_t raw = threadIdx.x;
    if (raw < 128) out[raw] = __float_as_uint(div_full(1.0f, e4m3_to_f32(raw)));
}

// out[raw], raw < 127: multiplier the AMAX variant applies for scale byte `raw`;
// out[127]: rcp.approx.ftz(6.0f), the factor it uses for amax / 6.
__global__ void amax_table_kernel(const float* gs_inv_ptr, float* out) {
    const uint32_t raw = threadIdx.x;
    const float gs_inv = *gs_inv_ptr;
    if (raw < 127) out[raw] = (raw == 0) ? 0.0f : rcp_approx_ftz(__fmul_rn(e4m3_to_f32(raw), rcp_approx_ftz(gs_inv)));
    else if (raw == 127) out[raw] = rcp_approx_ftz(6.0f);
}

}  // namespace
}  // namespace nvfp4

extern "C" int nvfp4_probe_div_full_table(uint32_t* out128, void* stream) {
    if (!out128) return NVFP4_ERR_NULL_POINTER;
    nvfp4::div_full_table_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(out128);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int nvfp4_probe_amax_out_scale_table(const float* gs_inv, float* out128, void* stream) {
    if (!gs_inv || !out128) return NVFP4_ERR_NULL_POINTER;
    nvfp4::amax_table_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(gs_inv, out128);
    return static_cast<int>(cudaGetLastError());
}
