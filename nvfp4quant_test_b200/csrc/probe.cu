// Small diagnostic kernels and the status-string table.
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

extern "C" const char* nvfp4_status_string(int status) {
    switch (status) {
        case NVFP4_OK: return "ok";
        case NVFP4_ERR_NULL_POINTER: return "a required pointer is NULL";
        case NVFP4_ERR_BAD_SHAPE: return "bad shape (sizes must be non-negative, n and padded_n multiples of 16, padded_n >= n, GEMM K a multiple of 64)";
        case NVFP4_ERR_BAD_ENUM: return "unknown variant, dtype or implementation id";
        case NVFP4_ERR_MISALIGNED: return "a pointer is not aligned as the header documents";
        case NVFP4_ERR_BAD_RANGE: return "candidate window must satisfy lower <= upper and hold at most 64 candidates";
        case NVFP4_ERR_WORKSPACE: return "workspace is NULL or too small";
        case NVFP4_ERR_UNSUPPORTED: return "unsupported configuration";
        case NVFP4_ERR_TOO_LARGE: return "problem exceeds the supported size";
        case NVFP4_ERR_STATIC_SCRATCH: return "input is larger than the library's built-in scratch array can serve (see nvfp4_global_scale_static_max_bytes)";
        default: break;
    }
    if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
    return "unknown status";
}

extern "C" int nvfp4_abi_version(void) { return 1; }
