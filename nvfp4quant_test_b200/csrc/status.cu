// Status strings and ABI version of the C ABI.
#include <cuda_runtime.h>

#include "nvfp4_b200.h"

namespace nvfp4 {
int g_dependent_launch = 1;   // see common.cuh
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
