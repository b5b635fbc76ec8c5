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

// 2: grouped GEMM launch, one-call quantizer chain, strided importance reduction, capture id (additions only: every
// version-1 entry point keeps its signature and meaning)
extern "C" int nvfp4_abi_version(void) { return 2; }

// 0 while `stream` is not being captured into a CUDA graph, else the id of the capture (unique per capture sequence of the
// process).  Host bookkeeping only: callers that hand out scratch buffers per stream use it to tell captures apart, because
// graphs captured one after the other on the same stream may later be replayed at the same time on different streams.
extern "C" int nvfp4_stream_capture_id(void* stream, unsigned long long* id_host) {
    if (!id_host) return NVFP4_ERR_NULL_POINTER;
    *id_host = 0;
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    unsigned long long id = 0;
    const cudaError_t e = cudaStreamGetCaptureInfo(static_cast<cudaStream_t>(stream), &status, &id);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (status == cudaStreamCaptureStatusActive) *id_host = id;
    return NVFP4_OK;
}
