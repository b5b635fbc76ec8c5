// Per-input-channel squared L2 norm of an activation batch: out[j] = sum_i x[i, j]^2 (fp32).
//
// This is the importance vector the reference feeds to the weighted quantizer ("the importance scores for
// weight tensors are based on the activation input-channel square norm, and vice versa", README.md:11 of
// efsotr/nvfp4quant_test; its driver script is not published, torch's `(x.float() ** 2).sum(0)` is the
// obvious spelling).  One pass over x; the summation order is fixed (rows strided by 64 per thread in ascending
// order, then a fixed binary tree over the 64 row groups), so the result is reproducible run to run.  A CTA owns
// 16 columns, so an 8192-column batch runs on 512 CTAs with eight loads in flight per thread.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace nvfp4 {
namespace {

constexpr int kSqThreads = 256;   // 64 row groups x 4 lanes
constexpr int kSqLanes = 4;       // lanes side by side on one row segment
constexpr int kSqGroups = kSqThreads / kSqLanes;
constexpr int kSqCols = 4 * kSqLanes;   // columns per CTA: 4 per lane (32 bytes of bf16 per row: one DRAM sector)
constexpr int kSqUnroll = 8;      // independent loads in flight per thread

template <int DT>
__device__ __forceinline__ void load4(const void* x, int64_t elem, float v[4]) {
    if (DT == NVFP4_DT_F32) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(x) + elem));
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
        const uint2 u = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(x) + elem));
        if (DT == NVFP4_DT_BF16) {
            v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xffff0000u);
            v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xffff0000u);
        } else {
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
            const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
            v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
        }
    }
}

template <int DT>
__global__ void __launch_bounds__(kSqThreads) channel_sqnorm_kernel(const void* x, int64_t m, int64_t n, int64_t ld,
                                                                    float* out) {
    const int lane = threadIdx.x % kSqLanes, rg = threadIdx.x / kSqLanes;
    const int64_t col = static_cast<int64_t>(blockIdx.x) * kSqCols + lane * 4;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (col < n) {   // n % 4 == 0 is required, so a lane's 4 columns are all inside or all outside
        int64_t r = rg;
        // rows rg, rg + 64, ... in ascending order; kSqUnroll loads are issued before the first is consumed
        for (; r + (kSqUnroll - 1) * kSqGroups < m; r += kSqUnroll * kSqGroups) {
            float v[kSqUnroll][4];
#pragma unroll
            for (int u = 0; u < kSqUnroll; ++u) load4<DT>(x, (r + u * kSqGroups) * ld + col, v[u]);
#pragma unroll
            for (int u = 0; u < kSqUnroll; ++u)
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[k] = __fmaf_rn(v[u][k], v[u][k], acc[k]);
        }
        for (; r < m; r += kSqGroups) {
            float v[4];
            load4<DT>(x, r * ld + col, v);
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[k] = __fmaf_rn(v[k], v[k], acc[k]);
        }
    }
    // fixed binary tree over the 64 row groups
    __shared__ float part[kSqGroups][kSqCols];
#pragma unroll
    for (int k = 0; k < 4; ++k) part[rg][lane * 4 + k] = acc[k];
    __syncthreads();
    for (int half = kSqGroups / 2; half >= 1; half >>= 1) {
        for (int idx = threadIdx.x; idx < half * kSqCols; idx += kSqThreads) {
            const int g = idx / kSqCols, c = idx - g * kSqCols;
            part[g][c] = __fadd_rn(part[g][c], part[g + half][c]);
        }
        __syncthreads();
    }
    if (threadIdx.x < kSqCols) {
        const int64_t oc = static_cast<int64_t>(blockIdx.x) * kSqCols + threadIdx.x;
        if (oc < n) out[oc] = part[0][threadIdx.x];
    }
}

}  // namespace
}  // namespace nvfp4

extern "C" int nvfp4_channel_sqnorm_launch_strided(const void* x, int x_dtype, int64_t m, int64_t n, int64_t ld, float* out,
                                                   void* stream) {
    using namespace nvfp4;
    if (x_dtype < NVFP4_DT_BF16 || x_dtype > NVFP4_DT_F32) return NVFP4_ERR_BAD_ENUM;
    if (m < 0 || n < 0 || (n % 4) != 0 || ld < n) return NVFP4_ERR_BAD_SHAPE;
    if (n == 0) return NVFP4_OK;
    if (!out || (!x && m > 0)) return NVFP4_ERR_NULL_POINTER;
    // a lane reads 4 consecutive elements (8 or 16 bytes) of a row: the row pitch keeps those pieces aligned
    if ((ld % 4) != 0) return NVFP4_ERR_BAD_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 3)) return NVFP4_ERR_MISALIGNED;
    const int64_t blocks = (n + kSqCols - 1) / kSqCols;
    if (blocks > 0x7fffffffLL) return NVFP4_ERR_TOO_LARGE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned g = static_cast<unsigned>(blocks);
    switch (x_dtype) {
        case NVFP4_DT_BF16: channel_sqnorm_kernel<NVFP4_DT_BF16><<<g, kSqThreads, 0, s>>>(x, m, n, ld, out); break;
        case NVFP4_DT_F16: channel_sqnorm_kernel<NVFP4_DT_F16><<<g, kSqThreads, 0, s>>>(x, m, n, ld, out); break;
        default: channel_sqnorm_kernel<NVFP4_DT_F32><<<g, kSqThreads, 0, s>>>(x, m, n, ld, out); break;
    }
    return static_cast<int>(cudaGetLastError());
}

extern "C" int nvfp4_channel_sqnorm_launch(const void* x, int x_dtype, int64_t m, int64_t n, float* out, void* stream) {
    return nvfp4_channel_sqnorm_launch_strided(x, x_dtype, m, n, n, out, stream);
}
