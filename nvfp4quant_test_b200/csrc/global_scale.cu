// Tensor-wide NVFP4 global scale: gs = amax|x| / (6 * fp8_max), gs_inv = 1 / gs.
//
// Follows helper.py:96-100 of efsotr/nvfp4quant_test (get_nvfp4_global_scale) as torch
// evaluates it on a CUDA tensor: a fp32 tensor divided by a host scalar is multiplied by
// the fp32 reciprocal of that scalar, and `.reciprocal()` is an IEEE fp32 division.
//
// One pass over x with 16-byte loads.  The maximum is taken on the magnitude BIT PATTERNS
// (sign cleared, unsigned compare): for non-negative floats that order equals the numeric
// order, and a NaN pattern is larger than +inf, so NaN propagates the way torch's max does.
// Blocks combine through a 2-word scratch (running maximum, arrival counter); the last
// block to arrive publishes the result and leaves the scratch zeroed for the next call.
#include <cuda_fp16.h>

#include "common.cuh"

namespace nvfp4 {
namespace {

constexpr int kGsThreads = 512;

__device__ __forceinline__ uint32_t umax2x16(uint32_t a, uint32_t b) { return __vmaxu2(a, b); }

template <int DT>
__global__ void __launch_bounds__(kGsThreads) global_scale_kernel(const void* x, int64_t numel, float fp8_max,
                                                                  float* out, uint32_t* scratch) {
    // launched as a programmatic dependent: x, the scratch words and `out` belong to the kernel before this one until
    // it has finished.  The kernel behind this one (the quantizer, which waits before it touches anything) may be
    // scheduled at once.
    griddep_launch();
    griddep_wait();
    constexpr int kPerVec = (DT == NVFP4_DT_F32) ? 4 : 8;
    const int64_t nvec = numel / kPerVec;
    x = after_wait(x);   // loads of x stay behind the wait
    const uint4* xv = static_cast<const uint4*>(x);
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kGsThreads;
    uint32_t acc = 0;
    auto fold = [&](const uint4& q) {
        if (DT == NVFP4_DT_F32) {
            acc = max(acc, max(max(q.x & 0x7fffffffu, q.y & 0x7fffffffu), max(q.z & 0x7fffffffu, q.w & 0x7fffffffu)));
        } else {
            acc = umax2x16(acc, umax2x16(umax2x16(q.x & 0x7fff7fffu, q.y & 0x7fff7fffu),
                                         umax2x16(q.z & 0x7fff7fffu, q.w & 0x7fff7fffu)));
        }
    };
    int64_t i = static_cast<int64_t>(blockIdx.x) * kGsThreads + threadIdx.x;
    // four independent 16-byte loads in flight per thread: with one, a resident grid holds too few bytes in
    // flight to cover the HBM latency
    for (; i + 3 * stride < nvec; i += 4 * stride) {
        const uint4 q0 = __ldg(xv + i), q1 = __ldg(xv + i + stride), q2 = __ldg(xv + i + 2 * stride),
                    q3 = __ldg(xv + i + 3 * stride);
        fold(q0);
        fold(q1);
        fold(q2);
        fold(q3);
    }
    // the last, partial round the same way (a few-token activation is nothing but this round): slots past the end
    // read as zeros, which never raise a maximum of magnitudes
    if (i < nvec) {
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        const uint4 q0 = __ldg(xv + i);
        const uint4 q1 = i + stride < nvec ? __ldg(xv + i + stride) : zero;
        const uint4 q2 = i + 2 * stride < nvec ? __ldg(xv + i + 2 * stride) : zero;
        fold(q0);
        fold(q1);
        fold(q2);
    }
    // ragged tail (numel not a multiple of the vector width): first threads of block 0
    if (blockIdx.x == 0) {
        const int64_t t = nvec * kPerVec + threadIdx.x;
        if (t < numel) {
            if (DT == NVFP4_DT_F32) acc = max(acc, static_cast<const uint32_t*>(x)[t] & 0x7fffffffu);
            else acc = umax2x16(acc, static_cast<const uint16_t*>(x)[t] & 0x7fffu);
        }
    }
    uint32_t bits;  // fp32 magnitude pattern of this thread's maximum
    if (DT == NVFP4_DT_F32) {
        bits = acc;
    } else {
        const uint32_t h = max(acc & 0xffffu, acc >> 16);
        if (DT == NVFP4_DT_BF16) bits = h << 16;
        else bits = __float_as_uint(__half2float(__ushort_as_half(static_cast<unsigned short>(h))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
    __shared__ uint32_t warp_max[kGsThreads / 32];
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = bits;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t b = 0;
        for (int i = 0; i < kGsThreads / 32; ++i) b = max(b, warp_max[i]);
        // a one-block grid (activations of a few tokens) has its maximum already: no trip through the scratch words,
        // whose three dependent atomics would cost more than the rest of the kernel
        bool last = gridDim.x == 1;
        uint32_t mx = b;
        if (!last) {
            atomicMax(&scratch[0], b);
            __threadfence();
            const uint32_t ticket = atomicAdd(&scratch[1], 1u);
            last = ticket == gridDim.x - 1;
            if (last) {
                __threadfence();
                mx = atomicExch(&scratch[0], 0u);
                scratch[1] = 0u;
            }
        }
        if (last) {
            const float amax = __uint_as_float(mx);
            const float inv_den = __fdiv_rn(1.0f, __fmul_rn(6.0f, fp8_max));
            const float gs = __fmul_rn(amax, inv_den);
            out[0] = gs;
            out[1] = __fdiv_rn(1.0f, gs);
        }
    }
}

}  // namespace
}  // namespace nvfp4

extern "C" int nvfp4_global_scale_launch(const void* x, int x_dtype, int64_t numel, float fp8_max, float* out,
                                         uint32_t* scratch, void* stream) {
    using namespace nvfp4;
    if (x_dtype < NVFP4_DT_BF16 || x_dtype > NVFP4_DT_F32) return NVFP4_ERR_BAD_ENUM;
    if (numel < 0) return NVFP4_ERR_BAD_SHAPE;
    if (!out || !scratch || (!x && numel > 0)) return NVFP4_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 3) ||
        (reinterpret_cast<uintptr_t>(scratch) & 3))
        return NVFP4_ERR_MISALIGNED;
    const int per_vec = (x_dtype == NVFP4_DT_F32) ? 4 : 8;
    const int64_t nvec = numel / per_vec;
    // up to four 16-byte loads per thread (all in flight at once) stay in one block, which needs no atomics
    int64_t blocks = nvec <= 4 * kGsThreads ? 1 : (nvec + kGsThreads - 1) / kGsThreads;
    // a few resident blocks per SM is enough to keep HBM busy; more only adds atomics
    // measured at 8192 x 8192 bf16: 1 CTA per SM 29.0 us, 2: 25.4, 3: 25.0, 4: 25.2-26.5, 8: 27.5, 16: 29.2
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t cap = static_cast<int64_t>(sms) * 3;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned g = static_cast<unsigned>(blocks);
    const dim3 grid(g), block(kGsThreads);
    switch (x_dtype) {
        case NVFP4_DT_BF16:
            return static_cast<int>(launch_dependent(global_scale_kernel<NVFP4_DT_BF16>, grid, block, 0, s, x, numel, fp8_max, out, scratch));
        case NVFP4_DT_F16:
            return static_cast<int>(launch_dependent(global_scale_kernel<NVFP4_DT_F16>, grid, block, 0, s, x, numel, fp8_max, out, scratch));
        default:
            return static_cast<int>(launch_dependent(global_scale_kernel<NVFP4_DT_F32>, grid, block, 0, s, x, numel, fp8_max, out, scratch));
    }
}
