// Global-scale reduction for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to obtain scratch memory at the point where they need
// the tensor-wide scale: a plugin that is handed raw device pointers by a runtime that owns every
// allocation, an inference engine that has frozen its memory pool before the first request, or
// code that runs while device allocation is forbidden.  cudaMalloc (and a framework allocator
// that may fall through to it) is not an option for them, yet the reduction needs a place where
// thread blocks can leave their partial maxima.
//
// nvfp4_global_scale_launch_static therefore keeps that scratch inside the library image: a
// file-scope __device__ array of NVFP4_STATIC_SCRATCH_WORDS 32-bit words (16.25 KiB), present
// on every GPU that loads the library until the process exits.  Each thread block reduces a fixed
// 128 KiB chunk of the input and writes one partial maximum into its slot; the last block to
// arrive folds the slots and writes the result.  The slot count bounds the input size: at most
// NVFP4_STATIC_MAX_BYTES (512 MiB) of input; larger tensors are rejected with NVFP4_ERR_STATIC_SCRATCH.
//
// Rules for callers
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress) with
//     that device current and caches it.  Make that first call outside any stream capture.
//   * All calls on a device share the one array.  The arrival counter is cleared at the start of
//     every call (an asynchronous 4-byte memset on `stream`) and partial slots are rewritten
//     before they are read, so stale contents of an earlier call never leak into a result.
//     Two calls that can run concurrently on the same GPU (different streams, or two host threads)
//     race on the array and must be serialised by the caller.
//   * Nothing is allocated or freed: no cudaMalloc / cudaFree, no library workspace.
// Results are bit-identical to nvfp4_global_scale_launch (maximum of magnitude bit patterns, then
// the same two fp32 operations).
#include <cuda_fp16.h>

#include <atomic>

#include "common.cuh"

namespace nvfp4 {
namespace {

constexpr int kThreads = 512;
constexpr int kVecPerThread = 16;                                   // 16-byte vectors per thread
constexpr int64_t kChunkBytes = int64_t(kThreads) * kVecPerThread * 16;   // 128 KiB per block
constexpr int kMaxBlocks = 4096;
constexpr int kHeaderWords = 64;                                    // word 0: arrival counter; rest: padding
constexpr int kScratchWords = kHeaderWords + kMaxBlocks;            // 4160 words = 16.25 KiB
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) uint32_t g_static_scratch[kScratchWords];

template <int DT>
__global__ void __launch_bounds__(kThreads) global_scale_static_kernel(const void* x, int64_t numel, float fp8_max,
                                                                       float* out, uint32_t* scratch) {
    constexpr int kPerVec = (DT == NVFP4_DT_F32) ? 4 : 8;
    const int64_t nvec = numel / kPerVec;
    const uint4* xv = static_cast<const uint4*>(x);
    const int64_t first = static_cast<int64_t>(blockIdx.x) * kThreads * kVecPerThread + threadIdx.x;
    uint32_t acc = 0;
#pragma unroll 4
    for (int k = 0; k < kVecPerThread; ++k) {
        const int64_t i = first + static_cast<int64_t>(k) * kThreads;
        if (i < nvec) {
            const uint4 q = __ldg(xv + i);
            if (DT == NVFP4_DT_F32)
                acc = max(acc, max(max(q.x & 0x7fffffffu, q.y & 0x7fffffffu), max(q.z & 0x7fffffffu, q.w & 0x7fffffffu)));
            else
                acc = __vmaxu2(acc, __vmaxu2(__vmaxu2(q.x & 0x7fff7fffu, q.y & 0x7fff7fffu),
                                             __vmaxu2(q.z & 0x7fff7fffu, q.w & 0x7fff7fffu)));
        }
    }
    if (blockIdx.x == 0) {  // elements past the last whole vector
        const int64_t t = nvec * kPerVec + threadIdx.x;
        if (t < numel) {
            if (DT == NVFP4_DT_F32) acc = max(acc, static_cast<const uint32_t*>(x)[t] & 0x7fffffffu);
            else acc = __vmaxu2(acc, static_cast<const uint16_t*>(x)[t] & 0x7fffu);
        }
    }
    uint32_t bits;
    if (DT == NVFP4_DT_F32) {
        bits = acc;
    } else {
        const uint32_t h = max(acc & 0xffffu, acc >> 16);
        bits = (DT == NVFP4_DT_BF16) ? (h << 16)
                                     : __float_as_uint(__half2float(__ushort_as_half(static_cast<unsigned short>(h))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
    __shared__ uint32_t warp_max[kThreads / 32];
    __shared__ bool is_last;
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = bits;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t b = 0;
        for (int i = 0; i < kThreads / 32; ++i) b = max(b, warp_max[i]);
        scratch[kHeaderWords + blockIdx.x] = b;
        __threadfence();
        is_last = atomicAdd(&scratch[0], 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    uint32_t m = 0;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += kThreads) m = max(m, __ldcg(&scratch[kHeaderWords + i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t b = 0;
        for (int i = 0; i < kThreads / 32; ++i) b = max(b, warp_max[i]);
        const float amax = __uint_as_float(b);
        const float inv_den = __fdiv_rn(1.0f, __fmul_rn(6.0f, fp8_max));
        const float gs = __fmul_rn(amax, inv_den);
        out[0] = gs;
        out[1] = __fdiv_rn(1.0f, gs);
        scratch[0] = 0u;
    }
}

// Device address of g_static_scratch, looked up once per device with that device current.  The address belongs to
// the device's primary context: it stays valid until that context is destroyed (cudaDeviceReset), after which this
// library must not be used from the old process state anyway.  Entries are atomics: two host threads making their
// first call at once both look the address up and store the same value.
uint32_t* static_scratch_for_current_device(cudaError_t* err) {
    static std::atomic<uint32_t*> cache[kMaxDevices] = {};
    int dev = -1;
    *err = cudaGetDevice(&dev);
    if (*err != cudaSuccess) return nullptr;
    if (dev < 0 || dev >= kMaxDevices) {
        *err = cudaErrorInvalidDevice;
        return nullptr;
    }
    uint32_t* addr = cache[dev].load(std::memory_order_acquire);
    if (!addr) {
        void* p = nullptr;
        *err = cudaGetSymbolAddress(&p, g_static_scratch);
        if (*err != cudaSuccess) return nullptr;
        addr = static_cast<uint32_t*>(p);
        cache[dev].store(addr, std::memory_order_release);
    }
    return addr;
}

}  // namespace
}  // namespace nvfp4

extern "C" int64_t nvfp4_global_scale_static_max_bytes(void) { return nvfp4::kChunkBytes * nvfp4::kMaxBlocks; }

extern "C" int nvfp4_global_scale_launch_static(const void* x, int x_dtype, int64_t numel, float fp8_max, float* out,
                                                void* stream) {
    using namespace nvfp4;
    if (x_dtype < NVFP4_DT_BF16 || x_dtype > NVFP4_DT_F32) return NVFP4_ERR_BAD_ENUM;
    if (numel < 0) return NVFP4_ERR_BAD_SHAPE;
    if (!out || (!x && numel > 0)) return NVFP4_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 3)) return NVFP4_ERR_MISALIGNED;
    const int64_t elem_bytes = (x_dtype == NVFP4_DT_F32) ? 4 : 2;
    if (numel > nvfp4_global_scale_static_max_bytes() / elem_bytes) return NVFP4_ERR_STATIC_SCRATCH;
    cudaError_t err = cudaSuccess;
    uint32_t* scratch = static_scratch_for_current_device(&err);
    if (!scratch) return static_cast<int>(err);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    err = cudaMemsetAsync(scratch, 0, sizeof(uint32_t), s);  // the arrival counter must start at zero
    if (err != cudaSuccess) return static_cast<int>(err);
    const int64_t bytes = numel * elem_bytes;
    int64_t blocks = (bytes + kChunkBytes - 1) / kChunkBytes;
    if (blocks < 1) blocks = 1;
    const unsigned g = static_cast<unsigned>(blocks);
    switch (x_dtype) {
        case NVFP4_DT_BF16: global_scale_static_kernel<NVFP4_DT_BF16><<<g, kThreads, 0, s>>>(x, numel, fp8_max, out, scratch); break;
        case NVFP4_DT_F16: global_scale_static_kernel<NVFP4_DT_F16><<<g, kThreads, 0, s>>>(x, numel, fp8_max, out, scratch); break;
        default: global_scale_static_kernel<NVFP4_DT_F32><<<g, kThreads, 0, s>>>(x, numel, fp8_max, out, scratch); break;
    }
    return static_cast<int>(cudaGetLastError());
}
