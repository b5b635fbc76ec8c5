// Shared device helpers for the NVFP4 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "nvfp4_b200.h"

namespace nvfp4 {

constexpr int kBlock = 16;  // elements per scale block

__host__ __device__ inline int64_t round_up_i64(int64_t x, int64_t y) { return (x + y - 1) / y * y; }

// div.full.f32: the approximate full-range division Triton's `/` lowers to.
__device__ __forceinline__ float div_full(float a, float b) {
    float r;
    asm("div.full.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

__device__ __forceinline__ float rcp_approx_ftz(float a) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
    return r;
}

// raw E4M3 byte -> fp32 (exact).
__device__ __forceinline__ float e4m3_to_f32(uint32_t raw) {
    uint32_t h2;
    uint16_t in = static_cast<uint16_t>(raw & 0xffu);
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(in));
    float f;
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.f32.f16 %0, lo; }" : "=f"(f) : "r"(h2));
    return f;
}

// fp32 -> raw E4M3 byte, round-to-nearest-even, saturating to 448, NaN -> 0x7f.
__device__ __forceinline__ uint32_t f32_to_e4m3(float x) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(x));
    return r & 0xffu;
}

// Eight fp32 -> 32 bits of E2M1 nibbles, element 0 in the lowest nibble.
__device__ __forceinline__ uint32_t f32x8_to_e2m1x8(float x0, float x1, float x2, float x3, float x4,
                                                    float x5, float x6, float x7) {
    uint32_t out;
    asm("{ .reg .b8 b0, b1, b2, b3;\n"
        "  cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
        "  cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
        "  cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
        "  cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
        "  mov.b32 %0, {b0, b1, b2, b3}; }"
        : "=r"(out)
        : "f"(x0), "f"(x1), "f"(x2), "f"(x3), "f"(x4), "f"(x5), "f"(x6), "f"(x7));
    return out;
}

// E2M1-round two fp32 values and return the rounded values as fp32.
__device__ __forceinline__ void e2m1_round_pair(float xa, float xb, float& qa, float& qb) {
    asm("{ .reg .b8 b; .reg .b32 h; .reg .b16 lo, hi;\n"
        "  cvt.rn.satfinite.e2m1x2.f32 b, %3, %2;\n"
        "  cvt.rn.f16x2.e2m1x2 h, b;\n"
        "  mov.b32 {lo, hi}, h;\n"
        "  cvt.f32.f16 %0, lo;\n"
        "  cvt.f32.f16 %1, hi; }"
        : "=f"(qa), "=f"(qb)
        : "f"(xa), "f"(xb));
}

// Packed fp32x2 arithmetic (one instruction, two IEEE-rounded lanes).
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization attribute may start
// while the kernel before it on the stream is still running; griddep_wait() is where it stops until that kernel has
// finished and its writes are visible (it returns at once when there is nothing to wait for).  griddep_launch() is
// the other half: the running kernel says that the next one may start being scheduled (a hint; harmless when the
// next launch did not ask for it).
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Reads that follow griddep_wait().  The compiler takes a non-coherent load (__ldg) to read memory that never changes
// and may move it ahead of any barrier, the wait included - where the kernel before this one has not written the data
// yet.  after_wait(p) hands a pointer back as a value produced behind the wait, so that loads through it stay there
// (volatile asm statements keep their order); load_f32_after_wait is a plain coherent load for single words.
template <class T>
__device__ __forceinline__ T* after_wait(T* p) {
    asm volatile("" : "+l"(p)::"memory");
    return p;
}
__device__ __forceinline__ float load_f32_after_wait(const float* p) {
    float v;
    asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

// 1 (default): the library's kernels are launched with the programmatic-stream-serialization attribute; 0: plain
// launches.  One switch for the whole library (testing hook: nvfp4_gemm_tune_pdl); defined in status.cu.
extern int g_dependent_launch;

// kernel<<<grid, block, smem, stream>>>(args...) as a programmatic dependent launch.  The kernel must call
// griddep_wait() before its first access to global memory that an earlier kernel on the stream may write or read.
template <typename... Params, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_dependent_launch ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Byte offset of block (row, col) in the 128x4-tiled scale layout.
__host__ __device__ inline int64_t swizzled_scale_offset(int64_t row, int64_t col, int64_t k_pad) {
    return (row >> 7) * (k_pad * 128) + (col >> 2) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (col & 3);
}

}  // namespace nvfp4
