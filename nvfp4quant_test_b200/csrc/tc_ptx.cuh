// tcgen05 / TMA / mbarrier wrappers and descriptor helpers shared by the NVFP4 GEMM kernels (sm_100a only).
// Included by gemm.cu alone: the status word below is one per library.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"

namespace nvfp4 {
namespace gemm {


constexpr int kBM = 128;          // rows of A per tile
constexpr int kBKBytes = 128;     // bytes of K per stage row (= 256 FP4 elements, one swizzle row)
constexpr int kBK = 256;          // elements of K per stage
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
// Every tile / pair kernel asks for the whole shared memory of an SM (227 KiB), whatever its ring needs: a CTA that
// takes all 512 TMEM columns must be alone on its SM, and identical footprints keep concurrently running GEMM
// kernels from being placed differently.
constexpr int kGemmDynSmemBytes = 232448;
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s: far above any legitimate wait
__device__ uint64_t g_gemm_wait_limit_ns = kWaitLimitNs;   // what the waits use; settable from the host (nvfp4_gemm_set_wait_limit_ns)

__device__ uint32_t g_gemm_status;  // 0 = ok; else (role << 24) | detail of the wait that expired

// Progress counters for debugging builds (-DNVFP4_GEMM_TRACE): how many CTAs of each kernel family passed each point.
#ifdef NVFP4_GEMM_TRACE
__device__ uint32_t* g_gemm_trace = nullptr;
__device__ __forceinline__ void trace_mark(int family, int point) {
    uint32_t* t = g_gemm_trace;
    if (t) atomicAdd(t + family * 16 + point, 1u);
}
#else
__device__ __forceinline__ void trace_mark(int, int) {}
#endif

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait.  Returns false (after recording `code`) when the limit expires or another role
// has already given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t code) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_timer_ns() - t0 > g_gemm_wait_limit_ns) {
            *abort_flag = 1;
            atomicCAS(&g_gemm_status, 0u, code);
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld_32x32b_x32(uint32_t taddr, uint32_t v[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One lane of a converged warp (elect.sync).  The MMA warp runs its loops with all 32 lanes so that stage
// indices, descriptors and TMEM addresses stay warp-uniform (they then live in uniform registers, which is
// what the tcgen05 instructions take); only the tcgen05 instruction itself is issued by the elected lane.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{ .reg .b32 rx; .reg .pred px; elect.sync rx|px, 0xffffffff; selp.u32 %0, 1, 0, px; }" : "=r"(pred));
    return pred != 0;
}
// Bounded wait executed by the whole warp; the answer is lane 0's, so it is uniform.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t code) {
    const bool ok = mbar_wait(bar, parity, abort_flag, code);
    return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
}

// Descriptors as (lo, hi) words: hi is a constant per operand kind, lo = (smem address >> 4) [| LBO], so stepping
// through a tile is one 32-bit add.  Keeps the single issuing thread to a few instructions per tcgen05 op.
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024 B, version 1, 128-byte swizzle
constexpr uint32_t kDescHiSf = (128u >> 4) | (1u << 14);                   // SBO 128 B, version 1, no swizzle
__device__ __forceinline__ void tc_cp_lohi(uint32_t taddr, uint32_t lo) {
    asm volatile("{ .reg .b64 d; mov.b64 d, {%1, %2}; tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d; }" ::"r"(taddr),
                 "r"(lo), "r"(kDescHiSf)
                 : "memory");
}
__device__ __forceinline__ void tc_mma_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t sfa_tmem,
                                            uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; .reg .b64 da, db; setp.ne.b32 p, %4, 0; mov.b64 da, {%1, %7}; mov.b64 db, {%2, %7};\n"
        "  tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %3, [%5], [%6], p; }" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem), "r"(kDescHiSw128)
        : "memory");
}

// Instruction descriptor: E2M1 x E2M1, UE4M3 scales, K-major A and B, M = 128, N = BN, K = 64.
template <int BN>
__device__ __forceinline__ constexpr uint32_t instr_desc() {
    return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) | (0u << 23) |
           (static_cast<uint32_t>(kBM >> 4) << 24);
}


}  // namespace gemm
}  // namespace nvfp4
