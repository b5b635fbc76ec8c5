// NVFP4 block-scaled GEMM for sm_100a:
//   out[M, N] (bf16) = alpha * sum_k dq(a)[m, k] * dq(b)[n, k]
// with a, b packed E2M1 (K-major) and one UE4M3 scale per 16 elements stored in the
// 128x4-tiled layout the quantizer writes.  Replaces vllm's cutlass_scaled_fp4_mm
// (vllm/_custom_ops.py:741-752), the consumer efsotr/nvfp4quant_test names at README.md:68.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      producer: TMA tile loads of A / B (128-byte swizzle) and bulk copies of the
//               scale tiles into a shared-memory ring (6 stages with 128-wide tiles, 4 with 256-wide)
//   warp 1      MMA issuer: tcgen05.cp scale tiles smem -> TMEM, then
//               tcgen05.mma.kind::mxf4nvf4.block_scale (K = 64 per instruction) into a TMEM
//               accumulator; tcgen05.commit releases ring slots / publishes the accumulator
//   warps 2-5   epilogue: tcgen05.ld the accumulator, * alpha, -> bf16, store
// No cluster multicast is used anywhere.  Every barrier wait is bounded: on expiry the kernel
// records a status word and every role leaves its loop, so a fault in the pipeline logic
// surfaces as an error code rather than a hung device.
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
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s: far above any legitimate wait

__device__ uint32_t g_gemm_status;  // 0 = ok; else (role << 24) | detail of the wait that expired

template <int BN>
struct Cfg {
    static constexpr int kNG = (BN + 127) / 128;            // 128-row scale groups a B tile touches (a 64-row tile: half of one)
    static constexpr int kAcc = (BN <= 128) ? 2 : 1;        // accumulator buffers in TMEM
    static constexpr int kABytes = kBM * kBKBytes;          // 16 KiB
    static constexpr int kBBytes = BN * kBKBytes;
    static constexpr int kSfaBytes = 2048;                  // 128 rows x 16 blocks
    static constexpr int kSfbBytes = 2048 * kNG;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    // ring depth: as many stages as fit in shared memory (the bytes in flight per SM are what keeps HBM busy when
    // few CTAs stream a long K)
    static constexpr int kStages = (BN == 64) ? 8 : (BN == 128) ? 6 : 4;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
    // scale factors sit behind the accumulators, in two sets used by alternate K tiles so that the
    // copies for the next K tile do not have to wait for the MMAs still reading the current set
    static constexpr int kSfSetCols = 16 + 16 * kNG;
    static constexpr int kSfaCol = kAcc * BN;               // TMEM column of the A scales (set 0)
    static constexpr int kSfbCol = kSfaCol + 16;            // TMEM column of the B scales (set 0)
    static_assert(kSfaCol + 2 * kSfSetCols <= kTmemCols, "TMEM budget");
};

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
        if (global_timer_ns() - t0 > kWaitLimitNs) {
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
// Bounded wait executed by the whole warp; the verdict is lane 0's, so it is uniform.
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

struct GemmParams {
    const uint8_t* sfa;
    const uint8_t* sfb;
    const float* alpha;
    __nv_bfloat16* out;
    int M, N, K;
    int64_t sf_group_stride;  // bytes between consecutive 128-row scale groups = round_up(K/16, 4) * 128
    int sfa_groups, sfb_groups;  // 128-row groups present in each scale buffer
    // single-CTA kernel only: K is cut into k_splits ranges of k_tiles_per_split stages; with more than one range
    // each work item writes an fp32 partial tile to `partial` ([k_splits, M, N]) and a second kernel sums them.
    int k_splits, k_tiles_per_split;
    int k_rotate;             // != 0: each tile starts its K loop at a different stage (spreads requests for shared A rows)
    float* partial;
    int raster_group;         // m-tiles per band of the tile numbering (see tile_to_mn)
};

// Tile index -> (m tile, n tile).  Tiles are numbered in bands of `group` m-tiles: inside a band the m index runs
// fastest, then n.  The CTAs that run at the same time then cover a roughly square patch of the output, so every A
// tile and every B tile is being fetched by a moderate number of CTAs at once instead of one B tile by all of them.
__device__ __forceinline__ void tile_to_mn(int tile, int m_tiles, int n_tiles, int group, int& mt, int& nt) {
    const int band = tile / (group * n_tiles);
    const int first_m = band * group;
    const int rows = min(group, m_tiles - first_m);
    const int in_band = tile - band * group * n_tiles;
    nt = in_band / rows;
    mt = first_m + in_band - nt * rows;
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - raw_addr);
    // ring: [stage][A | B | SFA | SFB]; then barriers
    uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + C::kStages * C::kStageBytes);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (C::kStages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * C::kStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * C::kStages + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * C::kStages + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t*>(tmem_slot))),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int m_tiles = (p.M + kBM - 1) / kBM;
    const int n_tiles = (p.N + BN - 1) / BN;
    const int mn_tiles = m_tiles * n_tiles;
    const int total_tiles = mn_tiles * p.k_splits;   // work items: (K range, n tile, m tile)
    const int k_tiles = (p.K + kBK - 1) / kBK;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        {
            const bool issuer = elect_one();
            if (issuer) {
                asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
                asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
            }
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int ks = tile / mn_tiles, t2 = tile - ks * mn_tiles;
                int mt, nt;
                tile_to_mn(t2, m_tiles, n_tiles, p.raster_group, mt, nt);
                const int kt_begin = ks * p.k_tiles_per_split;
                const int kcount = min(k_tiles, kt_begin + p.k_tiles_per_split) - kt_begin;
                const int rot = p.k_rotate ? (t2 * 5) % kcount : 0;
                for (int i = 0; i < kcount; ++i) {
                    const int kt = kt_begin + (i + rot) % kcount;
                    if (!(ok = mbar_wait_warp(empty_bar(stage), phase ^ 1u, abort_flag, (1u << 24) | kt))) break;
                    const int kb_count = min(4, (p.K - kt * kBK + 63) / 64);  // 64-element K blocks in this stage
                    const uint32_t sf_bytes = 512u * kb_count;
                    int sfb_present = 0;
                    const int grp0 = BN == 64 ? (nt >> 1) : nt * C::kNG;   // first 128-row scale group of this B tile
                    for (int g = 0; g < C::kNG; ++g) sfb_present += (grp0 + g < p.sfb_groups) ? 1 : 0;
                    const uint32_t tx = C::kABytes + C::kBBytes + sf_bytes * (1 + sfb_present);
                    const uint32_t sbase = base + stage * C::kStageBytes;
                    if (issuer) {
                    mbar_expect_tx(full_bar(stage), tx);
                    tma_load_2d(sbase, &tmap_a, kt * kBKBytes, mt * kBM, full_bar(stage));
                    tma_load_2d(sbase + C::kABytes, &tmap_b, kt * kBKBytes, nt * BN, full_bar(stage));
                    bulk_load_1d(sbase + C::kABytes + C::kBBytes,
                                 p.sfa + static_cast<int64_t>(mt) * p.sf_group_stride + static_cast<int64_t>(kt) * 2048,
                                 sf_bytes, full_bar(stage));
                    for (int g = 0; g < C::kNG; ++g) {
                        const int grp = grp0 + g;
                        if (grp < p.sfb_groups)
                            bulk_load_1d(sbase + C::kABytes + C::kBBytes + C::kSfaBytes + g * 2048,
                                         p.sfb + static_cast<int64_t>(grp) * p.sf_group_stride +
                                             static_cast<int64_t>(kt) * 2048,
                                         sf_bytes, full_bar(stage));
                    }
                    }
                    __syncwarp();
                    if (++stage == C::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        {
            const bool issuer = elect_one();
            constexpr uint32_t idesc = instr_desc<BN>();
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                if (!(ok = mbar_wait_warp(tempty_bar(acc), acc_phase ^ 1u, abort_flag, (2u << 24) | 0xffff))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                const int ks = tile / mn_tiles, t2 = tile - ks * mn_tiles;
                // a 64-row B tile is one half of a 128-row scale group: rows 64..127 sit two TMEM columns further on
                uint32_t sfb_half = 0;
                if (BN == 64) {
                    int mt, nt;
                    tile_to_mn(t2, m_tiles, n_tiles, p.raster_group, mt, nt);
                    sfb_half = 2u * (nt & 1);
                }
                const int kt_begin = ks * p.k_tiles_per_split;
                const int kcount = min(k_tiles, kt_begin + p.k_tiles_per_split) - kt_begin;
                const int rot = p.k_rotate ? (t2 * 5) % kcount : 0;
                for (int i = 0; i < kcount; ++i) {
                    const int kt = kt_begin + (i + rot) % kcount;
                    if (!(ok = mbar_wait_warp(full_bar(stage), phase, abort_flag, (2u << 24) | kt))) break;
                    tc_fence_after();
                    const int kb_count = min(4, (p.K - kt * kBK + 63) / 64);
                    const uint32_t sbase = base + stage * C::kStageBytes;
                    const uint32_t a_lo = ((sbase & 0x3ffffu) >> 4) | (1u << 16);
                    const uint32_t b_lo = a_lo + (C::kABytes >> 4);
                    const uint32_t sfa_lo = ((sbase + C::kABytes + C::kBBytes) & 0x3ffffu) >> 4;
                    const uint32_t sfb_lo = sfa_lo + (C::kSfaBytes >> 4);
                    const uint32_t set = (i & 1) * C::kSfSetCols;
                    const uint32_t sfa_t = tmem_base + C::kSfaCol + set;
                    const uint32_t sfb_t = tmem_base + C::kSfbCol + set;
                    const uint32_t sfb_use = sfb_t + sfb_half;
                    const uint32_t first = i > 0 ? 1u : 0u;
                    if (!issuer) {
                        // nothing to issue on this lane
                    } else if (kb_count == 4) {
#pragma unroll
                        for (int kb = 0; kb < 4; ++kb) {
                            tc_cp_lohi(sfa_t + 4 * kb, sfa_lo + 32 * kb);
#pragma unroll
                            for (int g = 0; g < C::kNG; ++g)
                                tc_cp_lohi(sfb_t + 4 * C::kNG * kb + 4 * g, sfb_lo + 128 * g + 32 * kb);
                        }
#pragma unroll
                        for (int kb = 0; kb < 4; ++kb)   // 32 bytes of K per instruction: start address + 2 (x16 B)
                            tc_mma_lohi(d_tmem, a_lo + 2 * kb, b_lo + 2 * kb, idesc, sfa_t + 4 * kb, sfb_use + 4 * C::kNG * kb,
                                        kb == 0 ? first : 1u);
                    } else {
                        for (int kb = 0; kb < kb_count; ++kb) {
                            tc_cp_lohi(sfa_t + 4 * kb, sfa_lo + 32 * kb);
                            for (int g = 0; g < C::kNG; ++g)
                                tc_cp_lohi(sfb_t + 4 * C::kNG * kb + 4 * g, sfb_lo + 128 * g + 32 * kb);
                        }
                        for (int kb = 0; kb < kb_count; ++kb)
                            tc_mma_lohi(d_tmem, a_lo + 2 * kb, b_lo + 2 * kb, idesc, sfa_t + 4 * kb, sfb_use + 4 * C::kNG * kb,
                                        kb == 0 ? first : 1u);
                    }
                    if (issuer) tc_commit(empty_bar(stage));  // slot reusable once these MMAs have read it
                    __syncwarp();
                    if (++stage == C::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                if (issuer) tc_commit(tfull_bar(acc));  // accumulator complete
                __syncwarp();
                if (++acc == C::kAcc) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int sp = warp & 3;  // TMEM sub-partition this warp may read: lanes 32*sp .. 32*sp+31
        const float alpha = __ldg(p.alpha);
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        const bool vec_ok = (p.N % 8) == 0;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
            const int ks = tile / mn_tiles, t2 = tile - ks * mn_tiles;
            int mt, nt;
            tile_to_mn(t2, m_tiles, n_tiles, p.raster_group, mt, nt);
            ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, (3u << 24) | (tile & 0xffff));
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            tc_fence_after();
            const int row = mt * kBM + sp * 32 + lane;
            __nv_bfloat16* orow = p.out + static_cast<int64_t>(row) * p.N;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tc_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(sp * 32) << 16) + acc * BN + c * 32, v);
                tc_ld_wait();
                const int col0 = nt * BN + c * 32;
                if (p.k_splits > 1) {
                    // fp32 partial of this K range; alpha and the bf16 rounding happen in the reduction kernel
                    if (row < p.M && col0 < p.N) {
                        float* prow = p.partial + (static_cast<int64_t>(ks) * p.M + row) * p.N + col0;
                        if ((p.N % 4) == 0 && col0 + 32 <= p.N) {
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                *reinterpret_cast<uint4*>(prow + 4 * q) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                        } else {
                            for (int e = 0; e < 32; ++e)
                                if (col0 + e < p.N) prow[e] = __uint_as_float(v[e]);
                        }
                    }
                } else if (row < p.M && col0 < p.N) {
                    if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float lo = __fmul_rn(__uint_as_float(v[q * 8 + 2 * e]), alpha);
                                const float hi = __fmul_rn(__uint_as_float(v[q * 8 + 2 * e + 1]), alpha);
                                __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
                                w[e] = *reinterpret_cast<uint32_t*>(&b2);
                            }
                            *reinterpret_cast<uint4*>(orow + col0 + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
                        for (int e = 0; e < 32; ++e)
                            if (col0 + e < p.N) orow[col0 + e] = __float2bfloat16_rn(__fmul_rn(__uint_as_float(v[e]), alpha));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            if (++acc == C::kAcc) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    if (*abort_flag) {
        // give any bulk copy still in flight time to land before shared memory is released
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// out[m, n] = bf16(alpha * sum over K ranges of partial[s][m][n]); ranges are added in ascending order.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, const float* alpha_ptr,
                                                            __nv_bfloat16* __restrict__ out, int64_t mn, int splits) {
    const float alpha = __ldg(alpha_ptr);
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < mn; i += static_cast<int64_t>(gridDim.x) * 256) {
        float acc = partial[i];
        for (int s = 1; s < splits; ++s) acc = __fadd_rn(acc, partial[static_cast<int64_t>(s) * mn + i]);
        out[i] = __float2bfloat16_rn(__fmul_rn(acc, alpha));
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// [rows, k_bytes] row-major byte matrix, box = 128 bytes x box_rows, 128-byte swizzle, zero fill.
static int make_operand_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t k_bytes, int box_rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return NVFP4_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(k_bytes), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(k_bytes)};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(kBKBytes), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? NVFP4_OK : NVFP4_ERR_UNSUPPORTED;
}

template <int BN>
static int launch(const uint8_t* a, const uint8_t* b, const GemmParams& p, cudaStream_t stream) {
    using C = Cfg<BN>;
    CUtensorMap ma, mb;
    int st = make_operand_map(&ma, a, p.M, p.K / 2, kBM);
    if (st != NVFP4_OK) return st;
    st = make_operand_map(&mb, b, p.N, p.K / 2, BN);
    if (st != NVFP4_OK) return st;
    // function attributes are per device; setting it on every launch keeps multi-device processes correct
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = ((p.M + kBM - 1) / kBM) * ((p.N + BN - 1) / BN) * p.k_splits;
    const int grid = tiles < sms ? tiles : sms;
    gemm_kernel<BN><<<grid, kThreads, C::kSmemBytes, stream>>>(ma, mb, p);
    e = cudaGetLastError();
    if (e != cudaSuccess || p.k_splits == 1) return static_cast<int>(e);
    const int64_t mn = static_cast<int64_t>(p.M) * p.N;
    int64_t rblocks = (mn + 255) / 256;
    if (rblocks > 148 * 8) rblocks = 148 * 8;
    splitk_reduce_kernel<<<static_cast<unsigned>(rblocks), 256, 0, stream>>>(p.partial, p.alpha, p.out, mn, p.k_splits);
    return static_cast<int>(cudaGetLastError());
}


// =============================================================================================
// Two-CTA variant (cta_group::2): a CTA pair owns a 256 x 256 output tile.  Each CTA loads its own
// 128 rows of A and HALF of the B tile (128 of the 256 weight rows); the pair's tensor cores read
// both halves, so B crosses L2 -> shared memory once per pair instead of once per CTA.  No
// multicast load is involved: every TMA copy has exactly one destination CTA.  The CTA with
// cluster rank 0 issues all MMAs; copies of both CTAs report to rank 0's "full" barrier
// (cp.async.bulk.tensor ... .cta_group::2), and tcgen05.commit signals the "empty" and
// "accumulator ready" barriers of both CTAs.
// =============================================================================================
namespace pair {

// Tile-width dependent constants of the pair kernel.  BN = 256: one accumulator (256 columns) per CTA.
// BN = 192: two accumulators (2 x 192 columns), so the epilogue of one tile overlaps the MMAs of the next.
template <int BN>
struct PairCfg {
    static constexpr int kAcc = (BN == 192) ? 2 : 1;
    static constexpr int kABytes = 128 * kBKBytes;          // this CTA's 128 rows of A
    static constexpr int kBBytes = (BN / 2) * kBKBytes;     // this CTA's half of the B rows
    static constexpr int kSfaBytes = 2048;                  // scales of this CTA's A rows
    static constexpr int kSfbBytes = 4096;                  // two 128-row scale groups cover the B tile
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    static constexpr int kStages = (BN == 192) ? 6 : 5;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
    static constexpr int kSfaCol = kAcc * BN;               // scale set 0; set 1 follows 48 columns later
    static constexpr int kSfbCol = kSfaCol + 16;
    static constexpr int kSfSetCols = 48;
    static_assert(kSfaCol + 2 * kSfSetCols <= kTmemCols, "TMEM budget");
    static_assert(kStageBytes % 1024 == 0, "stage alignment for the 128-byte swizzle");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// tile load whose completion bytes are reported to a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar_cluster)
        : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"(static_cast<uint16_t>(3))
                 : "memory");
}
__device__ __forceinline__ void tc_cp_pair(uint32_t taddr, uint32_t lo) {
    asm volatile("{ .reg .b64 d; mov.b64 d, {%1, %2}; tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], d; }" ::"r"(taddr),
                 "r"(lo), "r"(kDescHiSf)
                 : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; .reg .b64 da, db; setp.ne.b32 p, %4, 0; mov.b64 da, {%1, %7}; mov.b64 db, {%2, %7};\n"
        "  tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %3, [%5], [%6], p; }" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem), "r"(kDescHiSw128)
        : "memory");
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                 const GemmParams p) {
    using C = PairCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - raw_addr);
    uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + C::kStages * C::kStageBytes);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (C::kStages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * C::kStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * C::kStages + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * C::kStages + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();           // 0 = leader (issues the MMAs)
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full_bar(s), 1);    // leader's producer; bytes of both CTAs' copies land here
            mbar_init(empty_bar(s), 1);   // one tcgen05.commit
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 8);  // 4 epilogue warps of each CTA
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t*>(tmem_slot))),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the peer's barriers exist before anything is signalled across CTAs
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int m_tiles = (p.M + 255) / 256;
    const int n_tiles = (p.N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    const int k_tiles = (p.K + kBK - 1) / kBK;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (both CTAs)
        {
            const bool issuer = elect_one();
            if (issuer) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_sfa) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_sfb) : "memory");
            }
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair_id; ok && tile < total_tiles; tile += num_pairs) {
                int mt, nt;
                tile_to_mn(tile, m_tiles, n_tiles, p.raster_group, mt, nt);
                for (int kt = 0; kt < k_tiles; ++kt) {
                    if (!(ok = mbar_wait_warp(empty_bar(stage), phase ^ 1u, abort_flag, (1u << 24) | kt))) break;
                    if (issuer) {
                    if (rank == 0) mbar_expect_tx(full_bar(stage), 2u * C::kStageBytes);
                    const uint32_t lead_full = map_to_cta(full_bar(stage), 0);
                    const uint32_t sbase = base + stage * C::kStageBytes;
                    tma_load_2d_pair(sbase, &tmap_a, kt * kBKBytes, mt * 256 + static_cast<int>(rank) * 128, lead_full);
                    tma_load_2d_pair(sbase + C::kABytes, &tmap_b, kt * kBKBytes, nt * BN + static_cast<int>(rank) * (BN / 2), lead_full);
                    // scale tiles: x counts 8-byte elements (2048 B per K tile), y = 128-row group
                    tma_load_2d_pair(sbase + C::kABytes + C::kBBytes, &tmap_sfa, kt * 256, mt * 2 + static_cast<int>(rank), lead_full);
                    tma_load_2d_pair(sbase + C::kABytes + C::kBBytes + C::kSfaBytes, &tmap_sfb, kt * 256, (nt * BN) / 128, lead_full);
                    tma_load_2d_pair(sbase + C::kABytes + C::kBBytes + C::kSfaBytes + 2048, &tmap_sfb, kt * 256, (nt * BN) / 128 + 1, lead_full);
                    }
                    __syncwarp();
                    if (++stage == C::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader only)
        if (rank == 0) {
            const bool issuer = elect_one();
            constexpr uint32_t idesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                                       (static_cast<uint32_t>(256 >> 4) << 24);
            int stage = 0;
            uint32_t phase = 0, acc_phase = 0;
            int acc = 0;
            bool ok = true;
            for (int tile = pair_id; ok && tile < total_tiles; tile += num_pairs) {
                if (!(ok = mbar_wait_warp(tempty_bar(acc), acc_phase ^ 1u, abort_flag, (2u << 24) | 0xffff))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                // a 192-wide tile starts 0 or 64 rows into its first scale group: 64 rows = 2 TMEM columns
                int mt_unused, nt_of_tile;
                tile_to_mn(tile, m_tiles, n_tiles, p.raster_group, mt_unused, nt_of_tile);
                const uint32_t sfb_shift = (nt_of_tile * BN % 128) / 32;
                for (int kt = 0; kt < k_tiles; ++kt) {
                    if (!(ok = mbar_wait_warp(full_bar(stage), phase, abort_flag, (2u << 24) | kt))) break;
                    tc_fence_after();
                    const int kb_count = min(4, (p.K - kt * kBK + 63) / 64);
                    const uint32_t sbase = base + stage * C::kStageBytes;
                    const uint32_t a_lo = ((sbase & 0x3ffffu) >> 4) | (1u << 16);
                    const uint32_t b_lo = a_lo + (C::kABytes >> 4);
                    const uint32_t sfa_lo = ((sbase + C::kABytes + C::kBBytes) & 0x3ffffu) >> 4;
                    const uint32_t sfb_lo = sfa_lo + (C::kSfaBytes >> 4);
                    const uint32_t set = (kt & 1) * C::kSfSetCols;
                    const uint32_t sfa_t = tmem_base + C::kSfaCol + set;
                    const uint32_t sfb_t = tmem_base + C::kSfbCol + set;
                    const uint32_t first = kt > 0 ? 1u : 0u;
                    if (!issuer) {
                        // nothing to issue on this lane
                    } else if (kb_count == 4) {
#pragma unroll
                        for (int kb = 0; kb < 4; ++kb) {
                            tc_cp_pair(sfa_t + 4 * kb, sfa_lo + 32 * kb);
                            tc_cp_pair(sfb_t + 8 * kb, sfb_lo + 32 * kb);
                            tc_cp_pair(sfb_t + 8 * kb + 4, sfb_lo + 128 + 32 * kb);
                        }
#pragma unroll
                        for (int kb = 0; kb < 4; ++kb)
                            tc_mma_pair(d_tmem, a_lo + 2 * kb, b_lo + 2 * kb, idesc, sfa_t + 4 * kb, sfb_t + 8 * kb + sfb_shift,
                                        kb == 0 ? first : 1u);
                    } else {
                        for (int kb = 0; kb < kb_count; ++kb) {
                            tc_cp_pair(sfa_t + 4 * kb, sfa_lo + 32 * kb);
                            tc_cp_pair(sfb_t + 8 * kb, sfb_lo + 32 * kb);
                            tc_cp_pair(sfb_t + 8 * kb + 4, sfb_lo + 128 + 32 * kb);
                        }
                        for (int kb = 0; kb < kb_count; ++kb)
                            tc_mma_pair(d_tmem, a_lo + 2 * kb, b_lo + 2 * kb, idesc, sfa_t + 4 * kb, sfb_t + 8 * kb + sfb_shift,
                                        kb == 0 ? first : 1u);
                    }
                    if (issuer) tc_commit_pair(empty_bar(stage));   // frees this slot in both CTAs
                    __syncwarp();
                    if (++stage == C::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                if (issuer) tc_commit_pair(tfull_bar(acc));         // accumulators of both CTAs are complete
                __syncwarp();
                if (++acc == C::kAcc) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (both CTAs)
        const int sp = warp & 3;
        const float alpha = __ldg(p.alpha);
        uint32_t acc_phase = 0;
        int acc = 0;
        bool ok = true;
        const bool vec_ok = (p.N % 8) == 0;
        for (int tile = pair_id; ok && tile < total_tiles; tile += num_pairs) {
            int mt, nt;
            tile_to_mn(tile, m_tiles, n_tiles, p.raster_group, mt, nt);
            ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, (3u << 24) | (tile & 0xffff));
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            tc_fence_after();
            const int row = mt * 256 + static_cast<int>(rank) * 128 + sp * 32 + lane;
            __nv_bfloat16* orow = p.out + static_cast<int64_t>(row) * p.N;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tc_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(sp * 32) << 16) + acc * BN + c * 32, v);
                tc_ld_wait();
                const int col0 = nt * BN + c * 32;
                if (row < p.M && col0 < p.N) {
                    if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float lo = __fmul_rn(__uint_as_float(v[q * 8 + 2 * e]), alpha);
                                const float hi = __fmul_rn(__uint_as_float(v[q * 8 + 2 * e + 1]), alpha);
                                __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
                                w[e] = *reinterpret_cast<uint32_t*>(&b2);
                            }
                            *reinterpret_cast<uint4*>(orow + col0 + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
                        for (int e = 0; e < 32; ++e)
                            if (col0 + e < p.N) orow[col0 + e] = __float2bfloat16_rn(__fmul_rn(__uint_as_float(v[e]), alpha));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
            if (++acc == C::kAcc) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // neither CTA leaves while its partner may still signal or read it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// Scale buffer as a 2-D array of 8-byte words: row = 128-row group, 2048 B (one K tile) per box.
static int make_scale_map(CUtensorMap* map, const void* ptr, int64_t groups, int64_t group_stride_bytes) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return NVFP4_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(group_stride_bytes / 8), static_cast<cuuint64_t>(groups)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(group_stride_bytes)};
    cuuint32_t box[2] = {256, 1};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? NVFP4_OK : NVFP4_ERR_UNSUPPORTED;
}

template <int BN>
static int launch_pair(const uint8_t* a, const uint8_t* b, const GemmParams& p, cudaStream_t stream) {
    using C = PairCfg<BN>;
    CUtensorMap ma, mb, msa, msb;
    int st = make_operand_map(&ma, a, p.M, p.K / 2, 128);
    if (st == NVFP4_OK) st = make_operand_map(&mb, b, p.N, p.K / 2, BN / 2);
    if (st == NVFP4_OK) st = make_scale_map(&msa, p.sfa, p.sfa_groups, p.sf_group_stride);
    if (st == NVFP4_OK) st = make_scale_map(&msb, p.sfb, p.sfb_groups, p.sf_group_stride);
    if (st != NVFP4_OK) return st;
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = ((p.M + 255) / 256) * ((p.N + BN - 1) / BN);
    const int pairs = tiles < sms / 2 ? tiles : sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<BN>, ma, mb, msa, msb, p);
    return static_cast<int>(e);
}

}  // namespace pair

// =============================================================================================
// Skinny variant for decode-sized batches (M <= 128).  The roles of the operands are swapped: the 128 rows of
// the MMA are WEIGHT rows and its N dimension is the (padded) token count BT = 16 / 32 / 64 / 128, so the tensor
// cores spend BT/128 of the time a 128-row token tile of mostly padding would take and the kernel is a
// stream of the weights.  One CTA owns 128 weight rows and one K range; the K ranges of a tile are the CTAs
// of one thread-block cluster (1..8), which lets a shape with few weight tiles still pull from every SM.
// The partial accumulators are combined by a reduce-scatter through distributed shared memory: the token
// columns are dealt out to the ranks, every rank writes its partial tile to its own shared memory and sends
// each other rank the columns that rank owns with one bulk copy (cp.async.bulk shared::cta -> shared::cluster,
// completion counted on the receiver's mbarrier); the owner adds the partials in ascending rank order, applies
// alpha and stores bf16.  One kernel, no workspace, and the result does not depend on timing.  Every copy has
// one destination CTA (no multicast).
// =============================================================================================
namespace skinny {

using pair::cluster_ctarank;
using pair::cluster_sync_all;
using pair::map_to_cta;

constexpr int kMaxStages = 8;
// TMEM: accumulator in columns 0..BT-1, then two scale sets of 32 columns

template <int BT>
struct SkinnyCfg {
    static constexpr int kWBytes = 128 * kBKBytes;     // 128 weight rows x 256 codes
    static constexpr int kXBytes = BT * kBKBytes;      // BT token rows x 256 codes
    static constexpr int kSfBytes = 2048;              // one 128-row scale group x 16 blocks, for each operand
    static constexpr int kStageBytes = kWBytes + kXBytes + 2 * kSfBytes;
    static constexpr int kSfCol = BT <= 64 ? 64 : 128; // scale set 0: weights +0..15, tokens +16..31; set 1: +32
    static constexpr int kTmemCols = BT <= 64 ? 128 : 256;
    static constexpr int kMaxStages = (BT <= 64) ? 8 : 6;
    static_assert(kStageBytes % 1024 == 0, "stage alignment for the 128-byte swizzle");
    static_assert(BT % 16 == 0 && BT >= 16 && BT <= 128, "token tile");
};

__device__ __forceinline__ void tc_ld_32x32b_x16(uint32_t taddr, uint32_t v[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
// shared memory of this CTA -> shared memory of a CTA of the cluster; the bytes are counted on the receiver's barrier
__device__ __forceinline__ void bulk_copy_to_cta(uint32_t dst_cluster, uint32_t src_cta, uint32_t bytes, uint32_t bar_cluster) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_cluster),
                 "r"(src_cta), "r"(bytes), "r"(bar_cluster)
                 : "memory");
}

struct SkinnyParams {
    const uint8_t* sfx;   // token scales (group 0 of the tiled layout)
    const uint8_t* sfw;   // weight scales
    const float* alpha;
    __nv_bfloat16* out;   // [M, N]
    int M, N, K;
    int64_t sf_group_stride;
    int k_tiles_per_rank;
    int stages;
};

template <int BT>
__global__ void __launch_bounds__(kThreads)
skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const SkinnyParams p) {
    using C = SkinnyCfg<BT>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - raw_addr);
    const int nstages = p.stages;
    uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + nstages * C::kStageBytes);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
    const uint32_t tfull_bar = bar_base + 8u * (2 * kMaxStages);
    const uint32_t recv_bar = bar_base + 8u * (2 * kMaxStages + 1);   // partials from the other ranks have landed
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * kMaxStages + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    uint32_t ranks;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(ranks));
    const int nt = blockIdx.x / ranks;                  // 128-row weight tile (clusters run along x)
    // reduce-scatter: token column c belongs to rank c / cols_per_rank
    const uint32_t m_cols = static_cast<uint32_t>(min(p.M, BT));
    const uint32_t cols_per_rank = (m_cols + ranks - 1) / ranks;
    const uint32_t my_first = rank * cols_per_rank;
    const uint32_t my_cols = my_first < m_cols ? min(cols_per_rank, m_cols - my_first) : 0u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tfull_bar, 1);
        mbar_init(recv_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // (ranks - 1) senders x my columns x 128 rows x 4 bytes; armed before any rank can send (they send after
        // the cluster barrier below the main loop)
        if (ranks > 1 && my_cols > 0) mbar_expect_tx(recv_bar, (ranks - 1) * my_cols * 512u);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t*>(tmem_slot))),
                     "r"(C::kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int k_tiles = (p.K + kBK - 1) / kBK;
    const int kt_begin = static_cast<int>(rank) * p.k_tiles_per_rank;
    const int kcount = max(0, min(k_tiles, kt_begin + p.k_tiles_per_rank) - kt_begin);   // host: never 0

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        const bool issuer = elect_one();
        if (issuer) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
        }
        int stage = 0;
        uint32_t phase = 0;
        for (int i = 0; i < kcount; ++i) {
            const int kt = kt_begin + i;
            if (!mbar_wait_warp(empty_bar(stage), phase ^ 1u, abort_flag, (7u << 24) | kt)) break;
            const int kb_count = min(4, (p.K - kt * kBK + 63) / 64);
            const uint32_t sf_bytes = 512u * kb_count;
            const uint32_t sbase = base + stage * C::kStageBytes;
            if (issuer) {
                mbar_expect_tx(full_bar(stage), C::kWBytes + C::kXBytes + 2 * sf_bytes);
                tma_load_2d(sbase, &tmap_w, kt * kBKBytes, nt * 128, full_bar(stage));
                tma_load_2d(sbase + C::kWBytes, &tmap_x, kt * kBKBytes, 0, full_bar(stage));
                bulk_load_1d(sbase + C::kWBytes + C::kXBytes,
                             p.sfw + static_cast<int64_t>(nt) * p.sf_group_stride + static_cast<int64_t>(kt) * 2048, sf_bytes,
                             full_bar(stage));
                bulk_load_1d(sbase + C::kWBytes + C::kXBytes + C::kSfBytes, p.sfx + static_cast<int64_t>(kt) * 2048, sf_bytes,
                             full_bar(stage));
            }
            __syncwarp();
            if (++stage == nstages) {
                stage = 0;
                phase ^= 1u;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        const bool issuer = elect_one();
        constexpr uint32_t idesc = instr_desc<BT>();
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int i = 0; i < kcount; ++i) {
            if (!(ok = mbar_wait_warp(full_bar(stage), phase, abort_flag, (8u << 24) | i))) break;
            tc_fence_after();
            const int kb_count = min(4, (p.K - (kt_begin + i) * kBK + 63) / 64);
            const uint32_t sbase = base + stage * C::kStageBytes;
            const uint32_t w_lo = ((sbase & 0x3ffffu) >> 4) | (1u << 16);
            const uint32_t x_lo = w_lo + (C::kWBytes >> 4);
            const uint32_t sfw_lo = ((sbase + C::kWBytes + C::kXBytes) & 0x3ffffu) >> 4;
            const uint32_t sfx_lo = sfw_lo + (C::kSfBytes >> 4);
            const uint32_t sfw_t = tmem_base + C::kSfCol + (i & 1) * 32;
            const uint32_t sfx_t = sfw_t + 16;
            if (issuer) {
                for (int kb = 0; kb < kb_count; ++kb) {
                    tc_cp_lohi(sfw_t + 4 * kb, sfw_lo + 32 * kb);
                    tc_cp_lohi(sfx_t + 4 * kb, sfx_lo + 32 * kb);
                }
                for (int kb = 0; kb < kb_count; ++kb)
                    tc_mma_lohi(tmem_base, w_lo + 2 * kb, x_lo + 2 * kb, idesc, sfw_t + 4 * kb, sfx_t + 4 * kb,
                                (i > 0 || kb > 0) ? 1u : 0u);
                tc_commit(empty_bar(stage));
            }
            __syncwarp();
            if (++stage == nstages) {
                stage = 0;
                phase ^= 1u;
            }
        }
        if (ok && issuer) tc_commit(tfull_bar);
        __syncwarp();
    }

    // ---------------------------------------------------------------------- epilogue
    // Thread (sub-partition sp, lane) of warps 2..5 owns weight row nt*128 + 32*sp + lane; TMEM column m of its
    // lane is the partial sum for token m.  Columns are handled 16 at a time to keep the register count low.
    const int sp = warp & 3;
    const int n_local = sp * 32 + lane;
    const int n = nt * 128 + n_local;
    bool have = false;
    if (warp >= 2) {
        bool ok = mbar_wait(tfull_bar, 0, abort_flag, (9u << 24) | nt);
        have = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (have) tc_fence_after();
    }
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(sp * 32) << 16);
    if (ranks == 1) {
        if (warp >= 2 && have) {
            const float alpha = __ldg(p.alpha);
#pragma unroll 1
            for (int c = 0; c < BT / 16 && c * 16 < p.M; ++c) {
                uint32_t v[16];
                tc_ld_32x32b_x16(t_lane + c * 16, v);
                tc_ld_wait();
                if (n < p.N) {
#pragma unroll
                    for (int e = 0; e < 16; ++e)
                        if (c * 16 + e < p.M)
                            p.out[static_cast<int64_t>(c * 16 + e) * p.N + n] =
                                __float2bfloat16_rn(__fmul_rn(__uint_as_float(v[e]), alpha));
                }
            }
        }
    } else {
        // The ring is idle once the accumulator is complete (all copies landed and were consumed), so it is reused:
        // `part` [token column][128 rows] fp32 = this rank's partial tile, `recv` [sending rank][owned column][128 rows].
        float* part = reinterpret_cast<float*>(aligned);
        float* recv = part + BT * 128;
        if (warp >= 2 && have) {
#pragma unroll 1
            for (int c = 0; c < BT / 16 && c * 16 < p.M; ++c) {
                uint32_t v[16];
                tc_ld_32x32b_x16(t_lane + c * 16, v);
                tc_ld_wait();
#pragma unroll
                for (int e = 0; e < 16; ++e)
                    if (c * 16 + e < p.M) part[(c * 16 + e) * 128 + n_local] = __uint_as_float(v[e]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the bulk copies below read `part`
        }
        // every rank has left its main loop: the `recv` areas may be written
        cluster_sync_all();
        if (warp == 2 && have && elect_one()) {
            for (uint32_t o = 0; o < ranks; ++o) {
                const uint32_t first = o * cols_per_rank;
                if (o == rank || first >= m_cols) continue;
                const uint32_t cols = min(cols_per_rank, m_cols - first);
                bulk_copy_to_cta(map_to_cta(smem_u32(recv + (rank * cols_per_rank) * 128), o), smem_u32(part + first * 128),
                                 cols * 512u, map_to_cta(recv_bar, o));
            }
        }
        if (warp >= 2 && have && my_cols > 0) {
            bool ok = mbar_wait(recv_bar, 0, abort_flag, (10u << 24) | nt);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (ok && n < p.N) {
                const float alpha = __ldg(p.alpha);
                // this rank's own partial sits in `recv` terms at part[my_first ..]; eight columns at a time so that
                // the shared-memory loads of one rank's partials are in flight together
                const float* own = part + my_first * 128 + n_local;
                __nv_bfloat16* dst = p.out + static_cast<int64_t>(my_first) * p.N + n;
                for (uint32_t c0 = 0; c0 < my_cols; c0 += 8) {
                    float acc[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
                    for (uint32_t r = 0; r < ranks; ++r) {
                        const float* src = (r == rank) ? own : recv + (r * cols_per_rank) * 128 + n_local;
                        float v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[j] = (c0 + j < my_cols) ? src[(c0 + j) * 128] : 0.0f;
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[j] = r == 0 ? v[j] : __fadd_rn(acc[j], v[j]);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (c0 + j < my_cols)
                            dst[static_cast<int64_t>(c0 + j) * p.N] = __float2bfloat16_rn(__fmul_rn(acc[j], alpha));
                }
            }
        }
        // no rank may leave while another still copies out of its `part`
        cluster_sync_all();
    }

    // ---------------------------------------------------------------------- teardown
    if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::kTmemCols) : "memory");
    }
}

// K ranges per weight tile: the largest power of two that keeps every CTA of the grid resident at once (one per
// SM), with at least two K stages each and at most 8 (the portable cluster size).  With small token tiles two
// CTAs fit on an SM, and where the K range is already cut, cutting it once more measured faster (16 x 8192 x 8192:
// 12.2 -> 11.4 us); going from one range to two when the tiles already cover most SMs did not (16 x 14336 x 4096:
// 10.5 -> 11.1 us).  Cluster sizes that are not a power of two measured slower (6144 x 4096: 3 ranges 11.9 us,
// 2 ranges 8.0 us).
static int choose_ranks(int n_tiles, int k_tiles, int sms, int forced, int bt) {
    int r = 1;
    if (forced > 0) {
        r = forced;
    } else {
        while (r < 8 && n_tiles * (2 * r) <= sms) r *= 2;
        if (bt <= 32 && r >= 2 && r < 8 && n_tiles * (2 * r) <= 2 * sms - 40 && k_tiles / (2 * r) >= 4) r *= 2;
    }
    if (r > 8) r = 8;
    while (r > 1 && r > k_tiles / 2) --r;
    return r;
}

template <int BT>
static int launch_skinny(const uint8_t* x, const uint8_t* w, const GemmParams& g, int forced_ranks, cudaStream_t stream) {
    using C = SkinnyCfg<BT>;
    CUtensorMap mw, mx;
    int st = make_operand_map(&mw, w, g.N, g.K / 2, 128);
    if (st == NVFP4_OK) st = make_operand_map(&mx, x, g.M, g.K / 2, BT);
    if (st != NVFP4_OK) return st;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int n_tiles = (g.N + 127) / 128;
    const int k_tiles = (g.K + kBK - 1) / kBK;
    int ranks = choose_ranks(n_tiles, k_tiles, sms, forced_ranks, BT);
    SkinnyParams p;
    p.sfx = g.sfa;
    p.sfw = g.sfb;
    p.alpha = g.alpha;
    p.out = g.out;
    p.M = g.M;
    p.N = g.N;
    p.K = g.K;
    p.sf_group_stride = g.sf_group_stride;
    p.k_tiles_per_rank = (k_tiles + ranks - 1) / ranks;
    ranks = (k_tiles + p.k_tiles_per_rank - 1) / p.k_tiles_per_rank;   // no empty range
    // one CTA per SM with a deep ring when the whole grid is resident at once, else two CTAs per SM
    p.stages = (n_tiles * ranks <= sms) ? C::kMaxStages : 4;
    if (p.stages > p.k_tiles_per_rank) p.stages = p.k_tiles_per_rank < 2 ? 2 : p.k_tiles_per_rank;
    // the ring doubles as the reduce-scatter buffers: the partial tile plus one slot per rank of the owned columns
    while (ranks > 1 && (2 * BT + 8) * 512 > p.stages * C::kStageBytes) ++p.stages;
    if (p.stages > C::kMaxStages) return NVFP4_ERR_UNSUPPORTED;
    const int smem = p.stages * C::kStageBytes + 1024 + 256;
    cudaError_t e = cudaFuncSetAttribute(skinny_kernel<BT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kMaxStages * C::kStageBytes + 1024 + 256);
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles * ranks, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ranks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, skinny_kernel<BT>, mw, mx, p);
    return static_cast<int>(e);
}

}  // namespace skinny

}  // namespace gemm
}  // namespace nvfp4

static int g_gemm_force_path = 0;
constexpr int64_t kSkinnyMaxM = 128;   // what the skinny kernel accepts
constexpr int64_t kSkinnyAutoM = 32;   // what it is chosen for by default
static int g_gemm_force_splits = 0;    // 0 = by shape
static int g_gemm_force_rotate = -1;   // -1 = by shape
static int g_gemm_raster_group = 0;    // 0 = default

// K ranges for the single-CTA kernel.  Measured on B200 (M <= 128, K = 8192): cutting K never paid, the fixed
// cost of a second kernel and of the partial tiles outweighs the extra SMs, so the default is one range and the
// feature stays available through nvfp4_gemm_tune for shapes with very few tiles and very long K.
static int choose_k_splits(int64_t, int64_t, int64_t K) {
    if (g_gemm_force_splits <= 0) return 1;
    const int64_t k_tiles = (K + 255) / 256;
    return static_cast<int>(g_gemm_force_splits < k_tiles ? g_gemm_force_splits : k_tiles);
}

extern "C" size_t nvfp4_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const int splits = choose_k_splits(M, N, K);
    return splits > 1 ? static_cast<size_t>(splits) * static_cast<size_t>(M) * static_cast<size_t>(N) * sizeof(float) : 0;
}

// Testing hook: K ranges (0 = by shape) and K-loop rotation (-1 = by shape, 0 = off, 1 = on) of the single-CTA kernel.
// Testing hook: m-tiles per band of the tile numbering (0 = default).
extern "C" int nvfp4_gemm_tune_raster(int group) {
    if (group < 0 || group > 4096) return NVFP4_ERR_BAD_ENUM;
    g_gemm_raster_group = group;
    return NVFP4_OK;
}

extern "C" int nvfp4_gemm_tune(int k_splits, int k_rotate) {
    if (k_splits < 0 || k_splits > 16 || k_rotate < -1 || k_rotate > 1) return NVFP4_ERR_BAD_ENUM;
    g_gemm_force_splits = k_splits;
    g_gemm_force_rotate = k_rotate;
    return NVFP4_OK;
}

// Testing hook: 0 = choose the kernel by shape, 1 = 128x128 tiles, 2 = 128x256 tiles, 3 = CTA-pair 256x256 tiles,
// 4 = CTA-pair 256x192 tiles with two accumulators, 5 = skinny kernel (M <= 128; nvfp4_gemm_tune's k_splits then
// sets its K ranges per weight tile; larger M falls back to the choice by shape), 6 = 128x64 tiles.
extern "C" int nvfp4_gemm_force_path(int path) {
    if (path < 0 || path > 6) return NVFP4_ERR_BAD_ENUM;
    g_gemm_force_path = path;
    return NVFP4_OK;
}

extern "C" int nvfp4_gemm_launch(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                                 const float* alpha, void* out_bf16, int64_t M, int64_t N, int64_t K, void* workspace,
                                 size_t workspace_bytes, void* stream) {
    using namespace nvfp4;
    if (M < 0 || N < 0 || K < 0 || (K % 64) != 0) return NVFP4_ERR_BAD_SHAPE;
    if (M == 0 || N == 0) return NVFP4_OK;
    if (M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL) return NVFP4_ERR_TOO_LARGE;
    if (!a || !b || !sfa || !sfb || !alpha || !out_bf16) return NVFP4_ERR_NULL_POINTER;
    if (K == 0) return NVFP4_ERR_BAD_SHAPE;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) ||
        (reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15) ||
        (reinterpret_cast<uintptr_t>(out_bf16) & 15) || (reinterpret_cast<uintptr_t>(alpha) & 3))
        return NVFP4_ERR_MISALIGNED;
    gemm::GemmParams p;
    p.sfa = sfa;
    p.sfb = sfb;
    p.alpha = alpha;
    p.out = static_cast<__nv_bfloat16*>(out_bf16);
    p.M = static_cast<int>(M);
    p.N = static_cast<int>(N);
    p.K = static_cast<int>(K);
    p.sf_group_stride = round_up_i64(K / 16, 4) * 128;
    p.sfa_groups = static_cast<int>((M + 127) / 128);
    p.sfb_groups = static_cast<int>((N + 127) / 128);
    p.k_splits = choose_k_splits(M, N, K);
    const int k_tiles_total = static_cast<int>((K + 255) / 256);
    p.k_tiles_per_split = (k_tiles_total + p.k_splits - 1) / p.k_splits;
    p.k_splits = (k_tiles_total + p.k_tiles_per_split - 1) / p.k_tiles_per_split;   // no empty range
    p.k_rotate = g_gemm_force_rotate > 0 ? 1 : 0;
    p.partial = static_cast<float*>(workspace);
    // default: one band over all m-tiles (band sizes 1..16 measured within noise of it on B200)
    p.raster_group = g_gemm_raster_group > 0 ? g_gemm_raster_group : (1 << 20);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Decode-sized batches: weight rows on the MMA's 128 rows, tokens on its N dimension, K ranges across a cluster.
    // Measured on B200 with the weights streaming from HBM: faster than every other kernel up to 32 tokens; from 33
    // to 128 tokens only where few weight tiles meet a long K (at least 4 K ranges of at least 12 stages each, e.g.
    // 64 x 4096 x 14336: 13.2 us against 19.4 us), because its epilogue grows with the token tile.
    bool skinny = false;
    if (g_gemm_force_path == 5) {
        skinny = M <= kSkinnyMaxM;
    } else if (g_gemm_force_path == 0 && g_gemm_force_splits == 0 && M <= kSkinnyMaxM) {
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const int ranks = gemm::skinny::choose_ranks(static_cast<int>((N + 127) / 128), k_tiles_total, sms, 0, M <= 64 ? 64 : 128);
        skinny = M <= kSkinnyAutoM || (ranks >= 4 && k_tiles_total / ranks >= 12);
    }
    if (skinny) {
        const int forced = g_gemm_force_path == 5 ? g_gemm_force_splits : 0;
        if (M <= 16) return gemm::skinny::launch_skinny<16>(a, b, p, forced, s);
        if (M <= 32) return gemm::skinny::launch_skinny<32>(a, b, p, forced, s);
        if (M <= 64) return gemm::skinny::launch_skinny<64>(a, b, p, forced, s);
        return gemm::skinny::launch_skinny<128>(a, b, p, forced, s);
    }
    if (p.k_splits > 1) {
        const size_t need = static_cast<size_t>(p.k_splits) * static_cast<size_t>(M) * static_cast<size_t>(N) * sizeof(float);
        if (!workspace || workspace_bytes < need) return NVFP4_ERR_WORKSPACE;
        if (reinterpret_cast<uintptr_t>(workspace) & 15) return NVFP4_ERR_MISALIGNED;
    }
    // Kernel choice by a small cost model fitted to measurements on B200: time ~ waves x cost of one tile, where a
    // wave is 148 single-CTA tiles or 74 CTA-pair tiles.  Relative tile costs: 128x64 -> 0.45, 128x128 -> 0.7, 128x256 -> 1.0,
    // pair 256x192 -> 0.68 (0.75 of the MMA work per SM, and its epilogue overlaps the next tile).
    int path = g_gemm_force_path == 5 ? 0 : g_gemm_force_path;   // 0 = choose by shape
    if (path == 0) {
        const int64_t mt = (M + 127) / 128;
        const double c1 = static_cast<double>((mt * ((N + 127) / 128) + 147) / 148) * 0.7;
        const double c2 = static_cast<double>((mt * ((N + 255) / 256) + 147) / 148) * 1.0;
        const double c4 = static_cast<double>((((M + 255) / 256) * ((N + 191) / 192) + 73) / 74) * 0.68;
        path = (c1 <= c2) ? 1 : 2;
        double best = c1 <= c2 ? c1 : c2;
        if (M > 128 && N > 128 && p.k_splits == 1 && c4 <= best) {
            path = 4;
            best = c4;
        }
        // few, long tiles (one or two token tiles): 64 weight rows per CTA put twice as many SMs on the weight stream
        const double c6 = static_cast<double>((mt * ((N + 63) / 64) + 147) / 148) * 0.45;
        if (mt <= 2 && c6 < best) path = 6;
    }
    if (p.k_splits > 1 && path != 1 && path != 2 && path != 6) path = 1;
    if (path == 3) return gemm::pair::launch_pair<256>(a, b, p, s);
    if (path == 4) return gemm::pair::launch_pair<192>(a, b, p, s);
    if (path == 2) return gemm::launch<256>(a, b, p, s);
    if (path == 6) return gemm::launch<64>(a, b, p, s);
    return gemm::launch<128>(a, b, p, s);
}

extern "C" int nvfp4_gemm_last_status(void* stream, uint32_t* status_host) {
    if (!status_host) return NVFP4_ERR_NULL_POINTER;
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return static_cast<int>(e);
    uint32_t zero = 0;
    e = cudaMemcpyFromSymbol(status_host, nvfp4::gemm::g_gemm_status, sizeof(uint32_t));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (*status_host != 0) e = cudaMemcpyToSymbol(nvfp4::gemm::g_gemm_status, &zero, sizeof(uint32_t));
    return static_cast<int>(e);
}
