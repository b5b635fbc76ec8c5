// Decode-sized kernel of the NVFP4 GEMM: weights on the MMA rows, K ranges across a thread-block cluster.
#pragma once

#include "gemm_pair.cuh"

namespace nvfp4 {
namespace gemm {

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

// One launch may multiply the same token tile with several weight matrices of equal K (a layer's q / k / v, or gate /
// up projections): the weight tiles of all of them are numbered through, and a CTA looks up whose tile it owns.  The
// launch's fixed costs (prologue, ramp-up and drain of the weight stream) are then paid once per group.
constexpr int kMaxGroup = 8;

struct SkinnyWeight {
    const uint8_t* sfw;   // weight scales
    const float* alpha;   // output scale of this weight (times alpha_x when that is given)
    __nv_bfloat16* out;   // [M, N]
    int N;
    int tile_end;         // number of 128-row tiles of this and all earlier weights of the group
};

struct SkinnyParams {
    const uint8_t* sfx;   // token scales (group 0 of the tiled layout)
    const float* alpha_x; // optional common factor of every output scale
    int M, K;
    int64_t sf_group_stride;
    int k_tiles_per_rank;
    int stages;
    int n_weights;
    int weights_ready;    // != 0: all weights are prepared weights (constant while in use): read them before griddep_wait()
    SkinnyWeight w[kMaxGroup];
};

struct SkinnyMaps {
    CUtensorMap m[kMaxGroup];   // one per weight: [N, K/2] bytes in boxes of 128 rows x 128 bytes
};

template <int BT>
__global__ void __launch_bounds__(kThreads)
skinny_kernel(const __grid_constant__ SkinnyMaps maps, const __grid_constant__ CUtensorMap tmap_x, const SkinnyParams p) {
    using C = SkinnyCfg<BT>;
    extern __shared__ uint8_t smem_raw[];
    // The kernel queued behind this one may be scheduled at once: ahead of its own wait it reads nothing but a
    // prepared (constant) weight, and that wait covers this kernel's completion.
    griddep_launch();
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
    // clusters run along x: cluster index = 128-row weight tile, numbered through the weights of the group
    const int tile = blockIdx.x / ranks;
    int gi = 0;
    while (gi + 1 < p.n_weights && tile >= p.w[gi].tile_end) ++gi;
    const int nt = tile - (gi > 0 ? p.w[gi - 1].tile_end : 0);
    const CUtensorMap* tmap_w = &maps.m[gi];
    const uint8_t* const sfw = p.w[gi].sfw;
    const int N = p.w[gi].N;
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
    const int k_tiles = (p.K + kBK - 1) / kBK;
    const int kt_begin = static_cast<int>(rank) * p.k_tiles_per_rank;
    const int kcount = max(0, min(k_tiles, kt_begin + p.k_tiles_per_rank) - kt_begin);   // host: never 0

    // Producer state (warp 0).  The first ring-full of copies is issued BEFORE the CTA-wide barrier of the prologue:
    // the copies need the mbarriers (initialised by this warp's thread 0 just above) but neither TMEM nor the other
    // warps, so the first HBM round trip overlaps the TMEM allocation and the barrier instead of following them.
    int p_stage = 0, p_next = 0;
    uint32_t p_phase = 0;
    bool p_ok = true;
    auto produce = [&](int end) {
        const bool issuer = elect_one();
        for (; p_ok && p_next < end; ++p_next) {
            const int kt = kt_begin + p_next;
            const int stage = p_stage;
            const uint32_t phase = p_phase;
            if (!(p_ok = mbar_wait_warp(empty_bar(stage), phase ^ 1u, abort_flag, (7u << 24) | kt))) break;
            const int kb_count = min(4, (p.K - kt * kBK + 63) / 64);
            const uint32_t sf_bytes = 512u * kb_count;
            const uint32_t sbase = base + stage * C::kStageBytes;
            if (issuer) {
                mbar_expect_tx(full_bar(stage), C::kWBytes + C::kXBytes + 2 * sf_bytes);
                tma_load_2d(sbase, tmap_w, kt * kBKBytes, nt * 128, full_bar(stage));
                tma_load_2d(sbase + C::kWBytes, &tmap_x, kt * kBKBytes, 0, full_bar(stage));
                bulk_load_1d(sbase + C::kWBytes + C::kXBytes,
                             sfw + static_cast<int64_t>(nt) * p.sf_group_stride + static_cast<int64_t>(kt) * 2048, sf_bytes,
                             full_bar(stage));
                bulk_load_1d(sbase + C::kWBytes + C::kXBytes + C::kSfBytes, p.sfx + static_cast<int64_t>(kt) * 2048, sf_bytes,
                             full_bar(stage));
            }
            __syncwarp();
            if (++p_stage == nstages) {
                p_stage = 0;
                p_phase ^= 1u;
            }
        }
    };
    if (warp == 0) {
        __syncwarp();   // thread 0's barrier initialisation above, before any lane of this warp uses the barriers
        if (elect_one()) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(tmap_w) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
        }
        // First ring-full.  The weights do not depend on whatever ran before this kernel on the stream, the token tile
        // and its scales (the quantizer's output) do: with a programmatic dependent launch the weight copies go out
        // at once, the rest after griddep_wait().
        const int first = min(kcount, nstages);
        const bool issuer = elect_one();
        if (!p.weights_ready) griddep_wait();   // raw weight pointers: they may be the previous kernel's output too
        if (issuer) {
            for (int i = 0; i < first; ++i) {
                const int kt = kt_begin + i;
                const uint32_t sf_bytes = 512u * min(4, (p.K - kt * kBK + 63) / 64);
                const uint32_t sbase = base + i * C::kStageBytes;
                mbar_expect_tx(full_bar(i), C::kWBytes + C::kXBytes + 2 * sf_bytes);
                tma_load_2d(sbase, tmap_w, kt * kBKBytes, nt * 128, full_bar(i));
                bulk_load_1d(sbase + C::kWBytes + C::kXBytes,
                             sfw + static_cast<int64_t>(nt) * p.sf_group_stride + static_cast<int64_t>(kt) * 2048, sf_bytes,
                             full_bar(i));
            }
        }
        griddep_wait();
        if (issuer) {
            for (int i = 0; i < first; ++i) {
                const int kt = kt_begin + i;
                const uint32_t sf_bytes = 512u * min(4, (p.K - kt * kBK + 63) / 64);
                const uint32_t sbase = base + i * C::kStageBytes;
                tma_load_2d(sbase + C::kWBytes, &tmap_x, kt * kBKBytes, 0, full_bar(i));
                bulk_load_1d(sbase + C::kWBytes + C::kXBytes + C::kSfBytes, p.sfx + static_cast<int64_t>(kt) * 2048, sf_bytes,
                             full_bar(i));
            }
        }
        __syncwarp();
        p_next = first;
        p_stage = first == nstages ? 0 : first;
        p_phase = first == nstages ? 1u : 0u;
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
    if (warp >= 2) griddep_wait();   // the epilogue reads alpha (and writes out): only once the previous kernel is done

    if (warp == 0) {
        // ------------------------------------------------------------------ producer, stages after the first ring-full
        produce(kcount);
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
            const float alpha = load_alpha(p.w[gi].alpha, p.alpha_x);
            __nv_bfloat16* const out = p.w[gi].out;
#pragma unroll 1
            for (int c = 0; c < BT / 16 && c * 16 < p.M; ++c) {
                uint32_t v[16];
                tc_ld_32x32b_x16(t_lane + c * 16, v);
                tc_ld_wait();
                if (n < N) {
#pragma unroll
                    for (int e = 0; e < 16; ++e)
                        if (c * 16 + e < p.M)
                            out[static_cast<int64_t>(c * 16 + e) * N + n] =
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
            if (ok && n < N) {
                const float alpha = load_alpha(p.w[gi].alpha, p.alpha_x);
                // this rank's own partial sits in `recv` terms at part[my_first ..]; eight columns at a time so that
                // the shared-memory loads of one rank's partials are in flight together
                const float* own = part + my_first * 128 + n_local;
                __nv_bfloat16* dst = p.w[gi].out + static_cast<int64_t>(my_first) * N + n;
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
                            dst[static_cast<int64_t>(c0 + j) * N] = __float2bfloat16_rn(__fmul_rn(acc[j], alpha));
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

// One weight of a grouped launch, as the host sees it.
struct SkinnyItem {
    const uint8_t* w;         // codes [N, K/2]
    const uint8_t* sfw;       // tiled scales
    const float* alpha;
    __nv_bfloat16* out;       // [M, N]
    int64_t N;
    const WeightHandle* wh;   // prepared tensor maps, or NULL
};

// Ring depth: the deepest ring with which the whole grid is resident at once (as many CTAs per SM as that takes, at
// most what the TMEM columns allow), since a CTA that has to wait for a free SM starts its weight stream late.
template <int BT>
static int choose_stages(int ctas, int sms) {
    using C = SkinnyCfg<BT>;
    constexpr int kMaxPerSm = kTmemCols / C::kTmemCols;
    int per_sm = (ctas + sms - 1) / sms;
    if (per_sm < 1) per_sm = 1;
    if (per_sm > kMaxPerSm) per_sm = kMaxPerSm;
    // an SM has 233472 bytes of shared memory, of which 1 KiB per resident CTA is reserved; a CTA asks for its ring
    // plus 1 KiB of alignment slack plus 256 bytes of barriers
    int stages = (233472 / per_sm - 1024 - 1024 - 256) / C::kStageBytes;
    if (stages > C::kMaxStages) stages = C::kMaxStages;
    // with CTAs sharing an SM a fifth stage, which would still fit, measured slower than four (Llama-3-8B-shaped decode
    // chain of 32 layers at 1 / 16 tokens: 1.30 / 1.48 ms against 1.25 / 1.43; 16 x 28672 x 8192: 23.3 against 23.0 us)
    if (per_sm >= 2 && stages > 4) stages = 4;
    if (stages < 2) stages = 2;
    return stages;
}

template <int BT>
static int launch_skinny_group(const uint8_t* x, const uint8_t* sfx, const float* alpha_x, int M, int K,
                               int64_t sf_group_stride, const SkinnyItem* items, int n_items, int forced_ranks,
                               cudaStream_t stream) {
    using C = SkinnyCfg<BT>;
    if (n_items < 1 || n_items > kMaxGroup) return NVFP4_ERR_BAD_RANGE;
    SkinnyMaps maps;
    CUtensorMap mx;
    int st = make_operand_map(&mx, x, M, K / 2, BT);
    SkinnyParams p;
    int n_tiles = 0;
    p.weights_ready = 1;
    for (int i = 0; i < n_items && st == NVFP4_OK; ++i) {
        const SkinnyItem& it = items[i];
        if (!it.wh) p.weights_ready = 0;
        if (it.wh) maps.m[i] = it.wh->rows128;
        else st = make_operand_map(&maps.m[i], it.w, it.N, K / 2, 128);
        n_tiles += static_cast<int>((it.N + 127) / 128);
        p.w[i].sfw = it.sfw;
        p.w[i].alpha = it.alpha;
        p.w[i].out = it.out;
        p.w[i].N = static_cast<int>(it.N);
        p.w[i].tile_end = n_tiles;
    }
    if (st != NVFP4_OK) return st;
    for (int i = n_items; i < kMaxGroup; ++i) {   // unused slots: defined values, never dereferenced
        maps.m[i] = maps.m[0];
        p.w[i] = p.w[n_items - 1];
    }
    const DeviceInfo di = device_info();
    const int sms = di.sms;
    const int k_tiles = (K + kBK - 1) / kBK;
    int ranks = choose_ranks(n_tiles, k_tiles, sms, forced_ranks, BT);
    p.sfx = sfx;
    p.alpha_x = alpha_x;
    p.M = M;
    p.K = K;
    p.sf_group_stride = sf_group_stride;
    p.n_weights = n_items;
    p.k_tiles_per_rank = (k_tiles + ranks - 1) / ranks;
    ranks = (k_tiles + p.k_tiles_per_rank - 1) / p.k_tiles_per_rank;   // no empty range
    p.stages = choose_stages<BT>(n_tiles * ranks, sms);
    if (p.stages > p.k_tiles_per_rank) p.stages = p.k_tiles_per_rank < 2 ? 2 : p.k_tiles_per_rank;
    // the ring doubles as the reduce-scatter buffers: the partial tile plus one slot per rank of the owned columns
    while (ranks > 1 && (2 * BT + 8) * 512 > p.stages * C::kStageBytes) ++p.stages;
    if (p.stages > C::kMaxStages) return NVFP4_ERR_UNSUPPORTED;
    // Co-resident CTAs must never want more than the 512 TMEM columns of an SM between them (a CTA that waits in
    // tcgen05.alloc while its cluster peers wait for it is a deadlock).  Shared memory is what bounds co-residency, so
    // every CTA asks for at least the share of the SM's shared memory that matches its share of the TMEM columns
    // (1 KiB per CTA is reserved by the system): whatever mix of these kernels fits an SM then fits its TMEM too.
    constexpr int kMinSmem = 233472 / (kTmemCols / C::kTmemCols) - 1024;   // 128 columns: 57344 (4 CTAs), 256: 115712 (2)
    int smem = p.stages * C::kStageBytes + 1024 + 256;
    if (smem < kMinSmem) smem = kMinSmem;
    static_assert(C::kMaxStages * C::kStageBytes + 1024 + 256 <= kGemmDynSmemBytes, "ring does not fit");
    static bool attr_done[64] = {false};
    cudaError_t e = allow_full_smem(skinny_kernel<BT>, attr_done, di.device);
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles * ranks, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ranks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // programmatic dependent launch: this kernel may be scheduled while its predecessor on the stream is finishing
    // (it stops at griddep_wait() before touching anything the predecessor may have written)
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_dependent_launch ? 2 : 1;
    e = cudaLaunchKernelEx(&cfg, skinny_kernel<BT>, maps, mx, p);
    return static_cast<int>(e);
}

template <int BT>
static int launch_skinny(const uint8_t* x, const uint8_t* w, const GemmParams& g, int forced_ranks, cudaStream_t stream,
                         const WeightHandle* wh) {
    SkinnyItem it;
    it.w = w;
    it.sfw = g.sfb;
    it.alpha = g.alpha;
    it.out = g.out;
    it.N = g.N;
    it.wh = wh;
    return launch_skinny_group<BT>(x, g.sfa, g.alpha2, g.M, g.K, g.sf_group_stride, &it, 1, forced_ranks, stream);
}

}  // namespace skinny

}  // namespace gemm
}  // namespace nvfp4
