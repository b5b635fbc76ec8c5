// CTA-pair kernels of the NVFP4 GEMM (cta_group::2, 256 x 192 / 256 x 256 output tiles).
#pragma once

#include "gemm_tile.cuh"

namespace nvfp4 {
namespace gemm {

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
// BN = 192 / 128: two accumulators (2 x BN columns), so the epilogue of one tile overlaps the MMAs of the next.
// BN = 128 (256 x 128 tiles) is for a few hundred tokens: twice the CTAs of the wider tiles on the weight stream,
// and each CTA still loads only half of the tile's weight rows.
template <int BN>
struct PairCfg {
    static constexpr int kAcc = (BN <= 192) ? 2 : 1;
    static constexpr int kABytes = 128 * kBKBytes;          // this CTA's 128 rows of A
    static constexpr int kBBytes = (BN / 2) * kBKBytes;     // this CTA's half of the B rows
    static constexpr int kSfaBytes = 2048;                  // scales of this CTA's A rows
    static constexpr int kSfbBytes = 4096;                  // two 128-row scale groups cover the B tile
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    static constexpr int kStages = (BN == 128) ? 7 : (BN == 192) ? 6 : 5;
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
    // The kernel queued behind this one may be scheduled at once: ahead of its own wait it reads nothing but a
    // prepared (constant) weight, and that wait covers this kernel's completion.
    griddep_launch();
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
    if (threadIdx.x == 0) trace_mark(1, 0);

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
        if (lane == 0) trace_mark(1, 1);
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) trace_mark(1, 9);
    cluster_sync_all();   // the peer's barriers exist before anything is signalled across CTAs
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) trace_mark(1, 2);
    if (warp >= 2) griddep_wait();    // the epilogue reads alpha and writes the output: only after the previous kernel

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
            // weight half (B rows and their scales: independent of whatever ran before this kernel) and token half (A rows
            // and their scales) of a stage; the weight halves of the first ring-full are issued before griddep_wait()
            auto issue = [&](int st, int mt, int nt, int kt, bool weights, bool tokens) {
                const uint32_t lead_full = map_to_cta(full_bar(st), 0);
                const uint32_t sbase = base + st * C::kStageBytes;
                if (weights) {
                    if (rank == 0) mbar_expect_tx(full_bar(st), 2u * C::kStageBytes);
                    tma_load_2d_pair(sbase + C::kABytes, &tmap_b, kt * kBKBytes, nt * BN + static_cast<int>(rank) * (BN / 2), lead_full);
                    // scale tiles: x counts 8-byte elements (2048 B per K tile), y = 128-row group
                    tma_load_2d_pair(sbase + C::kABytes + C::kBBytes + C::kSfaBytes, &tmap_sfb, kt * 256, (nt * BN) / 128, lead_full);
                    tma_load_2d_pair(sbase + C::kABytes + C::kBBytes + C::kSfaBytes + 2048, &tmap_sfb, kt * 256, (nt * BN) / 128 + 1, lead_full);
                }
                if (tokens) {
                    tma_load_2d_pair(sbase, &tmap_a, kt * kBKBytes, mt * 256 + static_cast<int>(rank) * 128, lead_full);
                    tma_load_2d_pair(sbase + C::kABytes + C::kBBytes, &tmap_sfa, kt * 256, mt * 2 + static_cast<int>(rank), lead_full);
                }
            };
            int early = 0;
            if (!p.weights_ready) griddep_wait();
            if (pair_id < total_tiles) {
                int mt, nt;
                tile_to_mn(pair_id, m_tiles, n_tiles, p.raster_group, mt, nt);
                early = min(k_tiles, C::kStages);
                if (issuer)
                    for (int i = 0; i < early; ++i) issue(i, mt, nt, i, true, false);
                __syncwarp();
            }
            griddep_wait();
            for (int tile = pair_id; ok && tile < total_tiles; tile += num_pairs) {
                int mt, nt;
                tile_to_mn(tile, m_tiles, n_tiles, p.raster_group, mt, nt);
                for (int kt = 0; kt < k_tiles; ++kt) {
                    if (!(ok = mbar_wait_warp(empty_bar(stage), phase ^ 1u, abort_flag, (1u << 24) | kt))) break;
                    if (issuer) issue(stage, mt, nt, kt, early == 0, true);
                    if (early > 0) --early;
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
        const float alpha = load_alpha(p.alpha, p.alpha2);
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

    if (lane == 0) trace_mark(1, warp == 0 ? 3 : warp == 1 ? 4 : 5);
    // ---------------------------------------------------------------------- teardown
    if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) trace_mark(1, 6);
    cluster_sync_all();   // neither CTA leaves while its partner may still signal or read it
    if (threadIdx.x == 0) trace_mark(1, 7);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
        if (lane == 0) trace_mark(1, 8);
    }
    // cta_group::2 allocation state spans both SMs of the pair.  If one CTA left right after its own dealloc, another
    // kernel's CTA could start on that SM and allocate while the partner's dealloc for the pair is still to come;
    // with several GEMM kernels running at once that left a later tcgen05.alloc waiting for ever.  Both CTAs
    // therefore stay until both deallocations have been issued.
    cluster_sync_all();
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
static int launch_pair(const uint8_t* a, const uint8_t* b, const GemmParams& p, cudaStream_t stream, const WeightHandle* wh) {
    using C = PairCfg<BN>;
    CUtensorMap ma, msa, mb_local, msb_local;
    int st = make_operand_map(&ma, a, p.M, p.K / 2, 128);
    if (st == NVFP4_OK) st = make_scale_map(&msa, p.sfa, p.sfa_groups, p.sf_group_stride);
    if (st == NVFP4_OK && !wh) st = make_operand_map(&mb_local, b, p.N, p.K / 2, BN / 2);
    if (st == NVFP4_OK && !wh) st = make_scale_map(&msb_local, p.sfb, p.sfb_groups, p.sf_group_stride);
    if (st != NVFP4_OK) return st;
    const CUtensorMap& mb = wh ? *wh->by_rows(BN / 2) : mb_local;
    const CUtensorMap& msb = wh ? wh->scales : msb_local;
    static_assert(C::kSmemBytes <= kGemmDynSmemBytes, "ring does not fit");
    const DeviceInfo di = device_info();
    static bool attr_done[64] = {false};
    cudaError_t e = allow_full_smem(gemm_pair_kernel<BN>, attr_done, di.device);
    if (e != cudaSuccess) return static_cast<int>(e);
    const int sms = di.sms;
    const int tiles = ((p.M + 255) / 256) * ((p.N + BN - 1) / BN);
    const int pairs = tiles < sms / 2 ? tiles : sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kGemmDynSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // may start while its predecessor finishes
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_dependent_launch ? 2 : 1;
    e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<BN>, ma, mb, msa, msb, p);
    return static_cast<int>(e);
}

}  // namespace pair

}  // namespace gemm
}  // namespace nvfp4
