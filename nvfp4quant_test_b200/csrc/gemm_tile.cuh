// Tile kernels of the NVFP4 GEMM: one persistent CTA per SM, 128 x 64 / 128 x 128 / 128 x 256 output tiles.
#pragma once

#include "tc_ptx.cuh"

namespace nvfp4 {
namespace gemm {

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

struct GemmParams {
    const uint8_t* sfa;
    const uint8_t* sfb;
    const float* alpha;
    const float* alpha2;      // optional second factor: the output scale is alpha[0] * alpha2[0] (one fp32 multiplication)
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
    // != 0: the weight operand is a prepared weight, constant while launches with it are in flight, and may be read
    // before griddep_wait(); 0 (raw pointers): it may be the output of the kernel just before this one, like the tokens
    int weights_ready;
};

// Output scale of a launch: alpha[0], or alpha[0] * alpha2[0] rounded once (what a separate fp32 multiplication of the
// activation's and the weight's global scales gives).
__device__ __forceinline__ float load_alpha(const float* alpha, const float* alpha2) {
    // called behind griddep_wait(): the scales may be the work of the kernels before this one
    const float a = load_f32_after_wait(alpha);
    return alpha2 ? __fmul_rn(a, load_f32_after_wait(alpha2)) : a;
}

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
    // The kernel queued behind this one may be scheduled at once: ahead of its own wait it reads nothing but a
    // prepared (constant) weight, and that wait covers this kernel's completion.
    griddep_launch();
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
    if (threadIdx.x == 0) trace_mark(0, 0);

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
        if (lane == 0) trace_mark(0, 1);
    }
    // The producer warp initialised the mbarriers itself (thread 0) and needs neither TMEM nor the other warps, so it
    // only ARRIVES on the prologue barrier and starts its copies at once; the first HBM round trip then overlaps the
    // TMEM allocation.  Warps 1..5 wait for the arrival (barrier initialisation, TMEM address).
    tc_fence_before();
    if (warp == 0) {
        __syncwarp();
        asm volatile("bar.arrive 1, %0;" ::"n"(kThreads) : "memory");
    } else {
        asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
    }
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;   // meaningful in warps 1..5 only
    if (threadIdx.x == 32) trace_mark(0, 2);
    if (warp >= 2) griddep_wait();    // alpha, and the output buffer, belong to whatever ran before: epilogue only after it

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
            // Stage copies come in two halves: the weight half (B tile and its scales) depends on nothing that ran
            // before this kernel, the token half (A tile and its scales) may be the previous kernel's output.  The
            // weight halves of the first ring-full go out before griddep_wait(), so that with a programmatic dependent
            // launch the weight stream starts while the previous kernel is still finishing; `early` counts them.
            auto issue = [&](int st, int mt, int nt, int kt, bool weights, bool tokens) {
                const int kb_count = min(4, (p.K - kt * kBK + 63) / 64);  // 64-element K blocks in this stage
                const uint32_t sf_bytes = 512u * kb_count;
                int sfb_present = 0;
                const int grp0 = BN == 64 ? (nt >> 1) : nt * C::kNG;   // first 128-row scale group of this B tile
                for (int g = 0; g < C::kNG; ++g) sfb_present += (grp0 + g < p.sfb_groups) ? 1 : 0;
                const uint32_t sbase = base + st * C::kStageBytes;
                if (weights) {
                    mbar_expect_tx(full_bar(st), C::kABytes + C::kBBytes + sf_bytes * (1 + sfb_present));
                    tma_load_2d(sbase + C::kABytes, &tmap_b, kt * kBKBytes, nt * BN, full_bar(st));
                    for (int g = 0; g < C::kNG; ++g) {
                        const int grp = grp0 + g;
                        if (grp < p.sfb_groups)
                            bulk_load_1d(sbase + C::kABytes + C::kBBytes + C::kSfaBytes + g * 2048,
                                         p.sfb + static_cast<int64_t>(grp) * p.sf_group_stride +
                                             static_cast<int64_t>(kt) * 2048,
                                         sf_bytes, full_bar(st));
                    }
                }
                if (tokens) {
                    tma_load_2d(sbase, &tmap_a, kt * kBKBytes, mt * kBM, full_bar(st));
                    bulk_load_1d(sbase + C::kABytes + C::kBBytes,
                                 p.sfa + static_cast<int64_t>(mt) * p.sf_group_stride + static_cast<int64_t>(kt) * 2048,
                                 sf_bytes, full_bar(st));
                }
            };
            int early = 0;
            if (!p.weights_ready) griddep_wait();
            if (static_cast<int>(blockIdx.x) < total_tiles && !p.k_rotate) {
                const int ks = blockIdx.x / mn_tiles, t2 = blockIdx.x - ks * mn_tiles;
                int mt, nt;
                tile_to_mn(t2, m_tiles, n_tiles, p.raster_group, mt, nt);
                const int kt_begin = ks * p.k_tiles_per_split;
                const int kcount = min(k_tiles, kt_begin + p.k_tiles_per_split) - kt_begin;
                early = min(kcount, C::kStages);
                if (issuer)
                    for (int i = 0; i < early; ++i) issue(i, mt, nt, kt_begin + i, true, false);
                __syncwarp();
            }
            griddep_wait();
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
        const float alpha = load_alpha(p.alpha, p.alpha2);
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

    if (lane == 0) trace_mark(0, warp == 0 ? 3 : warp == 1 ? 4 : 5);
    // ---------------------------------------------------------------------- teardown
    if (*abort_flag) {
        // give any bulk copy still in flight time to land before shared memory is released
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) trace_mark(0, 6);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
        if (lane == 0) trace_mark(0, 8);
    }
}

// out[m, n] = bf16(alpha * sum over K ranges of partial[s][m][n]); ranges are added in ascending order.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, const float* alpha_ptr,
                                                            const float* alpha2_ptr, __nv_bfloat16* __restrict__ out,
                                                            int64_t mn, int splits) {
    const float alpha = load_alpha(alpha_ptr, alpha2_ptr);
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

// Per-device facts the launchers need on every call, looked up once per device.

struct DeviceInfo {
    int device;
    int sms;
};
static DeviceInfo device_info() {
    static int sm_count[64] = {0};
    DeviceInfo d{0, 148};
    if (cudaGetDevice(&d.device) != cudaSuccess || d.device < 0 || d.device >= 64) return d;
    if (sm_count[d.device] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, d.device) == cudaSuccess && v > 0) sm_count[d.device] = v;
    }
    if (sm_count[d.device] > 0) d.sms = sm_count[d.device];
    return d;
}
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is per device and sticky: once per (kernel, device) is enough.
template <class Kernel>
static cudaError_t allow_full_smem(Kernel kernel, bool* done_per_device, int device) {
    if (device >= 0 && device < 64 && done_per_device[device]) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmDynSmemBytes);
    if (e == cudaSuccess && device >= 0 && device < 64) done_per_device[device] = true;
    return e;
}

// A weight matrix prepared once for many GEMM calls: its tensor maps for every tile height the kernels use.
struct WeightHandle {
    uint32_t magic;
    int device;
    const uint8_t* b;
    const uint8_t* sfb;
    int64_t N, K;
    CUtensorMap rows64, rows96, rows128, rows256;   // operand maps by box height
    CUtensorMap scales;                             // scale groups as rows of 8-byte words (pair kernels)
    const CUtensorMap* by_rows(int rows) const {
        return rows == 64 ? &rows64 : rows == 96 ? &rows96 : rows == 128 ? &rows128 : &rows256;
    }
};
constexpr uint32_t kWeightMagic = 0x4e56463u;

template <int BN>
static int launch(const uint8_t* a, const uint8_t* b, const GemmParams& p, cudaStream_t stream, const WeightHandle* wh) {
    using C = Cfg<BN>;
    CUtensorMap ma, mb_local;
    int st = make_operand_map(&ma, a, p.M, p.K / 2, kBM);
    if (st != NVFP4_OK) return st;
    if (!wh) {
        st = make_operand_map(&mb_local, b, p.N, p.K / 2, BN);
        if (st != NVFP4_OK) return st;
    }
    const CUtensorMap& mb = wh ? *wh->by_rows(BN) : mb_local;
    static_assert(C::kSmemBytes <= kGemmDynSmemBytes, "ring does not fit");
    const DeviceInfo di = device_info();
    static bool attr_done[64] = {false};
    cudaError_t e = allow_full_smem(gemm_kernel<BN>, attr_done, di.device);
    if (e != cudaSuccess) return static_cast<int>(e);
    const int sms = di.sms;
    const int tiles = ((p.M + kBM - 1) / kBM) * ((p.N + BN - 1) / BN) * p.k_splits;
    const int grid = tiles < sms ? tiles : sms;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kGemmDynSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // may start while its predecessor finishes
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_dependent_launch ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, gemm_kernel<BN>, ma, mb, p);
    if (e != cudaSuccess || p.k_splits == 1) return static_cast<int>(e);
    const int64_t mn = static_cast<int64_t>(p.M) * p.N;
    int64_t rblocks = (mn + 255) / 256;
    if (rblocks > 148 * 8) rblocks = 148 * 8;
    splitk_reduce_kernel<<<static_cast<unsigned>(rblocks), 256, 0, stream>>>(p.partial, p.alpha, p.alpha2, p.out, mn, p.k_splits);
    return static_cast<int>(cudaGetLastError());
}



}  // namespace gemm
}  // namespace nvfp4
