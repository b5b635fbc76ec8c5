// NVFP4 block-scaled GEMM for sm_100a:
//   out[M, N] (bf16) = alpha * sum_k dq(a)[m, k] * dq(b)[n, k]
// with a, b packed E2M1 (K-major) and one UE4M3 scale per 16 elements stored in the
// 128x4-tiled layout the quantizer writes.  Replaces vllm's cutlass_scaled_fp4_mm
// (vllm/_custom_ops.py:741-752), the consumer efsotr/nvfp4quant_test names at README.md:68.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      producer: TMA tile loads of A / B (128-byte swizzle) and bulk copies of the
//               scale tiles into a 4-stage shared-memory ring
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
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s: far above any legitimate wait

__device__ uint32_t g_gemm_status;  // 0 = ok; else (role << 24) | detail of the wait that expired

template <int BN>
struct Cfg {
    static constexpr int kNG = BN / 128;                    // 128-row scale groups per B tile
    static constexpr int kAcc = (BN == 128) ? 2 : 1;        // accumulator buffers in TMEM
    static constexpr int kABytes = kBM * kBKBytes;          // 16 KiB
    static constexpr int kBBytes = BN * kBKBytes;
    static constexpr int kSfaBytes = 2048;                  // 128 rows x 16 blocks
    static constexpr int kSfbBytes = 2048 * kNG;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
    static constexpr int kSfaCol = kAcc * BN;               // TMEM column of the A scales
    static constexpr int kSfbCol = kSfaCol + 16;            // TMEM column of the B scales
    static_assert(kSfbCol + 16 * kNG <= kTmemCols, "TMEM budget");
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
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p; }" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
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

// K-major operand tile, 128-byte swizzle: rows are 128 B apart, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3ffffu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Scale tile: 32 rows x 16 B, unswizzled; 8-row core matrices 128 B apart.
__device__ __forceinline__ uint64_t smem_desc_sf(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3ffffu) >> 4) | (static_cast<uint64_t>(128 >> 4) << 32) | (1ull << 46);
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
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - raw_addr);
    // ring: [stage][A | B | SFA | SFB]; then barriers
    uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + kStages * C::kStageBytes);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * kStages + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
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
    const int total_tiles = m_tiles * n_tiles;
    const int k_tiles = (p.K + kBK - 1) / kBK;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int mt = tile % m_tiles, nt = tile / m_tiles;
                for (int kt = 0; kt < k_tiles; ++kt) {
                    if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, (1u << 24) | kt))) break;
                    const int kb_count = min(4, (p.K - kt * kBK + 63) / 64);  // 64-element K blocks in this stage
                    const uint32_t sf_bytes = 512u * kb_count;
                    int sfb_present = 0;
                    for (int g = 0; g < C::kNG; ++g) sfb_present += (nt * C::kNG + g < p.sfb_groups) ? 1 : 0;
                    const uint32_t tx = C::kABytes + C::kBBytes + sf_bytes * (1 + sfb_present);
                    mbar_expect_tx(full_bar(stage), tx);
                    const uint32_t sbase = base + stage * C::kStageBytes;
                    tma_load_2d(sbase, &tmap_a, kt * kBKBytes, mt * kBM, full_bar(stage));
                    tma_load_2d(sbase + C::kABytes, &tmap_b, kt * kBKBytes, nt * BN, full_bar(stage));
                    bulk_load_1d(sbase + C::kABytes + C::kBBytes,
                                 p.sfa + static_cast<int64_t>(mt) * p.sf_group_stride + static_cast<int64_t>(kt) * 2048,
                                 sf_bytes, full_bar(stage));
                    for (int g = 0; g < C::kNG; ++g) {
                        const int grp = nt * C::kNG + g;
                        if (grp < p.sfb_groups)
                            bulk_load_1d(sbase + C::kABytes + C::kBBytes + C::kSfaBytes + g * 2048,
                                         p.sfb + static_cast<int64_t>(grp) * p.sf_group_stride +
                                             static_cast<int64_t>(kt) * 2048,
                                         sf_bytes, full_bar(stage));
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc<BN>();
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                if (!(ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, (2u << 24) | 0xffff))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kt = 0; kt < k_tiles; ++kt) {
                    if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, (2u << 24) | kt))) break;
                    tc_fence_after();
                    const int kb_count = min(4, (p.K - kt * kBK + 63) / 64);
                    const uint32_t sbase = base + stage * C::kStageBytes;
                    const uint32_t sfa_s = sbase + C::kABytes + C::kBBytes;
                    const uint32_t sfb_s = sfa_s + C::kSfaBytes;
                    for (int kb = 0; kb < kb_count; ++kb) {
                        tc_cp_32x128b_warpx4(tmem_base + C::kSfaCol + 4 * kb, smem_desc_sf(sfa_s + 512 * kb));
                        for (int g = 0; g < C::kNG; ++g)
                            tc_cp_32x128b_warpx4(tmem_base + C::kSfbCol + 4 * C::kNG * kb + 4 * g,
                                                 smem_desc_sf(sfb_s + 2048 * g + 512 * kb));
                    }
                    const uint64_t adesc = smem_desc_sw128(sbase);
                    const uint64_t bdesc = smem_desc_sw128(sbase + C::kABytes);
                    for (int kb = 0; kb < kb_count; ++kb) {
                        // 32 bytes of K per instruction: advance the descriptor start address by 2 (x16 B)
                        tc_mma_nvf4(d_tmem, adesc + 2u * kb, bdesc + 2u * kb, idesc, tmem_base + C::kSfaCol + 4 * kb,
                                    tmem_base + C::kSfbCol + 4 * C::kNG * kb, (kt > 0 || kb > 0) ? 1u : 0u);
                    }
                    tc_commit(empty_bar(stage));  // slot reusable once these MMAs have read it
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                tc_commit(tfull_bar(acc));  // accumulator complete
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
            const int mt = tile % m_tiles, nt = tile / m_tiles;
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
    const int tiles = ((p.M + kBM - 1) / kBM) * ((p.N + BN - 1) / BN);
    const int grid = tiles < sms ? tiles : sms;
    gemm_kernel<BN><<<grid, kThreads, C::kSmemBytes, stream>>>(ma, mb, p);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace gemm
}  // namespace nvfp4

extern "C" size_t nvfp4_gemm_workspace_bytes(int64_t, int64_t, int64_t) { return 0; }

extern "C" int nvfp4_gemm_launch(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                                 const float* alpha, void* out_bf16, int64_t M, int64_t N, int64_t K, void* workspace,
                                 size_t workspace_bytes, void* stream) {
    using namespace nvfp4;
    (void)workspace;
    (void)workspace_bytes;
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
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Wide tiles feed the tensor pipe best; narrow ones keep more SMs busy when there are few tiles.
    const int64_t wide_tiles = ((M + 127) / 128) * ((N + 255) / 256);
    if (N > 128 && wide_tiles >= 148) return gemm::launch<256>(a, b, p, s);
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
