// NVFP4 quantizer for sm_100a: ScaleSweep (unweighted and importance-weighted)
// and the amax baseline, one kernel family.
//
// Behaviour follows efsotr/nvfp4quant_test:
//   kernels/kernel_ScaleSweep_MSE.py:271-377  (unweighted sweep, RNE base, -3..+7)
//   kernels/kernel_ScaleSweep.py:290-416      (weighted sweep, floor base, -8..+7)
// and, for the amax variant, the NVFP4 recipe of vllm's scaled_fp4_quant.
//
// Bit-exactness rules kept here: fp32 everywhere with explicit round-to-nearest
// operations (no contraction), `1/scale` through div.full.f32, squared errors
// accumulated as one serial FMA chain over elements 0..15 (unweighted) or as the
// fixed pairwise tree (weighted), candidates visited in ascending raw order with
// a strict `<`, so the lowest raw code wins ties.
//
// Mapping: one 16-element block per thread; a warp covers 32 consecutive blocks
// of one row (1 KiB of bf16).  Three interchangeable loop bodies give identical
// bytes: the scalar transcription (1), one candidate per trip with packed
// multiplies and the mixed-precision subtract (2), and the default (3): two
// candidates per trip whose FMA chains share one f32x2 instruction (each lane of
// a packed instruction is an independent IEEE operation).
//
// Body 4 is body 3 with the tensor-wide global scale (helper.py:96-100: amax / (6 * fp8_max) and its reciprocal)
// computed inside the same launch: every thread keeps its block in registers, the CTAs combine their maxima
// through a scratch word and wait for one another (cooperative launch: all CTAs are resident; the wait is bounded
// by the global timer), then the sweep runs as usual.  x is read from HBM once and one launch replaces two; the
// tensor must fit the resident grid (about 3 M elements on a B200).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace nvfp4 {
namespace {

constexpr int kThreads = 256;
// Resident CTAs per SM the register allocation aims for: the unweighted sweep fits 5 (48 registers) without
// spilling; the weighted one keeps 16 importance weights live and needs 64 registers (4 CTAs).
#ifndef NVFP4_QUANT_MIN_BLOCKS
#define NVFP4_QUANT_MIN_BLOCKS 5
#endif
// The two-dimensional-grid body has less index arithmetic alive and takes one more CTA per SM (40 registers, a few
// bytes of spill outside the loop): 121.1 -> 118.5 us at 8192 x 8192; the flat body gets slower with the same bound.
// Weighted sweep, two-dimensional grid, at 8192 x 8192: 5 CTAs (48 registers, spills) 223 us, 4 CTAs (64) 192 us,
// 3 CTAs (80) 199 us, 2 CTAs (90, importance pairs kept in registers) 205 us.
#ifndef NVFP4_QUANT_MIN_BLOCKS_2D
#define NVFP4_QUANT_MIN_BLOCKS_2D 6
#endif
#ifndef NVFP4_QUANT_MIN_BLOCKS_W2D
#define NVFP4_QUANT_MIN_BLOCKS_W2D 4
#endif
// Body 9 (a few tokens): CTAs of 64 threads over the slots of the real rows only.  A 256-thread CTA puts two warps on
// every scheduler of one SM, and a warp's sweep is ~750 instructions; 64-thread CTAs spread the same blocks over four
// times as many SMs with at most one warp per scheduler.  The padding rows of the tiled scale layout (127 of 128 for
// one token) get a few CTAs at the end of the grid that write their zero words.
constexpr int kSmallThreads = 64;
// Real 16-element blocks up to which body 9 is the default.  Measured in a chain of launches (us, body 9 against the
// better of the other bodies): unweighted 1 x 4096 1.72 / 2.38, 1 x 14336 1.78 / 2.74, 32 x 8192 1.94 / 2.81, 64 x 8192
// 2.50 / 2.84, 128 x 4096 2.55 / 2.54, 96 x 8192 3.57 / 3.37; weighted 1 x 8192 2.35 / 3.85, 48 x 8192 3.59 / 4.87,
// 64 x 8192 3.61 / 4.07, 128 x 4096 3.59 / 3.40, 96 x 8192 6.39 / 5.28.
constexpr int64_t kSmallBlocks = 32768;
constexpr int64_t kSmallBlocksWeighted = 24576;
__host__ __device__ constexpr int block_threads(int impl) { return impl == 9 ? kSmallThreads : kThreads; }
constexpr int min_blocks(int variant, int impl) {
    if (impl == 9) return 8;
    return variant == NVFP4_VARIANT_WEIGHTED ? (impl >= 6 ? NVFP4_QUANT_MIN_BLOCKS_W2D : 4)
           : (impl >= 6 && variant == NVFP4_VARIANT_MSE) ? NVFP4_QUANT_MIN_BLOCKS_2D
                                                         : NVFP4_QUANT_MIN_BLOCKS;
}

struct QuantParams {
    const void* x;
    const float* importance;
    const float* gs_inv;
    uint8_t* codes;
    uint8_t* scales;
    int64_t m, n;
    int64_t bin, bout;      // 16-element blocks per input / output row
    int64_t width, rows;    // slot grid: scale columns / rows that get written
    int64_t k_pad;          // padded scale columns (swizzled layout)
    int64_t total;          // rows * width
    int lower, ncand;
    int swizzled;
    // fused global-scale variant only
    float fp8_max;
    float* gs_out;          // [2]: global scale, its reciprocal
    uint32_t* fused_scratch;  // [4]: running maximum, arrivals, readers, unused; zero between calls
};

__device__ uint32_t g_quant_status;   // 0 = ok; 1 = the grid-wide wait of the fused kernel gave up
constexpr uint64_t kFusedWaitLimitNs = 2000000000ull;
__device__ uint64_t g_fused_wait_limit_ns = kFusedWaitLimitNs;   // settable from the host (nvfp4_quant_fused_set_wait_limit_ns)

template <int DT>
__device__ __forceinline__ void load16(const void* base, int64_t elem, float v[16]);

template <>
__device__ __forceinline__ void load16<NVFP4_DT_BF16>(const void* base, int64_t elem, float v[16]) {
    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + elem);
    uint4 a = __ldg(p), b = __ldg(p + 1);
    uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <>
__device__ __forceinline__ void load16<NVFP4_DT_F16>(const void* base, int64_t elem, float v[16]) {
    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + elem);
    uint4 a = __ldg(p), b = __ldg(p + 1);
    uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

template <>
__device__ __forceinline__ void load16<NVFP4_DT_F32>(const void* base, int64_t elem, float v[16]) {
    const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float4 f = __ldg(p + i);
        v[4 * i] = f.x;
        v[4 * i + 1] = f.y;
        v[4 * i + 2] = f.z;
        v[4 * i + 3] = f.w;
    }
}

__device__ __forceinline__ float max_abs16(const float v[16]) {
    float m[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1]));
    return fmaxf(fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3])), fmaxf(fmaxf(m[4], m[5]), fmaxf(m[6], m[7])));
}

// Candidate table: entry k describes raw code clamp(k - kTabPad, 1, 126), so a sweep that starts at
// tab[first + kTabPad] reads consecutive entries and needs no per-candidate clamping.
// .x = .y = 1/s (div.full.f32), .z = s*s, .w = the raw code (bit pattern).
constexpr int kTabPad = 64;
constexpr int kTabSize = 256;

// ---- scalar transcription: one candidate at a time --------------------------------------
template <bool WEIGHTED>
__device__ __forceinline__ uint32_t sweep_scalar(const float v[16], const float w[16], int first_idx, int ncand,
                                                 const float4* tab) {
    float best = __int_as_float(0x7f800000);
    uint32_t best_raw = 0;
#pragma unroll 1
    for (int i = 0; i < ncand; ++i) {
        const float4 e4 = tab[first_idx + i];
        const float2 e = make_float2(e4.x, e4.z);
        const uint32_t raw = __float_as_uint(e4.w);
        float err;
        if (!WEIGHTED) {
            float acc = 0.0f;
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                float x0 = __fmul_rn(v[2 * p], e.x), x1 = __fmul_rn(v[2 * p + 1], e.x), q0, q1;
                e2m1_round_pair(x0, x1, q0, q1);
                float d0 = __fsub_rn(q0, x0), d1 = __fsub_rn(q1, x1);
                acc = __fmaf_rn(d0, d0, acc);  // fma(d, d, +0) == mul.rn(d, d) for the first term
                acc = __fmaf_rn(d1, d1, acc);
            }
            err = __fmul_rn(acc, e.y);
        } else {
            float pe[8];
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                float x0 = __fmul_rn(v[2 * p], e.x), x1 = __fmul_rn(v[2 * p + 1], e.x), q0, q1;
                e2m1_round_pair(x0, x1, q0, q1);
                float d0 = __fsub_rn(q0, x0), d1 = __fsub_rn(q1, x1);
                float a = __fmul_rn(__fmul_rn(d0, d0), w[2 * p]);
                pe[p] = __fmaf_rn(__fmul_rn(d1, d1), w[2 * p + 1], a);
            }
            float t = __fadd_rn(__fadd_rn(__fadd_rn(pe[0], pe[1]), __fadd_rn(pe[2], pe[3])),
                                __fadd_rn(__fadd_rn(pe[4], pe[5]), __fadd_rn(pe[6], pe[7])));
            err = __fmul_rn(t, e.y);
        }
        if (err < best) {
            best = err;
            best_raw = raw;
        }
    }
    return best_raw;
}

// ---- paired: two candidates per loop trip; element pairs share the multiply and both
// conversions, the difference uses the mixed-precision subtract (f16 grid value minus fp32 x,
// one full-rate instruction, exact like cvt + sub), and the two candidates' accumulations
// share one f32x2 instruction -------------------------------------------------------------
__device__ __forceinline__ void e2m1_diff_pair(uint64_t x2, float& d0, float& d1) {
    asm("{ .reg .b8 b; .reg .b32 h; .reg .b16 lo, hi; .reg .f32 x0, x1;\n"
        "  mov.b64 {x0, x1}, %2;\n"
        "  cvt.rn.satfinite.e2m1x2.f32 b, x1, x0;\n"
        "  cvt.rn.f16x2.e2m1x2 h, b;\n"
        "  mov.b32 {lo, hi}, h;\n"
        "  sub.rn.f32.f16 %0, lo, x0;\n"
        "  sub.rn.f32.f16 %1, hi, x1; }"
        : "=f"(d0), "=f"(d1)
        : "l"(x2));
}

// NC > 0: the candidate count is the compile-time constant NC and the trips are unrolled (the table index and the
// loop control leave the instruction stream); NC = 0: `ncand` at run time, one rolled loop.
template <bool WEIGHTED, int NC = 0>
__device__ __forceinline__ uint32_t sweep_paired(const float v[16], const float w[16], int first_idx, int ncand_rt,
                                                 const float4* tab) {
    const int ncand = NC > 0 ? NC : ncand_rt;
    uint64_t vp[8];  // (v[2p], v[2p+1])
#pragma unroll
    for (int p = 0; p < 8; ++p) vp[p] = pack_f32x2(v[2 * p], v[2 * p + 1]);
    float best = __int_as_float(0x7f800000);
    uint32_t best_raw = 0;
    auto trip = [&](int i) {
        const float4 ea = tab[first_idx + i], eb = tab[first_idx + i + 1];
        const uint32_t raw_a = __float_as_uint(ea.w), raw_b = __float_as_uint(eb.w);
        const uint64_t inv_a = pack_f32x2(ea.x, ea.y), inv_b = pack_f32x2(eb.x, eb.y);
        uint64_t tot2;
        if (!WEIGHTED) {
            uint64_t acc2 = 0;  // (+0, +0): candidate a in the low lane, b in the high lane
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                float a0, a1, b0, b1;
                e2m1_diff_pair(mul_f32x2(vp[p], inv_a), a0, a1);
                e2m1_diff_pair(mul_f32x2(vp[p], inv_b), b0, b1);
                const uint64_t d0 = pack_f32x2(a0, b0), d1 = pack_f32x2(a1, b1);
                acc2 = fma_f32x2(d0, d0, acc2);
                acc2 = fma_f32x2(d1, d1, acc2);
            }
            tot2 = acc2;
        } else {
            uint64_t pe[8];
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                float a0, a1, b0, b1;
                e2m1_diff_pair(mul_f32x2(vp[p], inv_a), a0, a1);
                e2m1_diff_pair(mul_f32x2(vp[p], inv_b), b0, b1);
                const uint64_t d0 = pack_f32x2(a0, b0), d1 = pack_f32x2(a1, b1);
                const uint64_t t = mul_f32x2(mul_f32x2(d0, d0), pack_f32x2(w[2 * p], w[2 * p]));
                pe[p] = fma_f32x2(mul_f32x2(d1, d1), pack_f32x2(w[2 * p + 1], w[2 * p + 1]), t);
            }
            tot2 = add_f32x2(add_f32x2(add_f32x2(pe[0], pe[1]), add_f32x2(pe[2], pe[3])),
                             add_f32x2(add_f32x2(pe[4], pe[5]), add_f32x2(pe[6], pe[7])));
        }
        float err_a, err_b;
        unpack_f32x2(mul_f32x2(tot2, pack_f32x2(ea.z, eb.z)), err_a, err_b);
        if (err_a < best) {
            best = err_a;
            best_raw = raw_a;
        }
        if (err_b < best) {
            best = err_b;
            best_raw = raw_b;
        }
    };
    if (NC > 0 && !WEIGHTED) {
#pragma unroll
        for (int i = 0; i + 1 < NC; i += 2) trip(i);
    } else if (NC > 0) {
#pragma unroll 2
        for (int i = 0; i + 1 < NC; i += 2) trip(i);
    } else {
#pragma unroll 1
        for (int i = 0; i + 1 < ncand; i += 2) trip(i);
    }
    if (ncand & 1) {  // odd count: the last candidate alone, scalar chain
        const float4 e4 = tab[first_idx + ncand - 1];
        const float2 e = make_float2(e4.x, e4.z);
        const uint32_t raw = __float_as_uint(e4.w);
        const uint64_t inv2 = pack_f32x2(e4.x, e4.y);
        float err;
        if (!WEIGHTED) {
            float acc = 0.0f;
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                float d0, d1;
                e2m1_diff_pair(mul_f32x2(vp[p], inv2), d0, d1);
                acc = __fmaf_rn(d0, d0, acc);
                acc = __fmaf_rn(d1, d1, acc);
            }
            err = __fmul_rn(acc, e.y);
        } else {
            float pe[8];
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                float d0, d1;
                e2m1_diff_pair(mul_f32x2(vp[p], inv2), d0, d1);
                const float a = __fmul_rn(__fmul_rn(d0, d0), w[2 * p]);
                pe[p] = __fmaf_rn(__fmul_rn(d1, d1), w[2 * p + 1], a);
            }
            const float t = __fadd_rn(__fadd_rn(__fadd_rn(pe[0], pe[1]), __fadd_rn(pe[2], pe[3])),
                                      __fadd_rn(__fadd_rn(pe[4], pe[5]), __fadd_rn(pe[6], pe[7])));
            err = __fmul_rn(t, e.y);
        }
        if (err < best) {
            best = err;
            best_raw = raw;
        }
    }
    return best_raw;
}

// ---- one candidate per trip, element pairs share the multiply, scalar FMA chain ----------------
template <bool WEIGHTED>
__device__ __forceinline__ uint32_t sweep_single(const float v[16], const float w[16], int first_idx, int ncand,
                                                 const float4* tab) {
    uint64_t vp[8];
#pragma unroll
    for (int p = 0; p < 8; ++p) vp[p] = pack_f32x2(v[2 * p], v[2 * p + 1]);
    float best = __int_as_float(0x7f800000);
    uint32_t best_raw = 0;
#pragma unroll 1
    for (int i = 0; i < ncand; ++i) {
        const float4 e4 = tab[first_idx + i];
        const float2 e = make_float2(e4.x, e4.z);
        const uint32_t raw = __float_as_uint(e4.w);
        const uint64_t inv2 = pack_f32x2(e4.x, e4.y);
        float err;
        if (!WEIGHTED) {
            float acc = 0.0f;
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                float d0, d1;
                e2m1_diff_pair(mul_f32x2(vp[p], inv2), d0, d1);
                acc = __fmaf_rn(d0, d0, acc);
                acc = __fmaf_rn(d1, d1, acc);
            }
            err = __fmul_rn(acc, e.y);
        } else {
            float pe[8];
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                float d0, d1;
                e2m1_diff_pair(mul_f32x2(vp[p], inv2), d0, d1);
                const float a = __fmul_rn(__fmul_rn(d0, d0), w[2 * p]);
                pe[p] = __fmaf_rn(__fmul_rn(d1, d1), w[2 * p + 1], a);
            }
            const float t = __fadd_rn(__fadd_rn(__fadd_rn(pe[0], pe[1]), __fadd_rn(pe[2], pe[3])),
                                      __fadd_rn(__fadd_rn(pe[4], pe[5]), __fadd_rn(pe[6], pe[7])));
            err = __fmul_rn(t, e.y);
        }
        if (err < best) {
            best = err;
            best_raw = raw;
        }
    }
    return best_raw;
}

template <int DT, int VARIANT, int IMPL>
__global__ void __launch_bounds__(block_threads(IMPL), min_blocks(VARIANT, IMPL))
quant_kernel(const QuantParams p) {
    constexpr int T = block_threads(IMPL);   // threads per CTA
    static_assert(kTabSize % T == 0, "every thread builds the same number of table entries");
    __shared__ float4 tab[kTabSize];
    constexpr bool FUSED = IMPL == 4;
    static_assert(!FUSED || VARIANT != NVFP4_VARIANT_AMAX, "the fused variant covers the two sweeps");
    // Launched as a programmatic dependent: the input, the global scale and the output buffers may still be in use by
    // the kernel before this one on the stream, so everything waits.  The kernel BEHIND this one may be scheduled right
    // away, even before that wait is over: whatever it does ahead of its own wait (a GEMM streams a prepared, constant
    // weight) depends on neither this kernel nor the ones before it, and its wait covers this kernel's completion,
    // which in turn comes after this wait.
    griddep_launch();
    if (!FUSED) griddep_wait();
    // everything the kernel before this one may have written is read through pointers taken behind the wait
    const void* const x_in = after_wait(p.x);
    const float* const importance_in = after_wait(p.importance);
    float gs_inv = FUSED ? 0.0f : load_f32_after_wait(p.gs_inv);
    // Body 6 = body 3 with a two-dimensional grid: blockIdx.x is the row, blockIdx.y the 256-block column chunk.
    // The row is then uniform over the CTA, so the division below, the row part of the addresses and most of the
    // tiled scale offset leave the per-thread instruction stream.  Used when the slot grid is a whole number of
    // chunks wide (e.g. 512 blocks per row at 8192 columns); narrow or ragged widths keep the flat numbering.
    constexpr bool GRID2D = IMPL == 6 || IMPL == 7 || IMPL == 8;   // 7 = 6 with the reference's candidate count compiled in
    constexpr bool WHOLE = IMPL == 8;                              // 8 = 7 on tensors without any padding: no predicates
    constexpr bool SMALL = IMPL == 9;   // threads for the slots of the real rows only (see the end of the kernel)
    const int64_t id = GRID2D ? 0 : static_cast<int64_t>(blockIdx.x) * T + threadIdx.x;
    const bool in_range = GRID2D ? true : id < (SMALL ? p.m * p.width : p.total);
    int64_t row = 0, col = 0;
    if (GRID2D) {
        row = blockIdx.x;
        col = static_cast<int64_t>(blockIdx.y) * kThreads + threadIdx.x;
    } else if (in_range) {
        if (p.total <= 0x7fffffffLL) {  // 32-bit division is several times cheaper than the 64-bit one
            const uint32_t r32 = static_cast<uint32_t>(id) / static_cast<uint32_t>(p.width);
            row = r32;
            col = static_cast<uint32_t>(id) - r32 * static_cast<uint32_t>(p.width);
        } else {
            row = id / p.width;
            col = id - row * p.width;
        }
    }
    const bool valid = WHOLE ? true : (in_range && row < p.m && col < p.bout);
    if (SMALL && static_cast<int64_t>(blockIdx.x) * T >= p.m * p.width) {
        // A CTA behind the real rows' slots.  The rows m .. rows-1 of the tiled scale layout (127 of 128 for one token)
        // hold no data; these CTAs write their zero scale bytes, four 32-bit words (of four columns each) per thread,
        // and leave before the candidate table is built.  (Rows beyond m exist only in the tiled layout, whose width is
        // a multiple of 4; the launcher sizes this part of the grid, and at most 127 rows are padding.)
        const uint32_t words_per_row = static_cast<uint32_t>(p.width >> 2);
        const uint32_t words = static_cast<uint32_t>(p.rows - p.m) * words_per_row;
        const uint32_t real_ctas = static_cast<uint32_t>((p.m * p.width + T - 1) / T);
        const uint32_t fill_threads = (gridDim.x - real_ctas) * T;
        for (uint32_t wi = (blockIdx.x - real_ctas) * T + threadIdx.x; wi < words; wi += fill_threads) {
            const uint32_t r = wi / words_per_row;
            const uint32_t c = (wi - r * words_per_row) * 4u;
            *reinterpret_cast<uint32_t*>(p.scales + swizzled_scale_offset(p.m + r, c, p.k_pad)) = 0u;
        }
        return;
    }

    float v[16], w[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        v[j] = 0.0f;
        w[j] = 0.0f;
    }
    if (WHOLE || (valid && col < p.bin)) {
        load16<DT>(x_in, row * p.n + col * kBlock, v);
        if (VARIANT == NVFP4_VARIANT_WEIGHTED) load16<NVFP4_DT_F32>(importance_in, col * kBlock, w);
    }

    // The global scale and the block's elements were requested above; the candidate table is built while they are
    // on their way (at small batch sizes nothing else hides a trip to memory).  The amax variant needs no table: its
    // one multiplier per block is two reciprocals away from the scale byte, and without the table there is no
    // CTA-wide barrier between the loads and their use.
    if (VARIANT != NVFP4_VARIANT_AMAX) {
#pragma unroll
        for (int t = threadIdx.x; t < kTabSize; t += T) {   // one entry per thread with 256 threads, four with 64
            const uint32_t raw = static_cast<uint32_t>(min(max(t - kTabPad, 1), 126));
            const float s = e4m3_to_f32(raw);
            float4 e;
            e.x = e.y = div_full(1.0f, s);
            e.z = __fmul_rn(s, s);
            e.w = __uint_as_float(raw);
            tab[t] = e;
        }
        __syncthreads();
    }

    if (FUSED) {
        // tensor-wide maximum on fp32 magnitude bit patterns (a NaN pattern is larger than +inf, as torch's max wants)
        __shared__ uint32_t warp_max[kThreads / 32];
        __shared__ float gs_inv_shared;
        uint32_t bits = 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) bits = max(bits, __float_as_uint(v[j]) & 0x7fffffffu);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
        if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = bits;
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t b = 0;
            for (int i = 0; i < kThreads / 32; ++i) b = max(b, warp_max[i]);
            volatile uint32_t* sc = p.fused_scratch;
            atomicMax(p.fused_scratch, b);
            __threadfence();
            // scratch[3] != 0 is a testing hook: CTA 0 then withholds its arrival, so that every wait below runs into
            // the limit and the error path (status word, no hang) can be exercised
            if (!(blockIdx.x == 0 && sc[3] != 0u)) atomicAdd(p.fused_scratch + 1, 1u);
            // every CTA of a cooperative launch is resident, so the others will arrive; bounded all the same
            uint64_t t0 = 0;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
            while (sc[1] < gridDim.x) {
                uint64_t t1;
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
                if (t1 - t0 > g_fused_wait_limit_ns) {
                    atomicExch(&g_quant_status, 1u);
                    break;
                }
                __nanosleep(64);
            }
            __threadfence();
            const float amax = __uint_as_float(sc[0]);
            const float inv_den = __fdiv_rn(1.0f, __fmul_rn(6.0f, p.fp8_max));
            const float gs = __fmul_rn(amax, inv_den);
            const float gsi = __fdiv_rn(1.0f, gs);
            gs_inv_shared = gsi;
            __threadfence();
            // the last CTA to have read the maximum publishes the result and leaves the scratch zeroed
            if (atomicAdd(p.fused_scratch + 2, 1u) == gridDim.x - 1) {
                p.gs_out[0] = gs;
                p.gs_out[1] = gsi;
                sc[0] = 0u;
                sc[1] = 0u;
                sc[2] = 0u;
            }
        }
        __syncthreads();
        gs_inv = gs_inv_shared;
    }

    uint32_t sbyte = 0;
    float inv = 0.0f;
    // Body 5 = body 3 plus: a warp whose 32 slots are all padding (rows beyond m in the tiled scale layout: 127 of
    // 128 rows for a single token) has nothing to sweep and only writes its zero scale bytes below.  A separate
    // instantiation because the vote and branch cost the full-size kernel 6 % (8192 x 8192: 123.7 -> 131.8 us);
    // the launcher picks it when at least a quarter of the slot grid is padding rows.
    if ((IMPL == 5 || IMPL == 9) && !__any_sync(0xffffffffu, valid)) {
        // nothing
    } else if (VARIANT == NVFP4_VARIANT_AMAX) {
        const float amax = max_abs16(v);
        const float sf = __fmul_rn(gs_inv, __fmul_rn(amax, rcp_approx_ftz(6.0f)));
        sbyte = f32_to_e4m3(sf);
        const uint32_t raw = sbyte & 0x7fu;
        inv = (raw == 0) ? 0.0f : rcp_approx_ftz(__fmul_rn(e4m3_to_f32(raw), rcp_approx_ftz(gs_inv)));
    } else {
        const uint64_t gs2 = pack_f32x2(gs_inv, gs_inv);
#pragma unroll
        for (int q = 0; q < 8; ++q)   // packed multiply: each lane is the same IEEE product as a scalar mul.rn
            unpack_f32x2(mul_f32x2(pack_f32x2(v[2 * q], v[2 * q + 1]), gs2), v[2 * q], v[2 * q + 1]);
        const float amax = max_abs16(v);
        const float base_scale = __fmul_rn(amax, __uint_as_float(0x3E2AAAABu));  // fp32(1/6)
        const uint32_t base_fp8 = f32_to_e4m3(base_scale);
        int base_raw = static_cast<int>(base_fp8);
        if (VARIANT == NVFP4_VARIANT_WEIGHTED) base_raw -= (e4m3_to_f32(base_fp8) > base_scale) ? 1 : 0;
        constexpr bool W = VARIANT == NVFP4_VARIANT_WEIGHTED;
        // clamping the start once is enough: with it below -kTabPad every candidate is raw 1, above 127 every one 126
        const int first_idx = min(max(base_raw + p.lower, -kTabPad), 127) + kTabPad;
        sbyte = (IMPL == 1)   ? sweep_scalar<W>(v, w, first_idx, p.ncand, tab)
                : (IMPL == 2) ? sweep_single<W>(v, w, first_idx, p.ncand, tab)
                : (IMPL == 7 || IMPL == 8 || (IMPL == 9 && p.ncand == (W ? 16 : 11)))
                    ? sweep_paired<W, W ? 16 : 11>(v, w, first_idx, p.ncand, tab)
                    : sweep_paired<W>(v, w, first_idx, p.ncand, tab);
        // sbyte is 0 only when no candidate had a comparable (non-NaN, < inf) error: 1/0 as the reference computes it
        inv = (sbyte == 0) ? div_full(1.0f, 0.0f) : tab[sbyte + kTabPad].x;
    }

    if (valid) {
        const uint64_t inv2 = pack_f32x2(inv, inv);
        float x[16];
#pragma unroll
        for (int q = 0; q < 8; ++q)
            unpack_f32x2(mul_f32x2(pack_f32x2(v[2 * q], v[2 * q + 1]), inv2), x[2 * q], x[2 * q + 1]);
        const uint32_t lo = f32x8_to_e2m1x8(x[0], x[1], x[2], x[3], x[4], x[5], x[6], x[7]);
        const uint32_t hi = f32x8_to_e2m1x8(x[8], x[9], x[10], x[11], x[12], x[13], x[14], x[15]);
        *reinterpret_cast<uint2*>(p.codes + (row * p.bout + col) * 8) = make_uint2(lo, hi);
    } else {
        sbyte = 0;  // padding rows / columns of the scale buffer read as zero scales
    }

    // Scale store.  With width % 4 == 0 (always true for the swizzled layout) lanes
    // 4q..4q+3 hold four consecutive blocks of one row: merge them into one 32-bit store.
    if ((p.width & 3) == 0) {
        const uint32_t lane = threadIdx.x & 31;
        uint32_t word = sbyte << (8 * (lane & 3));
        word |= __shfl_xor_sync(0xffffffffu, word, 1);
        word |= __shfl_xor_sync(0xffffffffu, word, 2);
        if (in_range && (lane & 3) == 0) {
            const int64_t off = p.swizzled ? swizzled_scale_offset(row, col, p.k_pad) : row * p.width + col;
            *reinterpret_cast<uint32_t*>(p.scales + off) = word;
        }
    } else if (in_range) {
        p.scales[row * p.width + col] = static_cast<uint8_t>(sbyte);
    }
}


template <int DT, int VARIANT>
cudaError_t launch_impl(int impl, const QuantParams& p, cudaStream_t stream) {
    const int64_t grid = (p.total + kThreads - 1) / kThreads;
    // body 8: tensors without padding whose rows are whole 256-block chunks (every slot of the scale layout is a
    // real block): body 7 without its validity predicates
    const bool whole = VARIANT != NVFP4_VARIANT_AMAX && p.rows == p.m && p.bin == p.bout && p.bout == p.width &&
                       (p.width % kThreads) == 0 && p.width / kThreads <= 65535 && p.rows <= 0x7fffffffLL &&
                       (VARIANT == NVFP4_VARIANT_MSE ? p.ncand == 11 : p.ncand == 16);
    const bool small = VARIANT != NVFP4_VARIANT_AMAX &&
                       p.m * p.bout <= (VARIANT == NVFP4_VARIANT_WEIGHTED ? kSmallBlocksWeighted : kSmallBlocks);
    if constexpr (VARIANT != NVFP4_VARIANT_AMAX) {
        if ((impl == 8 || (impl == 0 && !small)) && whole) {
            const dim3 grid2(static_cast<unsigned>(p.rows), static_cast<unsigned>(p.width / kThreads));
            return launch_dependent(quant_kernel<DT, VARIANT, 8>, grid2, dim3(kThreads), 0, stream, p);
        }
    }
    // body 9: tensors of a few tokens (up to kSmallBlocks real blocks), where latency is all that matters
    if (impl == 9 || (impl == 0 && small)) {
        // CTAs for the slots of the real rows, then CTAs that zero the padding rows' scale words (4 words per thread)
        const int64_t pad_words = (p.rows - p.m) * (p.width >> 2);
        if (pad_words > 0x7fffffffLL) return cudaErrorInvalidValue;   // at most 127 rows: a width beyond 2^26 columns
        const int64_t grid9 = (p.m * p.width + kSmallThreads - 1) / kSmallThreads +
                              (pad_words + 4 * kSmallThreads - 1) / (4 * kSmallThreads);
        if (grid9 > 0x7fffffffLL) return cudaErrorInvalidValue;
        return launch_dependent(quant_kernel<DT, VARIANT, 9>, static_cast<unsigned>(grid9), dim3(kSmallThreads), 0, stream, p);
    }
    if (impl >= 8) impl = 0;
    cudaError_t e;
    if (impl == 1)
        e = launch_dependent(quant_kernel<DT, VARIANT, 1>, static_cast<unsigned>(grid), dim3(kThreads), 0, stream, p);
    else if (impl == 2)
        e = launch_dependent(quant_kernel<DT, VARIANT, 2>, static_cast<unsigned>(grid), dim3(kThreads), 0, stream, p);
    else if (impl == 5 || (impl == 0 && (p.rows - p.m) * 4 >= p.rows))
        e = launch_dependent(quant_kernel<DT, VARIANT, 5>, static_cast<unsigned>(grid), dim3(kThreads), 0, stream, p);
    else if ((impl == 6 || impl == 7 || impl == 0) && (p.width % kThreads) == 0 && p.width / kThreads <= 65535 &&
             p.rows <= 0x7fffffffLL) {
        const dim3 grid2(static_cast<unsigned>(p.rows), static_cast<unsigned>(p.width / kThreads));
        // the reference's own windows (11 candidates unweighted, 16 weighted) have an unrolled instantiation
        const bool fixed = VARIANT == NVFP4_VARIANT_MSE ? p.ncand == 11 : VARIANT == NVFP4_VARIANT_WEIGHTED && p.ncand == 16;
        if (fixed && (impl == 7 || (impl == 0 && VARIANT == NVFP4_VARIANT_MSE)))
            e = launch_dependent(quant_kernel<DT, VARIANT, 7>, grid2, dim3(kThreads), 0, stream, p);
        else
            e = launch_dependent(quant_kernel<DT, VARIANT, 6>, grid2, dim3(kThreads), 0, stream, p);
    }
    else
        e = launch_dependent(quant_kernel<DT, VARIANT, 3>, static_cast<unsigned>(grid), dim3(kThreads), 0, stream, p);
    return e;
}

template <int DT>
cudaError_t launch_variant(int variant, int impl, const QuantParams& p, cudaStream_t stream) {
    switch (variant) {
        case NVFP4_VARIANT_MSE: return launch_impl<DT, NVFP4_VARIANT_MSE>(impl, p, stream);
        case NVFP4_VARIANT_WEIGHTED: return launch_impl<DT, NVFP4_VARIANT_WEIGHTED>(impl, p, stream);
        default: return launch_impl<DT, NVFP4_VARIANT_AMAX>(impl, p, stream);
    }
}

}  // namespace
}  // namespace nvfp4

extern "C" int nvfp4_quant_launch_impl(int impl, int variant, const void* x, int x_dtype, const float* importance,
                                       const float* gs_inv, uint8_t* codes, uint8_t* scales, int64_t m, int64_t n,
                                       int64_t padded_n, int lower, int upper, int swizzled, void* stream) {
    using namespace nvfp4;
    if (variant < NVFP4_VARIANT_MSE || variant > NVFP4_VARIANT_AMAX) return NVFP4_ERR_BAD_ENUM;
    if (x_dtype < NVFP4_DT_BF16 || x_dtype > NVFP4_DT_F32) return NVFP4_ERR_BAD_ENUM;
    if (impl < 0 || impl > 9 || impl == 4) return NVFP4_ERR_BAD_ENUM;
    if (m < 0 || n < 0 || (n % kBlock) != 0 || (padded_n % kBlock) != 0 || padded_n < n) return NVFP4_ERR_BAD_SHAPE;
    if (variant != NVFP4_VARIANT_AMAX && (upper < lower || upper - lower + 1 > 64)) return NVFP4_ERR_BAD_RANGE;
    QuantParams p;
    p.m = m;
    p.n = n;
    p.bin = n / kBlock;
    p.bout = padded_n / kBlock;
    p.k_pad = round_up_i64(p.bout, 4);
    p.swizzled = swizzled ? 1 : 0;
    p.width = swizzled ? p.k_pad : p.bout;
    p.rows = swizzled ? round_up_i64(m, 128) : m;
    p.total = p.rows * p.width;
    if (p.total == 0) return NVFP4_OK;
    if ((p.total + kThreads - 1) / kThreads > 0x7fffffffLL) return NVFP4_ERR_TOO_LARGE;
    if (!gs_inv || !codes || !scales || (!x && m * n > 0)) return NVFP4_ERR_NULL_POINTER;
    if (variant == NVFP4_VARIANT_WEIGHTED && !importance && n > 0) return NVFP4_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(codes) & 7) ||
        (reinterpret_cast<uintptr_t>(gs_inv) & 3))
        return NVFP4_ERR_MISALIGNED;
    if (swizzled && (reinterpret_cast<uintptr_t>(scales) & 3)) return NVFP4_ERR_MISALIGNED;
    if (!swizzled && (p.width & 3) == 0 && (reinterpret_cast<uintptr_t>(scales) & 3)) return NVFP4_ERR_MISALIGNED;
    if (variant == NVFP4_VARIANT_WEIGHTED && (reinterpret_cast<uintptr_t>(importance) & 15)) return NVFP4_ERR_MISALIGNED;
    p.x = x;
    p.importance = importance;
    p.gs_inv = gs_inv;
    p.codes = codes;
    p.scales = scales;
    p.lower = lower;
    p.ncand = (variant == NVFP4_VARIANT_AMAX) ? 0 : upper - lower + 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t err;
    switch (x_dtype) {
        case NVFP4_DT_BF16: err = launch_variant<NVFP4_DT_BF16>(variant, impl, p, s); break;
        case NVFP4_DT_F16: err = launch_variant<NVFP4_DT_F16>(variant, impl, p, s); break;
        default: err = launch_variant<NVFP4_DT_F32>(variant, impl, p, s); break;
    }
    return static_cast<int>(err);
}

namespace nvfp4 {
namespace {
template <int DT, int VARIANT>
cudaError_t launch_fused(const QuantParams& p, int sms, cudaStream_t stream, bool* too_large) {
    const int64_t grid = (p.total + kThreads - 1) / kThreads;
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quant_kernel<DT, VARIANT, 4>, kThreads, 0);
    if (e != cudaSuccess) return e;
    if (grid > static_cast<int64_t>(per_sm) * sms) {
        *too_large = true;
        return cudaSuccess;
    }
    QuantParams q = p;
    void* args[] = {&q};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(quant_kernel<DT, VARIANT, 4>),
                                       dim3(static_cast<unsigned>(grid)), dim3(kThreads), args, 0, stream);
}
template <int DT>
cudaError_t launch_fused_variant(int variant, const QuantParams& p, int sms, cudaStream_t stream, bool* too_large) {
    if (variant == NVFP4_VARIANT_MSE) return launch_fused<DT, NVFP4_VARIANT_MSE>(p, sms, stream, too_large);
    return launch_fused<DT, NVFP4_VARIANT_WEIGHTED>(p, sms, stream, too_large);
}
}  // namespace
}  // namespace nvfp4

// Global scale, then the quantizer with that scale, as two launches from one host call: what get_nvfp4_global_scale followed
// by scalesweep_*_quant_out do (helper.py:96-100, bench.py:57-67 of the reference), for callers that pay per host call
// (an eager decode loop).  gs_out[0] = amax|x| / (6 * fp8_max), gs_out[1] = 1 / gs_out[0]; `scratch` = the 2 zeroed words
// of nvfp4_global_scale_launch.  Both kernels are programmatic dependent launches; bytes equal the two separate calls.
extern "C" int nvfp4_quant_chain_launch(int variant, const void* x, int x_dtype, const float* importance, float fp8_max,
                                        float* gs_out, uint32_t* scratch, uint8_t* codes, uint8_t* scales, int64_t m,
                                        int64_t n, int64_t padded_n, int lower, int upper, int swizzled, void* stream) {
    if (m <= 0 || n <= 0) return NVFP4_ERR_BAD_SHAPE;   // an empty tensor has no maximum
    if (!(fp8_max > 0.0f)) return NVFP4_ERR_BAD_RANGE;
    if (!gs_out) return NVFP4_ERR_NULL_POINTER;
    const int st = nvfp4_global_scale_launch(x, x_dtype, m * n, fp8_max, gs_out, scratch, stream);
    if (st != NVFP4_OK) return st;
    return nvfp4_quant_launch(variant, x, x_dtype, importance, gs_out + 1, codes, scales, m, n, padded_n, lower, upper,
                              swizzled, stream);
}

extern "C" int nvfp4_quant_fused_launch(int variant, const void* x, int x_dtype, const float* importance, float fp8_max,
                                        float* gs_out, uint32_t* scratch, uint8_t* codes, uint8_t* scales, int64_t m,
                                        int64_t n, int64_t padded_n, int lower, int upper, int swizzled, void* stream) {
    using namespace nvfp4;
    if (variant != NVFP4_VARIANT_MSE && variant != NVFP4_VARIANT_WEIGHTED) return NVFP4_ERR_BAD_ENUM;
    if (x_dtype < NVFP4_DT_BF16 || x_dtype > NVFP4_DT_F32) return NVFP4_ERR_BAD_ENUM;
    if (m < 0 || n < 0 || (n % kBlock) != 0 || (padded_n % kBlock) != 0 || padded_n < n) return NVFP4_ERR_BAD_SHAPE;
    if (upper < lower || upper - lower + 1 > 64) return NVFP4_ERR_BAD_RANGE;
    if (!(fp8_max > 0.0f)) return NVFP4_ERR_BAD_RANGE;
    QuantParams p;
    p.m = m;
    p.n = n;
    p.bin = n / kBlock;
    p.bout = padded_n / kBlock;
    p.k_pad = round_up_i64(p.bout, 4);
    p.swizzled = swizzled ? 1 : 0;
    p.width = swizzled ? p.k_pad : p.bout;
    p.rows = swizzled ? round_up_i64(m, 128) : m;
    p.total = p.rows * p.width;
    if (p.total == 0 || m * n == 0) return NVFP4_ERR_BAD_SHAPE;   // an empty tensor has no maximum
    if (!gs_out || !scratch || !codes || !scales || !x) return NVFP4_ERR_NULL_POINTER;
    if (variant == NVFP4_VARIANT_WEIGHTED && !importance) return NVFP4_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(codes) & 7) ||
        (reinterpret_cast<uintptr_t>(gs_out) & 3) || (reinterpret_cast<uintptr_t>(scratch) & 3))
        return NVFP4_ERR_MISALIGNED;
    if (swizzled && (reinterpret_cast<uintptr_t>(scales) & 3)) return NVFP4_ERR_MISALIGNED;
    if (!swizzled && (p.width & 3) == 0 && (reinterpret_cast<uintptr_t>(scales) & 3)) return NVFP4_ERR_MISALIGNED;
    if (variant == NVFP4_VARIANT_WEIGHTED && (reinterpret_cast<uintptr_t>(importance) & 15)) return NVFP4_ERR_MISALIGNED;
    p.x = x;
    p.importance = importance;
    p.gs_inv = nullptr;
    p.codes = codes;
    p.scales = scales;
    p.lower = lower;
    p.ncand = upper - lower + 1;
    p.fp8_max = fp8_max;
    p.gs_out = gs_out;
    p.fused_scratch = scratch;
    int dev = 0, sms = 0, coop = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (!coop) return NVFP4_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    bool too_large = false;
    cudaError_t err;
    switch (x_dtype) {
        case NVFP4_DT_BF16: err = launch_fused_variant<NVFP4_DT_BF16>(variant, p, sms, s, &too_large); break;
        case NVFP4_DT_F16: err = launch_fused_variant<NVFP4_DT_F16>(variant, p, sms, s, &too_large); break;
        default: err = launch_fused_variant<NVFP4_DT_F32>(variant, p, sms, s, &too_large); break;
    }
    if (too_large) return NVFP4_ERR_TOO_LARGE;
    return static_cast<int>(err);
}

extern "C" int nvfp4_quant_fused_last_status(void* stream, uint32_t* status_host) {
    if (!status_host) return NVFP4_ERR_NULL_POINTER;
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaMemcpyFromSymbol(status_host, nvfp4::g_quant_status, sizeof(uint32_t));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (*status_host != 0) {
        const uint32_t zero = 0;
        e = cudaMemcpyToSymbol(nvfp4::g_quant_status, &zero, sizeof(uint32_t));
    }
    return static_cast<int>(e);
}

extern "C" int nvfp4_quant_launch(int variant, const void* x, int x_dtype, const float* importance,
                                  const float* gs_inv, uint8_t* codes, uint8_t* scales, int64_t m, int64_t n,
                                  int64_t padded_n, int lower, int upper, int swizzled, void* stream) {
    return nvfp4_quant_launch_impl(0, variant, x, x_dtype, importance, gs_inv, codes, scales, m, n, padded_n, lower,
                                   upper, swizzled, stream);
}

// Testing hook: the limit (nanoseconds, 1 us .. 10 s) of the fused kernel's grid-wide wait on the current device;
// 0 restores the default of 2 s.  Synchronous.
extern "C" int nvfp4_quant_fused_set_wait_limit_ns(uint64_t ns) {
    if (ns == 0) ns = nvfp4::kFusedWaitLimitNs;
    if (ns < 1000ull || ns > 10000000000ull) return NVFP4_ERR_BAD_RANGE;
    return static_cast<int>(cudaMemcpyToSymbol(nvfp4::g_fused_wait_limit_ns, &ns, sizeof(ns)));
}
