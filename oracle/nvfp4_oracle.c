/*
 * CPU oracle for NVFP4 ScaleSweep quantization and the NVFP4 block-scaled GEMM.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * the reference's device kernels so that the CUDA product path can be compared
 * with it bit for bit.  Nothing in the product package links or calls it; only
 * the test-suite, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Reference locations restated here (paths inside efsotr/nvfp4quant_test):
 *   kernels/kernel_ScaleSweep_MSE.py:271-377   unweighted sweep kernel
 *   kernels/kernel_ScaleSweep_MSE.py:83-188    pair error, serial FMA chain, *(s*s)
 *   kernels/kernel_ScaleSweep_MSE.py:37-80     final E2M1 pack
 *   kernels/kernel_ScaleSweep_MSE.py:15-34     128x4 swizzled scale offset
 *   kernels/kernel_ScaleSweep.py:84-171        weighted pair error, fixed tree sum
 *   kernels/kernel_ScaleSweep.py:290-416       weighted sweep kernel (floor base)
 *   kernels/kernel_vllm.py:29-70               swizzle / unswizzle of scales
 *   helper.py:117-147                          E2M1 LUT, dequantize_base
 * Third party (vllm 0.22.0, not vendored by the reference): the amax quantizer
 * `scaled_fp4_quant` and the GEMM `cutlass_scaled_fp4_mm` (call sites
 * bench.py:118-125, README.md:68).  Their arithmetic is restated from the
 * published NVFP4 recipe: sf = e4m3(gs_inv * amax/6), x * 1/(sf * 1/gs_inv).
 *
 * Parity pins: (1) the 37 known-answer vectors of proof/nvfp4_bound_example.py
 * (sweep result == exhaustive optimum); (2) fixtures under tests/golden/ that
 * were produced by running the reference's own Triton kernels on a B200;
 * (3) the swizzle permutation of kernels/kernel_vllm.py.
 *
 * Numerics: fp32 throughout, single-rounding fmaf, no contraction (build with
 * -ffp-contract=off), denormals kept.  `1/scale` is the GPU's `div.full.f32`,
 * which is not IEEE division: only 126 denominators occur, so their results
 * are tabulated (div_full_table.h, captured from a B200).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <stdlib.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "div_full_table.h"

#define VARIANT_MSE 0
#define VARIANT_WEIGHTED 1
#define VARIANT_AMAX 2

#define DT_BF16 0
#define DT_F16 1
#define DT_F32 2

static inline float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ff;
    if (exp == 0) {
        if (man == 0) return bits_to_f32(sign);
        float v = (float)man * 0x1p-24f;
        return sign ? -v : v;
    }
    if (exp == 31) return bits_to_f32(sign | 0x7f800000u | (man << 13));
    return bits_to_f32(sign | ((exp + 112) << 23) | (man << 13));
}

static inline float load_elem(const void* x, int dtype, int64_t idx) {
    if (dtype == DT_BF16) return bits_to_f32((uint32_t)((const uint16_t*)x)[idx] << 16);
    if (dtype == DT_F16) return f16_to_f32(((const uint16_t*)x)[idx]);
    return ((const float*)x)[idx];
}

/* E4M3 (finite-only "fn" flavour): value of a raw byte. */
float nvfp4_oracle_e4m3_to_f32(uint8_t b) {
    int exp = (b >> 3) & 15, man = b & 7;
    float v;
    if (exp == 0) v = (float)man * 0x1p-9f;
    else if (exp == 15 && man == 7) v = NAN;
    else v = ldexpf(1.0f + (float)man * 0.125f, exp - 7);
    return (b & 0x80) ? -v : v;
}

/* fp32 -> E4M3, round-to-nearest-even, saturating to +-448, NaN -> 0x7f.
 * (kernels/kernel_ScaleSweep_MSE.py:321: `.to(tl.float8e4nv)`, which lowers to
 * cvt.rn.satfinite.e4m3x2.f32 on Blackwell.) */
uint8_t nvfp4_oracle_f32_to_e4m3(float x) {
    uint8_t sign = signbit(x) ? 0x80 : 0;
    float a = fabsf(x);
    if (isnan(a)) return 0x7f;
    if (a >= 448.0f) return sign | 0x7e;
    if (a < 0x1p-6f) {
        int q = (int)nearbyintf(a * 512.0f); /* exact product, RNE */
        return sign | (uint8_t)q;            /* q == 8 is the smallest normal */
    }
    int e;
    float m = frexpf(a, &e); /* a = m * 2^e, m in [0.5,1) */
    m *= 2.0f; e -= 1;       /* m in [1,2) */
    int q = (int)nearbyintf((m - 1.0f) * 8.0f);
    if (q == 8) { q = 0; e += 1; }
    int bits = ((e + 7) << 3) | q;
    if (bits > 0x7e) bits = 0x7e;
    return sign | (uint8_t)bits;
}

static const float E2M1_VALUE[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* fp32 -> E2M1 nibble: RNE on {0,.5,1,1.5,2,3,4,6}, saturating, sign kept on
 * zero, NaN -> +6 (cvt.rn.satfinite.e2m1x2.f32). */
static inline uint8_t f32_to_e2m1(float x) {
    if (isnan(x)) return 0x7;
    uint8_t sign = signbit(x) ? 0x8 : 0;
    float a = fabsf(x);
    uint8_t c;
    if (a <= 0.25f) c = 0;
    else if (a < 0.75f) c = 1;
    else if (a <= 1.25f) c = 2;
    else if (a < 1.75f) c = 3;
    else if (a <= 2.5f) c = 4;
    else if (a < 3.5f) c = 5;
    else if (a <= 5.0f) c = 6;
    else c = 7;
    return sign | c;
}

static inline float e2m1_to_f32(uint8_t nib) {
    float v = E2M1_VALUE[nib & 7];
    return (nib & 8) ? -v : v;
}

/* 1/s as the GPU computes it: div.full.f32 1.0, e4m3(raw). raw 0 -> +inf. */
static inline float inv_scale_of_raw(int raw) {
    if (raw <= 0) return INFINITY;
    return bits_to_f32(NVFP4_DIV_FULL_RCP_BITS[raw]);
}

int64_t nvfp4_oracle_swizzled_offset(int64_t row, int64_t col, int64_t k_pad) {
    return (row >> 7) * (k_pad * 128) + (col >> 2) * 512 + (row & 31) * 16 +
           ((row & 127) >> 5) * 4 + (col & 3);
}

/* Unweighted block error for one candidate: quantize x_j = v_j*inv, serial FMA
 * chain over j = 0..15 in pair order, then *(s*s). */
__attribute__((target_clones("default", "avx2,fma")))
static float mse_error(const float v[16], float inv, float s) {
    float acc = 0.0f;
    for (int j = 0; j < 16; ++j) {
        float x = v[j] * inv;
        float d = e2m1_to_f32(f32_to_e2m1(x)) - x;
        acc = (j == 0) ? d * d : fmaf(d, d, acc);
    }
    return acc * (s * s);
}

__attribute__((target_clones("default", "avx2,fma")))
static float weighted_error(const float v[16], const float w[16], float inv, float s) {
    float e[8];
    for (int p = 0; p < 8; ++p) {
        float x0 = v[2 * p] * inv, x1 = v[2 * p + 1] * inv;
        float d0 = e2m1_to_f32(f32_to_e2m1(x0)) - x0;
        float d1 = e2m1_to_f32(f32_to_e2m1(x1)) - x1;
        float a = d0 * d0;
        float b = d1 * d1;
        a = a * w[2 * p];
        e[p] = fmaf(b, w[2 * p + 1], a);
    }
    float t = ((e[0] + e[1]) + (e[2] + e[3])) + ((e[4] + e[5]) + (e[6] + e[7]));
    return t * (s * s);
}

static void pack_block(const float v[16], float inv, uint8_t out[8]) {
    for (int j = 0; j < 8; ++j) {
        uint8_t lo = f32_to_e2m1(v[2 * j] * inv);
        uint8_t hi = f32_to_e2m1(v[2 * j + 1] * inv);
        out[j] = (uint8_t)((hi << 4) | lo);
    }
}

/* Sweep one block; returns the chosen raw E4M3 byte. */
static int sweep_block(int variant, const float v[16], const float* w, int lower, int upper) {
    float amax = 0.0f;
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
    float base_scale = amax * bits_to_f32(0x3E2AAAABu); /* fp32(1/6) */
    uint8_t base_fp8 = nvfp4_oracle_f32_to_e4m3(base_scale);
    int base_raw = base_fp8;
    if (variant == VARIANT_WEIGHTED && nvfp4_oracle_e4m3_to_f32(base_fp8) > base_scale) base_raw -= 1;
    float best = INFINITY;
    int best_raw = 0;
    for (int i = 0; i <= upper - lower; ++i) {
        int raw = base_raw + lower + i;
        if (raw < 1) raw = 1;
        if (raw > 126) raw = 126;
        float s = nvfp4_oracle_e4m3_to_f32((uint8_t)raw);
        float inv = inv_scale_of_raw(raw);
        float err = (variant == VARIANT_WEIGHTED) ? weighted_error(v, w, inv, s) : mse_error(v, inv, s);
        if (err < best) { best = err; best_raw = raw; }
    }
    return best_raw;
}

/*
 * Quantize x[m, n] into codes[m, padded_n/2] and block scales.
 *   scales: swizzled -> byte offset nvfp4_oracle_swizzled_offset(row, col, round_up(padded_n/16, 4))
 *           linear   -> row * (padded_n/16) + col
 * Only the logical region (m rows, padded_n/16 blocks) is written, like the
 * reference; the caller owns the padding bytes.
 * amax_out_scale_table: optional 127 floats, entry r = the GPU's
 *   rcp.approx.ftz(e4m3(r) * rcp.approx.ftz(gs_inv)); NULL -> IEEE division.
 * amax_sixth: the factor used for amax/6 by the amax variant (0 -> fp32(1/6)).
 * Returns 0, or -1 on bad arguments.
 */
int nvfp4_oracle_quant(int variant, const void* x, int x_dtype, const float* importance,
                       float gs_inv, uint8_t* codes, uint8_t* scales, int64_t m, int64_t n,
                       int64_t padded_n, int lower, int upper, int swizzled,
                       const float* amax_out_scale_table, float amax_sixth, int nthreads) {
    if (m < 0 || n < 0 || n % 16 || padded_n % 16 || padded_n < n) return -1;
    if (variant == VARIANT_WEIGHTED && !importance) return -1;
    if (variant != VARIANT_AMAX && upper < lower) return -1;
    const int64_t bin = n / 16, bout = padded_n / 16, k_pad = (bout + 3) / 4 * 4;
    if (amax_sixth == 0.0f) amax_sixth = bits_to_f32(0x3E2AAAABu);
#ifdef _OPENMP
    if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < m; ++row) {
        for (int64_t col = 0; col < bout; ++col) {
            float v[16], w[16];
            if (col < bin) {
                for (int j = 0; j < 16; ++j) v[j] = load_elem(x, x_dtype, row * n + col * 16 + j);
            } else {
                for (int j = 0; j < 16; ++j) v[j] = 0.0f;
            }
            uint8_t sbyte;
            float inv;
            if (variant == VARIANT_AMAX) {
                /* amax taken on the raw elements, as the vllm op does */
                float amax = 0.0f;
                for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
                float sf = gs_inv * (amax * amax_sixth);
                sbyte = nvfp4_oracle_f32_to_e4m3(sf);
                float sfv = nvfp4_oracle_e4m3_to_f32(sbyte);
                if (sfv == 0.0f) inv = 0.0f;
                else if (amax_out_scale_table) inv = amax_out_scale_table[sbyte & 0x7f];
                else inv = 1.0f / (sfv * (1.0f / gs_inv));
            } else {
                for (int j = 0; j < 16; ++j) {
                    v[j] = v[j] * gs_inv;
                    w[j] = (variant == VARIANT_WEIGHTED && col < bin) ? importance[col * 16 + j] : 0.0f;
                }
                int raw = sweep_block(variant, v, w, lower, upper);
                sbyte = (uint8_t)raw;
                inv = inv_scale_of_raw(raw);
            }
            pack_block(v, inv, codes + (row * bout + col) * 8);
            int64_t off = swizzled ? nvfp4_oracle_swizzled_offset(row, col, k_pad) : row * bout + col;
            scales[off] = sbyte;
        }
    }
    return 0;
}

/* Exhaustive search over all 126 positive finite scales (raw 1..126) with the
 * same fp32 error; used to check that the windowed sweep finds the optimum. */
int nvfp4_oracle_best_raw_exhaustive(const float v[16]) {
    float best = INFINITY;
    int best_raw = 0;
    for (int raw = 1; raw <= 126; ++raw) {
        float err = mse_error(v, inv_scale_of_raw(raw), nvfp4_oracle_e4m3_to_f32((uint8_t)raw));
        if (err < best) { best = err; best_raw = raw; }
    }
    return best_raw;
}

/* Sweep one fp32 block with gs_inv = 1 and return the raw scale byte. */
int nvfp4_oracle_sweep_block_f32(int variant, const float v[16], const float* w, int lower, int upper) {
    return sweep_block(variant, v, w, lower, upper);
}

/* deq[m, n] = LUT[nibble] * e4m3(scale) * gs  (helper.py:144-147). */
int nvfp4_oracle_dequant(const uint8_t* codes, const uint8_t* scales, float gs, float* out,
                         int64_t m, int64_t n, int swizzled) {
    if (n % 16) return -1;
    const int64_t b = n / 16, k_pad = (b + 3) / 4 * 4;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < m; ++row)
        for (int64_t col = 0; col < b; ++col) {
            int64_t off = swizzled ? nvfp4_oracle_swizzled_offset(row, col, k_pad) : row * b + col;
            float s = nvfp4_oracle_e4m3_to_f32(scales[off]);
            for (int j = 0; j < 8; ++j) {
                uint8_t byte = codes[(row * b + col) * 8 + j];
                out[row * n + col * 16 + 2 * j] = e2m1_to_f32(byte & 0xf) * s * gs;
                out[row * n + col * 16 + 2 * j + 1] = e2m1_to_f32(byte >> 4) * s * gs;
            }
        }
    return 0;
}

/*
 * out[M, N] = alpha * sum_k a[m,k] sfa[m,k/16] b[n,k] sfb[n,k/16], accumulated in
 * double (the products code*scale are exact in double).  a: [M, K/2], b: [N, K/2],
 * scales swizzled with k_pad = round_up(K/16, 4).  Result left in fp32 (the
 * caller rounds to bf16).
 */
int nvfp4_oracle_gemm(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                      float alpha, float* out, int64_t M, int64_t N, int64_t K) {
    if (K % 16) return -1;
    const int64_t kb = K / 16, k_pad = (kb + 3) / 4 * 4;
    float* da = (float*)malloc(sizeof(float) * (size_t)(M * K));
    float* db = (float*)malloc(sizeof(float) * (size_t)(N * K));
    if (!da || !db) { free(da); free(db); return -2; }
    nvfp4_oracle_dequant(a, sfa, 1.0f, da, M, K, 1);
    nvfp4_oracle_dequant(b, sfb, 1.0f, db, N, K, 1);
    (void)k_pad;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M; ++i)
        for (int64_t j = 0; j < N; ++j) {
            double acc = 0.0;
            const float* pa = da + i * K;
            const float* pb = db + j * K;
            for (int64_t k = 0; k < K; ++k) acc += (double)pa[k] * (double)pb[k];
            out[i * N + j] = (float)((double)alpha * acc);
        }
    free(da);
    free(db);
    return 0;
}

int nvfp4_oracle_div_full_table_is_measured(void) { return NVFP4_DIV_FULL_TABLE_MEASURED; }
uint32_t nvfp4_oracle_div_full_bits(int raw) { return NVFP4_DIV_FULL_RCP_BITS[raw & 127]; }

/*
 * For nblocks fp32 blocks (gs_inv = 1): hist[off + 64] += 1 where off = exhaustive optimum raw - base raw,
 * base = RNE_E4M3(amax/6).  Blocks whose base code is >= 120 (within reach of saturation) or < 16 (window touches
 * the subnormal codes, where scales are equally spaced and the claim does not apply) are counted in *skipped.
 * Supports the reference's claim (proof/proof.md) that for normal scales away from saturation a minimiser lies in
 * [base-3, base+7].
 */
void nvfp4_oracle_offset_histogram(const float* x, int64_t nblocks, int64_t hist[128], int64_t* skipped) {
    int64_t local_skipped = 0;
#pragma omp parallel
    {
        int64_t h[128];
        int64_t sk = 0;
        memset(h, 0, sizeof(h));
#pragma omp for schedule(static)
        for (int64_t b = 0; b < nblocks; ++b) {
            const float* v = x + b * 16;
            float amax = 0.0f;
            for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
            int base = nvfp4_oracle_f32_to_e4m3(amax * bits_to_f32(0x3E2AAAABu));
            if (amax == 0.0f || base >= 120 || base < 16) { ++sk; continue; }
            int best = nvfp4_oracle_best_raw_exhaustive(v);
            int off = best - base;
            if (off < -64) off = -64;
            if (off > 63) off = 63;
            ++h[off + 64];
        }
#pragma omp critical
        {
            for (int i = 0; i < 128; ++i) hist[i] += h[i];
            local_skipped += sk;
        }
    }
    *skipped = local_skipped;
}

/*
 * Pruning study for the unweighted sweep (kernels/kernel_ScaleSweep_MSE.py:326-346), in the kernel's own fp32
 * arithmetic.  For a candidate scale s whose grid cannot hold the block maximum (x = amax * (1/s) > 6), the block
 * error is at least the error of that one element: RN(RN(d*d) * RN(s*s)) with d = RN(6 - x).  The bound needs no
 * rounding margin: every other term of the serial FMA chain is >= 0 and round-to-nearest is monotone, so the
 * chain can only be larger.  A candidate whose bound is strictly above the least error among the non-saturating
 * candidates can neither win nor tie and may be skipped.
 *   surv_hist[k]      blocks that keep k candidates under that rule (k = 0..ncand)
 *   warp_hist[k]      groups of 32 consecutive blocks whose largest survivor count is k (the trip count of a warp
 *                     that holds one block per lane)
 *   pruned_by_off[i]  blocks in which candidate i (offset lower + i) was pruned
 *   prefix_elems[i]   sum over blocks of the elements of candidate i's chain that have to be accumulated before its
 *                     partial error exceeds the block's final minimum (16 for a winner): the work a branch-and-bound
 *                     over chain prefixes with perfect knowledge of the minimum would still do
 * Returns the number of blocks in which pruning would have changed the chosen scale (must be 0).
 */
int64_t nvfp4_oracle_prune_study(const float* x, int64_t nblocks, float gs_inv, int lower, int upper,
                                 int64_t* surv_hist, int64_t* warp_hist, int64_t* pruned_by_off, int64_t* prefix_elems) {
    const int nc = upper - lower + 1;
    if (nc < 1 || nc > 64) return -1;
    int64_t wrong = 0;
    int warp_max = 0;
    for (int64_t b = 0; b < nblocks; ++b) {
        float v[16];
        float amax = 0.0f;
        for (int j = 0; j < 16; ++j) {
            v[j] = x[b * 16 + j] * gs_inv;
            amax = fmaxf(amax, fabsf(v[j]));
        }
        int base = nvfp4_oracle_f32_to_e4m3(amax * bits_to_f32(0x3E2AAAABu));
        float err[64], bound[64];
        int raws[64];
        float best_ns = INFINITY;    /* least error among candidates that do not saturate the maximum */
        for (int i = 0; i < nc; ++i) {
            int raw = base + lower + i;
            if (raw < 1) raw = 1;
            if (raw > 126) raw = 126;
            raws[i] = raw;
            float s = nvfp4_oracle_e4m3_to_f32((uint8_t)raw), inv = inv_scale_of_raw(raw);
            err[i] = mse_error(v, inv, s);
            float xm = amax * inv;
            if (xm > 6.0f) {
                float d = 6.0f - xm;
                bound[i] = (d * d) * (s * s);
            } else {
                bound[i] = -1.0f;    /* not a saturating candidate: always evaluated */
                if (err[i] < best_ns) best_ns = err[i];
            }
        }
        /* reference result */
        float best = INFINITY;
        int best_raw = 0;
        for (int i = 0; i < nc; ++i)
            if (err[i] < best) { best = err[i]; best_raw = raws[i]; }
        /* pruned result: saturating candidates are looked at after the others, lowest raw wins ties */
        float pbest = INFINITY;
        int praw = 0, kept = 0;
        for (int i = 0; i < nc; ++i) {
            if (bound[i] >= 0.0f && bound[i] > best_ns) { ++pruned_by_off[i]; continue; }
            ++kept;
            if (err[i] < pbest || (err[i] == pbest && raws[i] < praw)) { pbest = err[i]; praw = raws[i]; }
        }
        if (praw != best_raw) ++wrong;
        ++surv_hist[kept];
        if (kept > warp_max) warp_max = kept;
        if ((b & 31) == 31 || b == nblocks - 1) { ++warp_hist[warp_max]; warp_max = 0; }
        for (int i = 0; i < nc; ++i) {
            float inv = inv_scale_of_raw(raws[i]), s = nvfp4_oracle_e4m3_to_f32((uint8_t)raws[i]);
            float acc = 0.0f;
            int j = 0;
            for (; j < 16; ++j) {
                float xx = v[j] * inv;
                float d = e2m1_to_f32(f32_to_e2m1(xx)) - xx;
                acc = (j == 0) ? d * d : fmaf(d, d, acc);
                if (acc * (s * s) > best) { ++j; break; }
            }
            prefix_elems[i] += j;
        }
    }
    return wrong;
}
