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
//
// Launches are programmatic dependent launches (see common.cuh): a kernel lets the one queued behind it be scheduled from its
// first instruction and itself waits before it touches anything an earlier kernel may have written; a prepared weight is a
// constant by contract and is streamed ahead of that wait.  nvfp4_gemm_launch_grouped multiplies one activation with several
// prepared weights in one launch of the decode-sized kernel.
//
// This file holds the C entry points and the kernel choice; the kernels live in gemm_tile.cuh (one CTA per tile),
// gemm_pair.cuh (CTA pairs, cta_group::2) and gemm_skinny.cuh (decode-sized batches, K ranges across a cluster),
// all on the PTX wrappers of tc_ptx.cuh.  One translation unit, so that there is one status word.
#include <cstdint>
#include <new>

#include "gemm_tile.cuh"
#include "gemm_pair.cuh"
#include "gemm_skinny.cuh"
#include "gemm_peak.cuh"

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

// Testing hook: 0 = launch the library's kernels (GEMM, quantizer, global scale) without the programmatic-dependent-launch
// attribute, 1 = with (default).
extern "C" int nvfp4_gemm_tune_pdl(int enabled) {
    nvfp4::g_dependent_launch = enabled ? 1 : 0;
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
// sets its K ranges per weight tile; larger M falls back to the choice by shape), 6 = 128x64 tiles,
// 7 = CTA-pair 256x128 tiles.
extern "C" int nvfp4_gemm_force_path(int path) {
    if (path < 0 || path > 7) return NVFP4_ERR_BAD_ENUM;
    g_gemm_force_path = path;
    return NVFP4_OK;
}

// Measured kernel choice (generated file, see its first lines): {M, N, K, path} for a grid of shapes on a 148-SM B200.
struct PlanRow {
    int M, N, K, path;
};
static const PlanRow kPlanTable[] = {
#include "gemm_plan_table.inc"
};
// Fastest measured kernel for (N, K) at the smallest tabulated M >= the launch's M; 0 when the shape is not tabulated.
static int table_path(int64_t M, int64_t N, int64_t K) {
    int64_t best_m = INT64_MAX;
    int path = 0;
    for (const PlanRow& r : kPlanTable)
        if (r.N == N && r.K == K && r.M >= M && r.M < best_m) {
            best_m = r.M;
            path = r.path;
        }
    return path;
}

// Kernel choice for one shape: host arithmetic only.  *path: 1 = 128x128 tiles, 2 = 128x256, 3 = pair 256x256,
// 4 = pair 256x192, 5 = skinny, 6 = 128x64, 7 = pair 256x128; *k_ranges: cluster size of the skinny kernel (1 for the others).
static void plan_gemm(int64_t M, int64_t N, int64_t K, int sms, int k_splits, int* path_out, int* ranges_out) {
    const int k_tiles_total = static_cast<int>((K + 255) / 256);
    const int n_tiles = static_cast<int>((N + 127) / 128);
    *ranges_out = 1;
    // Decode-sized batches: weight rows on the MMA's 128 rows, tokens on its N dimension, K ranges across a cluster.
    // Measured on B200 with the weights streaming from HBM: faster than every other kernel up to 32 tokens; from 33
    // to 128 tokens only where few weight tiles meet a long K (at least 4 K ranges of at least 12 stages each, e.g.
    // 64 x 4096 x 14336: 13.2 us against 19.4 us), because its epilogue grows with the token tile.
    bool skinny = false;
    if (g_gemm_force_path == 5) {
        skinny = M <= kSkinnyMaxM;
    } else if (g_gemm_force_path == 0 && g_gemm_force_splits == 0 && M <= kSkinnyMaxM) {
        const int ranks = nvfp4::gemm::skinny::choose_ranks(n_tiles, k_tiles_total, sms, 0, M <= 64 ? 64 : 128);
        // measured with the weights streaming from HBM (microseconds, decode-sized kernel against the best tile / pair
        // kernel): 48 x 4096 x 4096 6.5 / 7.3, 48 x 6144 x 4096 7.6 / 8.8, 48 x 8192 x 8192 11.7 / 12.1, but 48 x 28672 x
        // 8192 33.9 / 27.4; 64 x 1024 x 4096 5.0 / 6.3, 64 x 6144 x 4096 8.1 / 7.7
        skinny = M <= kSkinnyAutoM || (M <= 48 && n_tiles <= 64) || (M <= 64 && n_tiles <= 8) ||
                 (ranks >= 4 && k_tiles_total / ranks >= 12);
    }
    if (skinny) {
        const int forced = g_gemm_force_path == 5 ? g_gemm_force_splits : 0;
        const int bt = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
        int ranks = nvfp4::gemm::skinny::choose_ranks(n_tiles, k_tiles_total, sms, forced, bt);
        const int per = (k_tiles_total + ranks - 1) / ranks;
        ranks = (k_tiles_total + per - 1) / per;   // no empty range
        *path_out = 5;
        *ranges_out = ranks;
        return;
    }
    // Kernel choice by a small cost model fitted to measurements on B200: time ~ waves x cost of one tile, where a
    // wave is one single-CTA tile per SM or one CTA-pair tile per two SMs (148 / 74 on a B200).  Relative tile costs: 128x64 -> 0.45, 128x128 -> 0.7, 128x256 -> 1.0,
    // pair 256x192 -> 0.68 (0.75 of the MMA work per SM, and its epilogue overlaps the next tile), pair 256x256 -> 0.96,
    // pair 256x128 -> 0.6.
    int path = g_gemm_force_path == 5 ? 0 : g_gemm_force_path;   // 0 = choose by shape
    // shapes of the measured table (on the GPU it was measured on) take the kernel that was fastest there
    if (path == 0 && k_splits == 1 && sms == 148) path = table_path(M, N, K);
    if (path == 0) {
        const int64_t mt = (M + 127) / 128;
        const int64_t wave1 = sms, wave2 = sms / 2 > 0 ? sms / 2 : 1;   // tiles per wave: single CTAs, CTA pairs
        const double c1 = static_cast<double>((mt * ((N + 127) / 128) + wave1 - 1) / wave1) * 0.7;
        const double c2 = static_cast<double>((mt * ((N + 255) / 256) + wave1 - 1) / wave1) * 1.0;
        const double c4 = static_cast<double>((((M + 255) / 256) * ((N + 191) / 192) + wave2 - 1) / wave2) * 0.68;
        path = (c1 <= c2) ? 1 : 2;
        double best = c1 <= c2 ? c1 : c2;
        // the pair kernels need a clear margin: at equal wave counts the single-CTA kernels put more CTAs on the
        // weight stream (512 x 4096 x 4096: 128x128 tiles 9.8 us, pair 256x192 10.5 us)
        // ... while per K stage the pair is cheaper, so from ~26 stages on it wins again (512 x 4096 x 14336: 19.8 / 21.7 us)
        const double margin = k_tiles_total >= 26 ? 0.0 : 0.03;
        if (M > 128 && N > 128 && k_splits == 1 && c4 < best - margin) {
            path = 4;
            best = c4;
        }
        // pair 256x256: 0.96 per wave of 74 pairs; wins where it needs fewer waves than the others (1024 x 4096 x
        // 14336: 25.4 us against 28.1 us with 128x256 tiles)
        const double c3 = static_cast<double>((((M + 255) / 256) * ((N + 255) / 256) + wave2 - 1) / wave2) * 0.96;
        if (M > 128 && N > 128 && k_splits == 1 && c3 < best) {
            path = 3;
            best = c3;
        }
        // pair 256x128: 0.6 per wave; the kernel for a few hundred tokens (256 x 8192 x 8192: 13.4 us against 14.8 us
        // with 128x128 tiles): as many CTAs as those, each loading only half of its tile's weight rows
        const double c7 = static_cast<double>((((M + 255) / 256) * ((N + 127) / 128) + wave2 - 1) / wave2) * 0.6;
        // (with one token tile the second CTA of a pair has no rows, yet from ~20 K stages on sharing the weight
        // rows still wins: 64 x 8192 x 8192 12.6 us against 13.3 us with 128x64 tiles)
        if ((M > 128 || k_tiles_total >= 20) && N > 128 && k_splits == 1 && c7 < best) {
            path = 7;
            best = c7;
        }
        // few tiles (one or two token tiles): 64 weight rows per CTA put twice as many SMs on the weight stream; every
        // CTA re-reads the token tile, which costs per K stage, so from ~20 stages on it is rated 1.4x
        // (256 x 4096 x 14336: 20.0 us against 16.6 us with pair 256x128)
        const double c6 = static_cast<double>((mt * ((N + 63) / 64) + wave1 - 1) / wave1) * 0.45 * (k_tiles_total >= 20 ? 1.4 : 1.0);
        if (mt <= 2 && c6 < best) path = 6;
    }
    if (k_splits > 1 && path != 1 && path != 2 && path != 6) path = 1;
    *path_out = path;
}

// Testing hook: the kernel nvfp4_gemm_launch would pick for this shape on a GPU with `sms` SMs (under the current
// force / tune settings).  No GPU is touched.
extern "C" int nvfp4_gemm_plan(int64_t M, int64_t N, int64_t K, int sms, int* path, int* k_ranges) {
    if (!path || !k_ranges) return NVFP4_ERR_NULL_POINTER;
    if (M <= 0 || N <= 0 || K <= 0 || (K % 64) != 0 || sms <= 0) return NVFP4_ERR_BAD_SHAPE;
    plan_gemm(M, N, K, sms, choose_k_splits(M, N, K), path, k_ranges);
    return NVFP4_OK;
}

static int gemm_launch_impl(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                            const float* alpha, void* out_bf16, int64_t M, int64_t N, int64_t K, void* workspace,
                            size_t workspace_bytes, void* stream, const nvfp4::gemm::WeightHandle* wh,
                            const float* alpha2 = nullptr) {
    using namespace nvfp4;
    if (M < 0 || N < 0 || K < 0 || (K % 64) != 0) return NVFP4_ERR_BAD_SHAPE;
    if (M == 0 || N == 0) return NVFP4_OK;
    if (M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL) return NVFP4_ERR_TOO_LARGE;
    if (!a || !b || !sfa || !sfb || !alpha || !out_bf16) return NVFP4_ERR_NULL_POINTER;
    if (K == 0) return NVFP4_ERR_BAD_SHAPE;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) ||
        (reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15) ||
        (reinterpret_cast<uintptr_t>(out_bf16) & 15) || (reinterpret_cast<uintptr_t>(alpha) & 3) ||
        (reinterpret_cast<uintptr_t>(alpha2) & 3))
        return NVFP4_ERR_MISALIGNED;
    gemm::GemmParams p;
    p.sfa = sfa;
    p.sfb = sfb;
    p.alpha = alpha;
    p.alpha2 = alpha2;
    p.weights_ready = wh ? 1 : 0;
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
    const int sms = gemm::device_info().sms;
    int path = 0, ranges = 1;
    plan_gemm(M, N, K, sms, p.k_splits, &path, &ranges);
    if (path == 5) {
        const int forced = g_gemm_force_path == 5 ? g_gemm_force_splits : 0;
        if (M <= 16) return gemm::skinny::launch_skinny<16>(a, b, p, forced, s, wh);
        if (M <= 32) return gemm::skinny::launch_skinny<32>(a, b, p, forced, s, wh);
        if (M <= 64) return gemm::skinny::launch_skinny<64>(a, b, p, forced, s, wh);
        return gemm::skinny::launch_skinny<128>(a, b, p, forced, s, wh);
    }
    if (p.k_splits > 1) {
        const size_t need = static_cast<size_t>(p.k_splits) * static_cast<size_t>(M) * static_cast<size_t>(N) * sizeof(float);
        if (!workspace || workspace_bytes < need) return NVFP4_ERR_WORKSPACE;
        if (reinterpret_cast<uintptr_t>(workspace) & 15) return NVFP4_ERR_MISALIGNED;
    }
    if (path == 3) return gemm::pair::launch_pair<256>(a, b, p, s, wh);
    if (path == 4) return gemm::pair::launch_pair<192>(a, b, p, s, wh);
    if (path == 7) return gemm::pair::launch_pair<128>(a, b, p, s, wh);
    if (path == 2) return gemm::launch<256>(a, b, p, s, wh);
    if (path == 6) return gemm::launch<64>(a, b, p, s, wh);
    return gemm::launch<128>(a, b, p, s, wh);
}

extern "C" int nvfp4_gemm_launch(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                                 const float* alpha, void* out_bf16, int64_t M, int64_t N, int64_t K, void* workspace,
                                 size_t workspace_bytes, void* stream) {
    return gemm_launch_impl(a, b, sfa, sfb, alpha, out_bf16, M, N, K, workspace, workspace_bytes, stream, nullptr);
}

// A weight matrix used by many GEMM calls (a model's linear layer): its tensor maps are encoded once here instead
// of on every launch.  The handle is a small host object; it refers to `b` / `sfb`, which the caller keeps alive and
// unchanged in place (their contents may change, their addresses and shape may not) until nvfp4_gemm_release.
extern "C" int nvfp4_gemm_prepare(const uint8_t* b, const uint8_t* sfb, int64_t N, int64_t K, void** handle_out) {
    using namespace nvfp4;
    if (!handle_out) return NVFP4_ERR_NULL_POINTER;
    *handle_out = nullptr;
    if (N <= 0 || K <= 0 || (K % 64) != 0) return NVFP4_ERR_BAD_SHAPE;
    if (N > 0x7fffff00LL || K > 0x7fffff00LL) return NVFP4_ERR_TOO_LARGE;
    if (!b || !sfb) return NVFP4_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(b) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15)) return NVFP4_ERR_MISALIGNED;
    gemm::WeightHandle* h = new (std::nothrow) gemm::WeightHandle();
    if (!h) return NVFP4_ERR_UNSUPPORTED;
    h->magic = gemm::kWeightMagic;
    h->device = gemm::device_info().device;
    h->b = b;
    h->sfb = sfb;
    h->N = N;
    h->K = K;
    int st = gemm::make_operand_map(&h->rows64, b, N, K / 2, 64);
    if (st == NVFP4_OK) st = gemm::make_operand_map(&h->rows96, b, N, K / 2, 96);
    if (st == NVFP4_OK) st = gemm::make_operand_map(&h->rows128, b, N, K / 2, 128);
    if (st == NVFP4_OK) st = gemm::make_operand_map(&h->rows256, b, N, K / 2, 256);
    if (st == NVFP4_OK)
        st = gemm::pair::make_scale_map(&h->scales, sfb, (N + 127) / 128, round_up_i64(K / 16, 4) * 128);
    if (st != NVFP4_OK) {
        delete h;
        return st;
    }
    *handle_out = h;
    return NVFP4_OK;
}

extern "C" int nvfp4_gemm_release(void* handle) {
    auto* h = static_cast<nvfp4::gemm::WeightHandle*>(handle);
    if (!h) return NVFP4_OK;
    if (h->magic != nvfp4::gemm::kWeightMagic) return NVFP4_ERR_BAD_ENUM;
    h->magic = 0;
    delete h;
    return NVFP4_OK;
}

// out[M, N] = alpha * dq(a) dq(weight)^T with a prepared weight: the same kernels and bits as nvfp4_gemm_launch.
extern "C" int nvfp4_gemm_launch_prepared(void* handle, const uint8_t* a, const uint8_t* sfa, const float* alpha,
                                          void* out_bf16, int64_t M, void* workspace, size_t workspace_bytes, void* stream) {
    auto* h = static_cast<const nvfp4::gemm::WeightHandle*>(handle);
    if (!h) return NVFP4_ERR_NULL_POINTER;
    if (h->magic != nvfp4::gemm::kWeightMagic) return NVFP4_ERR_BAD_ENUM;
    if (h->device != nvfp4::gemm::device_info().device) return NVFP4_ERR_UNSUPPORTED;   // prepared on another device
    return gemm_launch_impl(a, h->b, sfa, h->sfb, alpha, out_bf16, M, h->N, h->K, workspace, workspace_bytes, stream, h);
}

// One activation against several prepared weights of equal K, e.g. a layer's q / k / v projections:
//   outs[i][M, N_i] = alpha_w[i][0] * alpha_a[0] * dq(a) dq(weight_i)^T      (alpha_a may be NULL: factor 1)
// Decode-sized batches on shapes the decode-sized kernel is chosen for go out as ONE launch per 8 weights; everything
// else as one launch per weight.  Each output has the bits nvfp4_gemm_launch_prepared gives for the same weight with
// alpha = alpha_w[i][0] * alpha_a[0] whenever the K ranges per tile agree (they are chosen from the group's total tile count).
extern "C" int nvfp4_gemm_launch_grouped(void* const* handles, int n_weights, const uint8_t* a, const uint8_t* sfa,
                                         const float* alpha_a, const float* const* alpha_w, void* const* outs_bf16,
                                         int64_t M, void* stream) {
    using namespace nvfp4;
    if (n_weights < 0 || n_weights > 64) return NVFP4_ERR_BAD_RANGE;
    if (n_weights == 0) return NVFP4_OK;
    if (!handles || !alpha_w || !outs_bf16) return NVFP4_ERR_NULL_POINTER;
    if (M < 0) return NVFP4_ERR_BAD_SHAPE;
    const int device = gemm::device_info().device;
    int64_t K = 0, n_total = 0;
    for (int i = 0; i < n_weights; ++i) {
        auto* h = static_cast<const gemm::WeightHandle*>(handles[i]);
        if (!h || !alpha_w[i] || !outs_bf16[i]) return NVFP4_ERR_NULL_POINTER;
        if (h->magic != gemm::kWeightMagic) return NVFP4_ERR_BAD_ENUM;
        if (h->device != device) return NVFP4_ERR_UNSUPPORTED;
        if (i == 0) K = h->K;
        else if (h->K != K) return NVFP4_ERR_BAD_SHAPE;
        if ((reinterpret_cast<uintptr_t>(outs_bf16[i]) & 15) || (reinterpret_cast<uintptr_t>(alpha_w[i]) & 3))
            return NVFP4_ERR_MISALIGNED;
        n_total += (h->N + 127) / 128 * 128;
    }
    if (M == 0) return NVFP4_OK;
    if (!a || !sfa) return NVFP4_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(sfa) & 15) ||
        (reinterpret_cast<uintptr_t>(alpha_a) & 3))
        return NVFP4_ERR_MISALIGNED;
    if (M > 0x7fffff00LL || n_total > 0x7fffff00LL) return NVFP4_ERR_TOO_LARGE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int path = 0, ranges = 1;
    if (n_weights > 1) {
        plan_gemm(M, n_total, K, gemm::device_info().sms, choose_k_splits(M, n_total, K), &path, &ranges);
        // One launch for the group beats one tile-kernel launch per weight up to 64 tokens (Llama-3-8B-shaped stack, 32
        // layers, ms: 48 tokens 1.75 against 1.89, 64 tokens 1.81 against 1.84; 96 tokens 2.05 against 1.95).
        if (M <= 64 && g_gemm_force_path == 0 && g_gemm_force_splits == 0) path = 5;
    }
    if (path == 5) {
        const int forced = g_gemm_force_path == 5 ? g_gemm_force_splits : 0;
        const int64_t stride = round_up_i64(K / 16, 4) * 128;
        for (int first = 0; first < n_weights; first += gemm::skinny::kMaxGroup) {
            const int n = n_weights - first < gemm::skinny::kMaxGroup ? n_weights - first : gemm::skinny::kMaxGroup;
            gemm::skinny::SkinnyItem items[gemm::skinny::kMaxGroup];
            for (int i = 0; i < n; ++i) {
                auto* h = static_cast<const gemm::WeightHandle*>(handles[first + i]);
                items[i].w = h->b;
                items[i].sfw = h->sfb;
                items[i].alpha = alpha_w[first + i];
                items[i].out = static_cast<__nv_bfloat16*>(outs_bf16[first + i]);
                items[i].N = h->N;
                items[i].wh = h;
            }
            const int m = static_cast<int>(M), k = static_cast<int>(K);
            int st;
            if (M <= 16) st = gemm::skinny::launch_skinny_group<16>(a, sfa, alpha_a, m, k, stride, items, n, forced, s);
            else if (M <= 32) st = gemm::skinny::launch_skinny_group<32>(a, sfa, alpha_a, m, k, stride, items, n, forced, s);
            else if (M <= 64) st = gemm::skinny::launch_skinny_group<64>(a, sfa, alpha_a, m, k, stride, items, n, forced, s);
            else st = gemm::skinny::launch_skinny_group<128>(a, sfa, alpha_a, m, k, stride, items, n, forced, s);
            if (st != NVFP4_OK) return st;
        }
        return NVFP4_OK;
    }
    for (int i = 0; i < n_weights; ++i) {
        auto* h = static_cast<const gemm::WeightHandle*>(handles[i]);
        const int st = gemm_launch_impl(a, h->b, sfa, h->sfb, alpha_w[i], outs_bf16[i], M, h->N, h->K, nullptr, 0, stream, h,
                                        alpha_a);
        if (st != NVFP4_OK) return st;
    }
    return NVFP4_OK;
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


// Tensor-pipe rate probe: `stages` x 4 block-scaled FP4 MMAs per SM on operands resident in shared memory; time the
// launch with events on `stream`.  pair == 0: one CTA per SM, M = 128, N = 256, K = 64 per instruction; pair != 0:
// a CTA pair (cta_group::2) per two SMs, M = 256, N = 256, K = 64 per instruction -- the form the large-shape
// kernels use; pair == 2 (testing hook): the pair == 0 kernel with its last tcgen05.commit left out, so that its
// final wait ends at the wait limit and the status word is set (nothing faults, TMEM is freed).  Work done either way: *sms_out * stages * 4 * 2 * 128 * 256 * 64 flop (*sms_out = SMs used).
// Bounded: stages <= 1 << 20.
extern "C" int nvfp4_gemm_peak_probe(int stages, int pair_mode, int* sms_out, void* stream) {
    using namespace nvfp4::gemm;
    if (stages <= 0 || stages > (1 << 20)) return NVFP4_ERR_BAD_RANGE;
    if (pair_mode < 0 || pair_mode > 2) return NVFP4_ERR_BAD_ENUM;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (pair_mode != 1) {
        e = cudaFuncSetAttribute(peak::fp4_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmDynSmemBytes);
        if (e != cudaSuccess) return static_cast<int>(e);
        if (sms_out) *sms_out = sms;
        // whole SM: it takes all TMEM columns
        peak::fp4_peak_kernel<<<sms, peak::kPeakThreads, kGemmDynSmemBytes, s>>>(stages, pair_mode == 2 ? 1 : 0);
        return static_cast<int>(cudaGetLastError());
    }
    e = cudaFuncSetAttribute(peak::fp4_peak_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmDynSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    const int ctas = sms / 2 * 2;
    if (sms_out) *sms_out = ctas;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas, 1, 1);
    cfg.blockDim = dim3(peak::kPeakThreads, 1, 1);
    cfg.dynamicSmemBytes = kGemmDynSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, peak::fp4_peak_pair_kernel, stages));
}

// Testing hook: the limit (nanoseconds, 1 us .. 10 s) after which a wait inside the GEMM kernels of the current device
// gives up and records a status word; 0 restores the default of 2 s.  Synchronous (it copies to a device symbol).
extern "C" int nvfp4_gemm_set_wait_limit_ns(uint64_t ns) {
    if (ns == 0) ns = nvfp4::gemm::kWaitLimitNs;
    if (ns < 1000ull || ns > 10000000000ull) return NVFP4_ERR_BAD_RANGE;
    return static_cast<int>(cudaMemcpyToSymbol(nvfp4::gemm::g_gemm_wait_limit_ns, &ns, sizeof(ns)));
}

#ifdef NVFP4_GEMM_TRACE
// Debugging builds only: device buffer of 64 counters the kernels add their progress marks to (NULL = off).
extern "C" int nvfp4_gemm_set_trace(uint32_t* counters) {
    return static_cast<int>(cudaMemcpyToSymbol(nvfp4::gemm::g_gemm_trace, &counters, sizeof(counters)));
}
#endif
