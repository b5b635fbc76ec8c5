/*
 * C ABI of libnvfp4_b200.so: NVFP4 ScaleSweep quantization and the NVFP4
 * block-scaled GEMM for NVIDIA B200 (sm_100a).
 *
 * Every pointer is a DEVICE pointer unless its name ends in `_host`.  Launches
 * are asynchronous on `stream` (a cudaStream_t passed as void*; NULL = the
 * legacy default stream).  Launch calls never synchronise the device, copy to the
 * host or allocate memory; the few calls that do synchronise (the *_last_status
 * readers and the set_wait_limit hooks) say so.  Return value: 0 = ok, < 0 =
 * NVFP4_ERR_* (nothing was launched), > 0 = a cudaError_t reported by the launch.
 *
 * The "replaces" notes name the interface of efsotr/nvfp4quant_test (paths
 * inside that project) or of vllm 0.22.0, which that project calls.
 */
#ifndef NVFP4_B200_H_
#define NVFP4_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    NVFP4_OK = 0,
    NVFP4_ERR_NULL_POINTER = -1,
    NVFP4_ERR_BAD_SHAPE = -2,    /* n or padded_n not a multiple of 16, padded_n < n, K % 64, ... */
    NVFP4_ERR_BAD_ENUM = -3,     /* unknown variant / dtype / implementation */
    NVFP4_ERR_MISALIGNED = -4,   /* a pointer is not aligned as documented */
    NVFP4_ERR_BAD_RANGE = -5,    /* upper < lower or more than 64 candidates */
    NVFP4_ERR_WORKSPACE = -6,    /* workspace too small */
    NVFP4_ERR_UNSUPPORTED = -7,
    NVFP4_ERR_TOO_LARGE = -8,
    NVFP4_ERR_STATIC_SCRATCH = -9 /* input needs more scratch than the library's built-in array holds */
};

enum { NVFP4_VARIANT_MSE = 0, NVFP4_VARIANT_WEIGHTED = 1, NVFP4_VARIANT_AMAX = 2 };
enum { NVFP4_DT_BF16 = 0, NVFP4_DT_F16 = 1, NVFP4_DT_F32 = 2 };

/*
 * Quantize x[m, n] (row-major, contiguous) to packed E2M1 codes and one E4M3
 * scale per 16 elements.
 *
 *   variant   MSE:      sweep raw E4M3 codes base+lower..base+upper around
 *                       base = RNE_E4M3(amax/6), pick the least fp32 squared error,
 *                       lowest raw code on ties.
 *                       replaces kernels/kernel_ScaleSweep_MSE.py:380-413
 *                       (scalesweep_mse_nvfp4_quant_out) and the Triton kernel :271-377.
 *             WEIGHTED: same with per-column weights importance[n] and a
 *                       floor-rounded base.
 *                       replaces kernels/kernel_ScaleSweep.py:436-480 and :290-416.
 *             AMAX:     scale = E4M3(gs_inv * amax/6), no sweep.
 *                       replaces vllm `_C::scaled_fp4_quant.out`
 *                       (vllm/_custom_ops.py:1600-1665; call site bench.py:118-125).
 *   x         16-byte aligned; x_dtype one of NVFP4_DT_*.
 *   importance  n floats (WEIGHTED only, else may be NULL).
 *   gs_inv    one float on the device: 1 / global_scale.
 *   codes     uint8 [m, padded_n/2], 8-byte aligned; byte j of a row holds
 *             element 2j in its low nibble, 2j+1 in its high nibble.
 *   scales    swizzled != 0: uint8 [round_up(m,128) * round_up(padded_n/16, 4)] in the
 *             128x4 tile order of the tcgen05 scale-factor layout
 *             (kernels/kernel_vllm.py:9-26); rows >= m and columns >= padded_n/16
 *             are written as 0.  4-byte aligned.
 *             swizzled == 0: uint8 [m, padded_n/16] row-major.
 *   padded_n  >= n, multiple of 16; columns n..padded_n quantize as zeros.
 *   lower, upper  candidate window (ignored by AMAX); the reference uses -3..7
 *             (MSE) and -8..7 (WEIGHTED).
 */
int nvfp4_quant_launch(int variant, const void* x, int x_dtype, const float* importance,
                       const float* gs_inv, uint8_t* codes, uint8_t* scales, int64_t m, int64_t n,
                       int64_t padded_n, int lower, int upper, int swizzled, void* stream);

/* Same, choosing the kernel body: 0 = default (9 for tensors of a few tokens, see there; else 5 when a quarter or more
 * of the scale layout's rows are padding, else 8 / 7 / 6 where they apply, else 3), 1 = scalar (one candidate at a time, the plainest transcription), 2 = one candidate per trip with
 * packed multiplies and the mixed-precision subtract, 3 = two candidates per trip sharing one f32x2 FMA chain,
 * 5 = 3 with warps that hold only padding rows skipping the sweep, 6 = 3 on a two-dimensional grid (row =
 * blockIdx.x, uniform over the CTA; taken by default when the row is a whole number of 256-block chunks wide,
 * otherwise 6 means 3), 7 = 6 with the reference's candidate count (11 unweighted, 16 weighted) compiled in and
 * the sweep unrolled (default for the unweighted sweep with the reference's window; other windows make it 6),
 * 8 = 7 without any validity predicate, for tensors in which every slot of the scale layout is a real block (m a
 * multiple of 128 in the tiled layout, padded_n == n, rows a whole number of 256-block chunks wide, the reference's
 * window); the default there, elsewhere 8 means the default; 9 = 3 in CTAs of 64 threads over the real rows' slots,
 * which spreads a tensor of a few tokens over four times as many SMs, plus a few CTAs that zero the padding rows of the
 * tiled scale layout (the default up to 32768 real blocks, e.g. 64 tokens x 8192; 24576 for the weighted sweep).
 * 4 is the fused form, which has its own entry point below.  All give identical bytes; exposed for testing and
 * timing. */
int nvfp4_quant_launch_impl(int impl, int variant, const void* x, int x_dtype, const float* importance,
                            const float* gs_inv, uint8_t* codes, uint8_t* scales, int64_t m, int64_t n,
                            int64_t padded_n, int lower, int upper, int swizzled, void* stream);

/*
 * out[0] = amax(|x|) / (6 * fp8_max), out[1] = 1 / out[0]  over numel elements.
 * replaces helper.py:96-100 (get_nvfp4_global_scale).
 * `scratch` = 2 uint32 that must be zero before the first call; the kernel
 * leaves them zero again, so one scratch serves any number of calls issued in
 * stream order.  Concurrent calls need separate scratch; so do launches recorded into different CUDA graphs that may be
 * replayed at the same time, even when they were captured on one stream (see nvfp4_stream_capture_id).
 */
int nvfp4_global_scale_launch(const void* x, int x_dtype, int64_t numel, float fp8_max, float* out,
                              uint32_t* scratch, void* stream);

/*
 * Global scale and ScaleSweep quantization in one launch: what get_nvfp4_global_scale (helper.py:96-100)
 * followed by scalesweep_*_quant_out (kernels/kernel_ScaleSweep_MSE.py:380-413, kernels/kernel_ScaleSweep.py:436-489)
 * compute, as the reference's bench chains them (bench.py:57-67), with identical bytes.  variant is
 * NVFP4_VARIANT_MSE or NVFP4_VARIANT_WEIGHTED; gs_out[0] = amax(|x|) / (6 * fp8_max), gs_out[1] = 1 / gs_out[0].
 * Every 16-element block stays in its thread's registers while the CTAs combine their maxima through
 * `scratch` and wait for one another (cooperative launch; the wait is bounded, see nvfp4_quant_fused_last_status),
 * so x crosses HBM once.  The tensor must fit the resident grid of the device (about 3 M elements on a B200):
 * otherwise NVFP4_ERR_TOO_LARGE is returned, nothing is launched, and the caller issues the two launches.
 * `scratch` = 4 uint32, zero before the first call; the kernel leaves them zero.  Calls that share a scratch
 * must be ordered on one stream.  (Testing hook: a non-zero scratch[3] makes CTA 0 withhold its arrival, so the
 * grid-wide wait runs into its limit and the status word is set.)
 */
int nvfp4_quant_fused_launch(int variant, const void* x, int x_dtype, const float* importance, float fp8_max,
                             float* gs_out, uint32_t* scratch, uint8_t* codes, uint8_t* scales, int64_t m, int64_t n,
                             int64_t padded_n, int lower, int upper, int swizzled, void* stream);
/*
 * The same two steps as two launches from ONE host call (global scale kernel, then the quantizer reading gs_out[1]):
 * for callers that pay per host call, e.g. an eager decode loop.  Any variant (amax included), any size; `scratch` = the
 * 2 zeroed uint32 of nvfp4_global_scale_launch.  Bytes and scales equal the two separate calls.
 */
int nvfp4_quant_chain_launch(int variant, const void* x, int x_dtype, const float* importance, float fp8_max,
                             float* gs_out, uint32_t* scratch, uint8_t* codes, uint8_t* scales, int64_t m, int64_t n,
                             int64_t padded_n, int lower, int upper, int swizzled, void* stream);
/* Synchronises `stream`; *status = 0, or 1 if a fused launch on this device gave up its grid-wide wait (its
 * outputs are then invalid and its scratch must be zeroed again).  Reading a non-zero status clears it. */
int nvfp4_quant_fused_last_status(void* stream, uint32_t* status);

/*
 * out[j] = sum_i x[i, j]^2 in fp32 for x[m, n] (n % 4 == 0, x 16-byte aligned): the per-input-channel squared
 * norm the reference uses as importance for the operand it multiplies with (README.md:11; the reference's
 * driver computes it with torch, no dedicated kernel).  Fixed summation order: reproducible run to run.
 */
int nvfp4_channel_sqnorm_launch(const void* x, int x_dtype, int64_t m, int64_t n, float* out, void* stream);
/* The same for a column slice of a wider batch: x points at the slice's first column, `ld` (>= n, % 4 == 0) is the
 * row pitch in elements.  Columns are independent and each sum runs over the rows in the same fixed order, so the
 * slices of several GPUs concatenate to the bits one GPU computes for the whole batch (multi-GPU weight quantization
 * shards the importance reduction this way; no counterpart in the reference, which runs on one GPU). */
int nvfp4_channel_sqnorm_launch_strided(const void* x, int x_dtype, int64_t m, int64_t n, int64_t ld, float* out,
                                        void* stream);

/*
 * The same result as nvfp4_global_scale_launch for callers that cannot allocate device memory
 * (this entry point has no counterpart in the reference).  Typical callers: a plugin that only
 * receives raw device pointers from a runtime which owns all allocations, a serving process whose
 * memory pool is frozen, code running where cudaMalloc is not permitted.  The block-level partial
 * maxima live in an array compiled into the library (16.25 KiB per GPU, held until process exit)
 * instead of caller-provided scratch, and the call performs no allocation of any kind.
 *   - Limit: numel * sizeof(element) <= nvfp4_global_scale_static_max_bytes() (512 MiB); larger
 *     inputs return NVFP4_ERR_STATIC_SCRATCH and launch nothing.
 *   - The first call on each device resolves the array's device address (with that device
 *     current); issue it before starting any stream capture.
 *   - All calls on one GPU share the array: calls that may overlap on the GPU (other streams or
 *     host threads) race and must be serialised by the caller.  Calls in one stream are safe; each
 *     call re-clears the counter it relies on.
 */
int nvfp4_global_scale_launch_static(const void* x, int x_dtype, int64_t numel, float fp8_max, float* out,
                                     void* stream);
int64_t nvfp4_global_scale_static_max_bytes(void);

/*
 * out[M, N] (bf16, row-major) = alpha * sum_k dq(a)[m,k] * dq(b)[n,k]
 *   a: uint8 [M, K/2], b: uint8 [N, K/2] packed E2M1, K-major, 16-byte aligned
 *   sfa / sfb: swizzled E4M3 scales as written by nvfp4_quant_launch for
 *              [M, K] and [N, K];  alpha: one float on the device.
 *   K % 64 == 0 required (K % 16 == 0 operands can be produced with padded_n).
 * fp32 accumulation on tcgen05 (kind::mxf4nvf4.block_scale) with TMEM accumulators.
 * replaces vllm `_C::cutlass_scaled_fp4_mm` (vllm/_custom_ops.py:741-752;
 * named at README.md:68).
 * workspace: nvfp4_gemm_workspace_bytes(M, N, K) bytes, 16-byte aligned (may be NULL when that is 0).
 * It is 0 for every shape unless K ranges were switched on through nvfp4_gemm_tune (a testing hook: the tile
 * kernels then write fp32 partial tiles that a second kernel sums); contents need no initialisation.
 * Launches of this library's GEMM kernels may overlap on the GPU (several streams): every kernel reserves shared
 * memory in proportion to the TMEM columns it takes, so CTAs that share an SM never wait for one another's TMEM.
 */
int nvfp4_gemm_launch(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                      const float* alpha, void* out_bf16, int64_t M, int64_t N, int64_t K,
                      void* workspace, size_t workspace_bytes, void* stream);
size_t nvfp4_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);

/*
 * The same GEMM for a weight that is used many times (a model's linear layer; no counterpart in vllm's op, which
 * takes raw tensors on every call).  nvfp4_gemm_prepare encodes the weight's tensor maps once and returns a handle;
 * nvfp4_gemm_launch_prepared(handle, a, sfa, alpha, out, M, ...) then computes out[M, N] exactly as
 * nvfp4_gemm_launch(a, b, sfa, sfb, alpha, out, M, N, K, ...) would, with less host work per call.
 * Ownership: the handle is a small HOST object owned by the caller and freed with nvfp4_gemm_release (NULL is
 * accepted).  It refers to b / sfb without owning them: keep both allocated at the same addresses with the same
 * shape while the handle lives.  A prepared weight is treated as a constant: a launch with the handle starts reading
 * b / sfb while kernels queued before it on the stream are still finishing (see nvfp4_gemm_tune_pdl), so their
 * contents must be complete before such a launch is issued - written before nvfp4_gemm_prepare, or rewritten in place
 * later and followed by a stream / event synchronisation on the host.  (nvfp4_gemm_launch, with raw pointers, makes no
 * such assumption: its weights may come from the kernel just before it.)  A handle belongs to the device that was
 * current in nvfp4_gemm_prepare; launching it with another device current returns NVFP4_ERR_UNSUPPORTED.  Handles may
 * be used from several host threads at once (they are read-only after creation).
 */
int nvfp4_gemm_prepare(const uint8_t* b, const uint8_t* sfb, int64_t N, int64_t K, void** handle_host);
int nvfp4_gemm_launch_prepared(void* handle, const uint8_t* a, const uint8_t* sfa, const float* alpha, void* out_bf16,
                               int64_t M, void* workspace, size_t workspace_bytes, void* stream);
int nvfp4_gemm_release(void* handle);
/*
 * One activation against several prepared weights of equal K in one call (a layer's q / k / v projections, or gate /
 * up: what serving stacks fuse into one wider linear layer; no counterpart in the reference, whose weights are
 * multiplied one by one):
 *   outs_bf16[i][M, N_i] = alpha_w[i][0] * alpha_a[0] * dq(a) dq(weight_i)^T,   i < n_weights <= 64.
 * alpha_w[i] points at one float on the device (the weight's global scale, or the finished output scale); alpha_a at
 * the common factor (the activation's global scale) or is NULL (factor 1).  The product is one fp32 multiplication,
 * so with alpha_a the result equals nvfp4_gemm_launch_prepared with alpha = alpha_w[i][0] * alpha_a[0] computed by a
 * separate fp32 multiplication, without that extra launch.  handles / alpha_w / outs_bf16 are HOST arrays read during the call.
 * Up to 64 tokens (and wherever the kernel choice takes the decode-sized kernel for the group's total N), up to 8 weights
 * go out as ONE launch whose weight tiles are numbered through the group (fixed costs paid once, every SM on the
 * combined weight stream); otherwise one launch per weight.  Outputs agree with the one-by-one calls to fp32 rounding before the bf16 store (bit for bit when
 * the K ranges per tile agree; they are chosen from the group's total tile count).  No workspace.
 */
int nvfp4_gemm_launch_grouped(void* const* handles, int n_weights, const uint8_t* a, const uint8_t* sfa,
                              const float* alpha_a, const float* const* alpha_w, void* const* outs_bf16, int64_t M,
                              void* stream);
/* Testing hook (process-wide): 0 = pick the GEMM kernel by shape (default), 1 = 128x128 tiles,
 * 2 = 128x256 tiles, 3 = CTA-pair 256x256 tiles, 4 = CTA-pair 256x192 tiles, 5 = skinny kernel for
 * M <= 128 (weights on the MMA rows, K ranges across a thread-block cluster; the default up to 32 tokens),
 * 6 = 128x64 tiles, 7 = CTA-pair 256x128 tiles.  Paths 1-4, 6 and 7 give identical bits; path 5 adds its K ranges in a fixed order and
 * agrees with them to fp32 rounding before the bf16 store (identical bits with one range). */
int nvfp4_gemm_force_path(int path);
/* Testing hook: *path = the kernel nvfp4_gemm_launch would take for this shape on a GPU with `sms` SMs under the
 * current force / tune settings (numbering of nvfp4_gemm_force_path), *k_ranges = the skinny kernel's cluster
 * size (1 for the other kernels).  Host arithmetic only: no GPU is touched. */
int nvfp4_gemm_plan(int64_t M, int64_t N, int64_t K, int sms, int* path, int* k_ranges);
/* Testing hook (process-wide): number of K ranges (0 = by shape) and K-loop rotation (-1 = by shape, 0 = off,
 * 1 = on) of the single-CTA tile kernels; while path 5 is forced, k_splits is the cluster size (K ranges per
 * weight tile, 1..8) of the skinny kernel instead.  nvfp4_gemm_workspace_bytes reflects the current setting
 * (the skinny kernel itself never needs a workspace). */
int nvfp4_gemm_tune(int k_splits, int k_rotate);
/* Testing hook (process-wide): 1 (default) = the GEMM kernels, the quantizer and the global-scale kernel are launched
 * as programmatic dependent launches (each may be scheduled while the kernel before it on the stream is finishing;
 * a GEMM starts on its weight stream, which does not depend on that kernel, and everything that does depend on it
 * waits), 0 = plain stream order. */
int nvfp4_gemm_tune_pdl(int enabled);
/* Testing hook (process-wide): m-tiles per band of the persistent kernels' tile numbering (0 = default). */
int nvfp4_gemm_tune_raster(int group);

/* Tensor-pipe rate probe (no counterpart in the reference; it supplies the measured denominator of the GEMM's
 * "fraction of FP4 peak"): every SM issues stages x 4 block-scaled FP4 MMAs (the GEMM's instruction, K = 64 each)
 * back to back on operands resident in shared memory, nothing else.  pair == 0: one CTA per SM, M = 128, N = 256;
 * pair == 1: CTA pairs (cta_group::2), M = 256, N = 256; pair == 2 (testing hook): the pair == 0 kernel with its
 * last commit left out, so that its final wait ends at the wait limit and sets the status word.  Time the launch with events on `stream`; work done =
 * *sms_used * stages * 4 * 2 * 128 * 256 * 64 flop.  1 <= stages <= 2^20.  Waits inside are bounded
 * (nvfp4_gemm_last_status reports an expiry). */
int nvfp4_gemm_peak_probe(int stages, int pair, int* sms_used_host, void* stream);

/* Device status word of the GEMMs on the current device: 0 = ok, else a bounded wait inside a kernel gave up
 * (the kernel returned without hanging).  One word per device: it tells that some launch since the last read
 * failed, not which one or on which stream.  Synchronises `stream`; reading a non-zero word clears it. */
int nvfp4_gemm_last_status(void* stream, uint32_t* status_host);

/* Testing hooks: the time (nanoseconds, 1 us .. 10 s; 0 = the default of 2 s) after which a wait inside the GEMM
 * kernels, or the grid-wide wait of the fused quantizer, gives up on the current device and records its status
 * word instead of waiting on.  Synchronous calls.  No counterpart in the reference. */
int nvfp4_gemm_set_wait_limit_ns(uint64_t ns);
int nvfp4_quant_fused_set_wait_limit_ns(uint64_t ns);

/* *id_host = 0 while `stream` is not being captured into a CUDA graph, else the id of the capture.  Host bookkeeping: the
 * scratch words of nvfp4_global_scale_launch / nvfp4_quant_fused_launch may be shared by launches that are ordered on one
 * stream, but graphs captured one after the other on the same stream can be replayed at the same time on different
 * streams, so every capture needs scratch of its own (the Python helpers key their scratch by this id). */
int nvfp4_stream_capture_id(void* stream, unsigned long long* id_host);
const char* nvfp4_status_string(int status);
int nvfp4_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4_B200_H_ */
