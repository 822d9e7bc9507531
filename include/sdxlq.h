/*
 * sdxlq — C ABI of the B200 (sm_100a) quantized-Linear operator.
 *
 * Drop-in boundary for the SDXL UNet projection path of the reference engine: everything
 * `sdxl::cuda::Ops::linear` / `Ops::linear_activation` dispatch to for a rank-2 weight
 * (include/sdxl/cuda/ops.hpp:21-30, src/cuda/ops_blas.cpp:244-397 of the reference). Plain
 * pointers and sizes only; all pointers are device pointers unless a comment says "host".
 * Every call is asynchronous on the context's stream and returns a status code; nothing
 * throws, aborts or synchronises unless stated.
 *
 * Enumerations keep the numeric values of the reference's enums so that a C++ shim can
 * static_cast between them.
 */
#ifndef SDXLQ_H_
#define SDXLQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status ---------------------------------------------------------------------------- */
typedef enum sdxlq_status {
    SDXLQ_OK = 0,
    SDXLQ_ERR_INVALID_ARGUMENT = 1,   /* the reference throws CudaError for these */
    SDXLQ_ERR_UNSUPPORTED_SHAPE = 2,
    SDXLQ_ERR_TIMEOUT = 3,            /* a bounded device-side wait ran out */
    SDXLQ_ERR_CUDA = 4,               /* a CUDA runtime/driver call failed */
    SDXLQ_ERR_WORKSPACE = 5           /* scratch workspace too small for the request */
} sdxlq_status;

/* ---- element types: numeric values of sdxl::cuda::ScalarType (tensor.hpp:17-24) --------- */
typedef enum sdxlq_dtype {
    SDXLQ_FP8_E4M3 = 0,
    SDXLQ_FP8_E5M2 = 1,
    SDXLQ_INT8 = 2,
    SDXLQ_FP16 = 3,
    SDXLQ_FP32 = 4,
    SDXLQ_INT32 = 5
} sdxlq_dtype;

/* sdxl::cuda::FP8ScaleMode (tensor.hpp:35-39); INT8 weights use PER_OUTPUT_CHANNEL. */
typedef enum sdxlq_scale_mode {
    SDXLQ_SCALE_NONE = 0,
    SDXLQ_SCALE_TENSOR_WIDE = 1,
    SDXLQ_SCALE_PER_OUTPUT_CHANNEL = 2
} sdxlq_scale_mode;

/* sdxl::cuda::FP8StorageLayout (tensor.hpp:45-48). */
typedef enum sdxlq_layout {
    SDXLQ_ROW_MAJOR_NK = 0,
    SDXLQ_K_MAJOR_KN = 1
} sdxlq_layout;

/* sdxl::cuda::LinearActivation (ops.hpp:15). */
typedef enum sdxlq_activation {
    SDXLQ_ACT_NONE = 0,
    SDXLQ_ACT_SILU = 1,
    SDXLQ_ACT_GELU = 2,
    SDXLQ_ACT_QUICK_GELU = 3,
    SDXLQ_ACT_GEGLU = 4
} sdxlq_activation;

/* ---- packed weight + scale metadata -------------------------------------------------------
 * The fields the reference carries on a weight `cuda::Tensor` (tensor.hpp:123-157):
 * data pointer, ScalarType, logical shape [N,K], FP8StorageLayout, dequant_scale_data(),
 * dequant_scale_count(), dequant_scale_mode(), convrot_group_size(). */
typedef struct sdxlq_weight {
    const void* data;            /* [N,K] row-major (or [K,N] when layout == K_MAJOR_KN) */
    int32_t dtype;               /* sdxlq_dtype: INT8, FP8_E4M3, FP8_E5M2 or FP16 */
    int32_t layout;              /* sdxlq_layout */
    uint64_t n;                  /* output features */
    uint64_t k;                  /* input features */
    const float* scales;         /* FP32 dequantisation scales, NULL for FP16 */
    uint64_t scale_count;        /* 1 (tensor wide) or n (per output channel) */
    int32_t scale_mode;          /* sdxlq_scale_mode */
    uint32_t convrot_group_size; /* 0 = no rotation, else 4, 16, 64 or 256 (INT8 only) */
} sdxlq_weight;

/* One Linear: Y[M,N] = act(X[M,K] * W[N,K]^T (+ bias)). Replaces one Ops::linear /
 * Ops::linear_activation call (ops_blas.cpp:244-397). */
typedef struct sdxlq_linear_desc {
    const void* x;               /* FP16 [M,K] contiguous row-major activations */
    uint64_t m;                  /* rows = product of all leading dimensions */
    sdxlq_weight weight;
    const void* bias;            /* FP16 [N] or NULL */
    int32_t activation;          /* sdxlq_activation; anything but NONE requires bias */
    int32_t reserved0;
    void* y;                     /* FP16 [M,N]; [M,N/2] for GEGLU */
    /* Optional reuse of already quantised activations (the three attention projections share
     * one input; the cross-attention K/V projections share the text context). When xq is set,
     * x is not read. INT8: xq INT8 [M,K] rotated with the weight's group size, xq_scales [M].
     * FP8: xq in the weight's FP8 format, xq_scales [1]. */
    const void* xq;
    const float* xq_scales;
    /* Optional: the raw INT32 accumulators [M,N] of the INT8 path (parity checks). */
    int32_t* acc_out;
    /* Optional FP16 [M,N] tensor added to the biased projection in FP16, y = __hadd(linear, residual):
     * the Ops::add_in_place that follows to_out, ff.net.2 and proj_out in the reference's transformer
     * block (src/cuda/unet.cpp:118, 132, 147, 179; add_in_place_kernel, src/cuda/ops_kernels.cu:60-64)
     * folded into the epilogue. May alias y (the hidden state updated in place). Requires
     * activation == NONE. */
    const void* residual;
    /* Hand-over of the FP8 activation quantiser's maximum between two projections (the GEGLU output of
     * ff.net.0.proj is the input of ff.net.2): quantize_tensor_fp8 (fp8_kernels.cu:157-190) reads its
     * input once for max |x| and once for the cast; the first read is saved when the kernel that wrote
     * x already knows the maximum.
     *   y_amax  optional device word (uint32): receives max |y| over this call's FP16 output as the bit
     *           pattern of the FP32 value, by atomic maximum. Zero it once after allocation; the
     *           consuming call puts it back to zero.
     *   x_amax  optional device word filled by the producer of x: FP8 weights only, ignored otherwise;
     *           the quantiser of this call skips its maximum pass, reads the word and clears it.
     * Results are bit-identical to the calls without the words. */
    void* y_amax;
    const void* x_amax;
} sdxlq_linear_desc;

/* sdxl::cuda::INT8ExecutionStats (runtime.hpp:106-112). Every INT8 Linear here runs on the
 * tensor cores, so imma_calls == linear_calls and the other counters stay 0. */
typedef struct sdxlq_int8_stats {
    uint64_t linear_calls;
    uint64_t tensor_core_calls;
    uint64_t dp4a_fallback_calls;
    uint64_t tensor_core_plan_misses;
    uint64_t tensor_core_execution_failures;
} sdxlq_int8_stats;

typedef struct sdxlq_context sdxlq_context;
typedef struct sdxlq_group_plan sdxlq_group_plan;

/* ---- context: stands in for what Ops needs from sdxl::cuda::Runtime (runtime.hpp:120-163:
 * device, stream, scratch arena, INT8 counters). ---------------------------------------- */

/* Creates a context on `device` that launches on `stream` (a cudaStream_t, may be NULL for the
 * default stream). `workspace_bytes` of scratch are allocated once here with cudaMalloc
 * (quantised activations and per-call tables); 0 selects 256 MiB. Not thread-safe: one
 * context per dispatch thread, like the reference Runtime. */
int sdxlq_context_create(int device, void* stream, size_t workspace_bytes, sdxlq_context** out);
void sdxlq_context_destroy(sdxlq_context* ctx);
int sdxlq_context_set_stream(sdxlq_context* ctx, void* stream);
/* Synchronises the stream and reports a device-side timeout flag or a sticky CUDA error. */
int sdxlq_context_check(sdxlq_context* ctx);
/* Host string describing the last non-OK status returned on this context (never NULL). */
const char* sdxlq_last_error(const sdxlq_context* ctx);
const char* sdxlq_status_string(int status);
/* Runtime::int8_execution_stats() (runtime.cpp:403-410). */
int sdxlq_get_stats(const sdxlq_context* ctx, sdxlq_int8_stats* out);

/* ---- the operator ------------------------------------------------------------------------ */

/* Ops::linear / Ops::linear_activation (ops_blas.cpp:244-397), dispatching on weight.dtype:
 * INT8 -> int8_convrot_linear (int8_convrot.cu:579-751), FP8 -> native_fp8_linear
 * (ops_blas.cpp:153-225, extended to per-output-channel weight scales), FP16 -> dense. */
int sdxlq_linear(sdxlq_context* ctx, const sdxlq_linear_desc* desc);

/* All `count` independent projections in one grouped launch per kernel kind (one activation-
 * quantise launch, one GEMM launch). Projections that read the same x with the same
 * quantisation share one quantised copy. No counterpart in the reference, which issues the
 * 743 projections of a UNet step one by one (src/cuda/unet.cpp:20-181).
 * Up to four projections that share one input per quantiser kind (the to_q/to_k/to_v of an
 * attention layer) travel in the kernel parameters: no table, no allocation, capturable. Larger
 * groups upload their tables through a pinned staging buffer and a stream-ordered allocation
 * (cudaMallocAsync / cudaFreeAsync on the context's stream): the call does not wait for the GPU,
 * but it cannot be recorded by a stream capture (build a plan for that). */
int sdxlq_linear_grouped(sdxlq_context* ctx, const sdxlq_linear_desc* descs, size_t count);

/* The same grouped launch split into build-once / run-many (descriptor tables stay on the
 * device). Pointers inside the descriptors must stay valid for the plan's lifetime. Creation
 * allocates with cudaMalloc and copies synchronously; running never allocates or synchronises.
 * A plan runs only on the context that created it (its tables address that context's workspace). */
int sdxlq_group_plan_create(sdxlq_context* ctx, const sdxlq_linear_desc* descs, size_t count,
                            sdxlq_group_plan** out);
int sdxlq_group_plan_run(sdxlq_context* ctx, sdxlq_group_plan* plan);
void sdxlq_group_plan_destroy(sdxlq_group_plan* plan);
/* Number of kernels one run of the plan launches. */
int sdxlq_group_plan_launches(const sdxlq_group_plan* plan);

/* The same Linear for callers that must not allocate device memory. It has no counterpart in
 * the reference (whose Ops::linear takes every temporary from the Runtime arena).
 *
 * Some hosts of this library cannot call cudaMalloc when they need a projection: an engine that
 * has handed all of the GPU's memory to its own pool and forbids driver allocations afterwards,
 * a plugin that runs inside a callback where the allocator's lock is already held, or a service
 * whose steady state is audited to be allocation-free. sdxlq_context_create allocates its
 * workspace, so it is off limits for them. This entry point needs no context: the quantised
 * activations (INT8: M*K bytes + 4*M; FP8: M*K bytes + 4) go to a 16 MiB array that is part of the
 * library image on every GPU that loads it, and nothing in the call allocates or frees device
 * memory. Projections that need more scratch than that are rejected with SDXLQ_ERR_WORKSPACE and
 * an explanatory message (FP16 weights need none and always fit).
 *
 *  - `device` must be the calling thread's current CUDA device. The first call on a device looks
 *    up the array's device address and the device's properties; make that first call outside any
 *    stream capture.
 *  - All calls on one GPU share the array, which still holds the previous call's data when the next
 *    one starts. Each call overwrites what it reads, but two calls whose kernels overlap on the GPU
 *    (different streams, no ordering between them) race on it: order them.
 *  - `message` (may be NULL) receives a NUL-terminated explanation when the status is not SDXLQ_OK.
 *  - A bounded device-side wait that runs out is not reported by this entry point. */
int sdxlq_linear_static(int device, void* stream, const sdxlq_linear_desc* desc, char* message,
                        size_t message_capacity);

/* ---- activation quantisers ---------------------------------------------------------------- */

/* activation_amax_kernel + quantize_activation_kernel (int8_convrot.cu:265-353) in one pass:
 * per-row optional regular-Hadamard rotation per group, per-row scale, INT8.
 * x_dtype is SDXLQ_FP16 or SDXLQ_FP32. xq [M,K] INT8, scales [M] FP32. */
int sdxlq_quantize_act_int8(sdxlq_context* ctx, const void* x, int32_t x_dtype, uint64_t m,
                            uint64_t k, uint32_t convrot_group_size, int8_t* xq, float* scales);

/* quantize_tensor_fp8 (fp8_kernels.cu:157-190): tensor-wide dynamic scale + saturating cast.
 * fmt is SDXLQ_FP8_E4M3 or SDXLQ_FP8_E5M2; q has `count` bytes; scale is one FP32. */
int sdxlq_quantize_act_fp8(sdxlq_context* ctx, const void* x_f16, uint64_t count, int32_t fmt,
                           uint8_t* q, float* scale);

/* ---- LayerNorm feeding a projection ------------------------------------------------------- */

/* Ops::layer_norm (include/sdxl/cuda/ops.hpp:39-42, src/cuda/ops_kernels.cu:185-256, 1425-1470) over the
 * last dimension of FP16 x[rows, width], optionally fused with the activation quantiser of the
 * projection that consumes the result, so that the normalised FP16 tensor is never written:
 *   out_dtype SDXLQ_FP16      y[rows, width] FP16, the reference's result.
 *   out_dtype SDXLQ_INT8      xq[rows, width] INT8 + xq_scales[rows]: LayerNorm, rounding to FP16, ConvRot
 *                             rotation (convrot_group_size, 0 = none) and per-row quantisation in one
 *                             call, equal to sdxlq_quantize_act_int8 applied to the FP16 result (one launch
 *                             without rotation; with rotation the FP16 rows pass through the context's
 *                             workspace on their way to the rotation kernel).
 *   out_dtype SDXLQ_FP8_E4M3 / SDXLQ_FP8_E5M2
 *                             xq[rows, width] FP8 + xq_scales[1], equal to sdxlq_quantize_act_fp8 applied
 *                             to the FP16 result (two launches: statistics, then normalise + cast).
 * Pass xq / xq_scales to sdxlq_linear_desc.xq / .xq_scales of every projection that reads the
 * normalised activations (to_q / to_k / to_v, ff.net.0.proj). The FP16 and FP8 forms want width a
 * multiple of 8, at most 2048, and 16-byte aligned rows (every SDXL width: 640, 1280);
 * SDXLQ_ERR_UNSUPPORTED_SHAPE otherwise. rows == 0 is a no-op. */
typedef struct sdxlq_layer_norm_desc {
    const void* x;               /* FP16 [rows, width] */
    uint64_t rows;
    uint64_t width;
    const void* gamma;           /* FP16 [width] */
    const void* beta;            /* FP16 [width] */
    float epsilon;               /* the reference's default is 1e-5 */
    int32_t out_dtype;
    uint32_t convrot_group_size; /* SDXLQ_INT8 only */
    uint32_t reserved;
    void* y;                     /* SDXLQ_FP16 */
    void* xq;                    /* quantised forms */
    float* xq_scales;
} sdxlq_layer_norm_desc;
int sdxlq_layer_norm(sdxlq_context* ctx, const sdxlq_layer_norm_desc* desc);

/* ---- harness scaffolding (not part of the projection path) --------------------------------- */

/* GroupNorm, optionally followed by SiLU, over channels-last FP16 activations x[batch, rows, channels]
 * (NHWC memory: rows = height * width): what Ops::group_norm_nchw / group_norm_silu_nchw
 * (include/sdxl/cuda/ops.hpp:43-52, src/cuda/ops_kernels.cu:258-308) compute, on the layout the
 * synthetic UNet loop keeps its convolution activations in, so that no layout copy surrounds the
 * norm. channel_bias (optional, [batch, channels] FP16) is added first with FP16 rounding: the
 * resnet's add_spatial_bias in front of norm2. y may alias x. channels must be a multiple of 8 and of
 * groups, at most 3072, with 16-byte aligned tensors; groups at most 64, batch at most 1024;
 * SDXLQ_ERR_UNSUPPORTED_SHAPE otherwise. Exists so
 * that the benchmark's UNet loop does not spend a quarter of its step on layout copies; it is not a
 * drop-in for the reference's NCHW operator. */
typedef struct sdxlq_group_norm_desc {
    const void* x;
    const void* channel_bias;
    const void* gamma;           /* FP16 [channels] */
    const void* beta;            /* FP16 [channels] */
    void* y;
    uint64_t batch;
    uint64_t rows;
    uint64_t channels;
    uint32_t groups;
    int32_t silu;
    float epsilon;
    uint32_t reserved;
} sdxlq_group_norm_desc;
int sdxlq_group_norm_nhwc(sdxlq_context* ctx, const sdxlq_group_norm_desc* desc);

/* y[r, c] = half(half(x[r, c] + bias[c]) + residual[r, c]) over channels-last FP16 x[rows, channels]: the
 * bias add of a convolution whose library call leaves the bias out, and the resnet's residual add
 * (Ops::add, src/cuda/unet.cpp:92), in one pass. channels a multiple of 8, all pointers 16-byte
 * aligned (SDXLQ_ERR_UNSUPPORTED_SHAPE otherwise); y may alias x or residual. */
int sdxlq_harness_bias_residual_add(sdxlq_context* ctx, const void* x, const void* bias, const void* residual, void* y,
                                    uint64_t rows, uint64_t channels);

/* ---- load-time weight packers ------------------------------------------------------------- */

/* upload_or_quantize_int8_weight (int8_convrot.cu:498-577) for a weight already on the device:
 * src_dtype FP16/FP32 -> rotate (group g, 0 = none) + per-row scale + INT8;
 * src_dtype INT8 -> copied unchanged (prequantised checkpoint; scales are supplied by the
 * caller and `scales` may be NULL). dst [N,K] INT8, scales [N]. */
int sdxlq_pack_weight_int8(sdxlq_context* ctx, const void* src, int32_t src_dtype, uint64_t n,
                           uint64_t k, uint32_t convrot_group_size, int8_t* dst, float* scales);

/* WeightStore::upload_tensor FP8 branch (weights.cu:119-170, 301-415): scale = max(amax /
 * FP8_MAX, 1e-12) (1 if amax == 0) tensor wide or per output row, q = FP8(value / scale);
 * a source already in `fmt` is copied with scales = 1. src_dtype FP16/FP32/FP8. */
int sdxlq_pack_weight_fp8(sdxlq_context* ctx, const void* src, int32_t src_dtype, uint64_t n,
                          uint64_t k, int32_t fmt, int32_t scale_mode, int32_t layout,
                          uint8_t* dst, float* scales);

/* valid_convrot_group_size (int8_convrot.cu:489-496). */
int sdxlq_valid_convrot_group_size(size_t group_size);

/* Scratch bytes sdxlq_linear / a grouped call needs for these descriptors (host arithmetic). */
size_t sdxlq_workspace_bytes(const sdxlq_linear_desc* descs, size_t count);

/* ---- diagnostics (no counterpart in the reference) ---------------------------------------- */

/* Overrides the accumulator tile width chosen per projection (multiple of 16, <= 256;
 * 0 restores the built-in choice). For tuning sweeps. */
int sdxlq_context_set_tile_n(sdxlq_context* ctx, int tile_n);

/* Selects the GEMM kernel flavour: 0 (default) runs every tile on one CTA (128 rows); 1 uses CTA
 * pairs (cta_group::2, 256-row tiles, each CTA loading half of the weight rows) for every projection
 * with more than 128 rows; -1 uses pairs only for projections of launches that fill the GPU several
 * times over. Results are bit-identical between the flavours. Pairs measured no faster than single
 * CTAs on B200 for this path, so they are opt-in. For tuning sweeps and tests. */
int sdxlq_context_set_pair_mode(sdxlq_context* ctx, int mode);

/* Per-kernel device timing. While enabled, every kernel launch of the library is bracketed by a
 * CUDA event pair recorded on the context's stream; sdxlq_profile_read synchronises, sums the
 * elapsed times per kernel class since the last read and resets. The FP8 quantiser counts as
 * two launches (amax + cast) timed together. */
enum {
    SDXLQ_KERNEL_QUANT_INT8 = 0,
    SDXLQ_KERNEL_QUANT_FP8 = 1,
    SDXLQ_KERNEL_GEMM = 2,
    SDXLQ_KERNEL_SMALL = 3,
    SDXLQ_KERNEL_LAYER_NORM = 4,
    SDXLQ_KERNEL_HARNESS = 5,         /* sdxlq_group_norm_nhwc */
    SDXLQ_KERNEL_CLASSES = 6
};
typedef struct sdxlq_kernel_times {
    double milliseconds[SDXLQ_KERNEL_CLASSES];
    uint64_t launches[SDXLQ_KERNEL_CLASSES];
} sdxlq_kernel_times;
int sdxlq_profile_enable(sdxlq_context* ctx, int enabled);
int sdxlq_profile_read(sdxlq_context* ctx, sdxlq_kernel_times* out);

/* Failure-detection self test: launches a one-thread kernel that waits, for at most
 * `limit_cycles` SM clocks, on a barrier nothing signals. The wait runs out, the kernel records
 * a timeout code and returns normally; the next sdxlq_context_check reports
 * SDXLQ_ERR_TIMEOUT and the context remains usable. */
int sdxlq_selftest_bounded_wait(sdxlq_context* ctx, long long limit_cycles);

/* Library build information: "sm_100a" and the kernel generation string. */
const char* sdxlq_build_info(void);

#ifdef __cplusplus
}
#endif

#endif /* SDXLQ_H_ */
