// Structures shared by the host dispatch code and the kernels, and the epilogue arithmetic
// shared by the tensor-core GEMM and the small-shape kernel.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace sdxlq {

// Operand kind of a GEMM problem (both operands have the same kind).
enum GemmKind : uint32_t { KIND_I8 = 0, KIND_E4M3 = 1, KIND_E5M2 = 2, KIND_F16 = 3 };

enum Activation : uint32_t { ACT_NONE = 0, ACT_SILU = 1, ACT_GELU = 2, ACT_QUICK_GELU = 3, ACT_GEGLU = 4 };

// Error word values written by a kernel whose bounded wait ran out.
enum DeviceError : uint32_t {
    DEV_OK = 0,
    DEV_TIMEOUT_PRODUCER = 0x100,
    DEV_TIMEOUT_MMA = 0x200,
    DEV_TIMEOUT_EPILOGUE = 0x300,
};

constexpr uint32_t kTileM = 128;          // rows of one output tile (UMMA M)
constexpr uint32_t kTileKBytes = 128;     // bytes of K per pipeline stage row (one swizzle span)
constexpr uint32_t kMaxTileN = 256;       // UMMA N limit
constexpr uint32_t kTmemColumns = 512;    // two accumulator buffers of up to 256 columns

// Everything the epilogue needs for one problem.
struct EpilogueParams {
    __half* y;                   // [M, n_out]
    int32_t* acc_out;            // optional raw INT32 accumulators [M, N]
    const float* a_scales;       // INT8: [M]; FP8: [1]; FP16: unused
    const float* w_scales;       // [N] or [1]; FP16: unused
    const __half* bias;          // [N] or null
    const __half* residual;      // optional [M, N] added to the biased projection (may alias y)
    uint32_t* y_amax;            // optional word: atomic maximum of |y| (FP32 bit pattern) over this problem's output
    uint32_t m, n, k;
    uint32_t n_out;              // n, or n / 2 for GEGLU
    uint32_t kind;               // GemmKind
    uint32_t activation;         // Activation
    uint32_t w_scale_per_channel;
    uint32_t vector_store_ok;    // y rows are 16-byte aligned and n_out % 8 == 0
    uint32_t vector_meta_ok;     // w_scales / bias (and their GEGLU gate halves) are 16-byte aligned
};

// One GEMM problem of a grouped launch. Tensor maps first (64-byte alignment required).
struct alignas(64) GemmProblem {
    CUtensorMap tmap_a;          // [M, K] activations (quantised), box {128 B, 128 rows}
    CUtensorMap tmap_b;          // [N, K] weights, box {128 B, tile_n rows} (tile_n / 2 for GEGLU)
    EpilogueParams ep;
    uint32_t tile_n;             // accumulator columns per tile (multiple of 16, <= 256)
    uint32_t tiles_m;
    uint32_t tiles_n;
    uint32_t k_blocks;           // ceil(K bytes / 128)
    uint32_t idesc;              // UMMA instruction descriptor
    uint32_t pad[1];
};

// One tile of a launch: everything the three kernel roles need to start on it, in one 64-byte
// record, so that a role can fetch the record of its next tile while it works on the current one
// and never chases a pointer between tiles.
enum TileFlags : uint16_t {
    TILE_HAS_BIAS = 1,          // bias != null
    TILE_SCALE_PER_CHANNEL = 2, // w_scales has one entry per weight row (else one entry)
    TILE_STORE_16 = 4,          // y rows 16-byte aligned and n_out % 8 == 0
    TILE_STORE_32 = 8,          // y rows 32-byte aligned and n_out % 16 == 0
    TILE_RAW_ACCUMULATORS = 16, // the problem also wants its INT32 accumulators (ep.acc_out)
    TILE_HAS_RESIDUAL = 32,     // ep.residual is added after the bias (no activation)
    TILE_OUTPUT_AMAX = 64,      // ep.y_amax receives the maximum of |y|
};

struct alignas(64) TileRef {
    uint32_t problem;            // index into the problem table (tensor maps, acc_out)
    uint16_t tile_m;
    uint16_t tile_n_index;
    uint32_t idesc;              // UMMA instruction descriptor
    uint32_t n_out;
    uint16_t k_blocks;
    uint16_t tile_n;             // accumulator columns of the tile
    uint8_t kind;                // GemmKind
    uint8_t activation;          // Activation
    uint16_t flags;              // TileFlags
    uint32_t m, n;
    const float* w_scales;
    const __half* bias;
    __half* y;
    const float* a_scales;
};
static_assert(sizeof(TileRef) == 64, "a tile record is one 64-byte line");

// The record of tile (tile_m, tile_n_index) of `problem` (table index `problem_index`).
__host__ __device__ inline TileRef make_tile_ref(const GemmProblem& problem, uint32_t problem_index, uint32_t tile_m,
                                                 uint32_t tile_n_index) {
    const EpilogueParams& ep = problem.ep;
    TileRef r;
    r.problem = problem_index;
    r.tile_m = static_cast<uint16_t>(tile_m);
    r.tile_n_index = static_cast<uint16_t>(tile_n_index);
    r.idesc = problem.idesc;
    r.n_out = ep.n_out;
    r.k_blocks = static_cast<uint16_t>(problem.k_blocks);
    r.tile_n = static_cast<uint16_t>(problem.tile_n);
    r.kind = static_cast<uint8_t>(ep.kind);
    r.activation = static_cast<uint8_t>(ep.activation);
    const bool store_32 = ep.vector_store_ok != 0 && ep.n_out % 16 == 0 && reinterpret_cast<uintptr_t>(ep.y) % 32 == 0;
    r.flags = static_cast<uint16_t>((ep.bias != nullptr ? TILE_HAS_BIAS : 0) |
                                    (ep.kind != KIND_F16 && ep.w_scale_per_channel != 0 ? TILE_SCALE_PER_CHANNEL : 0) |
                                    (ep.vector_store_ok != 0 ? TILE_STORE_16 : 0) | (store_32 ? TILE_STORE_32 : 0) |
                                    (ep.acc_out != nullptr ? TILE_RAW_ACCUMULATORS : 0) |
                                    (ep.residual != nullptr ? TILE_HAS_RESIDUAL : 0) | (ep.y_amax != nullptr ? TILE_OUTPUT_AMAX : 0));
    r.m = ep.m;
    r.n = ep.n;
    r.w_scales = ep.w_scales;
    r.bias = ep.bias;
    r.y = ep.y;
    r.a_scales = ep.a_scales;
    return r;
}

// Problems a launch can carry in its kernel parameters instead of a device table: a single call, or a
// small group (the three attention projections of one input) that then needs no table upload and
// can be issued inside a stream capture.
constexpr uint32_t kInlineProblems = 4;

struct GemmLaunchParams {
    const GemmProblem* problems; // device table (grouped plan) or null (`inline_problems` are used)
    const TileRef* tiles;        // device tile list (grouped plan) or null
    uint32_t num_tiles;
    uint32_t num_stages;
    uint32_t stage_bytes;        // bytes of one pipeline stage (A tile + B tile), multiple of 1024
    uint32_t b_offset;           // offset of the B tile inside a stage (= 128 rows * 128 B)
    uint32_t* error_word;        // device word set on a bounded-wait timeout
    long long wait_limit_cycles;
    uint32_t diagnostic_skip;    // tuning aid, results are meaningless when set. bit 0: no epilogue arithmetic or
                                 // stores; bit 1: no operand loads, no MMAs; bit 2: no operand loads; bit 3: no
                                 // MMAs; bit 5: one MMA per stage instead
                                 // of four; bit 6: only the A operand is loaded. Barriers are still signalled.
    uint32_t inline_count;       // problems in `inline_problems` (1 for a single call)
    uint32_t inline_tile_start[kInlineProblems + 1];   // first tile of each inline problem, then the tile count
    uint32_t pad1[3];
    GemmProblem inline_problems[kInlineProblems];
};

// ------------------------------------------------------------------------------------------
// Epilogue arithmetic. `acc_bits` is the raw 32-bit accumulator (INT32 for KIND_I8, FP32
// otherwise). Returns the FP16 projection before bias/activation:
//   INT8: half_rn((float(acc) * a_scale[row]) * w_scale[col])   (dequantize_gemm_f16_kernel)
//   FP8 : half_rn((acc * x_scale) * w_scale[col or 0])          (native FP8 Linear contract)
//   FP16: half_rn(acc)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ __half project_to_half(uint32_t acc_bits, uint32_t kind, float a_scale,
                                                  float w_scale) {
    float value;
    if (kind == KIND_I8) {
        value = __fmul_rn(__fmul_rn(static_cast<float>(static_cast<int32_t>(acc_bits)), a_scale), w_scale);
    } else if (kind == KIND_F16) {
        value = __uint_as_float(acc_bits);
    } else {
        value = __fmul_rn(__fmul_rn(__uint_as_float(acc_bits), a_scale), w_scale);
    }
    return __float2half_rn(value);
}

// 1 + erf(x / sqrt 2) = 2 * Phi(x), from erfc(t) = 2^(t * r(t)) with t = |x| / sqrt 2 clamped to
// 4.6 and r a degree-9 polynomial (least-squares fit of log2(erfc(t)) / t on Chebyshev nodes of
// [0, 4.6]): relative error of erfc below 1.5e-6 for t < 3 and absolute error below 6e-7
// everywhere, evaluated in FP32. For x >= 0 the result 2 - erfc(t) therefore carries an error
// below 6e-7; for x < 0 it is erfc(t) itself, which keeps its relative accuracy in the tail where
// the textbook 1 + erf(x) loses it to cancellation.
__device__ __forceinline__ float one_plus_erf(float x) {
    const float u = x * 0.7071067811865475f;
    const float t = fminf(fabsf(u), 4.6f);
    float r = -2.6164917699134094e-07f;
    r = fmaf(r, t, 6.632982149312738e-06f);
    r = fmaf(r, t, -7.087277481332421e-05f);
    r = fmaf(r, t, 0.0003955792635679245f);
    r = fmaf(r, t, -0.0009763258858583868f);
    r = fmaf(r, t, -0.0020724914502352476f);
    r = fmaf(r, t, 0.029831526800990105f);
    r = fmaf(r, t, -0.14946085214614868f);
    r = fmaf(r, t, -0.9181336760520935f);
    r = fmaf(r, t, -1.6279360055923462f);
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(r * t));
    return u >= 0.0f ? 2.0f - e : e;
}

// gelu(x) = 0.5 * x * (1 + erf(x / sqrt 2)), the exact-erf GELU of the reference
// (apply_linear_activation / bias_geglu_kernel, src/cuda/ops_kernels.cu:128-183).
__device__ __forceinline__ float gelu_erf(float x) {
    return (0.5f * x) * one_plus_erf(x);
}

// Two evaluations of one_plus_erf at once on the packed FP32 pipe (fma.rn.f32x2 rounds each half
// like the scalar fma.rn, so both halves equal the scalar function bit for bit).
__device__ __forceinline__ float2 one_plus_erf2(float2 x) {
    const float2 u = __fmul2_rn(x, make_float2(0.7071067811865475f, 0.7071067811865475f));
    const float2 t = make_float2(fminf(fabsf(u.x), 4.6f), fminf(fabsf(u.y), 4.6f));
    float2 r = make_float2(-2.6164917699134094e-07f, -2.6164917699134094e-07f);
    r = __ffma2_rn(r, t, make_float2(6.632982149312738e-06f, 6.632982149312738e-06f));
    r = __ffma2_rn(r, t, make_float2(-7.087277481332421e-05f, -7.087277481332421e-05f));
    r = __ffma2_rn(r, t, make_float2(0.0003955792635679245f, 0.0003955792635679245f));
    r = __ffma2_rn(r, t, make_float2(-0.0009763258858583868f, -0.0009763258858583868f));
    r = __ffma2_rn(r, t, make_float2(-0.0020724914502352476f, -0.0020724914502352476f));
    r = __ffma2_rn(r, t, make_float2(0.029831526800990105f, 0.029831526800990105f));
    r = __ffma2_rn(r, t, make_float2(-0.14946085214614868f, -0.14946085214614868f));
    r = __ffma2_rn(r, t, make_float2(-0.9181336760520935f, -0.9181336760520935f));
    r = __ffma2_rn(r, t, make_float2(-1.6279360055923462f, -1.6279360055923462f));
    const float2 exponent = __fmul2_rn(r, t);
    float2 e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(exponent.x));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(exponent.y));
    return make_float2(u.x >= 0.0f ? 2.0f - e.x : e.x, u.y >= 0.0f ? 2.0f - e.y : e.y);
}

__device__ __forceinline__ float2 gelu_erf2(float2 x) {
    return __fmul2_rn(__fmul2_rn(x, make_float2(0.5f, 0.5f)), one_plus_erf2(x));
}

// SiLU / GELU / QuickGELU on the FP32 value (ACT_NONE returns x).
__device__ __forceinline__ float activate(float x, uint32_t activation) {
    if (activation == ACT_SILU) return x / (1.0f + expf(-x));
    if (activation == ACT_GELU) return gelu_erf(x);
    if (activation == ACT_QUICK_GELU) return x / (1.0f + expf(-1.702f * x));
    return x;
}

// Bias + activation on an FP16 projection, as the reference runs them after the GEMM:
//   none     : __hadd(y, b)                                  (add_last_dim_bias_kernel)
//   SiLU/GELU/QuickGELU : half_rn(act(float(y) + float(b)))  (bias_activation_in_place_kernel)
__device__ __forceinline__ __half finish_scalar(__half y, bool has_bias, __half bias, uint32_t activation) {
    if (!has_bias) return y;
    if (activation == ACT_NONE) return __hadd(y, bias);
    return __float2half_rn(activate(__half2float(y) + __half2float(bias), activation));
}

// bias_geglu_kernel: out = half_rn((float(yv) + float(bv)) * gelu(float(yg) + float(bg))).
__device__ __forceinline__ __half finish_geglu(__half y_value, __half bias_value, __half y_gate,
                                               __half bias_gate) {
    const float value = __half2float(y_value) + __half2float(bias_value);
    const float gate = __half2float(y_gate) + __half2float(bias_gate);
    return __float2half_rn(value * gelu_erf(gate));
}

}  // namespace sdxlq
