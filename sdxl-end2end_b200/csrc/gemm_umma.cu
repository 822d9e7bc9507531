// Persistent, warp-specialised tcgen05 GEMM with fused dequant + bias + activation epilogue.
//
//   Y[M, N] = epilogue( A[M, K] * B[N, K]^T )      A, B both K-major, 8-bit (INT8 / FP8) or FP16
//
// Replaces, for every projection of the path, the reference's cuBLASLt call plus the kernels
// it runs afterwards: INT8 (src/cuda/int8_convrot.cu:634-698 GEMM, :388-402 dequant), FP8
// (src/cuda/ops_blas.cpp:153-225), FP16 (ops_blas.cpp:300-385), then add_last_dim_bias /
// bias_activation_in_place / bias_geglu (src/cuda/ops_kernels.cu:76-82, 142-183).
//
// One CTA per SM walks a tile list (all tiles of all problems of a grouped launch):
// (or one cluster of two CTAs per SM pair, see the kernel template)
//   warp 0    TMA producer  : cp.async.bulk.tensor 2D loads into a ring of 128B-swizzled stages
//   warp 1    MMA issuer    : tcgen05.mma (kind::i8 / kind::f8f6f4 / kind::f16), accumulators
//                             in TMEM, two accumulator buffers so the next tile's main loop
//                             overlaps this tile's epilogue
//   warps 2-9 epilogue      : tcgen05.ld -> scales, bias, activation / GEGLU -> FP16 stores
// Every wait is bounded: when one runs out the CTA raises an abort word, all roles leave their
// loops, TMEM is released and the kernel returns with an error code in global memory.

#include "internal.cuh"
#include "ptx.cuh"

#include <mutex>

namespace sdxlq {

// Tuning build only: cycle counters of CTA 0's roles, written behind the error word (words 16..47 of the
// control buffer) when the kernel ends. DIAG_ADD(counter, statement) times the statement.
#ifdef SDXLQ_DIAGNOSTICS
#define DIAG_DECL(name) long long name = 0
#define DIAG_ADD(name, ...) do { const long long diag_t0 = clock64(); __VA_ARGS__; name += clock64() - diag_t0; } while (0)
#define DIAG_WRITE(index, value) do { if (blockIdx.x == 0) params.error_word[16 + (index)] = static_cast<uint32_t>(value); } while (0)
#else
#define DIAG_DECL(name)
#define DIAG_ADD(name, ...) do { __VA_ARGS__; } while (0)
#define DIAG_WRITE(index, value)
#endif

namespace {

constexpr uint32_t kMaxStages = 8;
#ifndef SDXLQ_EPILOGUE_WARPS
#define SDXLQ_EPILOGUE_WARPS 8
#endif
constexpr uint32_t kEpilogueWarps = SDXLQ_EPILOGUE_WARPS;    // a multiple of 4: warps per TMEM lane quadrant x 4
constexpr uint32_t kWarpsPerQuadrant = kEpilogueWarps / 4;
// Warps 0-3 form the control warpgroup (warp 0 TMA producer, warp 1 MMA issuer, warps 2-3 stagers);
// the epilogue warps follow. Register reallocation (setmaxnreg) works on whole warpgroups, so
// the roles are laid out in groups of four warps: the control warpgroup hands most of its
// registers to the epilogue warpgroups once the kernel is set up.
constexpr uint32_t kControlWarps = 4;
constexpr uint32_t kThreads = 32 * (kControlWarps + kEpilogueWarps);
// Register split: the compiler budgets (64 K / threads) registers per thread, rounded down to a
// multiple of 8 (168 for 384 threads); the control warpgroup keeps 64 and the epilogue warps share
// what that frees: 128 * 64 + 256 * 216 <= 384 * 168.
constexpr uint32_t kControlRegisters = 64;
constexpr uint32_t kCompiledRegisters = 65536 / kThreads / 8 * 8;
constexpr uint32_t kEpilogueRegisters =
    (kCompiledRegisters * kThreads - 32 * kControlWarps * kControlRegisters) / (32 * kEpilogueWarps) / 8 * 8;
static_assert(32 * kControlWarps * kControlRegisters + 32 * kEpilogueWarps * kEpilogueRegisters <= kCompiledRegisters * kThreads,
              "the register split must fit the registers the block was launched with");

// The 512 accumulator columns of tensor memory are handed out in quarters of 128: a tile of up to
// 128 accumulator columns takes one quarter, a wider one two adjacent quarters (never wrapping
// around). The MMA issuer and the epilogue warps walk the same tile list and place every tile with
// the same rule, so no placement is communicated. With narrow tiles up to four tiles are in
// flight between the two roles, with wide tiles two.
constexpr uint32_t kAccQuarters = 4;
constexpr uint32_t kQuarterColumns = kTmemColumns / kAccQuarters;
constexpr uint32_t kSlots = 4;

struct AccumulatorRing {
    uint32_t cursor = 0;     // next free quarter
    uint32_t parity = 0;     // one bit per quarter, toggled at each use of the quarter by this role
    // Places a tile: returns its first quarter, sets `quarters` to how many it takes.
    __device__ __forceinline__ uint32_t place(uint32_t tile_n, uint32_t& quarters) {
        quarters = tile_n > kQuarterColumns ? 2u : 1u;
        if (cursor + quarters > kAccQuarters) cursor = 0;
        const uint32_t first = cursor;
        cursor = (cursor + quarters) & (kAccQuarters - 1u);
        return first;
    }
};

struct alignas(64) Control {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[kAccQuarters];    // MMA issuer -> epilogue: the tile whose first quarter this is, is complete
    uint64_t acc_empty[kAccQuarters];   // epilogue -> MMA issuer: this quarter of the accumulator columns is drained
    uint64_t staged[kSlots];            // stagers -> epilogue: the operand slot of this tile is filled
    uint64_t slot_free[kSlots];         // epilogue -> stagers: every epilogue warp of this CTA is done with the slot
    uint32_t tmem_base;
    uint32_t abort;
    uint32_t pad[2];
    // Per-tile epilogue operands, a ring of slots (tile i of the CTA uses slot i % kSlots), filled
    // by the stager warps while the tile's main loop runs: the tile record, the activation scale of
    // each of the CTA's 128 rows, and the weight scale and bias of every accumulator column.
    TileRef header[kSlots];
    alignas(16) float row_scale[kSlots][kTileM];
    alignas(16) float column_scale[kSlots][kMaxTileN];
    alignas(16) float column_bias[kSlots][kMaxTileN];         // the FP16 bias widened to FP32 (exact)
    alignas(16) __half column_bias_half[kSlots][kMaxTileN];
};

// The record of tile `index` of the launch. Launches that carry their problems in the kernel
// parameters (a single call, a small group) build it from there (constant bank): the tiles of
// problem p are numbered inline_tile_start[p] .. inline_tile_start[p + 1] - 1, row tiles fastest.
// Grouped plans read it from the tile list in global memory. Indices past the end read the last
// record, so a role may always fetch one tile ahead.
__device__ __forceinline__ TileRef load_tile(const GemmLaunchParams& params, uint32_t index) {
    index = min(index, params.num_tiles - 1u);
    if (params.problems == nullptr) {
        uint32_t p = 0;
#pragma unroll
        for (uint32_t i = 1; i < kInlineProblems; ++i) {
            if (i < params.inline_count && index >= params.inline_tile_start[i]) p = i;
        }
        const GemmProblem& problem = params.inline_problems[p];
        const uint32_t local = index - params.inline_tile_start[p];
        return make_tile_ref(problem, p, local % problem.tiles_m, local / problem.tiles_m);
    }
    const uint4* source = reinterpret_cast<const uint4*>(params.tiles + index);
    union {
        TileRef record;
        uint4 words[4];
    } u;
#pragma unroll
    for (int i = 0; i < 4; ++i) u.words[i] = __ldg(source + i);
    return u.record;
}

__device__ __forceinline__ const GemmProblem* tile_problem(const GemmLaunchParams& params, const TileRef& tile) {
    return params.problems == nullptr ? &params.inline_problems[tile.problem] : params.problems + tile.problem;
}

__device__ __forceinline__ void raise_abort(Control* control, uint32_t* error_word, uint32_t code) {
    *reinterpret_cast<volatile uint32_t*>(&control->abort) = 1;
    atomicCAS(error_word, 0u, code);
}

// Fills one slot with a tile's epilogue operands. Run by the two stager warps: `part` 0 takes the
// lower half of the columns and rows, `part` 1 the upper half. All loads are issued before the
// first store so that their latencies overlap.
// Column j of a GEGLU tile is value column n0 + j for j < tile_n / 2 and gate column
// n_out + n0 + (j - tile_n / 2) otherwise. Columns past the matrix edge get scale 0, bias 0; rows
// past it get activation scale 0.
__device__ __forceinline__ void stage_tile(const TileRef& tile, uint32_t first_row, uint32_t lane, uint32_t part,
                                           Control* control, uint32_t slot) {
    const bool geglu = tile.activation == ACT_GEGLU;
    const bool scaled = tile.kind != KIND_F16;
    const bool per_channel = (tile.flags & TILE_SCALE_PER_CHANNEL) != 0;
    const bool has_bias = (tile.flags & TILE_HAS_BIAS) != 0;
    const uint32_t tile_n = tile.tile_n;
    const uint32_t half = tile_n / 2;
    const uint32_t n0 = tile.tile_n_index * (geglu ? half : tile_n);
    constexpr uint32_t kColumns = kMaxTileN / 64u;      // columns per lane and part
    constexpr uint32_t kRows = kTileM / 64u;            // rows per lane and part
    float scale[kColumns];
    __half bias[kColumns];
    float a_scale[kRows];
#pragma unroll
    for (uint32_t i = 0; i < kColumns; ++i) {
        const uint32_t j = part * (kMaxTileN / 2u) + lane + 32u * i;
        const uint32_t local = (geglu && j >= half) ? j - half : j;
        const bool valid = j < tile_n && n0 + local < tile.n_out;
        const uint32_t column = (geglu && j >= half) ? tile.n_out + n0 + local : n0 + local;
        scale[i] = 0.0f;
        bias[i] = __half(0);
        if (valid) {
            scale[i] = scaled ? __ldg(tile.w_scales + (per_channel ? column : 0u)) : 1.0f;
            if (has_bias) bias[i] = tile.bias[column];
        }
    }
#pragma unroll
    for (uint32_t i = 0; i < kRows; ++i) {
        const uint32_t r = part * (kTileM / 2u) + lane + 32u * i;
        a_scale[i] = 1.0f;
        if (tile.kind == KIND_I8) a_scale[i] = first_row + r < tile.m ? __ldg(tile.a_scales + first_row + r) : 0.0f;
        else if (tile.kind != KIND_F16) a_scale[i] = __ldg(tile.a_scales);
    }
#pragma unroll
    for (uint32_t i = 0; i < kColumns; ++i) {
        const uint32_t j = part * (kMaxTileN / 2u) + lane + 32u * i;
        control->column_scale[slot][j] = scale[i];
        control->column_bias[slot][j] = __half2float(bias[i]);
        control->column_bias_half[slot][j] = bias[i];
    }
#pragma unroll
    for (uint32_t i = 0; i < kRows; ++i) control->row_scale[slot][part * (kTileM / 2u) + lane + 32u * i] = a_scale[i];
    if (part == 0 && lane == 0) control->header[slot] = tile;
}

__device__ __forceinline__ __half packed_half(const uint32_t word, int index) {
    return __ushort_as_half(static_cast<unsigned short>(index == 0 ? (word & 0xFFFFu) : (word >> 16)));
}

// 16 FP16 results of one output row, packed two per word -> global memory. `wide` (row pitch and
// base 32-byte aligned) writes the 32 bytes with one 256-bit store so that each lane fills a
// whole memory sector; `vector_ok` (16-byte aligned) uses two 128-bit stores.
__device__ __forceinline__ void store_row_16(__half* y, uint32_t n_out, bool vector_ok, bool wide, uint32_t row,
                                             uint32_t col0, const uint32_t (&words)[8]) {
    __half* destination = y + static_cast<size_t>(row) * n_out + col0;
    if (col0 + 16 <= n_out && wide) {
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(destination), "r"(words[0]),
                     "r"(words[1]), "r"(words[2]), "r"(words[3]), "r"(words[4]), "r"(words[5]), "r"(words[6]),
                     "r"(words[7])
                     : "memory");
    } else if (col0 + 16 <= n_out && vector_ok) {
        reinterpret_cast<uint4*>(destination)[0] = make_uint4(words[0], words[1], words[2], words[3]);
        reinterpret_cast<uint4*>(destination)[1] = make_uint4(words[4], words[5], words[6], words[7]);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (col0 + i < n_out) destination[i] = packed_half(words[i >> 1], i & 1);
        }
    }
}

// The 16 residual values that belong to one row's 16 outputs (packed two per word), loaded the way
// store_row_16 writes them: one 256-bit load, two 128-bit loads, or element by element at the edge.
__device__ __forceinline__ void load_row_16(const __half* source, uint32_t n_out, bool vector_ok, bool wide,
                                            uint32_t row, uint32_t col0, uint32_t (&words)[8]) {
    const __half* address = source + static_cast<size_t>(row) * n_out + col0;
    if (col0 + 16 <= n_out && wide) {
        asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(words[0]), "=r"(words[1]), "=r"(words[2]), "=r"(words[3]), "=r"(words[4]), "=r"(words[5]),
                       "=r"(words[6]), "=r"(words[7])
                     : "l"(address)
                     : "memory");
    } else if (col0 + 16 <= n_out && vector_ok) {
        const uint4 lo = reinterpret_cast<const uint4*>(address)[0];
        const uint4 hi = reinterpret_cast<const uint4*>(address)[1];
        words[0] = lo.x; words[1] = lo.y; words[2] = lo.z; words[3] = lo.w;
        words[4] = hi.x; words[5] = hi.y; words[6] = hi.z; words[7] = hi.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t lo = col0 + 2 * i < n_out ? __half_as_ushort(address[2 * i]) : 0u;
            const uint32_t hi = col0 + 2 * i + 1 < n_out ? __half_as_ushort(address[2 * i + 1]) : 0u;
            words[i] = lo | (hi << 16);
        }
    }
}

// Reads W consecutive staged FP32 values starting at column j0 (a multiple of 4) with 16-byte
// loads, as W / 2 pairs.
template <int W>
__device__ __forceinline__ void read_staged(const float* values, uint32_t j0, float2 (&out)[W / 2]) {
#pragma unroll
    for (int i = 0; i < W / 4; ++i) {
        const float4 v = *reinterpret_cast<const float4*>(values + j0 + 4 * i);
        out[2 * i] = make_float2(v.x, v.y);
        out[2 * i + 1] = make_float2(v.z, v.w);
    }
}

// W staged FP16 values, packed two per word.
template <int W>
__device__ __forceinline__ void read_staged_half(const __half* values, uint32_t j0, uint32_t (&out)[W / 2]) {
#pragma unroll
    for (int i = 0; i < W / 8; ++i) {
        const uint4 v = *reinterpret_cast<const uint4*>(values + j0 + 8 * i);
        out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w;
    }
}

// Two accumulators scaled to the projection values before their FP16 rounding:
// (acc * a_scale) * w_scale with both products rounded to FP32, as the reference's dequantisation
// computes them, here on the packed FP32 pipe (each half rounds like the scalar multiply).
template <uint32_t Kind>
__device__ __forceinline__ float2 dequantise2(uint32_t acc0, uint32_t acc1, float2 a_scale, float2 w_scale) {
    if (Kind == KIND_F16) return make_float2(__uint_as_float(acc0), __uint_as_float(acc1));
    const float2 raw = Kind == KIND_I8
                           ? make_float2(static_cast<float>(static_cast<int32_t>(acc0)), static_cast<float>(static_cast<int32_t>(acc1)))
                           : make_float2(__uint_as_float(acc0), __uint_as_float(acc1));
    return __fmul2_rn(__fmul2_rn(raw, a_scale), w_scale);
}

// Two FP32 values -> two FP16 values in one word (round to nearest even), .x in the low half.
__device__ __forceinline__ uint32_t to_half2_bits(float2 v) {
    const __half2 packed = __float22half2_rn(v);
    return *reinterpret_cast<const uint32_t*>(&packed);
}

__device__ __forceinline__ float2 from_half2_bits(uint32_t word) {
    return __half22float2(*reinterpret_cast<const __half2*>(&word));
}

// Everything one epilogue warp needs for its share of a tile, passed by value to the
// out-of-line epilogue variants.
struct EpilogueTile {
    __half* y;
    int32_t* acc_out;
    const __half* residual;         // [M, n_out] added after the bias, or null (may alias y)
    uint32_t* amax_out;             // word that receives max |y| of the problem's output, or null
    const float* column_scale;      // shared memory
    const float* column_bias;       // shared memory, FP32
    const __half* column_bias_half; // shared memory, FP16
    float a_scale;
    uint32_t n, n_out;
    uint32_t tile_n, n0;            // accumulator columns of the tile; first output column
    uint32_t row, tmem_row;
    uint32_t chunk_first;           // which of the warps of this TMEM lane quadrant
    uint32_t activation;            // Activation (read by the run-time activation variant)
    uint32_t flags;                 // bit 0 row in range, bit 1 has bias, bit 2 16-byte stores, bit 3 32-byte stores
                                    // (bits 4-8: tuning switches of the diagnostics build)
};

// 16 accumulator columns of one row -> 16 FP16 outputs (no GEGLU): dequantise, bias, activation.
// Act is ACT_NONE, ACT_GEGLU or kActRuntime (SiLU / GELU / QuickGELU chosen by t.activation at
// run time: the rare activations share one instance of the code).
constexpr uint32_t kActRuntime = 99;

template <uint32_t Kind, uint32_t Act>
__device__ __forceinline__ void finish_chunk_16(const EpilogueTile& t, uint32_t c0, const uint32_t (&acc)[16],
                                                float2 a_scale, bool has_bias, uint32_t (&out_words)[8]) {
    float2 w_scale[8];
    read_staged<16>(t.column_scale, c0, w_scale);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        out_words[i] = to_half2_bits(dequantise2<Kind>(acc[2 * i], acc[2 * i + 1], a_scale, w_scale[i]));
    }
    if (has_bias) {
        if (Act == ACT_NONE) {
            uint32_t bias_words[8];
            read_staged_half<16>(t.column_bias_half, c0, bias_words);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const __half2 sum = __hadd2(*reinterpret_cast<const __half2*>(&out_words[i]),
                                            *reinterpret_cast<const __half2*>(&bias_words[i]));
                out_words[i] = *reinterpret_cast<const uint32_t*>(&sum);
            }
        } else {
            float2 bias[8];
            read_staged<16>(t.column_bias, c0, bias);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 x = __fadd2_rn(from_half2_bits(out_words[i]), bias[i]);
                out_words[i] = to_half2_bits(t.activation == ACT_GELU
                                                 ? gelu_erf2(x)
                                                 : make_float2(activate(x.x, t.activation), activate(x.y, t.activation)));
            }
        }
    }
}

// 8 value and 8 gate accumulator columns of one row -> 8 FP16 GEGLU outputs (4 words).
template <uint32_t Kind>
__device__ __forceinline__ void finish_geglu_8(const EpilogueTile& t, uint32_t c, uint32_t half,
                                               const uint32_t (&acc_value)[8], const uint32_t (&acc_gate)[8],
                                               float2 a_scale, uint32_t* out_words) {
    float2 w_value[4], w_gate[4], b_value[4], b_gate[4];
    read_staged<8>(t.column_scale, c, w_value);
    read_staged<8>(t.column_scale, half + c, w_gate);
    read_staged<8>(t.column_bias, c, b_value);
    read_staged<8>(t.column_bias, half + c, b_gate);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // both projections are rounded to FP16 before the bias is added in FP32
        const float2 value = __fadd2_rn(
            from_half2_bits(to_half2_bits(dequantise2<Kind>(acc_value[2 * i], acc_value[2 * i + 1], a_scale, w_value[i]))),
            b_value[i]);
        const float2 gate = __fadd2_rn(
            from_half2_bits(to_half2_bits(dequantise2<Kind>(acc_gate[2 * i], acc_gate[2 * i + 1], a_scale, w_gate[i]))),
            b_gate[i]);
        out_words[i] = to_half2_bits(__fmul2_rn(value, gelu_erf2(gate)));
    }
}

// Drains this warp's share of one accumulator tile in chunks of 16 output columns (the warps of a TMEM
// lane quadrant take the chunks round-robin): tensor-memory load, wait, finish (dequantise, bias,
// activation), store, one chunk at a time, one output row per lane.
//
// Measured on B200 with parts of this function switched off (tuning build, 128 x 256 INT8 tiles, K = 640,
// main loop running): about 6000 cycles per tile, of which the stores account for 1900, the arithmetic
// for 1000 and the tensor-memory loads for nothing. Measured slower or no faster, same GPU, same run:
//  * a software-pipelined form (next chunk's load in flight while the current one is finished: larger
//    code, 7 % slower);
//  * swapping chunks between the four lanes of a quad with register shuffles so that every store writes
//    128 contiguous bytes per row (the shuffles and selects cost more issue slots than the stores save:
//    10 % slower);
//  * bulk tensor stores through shared memory, as 32-byte boxes per chunk (slower) and as 64-byte boxes
//    per pair of chunks with the 64-byte swizzle (conflict-free staging, a quarter of the store requests:
//    the same time within 2 %, 20 % slower on 128-column tiles) -- the cost of the stores is not the
//    load/store unit's transaction count;
//  * 12 or 16 epilogue warps (the time per tile does not change: the epilogue is not latency-bound
//    per warp);
//  * a second instance of the two hot variants for interior tiles, with the edge handling, the narrow
//    stores and the accumulator dump compiled out: 2 to 6 % faster on single K = 640 GEGLU projections,
//    9 % SLOWER on the UNet loop's projections as a whole (same GPU, same run), so it was taken out;
//  * kernels compiled for one activation as well as one operand class: no change.
// Also measured without gain (launch set-up rather than epilogue): the producer requesting the weight tiles of
// its first stages before griddepcontrol.wait and the activation tiles after it (18.40 against 18.27 ms per
// step at one image per GPU, no change at eight).
// Kind: 0 INT8, 1 FP8 (either format), 3 FP16.
// Arithmetic per output, as the reference runs it after the GEMM:
//   y = half_rn(dequantised accumulator)
//   no activation : __hadd(y, bias), then __hadd(.., residual)  (add_last_dim_bias_kernel, add_in_place_kernel)
//   SiLU/GELU/QuickGELU : half_rn(act(float(y) + float(bias))) (bias_activation_in_place_kernel)
//   GEGLU : half_rn((float(y_v) + float(b_v)) * gelu(float(y_g) + float(b_g)))   (bias_geglu_kernel)
template <uint32_t Kind, uint32_t Act>
__device__ __forceinline__ void epilogue_tile(const EpilogueTile& t) {
    const bool row_ok = (t.flags & 1u) != 0;
    const bool has_bias = (t.flags & 2u) != 0;
    const bool store_vector = (t.flags & 4u) != 0;
    const bool store_wide = (t.flags & 8u) != 0;
    const float2 a_scale = make_float2(t.a_scale, t.a_scale);
    int32_t* const acc_out = Kind == KIND_I8 ? t.acc_out : nullptr;
    constexpr uint32_t kStride = kWarpsPerQuadrant * 16u;
#ifdef SDXLQ_DIAGNOSTICS
    // tuning build: parts of the epilogue can be switched off to time the others
    const bool no_store = (t.flags & 16u) != 0, no_load = (t.flags & 32u) != 0, no_math = (t.flags & 64u) != 0;
    if ((t.flags & 128u) != 0) return;                      // nothing at all
    const uint32_t diag_limit = (t.flags & 256u) != 0 ? 32u : 0xFFFFFFFFu;     // one chunk per warp only
#else
    constexpr bool no_store = false, no_load = false, no_math = false;
    constexpr uint32_t diag_limit = 0xFFFFFFFFu;
#endif
    const uint32_t columns = Act == ACT_GEGLU ? t.tile_n / 2u : t.tile_n;        // output columns of the tile
    const uint32_t limit = min(diag_limit, min(columns, t.n_out > t.n0 ? t.n_out - t.n0 : 0u));
    const __half* const residual = Act == ACT_NONE ? t.residual : nullptr;
    const bool with_residual = residual != nullptr && row_ok;
    // max |y| over this lane's outputs of the tile, for the FP8 quantiser of the projection that reads y
    const bool want_amax = t.amax_out != nullptr;
    __half2 running_max = __float2half2_rn(0.0f);

    for (uint32_t c = t.chunk_first * 16u; c < limit; c += kStride) {
        const uint32_t col0 = t.n0 + c;
        uint32_t out_words[8];
        if (Act != ACT_GEGLU) {
            uint32_t acc[16];
            uint32_t extra[8] = {};
            if (no_load) {
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[i] = c + t.row + static_cast<uint32_t>(i);
            } else {
                ptx::tmem_ld_32x32b_x16(t.tmem_row + c, acc);
            }
            if (with_residual) load_row_16(residual, t.n_out, store_vector, store_wide, t.row, col0, extra);
            if (!no_load) ptx::tmem_ld_wait(acc);
            if (acc_out != nullptr && row_ok) {
                int32_t* raw = acc_out + static_cast<size_t>(t.row) * t.n + col0;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (col0 + i < t.n) raw[i] = static_cast<int32_t>(acc[i]);
                }
            }
            if (no_math) {
#pragma unroll
                for (int i = 0; i < 8; ++i) out_words[i] = acc[2 * i] ^ acc[2 * i + 1];
            } else {
                finish_chunk_16<Kind, Act>(t, c, acc, a_scale, has_bias, out_words);
            }
            if (Act == ACT_NONE && with_residual) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const __half2 sum = __hadd2(*reinterpret_cast<const __half2*>(&out_words[i]),
                                                *reinterpret_cast<const __half2*>(&extra[i]));
                    out_words[i] = *reinterpret_cast<const uint32_t*>(&sum);
                }
            }
        } else {
            const uint32_t half = t.tile_n / 2u;
#pragma unroll
            for (uint32_t step = 0; step < 2; ++step) {
                uint32_t value[8], gate[8];
                ptx::tmem_ld_32x32b_x8(t.tmem_row + c + 8u * step, value);
                ptx::tmem_ld_32x32b_x8(t.tmem_row + half + c + 8u * step, gate);
                ptx::tmem_ld_wait(value, gate);
                if (acc_out != nullptr && row_ok) {
                    int32_t* raw = acc_out + static_cast<size_t>(t.row) * t.n;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        if (col0 + 8u * step + i < t.n_out) {
                            raw[col0 + 8u * step + i] = static_cast<int32_t>(value[i]);
                            raw[t.n_out + col0 + 8u * step + i] = static_cast<int32_t>(gate[i]);
                        }
                    }
                }
                finish_geglu_8<Kind>(t, c + 8u * step, half, value, gate, a_scale, out_words + 4 * step);
            }
        }
        if (row_ok && (!no_store || (out_words[0] == 0x7E57C0DEu && out_words[7] == 0x7E57C0DEu))) {
            store_row_16(t.y, t.n_out, store_vector, store_wide, t.row, col0, out_words);
        }
        if (want_amax && row_ok) {
            // columns past the matrix edge hold zeros (scale 0, bias 0), so they cannot win the maximum
#pragma unroll
            for (int i = 0; i < 8; ++i) running_max = __hmax2(running_max, __habs2(*reinterpret_cast<const __half2*>(&out_words[i])));
        }
    }
    if (want_amax) {
        float maximum = fmaxf(__low2float(running_max), __high2float(running_max));
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, offset));
        if ((threadIdx.x & 31u) == 0 && maximum > 0.0f) atomicMax(t.amax_out, __float_as_uint(maximum));
    }
}

template <uint32_t Kind>
__device__ __forceinline__ void epilogue_dispatch(uint32_t activation, const EpilogueTile& t) {
    if (activation == ACT_NONE) epilogue_tile<Kind, ACT_NONE>(t);
    else if (activation == ACT_GEGLU) epilogue_tile<Kind, ACT_GEGLU>(t);
    else epilogue_tile<Kind, kActRuntime>(t);
}

}  // namespace

// Where the MMA issuer stands in the ring of pipeline stages, plus the loop constants.
struct MmaCursor {
    uint32_t stage, phase, num_stages;
    uint32_t full_base, empty_base;     // shared-memory addresses of full[0] / empty[0]
    uint32_t peer_empty_base;           // CTA pairs: empty[0] of the peer CTA as a shared::cluster address
    uint32_t a_lo_base;                 // descriptor low word of stage 0's A tile
    uint32_t stage_units, b_units;      // stage size and B offset in descriptor units (16 bytes)
    volatile uint32_t* abort_word;
    long long limit;
    uint32_t mode;                      // diagnostics: bit 0 no MMAs, bit 1 one MMA per stage
};

// Issues the MMAs of one tile: k_blocks stages of four MMAs each, into the accumulator at tmem_d.
// Returns false when a wait for a full stage ran out.
template <int KindTag, bool kPair>
__device__ __forceinline__ bool issue_tile_mmas(MmaCursor& c, uint32_t tmem_d, uint32_t idesc, uint32_t k_blocks) {
    uint32_t stage = c.stage, phase = c.phase;
    uint32_t accumulate = 0;
    for (uint32_t kb = 0; kb < k_blocks; ++kb) {
        if (!ptx::mbar_wait_bounded(c.full_base + stage * 8u, phase, c.abort_word, c.limit)) return false;
        ptx::tc_fence_after();
        const uint32_t a_lo = c.a_lo_base + stage * c.stage_units;
        if (c.mode == 0) {
            ptx::umma_stage<KindTag, kPair>(tmem_d, a_lo, a_lo + c.b_units, ptx::kUmmaDescHiSw128, idesc, accumulate);
        } else if (c.mode == 2 && KindTag != 0) {   // the one-MMA diagnostic exists for INT8 only
            ptx::umma_stage<KindTag, kPair>(tmem_d, a_lo, a_lo + c.b_units, ptx::kUmmaDescHiSw128, idesc, accumulate);
        } else if (c.mode == 2) {
            const uint64_t hi = static_cast<uint64_t>(ptx::kUmmaDescHiSw128) << 32;
            if (kPair) ptx::umma_i8_pair(tmem_d, hi | a_lo, hi | (a_lo + c.b_units), idesc, accumulate);
            else ptx::umma_i8(tmem_d, hi | a_lo, hi | (a_lo + c.b_units), idesc, accumulate);
        }
        accumulate = 1;
        const uint32_t empty_bar = c.empty_base + stage * 8u;
        if (kPair) {
            ptx::umma_commit_pair(empty_bar);                                 // frees the leader's stage
            ptx::umma_commit_pair(c.peer_empty_base + stage * 8u);            // and the peer's
        } else {
            ptx::umma_commit(empty_bar);
        }
        if (++stage == c.num_stages) { stage = 0; phase ^= 1u; }
    }
    c.stage = stage;
    c.phase = phase;
    return true;
}

// kPair = false: one CTA per 128-row tile (cta_group::1).
// kPair = true : a cluster of two CTAs per 256-row tile (cta_group::2). Each CTA loads its own 128
//   rows of A and half of the tile's B rows (for GEGLU: the leader the value rows, its peer the
//   gate rows); the leader's elected thread issues M=256 MMAs that read both CTAs' shared memory
//   and write 128 accumulator rows into each CTA's tensor memory. Every TMA load of the pair counts
//   on the leader's full barrier; the MMA completion is committed to both CTAs' empty / acc_full
//   barriers; both CTAs' epilogue warps arrive on the leader's acc_empty barriers.
//
// kClass fixes the operand class of every problem of the launch at compile time (0 INT8, 1 FP8, 2 FP16;
// the host picks the instance when all problems agree, which is every launch of one precision
// profile), so that the issuer and the epilogue warps carry one arithmetic variant instead of three;
// -1 keeps the per-tile switch for mixed launches.
template <bool kPair, int kClass>
__global__ void __launch_bounds__(kThreads, 1)
sdxlq_umma_gemm_kernel(const __grid_constant__ GemmLaunchParams params) {
    extern __shared__ __align__(128) uint8_t dynamic_smem[];
    Control* control = reinterpret_cast<Control*>(dynamic_smem);
    const uint32_t stages_base = (ptx::smem_u32(dynamic_smem) + sizeof(Control) + 1023u) & ~1023u;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t num_stages = params.num_stages;
    const uint32_t stage_bytes = params.stage_bytes;
    const uint32_t b_offset = params.b_offset;
    const uint32_t num_tiles = params.num_tiles;
    volatile uint32_t* abort_word = &control->abort;
    const long long limit = params.wait_limit_cycles;
#ifndef SDXLQ_DIAGNOSTICS
    // regular build: the tuning switches do not exist and the hot loops carry no tests for them
    // (1.5 % of the kernel time); build with -DSDXLQ_DIAGNOSTICS to get them
    constexpr bool skip_epilogue = false, skip_loads = false, skip_mma = false, one_mma_per_stage = false,
                   a_loads_only = false;
#else
    const bool skip_epilogue = (params.diagnostic_skip & 1u) != 0;
    const bool skip_loads = (params.diagnostic_skip & (2u | 4u)) != 0;
    const bool skip_mma = (params.diagnostic_skip & (2u | 8u)) != 0;
    const bool one_mma_per_stage = (params.diagnostic_skip & 32u) != 0;
    const bool a_loads_only = (params.diagnostic_skip & 64u) != 0;
#endif
    const uint32_t cta_rank = kPair ? ptx::cluster_cta_rank() : 0u;
    const bool leader = cta_rank == 0;
    const uint32_t first_tile = kPair ? blockIdx.x >> 1 : blockIdx.x;
    const uint32_t tile_stride = kPair ? gridDim.x >> 1 : gridDim.x;
    constexpr uint32_t kRowsPerTile = kPair ? 2 * kTileM : kTileM;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < num_stages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&control->full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&control->empty[s]), 1);
        }
        for (uint32_t b = 0; b < kAccQuarters; ++b) {
            ptx::mbar_init(ptx::smem_u32(&control->acc_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&control->acc_empty[b]), kPair ? 2 * kEpilogueWarps : kEpilogueWarps);
        }
        for (uint32_t b = 0; b < kSlots; ++b) {
            ptx::mbar_init(ptx::smem_u32(&control->staged[b]), 2);
            ptx::mbar_init(ptx::smem_u32(&control->slot_free[b]), kEpilogueWarps);
        }
        control->abort = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        if (kPair) {
            ptx::tmem_alloc_pair(ptx::smem_u32(&control->tmem_base), kTmemColumns);
            ptx::tmem_relinquish_pair();
        } else {
            ptx::tmem_alloc(ptx::smem_u32(&control->tmem_base), kTmemColumns);
            ptx::tmem_relinquish();
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (kPair) ptx::cluster_sync();          // the peer's barriers exist before anything signals them
    ptx::tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&control->tmem_base);

    // Everything above touched only this CTA's own state. From here on the roles read what the
    // kernels before this one wrote (quantised activations, their scales): wait for them to
    // complete when this grid was launched early; no effect otherwise.
    ptx::grid_dependency_wait();
    // ... and let the kernel behind this one (a quantiser, a LayerNorm) be scheduled: it fills the SMs as this
    // grid's CTAs leave them and waits for this grid's completion before it touches global memory.
    ptx::grid_launch_dependents();

    if (warp < kControlWarps) {
    ptx::setmaxnreg_dec<kControlRegisters>();
    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            uint32_t issued = 0;                     // stages handed to the copy engine so far
            const uint32_t full_base = ptx::smem_u32(&control->full[0]);
            const uint32_t empty_base = ptx::smem_u32(&control->empty[0]);
            const GemmProblem* bound = nullptr;
            bool ok = true;
            TileRef next = load_tile(params, first_tile);
            // diagnostic without loads: only the leader's arrivals count, its peer has nothing to do
            if (kPair && skip_loads && !leader) ok = false;
            for (uint32_t t = first_tile; ok && t < num_tiles; t += tile_stride) {
                const TileRef work = next;
                next = load_tile(params, t + tile_stride);      // in flight while this tile's loads are issued
                const GemmProblem* problem = tile_problem(params, work);
                const CUtensorMap* tmap_a = &problem->tmap_a;
                const CUtensorMap* tmap_b = &problem->tmap_b;
                if (params.problems != nullptr && problem != bound) {
                    ptx::fence_tensormap_acquire(tmap_a);
                    ptx::fence_tensormap_acquire(tmap_b);
                    bound = problem;
                }
                const bool geglu = work.activation == ACT_GEGLU;
                const uint32_t tile_n = work.tile_n;
                const uint32_t half = tile_n / 2;
                // bytes that land per stage, over both CTAs of a pair
                const uint32_t tx_bytes = (kPair ? 2 * kTileM + tile_n : kTileM + tile_n) * kTileKBytes;
                const int32_t k_step = (kClass < 0 ? work.kind == KIND_F16 : kClass == 2) ? 64 : 128;   // elements per stage
                const int32_t row_a = static_cast<int32_t>(work.tile_m * kRowsPerTile + cta_rank * kTileM);
                const int32_t row_b = static_cast<int32_t>(work.tile_n_index * (geglu ? half : tile_n));
                const int32_t row_gate = static_cast<int32_t>(work.n_out) + row_b;
                // pair: this CTA's half of the B rows (GEGLU: value rows in the leader, gate rows in the peer)
                const int32_t row_b_pair = geglu ? (leader ? row_b : row_gate)
                                                      : row_b + static_cast<int32_t>(cta_rank * half);
                // diagnostic without loads and MMAs: no stage hand-shakes either, the epilogue runs alone
                const uint32_t k_blocks = (skip_loads && skip_mma) ? 0u : work.k_blocks;
                int32_t k0 = 0;
                for (uint32_t kb = 0; kb < k_blocks; ++kb, k0 += k_step) {
                    if (!ptx::mbar_wait_bounded(empty_base + stage * 8u, phase ^ 1u, abort_word, limit)) {
                        raise_abort(control, params.error_word, DEV_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    const uint32_t full_bar = full_base + stage * 8u;
                    const uint32_t a_dst = stages_base + stage * stage_bytes;
                    const uint32_t b_dst = a_dst + b_offset;
                    if (skip_loads) {
                        if (leader) ptx::mbar_arrive(full_bar);
                    } else if (kPair) {
                        if (leader) ptx::mbar_expect_tx(full_bar, tx_bytes);
                        ptx::tma_load_2d_pair(a_dst, tmap_a, full_bar, k0, row_a);
                        ptx::tma_load_2d_pair(b_dst, tmap_b, full_bar, k0, row_b_pair);
                    } else if (a_loads_only) {      // diagnostic: half of the copy instructions, a third of the bytes
                        ptx::mbar_expect_tx(full_bar, kTileM * kTileKBytes);
                        ptx::tma_load_2d(a_dst, tmap_a, full_bar, k0, row_a);
                    } else {
                        ptx::mbar_expect_tx(full_bar, tx_bytes);
                        ptx::tma_load_2d(a_dst, tmap_a, full_bar, k0, row_a);
                        ptx::tma_load_2d(b_dst, tmap_b, full_bar, k0, row_b);
                        if (geglu) ptx::tma_load_2d(b_dst + half * kTileKBytes, tmap_b, full_bar, k0, row_gate);
                    }
                    ++issued;
                    if (++stage == num_stages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok && (!kPair || leader) && !skip_loads) {
                // Let the copies this thread started land before the CTA retires: the last
                // min(issued, num_stages) stages may still be in flight.
                const uint32_t pending = min(issued, num_stages);
                for (uint32_t i = issued - pending; i < issued; ++i) {
                    (void)ptx::mbar_wait_bounded(full_base + (i % num_stages) * 8u, (i / num_stages) & 1u, abort_word,
                                                 limit >> 4);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer ---------------------------------------
        // One thread issues every MMA of the CTA (of the pair). Its loop is the critical path of
        // the kernel: per stage it runs one barrier poll, one fence, one statement with the four
        // MMAs and one commit, all on 32-bit values kept in registers.
        if (lane == 0 && leader) {
            MmaCursor cursor;
            cursor.stage = 0;
            cursor.phase = 0;
            cursor.num_stages = num_stages;
            cursor.full_base = ptx::smem_u32(&control->full[0]);
            cursor.empty_base = ptx::smem_u32(&control->empty[0]);
            cursor.peer_empty_base = kPair ? ptx::map_to_cta(cursor.empty_base, 1) : 0u;
            cursor.a_lo_base = ptx::umma_desc_lo(stages_base);
            cursor.stage_units = stage_bytes >> 4;
            cursor.b_units = b_offset >> 4;
            cursor.abort_word = abort_word;
            cursor.limit = limit;
            cursor.mode = (skip_mma ? 1u : 0u) | (one_mma_per_stage ? 2u : 0u);
            AccumulatorRing ring;
            bool ok = true;
            DIAG_DECL(diag_acc_empty_wait); DIAG_DECL(diag_issue);
#ifdef SDXLQ_DIAGNOSTICS
            const long long diag_begin = clock64();
#endif
            TileRef next = load_tile(params, first_tile);
            for (uint32_t t = first_tile; ok && t < num_tiles; t += tile_stride) {
                const TileRef work = next;
                next = load_tile(params, t + tile_stride);      // in flight while this tile's MMAs are issued
                uint32_t quarters;
                const uint32_t first_quarter = ring.place(work.tile_n, quarters);
#ifdef SDXLQ_DIAGNOSTICS
                const long long diag_t_wait = clock64();
#endif
                for (uint32_t q = first_quarter; ok && q < first_quarter + quarters; ++q) {
                    // the quarter's previous user (if any) has been drained by every epilogue warp
                    ok = ptx::mbar_wait_bounded(ptx::smem_u32(&control->acc_empty[q]), ((ring.parity >> q) & 1u) ^ 1u,
                                                abort_word, limit);
                    ring.parity ^= 1u << q;
                }
#ifdef SDXLQ_DIAGNOSTICS
                const long long diag_t_issue = clock64();
                diag_acc_empty_wait += diag_t_issue - diag_t_wait;
#endif
                if (!ok) {
                    raise_abort(control, params.error_word, DEV_TIMEOUT_MMA);
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t tmem_d = tmem_base + first_quarter * kQuarterColumns;
                const uint32_t k_blocks = (skip_loads && skip_mma) ? 0u : work.k_blocks;
                if constexpr (kClass >= 0) {
                    ok = issue_tile_mmas<kClass, kPair>(cursor, tmem_d, work.idesc, k_blocks);
                } else {
                    if (work.kind == KIND_I8) ok = issue_tile_mmas<0, kPair>(cursor, tmem_d, work.idesc, k_blocks);
                    else if (work.kind == KIND_F16) ok = issue_tile_mmas<2, kPair>(cursor, tmem_d, work.idesc, k_blocks);
                    else ok = issue_tile_mmas<1, kPair>(cursor, tmem_d, work.idesc, k_blocks);
                }
                if (!ok) {
                    raise_abort(control, params.error_word, DEV_TIMEOUT_MMA + 1);
                    break;
                }
                const uint32_t full_bar = ptx::smem_u32(&control->acc_full[first_quarter]);
                if (kPair) {
                    ptx::umma_commit_pair(full_bar);
                    ptx::umma_commit_pair(ptx::map_to_cta(full_bar, 1));
                } else {
                    ptx::umma_commit(full_bar);
                }
#ifdef SDXLQ_DIAGNOSTICS
                diag_issue += clock64() - diag_t_issue;
#endif
            }
#ifdef SDXLQ_DIAGNOSTICS
            DIAG_WRITE(4, diag_acc_empty_wait); DIAG_WRITE(5, diag_issue); DIAG_WRITE(6, clock64() - diag_begin);
#endif
        }
    } else {
        // ------------------------------- stagers (warps 2 and 3) ---------------------------
        // Fill the epilogue's operand slot of each tile (tile record, row scales, column scales
        // and bias) while the tile's main loop runs, up to kSlots tiles ahead of the epilogue.
        uint32_t iteration = 0;
        DIAG_DECL(diag_slot_wait); DIAG_DECL(diag_stage); DIAG_DECL(diag_total);
#ifdef SDXLQ_DIAGNOSTICS
        const long long diag_begin = clock64();
#endif
        TileRef next = load_tile(params, first_tile);
        for (uint32_t t = first_tile; t < num_tiles; t += tile_stride, ++iteration) {
            const TileRef work = next;
            next = load_tile(params, t + tile_stride);
            const uint32_t slot = iteration % kSlots;
            uint32_t ok = 1;
            DIAG_ADD(diag_slot_wait,
            if (lane == 0) {
                ok = ptx::mbar_wait_bounded(ptx::smem_u32(&control->slot_free[slot]), ((iteration / kSlots) & 1u) ^ 1u,
                                            abort_word, limit) ? 1u : 0u;
                if (ok == 0) raise_abort(control, params.error_word, DEV_TIMEOUT_EPILOGUE + 1);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0));
            if (ok == 0) break;
            DIAG_ADD(diag_stage,
            stage_tile(work, work.tile_m * kRowsPerTile + cta_rank * kTileM, lane, warp - 2u, control, slot);
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&control->staged[slot])));
        }
#ifdef SDXLQ_DIAGNOSTICS
        diag_total = clock64() - diag_begin;
        if (warp == 2 && lane == 0) { DIAG_WRITE(0, diag_slot_wait); DIAG_WRITE(1, diag_stage); DIAG_WRITE(2, diag_total); DIAG_WRITE(3, iteration); }
#endif
    }
    } else {
        // ------------------------------- epilogue ------------------------------------------
        ptx::setmaxnreg_inc<kEpilogueRegisters>();
        // Warp w may touch TMEM lanes 32*(w % 4) .. +31. The warps of a quadrant take the column
        // chunks of the tile round-robin.
        const uint32_t quadrant = warp & 3u;
        const uint32_t chunk_first = (warp - kControlWarps) >> 2;      // 0 .. kWarpsPerQuadrant - 1
        const uint32_t row_in_cta = quadrant * 32u + lane;
        AccumulatorRing ring;
        uint32_t iteration = 0;
        DIAG_DECL(diag_staged_wait); DIAG_DECL(diag_acc_wait); DIAG_DECL(diag_work); DIAG_DECL(diag_setup); DIAG_DECL(diag_tail);
#ifdef SDXLQ_DIAGNOSTICS
        const long long diag_begin = clock64();
#endif
        for (uint32_t t = first_tile; t < num_tiles; t += tile_stride, ++iteration) {
            const uint32_t buffer = iteration % kSlots;
#ifdef SDXLQ_DIAGNOSTICS
            const long long diag_t_staged = clock64();
#endif
            if (!ptx::mbar_wait_bounded(ptx::smem_u32(&control->staged[buffer]), (iteration / kSlots) & 1u, abort_word, limit)) {
                raise_abort(control, params.error_word, DEV_TIMEOUT_EPILOGUE);
                break;
            }
#ifdef SDXLQ_DIAGNOSTICS
            const long long diag_t_setup = clock64();
            diag_staged_wait += diag_t_setup - diag_t_staged;
#endif
            const TileRef& work = control->header[buffer];
            const uint32_t tile_n = work.tile_n;
            const uint32_t activation = work.activation;
            const uint32_t kind = work.kind;
            const uint32_t flags = work.flags;
            EpilogueTile tile;
            tile.y = work.y;
            tile.acc_out = nullptr;
            if ((flags & TILE_RAW_ACCUMULATORS) != 0) tile.acc_out = tile_problem(params, work)->ep.acc_out;
            tile.residual = nullptr;
            if ((flags & TILE_HAS_RESIDUAL) != 0) tile.residual = tile_problem(params, work)->ep.residual;
            tile.amax_out = nullptr;
            if ((flags & TILE_OUTPUT_AMAX) != 0) tile.amax_out = tile_problem(params, work)->ep.y_amax;
            tile.column_scale = control->column_scale[buffer];
            tile.column_bias = control->column_bias[buffer];
            tile.column_bias_half = control->column_bias_half[buffer];
            tile.n = work.n;
            tile.n_out = work.n_out;
            tile.tile_n = tile_n;
            tile.n0 = work.tile_n_index * (activation == ACT_GEGLU ? tile_n / 2u : tile_n);
            tile.row = work.tile_m * kRowsPerTile + cta_rank * kTileM + row_in_cta;
            uint32_t quarters;
            const uint32_t first_quarter = ring.place(tile_n, quarters);
            tile.tmem_row = tmem_base + ((quadrant * 32u) << 16) + first_quarter * kQuarterColumns;
            tile.chunk_first = chunk_first;
            tile.activation = activation;
            tile.flags = (tile.row < work.m ? 1u : 0u) | ((flags & TILE_HAS_BIAS) != 0 ? 2u : 0u) |
                         ((flags & TILE_STORE_16) != 0 ? 4u : 0u) | ((flags & TILE_STORE_32) != 0 ? 8u : 0u);
#ifdef SDXLQ_DIAGNOSTICS
            tile.flags |= ((params.diagnostic_skip >> 7) & 31u) << 4;    // 128 no stores, 256 no accumulator loads, 512 no arithmetic,
                                                                         // 1024 empty epilogue function, 2048 one chunk per warp
#endif
            tile.a_scale = control->row_scale[buffer][row_in_cta];
#ifdef SDXLQ_DIAGNOSTICS
            const long long diag_t_acc = clock64();
            diag_setup += diag_t_acc - diag_t_setup;
#endif
            if (!ptx::mbar_wait_bounded(ptx::smem_u32(&control->acc_full[first_quarter]), (ring.parity >> first_quarter) & 1u,
                                        abort_word, limit)) {
                raise_abort(control, params.error_word, DEV_TIMEOUT_EPILOGUE);
                break;
            }
            ring.parity ^= 1u << first_quarter;
            ptx::tc_fence_after();
#ifdef SDXLQ_DIAGNOSTICS
            const long long diag_t_work = clock64();
            diag_acc_wait += diag_t_work - diag_t_acc;
#endif
            if (skip_epilogue) { /* diagnostic: accumulators are dropped */ }
            else if constexpr (kClass == 0) epilogue_dispatch<KIND_I8>(activation, tile);
            else if constexpr (kClass == 1) epilogue_dispatch<KIND_E4M3>(activation, tile);
            else if constexpr (kClass == 2) epilogue_dispatch<KIND_F16>(activation, tile);
            else if (kind == KIND_I8) epilogue_dispatch<KIND_I8>(activation, tile);
            else if (kind == KIND_F16) epilogue_dispatch<KIND_F16>(activation, tile);
            else epilogue_dispatch<KIND_E4M3>(activation, tile);
#ifdef SDXLQ_DIAGNOSTICS
            const long long diag_t_tail = clock64();
            diag_work += diag_t_tail - diag_t_work;
#endif
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                for (uint32_t q = first_quarter; q < first_quarter + quarters; ++q) {
                    const uint32_t empty_bar = ptx::smem_u32(&control->acc_empty[q]);
                    if (kPair) ptx::mbar_arrive_cluster(empty_bar & ptx::kPeerBitMask);   // the leader's barrier
                    else ptx::mbar_arrive(empty_bar);
                }
                ptx::mbar_arrive(ptx::smem_u32(&control->slot_free[buffer]));
            }
#ifdef SDXLQ_DIAGNOSTICS
            diag_tail += clock64() - diag_t_tail;
#endif
        }
#ifdef SDXLQ_DIAGNOSTICS
        if (warp == kControlWarps && lane == 0) {
            DIAG_WRITE(8, diag_staged_wait); DIAG_WRITE(9, diag_setup); DIAG_WRITE(10, diag_acc_wait); DIAG_WRITE(11, diag_work);
            DIAG_WRITE(12, diag_tail); DIAG_WRITE(13, clock64() - diag_begin); DIAG_WRITE(14, iteration);
        }
#endif
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (kPair) ptx::cluster_sync();          // neither CTA retires while its peer may still touch it
    if (warp == 1) {
        ptx::tc_fence_after();
        if (kPair) ptx::tmem_dealloc_pair(tmem_base, kTmemColumns);
        else ptx::tmem_dealloc(tmem_base, kTmemColumns);
    }
}

// Failure-detection probe: one thread waits, with a limit, on a barrier that nothing signals;
// the wait runs out, the timeout code is recorded and the kernel returns normally.
__global__ void sdxlq_bounded_wait_probe_kernel(uint32_t* error_word, long long limit_cycles) {
    __shared__ uint64_t barrier;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&barrier), 1);
        abort_flag = 0;
        ptx::fence_mbar_init();
        if (!ptx::mbar_wait_bounded(ptx::smem_u32(&barrier), 0, &abort_flag, limit_cycles)) {
            atomicCAS(error_word, 0u, static_cast<uint32_t>(DEV_TIMEOUT_EPILOGUE) + 0x80u);
        }
    }
}

cudaError_t launch_bounded_wait_probe(uint32_t* error_word, long long limit_cycles, cudaStream_t stream) {
    sdxlq_bounded_wait_probe_kernel<<<1, 32, 0, stream>>>(error_word, limit_cycles);
    return cudaGetLastError();
}

// Shared memory in front of the pipeline stages: the control block plus the slack needed to align
// the first stage to 1024 bytes.
size_t umma_gemm_control_bytes() { return (sizeof(Control) + 1023u + 1023u) / 1024u * 1024u; }

// Host-side launcher (called from the dispatch code). `grid` counts CTAs (even for the CTA-pair
// flavour, which is launched as clusters of two). The opt-in to more than 48 KB of dynamic shared
// memory is a per-device, process-wide property of the kernel, not of a context: both flavours are
// opted into the architectural maximum once per device, so that contexts with different tile
// geometries on one GPU cannot lower each other's limit. `operand_class` (0 INT8, 1 FP8, 2 FP16)
// selects the instance compiled for one operand class when every problem of the launch has it, -1
// the one that switches per tile.
cudaError_t launch_umma_gemm(const GemmLaunchParams& params, uint32_t grid, size_t dynamic_smem,
                             cudaStream_t stream, int device, bool pair, bool early_launch, int operand_class) {
    using Kernel = void (*)(GemmLaunchParams);
    static const Kernel kernels[2][4] = {
        {sdxlq_umma_gemm_kernel<false, -1>, sdxlq_umma_gemm_kernel<false, 0>, sdxlq_umma_gemm_kernel<false, 1>,
         sdxlq_umma_gemm_kernel<false, 2>},
        {sdxlq_umma_gemm_kernel<true, -1>, sdxlq_umma_gemm_kernel<true, 0>, sdxlq_umma_gemm_kernel<true, 1>,
         sdxlq_umma_gemm_kernel<true, 2>}};
    const int instance = (operand_class >= 0 && operand_class <= 2) ? operand_class + 1 : 0;
    const Kernel kernel = kernels[pair ? 1 : 0][instance];
    constexpr int kMaxDevices = 64;
    constexpr int kSharedMemoryOptIn = 232448;      // 227 KiB per CTA on sm_100
    static std::mutex opt_in_mutex;
    static bool opted_in[kMaxDevices][2][4] = {};
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    {
        std::lock_guard<std::mutex> lock(opt_in_mutex);
        if (!opted_in[device][pair ? 1 : 0][instance]) {
            const cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                            kSharedMemoryOptIn);
            if (status != cudaSuccess) return status;
            opted_in[device][pair ? 1 : 0][instance] = true;
        }
    }
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(grid, 1, 1);
    config.blockDim = dim3(kThreads, 1, 1);
    config.dynamicSmemBytes = dynamic_smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2] = {};
    unsigned count = 0;
    if (pair) {
        attributes[count].id = cudaLaunchAttributeClusterDimension;
        attributes[count].val.clusterDim.x = 2;
        attributes[count].val.clusterDim.y = 1;
        attributes[count].val.clusterDim.z = 1;
        ++count;
    }
    if (early_launch) {
        // Programmatic dependent launch: the grid may start (barrier set-up, tensor-memory
        // allocation) while the kernel before it on the stream drains; the kernel itself waits
        // (griddepcontrol.wait) before it reads anything that kernel wrote.
        attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    config.attrs = count != 0 ? attributes : nullptr;
    config.numAttrs = count;
    return cudaLaunchKernelEx(&config, kernel, params);
}

}  // namespace sdxlq
