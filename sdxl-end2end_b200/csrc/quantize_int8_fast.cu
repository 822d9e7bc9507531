// Throughput versions of the INT8 activation quantiser for FP16 rows whose pitch is a multiple of
// 16 bytes (every SDXL projection input). Same arithmetic, bit for bit, as the general kernel in
// quantize.cu, i.e. activation_amax_kernel + quantize_activation_kernel of the reference
// (src/cuda/int8_convrot.cu:265-353) fused into one pass:
//
//   plain_rows_kernel    no rotation: one warp per row, 16-byte loads strided over the lanes, the
//                        row kept as packed halves in registers, absmax in half precision (exact:
//                        the maximum of FP16 values is one of them), warp-shuffle reduction.
//   rotated_rows_kernel  regular-Hadamard groups of 4 / 16 / 64 / 256: four lanes own a 256-element
//                        chunk (lane q holds elements 32u + 8q .. +7 for u = 0..7), butterflies in
//                        registers with packed FP32x2 adds, two lane exchanges, and the reference's
//                        association for every output so that results match a sequential evaluation.

#include "quantize.cuh"

namespace sdxlq {

namespace {

__device__ __forceinline__ const QuantInt8Job& find_job(const QuantInt8Launch& launch, uint32_t block) {
    if (launch.jobs == nullptr) return launch.single;
    uint32_t lo = 0, hi = launch.num_jobs;          // last job with first_block <= block
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (launch.jobs[mid].first_block <= block) lo = mid; else hi = mid;
    }
    return launch.jobs[lo];
}

__device__ __forceinline__ float scale_from_amax(float maximum) {
    return maximum > 0.0f ? fmaxf(__fdiv_rn(maximum, 127.0f), 1.0e-30f) : 1.0f;
}

// clamp(rn(x), -128, 127) as a sign-extended 32-bit integer; NaN -> 0 (like __float2int_rn + clamp).
__device__ __forceinline__ uint32_t quantize_s8(float value) {
    uint32_t result;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(result) : "f"(value));
    return result;
}

// The low bytes of four integers -> one little-endian word.
__device__ __forceinline__ uint32_t pack_bytes(uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
    const uint32_t lo = __byte_perm(b0, b1, 0x0040);
    const uint32_t hi = __byte_perm(b2, b3, 0x0040);
    return __byte_perm(lo, hi, 0x5410);
}

__device__ __forceinline__ float half_lo(uint32_t word) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(word & 0xFFFFu)));
}
__device__ __forceinline__ float half_hi(uint32_t word) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(word >> 16)));
}

__device__ __forceinline__ uint2 quantize_vector(const uint4 raw, float inverse_scale) {
    const uint32_t q0 = quantize_s8(__fmul_rn(half_lo(raw.x), inverse_scale));
    const uint32_t q1 = quantize_s8(__fmul_rn(half_hi(raw.x), inverse_scale));
    const uint32_t q2 = quantize_s8(__fmul_rn(half_lo(raw.y), inverse_scale));
    const uint32_t q3 = quantize_s8(__fmul_rn(half_hi(raw.y), inverse_scale));
    const uint32_t q4 = quantize_s8(__fmul_rn(half_lo(raw.z), inverse_scale));
    const uint32_t q5 = quantize_s8(__fmul_rn(half_hi(raw.z), inverse_scale));
    const uint32_t q6 = quantize_s8(__fmul_rn(half_lo(raw.w), inverse_scale));
    const uint32_t q7 = quantize_s8(__fmul_rn(half_hi(raw.w), inverse_scale));
    return make_uint2(pack_bytes(q0, q1, q2, q3), pack_bytes(q4, q5, q6, q7));
}

__device__ __forceinline__ __half2 as_half2(uint32_t word) {
    return *reinterpret_cast<const __half2*>(&word);
}

// Finite-only |x| maximum of one 16-byte vector, the slow path used when a row holds infinities.
__device__ __forceinline__ float finite_max(const uint4 raw, float current) {
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float lo = fabsf(half_lo(words[i])), hi = fabsf(half_hi(words[i]));
        if (lo <= 3.402823466e+38f && lo > current) current = lo;
        if (hi <= 3.402823466e+38f && hi > current) current = hi;
    }
    return current;
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// No rotation: one warp per row.
// ------------------------------------------------------------------------------------------------
template <int MaxVectors>
__global__ void __launch_bounds__(256)
plain_rows_kernel(const __grid_constant__ QuantInt8Launch launch) {
    const QuantInt8Job& job = find_job(launch, blockIdx.x);
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row = (blockIdx.x - job.first_block) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= job.m) return;
    const uint32_t vectors = job.k >> 3;
    const uint4* source = reinterpret_cast<const uint4*>(static_cast<const __half*>(job.x) + static_cast<size_t>(row) * job.k);

    uint4 raw[MaxVectors];
    __half2 maximum2 = __float2half2_rn(0.0f);
#pragma unroll
    for (int v = 0; v < MaxVectors; ++v) {
        const uint32_t index = v * 32u + lane;
        raw[v] = index < vectors ? __ldg(source + index) : make_uint4(0u, 0u, 0u, 0u);
        maximum2 = __hmax2(maximum2, __habs2(as_half2(raw[v].x)));
        maximum2 = __hmax2(maximum2, __habs2(as_half2(raw[v].y)));
        maximum2 = __hmax2(maximum2, __habs2(as_half2(raw[v].z)));
        maximum2 = __hmax2(maximum2, __habs2(as_half2(raw[v].w)));
    }
    float maximum = fmaxf(__low2float(maximum2), __high2float(maximum2));
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, offset));
    }
    if (!(maximum <= 3.402823466e+38f)) {          // the row holds an infinity: finite values only
        maximum = 0.0f;
#pragma unroll
        for (int v = 0; v < MaxVectors; ++v) maximum = finite_max(raw[v], maximum);
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, offset));
        }
    }
    const float scale = scale_from_amax(maximum);
    const float inverse_scale = __fdiv_rn(1.0f, scale);
    if (lane == 0) job.scales[row] = scale;
    uint2* destination = reinterpret_cast<uint2*>(job.xq + static_cast<size_t>(row) * job.k);
#pragma unroll
    for (int v = 0; v < MaxVectors; ++v) {
        const uint32_t index = v * 32u + lane;
        if (index < vectors) destination[index] = quantize_vector(raw[v], inverse_scale);
    }
}

// ------------------------------------------------------------------------------------------------
// Rotated rows.
// ------------------------------------------------------------------------------------------------
namespace {

__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
// a - b with one rounding (b * -1 is exact).
__device__ __forceinline__ float2 sub2(float2 a, float2 b) { return __ffma2_rn(b, make_float2(-1.0f, -1.0f), a); }

// Packed radix-4 butterfly outputs with the reference's association.
__device__ __forceinline__ float2 bf0(float2 a, float2 b, float2 c, float2 d) { return sub2(add2(add2(a, b), c), d); }
__device__ __forceinline__ float2 bf1(float2 a, float2 b, float2 c, float2 d) { return add2(sub2(add2(a, b), c), d); }
__device__ __forceinline__ float2 bf2(float2 a, float2 b, float2 c, float2 d) { return add2(add2(sub2(a, b), c), d); }
__device__ __forceinline__ float2 bf3(float2 a, float2 b, float2 c, float2 d) { return add2(add2(sub2(b, a), c), d); }

__device__ __forceinline__ float sbf0(float a, float b, float c, float d) { return ((a + b) + c) - d; }
__device__ __forceinline__ float sbf1(float a, float b, float c, float d) { return ((a + b) - c) + d; }
__device__ __forceinline__ float sbf2(float a, float b, float c, float d) { return ((a - b) + c) + d; }
__device__ __forceinline__ float sbf3(float a, float b, float c, float d) { return ((-a + b) + c) + d; }

__device__ __forceinline__ float2 shuffle2(float2 value, int lane_mask) {
    return make_float2(__shfl_xor_sync(0xffffffffu, value.x, lane_mask), __shfl_xor_sync(0xffffffffu, value.y, lane_mask));
}

}  // namespace

// q[u][j] = (element 32u + 8*lane_in_quad + j, element 32u + 8*lane_in_quad + j + 4) of the chunk.
template <int Stages>
__global__ void __launch_bounds__(256, 2)
rotated_rows_kernel(const __grid_constant__ QuantInt8Launch launch) {
    __shared__ uint32_t row_max_bits[64];
    const QuantInt8Job& job = find_job(launch, blockIdx.x);
    if (job.stages != Stages) return;               // the launcher issues one launch per group size
    const uint32_t local_block = blockIdx.x - job.first_block;
    const uint32_t threads_per_row = job.threads_per_row;
    const uint32_t row_in_block = threadIdx.x / threads_per_row;
    const uint32_t thread_in_row = threadIdx.x - row_in_block * threads_per_row;
    const uint32_t row = local_block * job.rows_per_block + row_in_block;
    const bool active = row_in_block < job.rows_per_block && row < job.m;
    const uint32_t quad_lane = thread_in_row & 3u;
    const uint32_t base_col = (thread_in_row >> 2) * 256u + quad_lane * 8u;
    const uint32_t k = job.k;
    const __half* source = static_cast<const __half*>(job.x) + static_cast<size_t>(row) * k;
    if (threadIdx.x < 64) row_max_bits[threadIdx.x] = 0;

    float2 q[8][4];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const uint32_t col = base_col + 32u * u;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (active && col < k) raw = __ldg(reinterpret_cast<const uint4*>(source + col));
        q[u][0] = make_float2(half_lo(raw.x), half_lo(raw.z));
        q[u][1] = make_float2(half_hi(raw.x), half_hi(raw.z));
        q[u][2] = make_float2(half_lo(raw.y), half_lo(raw.w));
        q[u][3] = make_float2(half_hi(raw.y), half_hi(raw.w));
    }

    if (Stages >= 1) {          // stride 1: index bits 0-1 (j), in-lane; .x and .y are two tuples
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float2 a = q[u][0], b = q[u][1], c = q[u][2], d = q[u][3];
            q[u][0] = bf0(a, b, c, d);
            q[u][1] = bf1(a, b, c, d);
            q[u][2] = bf2(a, b, c, d);
            q[u][3] = bf3(a, b, c, d);
        }
    }
    if (Stages >= 2) {          // stride 4: index bit 2 = (.x | .y), bit 3 = quad lane bit 0
        const bool upper = (quad_lane & 1u) != 0;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float lo = q[u][j].x, hi = q[u][j].y;
                const float other_lo = __shfl_xor_sync(0xffffffffu, lo, 1);
                const float other_hi = __shfl_xor_sync(0xffffffffu, hi, 1);
                if (!upper) {   // holds a, b; partner holds c, d
                    q[u][j] = make_float2(sbf0(lo, hi, other_lo, other_hi), sbf1(lo, hi, other_lo, other_hi));
                } else {        // holds c, d; partner holds a, b
                    q[u][j] = make_float2(sbf2(other_lo, other_hi, lo, hi), sbf3(other_lo, other_hi, lo, hi));
                }
            }
        }
    }
    if (Stages >= 3) {          // stride 16: index bit 4 = quad lane bit 1, bit 5 = u bit 0
        const bool upper = (quad_lane & 2u) != 0;
#pragma unroll
        for (int w = 0; w < 8; w += 2) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 lo = q[w][j], hi = q[w + 1][j];
                const float2 other_lo = shuffle2(lo, 2);
                const float2 other_hi = shuffle2(hi, 2);
                if (!upper) {   // holds a (u even), c (u odd); partner holds b, d
                    q[w][j] = bf0(lo, other_lo, hi, other_hi);
                    q[w + 1][j] = bf2(lo, other_lo, hi, other_hi);
                } else {        // holds b, d; partner holds a, c
                    q[w][j] = bf1(other_lo, lo, other_hi, hi);
                    q[w + 1][j] = bf3(other_lo, lo, other_hi, hi);
                }
            }
        }
    }
    if (Stages >= 4) {          // stride 64: index bits 6-7 = u bits 1-2, in-lane
#pragma unroll
        for (int u0 = 0; u0 < 2; ++u0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 a = q[u0][j], b = q[u0 + 2][j], c = q[u0 + 4][j], d = q[u0 + 6][j];
                q[u0][j] = bf0(a, b, c, d);
                q[u0 + 2][j] = bf1(a, b, c, d);
                q[u0 + 4][j] = bf2(a, b, c, d);
                q[u0 + 6][j] = bf3(a, b, c, d);
            }
        }
    }

    // g^-1/2 = 2^-Stages exactly; the maximum skips NaN (fmaxf) and, through the slow path, inf.
    const float normalization = __uint_as_float((127u - Stages) << 23);
    const float2 normalization2 = make_float2(normalization, normalization);
    float local_max = 0.0f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            q[u][j] = __fmul2_rn(q[u][j], normalization2);
            local_max = fmaxf(local_max, fmaxf(fabsf(q[u][j].x), fabsf(q[u][j].y)));
        }
    }
    if (!(local_max <= 3.402823466e+38f)) {
        local_max = 0.0f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float x = fabsf(q[u][j].x), y = fabsf(q[u][j].y);
                if (x <= 3.402823466e+38f && x > local_max) local_max = x;
                if (y <= 3.402823466e+38f && y > local_max) local_max = y;
            }
        }
    }
    local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, 1));
    local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, 2));
    __syncthreads();            // row_max_bits cleared
    if (active && quad_lane == 0) atomicMax(row_max_bits + row_in_block, __float_as_uint(local_max));
    __syncthreads();
    const float scale = scale_from_amax(__uint_as_float(row_max_bits[active ? row_in_block : 0]));
    const float inverse_scale = __fdiv_rn(1.0f, scale);
    const float2 inverse2 = make_float2(inverse_scale, inverse_scale);
    if (active && thread_in_row == 0) job.scales[row] = scale;

    int8_t* destination = job.xq + static_cast<size_t>(row) * k;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const uint32_t col = base_col + 32u * u;
        if (!active || col >= k) continue;
        uint32_t low[4], high[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 scaled = __fmul2_rn(q[u][j], inverse2);
            low[j] = quantize_s8(scaled.x);
            high[j] = quantize_s8(scaled.y);
        }
        *reinterpret_cast<uint2*>(destination + col) =
            make_uint2(pack_bytes(low[0], low[1], low[2], low[3]), pack_bytes(high[0], high[1], high[2], high[3]));
    }
}

cudaError_t launch_int8_plain_rows(const QuantInt8Launch& launch, uint32_t blocks, uint32_t max_vectors,
                                   cudaStream_t stream) {
    if (max_vectors <= 3) plain_rows_kernel<3><<<blocks, 256, 0, stream>>>(launch);
    else if (max_vectors <= 10) plain_rows_kernel<10><<<blocks, 256, 0, stream>>>(launch);
    else plain_rows_kernel<20><<<blocks, 256, 0, stream>>>(launch);
    return cudaGetLastError();
}

cudaError_t launch_int8_rotated_rows(const QuantInt8Launch& launch, uint32_t blocks, uint32_t threads,
                                     uint32_t stages, cudaStream_t stream) {
    switch (stages) {
    case 1: rotated_rows_kernel<1><<<blocks, threads, 0, stream>>>(launch); break;
    case 2: rotated_rows_kernel<2><<<blocks, threads, 0, stream>>>(launch); break;
    case 3: rotated_rows_kernel<3><<<blocks, threads, 0, stream>>>(launch); break;
    default: rotated_rows_kernel<4><<<blocks, threads, 0, stream>>>(launch); break;
    }
    return cudaGetLastError();
}

}  // namespace sdxlq
