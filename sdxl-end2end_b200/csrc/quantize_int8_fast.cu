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
#include "int8_math.cuh"

namespace sdxlq {

namespace {

__device__ __forceinline__ const QuantInt8Job& find_job(const QuantInt8Launch& launch, uint32_t block) {
    if (launch.jobs == nullptr) return launch.single;
    if (launch.block_jobs != nullptr) return launch.jobs[launch.block_jobs[block]];
    uint32_t lo = 0, hi = launch.num_jobs;          // last job with first_block <= block
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (launch.jobs[mid].first_block <= block) lo = mid; else hi = mid;
    }
    return launch.jobs[lo];
}


}  // namespace

// ------------------------------------------------------------------------------------------------
// No rotation: one warp per row.
// ------------------------------------------------------------------------------------------------
template <int MaxVectors>
__global__ void __launch_bounds__(256)
plain_rows_kernel(const __grid_constant__ QuantInt8Launch launch) {
    wait_for_prior_kernels_then_release_next();
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
    wait_for_prior_kernels_then_release_next();
    const QuantInt8Job& job = find_job(launch, blockIdx.x);
    if (job.stages != Stages || job.pad != 0) return;   // one launch per group size; pad = 1: rotated256_rows_kernel
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

// ------------------------------------------------------------------------------------------------
// Rotated rows, groups of 256 (the default group size): every butterfly stage in registers on the
// packed FP32 pipe, one exchange through shared memory between stages 3 and 4, no lane shuffles.
//
// Four consecutive threads (a quad, inside one warp) own one 256-element group. Element e of the
// group = 64 r + 32 h + 16 y + l with r, h, y the index bits 7-6, 5, 4 and l the bits 3-0.
//   phase 1  each warp copies its threads' 64-element runs (thread T of the quad: r = T) from global
//            to shared memory with 16-byte asynchronous copies, coalesced, and each thread reads its
//            own run back: it now holds bits 5-0 in registers, as pairs P[h][l] = (y = 0, y = 1).
//   stages 1, 2 (strides 1, 4: bits 0-3) packed over the pair; stage 3 (stride 16: bits 4-5)
//            combines the two halves of P[0][l] and P[1][l], scalar.
//   exchange each thread writes its values to the quad's area of shared memory and reads back the
//            elements with bits 5-4 equal to its quad lane: it now holds bits 7-6 and 3-0, as runs
//            of four consecutive elements W[w][r] (l = 4 w .. 4 w + 3).
//   stage 4  (stride 64: bits 7-6) packed over consecutive elements.
// Then the row maximum (block-wide through shared memory), the scale, and the INT8 results: every
// thread stores four runs of 16 consecutive bytes.
// The 2^-4 normalisation is folded into the maximum and into the inverse scale: scaling by a power
// of two is exact (rotated FP16 data is a multiple of 2^-24, nowhere near the FP32 subnormals), so
// fl(fl(x * 2^-4) * (1 / s)) = fl(x * (2^-4 / s)) bit for bit.
//
// Measured on B200 (X[16384, 1280] and X[8192, 2560], 23 to 24 us, 0.42 to 0.53 of the copy bandwidth): the
// kernel is bound by instruction issue and dependency latency at 13 to 16 warps per SM (64 FP32 values
// and their successors per thread: 114 to 126 registers), not by memory. Tried and no faster, same GPU:
//  * a persistent grid that copies the next tile into a second staging buffer while it works on the
//    current one (loads fully overlapped; 11 % slower: more registers live across the loop);
//  * stage 3 on the packed pipe after regrouping neighbouring values into pairs, the integer cast as
//    fl(x / s) + 1.5 * 2^23 instead of cvt.rni (the conversion pipe goes from 29 % to 2 % busy, but the
//    regrouping moves cost more issue slots than the packed adds save: 13.4 against 11.8 million warp
//    instructions, same time). Note for anyone who retries the cast: a packed add.rn.f32x2 placed behind a
//    packed mul.rn.f32x2 was contracted into one packed fma (a single rounding; 5 of 2.6 million results off
//    by one at ties), the scalar add.rn.f32 was not.
//  * eight threads per group (32 values each, 64 registers, 32 warps per SM, all four stages packed, results
//    regrouped through shared memory for 32-byte stores): bit-identical, 21.9 against 21.8 us; the same kernel
//    persistent with the next tile's copies in flight behind the arithmetic: 27.6 us.
//  Twice the warps, fewer instructions and overlapped loads each leave the time where it is or make it worse;
//  what the three variants share is two block-wide barriers per tile around the row maximum.
// ------------------------------------------------------------------------------------------------
namespace {

__device__ __forceinline__ void cp_async_16(uint32_t smem_address, const void* global_address) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_address), "l"(global_address) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// in-place radix-4 butterfly on four packed values
__device__ __forceinline__ void butterfly2(float2& a, float2& b, float2& c, float2& d) {
    const float2 o0 = bf0(a, b, c, d), o1 = bf1(a, b, c, d), o2 = bf2(a, b, c, d), o3 = bf3(a, b, c, d);
    a = o0; b = o1; c = o2; d = o3;
}

}  // namespace

__global__ void __launch_bounds__(256, 2)
rotated256_rows_kernel(const __grid_constant__ QuantInt8Launch launch) {
    extern __shared__ __align__(16) uint8_t dynamic_smem[];
    __shared__ uint32_t row_max_bits[64];
    wait_for_prior_kernels_then_release_next();
    const QuantInt8Job& job = find_job(launch, blockIdx.x);
    if (job.stages != 4 || job.pad == 0) return;      // other group sizes / alignments: rotated_rows_kernel
    const uint32_t thread = threadIdx.x;
    const uint32_t lane = thread & 31u;
    const uint32_t warp_first = thread & ~31u;        // first thread of this warp
    const uint32_t quad_lane = thread & 3u;
    const uint32_t local_block = blockIdx.x - job.first_block;
    const uint32_t threads_per_row = job.threads_per_row;
    const uint32_t k = job.k;
    const uint32_t first_row = local_block * job.rows_per_block;
    const uint32_t active_threads = min(job.rows_per_block, job.m - first_row) * threads_per_row;
    const bool active = thread < active_threads;
    const uint32_t row_in_block = thread / threads_per_row;
    const uint32_t thread_in_row = thread - row_in_block * threads_per_row;
    uint8_t* staging = dynamic_smem;                                   // [threads][128 B] FP16 runs
    float* exchange = reinterpret_cast<float*>(dynamic_smem + blockDim.x * 128u);   // [threads][64] FP32
    if (thread < 64) row_max_bits[thread] = 0;

    // ---- phase 1: global -> shared (this warp's runs), then this thread's run -> registers ----
    {
        // The block's rows are contiguous in memory; thread T owns halves [64 T, 64 T + 64) of them,
        // i.e. 16-byte units 8 T .. 8 T + 7. Unit u of owner T sits at T * 128 + ((u ^ T) & 7) * 16.
        const uint4* block_source = reinterpret_cast<const uint4*>(static_cast<const __half*>(job.x) + static_cast<size_t>(first_row) * k);
        const uint32_t staging_address = static_cast<uint32_t>(__cvta_generic_to_shared(staging));
#pragma unroll
        for (int round = 0; round < 8; ++round) {
            const uint32_t unit = warp_first * 8u + round * 32u + lane;        // block-wide unit index
            const uint32_t owner = unit >> 3;
            if (owner < active_threads) {
                cp_async_16(staging_address + owner * 128u + (((unit ^ owner) & 7u) << 4), block_source + unit);
            }
        }
        cp_async_wait_all();
        __syncwarp();
    }
    float2 p[2][16];       // p[h][l] = (element 32 h + l, element 32 h + 16 + l) of this thread's run
    {
        const uint4* mine = reinterpret_cast<const uint4*>(staging + thread * 128u);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int v = 0; v < 2; ++v) {                 // v: which 8 of the 16 values of l
                uint4 low = make_uint4(0u, 0u, 0u, 0u), high = make_uint4(0u, 0u, 0u, 0u);
                if (active) {
                    low = mine[((4 * h + v) ^ thread) & 7u];          // elements 32 h + 8 v .. + 7
                    high = mine[((4 * h + 2 + v) ^ thread) & 7u];     // elements 32 h + 16 + 8 v .. + 7
                }
                const uint32_t lw[4] = {low.x, low.y, low.z, low.w}, hw[4] = {high.x, high.y, high.z, high.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    p[h][8 * v + 2 * i] = make_float2(half_lo(lw[i]), half_lo(hw[i]));
                    p[h][8 * v + 2 * i + 1] = make_float2(half_hi(lw[i]), half_hi(hw[i]));
                }
            }
        }
    }
    // ---- stages 1 and 2: index bits 0-1 and 2-3, packed over bit 4 ----
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int g = 0; g < 4; ++g) butterfly2(p[h][4 * g], p[h][4 * g + 1], p[h][4 * g + 2], p[h][4 * g + 3]);
#pragma unroll
        for (int g = 0; g < 4; ++g) butterfly2(p[h][g], p[h][g + 4], p[h][g + 8], p[h][g + 12]);
    }
    // ---- stage 3: index bits 4 (the pair) and 5 (h), scalar ----
#pragma unroll
    for (int l = 0; l < 16; ++l) {
        const float a = p[0][l].x, b = p[0][l].y, c = p[1][l].x, d = p[1][l].y;
        p[0][l] = make_float2(sbf0(a, b, c, d), sbf1(a, b, c, d));
        p[1][l] = make_float2(sbf2(a, b, c, d), sbf3(a, b, c, d));
    }
    // ---- exchange inside the quad ----
    // Destination thread D (quad lane q' = bits 5-4) keeps 16 units of four floats: unit 4 w + r
    // holds elements 64 r + 16 q' + 4 w .. + 3, at D * 64 + ((4 w + r) ^ (D & 7)) * 4 floats.
    float2 w2[4][4][2];    // w2[w][r][z]: elements 64 r + 16 q + 4 w + 2 z, + 1
    {
        const uint32_t quad_first = thread & ~3u;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int y = 0; y < 2; ++y) {
                const uint32_t destination = quad_first + 2u * h + y;
                float* area = exchange + destination * 64u;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint32_t unit = (4u * w + quad_lane) ^ (destination & 7u);
                    float4 value;
                    if (y == 0) value = make_float4(p[h][4 * w].x, p[h][4 * w + 1].x, p[h][4 * w + 2].x, p[h][4 * w + 3].x);
                    else value = make_float4(p[h][4 * w].y, p[h][4 * w + 1].y, p[h][4 * w + 2].y, p[h][4 * w + 3].y);
                    *reinterpret_cast<float4*>(area + unit * 4u) = value;
                }
            }
        }
        __syncwarp();
        const float* area = exchange + thread * 64u;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float4 value = *reinterpret_cast<const float4*>(area + (((4u * w + r) ^ (thread & 7u)) * 4u));
                w2[w][r][0] = make_float2(value.x, value.y);
                w2[w][r][1] = make_float2(value.z, value.w);
            }
        }
    }
    // ---- stage 4: index bits 6-7 (r), packed over consecutive elements ----
    float local_max = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
        for (int z = 0; z < 2; ++z) {
            butterfly2(w2[w][0][z], w2[w][1][z], w2[w][2][z], w2[w][3][z]);
#pragma unroll
            for (int r = 0; r < 4; ++r) local_max = fmaxf(local_max, fmaxf(fabsf(w2[w][r][z].x), fabsf(w2[w][r][z].y)));
        }
    }
    if (!(local_max <= 3.402823466e+38f)) {           // an infinity: the maximum runs over finite values only
        local_max = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
#pragma unroll
                for (int z = 0; z < 2; ++z) {
                    const float x = fabsf(w2[w][r][z].x), y = fabsf(w2[w][r][z].y);
                    if (x <= 3.402823466e+38f && x > local_max) local_max = x;
                    if (y <= 3.402823466e+38f && y > local_max) local_max = y;
                }
            }
        }
    }
    local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, 1));
    local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, 2));
    __syncthreads();            // row_max_bits cleared
    // the maximum of the normalised values: 2^-4 times the maximum found (exact)
    if (active && quad_lane == 0) atomicMax(row_max_bits + row_in_block, __float_as_uint(local_max * 0.0625f));
    __syncthreads();
    if (!active) return;
    const uint32_t row = first_row + row_in_block;
    const float scale = scale_from_amax(__uint_as_float(row_max_bits[row_in_block]));
    const float inverse_scale = __fdiv_rn(1.0f, scale) * 0.0625f;     // exact: folds the 2^-4 normalisation
    const float2 inverse2 = make_float2(inverse_scale, inverse_scale);
    if (thread_in_row == 0) job.scales[row] = scale;
    int8_t* destination = job.xq + static_cast<size_t>(row) * k + (thread_in_row >> 2) * 256u + quad_lane * 16u;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        uint32_t words[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float2 first = __fmul2_rn(w2[w][r][0], inverse2), second = __fmul2_rn(w2[w][r][1], inverse2);
            words[w] = pack_bytes(quantize_s8(first.x), quantize_s8(first.y), quantize_s8(second.x), quantize_s8(second.y));
        }
        *reinterpret_cast<uint4*>(destination + 64 * r) = make_uint4(words[0], words[1], words[2], words[3]);
    }
}

cudaError_t launch_int8_plain_rows(const QuantInt8Launch& launch, uint32_t blocks, uint32_t max_vectors,
                                   cudaStream_t stream, bool early_launch) {
    if (max_vectors <= 3) return launch_behind(plain_rows_kernel<3>, blocks, 256, 0, stream, early_launch, launch);
    if (max_vectors <= 10) return launch_behind(plain_rows_kernel<10>, blocks, 256, 0, stream, early_launch, launch);
    return launch_behind(plain_rows_kernel<20>, blocks, 256, 0, stream, early_launch, launch);
}

cudaError_t launch_int8_rotated_rows(const QuantInt8Launch& launch, uint32_t blocks, uint32_t threads,
                                     uint32_t stages, cudaStream_t stream, bool early_launch) {
    switch (stages) {
    case 1: return launch_behind(rotated_rows_kernel<1>, blocks, threads, 0, stream, early_launch, launch);
    case 2: return launch_behind(rotated_rows_kernel<2>, blocks, threads, 0, stream, early_launch, launch);
    case 3: return launch_behind(rotated_rows_kernel<3>, blocks, threads, 0, stream, early_launch, launch);
    default: return launch_behind(rotated_rows_kernel<4>, blocks, threads, 0, stream, early_launch, launch);
    }
}

// Groups of 256 with 16-byte aligned outputs (jobs marked with pad = 1).
cudaError_t launch_int8_rotated256_rows(const QuantInt8Launch& launch, uint32_t blocks, uint32_t threads,
                                        cudaStream_t stream, bool early_launch) {
    const size_t dynamic_smem = static_cast<size_t>(threads) * (128u + 256u);
    static bool opted_in[64] = {};
    int device = 0;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) return status;
    if (device < 0 || device >= 64 || !opted_in[device]) {
        status = cudaFuncSetAttribute(rotated256_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 256 * (128 + 256));
        if (status != cudaSuccess) return status;
        if (device >= 0 && device < 64) opted_in[device] = true;
    }
    return launch_behind(rotated256_rows_kernel, blocks, threads, dynamic_smem, stream, early_launch, launch);
}

}  // namespace sdxlq
