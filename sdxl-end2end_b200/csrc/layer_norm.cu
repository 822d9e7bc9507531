// LayerNorm over the last dimension, alone or fused with the FP8 activation quantiser that feeds the
// next projection.
//
// Arithmetic of the reference's layer_norm_kernel / layer_norm_fixed_kernel
// (src/cuda/ops_kernels.cu:185-256, launched by Ops::layer_norm at :1425-1470): FP32 sum -> mean,
// FP32 sum of the centred squares -> variance = max(0, sum / width), inverse = rsqrtf(variance +
// epsilon), y = half_rn((x - mean) * inverse * gamma + beta). The reference gives a row to a block and
// adds the partial sums through a shared-memory tree; here a warp owns a row, every lane adds its
// elements (even and odd ones in two accumulators) and the lanes are combined by a butterfly of
// shuffles. Only the order of the FP32 additions differs, which moves the sums in their last bits;
// results are deterministic.
//
// The row stays on the SM between the three steps (one 16-byte copy per eight elements, no re-read
// from memory), so the FP16 form moves 2 + 2 bytes per element. The FP8 form needs max |y| of the whole
// tensor before the first byte can be written: a statistics launch normalises and only reduces the
// maximum (2 bytes per element read), the cast launch normalises again and writes FP8 (2 read, 1
// written). 5 bytes per element against 9 for LayerNorm followed by the stand-alone quantiser.
// The unrotated INT8 form is one launch: the normalised row is kept as packed halves in the ring, its
// maximum is a warp reduction, and the bytes are written at once (2 read, 1 written).

#include "quantize.cuh"
#include "fp8_math.cuh"
#include "int8_math.cuh"


namespace sdxlq {

namespace {

enum : int { LN_F16 = 0, LN_FP8_STATS = 1, LN_FP8_CAST = 2, LN_INT8 = 3, LN_FP8_CAST_SAVED = 4 };   // _SAVED: row statistics from row_stats

constexpr uint32_t kRowsPerBlock = 8;      // one warp per row, 256 threads

__device__ __forceinline__ float warp_sum(float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_xor_sync(0xffffffffu, value, offset);
    return value;
}

__device__ __forceinline__ float2 pair_of(uint32_t word) { return __half22float2(as_half2(word)); }
__device__ __forceinline__ uint32_t word_of(const uint4& raw, int i) {
    return i == 0 ? raw.x : i == 1 ? raw.y : i == 2 ? raw.z : raw.w;
}

// kVectors 16-byte vectors per lane: rows of up to 256 * kVectors elements, one warp per row. The row is
// held as packed halves (converted on the fly in each of the three passes over the registers) and the
// next row of the warp is requested before the current one is worked on, so that the loads of one row
// overlap the arithmetic of the other. All FP32 arithmetic runs two elements at a time on the packed
// pipe (add / mul / fma .f32x2: each half rounds like the scalar instruction); gamma and beta sit in
// shared memory as FP32, split into the first and the second four elements of every vector so that the
// lanes' 16-byte reads do not collide. 67 to 80 registers: three blocks (24 warps) per SM, two for rows
// wider than 1280.
//
// FP8: the statistics launch leaves (mean, inverse deviation) of every row in row_stats (when the caller
// has room for them) so that the cast launch does not reduce the row again; the cast launch walks the
// rows from the last to the first, i.e. it starts with what the statistics launch read last and may
// still find in L2.
//
// Measured slower on B200 at the sizes of the UNet (65536 x 640, 16384 x 1280), same run: a ring of
// three or four rows per warp in shared memory filled by cp.async (deeper prefetch, 56 to 64 registers,
// 32 warps per SM) with the three passes reading shared memory (the load/store pipe becomes the busiest
// unit: 16 bytes of shared-memory traffic per element) -- 19 % slower; the same ring read once into
// registers, with gamma and beta as packed halves in registers -- 4 to 14 % slower on the FP8 forms.
template <int kVectors, int Mode>
__global__ void __launch_bounds__(256, kVectors > 5 ? 2 : 3)
layer_norm_rows_kernel(const __grid_constant__ LayerNormLaunch p) {
    // The cast launch of the FP8 form is scheduled while the statistics launch runs: it reads the rows (complete
    // since before the statistics launch released it) and only waits for that launch's maximum further down.
    // Every other form first waits for the kernels before it, then releases the kernel behind it.
    if constexpr (Mode == LN_FP8_CAST || Mode == LN_FP8_CAST_SAVED) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    else wait_for_prior_kernels_then_release_next();
    constexpr uint32_t kRowVectors = kVectors * 32;
    __shared__ float4 gamma_beta[4][kRowVectors];         // gamma 0-3, gamma 4-7, beta 0-3, beta 4-7 of each vector
    __shared__ uint32_t maximum_bits;
    __shared__ float warp_max[kRowsPerBlock];
    constexpr bool kCast = Mode == LN_FP8_CAST || Mode == LN_FP8_CAST_SAVED;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t vectors = p.width / 8;
    const float width = static_cast<float>(p.width);

    // The n-th row of this warp; the cast launch counts from the end of the tensor.
    const uint32_t stride = gridDim.x * kRowsPerBlock;
    const uint32_t first = blockIdx.x * kRowsPerBlock + warp;
    auto row_of = [&](uint32_t position) { return kCast ? p.rows - 1u - position : position; };
    uint4 raw[kVectors];
    auto request = [&](uint32_t at, uint4 (&into)[kVectors]) {
        const bool inside = at < p.rows;
        const uint4* source = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(inside ? row_of(at) : 0u) * p.width);
#pragma unroll
        for (int j = 0; j < kVectors; ++j) {
            const uint32_t vector = static_cast<uint32_t>(j) * 32u + lane;
            into[j] = (inside && vector < vectors) ? __ldg(source + vector) : make_uint4(0, 0, 0, 0);
        }
    };
    request(first, raw);                // (cast launch: the rows were complete before the statistics launch released it)

    for (uint32_t vector = threadIdx.x; vector < vectors; vector += blockDim.x) {
        const uint4 g = reinterpret_cast<const uint4*>(p.gamma)[vector];
        const uint4 b = reinterpret_cast<const uint4*>(p.beta)[vector];
        const float2 g0 = pair_of(g.x), g1 = pair_of(g.y), g2 = pair_of(g.z), g3 = pair_of(g.w);
        const float2 b0 = pair_of(b.x), b1 = pair_of(b.y), b2 = pair_of(b.z), b3 = pair_of(b.w);
        gamma_beta[0][vector] = make_float4(g0.x, g0.y, g1.x, g1.y);
        gamma_beta[1][vector] = make_float4(g2.x, g2.y, g3.x, g3.y);
        gamma_beta[2][vector] = make_float4(b0.x, b0.y, b1.x, b1.y);
        gamma_beta[3][vector] = make_float4(b2.x, b2.y, b3.x, b3.y);
    }

    float2 inverse_scale2 = make_float2(1.0f, 1.0f);
    if constexpr (kCast) {
        asm volatile("griddepcontrol.wait;" ::: "memory");       // the maximum of the statistics launch is complete
        // One thread reads the maximum and counts this block among its readers; the block that
        // completes the count clears both words for the next call (and for a replay of a captured graph).
        if (threadIdx.x == 0) {
            maximum_bits = *reinterpret_cast<volatile uint32_t*>(p.amax_bits);
            __threadfence();
            if (atomicAdd(p.done_count, 1u) == gridDim.x - 1u) {
                *p.amax_bits = 0;
                *p.done_count = 0;
            }
        }
    }
    __syncthreads();
    if constexpr (kCast) {
        const float scale = fp8_scale_from_amax(__uint_as_float(maximum_bits), p.fmt);
        const float inverse_scale = __fdiv_rn(1.0f, scale);
        inverse_scale2 = make_float2(inverse_scale, inverse_scale);
        if (blockIdx.x == 0 && threadIdx.x == 0) *p.scale_out = scale;
    }

    __half2 local_max2 = __float2half2_rn(0.0f);
    for (uint32_t position = first; position < p.rows; position += stride) {
        const uint32_t row = row_of(position);
        uint4 next[kVectors];
        request(position + stride, next);
        float mean, inverse;
        if constexpr (Mode == LN_FP8_CAST_SAVED) {
            const float2 stats = p.row_stats[row];
            mean = stats.x;
            inverse = stats.y;
        } else {
            float2 sum2 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int j = 0; j < kVectors; ++j) {          // vectors past the row hold zeros
#pragma unroll
                for (int i = 0; i < 4; ++i) sum2 = __fadd2_rn(sum2, pair_of(word_of(raw[j], i)));
            }
            mean = __fdiv_rn(warp_sum(sum2.x + sum2.y), width);
            const float2 minus_mean = make_float2(-mean, -mean);
            float2 squares2 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int j = 0; j < kVectors; ++j) {
                if (static_cast<uint32_t>(j) * 32u + lane < vectors) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 centred = __fadd2_rn(pair_of(word_of(raw[j], i)), minus_mean);
                        squares2 = __ffma2_rn(centred, centred, squares2);
                    }
                }
            }
            const float variance = fmaxf(0.0f, __fdiv_rn(warp_sum(squares2.x + squares2.y), width));
            inverse = rsqrtf(variance + p.epsilon);
            if (Mode == LN_FP8_STATS && p.row_stats != nullptr && lane == 0) p.row_stats[row] = make_float2(mean, inverse);
        }
        const float2 minus_mean = make_float2(-mean, -mean);
        const float2 inverse2 = make_float2(inverse, inverse);

#pragma unroll
        for (int j = 0; j < kVectors; ++j) {
            const uint32_t vector = static_cast<uint32_t>(j) * 32u + lane;
            if (vector >= vectors) continue;
            const float4 g_lo = gamma_beta[0][vector], g_hi = gamma_beta[1][vector];
            const float4 b_lo = gamma_beta[2][vector], b_hi = gamma_beta[3][vector];
            const float2 g[4] = {make_float2(g_lo.x, g_lo.y), make_float2(g_lo.z, g_lo.w), make_float2(g_hi.x, g_hi.y),
                                 make_float2(g_hi.z, g_hi.w)};
            const float2 b[4] = {make_float2(b_lo.x, b_lo.y), make_float2(b_lo.z, b_lo.w), make_float2(b_hi.x, b_hi.y),
                                 make_float2(b_hi.z, b_hi.w)};
            __half2 result[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // ((x - mean) * inverse) * gamma + beta, the product with gamma and the sum in one fma
                const float2 centred = __fadd2_rn(pair_of(word_of(raw[j], i)), minus_mean);
                result[i] = __float22half2_rn(__ffma2_rn(__fmul2_rn(centred, inverse2), g[i], b[i]));
            }
            if constexpr (Mode == LN_F16) {
                reinterpret_cast<uint4*>(p.y + static_cast<size_t>(row) * p.width)[vector] =
                    *reinterpret_cast<const uint4*>(result);
            } else if constexpr (Mode == LN_INT8) {
                raw[j] = *reinterpret_cast<const uint4*>(result);     // kept until the row's maximum is known
            } else if constexpr (Mode == LN_FP8_STATS) {
                // the maximum of FP16 values is one of them: exact in half precision
                local_max2 = __hmax2(local_max2, __hmax2(__habs2(result[0]), __habs2(result[1])));
                local_max2 = __hmax2(local_max2, __hmax2(__habs2(result[2]), __habs2(result[3])));
            } else {
                uint32_t packed[2];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 scaled = __fmul2_rn(__half22float2(result[i]), inverse_scale2);
                    const uint32_t two = encode_fp8x2(scaled.x, scaled.y, p.fmt);
                    if ((i & 1) == 0) packed[i >> 1] = two & 0xFFFFu;
                    else packed[i >> 1] |= (two & 0xFFFFu) << 16;
                }
                reinterpret_cast<uint2*>(p.q + static_cast<size_t>(row) * p.width)[vector] = make_uint2(packed[0], packed[1]);
            }
        }
        if constexpr (Mode == LN_INT8) {
            // per-row scale and cast of the unrotated INT8 quantiser (plain_rows_kernel), on the
            // normalised FP16 values now held in raw[]
            __half2 maximum2 = __float2half2_rn(0.0f);
#pragma unroll
            for (int j = 0; j < kVectors; ++j) {
                if (static_cast<uint32_t>(j) * 32u + lane >= vectors) continue;
                const uint4 y = raw[j];
                maximum2 = __hmax2(maximum2, __hmax2(__habs2(as_half2(y.x)), __habs2(as_half2(y.y))));
                maximum2 = __hmax2(maximum2, __hmax2(__habs2(as_half2(y.z)), __habs2(as_half2(y.w))));
            }
            float maximum = fmaxf(__low2float(maximum2), __high2float(maximum2));
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1) {
                maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, offset));
            }
            if (!(maximum <= 3.402823466e+38f)) {          // the row holds an infinity: finite values only
                maximum = 0.0f;
#pragma unroll
                for (int j = 0; j < kVectors; ++j) {
                    if (static_cast<uint32_t>(j) * 32u + lane < vectors) maximum = finite_max(raw[j], maximum);
                }
#pragma unroll
                for (int offset = 16; offset > 0; offset >>= 1) {
                    maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, offset));
                }
            }
            const float scale = scale_from_amax(maximum);
            const float inverse_row = __fdiv_rn(1.0f, scale);
            if (lane == 0) p.scale_out[row] = scale;
            uint2* destination = reinterpret_cast<uint2*>(p.q + static_cast<size_t>(row) * p.width);
#pragma unroll
            for (int j = 0; j < kVectors; ++j) {
                const uint32_t vector = static_cast<uint32_t>(j) * 32u + lane;
                if (vector < vectors) destination[vector] = quantize_vector(raw[j], inverse_row);
            }
        }
#pragma unroll
        for (int j = 0; j < kVectors; ++j) raw[j] = next[j];
    }

    if constexpr (Mode == LN_FP8_STATS) {
        // NaN never wins a maximum here (the half-precision maximum drops it, like the reference's fmaxf)
        float local_max = fmaxf(__low2float(local_max2), __high2float(local_max2));
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, offset));
        }
        if (lane == 0) warp_max[warp] = local_max;
        __syncthreads();
        if (threadIdx.x == 0) {
            float block_max = 0.0f;
            for (uint32_t w = 0; w < kRowsPerBlock; ++w) block_max = fmaxf(block_max, warp_max[w]);
            atomicMax(p.amax_bits, __float_as_uint(block_max));
        }
    }
}

uint32_t grid_for(uint32_t rows) {
    const uint32_t wanted = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
    return wanted < 148u * 3u ? (wanted == 0 ? 1u : wanted) : 148u * 3u;
}

template <int Mode>
cudaError_t launch_mode(const LayerNormLaunch& launch, cudaStream_t stream, bool dependent) {
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(grid_for(launch.rows), 1, 1);
    config.blockDim = dim3(256, 1, 1);
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = dependent ? &attribute : nullptr;
    config.numAttrs = dependent ? 1 : 0;
    const uint32_t vectors_per_lane = (launch.width / 8 + 31) / 32;
    if (vectors_per_lane <= 3) return cudaLaunchKernelEx(&config, layer_norm_rows_kernel<3, Mode>, launch);
    if (vectors_per_lane <= 5) return cudaLaunchKernelEx(&config, layer_norm_rows_kernel<5, Mode>, launch);
    return cudaLaunchKernelEx(&config, layer_norm_rows_kernel<8, Mode>, launch);
}

}  // namespace

cudaError_t launch_layer_norm_f16(const LayerNormLaunch& launch, cudaStream_t stream, bool early_launch) {
    return launch_mode<LN_F16>(launch, stream, early_launch);
}

cudaError_t launch_layer_norm_int8(const LayerNormLaunch& launch, cudaStream_t stream, bool early_launch) {
    return launch_mode<LN_INT8>(launch, stream, early_launch);
}

cudaError_t launch_layer_norm_fp8(const LayerNormLaunch& launch, cudaStream_t stream, bool early_launch) {
    const cudaError_t status = launch_mode<LN_FP8_STATS>(launch, stream, early_launch);
    if (status != cudaSuccess) return status;
    // The cast launch needs the maximum of the launch above: with the programmatic-dependency
    // attribute it is scheduled while that one drains and waits (griddepcontrol.wait) before it reads
    // the word; without the attribute the wait does nothing and the stream orders the two.
    return launch.row_stats != nullptr ? launch_mode<LN_FP8_CAST_SAVED>(launch, stream, early_launch)
                                       : launch_mode<LN_FP8_CAST>(launch, stream, early_launch);
}

}  // namespace sdxlq
