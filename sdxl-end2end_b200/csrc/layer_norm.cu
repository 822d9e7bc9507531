// LayerNorm over the last dimension, alone or fused with the FP8 activation quantiser that feeds the
// next projection.
//
// Arithmetic of the reference's layer_norm_kernel / layer_norm_fixed_kernel
// (src/cuda/ops_kernels.cu:185-256, launched by Ops::layer_norm at :1425-1470): FP32 sum -> mean,
// FP32 sum of the centred squares -> variance = max(0, sum / width), inverse = rsqrtf(variance +
// epsilon), y = half_rn((x - mean) * inverse * gamma + beta). The reference gives a row to a block and
// adds the partial sums through a shared-memory tree; here a warp owns a row, every lane adds its
// elements in column order and the lanes are combined by a butterfly of shuffles. Only the order of
// the FP32 additions differs, which moves the sums in their last bits; results are deterministic.
//
// The row stays in registers between the three steps (one 16-byte load per eight elements, no
// re-read), so the FP16 form moves 2 + 2 bytes per element. The FP8 form needs max |y| of the whole
// tensor before the first byte can be written: a statistics launch normalises and only reduces the
// maximum (2 bytes per element read), the cast launch normalises again and writes FP8 (2 read, 1
// written). 5 bytes per element against 9 for LayerNorm followed by the stand-alone quantiser.
// The unrotated INT8 form is one launch: the normalised row is kept as packed halves, its maximum is
// a warp reduction, and the bytes are written at once (2 read, 1 written).

#include "quantize.cuh"
#include "fp8_math.cuh"
#include "int8_math.cuh"

namespace sdxlq {

namespace {

enum : int { LN_F16 = 0, LN_FP8_STATS = 1, LN_FP8_CAST = 2, LN_INT8 = 3 };

constexpr uint32_t kRowsPerBlock = 8;      // one warp per row, 256 threads

__device__ __forceinline__ float warp_sum(float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_xor_sync(0xffffffffu, value, offset);
    return value;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&out)[8]) {
    const __half2* pairs = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(pairs[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}

// kVectors 16-byte vectors per lane: rows of up to 256 * kVectors elements. The row is held as packed
// halves (converted on the fly in each of the three passes over the registers) and the next row of
// the warp is requested before the current one is worked on, so that the loads of one row overlap
// the arithmetic of the other; gamma and beta sit in shared memory. That keeps the register need
// low enough for three blocks (24 warps) per SM (two for rows wider than 1280).
template <int kVectors, int Mode>
__global__ void __launch_bounds__(256, kVectors > 5 ? 2 : 3)
layer_norm_rows_kernel(const __grid_constant__ LayerNormLaunch p) {
    // A kernel launched behind this one with the programmatic-dependency attribute may begin its
    // set-up now; it waits for this kernel's completion before it reads the results.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ uint4 gamma_beta[2][kVectors * 32];
    __shared__ uint32_t maximum_bits;
    __shared__ float warp_max[kRowsPerBlock];
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t vectors = p.width / 8;
    const float width = static_cast<float>(p.width);

    for (uint32_t vector = threadIdx.x; vector < vectors; vector += blockDim.x) {
        gamma_beta[0][vector] = reinterpret_cast<const uint4*>(p.gamma)[vector];
        gamma_beta[1][vector] = reinterpret_cast<const uint4*>(p.beta)[vector];
    }

    const uint32_t stride = gridDim.x * kRowsPerBlock;
    uint32_t row = blockIdx.x * kRowsPerBlock + warp;
    uint4 raw[kVectors];
    auto request = [&](uint32_t which, uint4 (&into)[kVectors]) {
        const uint4* source = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(which) * p.width);
#pragma unroll
        for (int j = 0; j < kVectors; ++j) {
            const uint32_t vector = static_cast<uint32_t>(j) * 32u + lane;
            into[j] = (which < p.rows && vector < vectors) ? __ldg(source + vector) : make_uint4(0, 0, 0, 0);
        }
    };
    request(row, raw);                  // the input does not depend on the launch before this one

    float inverse_scale = 1.0f;
    if constexpr (Mode == LN_FP8_CAST) {
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
    if constexpr (Mode == LN_FP8_CAST) {
        const float scale = fp8_scale_from_amax(__uint_as_float(maximum_bits), p.fmt);
        inverse_scale = __fdiv_rn(1.0f, scale);
        if (blockIdx.x == 0 && threadIdx.x == 0) *p.scale_out = scale;
    }

    float local_max = 0.0f;
    for (; row < p.rows; row += stride) {
        uint4 next[kVectors];
        request(row + stride, next);
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < kVectors; ++j) {
            float f[8];
            unpack8(raw[j], f);          // vectors past the row hold zeros
#pragma unroll
            for (int i = 0; i < 8; ++i) sum += f[i];
        }
        const float mean = __fdiv_rn(warp_sum(sum), width);
        float squares = 0.0f;
#pragma unroll
        for (int j = 0; j < kVectors; ++j) {
            if (static_cast<uint32_t>(j) * 32u + lane < vectors) {
                float f[8];
                unpack8(raw[j], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float centred = f[i] - mean;
                    squares = fmaf(centred, centred, squares);
                }
            }
        }
        const float variance = fmaxf(0.0f, __fdiv_rn(warp_sum(squares), width));
        const float inverse = rsqrtf(variance + p.epsilon);

#pragma unroll
        for (int j = 0; j < kVectors; ++j) {
            const uint32_t vector = static_cast<uint32_t>(j) * 32u + lane;
            if (vector >= vectors) continue;
            float f[8], g[8], b[8];
            unpack8(raw[j], f);
            unpack8(gamma_beta[0][vector], g);
            unpack8(gamma_beta[1][vector], b);
            __half2 result[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float lo = fmaf(__fmul_rn(f[2 * i] - mean, inverse), g[2 * i], b[2 * i]);
                const float hi = fmaf(__fmul_rn(f[2 * i + 1] - mean, inverse), g[2 * i + 1], b[2 * i + 1]);
                result[i] = __floats2half2_rn(lo, hi);
            }
            if constexpr (Mode == LN_F16) {
                reinterpret_cast<uint4*>(p.y + static_cast<size_t>(row) * p.width)[vector] =
                    *reinterpret_cast<const uint4*>(result);
            } else if constexpr (Mode == LN_INT8) {
                raw[j] = *reinterpret_cast<const uint4*>(result);     // kept until the row's maximum is known
            } else if constexpr (Mode == LN_FP8_STATS) {
                // the maximum of FP16 values is one of them: exact in half precision
                __half2 m = __hmax2(__habs2(result[0]), __habs2(result[1]));
                m = __hmax2(m, __hmax2(__habs2(result[2]), __habs2(result[3])));
                const float2 both = __half22float2(m);
                local_max = fmaxf(local_max, fmaxf(both.x, both.y));
            } else {
                uint32_t packed[2];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 both = __half22float2(result[i]);
                    const uint32_t two = encode_fp8x2(__fmul_rn(both.x, inverse_scale), __fmul_rn(both.y, inverse_scale), p.fmt);
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
                maximum2 = __hmax2(maximum2, __hmax2(__habs2(as_half2(raw[j].x)), __habs2(as_half2(raw[j].y))));
                maximum2 = __hmax2(maximum2, __hmax2(__habs2(as_half2(raw[j].z)), __habs2(as_half2(raw[j].w))));
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
            const float inverse = __fdiv_rn(1.0f, scale);
            if (lane == 0) p.scale_out[row] = scale;
            uint2* destination = reinterpret_cast<uint2*>(p.q + static_cast<size_t>(row) * p.width);
#pragma unroll
            for (int j = 0; j < kVectors; ++j) {
                const uint32_t vector = static_cast<uint32_t>(j) * 32u + lane;
                if (vector < vectors) destination[vector] = quantize_vector(raw[j], inverse);
            }
        }
#pragma unroll
        for (int j = 0; j < kVectors; ++j) raw[j] = next[j];
    }

    if constexpr (Mode == LN_FP8_STATS) {
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, offset));
        }
        if (lane == 0) warp_max[warp] = local_max;
        __syncthreads();
        if (threadIdx.x == 0) {
            float block_max = 0.0f;
            for (uint32_t w = 0; w < kRowsPerBlock; ++w) block_max = fmaxf(block_max, warp_max[w]);
            // NaN never wins a maximum here (fmaxf drops it), like the reference's fmaxf reduction
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

cudaError_t launch_layer_norm_f16(const LayerNormLaunch& launch, cudaStream_t stream) {
    return launch_mode<LN_F16>(launch, stream, false);
}

cudaError_t launch_layer_norm_int8(const LayerNormLaunch& launch, cudaStream_t stream) {
    return launch_mode<LN_INT8>(launch, stream, false);
}

cudaError_t launch_layer_norm_fp8(const LayerNormLaunch& launch, cudaStream_t stream, bool early_launch) {
    const cudaError_t status = launch_mode<LN_FP8_STATS>(launch, stream, false);
    if (status != cudaSuccess) return status;
    // The cast launch needs the maximum of the launch above: with the programmatic-dependency
    // attribute it is scheduled while that one drains and waits (griddepcontrol.wait) before it reads
    // the word; without the attribute the wait does nothing and the stream orders the two.
    return launch_mode<LN_FP8_CAST>(launch, stream, early_launch);
}

}  // namespace sdxlq
