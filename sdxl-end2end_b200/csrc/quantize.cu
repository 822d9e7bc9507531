// Activation / weight quantisers.
//
// rotate_quantize_int8_kernel fuses the reference's activation_amax_kernel and
// quantize_activation_kernel (src/cuda/int8_convrot.cu:265-353; same arithmetic as the weight
// pair at :156-249) into one pass that keeps the row in registers:
//   rotated = regular-Hadamard(group) * g^-1/2, amax over the row, scale = max(amax/127, 1e-30)
//   (1 if amax == 0), q = clamp(rn(rotated * (1/scale)), -128, 127).
// Four lanes own one 256-element chunk of a row. Lane q of the quad holds, for u = 0..7, the 8
// consecutive elements starting at 32*u + 8*q, i.e. index bits {0,1,2,5,6,7}; bits {3,4} are the
// lane. The radix-4 butterfly stages of the reference (:121-150, strides 1, 4, 16, 64) then need
// one lane exchange each for strides 4 and 16 and none for strides 1 and 64. Every output is
// evaluated with the reference's own association ((a+b)+c)-d, ((a+b)-c)+d, ((a-b)+c)+d,
// ((-a+b)+c)+d, so results are bit-identical to a sequential evaluation. Group sizes 4, 16, 64
// are the same butterflies with the later stages skipped.
//
// fp8_amax_kernel / fp8_cast_kernel restate quantize_tensor_fp8 (src/cuda/fp8_kernels.cu:16-49,
// 157-190): tensor-wide amax, scale = max(amax / FP8_MAX, 1e-12) (1 if amax == 0),
// q = FP8_satfinite(x * (1/scale)).
//
// The weight packers restate source_amax / finalize_fp8_scales / pack_to_fp8
// (src/cuda/weights.cu:119-170).

#include "quantize.cuh"
#include "fp8_math.cuh"
#include "int8_math.cuh"

namespace sdxlq {

namespace {

__device__ __forceinline__ void load8(const __half* source, bool vector_ok, uint32_t valid, float (&out)[8]) {
    if (vector_ok && valid == 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(source);
        const __half2* pairs = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(pairs[i]);
            out[2 * i] = f.x;
            out[2 * i + 1] = f.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = static_cast<uint32_t>(i) < valid ? __half2float(source[i]) : 0.0f;
    }
}

__device__ __forceinline__ void load8(const float* source, bool vector_ok, uint32_t valid, float (&out)[8]) {
    if (vector_ok && valid == 8) {
        const float4 lo = reinterpret_cast<const float4*>(source)[0];
        const float4 hi = reinterpret_cast<const float4*>(source)[1];
        out[0] = lo.x; out[1] = lo.y; out[2] = lo.z; out[3] = lo.w;
        out[4] = hi.x; out[5] = hi.y; out[6] = hi.z; out[7] = hi.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = static_cast<uint32_t>(i) < valid ? source[i] : 0.0f;
    }
}

// The four outputs of one radix-4 butterfly, each with the reference's association.
__device__ __forceinline__ float bf0(float a, float b, float c, float d) { return ((a + b) + c) - d; }
__device__ __forceinline__ float bf1(float a, float b, float c, float d) { return ((a + b) - c) + d; }
__device__ __forceinline__ float bf2(float a, float b, float c, float d) { return ((a - b) + c) + d; }
__device__ __forceinline__ float bf3(float a, float b, float c, float d) { return ((-a + b) + c) + d; }

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

template <typename In, bool Normalize>
__device__ __forceinline__ void rotate_quantize_rows(const QuantInt8Job& job, uint32_t local_block,
                                                     uint32_t* row_max_bits, float* row_partials) {
    const uint32_t threads_per_row = job.threads_per_row;
    const uint32_t row_in_block = threadIdx.x / threads_per_row;
    const uint32_t thread_in_row = threadIdx.x - row_in_block * threads_per_row;
    const uint32_t row = local_block * job.rows_per_block + row_in_block;
    const bool active = row_in_block < job.rows_per_block && row < job.m;
    const uint32_t quad_lane = thread_in_row & 3u;
    const uint32_t base_col = (thread_in_row >> 2) * 256u + quad_lane * 8u;
    const uint32_t k = job.k;
    const bool vector_ok = job.vector_ok != 0;
    const In* source = static_cast<const In*>(job.x) + static_cast<size_t>(row) * k;

    if (threadIdx.x < job.rows_per_block) row_max_bits[threadIdx.x] = 0;

    float v[8][8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const uint32_t col = base_col + 32u * u;
        uint32_t valid = 0;
        if (active && col < k) valid = min(8u, k - col);
        if (valid != 0) {
            load8(source + col, vector_ok, valid, v[u]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[u][i] = 0.0f;
        }
    }

    if constexpr (Normalize) {
        // LayerNorm of the row before it is rotated, with the arithmetic of the reference's
        // layer_norm_kernel (src/cuda/ops_kernels.cu:185-256): FP32 mean, FP32 mean of the centred
        // squares clamped at 0, rsqrtf(variance + epsilon), and the result rounded to FP16 like the
        // tensor the reference would hand to its quantiser. The partial sums of a row's threads are
        // added in thread order, so the result does not depend on scheduling.
        const float width = static_cast<float>(k);
        const uint32_t first = row_in_block * threads_per_row;
        float partial = 0.0f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
#pragma unroll
            for (int i = 0; i < 8; ++i) partial += v[u][i];                  // absent elements hold 0
        }
        row_partials[threadIdx.x] = partial;
        __syncthreads();
        float total = 0.0f;
        if (active) for (uint32_t t = 0; t < threads_per_row; ++t) total += row_partials[first + t];
        const float mean = __fdiv_rn(total, width);
        __syncthreads();
        partial = 0.0f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t col = base_col + 32u * u;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float centred = v[u][i] - mean;
                if (active && col + i < k) partial = fmaf(centred, centred, partial);
            }
        }
        row_partials[threadIdx.x] = partial;
        __syncthreads();
        total = 0.0f;
        if (active) for (uint32_t t = 0; t < threads_per_row; ++t) total += row_partials[first + t];
        const float variance = fmaxf(0.0f, __fdiv_rn(total, width));
        const float inverse = rsqrtf(variance + job.epsilon);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t col = base_col + 32u * u;
            uint32_t valid = 0;
            if (active && col < k) valid = min(8u, k - col);
            if (valid == 0) continue;
            float gamma[8], beta[8];
            load8(job.gamma + col, vector_ok, valid, gamma);
            load8(job.beta + col, vector_ok, valid, beta);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float normalised = fmaf(__fmul_rn(v[u][i] - mean, inverse), gamma[i], beta[i]);
                v[u][i] = static_cast<uint32_t>(i) < valid ? __half2float(__float2half_rn(normalised)) : 0.0f;
            }
        }
    }

    const uint32_t stages = job.stages;
    if (stages >= 1) {          // stride 1: index bits 0-1, in-lane
#pragma unroll
        for (int u = 0; u < 8; ++u) {
#pragma unroll
            for (int h = 0; h < 8; h += 4) {
                const float a = v[u][h], b = v[u][h + 1], c = v[u][h + 2], d = v[u][h + 3];
                v[u][h] = bf0(a, b, c, d);
                v[u][h + 1] = bf1(a, b, c, d);
                v[u][h + 2] = bf2(a, b, c, d);
                v[u][h + 3] = bf3(a, b, c, d);
            }
        }
    }
    if (stages >= 2) {          // stride 4: index bit 2 in-lane, bit 3 = quad lane bit 0
        const bool upper = (quad_lane & 1u) != 0;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
#pragma unroll
            for (int off = 0; off < 4; ++off) {
                const float lo = v[u][off], hi = v[u][off + 4];
                const float other_lo = __shfl_xor_sync(0xffffffffu, lo, 1);
                const float other_hi = __shfl_xor_sync(0xffffffffu, hi, 1);
                if (!upper) {   // holds a, b; partner holds c, d
                    v[u][off] = bf0(lo, hi, other_lo, other_hi);
                    v[u][off + 4] = bf1(lo, hi, other_lo, other_hi);
                } else {        // holds c, d; partner holds a, b
                    v[u][off] = bf2(other_lo, other_hi, lo, hi);
                    v[u][off + 4] = bf3(other_lo, other_hi, lo, hi);
                }
            }
        }
    }
    if (stages >= 3) {          // stride 16: index bit 4 = quad lane bit 1, bit 5 = u bit 0
        const bool upper = (quad_lane & 2u) != 0;
#pragma unroll
        for (int w = 0; w < 8; w += 2) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float lo = v[w][i], hi = v[w + 1][i];
                const float other_lo = __shfl_xor_sync(0xffffffffu, lo, 2);
                const float other_hi = __shfl_xor_sync(0xffffffffu, hi, 2);
                if (!upper) {   // holds a (u even), c (u odd); partner holds b, d
                    v[w][i] = bf0(lo, other_lo, hi, other_hi);
                    v[w + 1][i] = bf2(lo, other_lo, hi, other_hi);
                } else {        // holds b, d; partner holds a, c
                    v[w][i] = bf1(other_lo, lo, other_hi, hi);
                    v[w + 1][i] = bf3(other_lo, lo, other_hi, hi);
                }
            }
        }
    }
    if (stages >= 4) {          // stride 64: index bits 6-7 = u bits 1-2, in-lane
#pragma unroll
        for (int u0 = 0; u0 < 2; ++u0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float a = v[u0][i], b = v[u0 + 2][i], c = v[u0 + 4][i], d = v[u0 + 6][i];
                v[u0][i] = bf0(a, b, c, d);
                v[u0 + 2][i] = bf1(a, b, c, d);
                v[u0 + 4][i] = bf2(a, b, c, d);
                v[u0 + 6][i] = bf3(a, b, c, d);
            }
        }
    }

    // g^-1/2 is the exact power of two 2^-stages.
    const float normalization = __uint_as_float((127u - stages) << 23);
    float local_max = 0.0f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[u][i] = __fmul_rn(v[u][i], normalization);
            const float magnitude = fabsf(v[u][i]);
            if (magnitude <= 3.402823466e+38f && magnitude > local_max) local_max = magnitude;   // finite only
        }
    }
    local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, 1));
    local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, 2));
    __syncthreads();            // row_max_bits cleared
    if (active && quad_lane == 0) atomicMax(row_max_bits + row_in_block, __float_as_uint(local_max));
    __syncthreads();
    const float maximum = __uint_as_float(row_max_bits[active ? row_in_block : 0]);
    const float scale = maximum > 0.0f ? fmaxf(__fdiv_rn(maximum, 127.0f), 1.0e-30f) : 1.0f;
    const float inverse_scale = __fdiv_rn(1.0f, scale);
    if (active && thread_in_row == 0) job.scales[row] = scale;

    int8_t* destination = job.xq + static_cast<size_t>(row) * k;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const uint32_t col = base_col + 32u * u;
        if (!active || col >= k) continue;
        uint32_t packed[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int quantized = __float2int_rn(__fmul_rn(v[u][i], inverse_scale));
            quantized = max(-128, min(127, quantized));
            packed[i >> 2] |= (static_cast<uint32_t>(quantized) & 0xFFu) << (8 * (i & 3));
        }
        if (vector_ok && col + 8 <= k) {
            *reinterpret_cast<uint2*>(destination + col) = make_uint2(packed[0], packed[1]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (col + i < k) destination[col + i] = static_cast<int8_t>((packed[i >> 2] >> (8 * (i & 3))) & 0xFFu);
            }
        }
    }
}

__global__ void __launch_bounds__(256, 2)
rotate_quantize_int8_kernel(const __grid_constant__ QuantInt8Launch launch) {
    __shared__ uint32_t row_max_bits[64];
    wait_for_prior_kernels_then_release_next();
    const QuantInt8Job& job = find_job(launch, blockIdx.x);
    const uint32_t local_block = blockIdx.x - job.first_block;
    if (job.x_is_f32) rotate_quantize_rows<float, false>(job, local_block, row_max_bits, nullptr);
    else rotate_quantize_rows<__half, false>(job, local_block, row_max_bits, nullptr);
}

// The same pass with a LayerNorm of the FP16 row in front of the rotation (every job carries gamma /
// beta). A kernel of its own so that its larger register need does not weigh on the one above.
__global__ void __launch_bounds__(256, 1)
normalize_rotate_quantize_int8_kernel(const __grid_constant__ QuantInt8Launch launch) {
    __shared__ uint32_t row_max_bits[64];
    __shared__ float row_partials[256];
    wait_for_prior_kernels_then_release_next();
    const QuantInt8Job& job = find_job(launch, blockIdx.x);
    rotate_quantize_rows<__half, true>(job, blockIdx.x - job.first_block, row_max_bits, row_partials);
}

cudaError_t launch_rotate_quantize_int8(const QuantInt8Launch& launch, uint32_t blocks, uint32_t threads,
                                        cudaStream_t stream, bool early_launch) {
    if (launch.single.gamma != nullptr) {
        return launch_behind(normalize_rotate_quantize_int8_kernel, blocks, threads, 0, stream, early_launch, launch);
    }
    return launch_behind(rotate_quantize_int8_kernel, blocks, threads, 0, stream, early_launch, launch);
}

// ------------------------------------------------------------------------------------------
// FP8 activations
// ------------------------------------------------------------------------------------------
namespace {

__device__ __forceinline__ uint32_t find_job_index(const QuantFp8Launch& launch, uint32_t block) {
    if (launch.jobs == nullptr) return 0;
    if (launch.block_jobs != nullptr) return launch.block_jobs[block];
    uint32_t lo = 0, hi = launch.num_jobs;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (launch.jobs[mid].first_block <= block) lo = mid; else hi = mid;
    }
    return lo;
}

}  // namespace

__global__ void __launch_bounds__(256)
fp8_amax_kernel(const __grid_constant__ QuantFp8Launch launch) {
    wait_for_prior_kernels_then_release_next();      // the cast kernel may be scheduled while this one runs
    const uint32_t job_index = find_job_index(launch, blockIdx.x);
    const QuantFp8Job& job = launch.jobs == nullptr ? launch.single : launch.jobs[job_index];
    if (job.amax_in != nullptr) return;                                  // the producer of x left the maximum
    const uint32_t local_block = blockIdx.x - job.first_block;
    const __half* source = static_cast<const __half*>(job.x);
    const size_t count = job.count;
    float local = 0.0f;
    if (job.vector_ok) {
        // Four 16-byte loads in flight per thread; the maximum of FP16 values is one of them, so it is
        // taken in half precision (NaN never wins, as with fmaxf).
        const size_t vectors = count / 8;
        const size_t step = static_cast<size_t>(job.num_blocks) * blockDim.x;
        const uint4* const vector_source = reinterpret_cast<const uint4*>(source);
        __half2 maximum2 = __float2half2_rn(0.0f);
        for (size_t index = static_cast<size_t>(local_block) * blockDim.x + threadIdx.x; index < vectors; index += 4 * step) {
            uint4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                raw[u] = index + u * step < vectors ? __ldg(vector_source + index + u * step) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                maximum2 = __hmax2(maximum2, __hmax2(__habs2(as_half2(raw[u].x)), __habs2(as_half2(raw[u].y))));
                maximum2 = __hmax2(maximum2, __hmax2(__habs2(as_half2(raw[u].z)), __habs2(as_half2(raw[u].w))));
            }
        }
        local = fmaxf(__low2float(maximum2), __high2float(maximum2));
        if (local_block == 0) {
            for (size_t index = vectors * 8 + threadIdx.x; index < count; index += blockDim.x) {
                local = fmaxf(local, fabsf(__half2float(source[index])));
            }
        }
    } else {
        for (size_t index = static_cast<size_t>(local_block) * blockDim.x + threadIdx.x; index < count;
             index += static_cast<size_t>(job.num_blocks) * blockDim.x) {
            local = fmaxf(local, fabsf(__half2float(source[index])));
        }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, offset));
    }
    __shared__ float warp_max[8];
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        float block_max = 0.0f;
        for (uint32_t w = 0; w < (blockDim.x + 31) / 32; ++w) block_max = fmaxf(block_max, warp_max[w]);
        atomicMax(launch.amax_bits + job_index, __float_as_uint(block_max));
    }
}

__global__ void __launch_bounds__(256)
fp8_cast_kernel(const __grid_constant__ QuantFp8Launch launch) {
    wait_for_prior_kernels_then_release_next();      // the maxima of fp8_amax_kernel (or of the producer of x) are complete
    const uint32_t job_index = find_job_index(launch, blockIdx.x);
    const QuantFp8Job& job = launch.jobs == nullptr ? launch.single : launch.jobs[job_index];
    const uint32_t local_block = blockIdx.x - job.first_block;
    // One thread reads the job's maximum and counts this block among its readers; the block that
    // completes the count clears the maximum and the counter, so the next call (and every replay of
    // a captured graph) finds both words zero without any host-side bookkeeping.
    __shared__ uint32_t maximum_bits;
    if (threadIdx.x == 0) {
        uint32_t* const word = job.amax_in != nullptr ? job.amax_in : launch.amax_bits + job_index;
        maximum_bits = *reinterpret_cast<volatile uint32_t*>(word);
        __threadfence();
        if (atomicAdd(launch.done_counts + job_index, 1u) == job.num_blocks - 1u) {
            *word = 0;
            launch.done_counts[job_index] = 0;
        }
    }
    __syncthreads();
    const float scale = fp8_scale_from_amax(__uint_as_float(maximum_bits), job.fmt);
    const float inverse_scale = __fdiv_rn(1.0f, scale);
    if (local_block == 0 && threadIdx.x == 0) *job.scale_out = scale;
    const __half* source = static_cast<const __half*>(job.x);
    uint8_t* destination = job.q;
    const size_t count = job.count;
    const uint32_t fmt = job.fmt;
    if (job.vector_ok) {
        // Four 16-byte loads in flight per thread, walking the tensor from its end to its start: what
        // the maximum kernel read last is what may still sit in L2.
        const size_t vectors = count / 8;
        const size_t step = static_cast<size_t>(job.num_blocks) * blockDim.x;
        const uint4* const vector_source = reinterpret_cast<const uint4*>(source);
        const float2 inverse_scale2 = make_float2(inverse_scale, inverse_scale);
        for (size_t index = static_cast<size_t>(local_block) * blockDim.x + threadIdx.x; index < vectors; index += 4 * step) {
            uint4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                raw[u] = index + u * step < vectors ? __ldg(vector_source + (vectors - 1 - (index + u * step))) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (index + u * step >= vectors) break;
                const uint32_t words[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
                uint32_t packed[2];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 scaled = __fmul2_rn(__half22float2(as_half2(words[i])), inverse_scale2);
                    const uint32_t two = encode_fp8x2(scaled.x, scaled.y, fmt);
                    if ((i & 1) == 0) packed[i >> 1] = two & 0xFFFFu;
                    else packed[i >> 1] |= (two & 0xFFFFu) << 16;
                }
                reinterpret_cast<uint2*>(destination)[vectors - 1 - (index + u * step)] = make_uint2(packed[0], packed[1]);
            }
        }
        if (local_block == 0) {
            for (size_t index = vectors * 8 + threadIdx.x; index < count; index += blockDim.x) {
                destination[index] = encode_fp8(__fmul_rn(__half2float(source[index]), inverse_scale), fmt);
            }
        }
    } else {
        for (size_t index = static_cast<size_t>(local_block) * blockDim.x + threadIdx.x; index < count;
             index += static_cast<size_t>(job.num_blocks) * blockDim.x) {
            destination[index] = encode_fp8(__fmul_rn(__half2float(source[index]), inverse_scale), fmt);
        }
    }
}

cudaError_t launch_fp8_quantize(const QuantFp8Launch& launch, uint32_t blocks, cudaStream_t stream, bool early_launch,
                                bool skip_maximum_pass) {
    // skip_maximum_pass: every job of the launch carries its maximum (amax_in), nothing to reduce
    if (!skip_maximum_pass) {
        const cudaError_t status = launch_behind(fp8_amax_kernel, blocks, 256, 0, stream, early_launch, launch);
        if (status != cudaSuccess) return status;
    }
    // The cast kernel needs the maxima of the kernel above. Launched with the programmatic-dependency
    // attribute it is scheduled while that kernel runs and waits (griddepcontrol.wait) before it reads
    // them; without the attribute the wait does nothing and the stream orders the two.
    return launch_behind(fp8_cast_kernel, blocks, 256, 0, stream, early_launch, launch);
}

// ------------------------------------------------------------------------------------------
// Load-time FP8 weight packers (not on the per-step path)
// ------------------------------------------------------------------------------------------
namespace {

__device__ __forceinline__ float read_weight(const void* source, int32_t dtype, size_t index) {
    if (dtype == 3) return __half2float(static_cast<const __half*>(source)[index]);
    if (dtype == 4) return static_cast<const float*>(source)[index];
    const __half_raw raw = __nv_cvt_fp8_to_halfraw(static_cast<const uint8_t*>(source)[index],
                                                   dtype == 0 ? __NV_E4M3 : __NV_E5M2);
    return __half2float(__half(raw));
}

}  // namespace

// One block per output row: amax over finite |w| of the row, combined into slot `row` (per
// channel) or slot 0 (tensor wide). `amax_bits` must be zero on entry.
__global__ void __launch_bounds__(256)
fp8_weight_amax_kernel(const void* source, int32_t dtype, uint32_t n, uint32_t k, uint32_t per_channel,
                       uint32_t* amax_bits) {
    const uint32_t row = blockIdx.x;
    float local = 0.0f;
    for (uint32_t col = threadIdx.x; col < k; col += blockDim.x) {
        const float magnitude = fabsf(read_weight(source, dtype, static_cast<size_t>(row) * k + col));
        if (magnitude <= 3.402823466e+38f && magnitude > local) local = magnitude;
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, offset));
    }
    if ((threadIdx.x & 31) == 0) atomicMax(amax_bits + (per_channel ? row : 0), __float_as_uint(local));
}

// scales[] holds the amax bit patterns on entry of the finalize kernel and the scales on exit.
__global__ void fp8_weight_finalize_kernel(float* scales, uint32_t count, uint32_t fmt) {
    const uint32_t index = blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= count) return;
    scales[index] = fp8_scale_from_amax(scales[index], fmt);
}

__global__ void __launch_bounds__(256)
fp8_weight_pack_kernel(const void* source, int32_t dtype, uint32_t n, uint32_t k, uint32_t fmt,
                       uint32_t per_channel, uint32_t k_major, const float* scales, uint8_t* destination) {
    const uint32_t row = blockIdx.x;
    const float scale = scales[per_channel ? row : 0];
    for (uint32_t col = threadIdx.x; col < k; col += blockDim.x) {
        const float value = read_weight(source, dtype, static_cast<size_t>(row) * k + col);
        const size_t index = k_major ? static_cast<size_t>(col) * n + row : static_cast<size_t>(row) * k + col;
        destination[index] = encode_fp8(__fdiv_rn(value, scale), fmt);
    }
}

__global__ void fill_f32_kernel(float* values, uint32_t count, float value) {
    const uint32_t index = blockIdx.x * blockDim.x + threadIdx.x;
    if (index < count) values[index] = value;
}

cudaError_t launch_fp8_weight_pack(const void* source, int32_t dtype, uint32_t n, uint32_t k, uint32_t fmt,
                                   uint32_t per_channel, uint32_t k_major, uint8_t* destination,
                                   float* scales, cudaStream_t stream) {
    const uint32_t scale_count = per_channel ? n : 1;
    cudaError_t status = cudaMemsetAsync(scales, 0, scale_count * sizeof(float), stream);
    if (status != cudaSuccess) return status;
    fp8_weight_amax_kernel<<<n, 256, 0, stream>>>(source, dtype, n, k, per_channel,
                                                  reinterpret_cast<uint32_t*>(scales));
    fp8_weight_finalize_kernel<<<(scale_count + 255) / 256, 256, 0, stream>>>(scales, scale_count, fmt);
    fp8_weight_pack_kernel<<<n, 256, 0, stream>>>(source, dtype, n, k, fmt, per_channel, k_major, scales,
                                                  destination);
    return cudaGetLastError();
}

cudaError_t launch_fill_f32(float* values, uint32_t count, float value, cudaStream_t stream) {
    fill_f32_kernel<<<(count + 255) / 256, 256, 0, stream>>>(values, count, value);
    return cudaGetLastError();
}

}  // namespace sdxlq
