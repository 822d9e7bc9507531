// GroupNorm (+ SiLU) for channels-last FP16 activations: scaffolding of the synthetic UNet loop, NOT part
// of the quantized-Linear path. The loop's convolutions run channels-last (what the tensor-core
// convolution kernels want); PyTorch's group_norm copies such a tensor to NCHW, normalises, and the
// next convolution copies it back: 18 bytes moved per element for a 6-byte operation. These two
// kernels read [batch, rows, channels] (NHWC memory) in place:
//   statistics  per (batch, row chunk): FP32 sum and sum of squares of every channel over the chunk's
//               rows (16-byte loads, eight channels per thread), folded to the groups in shared memory,
//               written as partial sums
//               (the block that finishes last for a batch element adds them up in a fixed order, in double
//               precision, and leaves mean and inverse standard deviation per group: deterministic)
//   apply       y = (x - mean) * inverse * gamma + beta, optional SiLU, FP16 out in the same layout
// with the arithmetic of the reference's group_norm_kernel (src/cuda/ops_kernels.cu:258-308:
// inverse = rsqrtf(max(0, variance) + epsilon), normalised / (1 + expf(-normalised)) for SiLU), except
// that the variance is E[x^2] - mean^2 from one pass instead of a second pass over centred values.
// An optional per-(batch, channel) FP16 bias is added first and rounded to FP16, which is the
// reference's add_spatial_bias (the resnet's time-embedding projection, src/cuda/unet.cpp:69-72)
// followed by the norm, without the tensor in between.

#include "quantize.cuh"

namespace sdxlq {

namespace {

constexpr uint32_t kMaxNormThreads = 384;       // a block is (channels / 8) vectors x as many rows as fit
constexpr uint32_t kMaxNormChannels = 8 * kMaxNormThreads;
constexpr uint32_t kRowsInFlight = 4;           // 16-byte loads every thread keeps outstanding

// Thread t of a block works on the 8 channels of vector t % V (V = channels / 8) of row slot t / V; the
// block covers R = blockDim / V rows at once and every thread keeps kRowsInFlight rows in flight. Sums are
// kept per channel, so the 16-byte vectors need not line up with the group boundaries (10, 30 or 60
// channels per group do not).
__device__ __forceinline__ void load_vector(const __half* row, uint32_t vector, const __half* bias_row, float (&out)[8]) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row) + vector);
    const __half2* pairs = reinterpret_cast<const __half2*>(&raw);
    if (bias_row == nullptr) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __half22float2(pairs[i]);
            out[2 * i] = v.x;
            out[2 * i + 1] = v.y;
        }
    } else {
        // add_spatial_bias: half_rn(float(x) + float(bias)), the tensor the reference normalises
        const uint4 bias_raw = __ldg(reinterpret_cast<const uint4*>(bias_row) + vector);
        const __half2* bias_pairs = reinterpret_cast<const __half2*>(&bias_raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __half22float2(__hadd2(pairs[i], bias_pairs[i]));
            out[2 * i] = v.x;
            out[2 * i + 1] = v.y;
        }
    }
}

__global__ void __launch_bounds__(kMaxNormThreads)
group_norm_stats_kernel(const GroupNormLaunch p) {
    __shared__ float channel_sums[kMaxNormThreads * 8][2];      // [row slot][channel]
    __shared__ uint32_t ticket;
    __shared__ double lane_sums[64][8][2];
    const uint32_t batch = blockIdx.y;
    const uint32_t chunk = blockIdx.x;
    const uint32_t vectors = p.channels / 8;
    const uint32_t rows_at_once = blockDim.x / vectors;
    const uint32_t slot = threadIdx.x / vectors;
    const uint32_t vector = threadIdx.x - slot * vectors;
    const uint32_t first_row = chunk * p.rows_per_chunk;
    const uint32_t last_row = min(p.rows, first_row + p.rows_per_chunk);
    const __half* base = p.x + static_cast<size_t>(batch) * p.rows * p.channels;
    const __half* bias_row = p.channel_bias != nullptr ? p.channel_bias + static_cast<size_t>(batch) * p.channels : nullptr;

    float sum[8] = {}, squares[8] = {};
    const uint32_t step = rows_at_once * kRowsInFlight;
    for (uint32_t row0 = first_row + slot; row0 < last_row; row0 += step) {
        float v[kRowsInFlight][8];
#pragma unroll
        for (uint32_t u = 0; u < kRowsInFlight; ++u) {
            const uint32_t row = row0 + u * rows_at_once;
            if (row < last_row) {
                load_vector(base + static_cast<size_t>(row) * p.channels, vector, bias_row, v[u]);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[u][i] = 0.0f;
            }
        }
#pragma unroll
        for (uint32_t u = 0; u < kRowsInFlight; ++u) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                sum[i] += v[u][i];
                squares[i] = fmaf(v[u][i], v[u][i], squares[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        channel_sums[slot * p.channels + vector * 8 + i][0] = sum[i];
        channel_sums[slot * p.channels + vector * 8 + i][1] = squares[i];
    }
    __syncthreads();
    // one thread per group adds its channels: row slots in order, channels in order
    if (threadIdx.x < p.groups) {
        const uint32_t channels_per_group = p.channels / p.groups;
        float total = 0.0f, total_squares = 0.0f;
        for (uint32_t s = 0; s < rows_at_once; ++s) {
            for (uint32_t j = 0; j < channels_per_group; ++j) {
                const uint32_t index = s * p.channels + threadIdx.x * channels_per_group + j;
                total += channel_sums[index][0];
                total_squares += channel_sums[index][1];
            }
        }
        float* out = p.partials + ((static_cast<size_t>(batch) * gridDim.x + chunk) * p.groups + threadIdx.x) * 2;
        out[0] = total;
        out[1] = total_squares;
    }
    // The block that finishes last for this batch element turns the partial sums into mean and inverse
    // standard deviation per group. Its additions run in a fixed order: L threads per group (8 when the
    // block has that many, else 4 or 2) take the chunks l, l + L, ... with four loads in flight each, then the
    // L results are added in order, in double precision.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket = atomicAdd(p.counters + batch, 1u);
    __syncthreads();
    if (ticket != gridDim.x - 1u) return;
    __threadfence();
    // a block has at least 193 threads and a launch at most 64 groups: 2 lanes always fit
    const uint32_t lanes = p.groups * 8u <= blockDim.x ? 8u : p.groups * 4u <= blockDim.x ? 4u : 2u;
    if (threadIdx.x < p.groups * lanes) {
        const uint32_t group = threadIdx.x / lanes, part = threadIdx.x % lanes;
        double total = 0.0, total_squares = 0.0;
        const float2* partial = reinterpret_cast<const float2*>(p.partials) + static_cast<size_t>(batch) * gridDim.x * p.groups + group;
        for (uint32_t c = part; c < gridDim.x; c += 4u * lanes) {
            float2 value[4];
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u) {
                const uint32_t chunk_index = c + u * lanes;
                value[u] = chunk_index < gridDim.x ? __ldcg(partial + static_cast<size_t>(chunk_index) * p.groups) : make_float2(0.0f, 0.0f);
            }
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u) {
                total += static_cast<double>(value[u].x);
                total_squares += static_cast<double>(value[u].y);
            }
        }
        lane_sums[group][part][0] = total;
        lane_sums[group][part][1] = total_squares;
    }
    __syncthreads();
    if (threadIdx.x < p.groups) {
        double total = 0.0, total_squares = 0.0;
        for (uint32_t part = 0; part < lanes; ++part) {
            total += lane_sums[threadIdx.x][part][0];
            total_squares += lane_sums[threadIdx.x][part][1];
        }
        const double count = static_cast<double>(p.rows) * (p.channels / p.groups);
        const double mean = total / count;
        const double variance = fmax(0.0, total_squares / count - mean * mean);
        float* final_values = p.finals + (static_cast<size_t>(batch) * 64u + threadIdx.x) * 2;
        final_values[0] = static_cast<float>(mean);
        final_values[1] = rsqrtf(static_cast<float>(variance) + p.epsilon);
    }
    if (threadIdx.x == 0) p.counters[batch] = 0;          // ready for the next launch (and for a graph replay)
}

__global__ void __launch_bounds__(kMaxNormThreads, 2)
group_norm_apply_kernel(const GroupNormLaunch p) {
    __shared__ float group_mean[64], group_inverse[64];
    const uint32_t batch = blockIdx.y;
    const uint32_t chunk = blockIdx.x;
    const uint32_t vectors = p.channels / 8;
    const uint32_t rows_at_once = blockDim.x / vectors;
    const uint32_t slot = threadIdx.x / vectors;
    const uint32_t vector = threadIdx.x - slot * vectors;
    if (threadIdx.x < p.groups) {
        const float* final_values = p.finals + (static_cast<size_t>(batch) * 64u + threadIdx.x) * 2;
        group_mean[threadIdx.x] = final_values[0];
        group_inverse[threadIdx.x] = final_values[1];
    }
    __syncthreads();

    const uint32_t channels_per_group = p.channels / p.groups;
    float mean[8], slope[8], beta[8];             // y = (x - mean) * (inverse * gamma) + beta
    {
        const uint4 gamma_raw = __ldg(reinterpret_cast<const uint4*>(p.gamma) + vector);
        const uint4 beta_raw = __ldg(reinterpret_cast<const uint4*>(p.beta) + vector);
        const __half* gamma_halves = reinterpret_cast<const __half*>(&gamma_raw);
        const __half* beta_halves = reinterpret_cast<const __half*>(&beta_raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t group = (vector * 8 + i) / channels_per_group;
            mean[i] = group_mean[group];
            slope[i] = group_inverse[group] * __half2float(gamma_halves[i]);
            beta[i] = __half2float(beta_halves[i]);
        }
    }
    const uint32_t first_row = chunk * p.rows_per_chunk;
    const uint32_t last_row = min(p.rows, first_row + p.rows_per_chunk);
    const __half* base = p.x + static_cast<size_t>(batch) * p.rows * p.channels;
    __half* out_base = p.y + static_cast<size_t>(batch) * p.rows * p.channels;
    const __half* bias_row = p.channel_bias != nullptr ? p.channel_bias + static_cast<size_t>(batch) * p.channels : nullptr;
    const uint32_t step = rows_at_once * kRowsInFlight;
    for (uint32_t row0 = first_row + slot; row0 < last_row; row0 += step) {
        float v[kRowsInFlight][8];
#pragma unroll
        for (uint32_t u = 0; u < kRowsInFlight; ++u) {
            const uint32_t row = row0 + u * rows_at_once;
            if (row < last_row) load_vector(base + static_cast<size_t>(row) * p.channels, vector, bias_row, v[u]);
        }
#pragma unroll
        for (uint32_t u = 0; u < kRowsInFlight; ++u) {
            const uint32_t row = row0 + u * rows_at_once;
            if (row >= last_row) break;
            uint4 out;
            __half2* out_pairs = reinterpret_cast<__half2*>(&out);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float lo = fmaf(v[u][2 * i] - mean[2 * i], slope[2 * i], beta[2 * i]);
                float hi = fmaf(v[u][2 * i + 1] - mean[2 * i + 1], slope[2 * i + 1], beta[2 * i + 1]);
                if (p.silu != 0) {
                    lo = __fdividef(lo, 1.0f + __expf(-lo));
                    hi = __fdividef(hi, 1.0f + __expf(-hi));
                }
                out_pairs[i] = __floats2half2_rn(lo, hi);
            }
            reinterpret_cast<uint4*>(out_base + static_cast<size_t>(row) * p.channels)[vector] = out;
        }
    }
}

// y[r, c] = half(half(x[r, c] + bias[c]) + residual[r, c]): a convolution's bias add and the resnet's
// residual add (Ops::add, src/cuda/unet.cpp:92) in one pass over the channels-last tensor instead of two.
// Eight channels per thread (16-byte accesses); channels is a multiple of 8.
__global__ void __launch_bounds__(256)
bias_residual_add_kernel(const __half* x, const __half* bias, const __half* residual, __half* y, size_t vectors,
                         uint32_t vectors_per_row) {
    for (size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; index < vectors;
         index += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint4 xv = reinterpret_cast<const uint4*>(x)[index];
        const uint4 bv = reinterpret_cast<const uint4*>(bias)[index % vectors_per_row];
        const uint4 rv = reinterpret_cast<const uint4*>(residual)[index];
        const __half2* xs = reinterpret_cast<const __half2*>(&xv);
        const __half2* bs = reinterpret_cast<const __half2*>(&bv);
        const __half2* rs = reinterpret_cast<const __half2*>(&rv);
        uint4 out;
        __half2* os = reinterpret_cast<__half2*>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) os[i] = __hadd2(__hadd2(xs[i], bs[i]), rs[i]);
        reinterpret_cast<uint4*>(y)[index] = out;
    }
}

}  // namespace

cudaError_t launch_bias_residual_add(const __half* x, const __half* bias, const __half* residual, __half* y, uint64_t rows,
                                     uint32_t channels, uint32_t sm_count, cudaStream_t stream) {
    const size_t vectors = static_cast<size_t>(rows) * channels / 8;
    const size_t wanted = (vectors + 255) / 256;
    const uint32_t blocks = static_cast<uint32_t>(wanted < static_cast<size_t>(sm_count) * 16 ? (wanted == 0 ? 1 : wanted) : sm_count * 16);
    bias_residual_add_kernel<<<blocks, 256, 0, stream>>>(x, bias, residual, y, vectors, channels / 8);
    return cudaGetLastError();
}

uint32_t group_norm_max_channels() { return kMaxNormChannels; }

cudaError_t launch_group_norm_nhwc(const GroupNormLaunch& launch, uint32_t chunks, cudaStream_t stream) {
    const dim3 grid(chunks, launch.batch, 1);
    const uint32_t vectors = launch.channels / 8;
    const uint32_t threads = vectors * (kMaxNormThreads / vectors);       // whole rows of vectors, at most 384 threads
    group_norm_stats_kernel<<<grid, threads, 0, stream>>>(launch);
    const cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return status;
    group_norm_apply_kernel<<<grid, threads, 0, stream>>>(launch);
    return cudaGetLastError();
}

}  // namespace sdxlq
