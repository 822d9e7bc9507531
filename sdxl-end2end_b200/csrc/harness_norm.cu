// GroupNorm (+ SiLU) for channels-last FP16 activations: scaffolding of the synthetic UNet loop, NOT part
// of the quantized-Linear path. The loop's convolutions run channels-last (what the tensor-core
// convolution kernels want); PyTorch's group_norm copies such a tensor to NCHW, normalises, and the
// next convolution copies it back: 18 bytes moved per element for a 6-byte operation. These two
// kernels read [batch, rows, channels] (NHWC memory) in place:
//   statistics  per (batch, row chunk): FP32 sum and sum of squares of every channel pair over the
//               chunk's rows, folded to the 32 groups in shared memory, written as partial sums
//   apply       every block first adds the partial sums of its batch element in chunk order (double
//               precision: deterministic, no atomics), then y = (x - mean) * inverse * gamma + beta,
//               optional SiLU, FP16 out in the same layout
// with the arithmetic of the reference's group_norm_kernel (src/cuda/ops_kernels.cu:258-308:
// inverse = rsqrtf(max(0, variance) + epsilon), normalised / (1 + expf(-normalised)) for SiLU), except
// that the variance is E[x^2] - mean^2 from one pass instead of a second pass over centred values.
// An optional per-(batch, channel) FP16 bias is added first and rounded to FP16, which is the
// reference's add_spatial_bias (the resnet's time-embedding projection, src/cuda/unet.cpp:69-72)
// followed by the norm, without the tensor in between.

#include "quantize.cuh"

namespace sdxlq {

namespace {

constexpr uint32_t kNormThreads = 320;          // channel pairs are dealt round-robin to the threads
constexpr uint32_t kMaxPairsPerThread = 4;      // channels <= 2 * 320 * 4 = 2560

__device__ __forceinline__ float2 load_pair(const __half* row, uint32_t pair, const __half* bias_row) {
    const float2 v = __half22float2(*reinterpret_cast<const __half2*>(row + 2 * pair));
    if (bias_row == nullptr) return v;
    // add_spatial_bias: half_rn(float(x) + float(bias)), the tensor the reference normalises
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(bias_row + 2 * pair));
    return __half22float2(__floats2half2_rn(v.x + b.x, v.y + b.y));
}

// Thread mapping shared by both kernels. With P = channels / 2 channel pairs per row:
//   P <= 320 threads: the block works on R = 320 / P rows at once, thread t on pair t % P of row slot t / P
//   P >  320        : one row at a time, thread t on pairs t, t + 320, ... (at most four)
// and every thread keeps about eight loads in flight (rows x pairs), so that enough loads are outstanding to cover the
// memory latency with four-byte accesses (a warp still reads 128 contiguous bytes per instruction).

struct NormMapping {
    uint32_t pairs, rows_at_once, slot, first_pair;
    bool active;
};

__device__ __forceinline__ NormMapping norm_mapping(uint32_t channels) {
    NormMapping m;
    m.pairs = channels / 2;
    if (m.pairs <= kNormThreads) {
        m.rows_at_once = kNormThreads / m.pairs;
        m.slot = threadIdx.x / m.pairs;
        m.first_pair = threadIdx.x - m.slot * m.pairs;
        m.active = m.slot < m.rows_at_once;
    } else {
        m.rows_at_once = 1;
        m.slot = 0;
        m.first_pair = threadIdx.x;
        m.active = true;
    }
    return m;
}

template <uint32_t kPairsPerThread>
__global__ void __launch_bounds__(kNormThreads)
group_norm_stats_kernel(const GroupNormLaunch p) {
    constexpr uint32_t kUnroll = kPairsPerThread == 1 ? 8 : (kPairsPerThread == 2 ? 4 : 2);
    __shared__ float pair_sums[kNormThreads * kPairsPerThread][2];     // [row slot][pair]
    const uint32_t batch = blockIdx.y;
    const uint32_t chunk = blockIdx.x;
    const NormMapping m = norm_mapping(p.channels);
    const uint32_t first_row = chunk * p.rows_per_chunk;
    const uint32_t last_row = min(p.rows, first_row + p.rows_per_chunk);
    const __half* base = p.x + static_cast<size_t>(batch) * p.rows * p.channels;
    const __half* bias_row = p.channel_bias != nullptr ? p.channel_bias + static_cast<size_t>(batch) * p.channels : nullptr;

    float sum[kPairsPerThread] = {}, squares[kPairsPerThread] = {};
    if (m.active) {
        const uint32_t step = m.rows_at_once * kUnroll;
        for (uint32_t row0 = first_row + m.slot; row0 < last_row; row0 += step) {
#pragma unroll
            for (uint32_t u = 0; u < kUnroll; ++u) {
                const uint32_t row = row0 + u * m.rows_at_once;
                if (row >= last_row) break;
                const __half* source = base + static_cast<size_t>(row) * p.channels;
#pragma unroll
                for (uint32_t i = 0; i < kPairsPerThread; ++i) {
                    const uint32_t pair = m.first_pair + i * kNormThreads;
                    if (pair < m.pairs) {
                        const float2 v = load_pair(source, pair, bias_row);
                        sum[i] += v.x + v.y;
                        squares[i] = fmaf(v.x, v.x, fmaf(v.y, v.y, squares[i]));
                    }
                }
            }
        }
#pragma unroll
        for (uint32_t i = 0; i < kPairsPerThread; ++i) {
            const uint32_t pair = m.first_pair + i * kNormThreads;
            if (pair < m.pairs) {
                pair_sums[m.slot * m.pairs + pair][0] = sum[i];
                pair_sums[m.slot * m.pairs + pair][1] = squares[i];
            }
        }
    }
    __syncthreads();
    // one thread per group adds its pairs: row slots in order, channels in order
    if (threadIdx.x < p.groups) {
        const uint32_t pairs_per_group = m.pairs / p.groups;
        float total = 0.0f, total_squares = 0.0f;
        for (uint32_t slot = 0; slot < m.rows_at_once; ++slot) {
            for (uint32_t j = 0; j < pairs_per_group; ++j) {
                const uint32_t index = slot * m.pairs + threadIdx.x * pairs_per_group + j;
                total += pair_sums[index][0];
                total_squares += pair_sums[index][1];
            }
        }
        float* out = p.partials + ((static_cast<size_t>(batch) * gridDim.x + chunk) * p.groups + threadIdx.x) * 2;
        out[0] = total;
        out[1] = total_squares;
    }
}

template <uint32_t kPairsPerThread>
__global__ void __launch_bounds__(kNormThreads)
group_norm_apply_kernel(const GroupNormLaunch p) {
    constexpr uint32_t kUnroll = kPairsPerThread == 1 ? 8 : (kPairsPerThread == 2 ? 4 : 2);
    __shared__ float group_mean[64], group_inverse[64];
    const uint32_t batch = blockIdx.y;
    const uint32_t chunk = blockIdx.x;
    const NormMapping m = norm_mapping(p.channels);
    const uint32_t pairs_per_group = m.pairs / p.groups;
    // Partial sums of this batch element, added in a fixed order by eight threads per group (thread l of a
    // group takes chunks l, l + 8, ...), then the eight results in order: deterministic, and the chain of
    // dependent additions is an eighth as long as with one thread per group.
    __shared__ double lane_sums[64][8][2];
    if (threadIdx.x < p.groups * 8u) {
        const uint32_t group = threadIdx.x >> 3, part = threadIdx.x & 7u;
        double total = 0.0, total_squares = 0.0;
        const float* partial = p.partials + (static_cast<size_t>(batch) * gridDim.x * p.groups + group) * 2;
        for (uint32_t c = part; c < gridDim.x; c += 8) {
            total += static_cast<double>(partial[static_cast<size_t>(c) * p.groups * 2]);
            total_squares += static_cast<double>(partial[static_cast<size_t>(c) * p.groups * 2 + 1]);
        }
        lane_sums[group][part][0] = total;
        lane_sums[group][part][1] = total_squares;
    }
    __syncthreads();
    if (threadIdx.x < p.groups) {
        double total = 0.0, total_squares = 0.0;
        for (uint32_t part = 0; part < 8; ++part) {
            total += lane_sums[threadIdx.x][part][0];
            total_squares += lane_sums[threadIdx.x][part][1];
        }
        const double count = static_cast<double>(p.rows) * (2.0 * pairs_per_group);
        const double mean = total / count;
        const double variance = fmax(0.0, total_squares / count - mean * mean);
        group_mean[threadIdx.x] = static_cast<float>(mean);
        group_inverse[threadIdx.x] = rsqrtf(static_cast<float>(variance) + p.epsilon);
    }
    __syncthreads();
    if (!m.active) return;

    float2 mean[kPairsPerThread], inverse[kPairsPerThread], gamma[kPairsPerThread], beta[kPairsPerThread];
#pragma unroll
    for (uint32_t i = 0; i < kPairsPerThread; ++i) {
        const uint32_t pair = m.first_pair + i * kNormThreads;
        if (pair < m.pairs) {
            const uint32_t group = pair / pairs_per_group;
            mean[i] = make_float2(group_mean[group], group_mean[group]);
            inverse[i] = make_float2(group_inverse[group], group_inverse[group]);
            gamma[i] = __half22float2(*reinterpret_cast<const __half2*>(p.gamma + 2 * pair));
            beta[i] = __half22float2(*reinterpret_cast<const __half2*>(p.beta + 2 * pair));
        }
    }
    const uint32_t first_row = chunk * p.rows_per_chunk;
    const uint32_t last_row = min(p.rows, first_row + p.rows_per_chunk);
    const __half* base = p.x + static_cast<size_t>(batch) * p.rows * p.channels;
    __half* out_base = p.y + static_cast<size_t>(batch) * p.rows * p.channels;
    const __half* bias_row = p.channel_bias != nullptr ? p.channel_bias + static_cast<size_t>(batch) * p.channels : nullptr;
    const uint32_t step = m.rows_at_once * kUnroll;
    for (uint32_t row0 = first_row + m.slot; row0 < last_row; row0 += step) {
        float2 v[kUnroll][kPairsPerThread];
#pragma unroll
        for (uint32_t u = 0; u < kUnroll; ++u) {
            const uint32_t row = row0 + u * m.rows_at_once;
            const __half* source = base + static_cast<size_t>(row) * p.channels;
#pragma unroll
            for (uint32_t i = 0; i < kPairsPerThread; ++i) {
                const uint32_t pair = m.first_pair + i * kNormThreads;
                if (row < last_row && pair < m.pairs) v[u][i] = load_pair(source, pair, bias_row);
            }
        }
#pragma unroll
        for (uint32_t u = 0; u < kUnroll; ++u) {
            const uint32_t row = row0 + u * m.rows_at_once;
            if (row >= last_row) break;
            __half* destination = out_base + static_cast<size_t>(row) * p.channels;
#pragma unroll
            for (uint32_t i = 0; i < kPairsPerThread; ++i) {
                const uint32_t pair = m.first_pair + i * kNormThreads;
                if (pair < m.pairs) {
                    float lo = fmaf((v[u][i].x - mean[i].x) * inverse[i].x, gamma[i].x, beta[i].x);
                    float hi = fmaf((v[u][i].y - mean[i].y) * inverse[i].y, gamma[i].y, beta[i].y);
                    if (p.silu != 0) {
                        lo = __fdividef(lo, 1.0f + __expf(-lo));
                        hi = __fdividef(hi, 1.0f + __expf(-hi));
                    }
                    *reinterpret_cast<__half2*>(destination + 2 * pair) = __floats2half2_rn(lo, hi);
                }
            }
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

uint32_t group_norm_max_channels() { return 2 * kNormThreads * kMaxPairsPerThread; }

cudaError_t launch_group_norm_nhwc(const GroupNormLaunch& launch, uint32_t chunks, cudaStream_t stream) {
    const dim3 grid(chunks, launch.batch, 1);
    const uint32_t pairs_per_thread = (launch.channels / 2 + kNormThreads - 1) / kNormThreads;
    switch (pairs_per_thread) {
    case 1: group_norm_stats_kernel<1><<<grid, kNormThreads, 0, stream>>>(launch); break;
    case 2: group_norm_stats_kernel<2><<<grid, kNormThreads, 0, stream>>>(launch); break;
    case 3: group_norm_stats_kernel<3><<<grid, kNormThreads, 0, stream>>>(launch); break;
    default: group_norm_stats_kernel<4><<<grid, kNormThreads, 0, stream>>>(launch); break;
    }
    const cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return status;
    switch (pairs_per_thread) {
    case 1: group_norm_apply_kernel<1><<<grid, kNormThreads, 0, stream>>>(launch); break;
    case 2: group_norm_apply_kernel<2><<<grid, kNormThreads, 0, stream>>>(launch); break;
    case 3: group_norm_apply_kernel<3><<<grid, kNormThreads, 0, stream>>>(launch); break;
    default: group_norm_apply_kernel<4><<<grid, kNormThreads, 0, stream>>>(launch); break;
    }
    return cudaGetLastError();
}

}  // namespace sdxlq
