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

__global__ void __launch_bounds__(kNormThreads)
group_norm_stats_kernel(const GroupNormLaunch p) {
    __shared__ float pair_sums[kNormThreads * kMaxPairsPerThread][2];
    const uint32_t batch = blockIdx.y;
    const uint32_t chunk = blockIdx.x;
    const uint32_t pairs = p.channels / 2;
    const uint32_t first_row = chunk * p.rows_per_chunk;
    const uint32_t last_row = min(p.rows, first_row + p.rows_per_chunk);
    const __half* base = p.x + static_cast<size_t>(batch) * p.rows * p.channels;
    const __half* bias_row = p.channel_bias != nullptr ? p.channel_bias + static_cast<size_t>(batch) * p.channels : nullptr;

    float sum[kMaxPairsPerThread] = {}, squares[kMaxPairsPerThread] = {};
    for (uint32_t row = first_row; row < last_row; ++row) {
        const __half* source = base + static_cast<size_t>(row) * p.channels;
#pragma unroll
        for (uint32_t i = 0; i < kMaxPairsPerThread; ++i) {
            const uint32_t pair = threadIdx.x + i * kNormThreads;
            if (pair < pairs) {
                const float2 v = load_pair(source, pair, bias_row);
                sum[i] += v.x + v.y;
                squares[i] = fmaf(v.x, v.x, fmaf(v.y, v.y, squares[i]));
            }
        }
    }
#pragma unroll
    for (uint32_t i = 0; i < kMaxPairsPerThread; ++i) {
        const uint32_t pair = threadIdx.x + i * kNormThreads;
        if (pair < pairs) {
            pair_sums[pair][0] = sum[i];
            pair_sums[pair][1] = squares[i];
        }
    }
    __syncthreads();
    // one thread per group adds its pairs in channel order
    if (threadIdx.x < p.groups) {
        const uint32_t pairs_per_group = pairs / p.groups;
        float total = 0.0f, total_squares = 0.0f;
        for (uint32_t j = 0; j < pairs_per_group; ++j) {
            total += pair_sums[threadIdx.x * pairs_per_group + j][0];
            total_squares += pair_sums[threadIdx.x * pairs_per_group + j][1];
        }
        float* out = p.partials + ((static_cast<size_t>(batch) * gridDim.x + chunk) * p.groups + threadIdx.x) * 2;
        out[0] = total;
        out[1] = total_squares;
    }
}

__global__ void __launch_bounds__(kNormThreads)
group_norm_apply_kernel(const GroupNormLaunch p) {
    __shared__ float group_mean[64], group_inverse[64];
    const uint32_t batch = blockIdx.y;
    const uint32_t chunk = blockIdx.x;
    const uint32_t pairs = p.channels / 2;
    const uint32_t pairs_per_group = pairs / p.groups;
    if (threadIdx.x < p.groups) {
        double total = 0.0, total_squares = 0.0;
        const float* partial = p.partials + (static_cast<size_t>(batch) * gridDim.x * p.groups + threadIdx.x) * 2;
        for (uint32_t c = 0; c < gridDim.x; ++c) {
            total += static_cast<double>(partial[static_cast<size_t>(c) * p.groups * 2]);
            total_squares += static_cast<double>(partial[static_cast<size_t>(c) * p.groups * 2 + 1]);
        }
        const double count = static_cast<double>(p.rows) * (2.0 * pairs_per_group);
        const double mean = total / count;
        const double variance = fmax(0.0, total_squares / count - mean * mean);
        group_mean[threadIdx.x] = static_cast<float>(mean);
        group_inverse[threadIdx.x] = rsqrtf(static_cast<float>(variance) + p.epsilon);
    }
    __syncthreads();

    float2 mean[kMaxPairsPerThread], inverse[kMaxPairsPerThread], gamma[kMaxPairsPerThread], beta[kMaxPairsPerThread];
#pragma unroll
    for (uint32_t i = 0; i < kMaxPairsPerThread; ++i) {
        const uint32_t pair = threadIdx.x + i * kNormThreads;
        if (pair < pairs) {
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
    for (uint32_t row = first_row; row < last_row; ++row) {
        const __half* source = base + static_cast<size_t>(row) * p.channels;
        __half* destination = out_base + static_cast<size_t>(row) * p.channels;
#pragma unroll
        for (uint32_t i = 0; i < kMaxPairsPerThread; ++i) {
            const uint32_t pair = threadIdx.x + i * kNormThreads;
            if (pair < pairs) {
                const float2 v = load_pair(source, pair, bias_row);
                float lo = fmaf((v.x - mean[i].x) * inverse[i].x, gamma[i].x, beta[i].x);
                float hi = fmaf((v.y - mean[i].y) * inverse[i].y, gamma[i].y, beta[i].y);
                if (p.silu != 0) {
                    lo = __fdividef(lo, 1.0f + __expf(-lo));
                    hi = __fdividef(hi, 1.0f + __expf(-hi));
                }
                *reinterpret_cast<__half2*>(destination + 2 * pair) = __floats2half2_rn(lo, hi);
            }
        }
    }
}

}  // namespace

uint32_t group_norm_max_channels() { return 2 * kNormThreads * kMaxPairsPerThread; }

cudaError_t launch_group_norm_nhwc(const GroupNormLaunch& launch, uint32_t chunks, cudaStream_t stream) {
    const dim3 grid(chunks, launch.batch, 1);
    group_norm_stats_kernel<<<grid, kNormThreads, 0, stream>>>(launch);
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return status;
    group_norm_apply_kernel<<<grid, kNormThreads, 0, stream>>>(launch);
    return cudaGetLastError();
}

}  // namespace sdxlq
