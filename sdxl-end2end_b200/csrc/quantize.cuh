// Job tables of the quantiser kernels (host <-> device).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace sdxlq {

// One [m, k] matrix to rotate + quantise row-wise to INT8.
struct QuantInt8Job {
    const void* x;               // FP16 or FP32 [m, k]
    int8_t* xq;                  // [m, k]
    float* scales;               // [m]
    uint32_t m, k;
    uint32_t stages;             // log4(group size): 0 = no rotation, 1..4 = groups of 4..256
    uint32_t threads_per_row;    // 4 * ceil(k / 256)
    uint32_t rows_per_block;     // block threads / threads_per_row
    uint32_t x_is_f32;
    uint32_t vector_ok;          // rows 16-byte aligned: 16-byte loads, 8-byte stores
    uint32_t first_block;        // first block of this job inside a grouped launch
    uint32_t num_blocks;
    uint32_t pad;                // 1: group of 256 with 16-byte aligned output rows (rotated256_rows_kernel)
    // LayerNorm over the row before the rotation (general kernel only): gamma == null means none.
    const __half* gamma;         // [k]
    const __half* beta;          // [k]
    float epsilon;
    uint32_t pad2;
};

struct QuantInt8Launch {
    const QuantInt8Job* jobs;    // device table (grouped) or null (`single` is used)
    const uint16_t* block_jobs;  // grouped: the job of every block of the launch, or null (the block searches `jobs`)
    uint32_t num_jobs;
    uint32_t pad;
    QuantInt8Job single;
};

// One tensor to quantise to FP8 with a tensor-wide dynamic scale.
struct QuantFp8Job {
    const void* x;               // FP16, `count` elements
    uint8_t* q;                  // `count` bytes
    float* scale_out;            // 1 float: the dequantisation scale
    uint64_t count;
    uint32_t fmt;                // 0 = E4M3, 1 = E5M2
    uint32_t vector_ok;
    uint32_t first_block;
    uint32_t num_blocks;
    uint32_t* amax_in;           // optional: the maximum of |x| as FP32 bits, filled by the producer of x; the
                                 // maximum kernel skips the job, the cast kernel reads this word and clears it
};

struct QuantFp8Launch {
    const QuantFp8Job* jobs;     // device table (grouped) or null
    const uint16_t* block_jobs;  // grouped: the job of every block of the launch, or null (the block searches `jobs`)
    uint32_t num_jobs;
    uint32_t pad;
    uint32_t* amax_bits;         // one scratch word per job, all zero on entry of the amax kernel
    uint32_t* done_counts;       // one word per job, zero on entry: cast blocks that have read the job's maximum;
                                 // the last one to read it puts both words back to zero for the next call
    QuantFp8Job single;
};

// Programmatic dependent launch, as every kernel of the projection path uses it: a kernel first waits for
// the kernels before it (griddepcontrol.wait: they have completed and their memory is visible), touching
// no global memory but constants before that, and then lets the kernel behind it be scheduled
// (griddepcontrol.launch_dependents), so that the next kernel's launch and set-up overlap this kernel's
// run. Waiting before triggering means that whatever a kernel finds complete, its dependents do too.
// Both instructions do nothing in a launch without the attribute.
__device__ __forceinline__ void wait_for_prior_kernels_then_release_next() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Launches `kernel`; `dependent` adds the programmatic-dependency attribute (the kernel may be scheduled
// while the kernel before it on the stream drains, see above).
template <typename... Params, typename... Args>
inline cudaError_t launch_behind(void (*kernel)(Params...), uint32_t blocks, uint32_t threads, size_t dynamic_smem,
                                 cudaStream_t stream, bool dependent, const Args&... args) {
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(blocks, 1, 1);
    config.blockDim = dim3(threads, 1, 1);
    config.dynamicSmemBytes = dynamic_smem;
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = dependent ? &attribute : nullptr;
    config.numAttrs = dependent ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, args...);
}

cudaError_t launch_rotate_quantize_int8(const QuantInt8Launch& launch, uint32_t blocks, uint32_t threads,
                                        cudaStream_t stream, bool early_launch);
cudaError_t launch_fp8_quantize(const QuantFp8Launch& launch, uint32_t blocks, cudaStream_t stream, bool early_launch,
                                bool skip_maximum_pass);
cudaError_t launch_fp8_weight_pack(const void* source, int32_t dtype, uint32_t n, uint32_t k, uint32_t fmt,
                                   uint32_t per_channel, uint32_t k_major, uint8_t* destination,
                                   float* scales, cudaStream_t stream);
cudaError_t launch_fill_f32(float* values, uint32_t count, float value, cudaStream_t stream);

// LayerNorm over the last dimension of FP16 x[rows, width] (width a multiple of 8, at most 2048, 16-byte
// aligned rows), one warp per row with the row in registers. Three outputs:
//   FP16            y[rows, width]
//   FP8             q[rows, width] in `fmt` with one tensor-wide dynamic scale: a statistics launch that only
//                   reduces max |y| into *amax_bits (and leaves the rows' statistics in row_stats), then a
//                   launch that normalises again and casts
//   INT8            q[rows, width] with per-row scales scale_out[rows], no rotation
struct LayerNormLaunch {
    const __half* x;
    const __half* gamma;
    const __half* beta;
    __half* y;
    uint8_t* q;
    float* scale_out;
    uint32_t* amax_bits;         // zero on entry; put back to zero by the cast launch
    uint32_t* done_count;        // zero on entry; put back to zero by the cast launch
    float2* row_stats;           // optional [rows] scratch: (mean, inverse deviation) from the statistics launch
                                 // to the cast launch; null: the cast launch reduces every row again
    uint32_t rows, width;
    uint32_t fmt;                // 0 = E4M3, 1 = E5M2
    float epsilon;
};
cudaError_t launch_layer_norm_f16(const LayerNormLaunch& launch, cudaStream_t stream, bool early_launch);
cudaError_t launch_layer_norm_int8(const LayerNormLaunch& launch, cudaStream_t stream, bool early_launch);
cudaError_t launch_layer_norm_fp8(const LayerNormLaunch& launch, cudaStream_t stream, bool early_launch);

// GroupNorm (+ SiLU) over channels-last FP16 activations [batch, rows, channels]: scaffolding of the UNet
// harness (see harness_norm.cu).
struct GroupNormLaunch {
    const __half* x;             // [batch, rows, channels]
    const __half* channel_bias;  // optional [batch, channels], added (and rounded to FP16) before the norm
    const __half* gamma;         // [channels]
    const __half* beta;          // [channels]
    __half* y;                   // [batch, rows, channels], may alias x
    float* partials;             // [batch, chunks, groups, 2] scratch
    float* finals;               // [batch, 64, 2] scratch: mean and inverse standard deviation per group
    uint32_t* counters;          // [batch] blocks of the statistics launch that are done; zero between launches
    uint32_t batch, rows, channels, groups;
    uint32_t rows_per_chunk;
    uint32_t silu;
    float epsilon;
};
uint32_t group_norm_max_channels();
cudaError_t launch_group_norm_nhwc(const GroupNormLaunch& launch, uint32_t chunks, cudaStream_t stream);
cudaError_t launch_bias_residual_add(const __half* x, const __half* bias, const __half* residual, __half* y, uint64_t rows,
                                     uint32_t channels, uint32_t sm_count, cudaStream_t stream);

}  // namespace sdxlq
