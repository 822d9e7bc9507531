// TEST INFRASTRUCTURE ONLY — never linked into the shipped library.
//
// Runs the reference's own CUDA code for this path on the GPU, compiled unmodified from the
// reference sources for sm_100 (recipe in oracle/Makefile, target `refcuda`):
//   quantize_tensor_fp8       src/cuda/fp8_kernels.cu:157-190 (fp16_amax / fp8_scale / fp16_to_fp8 kernels)
//   fp8_weight_only_linear    src/cuda/fp8_kernels.cu:51-149, 192-245 (WMMA kernel, FP16 accumulation)
//   Ops::linear / linear_activation   src/cuda/ops_blas.cpp:244-397 (cuBLASLt FP16, native FP8 through
//                                     cuBLASLt with the quantiser above, bias / activation kernels of
//                                     src/cuda/ops_kernels.cu)
//   Ops::layer_norm           src/cuda/ops_kernels.cu:185-256, 1425-1470
// through the reference's Runtime / Tensor classes (src/cuda/runtime.cpp, tensor.cu). Used by the
// GPU tests to check this repository's kernels, and the arithmetic of its oracle, against the
// reference's device code itself, and by the benchmark as a same-shape comparator. The INT8
// translation unit (src/cuda/int8_convrot.cu) is not part of this library: nvcc 12.9 aborts on it
// with an internal front-end error (see the Makefile); an INT8 weight therefore reaches a stub that
// throws. The attention back ends (cuDNN front end, the SM80 kernel) are stubbed the same way: no
// entry point here calls attention.
#include "sdxl/cuda/ops.hpp"
#include "sdxl/cuda/runtime.hpp"
#include "sdxl/cuda/tensor.hpp"
#include "src/cuda/cudnn_sdpa.hpp"
#include "src/cuda/flash_attention_sm80.hpp"
#include "src/cuda/fp8_internal.hpp"
#include "src/cuda/int8_convrot.hpp"

#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

namespace {

// One runtime per accumulation policy of the FP16 projections (RuntimeOptions::non_vae_accumulation:
// Float16 is the reference's default, Float32 its opt-in).
std::unique_ptr<sdxl::cuda::Runtime> g_runtime[2];

sdxl::cuda::Runtime& runtime(int fp32_accumulation = 0) {
    const int slot = fp32_accumulation != 0 ? 1 : 0;
    if (!g_runtime[slot]) {
        sdxl::cuda::RuntimeOptions options;
        options.device = 0;
        options.non_vae_accumulation =
            slot == 1 ? sdxl::cuda::NonVAEAccumulation::Float32 : sdxl::cuda::NonVAEAccumulation::Float16;
        g_runtime[slot] = std::make_unique<sdxl::cuda::Runtime>(options);
    }
    return *g_runtime[slot];
}

void report(char* error, std::uint64_t capacity, const char* text) {
    if (error == nullptr || capacity == 0) return;
    std::strncpy(error, text, static_cast<std::size_t>(capacity - 1));
    error[capacity - 1] = '\0';
}

sdxl::cuda::Tensor upload_bytes(const void* host, std::vector<std::size_t> shape, sdxl::cuda::ScalarType type,
                                sdxl::cuda::TensorRole role, bool persistent, int fp32_accumulation = 0) {
    sdxl::cuda::Runtime& rt = runtime(fp32_accumulation);
    sdxl::cuda::Tensor tensor = persistent ? sdxl::cuda::Tensor::allocate_persistent(rt, std::move(shape), type, role)
                                           : sdxl::cuda::Tensor::allocate(rt, std::move(shape), type, role);
    SDXL_CUDA_CHECK(cudaMemcpyAsync(tensor.data(), host, tensor.bytes(), cudaMemcpyHostToDevice, rt.stream()));
    return tensor;
}

// The operands of one Ops::linear_activation call, resident on the device.
struct LinearOperands {
    sdxl::cuda::Tensor input;
    sdxl::cuda::Tensor weight;
    sdxl::cuda::Tensor scale;
    sdxl::cuda::Tensor bias;
    bool has_bias = false;
};

// weight_type: 0 E4M3, 1 E5M2, 2 FP16.
LinearOperands upload_linear(const std::uint16_t* x, std::uint64_t m, std::uint64_t k, const void* w, std::uint64_t n,
                             int weight_type, const float* scales, std::uint64_t scale_count, const std::uint16_t* bias,
                             int fp32_accumulation) {
    using namespace sdxl::cuda;
    LinearOperands operands;
    operands.input = upload_bytes(x, {static_cast<std::size_t>(m), static_cast<std::size_t>(k)}, ScalarType::Float16,
                                  TensorRole::Model, false, fp32_accumulation);
    const ScalarType type = weight_type == 0   ? ScalarType::Float8E4M3
                            : weight_type == 1 ? ScalarType::Float8E5M2
                                               : ScalarType::Float16;
    operands.weight = upload_bytes(w, {static_cast<std::size_t>(n), static_cast<std::size_t>(k)}, type, TensorRole::Model,
                                   true, fp32_accumulation);
    if (weight_type != 2) {
        operands.scale = upload_bytes(scales, {static_cast<std::size_t>(scale_count)}, ScalarType::Float32,
                                      TensorRole::FP8ScaleMetadata, true, fp32_accumulation);
        operands.weight.attach_dequant_scale(operands.scale, scale_count == 1 ? FP8ScaleMode::TensorWide
                                                                             : FP8ScaleMode::PerOutputChannel);
    }
    if (bias != nullptr) {
        operands.bias = upload_bytes(bias, {static_cast<std::size_t>(n)}, ScalarType::Float16, TensorRole::Model, true,
                                     fp32_accumulation);
        operands.has_bias = true;
    }
    return operands;
}

sdxl::cuda::Tensor run_linear(const sdxl::cuda::Ops& ops, const LinearOperands& operands, int activation) {
    const auto kind = static_cast<sdxl::cuda::LinearActivation>(activation);
    if (!operands.has_bias) return ops.linear(operands.input, operands.weight, nullptr);
    return ops.linear_activation(operands.input, operands.weight, operands.bias, kind);
}

}  // namespace

// Parts of the reference this library leaves out; nothing above reaches them.
namespace sdxl::cuda {
Tensor int8_convrot_linear(const Runtime&, const Tensor&, const Tensor&) {
    throw CudaError("the INT8 translation unit is not part of this checker library");
}
bool cudnn_frontend_sdpa_compiled() noexcept { return false; }
void launch_cudnn_frontend_sdpa(const Runtime&, const Tensor&, const Tensor&, const Tensor&, Tensor&, std::size_t, bool) {
    throw CudaError("attention is not part of this checker library");
}
void launch_flash_attention_sm80_hdim64(const Runtime&, const Tensor&, const Tensor&, const Tensor&, const Tensor*, Tensor&,
                                        std::size_t, bool) {
    throw CudaError("attention is not part of this checker library");
}
}  // namespace sdxl::cuda

extern "C" {

// quantize_tensor_fp8 on FP16 bits x[rows, columns]; fmt 0 = E4M3, 1 = E5M2. Writes rows * columns
// FP8 bytes and the tensor-wide dequantisation scale. 0 ok, 1 the reference threw.
int refcuda_quantize_fp8(const std::uint16_t* x, std::uint64_t rows, std::uint64_t columns, int fmt, std::uint8_t* q,
                         float* scale, char* error, std::uint64_t error_capacity) {
    try {
        sdxl::cuda::Runtime& rt = runtime();
        const sdxl::cuda::Tensor input = upload_bytes(x, {static_cast<std::size_t>(rows), static_cast<std::size_t>(columns)},
                                                      sdxl::cuda::ScalarType::Float16, sdxl::cuda::TensorRole::Model, false);
        const sdxl::cuda::Tensor result = sdxl::cuda::quantize_tensor_fp8(
            rt, input, fmt == 0 ? sdxl::cuda::ScalarType::Float8E4M3 : sdxl::cuda::ScalarType::Float8E5M2);
        SDXL_CUDA_CHECK(cudaMemcpyAsync(q, result.data(), result.bytes(), cudaMemcpyDeviceToHost, rt.stream()));
        SDXL_CUDA_CHECK(cudaMemcpyAsync(scale, result.dequant_scale_data(), sizeof(float), cudaMemcpyDeviceToHost, rt.stream()));
        rt.synchronize();
        return 0;
    } catch (const std::exception& failure) {
        report(error, error_capacity, failure.what());
        return 1;
    }
}

// fp8_weight_only_linear: y[m, n] = x_f16[m, k] * (half(float(w_fp8) * scale))^T with FP16 accumulation.
// w holds n * k FP8 bytes, row-major [n, k] or, with k_major != 0, [k, n]; scale_count is 1 or n.
int refcuda_fp8_weight_only_linear(const std::uint16_t* x, std::uint64_t m, std::uint64_t k, const std::uint8_t* w,
                                   std::uint64_t n, int fmt, const float* scales, std::uint64_t scale_count, int k_major,
                                   std::uint16_t* y, char* error, std::uint64_t error_capacity) {
    try {
        sdxl::cuda::Runtime& rt = runtime();
        const sdxl::cuda::Tensor input = upload_bytes(x, {static_cast<std::size_t>(m), static_cast<std::size_t>(k)},
                                                      sdxl::cuda::ScalarType::Float16, sdxl::cuda::TensorRole::Model, false);
        sdxl::cuda::Tensor weight = upload_bytes(w, {static_cast<std::size_t>(n), static_cast<std::size_t>(k)},
                                                 fmt == 0 ? sdxl::cuda::ScalarType::Float8E4M3 : sdxl::cuda::ScalarType::Float8E5M2,
                                                 sdxl::cuda::TensorRole::Model, true);
        const sdxl::cuda::Tensor scale = upload_bytes(scales, {static_cast<std::size_t>(scale_count)}, sdxl::cuda::ScalarType::Float32,
                                                      sdxl::cuda::TensorRole::FP8ScaleMetadata, true);
        weight.attach_dequant_scale(scale, scale_count == 1 ? sdxl::cuda::FP8ScaleMode::TensorWide
                                                            : sdxl::cuda::FP8ScaleMode::PerOutputChannel);
        if (k_major != 0) weight.set_fp8_storage_layout(sdxl::cuda::FP8StorageLayout::KMajorKN);
        const sdxl::cuda::Tensor result = sdxl::cuda::fp8_weight_only_linear(rt, input, weight);
        SDXL_CUDA_CHECK(cudaMemcpyAsync(y, result.data(), result.bytes(), cudaMemcpyDeviceToHost, rt.stream()));
        rt.synchronize();
        return 0;
    } catch (const std::exception& failure) {
        report(error, error_capacity, failure.what());
        return 1;
    }
}

// Ops::linear (bias == nullptr) or Ops::linear_activation on FP16 activations x[m, k]. weight_type 0 E4M3,
// 1 E5M2, 2 FP16; activation is the reference's LinearActivation value (0 None, 1 SiLU, 2 GELU,
// 3 QuickGELU, 4 GEGLU: the output then has n / 2 columns). fp32_accumulation selects the runtime's
// NonVAEAccumulation for FP16 weights. y receives m * y_columns FP16 values.
int refcuda_ops_linear(const std::uint16_t* x, std::uint64_t m, std::uint64_t k, const void* w, std::uint64_t n,
                       int weight_type, const float* scales, std::uint64_t scale_count, const std::uint16_t* bias,
                       int activation, int fp32_accumulation, std::uint16_t* y, std::uint64_t y_columns, char* error,
                       std::uint64_t error_capacity) {
    try {
        sdxl::cuda::Runtime& rt = runtime(fp32_accumulation);
        const sdxl::cuda::Ops ops(rt);
        const LinearOperands operands = upload_linear(x, m, k, w, n, weight_type, scales, scale_count, bias, fp32_accumulation);
        const sdxl::cuda::Tensor result = run_linear(ops, operands, activation);
        if (result.elements() != m * y_columns) throw sdxl::cuda::CudaError("unexpected output extent");
        SDXL_CUDA_CHECK(cudaMemcpyAsync(y, result.data(), result.bytes(), cudaMemcpyDeviceToHost, rt.stream()));
        rt.synchronize();
        return 0;
    } catch (const std::exception& failure) {
        report(error, error_capacity, failure.what());
        return 1;
    }
}

// Device time of the same call, operands resident: `warmup` untimed calls, then `iterations` calls between
// two CUDA events on the reference's stream. Writes milliseconds per call.
int refcuda_time_linear(std::uint64_t m, std::uint64_t k, std::uint64_t n, int weight_type, int activation, int has_bias,
                        int fp32_accumulation, int warmup, int iterations, float* milliseconds, char* error,
                        std::uint64_t error_capacity) {
    try {
        sdxl::cuda::Runtime& rt = runtime(fp32_accumulation);
        const sdxl::cuda::Ops ops(rt);
        // Deterministic small-integer operands: the timing does not depend on the values.
        std::vector<std::uint16_t> x(m * k);
        for (std::size_t i = 0; i < x.size(); ++i) x[i] = static_cast<std::uint16_t>(0x3000U + (i * 2654435761ULL >> 20 & 0x3FFU));
        const std::size_t weight_bytes = n * k * (weight_type == 2 ? 2U : 1U);
        std::vector<std::uint8_t> w(weight_bytes);
        for (std::size_t i = 0; i < w.size(); ++i) w[i] = static_cast<std::uint8_t>(0x20U + (i * 40503ULL >> 7 & 0x1FU));
        std::vector<std::uint16_t> bias(n, 0x2E66U);
        const float scale = 0.01F;
        const LinearOperands operands = upload_linear(x.data(), m, k, w.data(), n, weight_type, &scale, 1,
                                                      has_bias != 0 ? bias.data() : nullptr, fp32_accumulation);
        for (int i = 0; i < warmup; ++i) (void)run_linear(ops, operands, activation);
        cudaEvent_t start = nullptr;
        cudaEvent_t stop = nullptr;
        SDXL_CUDA_CHECK(cudaEventCreate(&start));
        SDXL_CUDA_CHECK(cudaEventCreate(&stop));
        SDXL_CUDA_CHECK(cudaEventRecord(start, rt.stream()));
        for (int i = 0; i < iterations; ++i) (void)run_linear(ops, operands, activation);
        SDXL_CUDA_CHECK(cudaEventRecord(stop, rt.stream()));
        SDXL_CUDA_CHECK(cudaEventSynchronize(stop));
        float elapsed = 0.0F;
        SDXL_CUDA_CHECK(cudaEventElapsedTime(&elapsed, start, stop));
        cudaEventDestroy(start);
        cudaEventDestroy(stop);
        *milliseconds = elapsed / static_cast<float>(iterations > 0 ? iterations : 1);
        return 0;
    } catch (const std::exception& failure) {
        report(error, error_capacity, failure.what());
        return 1;
    }
}

// Ops::layer_norm over the last dimension of FP16 x[rows, width].
int refcuda_layer_norm(const std::uint16_t* x, std::uint64_t rows, std::uint64_t width, const std::uint16_t* gamma,
                       const std::uint16_t* beta, float epsilon, std::uint16_t* y, char* error, std::uint64_t error_capacity) {
    try {
        using namespace sdxl::cuda;
        Runtime& rt = runtime();
        const Ops ops(rt);
        const Tensor input = upload_bytes(x, {static_cast<std::size_t>(rows), static_cast<std::size_t>(width)},
                                          ScalarType::Float16, TensorRole::Model, false);
        const Tensor weight = upload_bytes(gamma, {static_cast<std::size_t>(width)}, ScalarType::Float16, TensorRole::Model, true);
        const Tensor bias = upload_bytes(beta, {static_cast<std::size_t>(width)}, ScalarType::Float16, TensorRole::Model, true);
        const Tensor result = ops.layer_norm(input, weight, bias, epsilon);
        SDXL_CUDA_CHECK(cudaMemcpyAsync(y, result.data(), result.bytes(), cudaMemcpyDeviceToHost, rt.stream()));
        rt.synchronize();
        return 0;
    } catch (const std::exception& failure) {
        report(error, error_capacity, failure.what());
        return 1;
    }
}

void refcuda_shutdown() {
    g_runtime[0].reset();
    g_runtime[1].reset();
}

}  // extern "C"
