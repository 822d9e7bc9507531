// TEST INFRASTRUCTURE ONLY — never linked into the shipped library.
//
// Runs the reference's own CUDA code for this path on the GPU, compiled unmodified from the
// reference sources for sm_100 (recipe in oracle/Makefile, target `refcuda`):
//   quantize_tensor_fp8       src/cuda/fp8_kernels.cu:157-190 (fp16_amax / fp8_scale / fp16_to_fp8 kernels)
//   fp8_weight_only_linear    src/cuda/fp8_kernels.cu:51-149, 192-245 (WMMA kernel, FP16 accumulation)
// through the reference's Runtime / Tensor classes (src/cuda/runtime.cpp, tensor.cu). Used by the
// GPU tests to check this repository's FP8 activation quantiser, and the weight-only arithmetic of
// its oracle, against the reference's device code itself. The INT8 translation unit
// (src/cuda/int8_convrot.cu) is not part of this library: nvcc 12.9 aborts on it with an internal
// front-end error (see the Makefile).
#include "sdxl/cuda/runtime.hpp"
#include "sdxl/cuda/tensor.hpp"
#include "src/cuda/fp8_internal.hpp"

#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <memory>
#include <string>

namespace {

std::unique_ptr<sdxl::cuda::Runtime> g_runtime;

sdxl::cuda::Runtime& runtime() {
    if (!g_runtime) {
        sdxl::cuda::RuntimeOptions options;
        options.device = 0;
        g_runtime = std::make_unique<sdxl::cuda::Runtime>(options);
    }
    return *g_runtime;
}

void report(char* error, std::uint64_t capacity, const char* text) {
    if (error == nullptr || capacity == 0) return;
    std::strncpy(error, text, static_cast<std::size_t>(capacity - 1));
    error[capacity - 1] = '\0';
}

sdxl::cuda::Tensor upload_bytes(const void* host, std::vector<std::size_t> shape, sdxl::cuda::ScalarType type,
                                sdxl::cuda::TensorRole role, bool persistent) {
    sdxl::cuda::Runtime& rt = runtime();
    sdxl::cuda::Tensor tensor = persistent ? sdxl::cuda::Tensor::allocate_persistent(rt, std::move(shape), type, role)
                                           : sdxl::cuda::Tensor::allocate(rt, std::move(shape), type, role);
    SDXL_CUDA_CHECK(cudaMemcpyAsync(tensor.data(), host, tensor.bytes(), cudaMemcpyHostToDevice, rt.stream()));
    return tensor;
}

}  // namespace

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

void refcuda_shutdown() { g_runtime.reset(); }

}  // extern "C"
