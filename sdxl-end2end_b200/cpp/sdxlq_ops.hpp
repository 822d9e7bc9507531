// C++20 host shim over the C ABI (include/sdxlq.h): the projection operators of the reference's
// `sdxl::cuda::Ops` (include/sdxl/cuda/ops.hpp:17-30 of the reference) with the same names,
// argument meaning and error behaviour, so that `Ops::linear` / `Ops::linear_activation`
// (src/cuda/ops_blas.cpp:244-397) can forward here.
//
// Header-only. `TensorRef` carries exactly the fields the reference's `cuda::Tensor` exposes to
// the operator (include/sdxl/cuda/tensor.hpp:99-157): data pointer, shape, ScalarType, TensorRole
// and the quantisation metadata (dequant scale pointer / count / mode, FP8 storage layout,
// ConvRot group size). It does not own memory: outputs come from the allocator the integrator
// passes in (the reference's `Tensor::allocate` on the runtime arena).
#pragma once

#include "sdxlq.h"

#include <cstddef>
#include <cstdint>
#include <functional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace sdxlq {

// sdxl::cuda::CudaError (include/sdxl/cuda/runtime.hpp:18-21).
class CudaError : public std::runtime_error {
public:
    explicit CudaError(const std::string& message, int status = SDXLQ_ERR_INVALID_ARGUMENT)
        : std::runtime_error(message), status_(status) {}
    [[nodiscard]] int status() const noexcept { return status_; }

private:
    int status_;
};

enum class ScalarType : std::uint8_t { Float8E4M3, Float8E5M2, Int8, Float16, Float32, Int32 };
enum class TensorRole : std::uint8_t { Model, SamplerState, VAE, FP8ScaleMetadata, QuantizationMetadata, HostInterop };
enum class FP8ScaleMode : std::uint8_t { None, TensorWide, PerOutputChannel };
enum class FP8StorageLayout : std::uint8_t { RowMajorNK, KMajorKN };
enum class LinearActivation : std::uint8_t { None, SiLU, GELU, QuickGELU, GEGLU };

[[nodiscard]] inline bool is_fp8(ScalarType type) noexcept {
    return type == ScalarType::Float8E4M3 || type == ScalarType::Float8E5M2;
}

[[nodiscard]] inline std::size_t scalar_size(ScalarType type) noexcept {
    switch (type) {
    case ScalarType::Float8E4M3:
    case ScalarType::Float8E5M2:
    case ScalarType::Int8: return 1;
    case ScalarType::Float16: return 2;
    default: return 4;
    }
}

// valid_convrot_group_size (src/cuda/int8_convrot.cu:489-496).
[[nodiscard]] inline bool valid_convrot_group_size(std::size_t group_size) noexcept {
    return sdxlq_valid_convrot_group_size(group_size) != 0;
}

struct TensorRef {
    void* data = nullptr;
    std::vector<std::size_t> shape;
    ScalarType type = ScalarType::Float16;
    TensorRole role = TensorRole::Model;
    const float* dequant_scale_data = nullptr;
    std::size_t dequant_scale_count = 0;
    FP8ScaleMode dequant_scale_mode = FP8ScaleMode::None;
    FP8StorageLayout fp8_storage_layout = FP8StorageLayout::RowMajorNK;
    std::size_t convrot_group_size = 0;

    [[nodiscard]] bool defined() const noexcept { return data != nullptr; }
    [[nodiscard]] std::size_t rank() const noexcept { return shape.size(); }
    [[nodiscard]] std::size_t size(std::size_t dimension) const { return shape.at(dimension); }
    [[nodiscard]] std::size_t elements() const noexcept {
        std::size_t total = 1;
        for (const std::size_t extent : shape) total *= extent;
        return total;
    }
    [[nodiscard]] bool has_dequant_scale() const noexcept { return dequant_scale_data != nullptr; }
};

// sdxl::cuda::INT8ExecutionStats (include/sdxl/cuda/runtime.hpp:106-112).
struct INT8ExecutionStats {
    std::size_t linear_calls = 0;
    std::size_t cublaslt_imma_calls = 0;       // tensor-core (tcgen05) calls here
    std::size_t dp4a_fallback_calls = 0;
    std::size_t tensor_core_plan_misses = 0;
    std::size_t tensor_core_execution_failures = 0;
};

// The slice of sdxl::cuda::Runtime the operator needs: device, stream, scratch, counters.
class Runtime final {
public:
    Runtime(int device, void* stream, std::size_t workspace_bytes = 0) {
        const int status = sdxlq_context_create(device, stream, workspace_bytes, &context_);
        if (status != SDXLQ_OK) throw CudaError(std::string("sdxlq_context_create: ") + sdxlq_status_string(status), status);
    }
    ~Runtime() { sdxlq_context_destroy(context_); }
    Runtime(const Runtime&) = delete;
    Runtime& operator=(const Runtime&) = delete;

    [[nodiscard]] sdxlq_context* context() const noexcept { return context_; }
    void synchronize() const { check(sdxlq_context_check(context_)); }
    [[nodiscard]] INT8ExecutionStats int8_execution_stats() const {
        sdxlq_int8_stats raw{};
        check(sdxlq_get_stats(context_, &raw));
        return INT8ExecutionStats{raw.linear_calls, raw.tensor_core_calls, raw.dp4a_fallback_calls,
                                  raw.tensor_core_plan_misses, raw.tensor_core_execution_failures};
    }
    void check(int status) const {
        if (status != SDXLQ_OK) throw CudaError(sdxlq_last_error(context_), status);
    }

private:
    sdxlq_context* context_ = nullptr;
};

class Ops final {
public:
    // `allocate(bytes)` returns stream-ordered device memory for an output tensor.
    using Allocator = std::function<void*(std::size_t)>;

    Ops(const Runtime& runtime, Allocator allocate) : runtime_(&runtime), allocate_(std::move(allocate)) {}

    // Ops::linear (src/cuda/ops_blas.cpp:244-386).
    [[nodiscard]] TensorRef linear(const TensorRef& input, const TensorRef& weight,
                                   const TensorRef* bias = nullptr) const {
        return run(input, weight, bias, LinearActivation::None);
    }

    // Ops::linear_activation (src/cuda/ops_blas.cpp:388-397).
    [[nodiscard]] TensorRef linear_activation(const TensorRef& input, const TensorRef& weight,
                                              const TensorRef& bias, LinearActivation activation) const {
        return run(input, weight, &bias, activation);
    }

    // Ops::linear followed by Ops::add_in_place(hidden, result) as the reference's transformer block
    // issues them (src/cuda/unet.cpp:114-118, 128-132, 143-147, 174-179), in one call: the FP16 add
    // runs in the projection's epilogue and `hidden` is updated in place.
    void linear_add_in_place(TensorRef& hidden, const TensorRef& input, const TensorRef& weight,
                             const TensorRef* bias = nullptr) const {
        TensorRef output = hidden;
        sdxlq_linear_desc desc = describe(input, weight, bias, LinearActivation::None, output, /*allocate_output=*/false);
        if (output.shape != hidden.shape || hidden.type != ScalarType::Float16) throw CudaError("CUDA add requires matching FP16 tensors");
        desc.y = hidden.data;
        desc.residual = hidden.data;
        runtime_->check(sdxlq_linear(runtime_->context(), &desc));
    }

    // Up to four projections of the same input in one launch per kernel kind and one quantisation of
    // the input: to_q / to_k / to_v of a transformer block (src/cuda/unet.cpp:110-112). Nothing is
    // allocated besides the outputs; the call can be recorded by a stream capture.
    [[nodiscard]] std::vector<TensorRef> linear_group(const TensorRef& input, const std::vector<const TensorRef*>& weights) const {
        std::vector<TensorRef> outputs(weights.size());
        std::vector<sdxlq_linear_desc> descs;
        descs.reserve(weights.size());
        for (std::size_t i = 0; i < weights.size(); ++i) {
            descs.push_back(describe(input, *weights[i], nullptr, LinearActivation::None, outputs[i]));
        }
        runtime_->check(sdxlq_linear_grouped(runtime_->context(), descs.data(), descs.size()));
        return outputs;
    }

    // Ops::layer_norm (include/sdxl/cuda/ops.hpp:39-42, src/cuda/ops_kernels.cu:1425-1470): FP16 in, FP16 out.
    [[nodiscard]] TensorRef layer_norm(const TensorRef& input, const TensorRef& weight, const TensorRef& bias,
                                       float epsilon = 1.0e-5F) const {
        sdxlq_layer_norm_desc desc = describe_norm(input, weight, bias, epsilon);
        TensorRef output = input;
        output.data = allocate_(input.elements() * sizeof(std::uint16_t));
        desc.out_dtype = SDXLQ_FP16;
        desc.y = output.data;
        runtime_->check(sdxlq_layer_norm(runtime_->context(), &desc));
        return output;
    }

    // Ops::layer_norm fused with the activation quantiser of the projection(s) that read the result
    // (to_q / to_k / to_v, attn2.to_q, ff.net.0.proj; src/cuda/unet.cpp:108-112, 121-124, 135-138): the
    // normalised FP16 tensor is never written. The result carries the quantised rows and their scale(s)
    // in the form `consumer` wants; pass it to linear_quantized.
    struct QuantizedActivations {
        void* data = nullptr;            // INT8 or FP8 [rows, width]
        float* scales = nullptr;         // [rows] (INT8) or [1] (FP8)
        std::vector<std::size_t> shape;
    };
    [[nodiscard]] QuantizedActivations layer_norm_quantized(const TensorRef& input, const TensorRef& weight,
                                                            const TensorRef& bias, const TensorRef& consumer,
                                                            float epsilon = 1.0e-5F) const {
        sdxlq_layer_norm_desc desc = describe_norm(input, weight, bias, epsilon);
        if (consumer.rank() != 2 || consumer.size(1) != desc.width) throw CudaError("CUDA linear feature mismatch");
        if (consumer.type != ScalarType::Int8 && !is_fp8(consumer.type)) {
            throw CudaError("layer_norm_quantized wants an INT8 or FP8 projection weight");
        }
        QuantizedActivations result;
        result.shape = input.shape;
        result.data = allocate_(input.elements());
        result.scales = static_cast<float*>(allocate_((consumer.type == ScalarType::Int8 ? desc.rows : 1) * sizeof(float)));
        desc.out_dtype = static_cast<std::int32_t>(consumer.type);
        desc.convrot_group_size = static_cast<std::uint32_t>(consumer.convrot_group_size);
        desc.xq = result.data;
        desc.xq_scales = result.scales;
        runtime_->check(sdxlq_layer_norm(runtime_->context(), &desc));
        return result;
    }

    // Ops::linear / linear_activation on rows that layer_norm_quantized (or quantize_*) produced.
    [[nodiscard]] TensorRef linear_quantized(const QuantizedActivations& input, const TensorRef& weight,
                                             const TensorRef* bias = nullptr,
                                             LinearActivation activation = LinearActivation::None) const {
        TensorRef shape_only;
        shape_only.shape = input.shape;
        shape_only.data = input.data;                   // only the shape is read: xq replaces x below
        TensorRef output;
        sdxlq_linear_desc desc = describe(shape_only, weight, bias, activation, output);
        desc.x = nullptr;
        desc.xq = input.data;
        desc.xq_scales = input.scales;
        runtime_->check(sdxlq_linear(runtime_->context(), &desc));
        return output;
    }

    // Ops::quantize_fp8 / quantize_e4m3 / quantize_e5m2 (src/cuda/ops_blas.cpp:231-242).
    [[nodiscard]] TensorRef quantize_fp8(const TensorRef& input, ScalarType fp8_type) const {
        if (input.type != ScalarType::Float16 || !is_fp8(fp8_type)) {
            throw CudaError("FP8 activation quantization requires float16 input and an FP8 destination");
        }
        TensorRef destination;
        destination.shape = input.shape;
        destination.type = fp8_type;
        destination.role = TensorRole::Model;
        destination.data = allocate_(input.elements());
        float* scale = static_cast<float*>(allocate_(sizeof(float)));
        runtime_->check(sdxlq_quantize_act_fp8(runtime_->context(), input.data, input.elements(),
                                               static_cast<std::int32_t>(fp8_type),
                                               static_cast<std::uint8_t*>(destination.data), scale));
        destination.dequant_scale_data = scale;
        destination.dequant_scale_count = 1;
        destination.dequant_scale_mode = FP8ScaleMode::TensorWide;
        return destination;
    }
    [[nodiscard]] TensorRef quantize_e4m3(const TensorRef& input) const { return quantize_fp8(input, ScalarType::Float8E4M3); }
    [[nodiscard]] TensorRef quantize_e5m2(const TensorRef& input) const { return quantize_fp8(input, ScalarType::Float8E5M2); }

    // A fixed set of projections run as one grouped launch per call (sdxlq_group_plan_*): built
    // once, run many times. Projections that read the same input with the same quantisation share
    // one quantised copy of it. Two uses at the reference's call sites (src/cuda/unet.cpp:98-149):
    //   * to_q / to_k / to_v of a transformer block on the same `normalized` tensor;
    //   * every cross-attention to_k / to_v of the UNet (140 projections) on the text encoder's
    //     hidden states, which do not change between denoising steps: run the set once per
    //     generation and keep its outputs for all steps, which takes the skinny K=2048 GEMMs out of
    //     the step loop.
    class ProjectionSet final {
    public:
        struct Entry {
            TensorRef input, weight;
            const TensorRef* bias = nullptr;
            LinearActivation activation = LinearActivation::None;
        };

        ProjectionSet(const Ops& ops, const std::vector<Entry>& entries) : runtime_(ops.runtime_) {
            std::vector<sdxlq_linear_desc> descs;
            descs.reserve(entries.size());
            for (const Entry& entry : entries) {
                TensorRef output;
                descs.push_back(ops.describe(entry.input, entry.weight, entry.bias, entry.activation, output));
                outputs_.push_back(output);
            }
            runtime_->check(sdxlq_group_plan_create(runtime_->context(), descs.data(), descs.size(), &plan_));
        }
        ProjectionSet(const ProjectionSet&) = delete;
        ProjectionSet& operator=(const ProjectionSet&) = delete;
        ~ProjectionSet() { sdxlq_group_plan_destroy(plan_); }

        // Enqueues the whole set on the runtime's stream; outputs()[i] belongs to entries[i].
        void run() const { runtime_->check(sdxlq_group_plan_run(runtime_->context(), plan_)); }
        [[nodiscard]] const std::vector<TensorRef>& outputs() const { return outputs_; }
        [[nodiscard]] int launches() const { return sdxlq_group_plan_launches(plan_); }

    private:
        const Runtime* runtime_ = nullptr;
        sdxlq_group_plan* plan_ = nullptr;
        std::vector<TensorRef> outputs_;
    };

private:
    [[nodiscard]] TensorRef run(const TensorRef& input, const TensorRef& weight, const TensorRef* bias,
                                LinearActivation activation) const {
        TensorRef output;
        const sdxlq_linear_desc desc = describe(input, weight, bias, activation, output);
        runtime_->check(sdxlq_linear(runtime_->context(), &desc));
        return output;
    }

    // Validates like Ops::linear, allocates the output and fills the C descriptor.
    // The checks of Ops::layer_norm (src/cuda/ops_kernels.cu:1425-1440), with its messages.
    [[nodiscard]] static sdxlq_layer_norm_desc describe_norm(const TensorRef& input, const TensorRef& weight,
                                                             const TensorRef& bias, float epsilon) {
        if (input.type != ScalarType::Float16 || weight.type != ScalarType::Float16 || bias.type != ScalarType::Float16 ||
            input.rank() < 1 || weight.rank() != 1 || bias.rank() != 1) {
            throw CudaError("CUDA layer_norm expects an FP16 input with rank-1 FP16 weight and bias");
        }
        const std::size_t width = input.shape.back();
        if (width == 0) throw CudaError("layer_norm requires a non-empty last dimension");
        if (weight.size(0) != width || bias.size(0) != width) throw CudaError("CUDA layer_norm width mismatch");
        sdxlq_layer_norm_desc desc{};
        desc.x = input.data;
        desc.rows = input.elements() / width;
        desc.width = width;
        desc.gamma = weight.data;
        desc.beta = bias.data;
        desc.epsilon = epsilon;
        return desc;
    }

    [[nodiscard]] sdxlq_linear_desc describe(const TensorRef& input, const TensorRef& weight, const TensorRef* bias,
                                             LinearActivation activation, TensorRef& output,
                                             bool allocate_output = true) const {
        // The type / role / rank checks of Ops::linear, with its messages.
        if (weight.type == ScalarType::Int8) {
            if (input.type != ScalarType::Float16 || input.role != TensorRole::Model || input.rank() < 2 ||
                weight.rank() != 2) {
                throw CudaError("INT8 linear requires FP16/FP32 model activations and a rank-2 INT8 weight");
            }
        } else if (is_fp8(weight.type)) {
            if (input.type != ScalarType::Float16 || input.role != TensorRole::Model || input.rank() < 2 ||
                weight.rank() != 2) {
                throw CudaError("FP8 UNet linear requires FP16 model activations and a rank-2 FP8 weight");
            }
        } else if (input.type != ScalarType::Float16 || weight.type != input.type || weight.role != input.role) {
            throw CudaError("CUDA linear expects matching FP16/FP32 tensors and roles, or FP8 weights");
        }
        if (input.rank() < 2 || weight.rank() != 2) throw CudaError("CUDA linear rank mismatch");
        const std::size_t k = input.shape.back();
        const std::size_t n = weight.size(0);
        if (weight.size(1) != k) throw CudaError("CUDA linear feature mismatch");
        if (bias != nullptr && (bias->type != ScalarType::Float16 || bias->role != input.role ||
                                bias->rank() != 1 || bias->size(0) != n)) {
            throw CudaError("CUDA linear bias mismatch");
        }
        const std::size_t m = input.elements() / k;

        output = TensorRef{};
        output.shape = input.shape;
        output.shape.back() = activation == LinearActivation::GEGLU ? n / 2 : n;
        output.type = ScalarType::Float16;
        output.role = input.role;
        output.data = allocate_output ? allocate_(output.elements() * sizeof(std::uint16_t)) : nullptr;

        sdxlq_linear_desc desc{};
        desc.x = input.data;
        desc.m = m;
        desc.weight.data = weight.data;
        desc.weight.dtype = static_cast<std::int32_t>(weight.type);
        desc.weight.layout = static_cast<std::int32_t>(weight.fp8_storage_layout);
        desc.weight.n = n;
        desc.weight.k = k;
        desc.weight.scales = weight.dequant_scale_data;
        desc.weight.scale_count = weight.dequant_scale_count;
        desc.weight.scale_mode = static_cast<std::int32_t>(weight.dequant_scale_mode);
        desc.weight.convrot_group_size = static_cast<std::uint32_t>(weight.convrot_group_size);
        desc.bias = bias != nullptr ? bias->data : nullptr;
        desc.activation = static_cast<std::int32_t>(activation);
        desc.y = output.data;
        return desc;
    }

    const Runtime* runtime_ = nullptr;
    Allocator allocate_;
};

}  // namespace sdxlq
