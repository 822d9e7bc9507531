// C++20 host side of the load-time half of the path: the option structs, metadata, eligibility
// rules, weight packers and the precision-profile parser of the reference, over the C ABI.
//
//   sdxl::QuantizationMetadata                    include/sdxl/model.hpp:17-23
//   sdxl::cuda::FP8WeightLoadOptions / INT8WeightLoadOptions / FP8Backend
//                                                 include/sdxl/cuda/weights.hpp:20-66
//   upload_or_quantize_int8_weight                src/cuda/int8_convrot.cu:498-577 (int8_convrot.hpp:11-16)
//   WeightStore::upload_tensor, FP8 branch        src/cuda/weights.cu:301-415
//   is_linear_weight / the FP8 eligibility rule   src/cuda/weights.cu:185-193, 484-486
//   parse_precision_profile / PrecisionProfile    src/cuda/engine.cpp:58-115, include/sdxl/cuda/engine.hpp:20-29
//   int8_require_tensor_cores                     src/cuda/engine.cpp:191-194
//
// Same names, same rules, same CudaError messages. Sources are tensors already on the device (the
// reference stages the checkpoint bytes with cudaMallocAsync first; that staging stays with the
// integrator's loader). Outputs come from the integrator's persistent allocator.
#pragma once

#include "sdxlq_ops.hpp"

#include <algorithm>
#include <cctype>
#include <string>
#include <string_view>

namespace sdxlq {

enum class FP8Format : std::uint8_t { Auto, E4M3, E5M2 };
enum class FP8Backend : std::uint8_t { Auto, Native, WeightOnly };
enum class FP8BackendPreference : std::uint8_t { Auto, NativeOnly, WeightOnly };

struct FP8WeightLoadOptions {
    bool quantize_linear_weights = true;
    bool preserve_native_fp8 = true;
    FP8Format format = FP8Format::Auto;
    FP8ScaleMode scale_mode = FP8ScaleMode::TensorWide;
    FP8Backend backend = FP8Backend::Auto;
};

struct INT8WeightLoadOptions {
    bool quantize_floating_weights = true;
    bool require_prequantized = false;
    bool strict = false;
    bool require_tensor_cores = false;
    bool enable_convrot = true;
    std::size_t convrot_group_size = 256;
};

// Quantisation metadata of a prequantised checkpoint weight. `weight_scale` lives on the device
// here (FP32, [N] or [N, 1]); the reference reads it from the mapped file and uploads it.
struct QuantizationMetadata {
    const float* weight_scale = nullptr;
    std::size_t weight_scale_count = 0;
    const float* input_scale = nullptr;
    bool convrot = false;
    bool per_row = false;
    std::size_t convrot_group_size = 0;
};

struct PrecisionProfile {
    bool fp8 = true;
    bool int8 = false;
    bool int8_clip = true;
    FP8WeightLoadOptions weights;
    INT8WeightLoadOptions int8_weights;
    FP8BackendPreference runtime_backend = FP8BackendPreference::Auto;
    std::string canonical = "fp8-auto";

    // RuntimeOptions::int8_require_tensor_cores as SDXLEngine derives it (engine.cpp:191-194). Every
    // INT8 Linear here runs on the tensor cores, so the requirement always holds.
    [[nodiscard]] bool int8_require_tensor_cores() const noexcept {
        return int8 && (int8_weights.require_tensor_cores || int8_weights.strict);
    }
};

// parse_precision_profile (src/cuda/engine.cpp:58-115): profile string -> loader options.
[[nodiscard]] inline PrecisionProfile parse_precision_profile(std::string value) {
    std::transform(value.begin(), value.end(), value.begin(), [](unsigned char c) { return static_cast<char>(std::tolower(c)); });
    if (value == "fp8") value = "fp8-auto";
    if (value == "int8") value = "int8-convrot";
    PrecisionProfile profile;
    profile.canonical = value;
    const auto has = [&](std::string_view part) { return value.find(part) != std::string::npos; };
    if (value == "fp16") {
        profile.fp8 = false;
        return profile;
    }
    if (value.rfind("int8", 0) == 0) {
        profile.fp8 = false;
        profile.int8 = true;
        profile.int8_clip = !has("unet-only");
        profile.int8_weights.enable_convrot = !has("row");
        profile.int8_weights.strict = has("strict");
        profile.int8_weights.require_tensor_cores = profile.int8_weights.strict || has("tensorcore");
        profile.int8_weights.require_prequantized = has("prequantized") || has("prequant");
        profile.int8_weights.quantize_floating_weights = !profile.int8_weights.require_prequantized;
        static constexpr std::string_view known[] = {
            "int8-convrot", "int8-convrot-strict", "int8-convrot-prequantized", "int8-convrot-prequantized-strict",
            "int8-convrot-tensorcore", "int8-convrot-prequantized-tensorcore", "int8-row", "int8-row-strict",
            "int8-convrot-unet-only", "int8-convrot-unet-only-strict"};
        if (std::find(std::begin(known), std::end(known), value) == std::end(known)) {
            throw CudaError("unknown INT8 precision profile: " + value);
        }
        return profile;
    }
    profile.weights.format = FP8Format::Auto;
    profile.weights.scale_mode = FP8ScaleMode::TensorWide;
    profile.weights.backend = FP8Backend::Auto;
    if (has("e4m3")) profile.weights.format = FP8Format::E4M3;
    else if (has("e5m2")) profile.weights.format = FP8Format::E5M2;
    else if (value != "fp8-auto") throw CudaError("unknown precision profile: " + value);
    if (has("channel")) {
        profile.weights.scale_mode = FP8ScaleMode::PerOutputChannel;
        profile.weights.backend = FP8Backend::WeightOnly;
        profile.runtime_backend = FP8BackendPreference::WeightOnly;
    } else if (has("native")) {
        profile.weights.backend = FP8Backend::Native;
        profile.runtime_backend = FP8BackendPreference::NativeOnly;
    } else if (has("weight")) {
        profile.weights.backend = FP8Backend::WeightOnly;
        profile.runtime_backend = FP8BackendPreference::WeightOnly;
    }
    return profile;
}

// is_linear_weight (src/cuda/weights.cu:185-193): which parameters load_prefixes_int8 quantises.
[[nodiscard]] inline bool is_linear_weight(std::string_view logical_name, std::size_t rank) noexcept {
    if (!logical_name.ends_with(".weight") || rank != 2) return false;
    return logical_name.find("embeddings.") == std::string_view::npos &&
           logical_name.find("token_embedding") == std::string_view::npos &&
           logical_name.find("position_embedding") == std::string_view::npos;
}

// The eligibility test of load_unet_fp8 (src/cuda/weights.cu:484-486).
[[nodiscard]] inline bool is_fp8_eligible(std::string_view logical_name, std::size_t expected_rank,
                                          const FP8WeightLoadOptions& options) noexcept {
    return options.quantize_linear_weights && expected_rank == 2 && logical_name.ends_with(".weight");
}

// The FP8 format a weight is stored in (fp8_type_for, src/cuda/weights.cu:234-242): Auto keeps a
// native E5M2 checkpoint in E5M2 when native formats are preserved and stores everything else as E4M3.
[[nodiscard]] inline ScalarType fp8_type_for(ScalarType source_type, const FP8WeightLoadOptions& options) noexcept {
    if (options.format == FP8Format::E4M3) return ScalarType::Float8E4M3;
    if (options.format == FP8Format::E5M2) return ScalarType::Float8E5M2;
    if (options.preserve_native_fp8 && source_type == ScalarType::Float8E5M2) return ScalarType::Float8E5M2;
    return ScalarType::Float8E4M3;
}

// upload_or_quantize_int8_weight (src/cuda/int8_convrot.cu:498-577) for a rank-2 `source` that is
// already on the device: INT8 prequantised (+ metadata) or FP16 / FP32 to be rotated and quantised.
// `allocate(bytes)` is the integrator's persistent allocator (the reference's allocate_persistent).
[[nodiscard]] inline TensorRef upload_or_quantize_int8_weight(const Runtime& runtime, const TensorRef& source,
                                                              const QuantizationMetadata* metadata, TensorRole role,
                                                              const INT8WeightLoadOptions& options,
                                                              const Ops::Allocator& allocate) {
    if (source.rank() != 2) throw CudaError("native INT8 weight must be rank 2");
    const std::size_t rows = source.size(0), columns = source.size(1);
    if (rows == 0 || columns == 0) throw CudaError("native INT8 weight cannot be empty");
    const bool prequantized = source.type == ScalarType::Int8;
    if (options.require_prequantized && !prequantized) {
        throw CudaError("INT8 prequantized-only profile received a floating-point linear weight");
    }
    if (!prequantized && !options.quantize_floating_weights) throw CudaError("on-the-fly INT8 quantization is disabled");
    bool use_convrot = options.enable_convrot && options.convrot_group_size > 0 && columns % options.convrot_group_size == 0;
    std::size_t group = use_convrot ? options.convrot_group_size : 0;
    if (prequantized) {
        if (metadata == nullptr || metadata->weight_scale == nullptr) throw CudaError("prequantized INT8 weight is missing weight_scale");
        use_convrot = metadata->convrot;
        group = use_convrot ? metadata->convrot_group_size : 0;
        if (use_convrot && (!valid_convrot_group_size(group) || columns % group != 0)) {
            throw CudaError("prequantized ConvRot metadata is incompatible with weight shape");
        }
        if (metadata->weight_scale_count != rows) throw CudaError("prequantized INT8 weight_scale is not per-output-row");
    } else {
        if (use_convrot && !valid_convrot_group_size(group)) {
            throw CudaError("INT8 ConvRot group size must be a power of four between 4 and 256");
        }
        if (source.type != ScalarType::Float16 && source.type != ScalarType::Float32) {
            throw CudaError("native INT8 loading requires I8, F16 or F32 weights");
        }
    }
    TensorRef result;
    result.shape = {rows, columns};
    result.type = ScalarType::Int8;
    result.role = role;
    result.data = allocate(rows * columns);
    float* scales = prequantized ? const_cast<float*>(metadata->weight_scale) : static_cast<float*>(allocate(rows * sizeof(float)));
    runtime.check(sdxlq_pack_weight_int8(runtime.context(), source.data, static_cast<std::int32_t>(source.type), rows, columns,
                                         static_cast<std::uint32_t>(group), static_cast<std::int8_t*>(result.data), scales));
    result.dequant_scale_data = scales;
    result.dequant_scale_count = rows;
    result.dequant_scale_mode = FP8ScaleMode::PerOutputChannel;
    result.convrot_group_size = use_convrot ? group : 0;
    return result;
}

// The FP8 branch of WeightStore::upload_tensor (src/cuda/weights.cu:301-415): tensor-wide or
// per-output-row scale, q = FP8(value / scale); a source already stored in the target format is
// kept byte for byte with scales of 1 when preserve_native_fp8 is set. `layout` KMajorKN stores the
// matrix transposed ([K, N]), which the reference does for its weight-only kernel.
[[nodiscard]] inline TensorRef upload_fp8_weight(const Runtime& runtime, const TensorRef& source, TensorRole role,
                                                 const FP8WeightLoadOptions& options, const Ops::Allocator& allocate,
                                                 FP8StorageLayout layout = FP8StorageLayout::RowMajorNK) {
    if (options.scale_mode == FP8ScaleMode::PerOutputChannel && source.rank() != 2) {
        throw CudaError("per-output-channel FP8 scaling requires a rank-2 matrix");
    }
    if (source.rank() != 2) throw CudaError("FP8 linear weights are rank 2");
    if (options.scale_mode == FP8ScaleMode::None) throw CudaError("CUDA weight upload target must be FP8, float16, or float32");
    const ScalarType target = fp8_type_for(source.type, options);
    const bool keep = is_fp8(source.type) && source.type == target && options.preserve_native_fp8;
    if (!keep && source.type != ScalarType::Float16 && source.type != ScalarType::Float32 && !is_fp8(source.type)) {
        throw CudaError("CUDA weight upload target must be FP8, float16, or float32");
    }
    const std::size_t rows = source.size(0), columns = source.size(1);
    const std::size_t scale_count = options.scale_mode == FP8ScaleMode::PerOutputChannel ? rows : 1;
    TensorRef result;
    result.shape = {rows, columns};
    result.type = target;
    result.role = role;
    result.fp8_storage_layout = layout;
    result.data = allocate(rows * columns);
    float* scales = static_cast<float*>(allocate(scale_count * sizeof(float)));
    runtime.check(sdxlq_pack_weight_fp8(runtime.context(), source.data, static_cast<std::int32_t>(source.type), rows, columns,
                                        static_cast<std::int32_t>(target), static_cast<std::int32_t>(options.scale_mode),
                                        static_cast<std::int32_t>(layout), static_cast<std::uint8_t*>(result.data), scales));
    result.dequant_scale_data = scales;
    result.dequant_scale_count = scale_count;
    result.dequant_scale_mode = options.scale_mode;
    return result;
}

}  // namespace sdxlq
