// TEST INFRASTRUCTURE ONLY — never linked into the shipped library.
//
// Exposes the reference's own CPU `linear_2d` and `geglu` (src/unet.cpp:202-235,
// 483-493 of the reference project) through a C ABI so that the restated oracle
// can be validated against the unmodified reference arithmetic, and so that the
// benchmark's CPU arm can time it.
//
// Those functions live in an anonymous namespace, so this translation unit
// includes the reference source file textually at build time (the include path is
// supplied by oracle/Makefile via -I<reference root>); no reference source is
// copied into this repository.

#include "src/unet.cpp"

#include "sdxl/scheduler.hpp"

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <filesystem>
#include <string>
#include <utility>
#include <vector>

namespace {

sdxl::TensorView make_view(const void* data, int dtype, const std::uint64_t* shape, int rank) {
    sdxl::TensorView view;
    view.data = static_cast<const std::byte*>(data);
    switch (dtype) {
    case 0: view.dtype = sdxl::DType::F16; break;
    case 1: view.dtype = sdxl::DType::F32; break;
    case 2: view.dtype = sdxl::DType::F8E4M3FN; break;
    case 3: view.dtype = sdxl::DType::F8E5M2; break;
    default: view.dtype = sdxl::DType::F32; break;
    }
    const std::int64_t element = (dtype == 0) ? 2 : (dtype == 1 ? 4 : 1);
    view.shape.assign(shape, shape + rank);
    view.strides_bytes.assign(static_cast<std::size_t>(rank), 0);
    std::int64_t stride = element;
    for (int d = rank - 1; d >= 0; --d) {
        view.strides_bytes[static_cast<std::size_t>(d)] = stride;
        stride *= static_cast<std::int64_t>(shape[d]);
    }
    view.storage_bytes = static_cast<std::uint64_t>(stride);
    view.source_key = "harness";
    return view;
}

} // namespace

extern "C" {

// Y[rows, out] = X[rows, in] * W[out, in]^T (+ bias); W/bias dtype: 0=f16, 1=f32, 2=e4m3fn, 3=e5m2.
// Returns 0 on success, 1 when the reference threw.
int ref_linear_2d(const float* input, std::uint64_t rows, std::uint64_t in_features,
                  const void* weight, int weight_dtype, std::uint64_t out_features,
                  const void* bias, int bias_dtype, float* output) {
    try {
        sdxl::FloatTensor x;
        x.shape = {static_cast<std::size_t>(rows), static_cast<std::size_t>(in_features)};
        x.values.assign(input, input + rows * in_features);
        const std::uint64_t wshape[2] = {out_features, in_features};
        const sdxl::TensorView w = make_view(weight, weight_dtype, wshape, 2);
        sdxl::FloatTensor y;
        if (bias != nullptr) {
            const std::uint64_t bshape[1] = {out_features};
            const sdxl::TensorView b = make_view(bias, bias_dtype, bshape, 1);
            y = sdxl::linear_2d(x, w, &b);
        } else {
            y = sdxl::linear_2d(x, w, nullptr);
        }
        std::memcpy(output, y.values.data(), y.values.size() * sizeof(float));
        return 0;
    } catch (...) {
        return 1;
    }
}

// out[rows, width] = in[rows, :width] * gelu(in[rows, width:2*width])
int ref_geglu(const float* input, std::uint64_t rows, std::uint64_t width2, float* output) {
    try {
        sdxl::FloatTensor x;
        x.shape = {1, static_cast<std::size_t>(rows), static_cast<std::size_t>(width2)};
        x.values.assign(input, input + rows * width2);
        const sdxl::FloatTensor y = sdxl::geglu(x);
        std::memcpy(output, y.values.data(), y.values.size() * sizeof(float));
        return 0;
    } catch (...) {
        return 1;
    }
}

float ref_gelu(float x) { return sdxl::gelu(x); }

// Opens a safetensors file with the reference's own parser (sdxl::SafeTensorFile,
// src/safetensors.cpp) and reports one tensor: dtype as the reference's DType value, rank, shape
// (up to 4 dimensions), byte count, and up to `capacity` leading bytes of its data. Returns 0 on
// success, 1 when the reference threw (malformed file, missing key), 2 for a rank above 4.
int ref_safetensors_probe(const char* path, const char* key, int* dtype, int* rank, std::uint64_t* shape,
                          std::uint64_t* bytes, unsigned char* data, std::uint64_t capacity) {
    try {
        const sdxl::SafeTensorFile file{std::filesystem::path(path)};
        const sdxl::TensorView view = file.tensor(key);
        if (view.shape.size() > 4) return 2;
        *dtype = static_cast<int>(view.dtype);
        *rank = static_cast<int>(view.shape.size());
        for (std::size_t d = 0; d < view.shape.size(); ++d) shape[d] = view.shape[d];
        *bytes = view.logical_bytes();
        const std::uint64_t count = *bytes < capacity ? *bytes : capacity;
        std::memcpy(data, view.data, static_cast<std::size_t>(count));
        return 0;
    } catch (const std::exception&) {
        return 1;
    }
}

// ---- the reference's parameter graph and CPU UNet executor ------------------------------------
//
// A handle owns an sdxl::SDXLModel built from the given UNet configuration (every other field as
// in SDXLConfig::base_1_0, src/sdxl.cpp:869-892). Parameters are bound to caller-owned FP32
// buffers by name, like the reference's tests bind their miniature models
// (tests/unet_scheduler_test.cpp:18-60), and SDXLUNet::forward (src/unet.cpp:699-807) runs on them.
struct RefUNet {
    sdxl::SDXLModel model;
    std::vector<std::pair<std::string, sdxl::ParameterSlot*>> unet_parameters;   // sorted by name
    explicit RefUNet(sdxl::SDXLConfig config) : model(std::move(config)) {
        for (auto& [name, slot] : model.graph().parameter_index()) {
            if (name.rfind("unet.", 0) == 0) unet_parameters.emplace_back(name, slot);
        }
        std::sort(unet_parameters.begin(), unet_parameters.end(),
                  [](const auto& l, const auto& r) { return l.first < r.first; });
    }
};

// config: channels[3], heads[3], transformer_depth[3], cross_attention_dim, time_embed_dim,
// addition_time_embed_dim, addition_input_dim, layers_per_block, norm_groups (15 values);
// null selects base_1_0.
void* ref_unet_create(const std::uint64_t* config) {
    try {
        sdxl::SDXLConfig cfg = sdxl::SDXLConfig::base_1_0();
        if (config != nullptr) {
            cfg.unet_channels = {config[0], config[1], config[2]};
            cfg.unet_heads = {config[3], config[4], config[5]};
            cfg.unet_transformer_depth = {config[6], config[7], config[8]};
            cfg.unet_cross_attention_dim = config[9];
            cfg.unet_time_embed_dim = config[10];
            cfg.unet_addition_time_embed_dim = config[11];
            cfg.unet_addition_input_dim = config[12];
            cfg.unet_layers_per_block = config[13];
            cfg.unet_norm_groups = config[14];
        }
        return new RefUNet(std::move(cfg));
    } catch (...) {
        return nullptr;
    }
}

void ref_unet_destroy(void* handle) { delete static_cast<RefUNet*>(handle); }

std::uint64_t ref_unet_parameter_count(void* handle) {
    return static_cast<RefUNet*>(handle)->unet_parameters.size();
}

// Name (with its "unet." prefix), rank and expected shape (up to 4 dimensions) of parameter `index`.
int ref_unet_parameter(void* handle, std::uint64_t index, char* name, std::uint64_t name_capacity, int* rank,
                       std::uint64_t* shape) {
    RefUNet* unet = static_cast<RefUNet*>(handle);
    if (index >= unet->unet_parameters.size()) return 1;
    const auto& [key, slot] = unet->unet_parameters[index];
    if (key.size() + 1 > name_capacity || slot->expected_shape.size() > 4) return 2;
    std::memcpy(name, key.c_str(), key.size() + 1);
    *rank = static_cast<int>(slot->expected_shape.size());
    for (std::size_t d = 0; d < slot->expected_shape.size(); ++d) shape[d] = slot->expected_shape[d];
    return 0;
}

// Binds parameter `name` to `count` caller-owned FP32 values (contiguous, expected shape).
int ref_unet_bind_f32(void* handle, const char* name, const float* values, std::uint64_t count) {
    RefUNet* unet = static_cast<RefUNet*>(handle);
    sdxl::ParameterSlot* slot = unet->model.graph().find_parameter(name);
    if (slot == nullptr) return 1;
    std::uint64_t expected = 1;
    for (const std::uint64_t dimension : slot->expected_shape) expected *= dimension;
    if (expected != count) return 2;
    slot->tensor = make_view(values, 1, slot->expected_shape.data(), static_cast<int>(slot->expected_shape.size()));
    return 0;
}

// SDXLUNet::forward. latents [batch,4,height,width], context [batch,tokens,cross], pooled
// [batch,pooled_width], time_ids [batch,6], all FP32; output like latents. 0 ok, 1 threw
// (message copied to `error`).
int ref_unet_forward(void* handle, const float* latents, std::uint64_t batch, std::uint64_t height, std::uint64_t width,
                     float timestep, const float* context, std::uint64_t tokens, const float* pooled,
                     std::uint64_t pooled_width, const float* time_ids, float* output, char* error,
                     std::uint64_t error_capacity) {
    try {
        RefUNet* unet = static_cast<RefUNet*>(handle);
        const std::size_t cross = static_cast<std::size_t>(unet->model.config().unet_cross_attention_dim);
        auto tensor = [](const float* data, std::vector<std::size_t> shape) {
            sdxl::FloatTensor t;
            std::size_t count = 1;
            for (const std::size_t d : shape) count *= d;
            t.shape = std::move(shape);
            t.values.assign(data, data + count);
            return t;
        };
        const sdxl::FloatTensor x = tensor(latents, {static_cast<std::size_t>(batch), 4, static_cast<std::size_t>(height), static_cast<std::size_t>(width)});
        const sdxl::FloatTensor c = tensor(context, {static_cast<std::size_t>(batch), static_cast<std::size_t>(tokens), cross});
        const sdxl::FloatTensor p = tensor(pooled, {static_cast<std::size_t>(batch), static_cast<std::size_t>(pooled_width)});
        const sdxl::FloatTensor ids = tensor(time_ids, {static_cast<std::size_t>(batch), 6});
        sdxl::UNetExecutionOptions options;
        options.check_finite_outputs = false;
        const sdxl::SDXLUNet executor(unet->model, options);
        const sdxl::FloatTensor y = executor.forward(x, timestep, c, p, ids);
        std::memcpy(output, y.values.data(), y.values.size() * sizeof(float));
        return 0;
    } catch (const std::exception& failure) {
        if (error != nullptr && error_capacity > 0) {
            std::strncpy(error, failure.what(), static_cast<std::size_t>(error_capacity - 1));
            error[error_capacity - 1] = '\0';
        }
        return 1;
    }
}

// SigmaSchedule(steps, Normal) with the default SchedulerConfig (src/scheduler.cpp:601-668):
// timesteps[steps], sigmas[steps + 1].
int ref_normal_sigma_schedule(std::uint64_t steps, float* timesteps, float* sigmas) {
    try {
        sdxl::SigmaSchedule schedule{sdxl::SchedulerConfig{}};
        schedule.set_timesteps(static_cast<std::size_t>(steps), sdxl::SchedulerKind::Normal);
        if (schedule.timesteps().size() != steps || schedule.sigmas().size() != steps + 1) return 2;
        std::memcpy(timesteps, schedule.timesteps().data(), steps * sizeof(float));
        std::memcpy(sigmas, schedule.sigmas().data(), (steps + 1) * sizeof(float));
        return 0;
    } catch (...) {
        return 1;
    }
}

} // extern "C"
