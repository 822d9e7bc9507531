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

#include <cstdint>
#include <cstring>
#include <filesystem>

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

} // extern "C"
