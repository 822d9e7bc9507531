// TEST INFRASTRUCTURE ONLY — never linked into the shipped library.
//
// Exposes the reference's threaded AVX2 `linear` (src/text_encoder.cpp:244-310 of
// the reference project: `dot_product` + output-block task split over
// `parallel_tasks`) through a C ABI. It is the reference's only multi-threaded
// CPU Linear, used as the "all host threads" CPU arm of the benchmark.
// The reference file is included textually at build time; nothing is copied.

#include "src/text_encoder.cpp"

#include <cstdint>
#include <cstring>

extern "C" {

// Y[rows, out] = X * W^T + bias with F32 or F16 weights (0=f16, 1=f32).
// threads == 0 selects hardware_concurrency() like the reference.
int ref_linear_threaded(const float* input, std::uint64_t rows, std::uint64_t in_features,
                        const void* weight, int weight_dtype, std::uint64_t out_features,
                        const void* bias, int bias_dtype, std::uint64_t threads, float* output) {
    try {
        auto make_view = [](const void* data, int dtype, std::vector<std::uint64_t> shape) {
            sdxl::TensorView view;
            view.data = static_cast<const std::byte*>(data);
            view.dtype = dtype == 0 ? sdxl::DType::F16 : sdxl::DType::F32;
            const std::int64_t element = dtype == 0 ? 2 : 4;
            view.shape = shape;
            view.strides_bytes.assign(shape.size(), 0);
            std::int64_t stride = element;
            for (std::size_t d = shape.size(); d-- > 0;) {
                view.strides_bytes[d] = stride;
                stride *= static_cast<std::int64_t>(shape[d]);
            }
            view.storage_bytes = static_cast<std::uint64_t>(stride);
            view.source_key = "harness";
            return view;
        };
        std::vector<float> x(input, input + rows * in_features);
        const sdxl::TensorView w = make_view(weight, weight_dtype, {out_features, in_features});
        sdxl::TextEncoderExecutionOptions options;
        options.thread_count = static_cast<std::size_t>(threads);
        std::vector<float> y;
        if (bias != nullptr) {
            const sdxl::TensorView b = make_view(bias, bias_dtype, {out_features});
            y = sdxl::linear(x, static_cast<std::size_t>(rows), static_cast<std::size_t>(in_features),
                             w, &b, options);
        } else {
            y = sdxl::linear(x, static_cast<std::size_t>(rows), static_cast<std::size_t>(in_features),
                             w, nullptr, options);
        }
        std::memcpy(output, y.data(), y.size() * sizeof(float));
        return 0;
    } catch (...) {
        return 1;
    }
}

unsigned ref_hardware_threads() {
    const unsigned detected = std::thread::hardware_concurrency();
    return detected == 0 ? 1U : detected;
}

} // extern "C"
