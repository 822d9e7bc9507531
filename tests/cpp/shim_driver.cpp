// Test program for the C++ host side (sdxlq_ops.hpp / sdxlq_weights.hpp): reads one case file
// written by the Python test, runs it on the GPU through sdxlq::Ops, writes the results.
//
// Case file (little endian): uint64 m, n, k, group, activation (0 none, 1 SiLU, 4 GEGLU), precision
// (0 INT8 from FP16 weights, 1 FP8 E4M3 per channel, 2 FP16), with_residual; then FP16 X [m,k],
// FP16 W [n,k], FP16 bias [n], FP16 residual [m, n_out].
// Result file: FP16 y [m, n_out] of linear / linear_activation (with the residual added in place
// when asked), then FP16 q,k,v-style group outputs: the same projection issued three times through
// linear_group, [3, m, n] (activation none only), then uint64 INT8 linear_calls counter.
#include "sdxlq_ops.hpp"
#include "sdxlq_weights.hpp"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <vector>

namespace {

void check(cudaError_t status, const char* what) {
    if (status != cudaSuccess) {
        std::cerr << what << ": " << cudaGetErrorString(status) << "\n";
        std::exit(3);
    }
}

struct DeviceArena {
    std::vector<void*> blocks;
    void* operator()(std::size_t bytes) {
        void* pointer = nullptr;
        check(cudaMalloc(&pointer, bytes == 0 ? 16 : bytes), "cudaMalloc");
        blocks.push_back(pointer);
        return pointer;
    }
    ~DeviceArena() { for (void* block : blocks) cudaFree(block); }
};

sdxlq::TensorRef upload(DeviceArena& arena, const std::vector<std::uint16_t>& host, std::vector<std::size_t> shape) {
    sdxlq::TensorRef tensor;
    tensor.shape = std::move(shape);
    tensor.type = sdxlq::ScalarType::Float16;
    tensor.data = arena(host.size() * 2);
    check(cudaMemcpy(tensor.data, host.data(), host.size() * 2, cudaMemcpyHostToDevice), "upload");
    return tensor;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc != 3) return 2;
    try {
        // host-only checks of the profile parser (the reference's strings and their options)
        const sdxlq::PrecisionProfile fp8 = sdxlq::parse_precision_profile("FP8");
        const sdxlq::PrecisionProfile channel = sdxlq::parse_precision_profile("fp8-e4m3-channel");
        const sdxlq::PrecisionProfile strict = sdxlq::parse_precision_profile("int8-convrot-strict");
        const sdxlq::PrecisionProfile row = sdxlq::parse_precision_profile("int8-row");
        bool threw = false;
        try { (void)sdxlq::parse_precision_profile("int8-nonsense"); } catch (const sdxlq::CudaError&) { threw = true; }
        if (fp8.canonical != "fp8-auto" || !fp8.fp8 || channel.weights.scale_mode != sdxlq::FP8ScaleMode::PerOutputChannel ||
            channel.runtime_backend != sdxlq::FP8BackendPreference::WeightOnly || !strict.int8 || !strict.int8_require_tensor_cores() ||
            row.int8_weights.enable_convrot || !threw || !sdxlq::is_linear_weight("unet.mid_block.attentions.0.proj_in.weight", 2) ||
            sdxlq::is_linear_weight("text_encoder.embeddings.token_embedding.weight", 2) ||
            sdxlq::is_linear_weight("unet.conv_in.weight", 4)) {
            std::cerr << "precision profile / eligibility rules differ from the reference\n";
            return 4;
        }

        std::ifstream in(argv[1], std::ios::binary);
        std::uint64_t header[7];
        in.read(reinterpret_cast<char*>(header), sizeof(header));
        const std::size_t m = header[0], n = header[1], k = header[2], group = header[3];
        const auto activation = static_cast<sdxlq::LinearActivation>(header[4]);
        const std::uint64_t precision = header[5];
        const bool with_residual = header[6] != 0;
        const std::size_t n_out = activation == sdxlq::LinearActivation::GEGLU ? n / 2 : n;
        std::vector<std::uint16_t> x(m * k), w(n * k), b(n), r(m * n_out);
        in.read(reinterpret_cast<char*>(x.data()), x.size() * 2);
        in.read(reinterpret_cast<char*>(w.data()), w.size() * 2);
        in.read(reinterpret_cast<char*>(b.data()), b.size() * 2);
        in.read(reinterpret_cast<char*>(r.data()), r.size() * 2);
        if (!in) return 5;

        check(cudaSetDevice(0), "cudaSetDevice");
        cudaStream_t stream = nullptr;
        check(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "stream");
        DeviceArena arena;
        sdxlq::Ops::Allocator allocate = [&arena](std::size_t bytes) { return arena(bytes); };
        sdxlq::Runtime runtime(0, stream, std::size_t(256) << 20);
        sdxlq::Ops ops(runtime, allocate);

        sdxlq::TensorRef input = upload(arena, x, {m, k});
        sdxlq::TensorRef source = upload(arena, w, {n, k});
        sdxlq::TensorRef bias = upload(arena, b, {n});
        sdxlq::TensorRef weight;
        if (precision == 0) {
            sdxlq::INT8WeightLoadOptions options;
            options.convrot_group_size = group;
            options.enable_convrot = group != 0;
            weight = sdxlq::upload_or_quantize_int8_weight(runtime, source, nullptr, sdxlq::TensorRole::Model, options, allocate);
        } else if (precision == 1) {
            sdxlq::FP8WeightLoadOptions options;
            options.format = sdxlq::FP8Format::E4M3;
            options.scale_mode = sdxlq::FP8ScaleMode::PerOutputChannel;
            weight = sdxlq::upload_fp8_weight(runtime, source, sdxlq::TensorRole::Model, options, allocate);
        } else {
            weight = source;
        }

        sdxlq::TensorRef y;
        if (with_residual) {
            y = upload(arena, r, {m, n_out});
            ops.linear_add_in_place(y, input, weight, &bias);
        } else if (activation == sdxlq::LinearActivation::None) {
            y = ops.linear(input, weight, &bias);
        } else {
            y = ops.linear_activation(input, weight, bias, activation);
        }
        std::vector<sdxlq::TensorRef> group_outputs;
        if (activation == sdxlq::LinearActivation::None) group_outputs = ops.linear_group(input, {&weight, &weight, &weight});
        runtime.synchronize();

        std::ofstream out(argv[2], std::ios::binary);
        std::vector<std::uint16_t> host(m * n_out);
        check(cudaMemcpy(host.data(), y.data, host.size() * 2, cudaMemcpyDeviceToHost), "download");
        out.write(reinterpret_cast<const char*>(host.data()), host.size() * 2);
        for (const sdxlq::TensorRef& tensor : group_outputs) {
            std::vector<std::uint16_t> part(m * n);
            check(cudaMemcpy(part.data(), tensor.data, part.size() * 2, cudaMemcpyDeviceToHost), "download");
            out.write(reinterpret_cast<const char*>(part.data()), part.size() * 2);
        }
        const std::uint64_t calls = runtime.int8_execution_stats().linear_calls;
        out.write(reinterpret_cast<const char*>(&calls), sizeof(calls));

        // LayerNorm in front of the projection: the fused form (quantised rows straight out of the norm)
        // against layer_norm followed by linear, bit for bit
        if (precision != 2 && k <= 2048 && activation == sdxlq::LinearActivation::None) {
            std::vector<std::uint16_t> gamma_host(k, 0x3C00), beta_host(x.begin(), x.begin() + static_cast<std::ptrdiff_t>(k));
            sdxlq::TensorRef gamma = upload(arena, gamma_host, {k});
            sdxlq::TensorRef beta = upload(arena, beta_host, {k});
            const sdxlq::TensorRef normalised = ops.layer_norm(input, gamma, beta);
            const sdxlq::TensorRef separate = ops.linear(normalised, weight, &bias);
            const sdxlq::Ops::QuantizedActivations rows = ops.layer_norm_quantized(input, gamma, beta, weight);
            const sdxlq::TensorRef fused = ops.linear_quantized(rows, weight, &bias);
            runtime.synchronize();
            std::vector<std::uint16_t> a(m * n), c(m * n);
            check(cudaMemcpy(a.data(), separate.data, a.size() * 2, cudaMemcpyDeviceToHost), "download");
            check(cudaMemcpy(c.data(), fused.data, c.size() * 2, cudaMemcpyDeviceToHost), "download");
            if (a != c) {
                std::cerr << "fused LayerNorm projection differs from layer_norm + linear\n";
                return 7;
            }
        }

        // error behaviour: the reference's message for a feature mismatch
        sdxlq::TensorRef wrong = input;
        wrong.shape = {m, k + 1};
        bool mismatch = false;
        try { (void)ops.linear(wrong, weight); } catch (const sdxlq::CudaError& error) { mismatch = std::string(error.what()) == "CUDA linear feature mismatch"; }
        if (!mismatch) return 6;
        return 0;
    } catch (const std::exception& failure) {
        std::cerr << "shim_driver: " << failure.what() << "\n";
        return 1;
    }
}
