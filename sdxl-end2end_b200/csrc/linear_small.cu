// Small-shape Linear: the same operator as the tensor-core GEMM for shapes a TMA tensor map
// cannot describe (row pitch not a multiple of 16 bytes, e.g. the 2x4 / 2x2 known-answer
// cases of the reference's operator test) and for K-major FP8 weights
// (FP8StorageLayout::KMajorKN). One thread per output element; identical epilogue arithmetic.

#include "internal.cuh"

#include <cuda_fp8.h>

namespace sdxlq {

struct SmallLinearParams {
    const void* a;               // quantised activations (INT8 / FP8) or FP16 activations, [M, K]
    const void* b;               // weights [N, K] (or [K, N] when k_major)
    EpilogueParams ep;
    uint32_t k_major;
};

namespace {

__device__ __forceinline__ float decode_fp8(uint8_t bits, uint32_t kind) {
    const __half_raw raw = __nv_cvt_fp8_to_halfraw(bits, kind == KIND_E4M3 ? __NV_E4M3 : __NV_E5M2);
    return __half2float(__half(raw));
}

__device__ __forceinline__ uint32_t dot_bits(const SmallLinearParams& p, uint32_t row, uint32_t col) {
    const EpilogueParams& ep = p.ep;
    const uint32_t k = ep.k;
    if (ep.kind == KIND_I8) {
        const int8_t* a = static_cast<const int8_t*>(p.a) + static_cast<size_t>(row) * k;
        const int8_t* b = static_cast<const int8_t*>(p.b) + static_cast<size_t>(col) * k;
        int32_t sum = 0;
        for (uint32_t i = 0; i < k; ++i) sum += static_cast<int32_t>(a[i]) * static_cast<int32_t>(b[i]);
        return static_cast<uint32_t>(sum);
    }
    float sum = 0.0f;
    if (ep.kind == KIND_F16) {
        const __half* a = static_cast<const __half*>(p.a) + static_cast<size_t>(row) * k;
        const __half* b = static_cast<const __half*>(p.b) + static_cast<size_t>(col) * k;
        for (uint32_t i = 0; i < k; ++i) sum = fmaf(__half2float(a[i]), __half2float(b[i]), sum);
    } else {
        const uint8_t* a = static_cast<const uint8_t*>(p.a) + static_cast<size_t>(row) * k;
        const uint8_t* b = static_cast<const uint8_t*>(p.b);
        for (uint32_t i = 0; i < k; ++i) {
            const size_t index = p.k_major ? static_cast<size_t>(i) * ep.n + col : static_cast<size_t>(col) * k + i;
            sum = fmaf(decode_fp8(a[i], ep.kind), decode_fp8(b[index], ep.kind), sum);
        }
    }
    return __float_as_uint(sum);
}

}  // namespace

__global__ void __launch_bounds__(256)
sdxlq_small_linear_kernel(const __grid_constant__ SmallLinearParams p) {
    const EpilogueParams& ep = p.ep;
    const size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= static_cast<size_t>(ep.m) * ep.n_out) return;
    const uint32_t row = static_cast<uint32_t>(index / ep.n_out);
    const uint32_t col = static_cast<uint32_t>(index % ep.n_out);
    const uint32_t kind = ep.kind;
    float a_scale = 1.0f;
    if (kind == KIND_I8) a_scale = ep.a_scales[row];
    else if (kind != KIND_F16) a_scale = ep.a_scales[0];
    const bool scaled = kind != KIND_F16;
    const bool has_bias = ep.bias != nullptr;

    const uint32_t acc = dot_bits(p, row, col);
    if (ep.acc_out != nullptr) ep.acc_out[static_cast<size_t>(row) * ep.n + col] = static_cast<int32_t>(acc);
    const float w_scale = scaled ? ep.w_scales[ep.w_scale_per_channel ? col : 0] : 1.0f;
    const __half y = project_to_half(acc, kind, a_scale, w_scale);
    __half result;
    if (ep.activation == ACT_GEGLU) {
        const uint32_t gate_col = ep.n_out + col;
        const uint32_t gate_acc = dot_bits(p, row, gate_col);
        if (ep.acc_out != nullptr) ep.acc_out[static_cast<size_t>(row) * ep.n + gate_col] = static_cast<int32_t>(gate_acc);
        const float gate_scale = scaled ? ep.w_scales[ep.w_scale_per_channel ? gate_col : 0] : 1.0f;
        const __half y_gate = project_to_half(gate_acc, kind, a_scale, gate_scale);
        result = finish_geglu(y, ep.bias[col], y_gate, ep.bias[gate_col]);
    } else {
        result = finish_scalar(y, has_bias, has_bias ? ep.bias[col] : __half(0), ep.activation);
        // Ops::add_in_place after the Linear, folded in (may alias y: each thread reads its element first)
        if (ep.residual != nullptr) result = __hadd(result, ep.residual[static_cast<size_t>(row) * ep.n_out + col]);
    }
    ep.y[static_cast<size_t>(row) * ep.n_out + col] = result;
    // the maximum of |y| for the consumer's FP8 quantiser (bit patterns of non-negative floats order like integers)
    if (ep.y_amax != nullptr) atomicMax(ep.y_amax, __float_as_uint(fabsf(__half2float(result))));
}

cudaError_t launch_small_linear(const void* a, const void* b, const EpilogueParams& ep, uint32_t k_major,
                                cudaStream_t stream) {
    SmallLinearParams params;
    params.a = a;
    params.b = b;
    params.ep = ep;
    params.k_major = k_major;
    const size_t outputs = static_cast<size_t>(ep.m) * ep.n_out;
    if (outputs == 0) return cudaSuccess;
    sdxlq_small_linear_kernel<<<static_cast<unsigned>((outputs + 255) / 256), 256, 0, stream>>>(params);
    return cudaGetLastError();
}

}  // namespace sdxlq
