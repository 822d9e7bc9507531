// FP8 scale and cast arithmetic shared by the activation quantiser and the LayerNorm -> FP8 kernels:
// quantize_tensor_fp8 of the reference (src/cuda/fp8_kernels.cu:16-49): scale = max(amax / FP8_MAX, 1e-12)
// (1 if amax == 0), q = FP8_satfinite(x * (1 / scale)).
#pragma once

#include <cuda_fp8.h>
#include <cstdint>

namespace sdxlq {

__device__ __forceinline__ float fp8_scale_from_amax(float maximum, uint32_t fmt) {
    const float fp8_maximum = fmt == 0 ? 448.0f : 57344.0f;
    return maximum > 0.0f ? fmaxf(__fdiv_rn(maximum, fp8_maximum), 1.0e-12f) : 1.0f;
}

__device__ __forceinline__ uint32_t encode_fp8x2(float lo, float hi, uint32_t fmt) {
    const float2 pair = make_float2(lo, hi);
    return fmt == 0 ? __nv_cvt_float2_to_fp8x2(pair, __NV_SATFINITE, __NV_E4M3)
                    : __nv_cvt_float2_to_fp8x2(pair, __NV_SATFINITE, __NV_E5M2);
}

__device__ __forceinline__ uint8_t encode_fp8(float value, uint32_t fmt) {
    return fmt == 0 ? __nv_cvt_float_to_fp8(value, __NV_SATFINITE, __NV_E4M3)
                    : __nv_cvt_float_to_fp8(value, __NV_SATFINITE, __NV_E5M2);
}

}  // namespace sdxlq
