// Per-row INT8 scale and cast arithmetic shared by the throughput quantisers and the LayerNorm -> INT8
// kernel: activation_amax_kernel + quantize_activation_kernel of the reference
// (src/cuda/int8_convrot.cu:265-353): scale = max(amax / 127, 1e-30) (1 if amax == 0, amax over finite
// values only), q = clamp(rn(x * (1 / scale)), -128, 127).
#pragma once

#include <cuda_fp16.h>
#include <cstdint>

namespace sdxlq {

__device__ __forceinline__ float scale_from_amax(float maximum) {
    return maximum > 0.0f ? fmaxf(__fdiv_rn(maximum, 127.0f), 1.0e-30f) : 1.0f;
}

// clamp(rn(x), -128, 127) as a sign-extended 32-bit integer; NaN -> 0 (like __float2int_rn + clamp).
__device__ __forceinline__ uint32_t quantize_s8(float value) {
    uint32_t result;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(result) : "f"(value));
    return result;
}

// The low bytes of four integers -> one little-endian word.
__device__ __forceinline__ uint32_t pack_bytes(uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
    const uint32_t lo = __byte_perm(b0, b1, 0x0040);
    const uint32_t hi = __byte_perm(b2, b3, 0x0040);
    return __byte_perm(lo, hi, 0x5410);
}

__device__ __forceinline__ float half_lo(uint32_t word) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(word & 0xFFFFu)));
}
__device__ __forceinline__ float half_hi(uint32_t word) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(word >> 16)));
}

__device__ __forceinline__ uint2 quantize_vector(const uint4 raw, float inverse_scale) {
    const uint32_t q0 = quantize_s8(__fmul_rn(half_lo(raw.x), inverse_scale));
    const uint32_t q1 = quantize_s8(__fmul_rn(half_hi(raw.x), inverse_scale));
    const uint32_t q2 = quantize_s8(__fmul_rn(half_lo(raw.y), inverse_scale));
    const uint32_t q3 = quantize_s8(__fmul_rn(half_hi(raw.y), inverse_scale));
    const uint32_t q4 = quantize_s8(__fmul_rn(half_lo(raw.z), inverse_scale));
    const uint32_t q5 = quantize_s8(__fmul_rn(half_hi(raw.z), inverse_scale));
    const uint32_t q6 = quantize_s8(__fmul_rn(half_lo(raw.w), inverse_scale));
    const uint32_t q7 = quantize_s8(__fmul_rn(half_hi(raw.w), inverse_scale));
    return make_uint2(pack_bytes(q0, q1, q2, q3), pack_bytes(q4, q5, q6, q7));
}

__device__ __forceinline__ __half2 as_half2(uint32_t word) {
    return *reinterpret_cast<const __half2*>(&word);
}

// Finite-only |x| maximum of one 16-byte vector, the slow path used when a row holds infinities.
__device__ __forceinline__ float finite_max(const uint4 raw, float current) {
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float lo = fabsf(half_lo(words[i])), hi = fabsf(half_hi(words[i]));
        if (lo <= 3.402823466e+38f && lo > current) current = lo;
        if (hi <= 3.402823466e+38f && hi > current) current = hi;
    }
    return current;
}

}  // namespace sdxlq
