// Per-token FP8 (E4M3FN) wire format helpers, used inside the dispatch send and receive warps.
//
// Rules (reference: csrc/kernels/host_staged/quantization.cuh:16-71): scale = amax/448 floored at
// the smallest normal FP32, 1 for an all-zero row; encode = cvt.rn.satfinite.e4m3(x * (1/scale));
// decode = bf16_rn(float(fp8) * scale).  Unlike the reference there is no staging pass through
// HBM: a send warp reduces amax over the row it already holds and converts on the way out.
#pragma once

#include <cstdint>

#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace bep {

constexpr float kFp8Max = 448.0f;
constexpr float kFp32MinNormal = 1.17549435e-38f;

__device__ __forceinline__ float fp8_scale_from_amax(float amax) {
    return amax == 0.0f ? 1.0f : fmaxf(amax / kFp8Max, kFp32MinNormal);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// |max| over the 8 BF16 values packed in a 16-byte chunk
__device__ __forceinline__ float chunk_amax(const uint4& v) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
    return m;
}

// 8 BF16 -> 8 E4M3 bytes
__device__ __forceinline__ uint2 chunk_to_fp8(const uint4& v, float inv_scale) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    std::uint32_t out[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float2 a = __bfloat1622float2(h[2 * i]);
        float2 b = __bfloat1622float2(h[2 * i + 1]);
        a.x *= inv_scale; a.y *= inv_scale; b.x *= inv_scale; b.y *= inv_scale;
        const std::uint32_t lo = __nv_cvt_float2_to_fp8x2(a, __NV_SATFINITE, __NV_E4M3);
        const std::uint32_t hi = __nv_cvt_float2_to_fp8x2(b, __NV_SATFINITE, __NV_E4M3);
        out[i] = lo | (hi << 16);
    }
    return make_uint2(out[0], out[1]);
}

// 8 E4M3 bytes -> 8 BF16
__device__ __forceinline__ uint4 chunk_from_fp8(const uint2& v, float scale) {
    const std::uint16_t* p = reinterpret_cast<const std::uint16_t*>(&v);
    uint4 out;
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2_raw raw = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(p[i]), __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&raw));
        o[i] = __floats2bfloat162_rn(f.x * scale, f.y * scale);
    }
    return out;
}

__device__ __forceinline__ std::uint8_t scalar_to_fp8(__nv_bfloat16 v, float inv_scale) {
    return static_cast<std::uint8_t>(__nv_cvt_float_to_fp8(__bfloat162float(v) * inv_scale, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ __nv_bfloat16 scalar_from_fp8(std::uint8_t v, float scale) {
    const __half_raw raw = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(v), __NV_E4M3);
    return __float2bfloat16_rn(__half2float(*reinterpret_cast<const __half*>(&raw)) * scale);
}

}  // namespace bep
