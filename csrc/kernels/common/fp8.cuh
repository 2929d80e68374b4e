// fp8 e4m3 block-scaling helpers shared by the quantisation kernels and by the
// dispatch kernel that quantises tokens on their way out.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace slime {

constexpr float kFp8Max      = 448.0f;
constexpr float kFp8AmaxFloor = 1e-4f;

// Block scaling: with c = max(amax, floor), scale = c / 448 is what the consumer multiplies by and
// inv = 448 / c is what the producer multiplies by. Both are IEEE divisions, done once per block, so
// that the per-element work is one multiply and the result can be restated bit for bit on the host.
struct Fp8Scale {
    float scale;
    float inv;
};

__device__ __forceinline__ Fp8Scale fp8_scale_from_amax(float amax)
{
    const float c = fmaxf(amax, kFp8AmaxFloor);
    return {__fdiv_rn(c, kFp8Max), __fdiv_rn(kFp8Max, c)};
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& raw, float* v)
{
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(p[i]);
        v[2 * i]       = f.x;
        v[2 * i + 1]   = f.y;
    }
}

__device__ __forceinline__ uint4 pack_bf16x8(const float* v)
{
    uint4           out;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return out;
}

// q[i] = rne_sat(v[i] * inv), eight values packed little-endian.
__device__ __forceinline__ uint2 quant_fp8x8(const float* v, float inv)
{
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float2 a = make_float2(__fmul_rn(v[4 * h + 0], inv), __fmul_rn(v[4 * h + 1], inv));
        const float2 b = make_float2(__fmul_rn(v[4 * h + 2], inv), __fmul_rn(v[4 * h + 3], inv));
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(a, __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(b, __NV_SATFINITE, __NV_E4M3);
        w[h]              = lo | (hi << 16);
    }
    return make_uint2(w[0], w[1]);
}

__device__ __forceinline__ void dequant_fp8x8(const uint2& raw, float scale, float* v)
{
    const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const __nv_fp8x2_storage_t s  = static_cast<__nv_fp8x2_storage_t>((w[h] >> (16 * j)) & 0xffffu);
            const __half2_raw          hr = __nv_cvt_fp8x2_to_halfraw2(s, __NV_E4M3);
            const float2               f  = __half22float2(*reinterpret_cast<const __half2*>(&hr));
            v[4 * h + 2 * j]              = f.x * scale;
            v[4 * h + 2 * j + 1]          = f.y * scale;
        }
    }
}

}  // namespace slime
