// Device helpers shared by the bandwidth-bound kernels: 4-element vector access
// for the operand formats of the contractions and the reference's scalar math.
#pragma once
#include "common.cuh"

namespace ts2 {

template <int FT>
struct Fast;

// e4m3 bytes, saturating round-to-nearest-even (activations and gradients)
template <>
struct Fast<0> {
    static constexpr int SIZE = 1;
    static __device__ __forceinline__ void store4(void *base, size_t idx, float4 v)
    {
        __nv_fp8x4_e4m3 p(v);
        *(uint32_t *)((uint8_t *)base + idx) = p.__x;
    }
    static __device__ __forceinline__ void zero4(void *base, size_t idx) { *(uint32_t *)((uint8_t *)base + idx) = 0u; }
    static __device__ __forceinline__ float4 load4(const void *base, size_t idx)
    {
        uint32_t raw = *(const uint32_t *)((const uint8_t *)base + idx);
        __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(raw & 0xffff), __NV_E4M3);
        __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(raw >> 16), __NV_E4M3);
        float2 a = __half22float2(*(__half2 *)&lo), b = __half22float2(*(__half2 *)&hi);
        return make_float4(a.x, a.y, b.x, b.y);
    }
};

template <>
struct Fast<1> {
    static constexpr int SIZE = 2;
    static __device__ __forceinline__ void store4(void *base, size_t idx, float4 v)
    {
        __half2 a = sat_half2(v.x, v.y), b = sat_half2(v.z, v.w);
        *(uint2 *)((__half *)base + idx) = make_uint2(*(uint32_t *)&a, *(uint32_t *)&b);
    }
    static __device__ __forceinline__ void zero4(void *base, size_t idx) { *(uint2 *)((__half *)base + idx) = make_uint2(0u, 0u); }
    static __device__ __forceinline__ float4 load4(const void *base, size_t idx)
    {
        uint2 raw = *(const uint2 *)((const __half *)base + idx);
        float2 a = __half22float2(*(__half2 *)&raw.x), b = __half22float2(*(__half2 *)&raw.y);
        return make_float4(a.x, a.y, b.x, b.y);
    }
};

// int8, round to nearest even, saturating (CvtToI8, src/lib/cuda/cuda_util.cuh:61-66)
__device__ __forceinline__ uint32_t sat_i8(float x)
{
    int32_t r;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(x));
    return (uint32_t)r & 0xffu;
}
template <>
struct Fast<2> {
    static constexpr int SIZE = 1;
    static __device__ __forceinline__ void store4(void *base, size_t idx, float4 v)
    {
        *(uint32_t *)((uint8_t *)base + idx) = sat_i8(v.x) | (sat_i8(v.y) << 8) | (sat_i8(v.z) << 16) | (sat_i8(v.w) << 24);
    }
    static __device__ __forceinline__ void zero4(void *base, size_t idx) { *(uint32_t *)((uint8_t *)base + idx) = 0u; }
    static __device__ __forceinline__ float4 load4(const void *base, size_t idx)
    {
        const char4 raw = *(const char4 *)((const uint8_t *)base + idx);
        return make_float4((float)raw.x, (float)raw.y, (float)raw.z, (float)raw.w);
    }
};

__device__ __forceinline__ float4 load_half4(const __half *p)
{
    uint2 raw = *(const uint2 *)p;
    float2 a = __half22float2(*(__half2 *)&raw.x), b = __half22float2(*(__half2 *)&raw.y);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store_half4(__half *p, float4 v)
{
    __half2 a = sat_half2(v.x, v.y), b = sat_half2(v.z, v.w);
    *(uint2 *)p = make_uint2(*(uint32_t *)&a, *(uint32_t *)&b);
}

__device__ __forceinline__ float dot4(float4 a, float4 b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }
__device__ __forceinline__ float4 scale4(float4 a, float s) { return make_float4(a.x * s, a.y * s, a.z * s, a.w * s); }
__device__ __forceinline__ float4 axpy4(float a, float4 x, float4 y)
{
    return make_float4(a * x.x + y.x, a * x.y + y.y, a * x.z + y.z, a * x.w + y.w);
}

// CpuComputeLolu, src/gpt/compute/cpu_util.cpp:139-151 (LOLU_SCALE = 2): exp(2x) / (1 + exp(2x)) with the
// result pinned to 0 / 1 beyond |2x| > 20.  Written as 1 / (1 + exp(-2x)) with the hardware exponential and
// reciprocal (relative error ~1e-6, far below the fp16 / e4m3 rounding of the result); the saturation is
// what the formula gives by itself (exp(20) ~ 4.9e8), so the two branches of the reference are kept only to
// return exactly 0 and 1.
__device__ __forceinline__ float lolu_mult(float gate)
{
    const float arg = gate * 2.f;
    const float r = __fdividef(1.f, 1.f + __expf(-arg));
    return arg < -20.f ? 0.f : (arg > 20.f ? 1.f : r);
}

// The same multiplier where the result is stored as e4m3 (FT == 0): sigmoid(2 g) = 0.5 + 0.5 tanh(g) with the
// one-instruction tanh (relative error 2^-11, far below the e4m3 step); the fp16 pipeline keeps the exact form.
template <int FT>
__device__ __forceinline__ float lolu_mult_ft(float gate)
{
    if (FT == 0) { // FT 1 (fp16) and 2 (int8, steps of 1/24 of the rms) keep the exact form
        float th;
        asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(gate));
        return fmaf(th, 0.5f, 0.5f);
    }
    return lolu_mult(gate);
}

// Packed fp16 arithmetic for the e4m3 pipeline's element-wise kernels.  Those kernels were bound by instruction issue,
// not by memory (about 190 warp instructions per 128 elements: three fp16 -> fp32 conversions, one MUFU and an
// fp32 -> e4m3 conversion per element): in packed fp16 one instruction serves two elements, the exponential included,
// and the result converts to two e4m3 bytes in one step.  fp16 carries 11 bits, the e4m3 results 4.
__device__ __forceinline__ __half2 h2_from_bits(uint32_t w) { return *(const __half2 *)&w; }
__device__ __forceinline__ uint32_t bits_from_h2(__half2 v) { return *(const uint32_t *)&v; }
__device__ __forceinline__ __half2 tanh_h2(__half2 v)
{
    uint32_t r;
    asm("tanh.approx.f16x2 %0, %1;" : "=r"(r) : "r"(bits_from_h2(v)));
    return h2_from_bits(r);
}
// sigmoid(2 g) = 0.5 + 0.5 tanh(g) for two gates
__device__ __forceinline__ __half2 lolu_mult_h2(__half2 gate)
{
    const __half2 half = __float2half2_rn(0.5f);
    return __hfma2(tanh_h2(gate), half, half);
}
// two fp16 -> two e4m3 bytes (low element in the low byte), nearest even, saturating (an infinity becomes 448)
__device__ __forceinline__ uint32_t e4m3x2_from_h2(__half2 v)
{
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(r) : "r"(bits_from_h2(v)));
    return r;
}
__device__ __forceinline__ uint32_t e4m3x4_from_h2(__half2 lo, __half2 hi) { return e4m3x2_from_h2(lo) | (e4m3x2_from_h2(hi) << 16); }

// scale of one 128-wide tile: sqrt(128 / sum of squares), 0 for an all-zero tile
__device__ __forceinline__ float tile_scale(float sum2) { return sum2 == 0.f ? 0.f : 11.3137085f * rsqrtf(sum2); }

// Weight encoder of the reference's CPU path for e4m3 (ConvertToFp8e4m3,
// src/gpt/model_params/sse_utils.h:161-204): round half away from zero on the 4th
// mantissa bit, values below 2^-7 become 0, saturate to +-448.  Bit-exact with it.
__device__ __forceinline__ uint8_t encode_e4m3_weight(float v)
{
    uint32_t bits = __float_as_uint(v);
    float f0 = __uint_as_float(bits & 0xFF800000u), f1 = __uint_as_float(bits & 0xFF880000u);
    v = __fadd_rn(v, __fsub_rn(f1, f0));
    bits = __float_as_uint(v);
    int sign = bits >> 31;
    int exponent = (int)((bits & 0x7F800000u) >> 23) - 120;
    int mantissa = (bits & 0x007FFFFFu) >> 20;
    int fp8 = (sign << 7) | (exponent << 3) | mantissa;
    if (exponent > 15)
        fp8 = (sign << 7) | 0x7f;
    if (exponent < 0)
        fp8 = 0;
    fp8 &= 0xff;
    if (fp8 == 0xff)
        fp8 = 0xfe;
    if (fp8 == 0x7f)
        fp8 = 0x7e;
    return (uint8_t)fp8;
}

} // namespace ts2
