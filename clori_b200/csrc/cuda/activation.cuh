// Device-side pieces of the activation fake quantisation shared by the kernels that apply it.
#pragma once

#include "common.cuh"

#include <cuda_fp8.h>

namespace yvx {

// nearest FP8 E4M3 value to a magnitude in [0, 448]: 2^-9 steps below 2^-5, eight steps
// per binade above; rintf rounds halves to the even multiple = the even code
__device__ __forceinline__ float activation_nearest_fp8(float m)
{
    if (m < 0.03125f) return __fmul_rn(rintf(__fmul_rn(m, 512.0f)), 0.001953125f);
    const uint32_t step = (__float_as_uint(m) & 0x7f800000u) - (3u << 23);
    // dividing by a power of two = multiplying by its (exact) reciprocal
    return __fmul_rn(rintf(__fmul_rn(m, __uint_as_float(0x7f000000u - step))), __uint_as_float(step));
}

// the same through the conversion instructions (round to nearest even, saturating at 448):
// float -> e4m3 -> half -> float, every step after the first exact
__device__ __forceinline__ float activation_nearest_fp8_cvt(float m)
{
    const __nv_fp8_storage_t code = __nv_cvt_float_to_fp8(m, __NV_SATFINITE, __NV_E4M3);
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(code, __NV_E4M3)));
}

// nearest of {0, 0.5, 1, 1.5, 2, 3, 4, 6} to a magnitude in [0, 6]
__device__ __forceinline__ float activation_nearest_fp4(float m)
{
    if (m < 2.0f) return __fmul_rn(rintf(__fmul_rn(m, 2.0f)), 0.5f);
    if (m < 4.0f) return rintf(m);
    return __fmul_rn(rintf(__fmul_rn(m, 0.5f)), 2.0f);
}

// One 128-lane segment of a row held as four adjacent lanes per thread of a warp, quantised in
// place. A block of 4 * group lanes is `group` neighbouring threads (a power of two), which find
// their largest magnitude by shuffles. With the transform the segment is the whole (zero-padded)
// row: strides 1 and 2 are inside a thread, strides 4 to 64 are exchanges with the thread whose
// index differs in one bit, the lower index holding the left operand as in the serial loop.
// All 32 threads must call it; threads outside the row pass zeros.
template <bool HADAMARD>
__device__ __forceinline__ void activation_segment(float (&v)[4], unsigned int lane, unsigned int group, bool fp8,
                                                   float hadamard_scale)
{
    const float limit = fp8 ? 448.0f : 6.0f;
    const float floor_amax = fp8 ? 1.0e-4f : __uint_as_float(0x01c00000u);  // 6 * 2^-126
    if (HADAMARD) {
        float t0 = __fadd_rn(v[0], v[1]), t1 = __fsub_rn(v[0], v[1]);
        float t2 = __fadd_rn(v[2], v[3]), t3 = __fsub_rn(v[2], v[3]);
        v[0] = __fadd_rn(t0, t2), v[2] = __fsub_rn(t0, t2);
        v[1] = __fadd_rn(t1, t3), v[3] = __fsub_rn(t1, t3);
#pragma unroll
        for (unsigned int m = 1u; m < 32u; m <<= 1) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float other = __shfl_xor_sync(0xffffffffu, v[k], m);
                v[k] = (lane & m) ? __fsub_rn(other, v[k]) : __fadd_rn(v[k], other);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = __fmul_rn(v[k], hadamard_scale);
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = fmaxf(amax, floor_amax);
    for (unsigned int m = 1u; m < group; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    // amax / limit rounded up to a power of two, kept as an 8-bit exponent in [0, 254]; exponent 0
    // stands for 2^-127. 1 / scale is a power of two as well, so the division is a product.
    const uint32_t ratio = __float_as_uint(__fdiv_rn(amax, limit));
    uint32_t exponent = (ratio >> 23) + ((ratio & 0x007fffffu) ? 1u : 0u);
    exponent = exponent > 254u ? 254u : exponent;
    const float scale = __uint_as_float(exponent ? exponent << 23 : 0x00400000u);
    const float inverse = __uint_as_float(exponent == 254u ? 0x00400000u : (254u - exponent) << 23);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float magnitude = fminf(fabsf(__fmul_rn(v[k], inverse)), limit);
        const float nearest = fp8 ? activation_nearest_fp8_cvt(magnitude) : activation_nearest_fp4(magnitude);
        v[k] = __bfloat162float(__float2bfloat16_rn(__fmul_rn(copysignf(nearest, v[k]), scale)));  // finite here
    }
}

}  // namespace yvx
