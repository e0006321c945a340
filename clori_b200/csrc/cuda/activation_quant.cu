// Activation fake quantisation of rows in place: optional Hadamard transform, then per
// block a power-of-two scale and the nearest FP8 E4M3 / FP4 E2M1 value, published as bf16.
//
// Replaces yvex_attention_activation_apply (src/graph/core.c:829-945, with
// yvex_attention_hadamard_cpu and attention_fake_quant_block, src/graph/numeric.c:
// 1008-1078 and 1210-1258) and its CUDA twin yvex_attention_activation_quantize
// (src/backend/cuda/kernels.cu:1136). The reference's encoder searches all codes for the
// nearest value with ties to the even code; for these two formats that is round-to-
// nearest-even on a grid whose step depends on the binade, which is what this kernel
// computes directly. Each butterfly output is one single-precision add or subtract of
// the same two operands as on the CPU, the scale is a power of two, and the product with
// it is exact, so results are bit-equal whatever the order the threads run in.
// One CTA per row; a warp owns a quantisation block at a time.
#include "common.cuh"

#include <cuda_fp8.h>

namespace yvx {

constexpr int kActivationThreads = 128;

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

__global__ void __launch_bounds__(kActivationThreads)
activation_quant_kernel(const yvx_activation_args a, unsigned int padded)
{
    extern __shared__ float row[];
    const unsigned int tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    float *values = a.values + (unsigned long long)blockIdx.x * a.row_stride;
    const unsigned int count = (unsigned int)a.count;
    bool finite = true;
    for (unsigned int i = tid; i < padded; i += kActivationThreads) {
        const float v = i < count ? values[i] : 0.0f;
        finite = finite && isfinite(v);
        row[i] = v;
    }
    if (a.hadamard) {
        for (unsigned int step = 1u; step < padded; step <<= 1) {
            __syncthreads();
            for (unsigned int pair = tid; pair < padded / 2u; pair += kActivationThreads) {
                const unsigned int i = (pair / step) * 2u * step + pair % step;
                const float left = row[i], right = row[i + step];
                row[i] = __fadd_rn(left, right);
                row[i + step] = __fsub_rn(left, right);
            }
        }
        __syncthreads();
        for (unsigned int i = tid; i < count; i += kActivationThreads)
            row[i] = __fmul_rn(row[i], a.hadamard_scale);
    }
    __syncthreads();
    const bool fp8 = a.quantization == 8u;
    const float limit = fp8 ? 448.0f : 6.0f;
    const float floor_amax = fp8 ? 1.0e-4f : __uint_as_float(0x01c00000u);  // 6 * 2^-126
    for (unsigned int block = warp; block < count / a.block_width; block += kActivationThreads / 32) {
        const unsigned int base = block * a.block_width;
        float amax = floor_amax;
        for (unsigned int e = lane; e < a.block_width; e += 32u) {
            const float v = row[base + e];
            finite = finite && isfinite(v);
            amax = fmaxf(amax, fabsf(v));
        }
        amax = warp_max(amax);
        // amax / limit rounded up to a power of two, kept as an 8-bit exponent in [0, 254];
        // exponent 0 stands for 2^-127
        const uint32_t ratio = __float_as_uint(__fdiv_rn(amax, limit));
        uint32_t exponent = (ratio >> 23) + ((ratio & 0x007fffffu) ? 1u : 0u);
        exponent = exponent > 254u ? 254u : exponent;
        const float scale = __uint_as_float(exponent ? exponent << 23 : 0x00400000u);
        for (unsigned int e = lane; e < a.block_width; e += 32u) {
            const float v = row[base + e];
            float normalized = __fdiv_rn(v, scale);
            float magnitude = fminf(fabsf(normalized), limit);
            const float nearest = fp8 ? activation_nearest_fp8(magnitude) : activation_nearest_fp4(magnitude);
            const float restored = __fmul_rn(copysignf(nearest, v), scale);
            values[base + e] = __uint_as_float((uint32_t)bf16_bits_rne(restored) << 16);
        }
    }
    if (!finite) atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
}

// One warp per row, four adjacent lanes per thread, 16-byte accesses, no shared memory:
// rows are walked in segments of 128 lanes; a block of block_width lanes is block_width / 4
// neighbouring threads, which find their largest magnitude by shuffles. With the transform
// the row is one segment (at most 128 lanes): strides 1 and 2 are inside a thread, strides
// 4 to 64 are exchanges with the thread whose index differs in one bit, the lower index
// holding the left operand as in the serial loop.
template <bool HADAMARD>
__global__ void __launch_bounds__(kActivationThreads)
activation_quant_warp_kernel(const yvx_activation_args a)
{
    const unsigned int lane = threadIdx.x & 31u;
    const unsigned long long r = (unsigned long long)blockIdx.x * (kActivationThreads / 32) + (threadIdx.x >> 5);
    if (r >= a.rows) return;
    float *values = a.values + r * a.row_stride;
    const unsigned int count = (unsigned int)a.count;
    const unsigned int group = a.block_width / 4u;
    const bool fp8 = a.quantization == 8u;
    const float limit = fp8 ? 448.0f : 6.0f;
    const float floor_amax = fp8 ? 1.0e-4f : __uint_as_float(0x01c00000u);  // 6 * 2^-126
    bool finite = true;
#pragma unroll 4
    for (unsigned int start = 0u; start < (HADAMARD ? 1u : count); start += 128u) {
        const unsigned int base = start + lane * 4u;
        const bool active = base < count;
        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (active) {
            const float4 x = *reinterpret_cast<const float4 *>(values + base);
            v[0] = x.x, v[1] = x.y, v[2] = x.z, v[3] = x.w;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) finite = finite && isfinite(v[k]);
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
            for (int k = 0; k < 4; ++k) v[k] = __fmul_rn(v[k], a.hadamard_scale);
        }
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        amax = fmaxf(amax, floor_amax);
        for (unsigned int m = 1u; m < group; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
        const uint32_t ratio = __float_as_uint(__fdiv_rn(amax, limit));
        uint32_t exponent = (ratio >> 23) + ((ratio & 0x007fffffu) ? 1u : 0u);
        exponent = exponent > 254u ? 254u : exponent;
        const float scale = __uint_as_float(exponent ? exponent << 23 : 0x00400000u);
        // 1 / scale is a power of two as well (2^-127 for the largest scale), so the division is a product
        const float inverse = __uint_as_float(exponent == 254u ? 0x00400000u : (254u - exponent) << 23);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float magnitude = fminf(fabsf(__fmul_rn(v[k], inverse)), limit);
            const float nearest = fp8 ? activation_nearest_fp8_cvt(magnitude) : activation_nearest_fp4(magnitude);
            v[k] = __bfloat162float(__float2bfloat16_rn(__fmul_rn(copysignf(nearest, v[k]), scale)));  // finite here
        }
        if (active) *reinterpret_cast<float4 *>(values + base) = make_float4(v[0], v[1], v[2], v[3]);
    }
    if (!finite) atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
}

}  // namespace yvx

extern "C" int yvx_cuda_activation_quant(const yvx_activation_args *a, void *stream)
{
    if (!a || !a->values || !a->status || !a->count || !a->block_width ||
        (a->quantization != 8u && a->quantization != 4u) || a->row_stride < a->count)
        return YVEX_ERR_INVALID_ARG;
    if (a->count % a->block_width) return YVEX_ERR_BOUNDS;
    if (a->count > 8192ull || a->block_width > 1024u || a->rows > 0x7fffffffull) return YVEX_ERR_UNSUPPORTED;
    if (!a->rows) return 0;
    // warp-per-row path: 16-byte rows, blocks of 4 << k lanes that tile a 128-lane segment; with the
    // transform the (padded) row must be exactly one segment
    const bool vector = !((unsigned long long)a->values & 15ull) && !(a->row_stride & 3ull) && !(a->count & 3ull) &&
                        a->block_width >= 4u && a->block_width <= 128u && !(a->block_width & (a->block_width - 1u));
    const unsigned int warp_grid = (unsigned int)((a->rows + 3ull) / 4ull);
    if (vector && !a->hadamard) {
        yvx::activation_quant_warp_kernel<false><<<warp_grid, yvx::kActivationThreads, 0, (cudaStream_t)stream>>>(*a);
        return yvx_cuda_check(cudaGetLastError(), "activation_quant_warp_kernel");
    }
    if (vector && a->count > 64ull && a->count <= 128ull) {
        yvx::activation_quant_warp_kernel<true><<<warp_grid, yvx::kActivationThreads, 0, (cudaStream_t)stream>>>(*a);
        return yvx_cuda_check(cudaGetLastError(), "activation_quant_warp_kernel");
    }
    unsigned int padded = 1u;
    while (padded < a->count) padded <<= 1;
    if (!a->hadamard) padded = (unsigned int)a->count;
    yvx::activation_quant_kernel<<<(unsigned int)a->rows, yvx::kActivationThreads, padded * sizeof(float),
                                   (cudaStream_t)stream>>>(*a, padded);
    return yvx_cuda_check(cudaGetLastError(), "activation_quant_kernel");
}
