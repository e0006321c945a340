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
#include "activation.cuh"

namespace yvx {

constexpr int kActivationThreads = 128;

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
        activation_segment<HADAMARD>(v, lane, group, fp8, a.hadamard_scale);
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
