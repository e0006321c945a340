// Device-side seeded fills for the benchmark workloads: the full-size KV pools
// are several GB, so they are generated where they live. Counter-based
// (splitmix64 of seed and element index), hence independent of launch shape.
#include "common.cuh"

namespace yvx {

__device__ __forceinline__ uint64_t splitmix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// Box-Muller on two 32-bit uniforms drawn from one 64-bit hash; each thread
// produces the pair (2i, 2i+1).
__global__ void fill_normal_kernel(void *dst, int dtype, unsigned long long count,
                                   unsigned long long seed, float sigma)
{
    const unsigned long long pair =
        (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = pair; i * 2ull < count; i += stride) {
        const uint64_t h = splitmix64(seed * 0xD1342543DE82EF95ull + i);
        const float u1 = ((float)(uint32_t)(h >> 32) + 1.0f) * (1.0f / 4294967296.0f);
        const float u2 = (float)(uint32_t)h * (1.0f / 4294967296.0f);
        const float radius = sqrtf(-2.0f * logf(u1)) * sigma;
        float s, c;
        sincospif(2.0f * u2, &s, &c);
        const float a = radius * c, b = radius * s;
        if (dtype == YVEX_DTYPE_BF16) {
            unsigned short *out = reinterpret_cast<unsigned short *>(dst);
            out[2 * i] = bf16_bits_rne(a);
            if (2 * i + 1 < count) out[2 * i + 1] = bf16_bits_rne(b);
        } else if (dtype == -YVEX_DTYPE_F32) {
            // F32 storage of values that bf16 holds exactly (what the reference's linears publish)
            float *out = reinterpret_cast<float *>(dst);
            out[2 * i] = __uint_as_float((uint32_t)bf16_bits_rne(a) << 16);
            if (2 * i + 1 < count) out[2 * i + 1] = __uint_as_float((uint32_t)bf16_bits_rne(b) << 16);
        } else {
            float *out = reinterpret_cast<float *>(dst);
            out[2 * i] = a;
            if (2 * i + 1 < count) out[2 * i + 1] = b;
        }
    }
}

// int8 lanes uniform in [-127, 127].
__global__ void fill_lanes_kernel(signed char *dst, unsigned long long count,
                                  unsigned long long seed)
{
    const unsigned long long start =
        ((unsigned long long)blockIdx.x * blockDim.x + threadIdx.x) * 8ull;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x * 8ull;
    for (unsigned long long i = start; i < count; i += stride) {
        uint64_t h = splitmix64(seed * 0xD1342543DE82EF95ull + i);
        for (int j = 0; j < 8 && i + j < count; ++j) {
            // 255 values from one byte-sized draw; 0xFF re-hashes to stay uniform.
            uint32_t byte = (uint32_t)(h >> (8 * j)) & 0xffu;
            uint64_t again = h;
            while (byte == 255u) {
                again = splitmix64(again + j + 1);
                byte = (uint32_t)again & 0xffu;
            }
            dst[i + j] = (signed char)((int)byte - 127);
        }
    }
}

// f16 scales uniform in [lo, hi).
__global__ void fill_scales_kernel(__half *dst, unsigned long long count,
                                   unsigned long long seed, float lo, float hi)
{
    const unsigned long long start = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = start; i < count; i += stride) {
        const uint64_t h = splitmix64(seed * 0xD1342543DE82EF95ull + i);
        const float u = (float)(uint32_t)(h >> 32) * (1.0f / 4294967296.0f);
        dst[i] = __float2half_rn(lo + (hi - lo) * u);
    }
}

}  // namespace yvx

extern "C" {

int yvx_cuda_fill_normal(void *dst, int dtype, unsigned long long count,
                         unsigned long long seed, float sigma, void *stream)
{
    if (!dst || !count || (dtype != YVEX_DTYPE_F32 && dtype != YVEX_DTYPE_BF16 && dtype != -YVEX_DTYPE_F32))
        return YVEX_ERR_INVALID_ARG;
    yvx::fill_normal_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>(dst, dtype, count, seed, sigma);
    return yvx_cuda_check(cudaGetLastError(), "fill_normal_kernel");
}

int yvx_cuda_fill_q8_lanes(void *dst, unsigned long long count, unsigned long long seed,
                           void *stream)
{
    if (!dst || !count) return YVEX_ERR_INVALID_ARG;
    yvx::fill_lanes_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>((signed char *)dst, count, seed);
    return yvx_cuda_check(cudaGetLastError(), "fill_lanes_kernel");
}

int yvx_cuda_fill_f16_uniform(void *dst, unsigned long long count, unsigned long long seed,
                              float lo, float hi, void *stream)
{
    if (!dst || !count) return YVEX_ERR_INVALID_ARG;
    yvx::fill_scales_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>((__half *)dst, count, seed, lo, hi);
    return yvx_cuda_check(cudaGetLastError(), "fill_scales_kernel");
}

}  // extern "C"

namespace yvx {

// Q8 records: lanes uniform in [-127,127] (stored as lane + 128) in the lane regions and f16
// scales uniform in [lo, hi) in the scale regions of every 17408-byte record.
__global__ void fill_q8_records_kernel(unsigned char *records, unsigned long long record_count,
                                       unsigned long long seed, float lo, float hi)
{
    const unsigned long long words_per_record = 17408ull / 4ull;
    const unsigned long long total = record_count * words_per_record;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += stride) {
        const unsigned long long within = (i % words_per_record) * 4ull;
        uint64_t h = splitmix64(seed * 0xD1342543DE82EF95ull + i);
        uint32_t word;
        if (within < 16384ull) {
            word = 0u;
            for (int j = 0; j < 4; ++j) {
                uint32_t byte = (uint32_t)(h >> (8 * j)) & 0xffu;
                uint64_t again = h;
                while (byte == 255u) {
                    again = splitmix64(again + j + 1);
                    byte = (uint32_t)again & 0xffu;
                }
                word |= ((byte + 1u) & 0xffu) << (8 * j);  // (byte - 127) + 128
            }
        } else {
            const float u0 = (float)(uint32_t)(h >> 32) * (1.0f / 4294967296.0f);
            const float u1 = (float)(uint32_t)h * (1.0f / 4294967296.0f);
            word = (uint32_t)__half_as_ushort(__float2half_rn(lo + (hi - lo) * u0)) |
                   ((uint32_t)__half_as_ushort(__float2half_rn(lo + (hi - lo) * u1)) << 16);
        }
        reinterpret_cast<uint32_t *>(records)[i] = word;
    }
}

}  // namespace yvx

extern "C" int yvx_cuda_fill_q8_records(void *records, unsigned long long record_count,
                                        unsigned long long seed, float lo, float hi, void *stream)
{
    if (!records || !record_count) return YVEX_ERR_INVALID_ARG;
    yvx::fill_q8_records_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>(
        (unsigned char *)records, record_count, seed, lo, hi);
    return yvx_cuda_check(cudaGetLastError(), "fill_q8_records_kernel");
}

namespace yvx {

__device__ __forceinline__ float normal_element(unsigned long long seed, unsigned long long e, float sigma)
{
    const uint64_t h = splitmix64(seed * 0xD1342543DE82EF95ull + (e >> 1));
    const float u1 = ((float)(uint32_t)(h >> 32) + 1.0f) * (1.0f / 4294967296.0f);
    const float u2 = (float)(uint32_t)h * (1.0f / 4294967296.0f);
    const float radius = sqrtf(-2.0f * logf(u1)) * sigma;
    float s, c;
    sincospif(2.0f * u2, &s, &c);
    return (e & 1ull) ? radius * s : radius * c;
}

// The values fill_normal_kernel would write as F32, rotated before the bf16 rounding:
// rotate-half over the full head width, pairs (lane, lane + dim/2), frequency
// theta^(-2*pair/dim), cosine and sine tables rounded to bf16 (the convention of the
// reference's rotary tables, src/runtime/decoder.c:1080-1094). Rows are
// [session][token][head][dim]; the position of a row is its token index.
__global__ void fill_normal_rope_kernel(unsigned short *dst, unsigned long long rows,
                                        unsigned int tokens, unsigned int heads, unsigned int dim,
                                        unsigned long long seed, float sigma, double theta)
{
    const unsigned int half = dim / 2u;
    const unsigned long long pairs = rows * heads * half;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < pairs;
         i += stride) {
        const unsigned int pair = (unsigned int)(i % half);
        const unsigned long long vector = i / half;           // row * heads + head
        const unsigned long long row = vector / heads;
        const unsigned int position = (unsigned int)(row % tokens);
        const unsigned long long lo_index = vector * dim + pair, hi_index = lo_index + half;
        const float lo = normal_element(seed, lo_index, sigma), hi = normal_element(seed, hi_index, sigma);
        const double angle = (double)position * pow(theta, -2.0 * (double)pair / (double)dim);
        const float c = __uint_as_float((uint32_t)bf16_bits_rne((float)cos(angle)) << 16);
        const float sn = __uint_as_float((uint32_t)bf16_bits_rne((float)sin(angle)) << 16);
        dst[lo_index] = bf16_bits_rne(__fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, sn)));
        dst[hi_index] = bf16_bits_rne(__fadd_rn(__fmul_rn(hi, c), __fmul_rn(lo, sn)));
    }
}

}  // namespace yvx

extern "C" int yvx_cuda_fill_normal_rope_bf16(void *dst, unsigned long long rows, unsigned int tokens,
                                              unsigned int heads, unsigned int dim,
                                              unsigned long long seed, float sigma, double theta,
                                              void *stream)
{
    if (!dst || !rows || !tokens || !heads || !dim || (dim & 1u) || !(theta > 1.0))
        return YVEX_ERR_INVALID_ARG;
    yvx::fill_normal_rope_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>(
        (unsigned short *)dst, rows, tokens, heads, dim, seed, sigma, theta);
    return yvx_cuda_check(cudaGetLastError(), "fill_normal_rope_kernel");
}
