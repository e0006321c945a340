// Projections of the encoded (latent) attention operator: encoded weight rows times
// activation rows, and the decode of encoded rows to F32.
//
// Replaces, for the weight encodings admitted here (F32, F16, BF16, Q8_0), the
// reference's yvex_qtype_matvec / yvex_qtype_split_matvec / yvex_qtype_grouped_rows
// (src/backend/cuda/kernels.cu:436-866) and yvex_encoded_row_decode, as the stages of
// src/backend/cuda/attention.c:1162-1236 and :1424-1451 use them (q_a, q_b, kv, the
// compressor and indexer projections, grouped out_a, out_b, the norm weights, sinks and
// position biases). CPU twin: yvex_attention_dot_batch over yvex_quant_cpu_dot
// (src/graph/core.c:1107-1215, src/gguf/quant_compute.c:116-181): every lane decoded to
// float, products and the running sum in double, the sum narrowed to float.
//
// The work is bandwidth-shaped for decode-sized token counts: every weight byte is read
// once per tile of kMatvecTokens token rows. One warp owns one weight row; lanes stride
// over the row with 16-byte loads and keep one double accumulator per token of the tile.
// A product of two floats is exact in double, and for the value ranges of this operator
// (bf16-published activations, 8- to 24-bit weights) the partial sums stay exact as well,
// so the result does not depend on the order of the additions and equals the CPU twin's
// sequential sum bit for bit; where a sum is not exact the two differ by one rounding of
// a double, far below the bf16 publication that follows.
#include "common.cuh"

#include <cuda_fp16.h>

namespace yvx {

constexpr int kMatvecWarps = 8;
constexpr int kMatvecTokens = 4;

__device__ __forceinline__ float bf16_bits_to_float(unsigned short bits)
{
    return __uint_as_float((uint32_t)bits << 16);
}

// One weight lane against the same lane of every token row of the tile. Rows beyond the
// live ones alias the last live row (their sums are never stored), so no lane is guarded.
template <int TOKENS>
__device__ __forceinline__ void accumulate(double (&acc)[TOKENS], float w, const float *const (&x)[TOKENS],
                                           unsigned long long lane_index)
{
#pragma unroll
    for (int t = 0; t < TOKENS; ++t) acc[t] = fma((double)w, (double)__ldg(x[t] + lane_index), acc[t]);
}

// grid: x = ceil(rows / kMatvecWarps), y = token tile, z = group.
// Group g takes weight rows [g * rows, (g + 1) * rows), input lanes [g * width, (g + 1) *
// width) of every token row and output lanes [g * rows, (g + 1) * rows).
__global__ void __launch_bounds__(kMatvecWarps * 32)
qtype_matvec_kernel(const yvx_matvec_args a)
{
    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned long long row = (unsigned long long)blockIdx.x * kMatvecWarps + warp;
    if (row >= a.rows) return;
    const unsigned long long group = blockIdx.z;
    const unsigned long long token0 = (unsigned long long)blockIdx.y * kMatvecTokens;
    const unsigned int live = (unsigned int)min((unsigned long long)kMatvecTokens, a.tokens - token0);
    const unsigned char *encoded = reinterpret_cast<const unsigned char *>(a.weights) +
                                   (a.first_row + group * a.rows + row) * a.row_bytes;
    const float *x[kMatvecTokens];
    double acc[kMatvecTokens];
#pragma unroll
    for (int t = 0; t < kMatvecTokens; ++t) {
        x[t] = a.input + (token0 + min((unsigned int)t, live - 1u)) * a.input_stride + group * a.width;
        acc[t] = 0.0;
    }

    if (a.qtype == YVX_QTYPE_Q8_0) {
        // 34-byte blocks: f16 scale, 32 int8 lanes; a lane of the warp takes a block at a time
        const unsigned long long blocks = a.width / 32ull;
        for (unsigned long long b = lane; b < blocks; b += 32ull) {
            const unsigned short *block = reinterpret_cast<const unsigned short *>(encoded + b * 34ull);
            const float d = __half2float(__ushort_as_half(block[0]));
            // the reference's decode refuses a negative or non-finite block scale
            if (!(d >= 0.0f) || isinf(d)) atomicCAS(a.status, 0, YVX_STATUS_CONTRACT);
#pragma unroll 4
            for (int j = 0; j < 16; ++j) {
                const unsigned short two = block[1 + j];
                const float w0 = d * (float)(signed char)(two & 0xffu);
                const float w1 = d * (float)(signed char)(two >> 8);
                accumulate(acc, w0, x, b * 32ull + 2ull * j);
                accumulate(acc, w1, x, b * 32ull + 2ull * j + 1ull);
            }
        }
    } else if (a.qtype == YVX_QTYPE_F32) {
        const float *w = reinterpret_cast<const float *>(encoded);
        for (unsigned long long i = lane; i < a.width; i += 32ull) accumulate(acc, __ldg(w + i), x, i);
    } else {
        // 16-bit encodings: eight lanes per 16-byte load when the row allows it
        const bool is_bf16 = a.qtype == YVX_QTYPE_BF16;
        const bool vector = (a.row_bytes & 15ull) == 0ull && (reinterpret_cast<uintptr_t>(a.weights) & 15u) == 0u &&
                            (a.width & 7ull) == 0ull;
        if (vector) {
            const uint4 *w = reinterpret_cast<const uint4 *>(encoded);
            for (unsigned long long i = lane; i < a.width / 8ull; i += 32ull) {
                const uint4 packed = __ldg(w + i);
                const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const unsigned short lo = (unsigned short)(words[j] & 0xffffu), hi = (unsigned short)(words[j] >> 16);
                    const float w0 = is_bf16 ? bf16_bits_to_float(lo) : __half2float(__ushort_as_half(lo));
                    const float w1 = is_bf16 ? bf16_bits_to_float(hi) : __half2float(__ushort_as_half(hi));
                    accumulate(acc, w0, x, i * 8ull + 2ull * j);
                    accumulate(acc, w1, x, i * 8ull + 2ull * j + 1ull);
                }
            }
        } else {
            const unsigned short *w = reinterpret_cast<const unsigned short *>(encoded);
            for (unsigned long long i = lane; i < a.width; i += 32ull) {
                const unsigned short bits = w[i];
                accumulate(acc, is_bf16 ? bf16_bits_to_float(bits) : __half2float(__ushort_as_half(bits)), x, i);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < kMatvecTokens; ++t)
#pragma unroll
        for (int offset = 16; offset; offset >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], offset);
    if (lane == 0) {
        for (unsigned int t = 0; t < live; ++t) {
            float value = (float)acc[t];
            if (!isfinite(value)) atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
            if (a.round_bf16) value = bf16_bits_to_float(bf16_bits_rne(value));
            if (!YVX_CHECKED_INDEX(token0 + t < a.tokens && group * a.rows + row < a.output_stride, a.status)) continue;
            a.output[(token0 + t) * a.output_stride + group * a.rows + row] = value;
        }
    }
}

// Encoded rows [first_row, first_row + rows) decoded to F32 [rows][width].
__global__ void qtype_decode_rows_kernel(const void *weights, unsigned int qtype, unsigned long long first_row,
                                         unsigned long long rows, unsigned long long width,
                                         unsigned long long row_bytes, float *out, int *status)
{
    const unsigned long long total = rows * width;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const unsigned long long row = i / width, lane = i % width;
        const unsigned char *encoded = reinterpret_cast<const unsigned char *>(weights) + (first_row + row) * row_bytes;
        float value;
        if (qtype == YVX_QTYPE_F32) {
            value = reinterpret_cast<const float *>(encoded)[lane];
        } else if (qtype == YVX_QTYPE_BF16) {
            value = bf16_bits_to_float(reinterpret_cast<const unsigned short *>(encoded)[lane]);
        } else if (qtype == YVX_QTYPE_F16) {
            value = __half2float(__ushort_as_half(reinterpret_cast<const unsigned short *>(encoded)[lane]));
        } else {
            const unsigned char *block = encoded + (lane / 32ull) * 34ull;
            const float d = __half2float(__ushort_as_half((unsigned short)(block[0] | (block[1] << 8))));
            if (!(d >= 0.0f) || isinf(d)) atomicCAS(status, 0, YVX_STATUS_CONTRACT);
            value = d * (float)(signed char)block[2 + lane % 32ull];
        }
        if (!isfinite(value)) atomicCAS(status, 0, YVX_STATUS_NONFINITE);
        out[i] = value;
    }
}

// In-place bf16 publication (round to nearest even) of F32 rows: values[row][0 .. width).
__global__ void round_bf16_rows_kernel(float *values, unsigned long long rows, unsigned long long width,
                                       unsigned long long row_stride, int *status)
{
    const unsigned long long total = rows * width;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        float *p = values + (i / width) * row_stride + i % width;
        const float value = *p;
        if (!isfinite(value)) atomicCAS(status, 0, YVX_STATUS_NONFINITE);
        *p = bf16_bits_to_float(bf16_bits_rne(value));
    }
}

static bool qtype_admitted(unsigned int qtype)
{
    return qtype == YVX_QTYPE_F32 || qtype == YVX_QTYPE_F16 || qtype == YVX_QTYPE_BF16 || qtype == YVX_QTYPE_Q8_0;
}

}  // namespace yvx

extern "C" {

unsigned long long yvx_cuda_qtype_row_bytes(unsigned int qtype, unsigned long long width)
{
    switch (qtype) {
    case YVX_QTYPE_F32: return width * 4ull;
    case YVX_QTYPE_F16:
    case YVX_QTYPE_BF16: return width * 2ull;
    case YVX_QTYPE_Q8_0: return width % 32ull ? 0ull : width / 32ull * 34ull;
    default: return 0ull;
    }
}

int yvx_cuda_qtype_matvec(const yvx_matvec_args *args, void *stream)
{
    using namespace yvx;
    if (!args || !args->weights || !args->input || !args->output || !args->status || !args->rows ||
        !args->width || !args->tokens || args->input_stride < args->width)
        return YVEX_ERR_INVALID_ARG;
    if (!qtype_admitted(args->qtype)) return YVEX_ERR_UNSUPPORTED;
    const unsigned long long groups = args->groups ? args->groups : 1ull;
    if (args->row_bytes != yvx_cuda_qtype_row_bytes(args->qtype, args->width) ||
        args->output_stride < groups * args->rows || args->input_stride < groups * args->width ||
        (args->qtype == YVX_QTYPE_Q8_0 && (reinterpret_cast<uintptr_t>(args->weights) & 1u)))
        return YVEX_ERR_BOUNDS;
    const unsigned long long ctas = (args->rows + kMatvecWarps - 1) / kMatvecWarps;
    const unsigned long long tiles = (args->tokens + kMatvecTokens - 1) / kMatvecTokens;
    if (ctas > 0x7fffffffull || tiles > 65535ull || groups > 65535ull) {
        yvx_cuda_set_error_text("the projection grid exceeds the launch limits");
        return YVEX_ERR_BOUNDS;
    }
    yvx_matvec_args a = *args;
    a.groups = groups;
    const dim3 grid((unsigned int)ctas, (unsigned int)tiles, (unsigned int)groups);
    qtype_matvec_kernel<<<grid, kMatvecWarps * 32, 0, (cudaStream_t)stream>>>(a);
    return yvx_cuda_check(cudaGetLastError(), "qtype_matvec_kernel");
}

int yvx_cuda_qtype_decode_rows(const void *weights, unsigned int qtype, unsigned long long first_row,
                               unsigned long long rows, unsigned long long width, float *out, int *status,
                               void *stream)
{
    using namespace yvx;
    if (!weights || !out || !status || !rows || !width) return YVEX_ERR_INVALID_ARG;
    if (!qtype_admitted(qtype)) return YVEX_ERR_UNSUPPORTED;
    const unsigned long long row_bytes = yvx_cuda_qtype_row_bytes(qtype, width);
    if (!row_bytes) return YVEX_ERR_BOUNDS;
    const unsigned long long total = rows * width;
    const unsigned int blocks = (unsigned int)min((total + 255ull) / 256ull, 148ull * 8ull);
    qtype_decode_rows_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(weights, qtype, first_row, rows, width,
                                                                      row_bytes, out, status);
    return yvx_cuda_check(cudaGetLastError(), "qtype_decode_rows_kernel");
}

int yvx_cuda_round_bf16_rows(float *values, unsigned long long rows, unsigned long long width,
                             unsigned long long row_stride, int *status, void *stream)
{
    using namespace yvx;
    if (!values || !status || !rows || !width || row_stride < width) return YVEX_ERR_INVALID_ARG;
    const unsigned long long total = rows * width;
    const unsigned int blocks = (unsigned int)min((total + 255ull) / 256ull, 148ull * 16ull);
    round_bf16_rows_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(values, rows, width, row_stride, status);
    return yvx_cuda_check(cudaGetLastError(), "round_bf16_rows_kernel");
}

}  // extern "C"
