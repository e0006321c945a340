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
#include "pipeline.cuh"

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

// The any-shape kernel (rows that are not 16-byte multiples, odd widths).
// grid: x = ceil(rows / kMatvecWarps), y = token tile, z = group.
// Group g takes weight rows [g * rows, (g + 1) * rows), input lanes [g * width, (g + 1) *
// width) of every token row and output lanes [g * rows, (g + 1) * rows).
__global__ void __launch_bounds__(kMatvecWarps * 32)
qtype_matvec_generic_kernel(const yvx_matvec_args a)
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


// ---- the streaming kernel ---------------------------------------------------------------
// Same sums, laid out for bandwidth. A CTA of 8 warps owns 8 * RW consecutive weight rows
// (a warp RW of them) and walks the row width in segments. Per segment the activation
// lanes of the token tile are converted to double ONCE into shared memory (skewed so that
// every access pattern below is conflict free) and every weight lane that follows costs
// one FP64 multiply-add per token plus its decode. Small CTAs (20 KB of activation lanes)
// keep many warps resident, which is what hides the FP64 and shared-memory latencies:
// persistent variants with one or two fat CTAs per SM measured 15-25 % slower.
//   Q8_0    row chunks of 32 blocks (1088 bytes) arrive by linear bulk copies into a
//           two-stage ring per warp; a lane owns one 34-byte block, reads it as the nine
//           words that hold it, and turns each signed byte into a double with one integer
//           XOR, one byte permute and one FP64 add (2^52 + u, minus 2^52 + 128 once per
//           block); the block's scale multiplies the block's sum once (the same value:
//           scale * lane is exact in single precision, and the sums are exact in double).
//   16-bit  16-byte loads of eight lanes per thread and row, sixteen in flight per thread;
//           sign, exponent and mantissa fields are placed by integer shifts into a double
//           whose exponent field still carries the narrow bias: a value 2^(narrow bias -
//           1023) times the weight, exact for zeros and subnormals too. The missing power
//           of two is put on the activations (BF16: all of it; F16, whose factor 2^1008
//           would overflow large activations: half there, half on the final sum). Powers of
//           two change no mantissa, so the sums are the same sums. An exponent field of all
//           ones (an infinite or NaN weight) raises the status word.
//   F32     one 4-byte load and one conversion per lane.
enum { kKindQ8 = 0, kKindHalf = 1, kKindF32 = 2 };
constexpr int kFastThreads = kMatvecWarps * 32;
constexpr int kQ8ChunkBlocks = 32, kQ8ChunkBytes = kQ8ChunkBlocks * 34, kQ8ChunkSlot = kQ8ChunkBytes + 16;

template <int TOKENS> struct FastShape {
    static constexpr int kSegment = TOKENS == 1 ? 2048 : 1024;   // activation lanes per segment
};
template <int KIND, int TOKENS> __host__ __device__ constexpr int fast_padded()
{
    constexpr int s = FastShape<TOKENS>::kSegment;
    return KIND == kKindQ8 ? s + s / 32 : KIND == kKindHalf ? s + s / 4 : s;
}
template <int KIND> __device__ __forceinline__ int fast_slot(int pos)
{
    return KIND == kKindQ8 ? pos + (pos >> 5) : KIND == kKindHalf ? pos + ((pos >> 3) << 1) : pos;
}
template <int KIND, int TOKENS, int RW> __host__ __device__ constexpr int fast_smem_bytes()
{
    return TOKENS * fast_padded<KIND, TOKENS>() * 8 +
           (KIND == kKindQ8 ? kMatvecWarps * 2 * RW * kQ8ChunkSlot + kMatvecWarps * 2 * 8 : 0);
}

template <int KIND, int TOKENS, int RW>
__global__ void __launch_bounds__(kFastThreads)
qtype_matvec_kernel(const yvx_matvec_args a)
{
    extern __shared__ __align__(16) unsigned char mv_smem[];
    constexpr int kSegment = FastShape<TOKENS>::kSegment, kPadded = fast_padded<KIND, TOKENS>();
    double *xd = reinterpret_cast<double *>(mv_smem);                 // [TOKENS][kPadded]
    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned long long group = blockIdx.z;
    const unsigned long long token0 = (unsigned long long)blockIdx.y * TOKENS;
    const unsigned int live = (unsigned int)min((unsigned long long)TOKENS, a.tokens - token0);
    const unsigned long long row0 = ((unsigned long long)blockIdx.x * kMatvecWarps + warp) * RW;
    const unsigned char *rows[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r)   // rows past the end alias the last one; their sums are never stored
        rows[r] = reinterpret_cast<const unsigned char *>(a.weights) +
                  (a.first_row + group * a.rows + min(row0 + r, a.rows - 1ull)) * a.row_bytes;
    const float *x[TOKENS];
#pragma unroll
    for (int t = 0; t < TOKENS; ++t)
        x[t] = a.input + (token0 + min((unsigned int)t, live - 1u)) * a.input_stride + group * a.width;
    double acc[RW][TOKENS];
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int t = 0; t < TOKENS; ++t) acc[r][t] = 0.0;

    // Q8_0: the warp's ring of row chunks
    unsigned char *ring = mv_smem + TOKENS * kPadded * 8 + warp * (2 * RW * kQ8ChunkSlot);
    uint64_t *bars = reinterpret_cast<uint64_t *>(mv_smem + TOKENS * kPadded * 8 + kMatvecWarps * 2 * RW * kQ8ChunkSlot) +
                     warp * 2;
    const unsigned long long blocks = a.width / 32ull;
    const unsigned int chunks = (unsigned int)((blocks + kQ8ChunkBlocks - 1) / kQ8ChunkBlocks);
    auto request = [&](unsigned int q) {   // lane 0: chunk q of the warp's rows into stage q & 1
        const unsigned int nb = (unsigned int)min((unsigned long long)kQ8ChunkBlocks, blocks - (unsigned long long)q * kQ8ChunkBlocks);
        const unsigned int bytes = nb * 34u;   // a multiple of 16: the launcher admits widths of whole 256 lanes
        fence_proxy_async();
        mbar_expect_tx(&bars[q & 1u], bytes * RW);
#pragma unroll
        for (int r = 0; r < RW; ++r)
            bulk_load(ring + ((q & 1u) * RW + r) * kQ8ChunkSlot, rows[r] + (unsigned long long)q * kQ8ChunkBytes, bytes,
                      &bars[q & 1u]);
    };
    if (KIND == kKindQ8) {
        if (lane == 0) {
            mbar_init(&bars[0], 1);
            mbar_init(&bars[1], 1);
            fence_barrier_init();
        }
        __syncwarp();
        if (lane == 0) {
            request(0);
            if (chunks > 1u) request(1);
        }
    }
    bool ok = true;
    unsigned int q = 0;   // Q8_0: next chunk to consume
    const bool is_bf16 = a.qtype == YVX_QTYPE_BF16;
    const double x_scale = KIND != kKindHalf ? 1.0 : is_bf16 ? 0x1p896 : 0x1p504;
    const double sum_scale = KIND == kKindHalf && !is_bf16 ? 0x1p504 : 1.0;
    uint32_t nonfinite = 0u;   // 16-bit weights: exponent fields of all ones seen

    for (unsigned long long seg0 = 0; seg0 < a.width; seg0 += kSegment) {
        const unsigned int seg_len = (unsigned int)min((unsigned long long)kSegment, a.width - seg0);
        __syncthreads();   // the previous segment's lanes have been read by every warp
        {
            // every load of the thread before its first conversion: one round trip, not one per lane
            constexpr int kPerThread = TOKENS * kSegment / kFastThreads;
            float staged[kPerThread];
#pragma unroll
            for (int k = 0; k < kPerThread; ++k) {
                const unsigned int i = threadIdx.x + (unsigned)k * kFastThreads, t = i / kSegment, pos = i % kSegment;
                staged[k] = pos < seg_len ? __ldg(x[t] + seg0 + pos) : 0.0f;
            }
#pragma unroll
            for (int k = 0; k < kPerThread; ++k) {
                const unsigned int i = threadIdx.x + (unsigned)k * kFastThreads, t = i / kSegment, pos = i % kSegment;
                if (pos < seg_len) xd[t * kPadded + fast_slot<KIND>((int)pos)] = (double)staged[k] * x_scale;
            }
        }
        __syncthreads();
        if (KIND == kKindQ8) {
            const unsigned int seg_chunks = (seg_len + 1023u) / 1024u;
            for (unsigned int c = 0; c < seg_chunks && ok; ++c, ++q) {
                if (!mbar_wait(&bars[q & 1u], (q >> 1) & 1u)) {
                    ok = false;
                    break;
                }
                const bool valid = (unsigned long long)q * kQ8ChunkBlocks + lane < blocks;
                // the lane's block: 34 bytes from 34 * lane, read as the nine words that hold them
                const unsigned int byte0 = 34u * lane, shift = (byte0 & 2u) * 8u;
                uint32_t data[RW][8];
                double scale[RW];
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    const uint32_t *words = reinterpret_cast<const uint32_t *>(
                        ring + ((q & 1u) * RW + r) * kQ8ChunkSlot + (byte0 & ~3u));
                    uint32_t w[9];
#pragma unroll
                    for (int j = 0; j < 9; ++j) w[j] = words[j];
                    const float d = __half2float(__ushort_as_half((unsigned short)((w[0] >> shift) & 0xffffu)));
                    // the reference's decode refuses a negative or non-finite block scale
                    if (valid && (!(d >= 0.0f) || isinf(d))) atomicCAS(a.status, 0, YVX_STATUS_CONTRACT);
                    scale[r] = (double)d;
#pragma unroll
                    for (int j = 0; j < 8; ++j)   // signed bytes -> biased unsigned bytes
                        data[r][j] = __funnelshift_rc(w[j], w[j + 1], 16u + shift) ^ 0x80808080u;
                }
                __syncwarp();   // every lane holds its blocks: the stage may be refilled
                if (lane == 0 && q + 2u < chunks) request(q + 2u);
                if (!valid) continue;
                const double *xs = xd + (c * kQ8ChunkBlocks + lane) * 33;
                double sum[RW][TOKENS], plain[TOKENS];
#pragma unroll
                for (int t = 0; t < TOKENS; ++t) {
                    plain[t] = 0.0;
#pragma unroll
                    for (int r = 0; r < RW; ++r) sum[r][t] = 0.0;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        double xv[TOKENS];
#pragma unroll
                        for (int t = 0; t < TOKENS; ++t) {
                            xv[t] = xs[t * kPadded + 4 * j + b];
                            plain[t] += xv[t];
                        }
#pragma unroll
                        for (int r = 0; r < RW; ++r) {
                            const double u = __hiloint2double(0x43300000, (int)__byte_perm(data[r][j], 0u, 0x4440u + b)) -
                                             4503599627370496.0;
#pragma unroll
                            for (int t = 0; t < TOKENS; ++t) sum[r][t] = fma(u, xv[t], sum[r][t]);
                        }
                    }
#pragma unroll
                for (int r = 0; r < RW; ++r)
#pragma unroll
                    for (int t = 0; t < TOKENS; ++t)
                        acc[r][t] = fma(scale[r], sum[r][t] - 128.0 * plain[t], acc[r][t]);
            }
        } else if (KIND == kKindHalf) {
            const unsigned int vectors = seg_len / 8u;
            // field placement: BF16 exponent+mantissa (15 bits) sit 3 bits lower in the double's
            // high word, F16's 6 bits lower; `field` keeps exactly those bits
            const uint32_t down = is_bf16 ? 3u : 6u, up = 16u - down;
            const uint32_t field = is_bf16 ? 0x0fffe000u : 0x01fffc00u;
            const uint32_t exponent = is_bf16 ? 0x7f807f80u : 0x7c007c00u, carry = is_bf16 ? 0x00800080u : 0x04000400u;
            // kDepth 16-byte loads per row in flight per lane before the first is used
            constexpr int kDepth = 16 / RW;
            for (unsigned int v0 = lane; v0 < vectors; v0 += 32u * kDepth) {
                uint4 held[kDepth][RW];
#pragma unroll
                for (int d = 0; d < kDepth; ++d)
#pragma unroll
                    for (int r = 0; r < RW; ++r)
                        held[d][r] = v0 + 32u * d < vectors
                                         ? __ldg(reinterpret_cast<const uint4 *>(rows[r] + seg0 * 2ull) + v0 + 32u * d)
                                         : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int d = 0; d < kDepth; ++d) {
                    const unsigned int v = v0 + 32u * d;
                    if (v >= vectors) break;
                    const double *xs = xd + 10u * v;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        double xv[TOKENS][2];
#pragma unroll
                        for (int t = 0; t < TOKENS; ++t) {
                            const double2 pair = *reinterpret_cast<const double2 *>(xs + t * kPadded + 2 * j);
                            xv[t][0] = pair.x;
                            xv[t][1] = pair.y;
                        }
#pragma unroll
                        for (int r = 0; r < RW; ++r) {
                            const uint32_t word = j == 0 ? held[d][r].x : j == 1 ? held[d][r].y : j == 2 ? held[d][r].z : held[d][r].w;
                            nonfinite |= ((word & exponent) + carry) & 0x80008000u;
                            const double w0 = __hiloint2double((int)(((word << up) & field) | ((word << 16) & 0x80000000u)), 0);
                            const double w1 = __hiloint2double((int)(((word >> down) & field) | (word & 0x80000000u)), 0);
#pragma unroll
                            for (int t = 0; t < TOKENS; ++t) acc[r][t] = fma(w1, xv[t][1], fma(w0, xv[t][0], acc[r][t]));
                        }
                    }
                }
            }
        } else {
#pragma unroll 4
            for (unsigned int pos = lane; pos < seg_len; pos += 32u) {
                double xv[TOKENS];
#pragma unroll
                for (int t = 0; t < TOKENS; ++t) xv[t] = xd[t * kPadded + pos];
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    const double w = (double)__ldg(reinterpret_cast<const float *>(rows[r]) + seg0 + pos);
#pragma unroll
                    for (int t = 0; t < TOKENS; ++t) acc[r][t] = fma(w, xv[t], acc[r][t]);
                }
            }
        }
    }
    if (!ok && lane == 0) atomicCAS(a.status, 0, YVX_STATUS_TIMEOUT);
    if (nonfinite) atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);   // an infinite or NaN weight
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int t = 0; t < TOKENS; ++t) {
#pragma unroll
            for (int offset = 16; offset; offset >>= 1) acc[r][t] += __shfl_xor_sync(0xffffffffu, acc[r][t], offset);
            acc[r][t] *= sum_scale;
        }
    if (lane == 0 && ok) {
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            if (row0 + r >= a.rows) break;
            for (unsigned int t = 0; t < live; ++t) {
                float value = (float)acc[r][t];
                if (!isfinite(value)) atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
                if (a.round_bf16) value = bf16_bits_to_float(bf16_bits_rne(value));
                if (!YVX_CHECKED_INDEX(token0 + t < a.tokens && group * a.rows + row0 + r < a.output_stride, a.status))
                    continue;
                a.output[(token0 + t) * a.output_stride + group * a.rows + row0 + r] = value;
            }
        }
    }
}

template <int KIND, int TOKENS, int RW>
static int fast_launch(const yvx_matvec_args &a, unsigned long long groups, cudaStream_t stream)
{
    constexpr int smem = fast_smem_bytes<KIND, TOKENS, RW>();
    static int configured_device = -1;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return YVEX_ERR_BACKEND;
    if (configured_device != device) {
        const cudaError_t error = cudaFuncSetAttribute(qtype_matvec_kernel<KIND, TOKENS, RW>,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (error != cudaSuccess) return yvx_cuda_check(error, "qtype_matvec_kernel attribute");
        configured_device = device;
    }
    const unsigned long long ctas = (a.rows + kMatvecWarps * RW - 1ull) / (kMatvecWarps * RW);
    const unsigned long long tiles = (a.tokens + TOKENS - 1ull) / TOKENS;
    if (ctas > 0x7fffffffull || tiles > 65535ull || groups > 65535ull) {
        yvx_cuda_set_error_text("the projection grid exceeds the launch limits");
        return YVEX_ERR_BOUNDS;
    }
    const dim3 grid((unsigned int)ctas, (unsigned int)tiles, (unsigned int)groups);
    qtype_matvec_kernel<KIND, TOKENS, RW><<<grid, kFastThreads, smem, stream>>>(a);
    return yvx_cuda_check(cudaGetLastError(), "qtype_matvec_kernel");
}

template <int KIND>
static int fast_dispatch(const yvx_matvec_args &a, unsigned long long groups, int sm_count, cudaStream_t stream)
{
    // rows per warp: as many as still leave two CTAs for every SM
    const unsigned long long per_cta_row = (unsigned long long)kMatvecWarps * 2ull * (unsigned long long)sm_count;
    const unsigned long long work = a.rows * groups;
    const int rw = work >= 4ull * per_cta_row ? 4 : work >= 2ull * per_cta_row ? 2 : 1;
    if (a.tokens == 1ull) {
        if (rw == 4) return fast_launch<KIND, 1, 4>(a, groups, stream);
        if (rw == 2) return fast_launch<KIND, 1, 2>(a, groups, stream);
        return fast_launch<KIND, 1, 1>(a, groups, stream);
    }
    if (rw == 4) return fast_launch<KIND, 4, 4>(a, groups, stream);
    if (rw == 2) return fast_launch<KIND, 4, 2>(a, groups, stream);
    return fast_launch<KIND, 4, 1>(a, groups, stream);
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
    // the streaming kernel wants rows that start on 16-byte boundaries
    static int sm_count = 0;
    if (!sm_count) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
            sm_count = 148;
    }
    const bool aligned = (reinterpret_cast<uintptr_t>(a.weights) & 15u) == 0u && (a.row_bytes & 15ull) == 0ull;
    if (aligned && a.qtype == YVX_QTYPE_Q8_0 && a.width % 256ull == 0ull)
        return fast_dispatch<kKindQ8>(a, groups, sm_count, (cudaStream_t)stream);
    if (aligned && (a.qtype == YVX_QTYPE_BF16 || a.qtype == YVX_QTYPE_F16) && a.width % 8ull == 0ull)
        return fast_dispatch<kKindHalf>(a, groups, sm_count, (cudaStream_t)stream);
    if (a.qtype == YVX_QTYPE_F32) return fast_dispatch<kKindF32>(a, groups, sm_count, (cudaStream_t)stream);
    const dim3 grid((unsigned int)ctas, (unsigned int)tiles, (unsigned int)groups);
    qtype_matvec_generic_kernel<<<grid, kMatvecWarps * 32, 0, (cudaStream_t)stream>>>(a);
    return yvx_cuda_check(cudaGetLastError(), "qtype_matvec_generic_kernel");
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
