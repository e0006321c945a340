// Rolling compressor over a chunk of tokens in one launch.
//
// Replaces yvex_attention_rolling_state (src/backend/cuda/kernels.cu:1536-1631 in
// the reference: one launch of ONE CTA per token, the whole state copied on every
// token) and its CPU twin yvex_attention_rolling_state_step_cpu
// (src/graph/attention.c:745-836). The transition is a ring insert, and an emission
// only reads the rows of its own group (and, with two halves, of the group before
// it), so every emission of a chunk is independent given the token rows and the state
// the chunk started from: CTA g computes emitted row g, the last state_slots CTAs
// write the state the serial process would end in. With norm_weights the CTA carries
// on through the publication chain of src/graph/attention_execute.c:776-806
// (bf16 round, RMS norm, bf16 round, rotation, bf16 round) while the row is still in
// registers. Per lane the softmax runs in double in the reference's order (previous
// half before current half, slot by slot), products and sums separately rounded.
#include "activation.cuh"

namespace yvx {

constexpr int kCompressorThreads = 256;
constexpr int kCompressorLanesPerThread = 4;  // head_dim <= 1024

struct compressor_row {
    const float *kv, *score, *ape;  // ape == nullptr: the score is stored with it already
};

// Row `token` (signed: negative means "before this chunk") of the chunk, else the
// given slot of the state the chunk started from.
__device__ __forceinline__ compressor_row compressor_source(const yvx_compressor_args &a,
                                                            long long token, unsigned long long cursor,
                                                            unsigned long long state_slot,
                                                            unsigned long long width)
{
    compressor_row r;
    if (token >= 0) {
        r.kv = a.token_kv + (unsigned long long)token * a.token_stride;
        r.score = a.token_score + (unsigned long long)token * a.token_stride;
        r.ape = a.ape + cursor * width;
    } else {
        r.kv = a.state_kv + state_slot * width;
        r.score = a.state_score + state_slot * width;
        r.ape = nullptr;
    }
    return r;
}

__device__ __forceinline__ float compressor_score(const compressor_row &r, unsigned long long column,
                                                  bool &finite)
{
    if (!r.ape) return r.score[column];
    const float token_score = r.score[column], ape = r.ape[column];
    finite = finite && isfinite(token_score) && isfinite(ape);
    return __fadd_rn(token_score, ape);
}

// float -> double is exact; for normal numbers it is a re-bias of the exponent and a shift
// of the mantissa, done on the integer pipe (the conversion instruction shares a narrow
// pipe with the other double-precision conversions). Zeros, subnormals, infinities and
// NaNs take the conversion instruction.
__device__ __forceinline__ double compressor_widen(float f)
{
    const uint32_t bits = __float_as_uint(f);
    if (((bits >> 23) & 0xffu) - 1u < 254u)
        return __hiloint2double((int)((bits & 0x80000000u) | (((bits & 0x7fffffffu) >> 3) + 0x38000000u)),
                                (int)(bits << 29));
    return (double)f;
}

__device__ __forceinline__ float compressor_bf16(float v)
{
    return __uint_as_float((uint32_t)bf16_bits_rne(v) << 16);
}

// The state after the last token, one slot per CTA: the row the serial process wrote
// to that slot last (a token of this chunk, else what the slot held before).
__device__ __forceinline__ void compressor_state_slot(const yvx_compressor_args &a, unsigned long long emitted,
                                                      unsigned long long slot, unsigned long long c0)
{
    const unsigned long long ratio = a.ratio;
    const unsigned long long width = a.overlap ? 2ull * a.head_dim : a.head_dim;
    const unsigned int tid = threadIdx.x;
    bool finite = true;
    const long long tokens = (long long)a.token_count;
    long long token;
    unsigned long long cursor, before_slot = slot;
    if (a.overlap && slot < ratio) {
        cursor = slot;
        if (!emitted) {
            token = -1;
        } else {
            const long long last = (long long)(ratio - c0 - 1ull + (emitted - 1ull) * ratio);
            token = last - (long long)(ratio - 1ull - cursor);
            before_slot = ratio + cursor;
        }
    } else {
        cursor = a.overlap ? slot - ratio : slot;
        const unsigned long long last_cursor = (c0 + a.token_count + ratio - 1ull) % ratio;
        token = tokens - 1 - (long long)((last_cursor + ratio - cursor) % ratio);
        if (!tokens) token = -1;
    }
    const compressor_row r = compressor_source(a, token, cursor, before_slot, width);
    for (unsigned long long column = tid; column < width; column += blockDim.x) {
        const float kv = r.kv[column];
        const float score = compressor_score(r, column, finite);
        if (r.ape) finite = finite && isfinite(kv);
        a.after_kv[slot * width + column] = kv;
        a.after_score[slot * width + column] = score;
    }
    if (!finite) atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
}

__global__ void __launch_bounds__(kCompressorThreads)
compressor_chunk_kernel(const yvx_compressor_args a, unsigned long long emitted)
{
    const unsigned long long ratio = a.ratio, hd = a.head_dim;
    const unsigned long long width = a.overlap ? 2ull * hd : hd;
    const unsigned long long c0 = a.start_position % ratio;
    const unsigned int tid = threadIdx.x;
    __shared__ double warp_part[kCompressorThreads / 32];
    bool finite = true;

    if (blockIdx.x >= emitted) {
        compressor_state_slot(a, emitted, blockIdx.x - emitted, c0);
        return;
    }

    // ---- emitted row g ----
    const unsigned long long g = blockIdx.x;
    const long long first_current = (long long)(g * ratio) - (long long)c0;
    const long long first_previous = first_current - (long long)ratio;
    // All lanes of a thread walk the slots together, so a row is resolved once per slot.
    // Pass 1 compares floats (widening is monotone, so the maximum is the same value).
    float value[kCompressorLanesPerThread], top[kCompressorLanesPerThread];
    double denominator[kCompressorLanesPerThread], sum[kCompressorLanesPerThread];
    const unsigned long long current_column = a.overlap ? hd : 0ull;
#pragma unroll
    for (int k = 0; k < kCompressorLanesPerThread; ++k) {
        top[k] = -INFINITY;
        denominator[k] = sum[k] = 0.0;
    }
    for (unsigned long long s = 0; s < ratio; ++s) {
        if (a.overlap) {
            const compressor_row p = compressor_source(a, first_previous + (long long)s, s,
                                                       g == 0ull ? s : ratio + s, width);
#pragma unroll
            for (int k = 0; k < kCompressorLanesPerThread; ++k) {
                const unsigned long long lane = tid + (unsigned long long)k * kCompressorThreads;
                if (lane < hd) top[k] = fmaxf(top[k], compressor_score(p, lane, finite));
            }
        }
        const compressor_row c = compressor_source(a, first_current + (long long)s, s,
                                                   a.overlap ? ratio + s : s, width);
#pragma unroll
        for (int k = 0; k < kCompressorLanesPerThread; ++k) {
            const unsigned long long lane = tid + (unsigned long long)k * kCompressorThreads;
            if (lane < hd) top[k] = fmaxf(top[k], compressor_score(c, lane + current_column, finite));
        }
    }
    for (unsigned long long s = 0; s < ratio; ++s) {
        if (a.overlap) {
            const compressor_row p = compressor_source(a, first_previous + (long long)s, s,
                                                       g == 0ull ? s : ratio + s, width);
#pragma unroll
            for (int k = 0; k < kCompressorLanesPerThread; ++k) {
                const unsigned long long lane = tid + (unsigned long long)k * kCompressorThreads;
                if (lane >= hd) continue;
                const double w = exp(__dsub_rn(compressor_widen(compressor_score(p, lane, finite)),
                                               compressor_widen(top[k])));
                const float kv = p.kv[lane];
                if (p.ape) finite = finite && isfinite(kv);
                denominator[k] = __dadd_rn(denominator[k], w);
                sum[k] = __dadd_rn(sum[k], __dmul_rn(w, compressor_widen(kv)));
            }
        }
        const compressor_row c = compressor_source(a, first_current + (long long)s, s,
                                                   a.overlap ? ratio + s : s, width);
#pragma unroll
        for (int k = 0; k < kCompressorLanesPerThread; ++k) {
            const unsigned long long lane = tid + (unsigned long long)k * kCompressorThreads;
            if (lane >= hd) continue;
            const double w = exp(__dsub_rn(compressor_widen(compressor_score(c, lane + current_column, finite)),
                                           compressor_widen(top[k])));
            const float kv = c.kv[lane + current_column];
            if (c.ape) finite = finite && isfinite(kv);
            denominator[k] = __dadd_rn(denominator[k], w);
            sum[k] = __dadd_rn(sum[k], __dmul_rn(w, compressor_widen(kv)));
        }
    }
#pragma unroll
    for (int k = 0; k < kCompressorLanesPerThread; ++k) {
        const unsigned long long lane = tid + (unsigned long long)k * kCompressorThreads;
        value[k] = 0.0f;
        if (lane >= hd) continue;
        finite = finite && isfinite(denominator[k]) && denominator[k] > 0.0 && isfinite(sum[k]);
        value[k] = __double2float_rn(__ddiv_rn(sum[k], denominator[k]));
        finite = finite && isfinite(value[k]);
    }

    if (a.norm_weights) {
        double squares = 0.0;
#pragma unroll
        for (int k = 0; k < kCompressorLanesPerThread; ++k) {
            value[k] = compressor_bf16(value[k]);
            squares = __dadd_rn(squares, __dmul_rn((double)value[k], (double)value[k]));
        }
#pragma unroll
        for (int offset = 16; offset; offset >>= 1)
            squares = __dadd_rn(squares, __shfl_xor_sync(0xffffffffu, squares, offset));
        if ((tid & 31u) == 0u) warp_part[tid >> 5] = squares;
        __syncthreads();
        double mean = 0.0;
#pragma unroll
        for (int w = 0; w < kCompressorThreads / 32; ++w) mean = __dadd_rn(mean, warp_part[w]);
        mean = __ddiv_rn(mean, (double)hd);
        const double inverse = __ddiv_rn(1.0, sqrt(__dadd_rn(mean, a.epsilon)));
        finite = finite && isfinite(inverse);
        const unsigned long long rope_start = a.rope_dims ? hd - a.rope_dims : hd;
        const unsigned long long position = a.start_position + (unsigned long long)first_current;
#pragma unroll
        for (int k = 0; k < kCompressorLanesPerThread; ++k) {
            const unsigned long long lane = tid + (unsigned long long)k * kCompressorThreads;
            const float weight = lane < hd ? a.norm_weights[lane] : 0.0f;
            const double scaled = __dmul_rn(__dmul_rn((double)value[k], inverse), (double)weight);
            float v = __double2float_rn(scaled);
            finite = finite && isfinite(weight) && isfinite(v);
            v = compressor_bf16(v);
            const float partner = __shfl_xor_sync(0xffffffffu, v, 1);
            if (lane >= rope_start && lane < hd) {
                const unsigned long long i = lane - rope_start;
                const double angle = __dmul_rn((double)position, a.rope_frequency[i >> 1]);
                double sn, c;
                sincos(angle, &sn, &c);
                const double x = (i & 1ull) ? (double)partner : (double)v;
                const double y = (i & 1ull) ? (double)v : (double)partner;
                const double rotated = (i & 1ull) ? __dadd_rn(__dmul_rn(x, sn), __dmul_rn(y, c))
                                                  : __dsub_rn(__dmul_rn(x, c), __dmul_rn(y, sn));
                v = __double2float_rn(rotated);
                finite = finite && isfinite(c) && isfinite(sn) && isfinite(v);
            }
            if (a.rope_dims) v = compressor_bf16(v);
            value[k] = v;
        }
    }
    if (!finite) {
        atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
        return;
    }
    float *out = a.compressed + g * a.compressed_stride;
#pragma unroll
    for (int k = 0; k < kCompressorLanesPerThread; ++k) {
        const unsigned long long lane = tid + (unsigned long long)k * kCompressorThreads;
        if (lane < hd) out[lane] = value[k];
    }
    if (tid == 0u && a.positions) a.positions[g] = a.start_position + (unsigned long long)first_current;
}

// The same emission with four adjacent lanes per thread and 16-byte accesses, for rows
// whose width, strides and addresses are multiples of four floats (every geometry the
// reference uses). A rotated pair (even lane, odd lane) lies inside one thread.
struct compressor_row4 {
    const float4 *kv, *score, *ape;
};

template <bool OVERLAP>
__device__ __forceinline__ compressor_row4 compressor_source4(const yvx_compressor_args &a, long long token,
                                                              unsigned long long cursor,
                                                              unsigned long long state_slot,
                                                              unsigned long long width, unsigned long long column)
{
    compressor_row4 r;
    if (token >= 0) {
        const unsigned long long offset = (unsigned long long)token * a.token_stride + column;
        r.kv = reinterpret_cast<const float4 *>(a.token_kv + offset);
        r.score = reinterpret_cast<const float4 *>(a.token_score + offset);
        r.ape = reinterpret_cast<const float4 *>(a.ape + cursor * width + column);
    } else {
        r.kv = reinterpret_cast<const float4 *>(a.state_kv + state_slot * width + column);
        r.score = reinterpret_cast<const float4 *>(a.state_score + state_slot * width + column);
        r.ape = nullptr;
    }
    return r;
}

__device__ __forceinline__ void compressor_load4(const compressor_row4 &r, float (&score)[4], bool &finite)
{
    const float4 s = __ldg(r.score);
    score[0] = s.x, score[1] = s.y, score[2] = s.z, score[3] = s.w;
    if (r.ape) {
        const float4 p = __ldg(r.ape);
        const float ape[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            finite = finite && isfinite(score[k]) && isfinite(ape[k]);
            score[k] = __fadd_rn(score[k], ape[k]);
        }
    }
}

template <bool OVERLAP>
__global__ void __launch_bounds__(kCompressorThreads, 4)
compressor_chunk4_kernel(const yvx_compressor_args a, unsigned long long emitted)
{
    const unsigned long long ratio = a.ratio, hd = a.head_dim;
    const unsigned long long width = OVERLAP ? 2ull * hd : hd;
    const unsigned long long c0 = a.start_position % ratio;
    const unsigned int tid = threadIdx.x;
    __shared__ double warp_part[kCompressorThreads / 32];
    if (blockIdx.x >= emitted) {
        compressor_state_slot(a, emitted, blockIdx.x - emitted, c0);
        return;
    }
    const unsigned long long g = blockIdx.x;
    const long long first_current = (long long)(g * ratio) - (long long)c0;
    const long long first_previous = first_current - (long long)ratio;
    const unsigned long long lane0 = 4ull * tid;
    const bool active = lane0 < hd;
    bool finite = true;
    float value[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (active) {
        float top[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        double denominator[4] = {0.0, 0.0, 0.0, 0.0}, sum[4] = {0.0, 0.0, 0.0, 0.0};
        float score[4];
        for (unsigned long long s = 0; s < ratio; ++s) {
            if (OVERLAP) {
                compressor_load4(compressor_source4<OVERLAP>(a, first_previous + (long long)s, s,
                                                             g == 0ull ? s : ratio + s, width, lane0),
                                 score, finite);
#pragma unroll
                for (int k = 0; k < 4; ++k) top[k] = fmaxf(top[k], score[k]);
            }
            compressor_load4(compressor_source4<OVERLAP>(a, first_current + (long long)s, s,
                                                         OVERLAP ? ratio + s : s, width,
                                                         lane0 + (OVERLAP ? hd : 0ull)),
                             score, finite);
#pragma unroll
            for (int k = 0; k < 4; ++k) top[k] = fmaxf(top[k], score[k]);
        }
        double top_wide[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) top_wide[k] = compressor_widen(top[k]);
        for (unsigned long long s = 0; s < ratio; ++s) {
#pragma unroll
            for (int half = OVERLAP ? 0 : 1; half < 2; ++half) {
                const compressor_row4 r =
                    half == 0 ? compressor_source4<OVERLAP>(a, first_previous + (long long)s, s,
                                                            g == 0ull ? s : ratio + s, width, lane0)
                              : compressor_source4<OVERLAP>(a, first_current + (long long)s, s,
                                                            OVERLAP ? ratio + s : s, width,
                                                            lane0 + (OVERLAP ? hd : 0ull));
                compressor_load4(r, score, finite);
                const float4 v = __ldg(r.kv);
                const float kv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const double w = exp(__dsub_rn(compressor_widen(score[k]), top_wide[k]));
                    if (r.ape) finite = finite && isfinite(kv[k]);
                    denominator[k] = __dadd_rn(denominator[k], w);
                    sum[k] = __dadd_rn(sum[k], __dmul_rn(w, compressor_widen(kv[k])));
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            finite = finite && isfinite(denominator[k]) && denominator[k] > 0.0 && isfinite(sum[k]);
            value[k] = __double2float_rn(__ddiv_rn(sum[k], denominator[k]));
            finite = finite && isfinite(value[k]);
        }
    }
    if (a.norm_weights) {
        double squares = 0.0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            value[k] = compressor_bf16(value[k]);
            squares = __dadd_rn(squares, __dmul_rn((double)value[k], (double)value[k]));
        }
#pragma unroll
        for (int offset = 16; offset; offset >>= 1)
            squares = __dadd_rn(squares, __shfl_xor_sync(0xffffffffu, squares, offset));
        if ((tid & 31u) == 0u) warp_part[tid >> 5] = squares;
        __syncthreads();
        double mean = 0.0;
#pragma unroll
        for (int w = 0; w < kCompressorThreads / 32; ++w)
            if (w < (int)(blockDim.x >> 5)) mean = __dadd_rn(mean, warp_part[w]);
        mean = __ddiv_rn(mean, (double)hd);
        const double inverse = __ddiv_rn(1.0, sqrt(__dadd_rn(mean, a.epsilon)));
        finite = finite && isfinite(inverse);
        if (active) {
            const unsigned long long rope_start = a.rope_dims ? hd - a.rope_dims : hd;
            const unsigned long long position = a.start_position + (unsigned long long)first_current;
            const float4 weights = __ldg(reinterpret_cast<const float4 *>(a.norm_weights + lane0));
            const float weight[4] = {weights.x, weights.y, weights.z, weights.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float v = __double2float_rn(__dmul_rn(__dmul_rn((double)value[k], inverse), (double)weight[k]));
                finite = finite && isfinite(weight[k]) && isfinite(v);
                value[k] = compressor_bf16(v);
            }
#pragma unroll
            for (int k = 0; k < 4; k += 2) {
                if (lane0 + k < rope_start) continue;
                const unsigned long long i = lane0 + k - rope_start;
                const double angle = __dmul_rn((double)position, a.rope_frequency[i >> 1]);
                double sn, c;
                sincos(angle, &sn, &c);
                const double x = (double)value[k], y = (double)value[k + 1];
                const float rx = __double2float_rn(__dsub_rn(__dmul_rn(x, c), __dmul_rn(y, sn)));
                const float ry = __double2float_rn(__dadd_rn(__dmul_rn(x, sn), __dmul_rn(y, c)));
                finite = finite && isfinite(c) && isfinite(sn) && isfinite(rx) && isfinite(ry);
                value[k] = rx, value[k + 1] = ry;
            }
            if (a.rope_dims) {
#pragma unroll
                for (int k = 0; k < 4; ++k) value[k] = compressor_bf16(value[k]);
            }
        }
    }
    if (a.activation_quantization) {
        // warp w holds lanes [128 w, 128 w + 128): one segment of the activation's layout
        const unsigned int count = (unsigned int)a.activation_count, segment = (tid >> 5) * 128u;
        if (segment < count) {
            const bool quantised = lane0 < count;
            float q[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) q[k] = quantised ? value[k] : 0.0f;
            const unsigned int group = (unsigned int)a.activation_block_width / 4u;
            if (a.activation_hadamard)
                activation_segment<true>(q, tid & 31u, group, a.activation_quantization == 8u,
                                         __fdiv_rn(1.0f, sqrtf((float)count)));
            else
                activation_segment<false>(q, tid & 31u, group, a.activation_quantization == 8u, 1.0f);
            if (quantised) {
#pragma unroll
                for (int k = 0; k < 4; ++k) value[k] = q[k];
            }
        }
    }
    if (!finite) {
        atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
        return;
    }
    if (active)
        *reinterpret_cast<float4 *>(a.compressed + g * a.compressed_stride + lane0) =
            make_float4(value[0], value[1], value[2], value[3]);
    if (tid == 0u && a.positions) a.positions[g] = a.start_position + (unsigned long long)first_current;
}

}  // namespace yvx

extern "C" int yvx_cuda_compressor_chunk(const yvx_compressor_args *a, void *stream,
                                         unsigned long long *emitted_out)
{
    if (emitted_out) *emitted_out = 0ull;
    if (!a || !a->ratio || !a->head_dim || !a->ape || !a->state_kv || !a->state_score ||
        !a->after_kv || !a->after_score || !a->status ||
        (a->token_count && (!a->token_kv || !a->token_score)))
        return YVEX_ERR_INVALID_ARG;
    const unsigned long long width = a->head_dim * (a->overlap ? 2ull : 1ull);
    const unsigned long long slots = a->ratio * (a->overlap ? 2ull : 1ull);
    if (a->after_kv == a->state_kv || a->after_score == a->state_score) return YVEX_ERR_INVALID_ARG;
    if (a->token_count && a->token_stride < width) return YVEX_ERR_FORMAT;
    if (a->head_dim > (unsigned long long)yvx::kCompressorThreads * yvx::kCompressorLanesPerThread ||
        (a->head_dim & 1ull) || a->ratio > (1ull << 20) || a->token_count > (1ull << 40))
        return YVEX_ERR_UNSUPPORTED;
    if (a->norm_weights) {
        if (!(a->epsilon > 0.0) || a->epsilon > 1.0e300) return YVEX_ERR_INVALID_ARG;
        if (a->rope_dims && (!a->rope_frequency || (a->rope_dims & 1ull) || a->rope_dims > a->head_dim))
            return YVEX_ERR_INVALID_ARG;
    }
    if (a->start_position > ~0ull - a->token_count) return YVEX_ERR_BOUNDS;
    const unsigned long long emitted = (a->start_position % a->ratio + a->token_count) / a->ratio;
    if (emitted && (!a->compressed || a->compressed_stride < a->head_dim)) return YVEX_ERR_FORMAT;
    if (emitted + slots > 0x7fffffffull) return YVEX_ERR_UNSUPPORTED;
    yvx_compressor_args args = *a;
    if (!args.norm_weights) args.rope_dims = 0ull;
    const unsigned long long misaligned =
        (unsigned long long)args.token_kv | (unsigned long long)args.token_score | (unsigned long long)args.ape |
        (unsigned long long)args.state_kv | (unsigned long long)args.state_score |
        (unsigned long long)args.compressed | (unsigned long long)args.norm_weights;
    const bool vector = !(a->head_dim & 3ull) && !(a->token_stride & 3ull) && !(a->compressed_stride & 3ull) &&
                        !(misaligned & 15ull);
    if (a->activation_quantization) {
        if (a->activation_quantization != 8u && a->activation_quantization != 4u) return YVEX_ERR_FORMAT;
        if (!a->activation_count || a->activation_count > a->head_dim || !a->activation_block_width)
            return YVEX_ERR_INVALID_ARG;
        if (a->activation_count % a->activation_block_width) return YVEX_ERR_BOUNDS;
        if (!vector || (a->activation_count & 3ull) || a->activation_block_width < 4ull ||
            a->activation_block_width > 128ull || (a->activation_block_width & (a->activation_block_width - 1ull)) ||
            (a->activation_hadamard && (a->activation_count <= 64ull || a->activation_count > 128ull)))
            return YVEX_ERR_UNSUPPORTED;
    }
    const unsigned int grid = (unsigned int)(emitted + slots);
    const unsigned int threads4 = (unsigned int)((a->head_dim / 4ull + 31ull) / 32ull * 32ull);
    if (vector && a->overlap)
        yvx::compressor_chunk4_kernel<true><<<grid, threads4, 0, (cudaStream_t)stream>>>(args, emitted);
    else if (vector)
        yvx::compressor_chunk4_kernel<false><<<grid, threads4, 0, (cudaStream_t)stream>>>(args, emitted);
    else
        yvx::compressor_chunk_kernel<<<grid, yvx::kCompressorThreads, 0, (cudaStream_t)stream>>>(args, emitted);
    if (emitted_out) *emitted_out = emitted;
    return yvx_cuda_check(cudaGetLastError(), "compressor_chunk_kernel");
}
