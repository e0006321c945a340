// Shared-latent attention reduce: every query head attends over ONE row per
// position, the row is both key and value, and a per-head sink logit joins the
// softmax denominator. Local pass over the sliding window, then a pass over
// compressed rows (selected indices or all rows up to the position).
//
// Replaces yvex_attention_reduce_native (src/backend/cuda/attention_kernels.cu:
// 259-406 in the reference: one CTA per (token, head), two block barriers per
// candidate row, output accumulated in global memory, every head re-reading the
// shared rows). Here one warp owns a (token, head) pair with the query and the
// accumulator in registers, eight heads of a token share a CTA so a row fetched
// once from L2 serves eight heads, and the softmax state never leaves the warp.
// Row visibility and the published value (quotient rounded to bf16, stored as
// F32) are the reference's; the reference's output rotation and second
// publication (src/graph/core.c:498-507) can be fused into the epilogue.
#include "common.cuh"

namespace yvx {

constexpr int kLatentWarps = 8;

__device__ __forceinline__ const float *latent_visible_row(const yvx_latent_reduce_args &a,
                                                           unsigned int pass,
                                                           unsigned long long ordinal,
                                                           unsigned long long candidate,
                                                           unsigned long long local_offset)
{
    const unsigned long long token_position = a.phase_start_position + ordinal;
    if (pass == 0u) {
        candidate += local_offset;
        const unsigned long long position = a.local_positions[candidate];
        if (!a.candidate_block_visible) {
            const unsigned long long first = token_position + 1ull > a.sliding_window
                                                 ? token_position + 1ull - a.sliding_window : 0ull;
            if (position < first || position > token_position) return nullptr;
        }
        return a.local + candidate * a.local_stride;
    }
    const unsigned long long index =
        a.attention_class == 2u ? candidate : a.selected[ordinal * a.topk_capacity + candidate];
    const unsigned long long position = a.compressed_positions[index];
    if (position > token_position || position > ~0ull - a.ratio + 1ull ||
        position + a.ratio - 1ull > token_position)
        return nullptr;
    return a.compressed + index * a.compressed_stride;
}

// grid: x = head tile (8 heads), y = token. SLOTS * 32 >= head_dim.
template <int SLOTS>
__global__ void __launch_bounds__(kLatentWarps * 32)
latent_reduce_kernel(const yvx_latent_reduce_args a)
{
    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned long long ordinal = blockIdx.y;
    const unsigned long long head = (unsigned long long)blockIdx.x * kLatentWarps + warp;
    if (head >= a.query_heads) return;
    const unsigned long long token_position = a.phase_start_position + ordinal;
    unsigned long long local_offset, local_count;
    if (a.candidate_block_visible) {
        local_offset = 0ull;
        local_count = a.initial_local_count + a.token_count;
    } else {
        const unsigned long long before = a.initial_local_count + ordinal;
        const unsigned long long history =
            token_position < a.sliding_window - 1ull ? token_position : a.sliding_window - 1ull;
        if (history > before) {
            if (lane == 0) atomicCAS(a.status, 0, YVX_STATUS_CONTRACT);
            return;
        }
        local_offset = before - history;
        local_count = history + 1ull;
    }
    const unsigned long long compressed_count =
        a.attention_class == 0u ? 0ull
        : a.attention_class == 1u
            ? a.selected_count[ordinal]
            : token_position / a.ratio + ((token_position + 1ull) % a.ratio == 0ull);

    const float log2e = 1.4426950408889634f;
    const float scale = rsqrtf((float)a.head_dim) * log2e;  // scores in log2 units
    const float *q = a.query + (ordinal * a.query_heads + head) * a.head_dim;
    float qr[SLOTS], acc[SLOTS];
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const unsigned long long d = lane + 32ull * s;
        qr[s] = d < a.head_dim ? q[d] * scale : 0.0f;
        acc[s] = 0.0f;
    }
    float m = a.sinks[head] * log2e, l = 1.0f;  // the sink seeds the maximum and the denominator
    bool finite = isfinite(m);
    for (unsigned int pass = 0; pass < 2u; ++pass) {
        const unsigned long long count = pass == 0u ? local_count : compressed_count;
        for (unsigned long long candidate = 0; candidate < count; ++candidate) {
            const float *row = latent_visible_row(a, pass, ordinal, candidate, local_offset);
            if (!row) continue;  // identical on every lane
            float r[SLOTS], dot = 0.0f;
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                const unsigned long long d = lane + 32ull * s;
                r[s] = d < a.head_dim ? row[d] : 0.0f;
                dot = fmaf(qr[s], r[s], dot);
            }
            dot = warp_sum(dot);
            finite = finite && isfinite(dot);
            if (dot <= m) {
                float w;
                asm("ex2.approx.f32 %0, %1;" : "=f"(w) : "f"(dot - m));
                l += w;
#pragma unroll
                for (int s = 0; s < SLOTS; ++s) acc[s] = fmaf(w, r[s], acc[s]);
            } else {
                float keep;
                asm("ex2.approx.f32 %0, %1;" : "=f"(keep) : "f"(m - dot));
                l = fmaf(l, keep, 1.0f);
#pragma unroll
                for (int s = 0; s < SLOTS; ++s) acc[s] = fmaf(acc[s], keep, r[s]);
                m = dot;
            }
        }
    }
    if (!finite || !isfinite(l) || l <= 0.0f) {
        if (lane == 0) atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
        return;
    }
    float *out = a.out + (ordinal * a.query_heads + head) * a.head_dim;
    const unsigned long long rope_start = a.rope_frequency ? a.head_dim - a.rope_dims : a.head_dim;
    bool published_finite = true;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const unsigned long long d = lane + 32ull * s;
        float published = acc[s] / l;
        published_finite = published_finite && isfinite(published);
        published = __uint_as_float((uint32_t)bf16_bits_rne(published) << 16);
        // Output rotation of the reference (rope_apply with inverse = 1, then the second
        // publication): pairs are adjacent lanes, so the partner sits in the neighbouring
        // lane of the same slot. Uniform per slot: every lane reaches the shuffle.
        if (rope_start < a.head_dim && 32ull * s + 32ull > rope_start) {
            const float partner = __shfl_xor_sync(0xffffffffu, published, 1);
            if (d >= rope_start && d < a.head_dim) {
                const unsigned long long i = d - rope_start;
                const double angle = __dmul_rn((double)token_position, a.rope_frequency[i >> 1]);
                double sn, c;
                sincos(angle, &sn, &c);
                sn = -sn;
                const double x = (i & 1ull) ? (double)partner : (double)published;
                const double y = (i & 1ull) ? (double)published : (double)partner;
                const double rotated = (i & 1ull) ? __dadd_rn(__dmul_rn(x, sn), __dmul_rn(y, c))
                                                  : __dsub_rn(__dmul_rn(x, c), __dmul_rn(y, sn));
                published_finite = published_finite && isfinite(c) && isfinite(sn);
                published = __uint_as_float((uint32_t)bf16_bits_rne(__double2float_rn(rotated)) << 16);
            }
        }
        if (d < a.head_dim) {
            if (!published_finite)
                atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
            else
                out[d] = published;
        }
    }
}

}  // namespace yvx

extern "C" int yvx_cuda_latent_reduce(const yvx_latent_reduce_args *a, void *stream)
{
    // Admission mirrors the reference kernel's contract checks (attention_kernels.cu:291-306).
    if (!a || !a->query || !a->local || !a->local_positions || !a->sinks || !a->out || !a->status ||
        !a->query_heads || !a->head_dim || !a->sliding_window || !a->token_count ||
        a->attention_class > 2u ||
        (a->candidate_block_visible != 0 && a->candidate_block_visible != 1) ||
        a->local_stride < a->head_dim ||
        (a->attention_class != 0u &&
         (!a->compressed || !a->compressed_positions || a->compressed_stride < a->head_dim)) ||
        (a->attention_class == 1u && (!a->selected || !a->selected_count || !a->topk_capacity)) ||
        (a->attention_class == 1u && a->ratio != 4ull) ||
        (a->attention_class == 2u && a->ratio != 128ull) ||
        (a->attention_class == 0u && a->ratio != 0ull))
        return YVEX_ERR_INVALID_ARG;
    if (a->rope_frequency &&
        (a->rope_dims < 2ull || a->rope_dims > a->head_dim || (a->rope_dims & 1ull) ||
         ((a->head_dim - a->rope_dims) & 1ull)))
        return YVEX_ERR_INVALID_ARG;
    if (a->head_dim > 512ull || a->token_count > 65535ull) return YVEX_ERR_UNSUPPORTED;
    const dim3 grid((unsigned int)((a->query_heads + yvx::kLatentWarps - 1) / yvx::kLatentWarps),
                    (unsigned int)a->token_count);
    cudaStream_t s = (cudaStream_t)stream;
    if (a->head_dim <= 128ull)
        yvx::latent_reduce_kernel<4><<<grid, yvx::kLatentWarps * 32, 0, s>>>(*a);
    else if (a->head_dim <= 256ull)
        yvx::latent_reduce_kernel<8><<<grid, yvx::kLatentWarps * 32, 0, s>>>(*a);
    else
        yvx::latent_reduce_kernel<16><<<grid, yvx::kLatentWarps * 32, 0, s>>>(*a);
    return yvx_cuda_check(cudaGetLastError(), "latent_reduce_kernel");
}
