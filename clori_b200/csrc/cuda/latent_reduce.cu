// Shared-latent attention reduce: every query head attends over ONE row per
// position, the row is both key and value, and a per-head sink logit joins the
// softmax denominator. Local pass over the sliding window, then a pass over
// compressed rows (selected indices or all rows up to the position).
//
// Replaces yvex_attention_reduce_native (src/backend/cuda/attention_kernels.cu:
// 259-406 in the reference: one CTA per (token, head), two block barriers per
// candidate row, output accumulated in global memory, every head re-reading the
// shared rows). Here one warp owns a (token, head) pair with the query and the
// accumulator in registers and eight heads of a token share a CTA. The CTA
// resolves a chunk of candidates to row pointers, brings the whole chunk into
// shared memory with asynchronous 16-byte copies (one memory latency per chunk
// instead of one per row, the next chunk in flight while the warps work on the
// current one), and each warp walks the rows from shared memory. A decode step
// has too few (token, head) pairs to fill the GPU, so the candidate list is also
// split across CTAs; the partial (m, l, acc) states are folded by a second small
// launch that also publishes. Row visibility and the published value (quotient
// rounded to bf16, stored as F32) are the reference's; the reference's output
// rotation and second publication (src/graph/core.c:498-507) can be fused into
// the epilogue.
#include "common.cuh"

namespace yvx {

constexpr int kLatentWarps = 8;
constexpr int kLatentBufferFloats = 8192;  // one staging buffer: 32 KB, two of them

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

// Publication of one (token, head): quotient, bf16, and with rope_frequency the
// reference's inverse rotation (rope_apply with inverse = 1) and second publication.
// Rotated pairs are adjacent lanes, so the partner sits in the neighbouring lane of the
// same slot; the branch around the shuffle is uniform per slot.
template <int SLOTS>
__device__ __forceinline__ void latent_publish(const yvx_latent_reduce_args &a, unsigned long long ordinal,
                                               unsigned long long head, unsigned int lane,
                                               const float (&acc)[SLOTS], float l, unsigned int first_slot = 0u)
{
    const unsigned long long token_position = a.phase_start_position + ordinal;
    float *out = a.out + (ordinal * a.query_heads + head) * a.head_dim;
    const unsigned long long rope_start = a.rope_frequency ? a.head_dim - a.rope_dims : a.head_dim;
    bool published_finite = true;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const unsigned long long d = lane + 32ull * (first_slot + s);
        float published = acc[s] / l;
        published_finite = published_finite && isfinite(published);
        published = __uint_as_float((uint32_t)bf16_bits_rne(published) << 16);
        if (rope_start < a.head_dim && 32ull * (first_slot + s) + 32ull > rope_start) {
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

__device__ __forceinline__ void latent_copy16(float *dst, const float *src)
{
    const unsigned int smem = (unsigned int)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(src) : "memory");
}

// grid: x = head tile (8 heads), y = token, z = split of the candidate list.
// SLOTS * 32 >= head_dim. Split z of a token covers candidates
// [z * per_split, (z + 1) * per_split) of the list "local rows, then compressed rows".
// splits == 1: publishes. Otherwise writes (acc[head_dim], m, l) to
// partials[((token * heads + head) * splits + z) * (head_dim + 2)].
template <int SLOTS>
__global__ void __launch_bounds__(kLatentWarps * 32)
latent_reduce_kernel(const yvx_latent_reduce_args a, const unsigned int splits,
                     const unsigned long long per_split, float *partials)
{
    constexpr unsigned int kRowFloats = SLOTS * 32;
    constexpr unsigned int kChunkRows = kLatentBufferFloats / kRowFloats;
    extern __shared__ __align__(16) float staged[];             // [2][kChunkRows][kRowFloats]
    __shared__ const float *row_of[2][kChunkRows];
    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned long long ordinal = blockIdx.y;
    const unsigned long long head = (unsigned long long)blockIdx.x * kLatentWarps + warp;
    const bool owner = head < a.query_heads;
    const unsigned long long token_position = a.phase_start_position + ordinal;
    unsigned long long local_offset, local_count;
    if (a.candidate_block_visible) {
        local_offset = 0ull;
        local_count = a.initial_local_count + a.token_count;
    } else {
        const unsigned long long before = a.initial_local_count + ordinal;
        const unsigned long long history =
            token_position < a.sliding_window - 1ull ? token_position : a.sliding_window - 1ull;
        if (history > before) {  // uniform over the CTA
            if (threadIdx.x == 0) atomicCAS(a.status, 0, YVX_STATUS_CONTRACT);
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
    const unsigned long long total = local_count + compressed_count;
    const unsigned long long begin = min((unsigned long long)blockIdx.z * per_split, total);
    const unsigned long long end = min(begin + per_split, total);

    const float log2e = 1.4426950408889634f;
    const float scale = rsqrtf((float)a.head_dim) * log2e;  // scores in log2 units
    float qr[SLOTS], acc[SLOTS];
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const unsigned long long d = lane + 32ull * s;
        qr[s] = owner && d < a.head_dim ? a.query[(ordinal * a.query_heads + head) * a.head_dim + d] * scale : 0.0f;
        acc[s] = 0.0f;
    }
    // the sink seeds the maximum and the denominator of the first split
    float m = -INFINITY, l = 0.0f;
    bool finite = true;
    if (blockIdx.z == 0u && owner) {
        m = a.sinks[head] * log2e;
        l = 1.0f;
        finite = isfinite(m);
    }
    // 16-byte copies need aligned rows; otherwise the rows are copied float by float
    const bool vector_rows =
        (a.head_dim & 3ull) == 0ull && (a.local_stride & 3ull) == 0ull &&
        (reinterpret_cast<unsigned long long>(a.local) & 15ull) == 0ull &&
        (a.attention_class == 0u || ((a.compressed_stride & 3ull) == 0ull &&
                                     (reinterpret_cast<unsigned long long>(a.compressed) & 15ull) == 0ull));
    const unsigned int chunks = (unsigned int)((end - begin + kChunkRows - 1u) / kChunkRows);

    // candidate of this thread in a chunk -> row pointer (nullptr: not visible / past the end)
    auto resolve = [&](unsigned int chunk) -> const float * {
        const unsigned long long c = begin + (unsigned long long)chunk * kChunkRows + threadIdx.x;
        if (threadIdx.x >= kChunkRows || chunk >= chunks || c >= end) return nullptr;
        return c < local_count ? latent_visible_row(a, 0u, ordinal, c, local_offset)
                               : latent_visible_row(a, 1u, ordinal, c - local_count, local_offset);
    };
    auto stage = [&](unsigned int chunk) {  // asynchronous copy of the chunk's rows
        float *buffer = staged + (chunk & 1u) * kLatentBufferFloats;
        if (vector_rows) {
            const unsigned int quads = (unsigned int)(a.head_dim >> 2);
            for (unsigned int i = threadIdx.x; i < kChunkRows * quads; i += blockDim.x) {
                const unsigned int r = i / quads, c = i % quads;
                const float *row = row_of[chunk & 1u][r];
                if (row) latent_copy16(buffer + r * kRowFloats + 4u * c, row + 4u * c);
            }
        } else {
            for (unsigned int i = threadIdx.x; i < kChunkRows * (unsigned int)a.head_dim; i += blockDim.x) {
                const unsigned int r = i / (unsigned int)a.head_dim, c = i % (unsigned int)a.head_dim;
                const float *row = row_of[chunk & 1u][r];
                if (row) buffer[r * kRowFloats + c] = row[c];
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // The first two chunks are resolved together (their index and position lookups overlap)
    // and both copies start before any row is used; later chunks are resolved while the
    // warps work, in the registers of the resolving threads.
    if (chunks) {
        const float *first_row = resolve(0), *second_row = resolve(1);
        if (threadIdx.x < kChunkRows) {
            row_of[0][threadIdx.x] = first_row;
            row_of[1][threadIdx.x] = second_row;
        }
        __syncthreads();
        stage(0);
        if (chunks > 1u) stage(1);
    }
    for (unsigned int chunk = 0; chunk < chunks; ++chunk) {
        const float *later_row = resolve(chunk + 2u);
        if (chunk + 1u < chunks) {
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // this chunk's rows are in shared memory for every warp
        const float *buffer = staged + (chunk & 1u) * kLatentBufferFloats;
        // Four rows per step: four independent dot products and reductions in flight, one
        // rescale of the running state per step.
        for (unsigned int r0 = 0; r0 < kChunkRows; r0 += 4u) {
            float v[4][SLOTS], dot[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const bool present = row_of[chunk & 1u][r0 + i] != nullptr;  // identical on every thread
                const float *row = buffer + (r0 + i) * kRowFloats;
                dot[i] = 0.0f;
#pragma unroll
                for (int s = 0; s < SLOTS; ++s) {
                    const unsigned long long d = lane + 32ull * s;
                    v[i][s] = present && d < a.head_dim ? row[d] : 0.0f;
                    dot[i] = fmaf(qr[s], v[i][s], dot[i]);
                }
            }
#pragma unroll
            for (int offset = 16; offset; offset >>= 1)
#pragma unroll
                for (int i = 0; i < 4; ++i) dot[i] += __shfl_xor_sync(0xffffffffu, dot[i], offset);
            float top = m;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                finite = finite && isfinite(dot[i]);
                if (row_of[chunk & 1u][r0 + i] == nullptr) dot[i] = -INFINITY;
                top = fmaxf(top, dot[i]);
            }
            if (top == -INFINITY) continue;  // no row yet and no sink in this split
            float keep, w[4];
            asm("ex2.approx.f32 %0, %1;" : "=f"(keep) : "f"(m - top));  // 0 when m is still -inf
            l *= keep;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                asm("ex2.approx.f32 %0, %1;" : "=f"(w[i]) : "f"(dot[i] - top));
                l += w[i];
            }
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                float x = acc[s] * keep;
#pragma unroll
                for (int i = 0; i < 4; ++i) x = fmaf(w[i], v[i][s], x);
                acc[s] = x;
            }
            m = top;
        }
        __syncthreads();  // every warp is done with this buffer and its row pointers
        if (chunk + 2u < chunks) {
            if (threadIdx.x < kChunkRows) row_of[chunk & 1u][threadIdx.x] = later_row;
            __syncthreads();
            stage(chunk + 2u);
        }
    }
    pdl_launch_dependents();
    if (!owner) return;
    if (!finite) {
        if (lane == 0) atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
        return;
    }
    if (splits == 1u) {
        if (!isfinite(l) || l <= 0.0f) {
            if (lane == 0) atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
            return;
        }
        latent_publish<SLOTS>(a, ordinal, head, lane, acc, l);
        return;
    }
    float *part = partials + ((ordinal * a.query_heads + head) * splits + blockIdx.z) * (a.head_dim + 2ull);
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const unsigned long long d = lane + 32ull * s;
        if (d < a.head_dim) part[d] = acc[s];
    }
    if (lane == 0) {
        part[a.head_dim] = m;
        part[a.head_dim + 1ull] = l;
    }
}

// Folds the splits of a (token, head) in split order and publishes. grid: x = head,
// y = token; SLOTS / 4 warps, each owning four 32-lane slots of the head's row, so that
// sixteen splits' worth of loads are in flight per warp.
template <int SLOTS>
__global__ void __launch_bounds__(SLOTS * 8)
latent_fold_kernel(const yvx_latent_reduce_args a, const unsigned int splits, const float *partials)
{
    constexpr int kOwn = 4, kFoldBatch = 16;
    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned int first_slot = warp * kOwn;
    const unsigned long long ordinal = blockIdx.y, head = blockIdx.x;
    pdl_wait();
    // a split that refused leaves its partial unwritten: nothing to publish
    if (*reinterpret_cast<volatile int *>(a.status) != YVX_STATUS_OK) return;
    const unsigned long long width = a.head_dim + 2ull;
    const float *part = partials + (ordinal * a.query_heads + head) * splits * width;
    float m = -INFINITY;
    for (unsigned int i = lane; i < splits; i += 32u) m = fmaxf(m, __ldcg(part + i * width + a.head_dim));
#pragma unroll
    for (int offset = 16; offset; offset >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, offset));
    float acc[kOwn], l = 0.0f;
#pragma unroll
    for (int s = 0; s < kOwn; ++s) acc[s] = 0.0f;
    // Lane i owns the weight of split base + i; the rows of the splits are then read with
    // loads that depend on nothing but the split index, a batch of them in flight at once.
    for (unsigned int base = 0; base < splits; base += 32u) {
        const unsigned int mine = base + lane;
        float w_lane = 0.0f;
        if (mine < splits) {
            const float mi = __ldcg(part + mine * width + a.head_dim);
            const float li = __ldcg(part + mine * width + a.head_dim + 1ull);
            asm("ex2.approx.f32 %0, %1;" : "=f"(w_lane) : "f"(mi - m));  // 0 for a split without rows
            l = fmaf(li, w_lane, l);
        }
        const unsigned int count = min(32u, splits - base);
        for (unsigned int j0 = 0; j0 < count; j0 += kFoldBatch) {
            float v[kFoldBatch][kOwn], w[kFoldBatch];
#pragma unroll
            for (int j = 0; j < kFoldBatch; ++j) {
                const bool live = j0 + j < count;
                const float *p = part + (base + j0 + (live ? j : 0)) * width;
                w[j] = __shfl_sync(0xffffffffu, w_lane, (j0 + j) & 31u);
                if (!live) w[j] = 0.0f;
#pragma unroll
                for (int s = 0; s < kOwn; ++s) {
                    const unsigned long long d = lane + 32ull * (first_slot + s);
                    v[j][s] = d < a.head_dim ? __ldcg(p + d) : 0.0f;
                }
            }
#pragma unroll
            for (int j = 0; j < kFoldBatch; ++j)
#pragma unroll
                for (int s = 0; s < kOwn; ++s) acc[s] = fmaf(v[j][s], w[j], acc[s]);
        }
    }
    l = warp_sum(l);
    if (!isfinite(l) || l <= 0.0f) {
        if (lane == 0) atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
        return;
    }
    latent_publish<kOwn>(a, ordinal, head, lane, acc, l, first_slot);
}

struct latent_plan {
    unsigned int splits;
    unsigned long long per_split;
};

// Deterministic in the arguments and the SM count: enough CTAs for two per SM, splits
// of whole staging chunks, never more splits than chunks in the longest candidate list.
static latent_plan latent_make_plan(const yvx_latent_reduce_args &a, int sms)
{
    const unsigned int slots = a.head_dim <= 128ull ? 4u : a.head_dim <= 256ull ? 8u : 16u;
    const unsigned long long chunk_rows = kLatentBufferFloats / (slots * 32u);
    const unsigned long long rows_local = a.initial_local_count + a.token_count;
    const unsigned long long max_local =
        a.candidate_block_visible || rows_local < a.sliding_window ? rows_local : a.sliding_window;
    const unsigned long long last = a.phase_start_position + a.token_count - 1ull;
    const unsigned long long max_compressed =
        a.attention_class == 0u ? 0ull : a.attention_class == 1u ? a.topk_capacity : last / a.ratio + 1ull;
    const unsigned long long max_total = max_local + max_compressed ? max_local + max_compressed : 1ull;
    const unsigned long long tiles = (a.query_heads + kLatentWarps - 1) / kLatentWarps * a.token_count;
    unsigned long long splits = (2ull * (unsigned long long)sms + tiles - 1ull) / tiles;
    const unsigned long long max_splits = (max_total + chunk_rows - 1ull) / chunk_rows;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1ull) splits = 1ull;
    unsigned long long per_split = (max_total + splits - 1ull) / splits;
    per_split = (per_split + chunk_rows - 1ull) / chunk_rows * chunk_rows;
    splits = (max_total + per_split - 1ull) / per_split;
    latent_plan plan = {(unsigned int)splits, per_split};
    return plan;
}

static int latent_sm_count()
{
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    return sms;
}

template <int SLOTS>
static int latent_launch(const yvx_latent_reduce_args &a, cudaStream_t s, unsigned int *launches)
{
    latent_plan plan = {1u, ~0ull >> 1};
    if (a.workspace) plan = latent_make_plan(a, latent_sm_count());
    if (plan.splits == 1u) plan.per_split = ~0ull >> 1;
    const size_t smem = 2u * kLatentBufferFloats * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(latent_reduce_kernel<SLOTS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return yvx_cuda_check(e, "latent_reduce_kernel attribute");
    const unsigned int tiles = (unsigned int)((a.query_heads + kLatentWarps - 1) / kLatentWarps);
    latent_reduce_kernel<SLOTS><<<dim3(tiles, (unsigned int)a.token_count, plan.splits), kLatentWarps * 32, smem, s>>>(
        a, plan.splits, plan.per_split, (float *)a.workspace);
    if (launches) *launches = 1u;
    if (plan.splits > 1u) {
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3((unsigned int)a.query_heads, (unsigned int)a.token_count, 1);
        config.blockDim = dim3(SLOTS * 8, 1, 1);
        config.stream = s;
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[0].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
        e = cudaLaunchKernelEx(&config, latent_fold_kernel<SLOTS>, a, plan.splits, (const float *)a.workspace);
        if (e != cudaSuccess) return yvx_cuda_check(e, "latent_fold_kernel");
        if (launches) *launches = 2u;
    }
    return yvx_cuda_check(cudaGetLastError(), "latent_reduce_kernel");
}

static int latent_admit(const yvx_latent_reduce_args *a)
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
    return 0;
}

}  // namespace yvx

extern "C" unsigned long long yvx_cuda_latent_reduce_workspace_bytes(const yvx_latent_reduce_args *a)
{
    if (yvx::latent_admit(a) != 0) return 0ull;
    const yvx::latent_plan plan = yvx::latent_make_plan(*a, yvx::latent_sm_count());
    if (plan.splits <= 1u) return 0ull;
    return a->token_count * a->query_heads * plan.splits * (a->head_dim + 2ull) * sizeof(float);
}

extern "C" int yvx_cuda_latent_reduce_launches(const yvx_latent_reduce_args *a, void *stream, unsigned int *launches)
{
    if (launches) *launches = 0u;
    const int admitted = yvx::latent_admit(a);
    if (admitted != 0) return admitted;
    cudaStream_t s = (cudaStream_t)stream;
    if (a->head_dim <= 128ull) return yvx::latent_launch<4>(*a, s, launches);
    if (a->head_dim <= 256ull) return yvx::latent_launch<8>(*a, s, launches);
    return yvx::latent_launch<16>(*a, s, launches);
}

extern "C" int yvx_cuda_latent_reduce(const yvx_latent_reduce_args *a, void *stream)
{
    return yvx_cuda_latent_reduce_launches(a, stream, nullptr);
}
