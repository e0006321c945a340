// Decode / verify over F32 KV rows under the exact-F32 contract (head_dim 128,
// at most 8 query vectors per KV head, contiguous KV), for launches too short
// for a streaming loop to reach the DRAM rate: a CTA's whole chunk (up to 112
// tokens of K and V for one KV head, 112 KB) is requested with TMA at the start,
// in sub-chunks of 16 tokens with their own mbarriers, and each warp consumes
// sub-chunks as they land. Seven sub-chunk buffers: two CTAs fit an SM only because
// nothing else lives in shared memory (the softmax weights of a sub-chunk go
// through the K rows the warp has just taken into registers; the merge reuses
// consumed buffers). With tickets the kernel also folds its own splits: the CTA
// that arrives last for a KV head combines every split's partial in split order
// and writes the output, so a decode step is ONE launch. All arithmetic is
// single-precision FMA.
//
//   scores   lanes own 4 dims; the 16 partial dot products per vector are summed
//            across lanes by a halving exchange (16 shuffles for 16 tokens, four
//            vectors interleaved), after which lanes 2t and 2t+1 hold token t's score
//   softmax  running max per vector (warp-uniform), exp2 domain
//   values   the 16 weights go through shared memory and come back as broadcast
//            loads; lanes own 4 output dims
//
// Same partial format and combine as the general kernel, which it replaces for
// these shapes (reference: yvex_gqa_f32_body, src/backend/cuda/
// transformer_kernels.cu:137-238, one CTA per query head walking all rows).
#include "exchange.cuh"
#include "pipeline.cuh"

namespace yvx {

constexpr int kF32Threads = 128, kF32Warps = 4;
constexpr int kF32HeadDim = 128;
constexpr int kF32Sub = 16;                       // tokens per sub-chunk
#ifndef F32_MAXSUBS
#define F32_MAXSUBS 7
#endif
constexpr int kF32MaxSubs = F32_MAXSUBS;                    // 112 tokens per CTA
constexpr int kF32Buffers = kF32MaxSubs;           // one buffer per sub-chunk: everything is in flight at once
constexpr int kF32SubBytes = kF32Sub * kF32HeadDim * 4;          // 8 KB
constexpr int kF32TailBytes = 384;                // barriers, merge statistics, the arrival flag
constexpr int kF32SmemBytes = 2 * kF32Buffers * kF32SubBytes + kF32TailBytes;
constexpr unsigned int kF32MaxSplits = 256;

struct F32Maps {
    CUtensorMap key, value;
};

__device__ __forceinline__ float f32_exp2(float x)
{
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Sums x[v][t] over the warp for 16 tokens of four vectors at once: afterwards
// every lane holds, per vector, the total of token (lane >> 1). The four vectors'
// exchanges are independent, so their shuffle latencies overlap.
__device__ __forceinline__ void reduce16x4(float (&x)[4][16], unsigned int lane, float (&total)[4])
{
#pragma unroll
    for (int width = 8, offset = 16; width >= 1; width >>= 1, offset >>= 1) {
        const bool upper = lane & offset;
#pragma unroll
        for (int i = 0; i < width; ++i)
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const float keep = upper ? x[v][i + width] : x[v][i];
                const float send = upper ? x[v][i] : x[v][i + width];
                x[v][i] = keep + __shfl_xor_sync(0xffffffffu, send, offset);
            }
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) total[v] = x[v][0] + __shfl_xor_sync(0xffffffffu, x[v][0], 1);
}

struct F32BlockSync {
    static __device__ __forceinline__ void sync() { __syncthreads(); }
};

// grid: x = split, y = kv head, z = session. VT = vectors per CTA (4 or 8).
template <int VT>
__global__ void __launch_bounds__(kF32Threads)
gqa_decode_f32_kernel(const yvx_gqa_problem p, const __grid_constant__ F32Maps maps, const int head_major,
                      const int cooperative)
{
    // No static shared memory: the dynamic window starts on a 1024-byte boundary and the two
    // resident CTAs of an SM need every byte (2 x (112 KB + 256 B + the 1 KB the system keeps)).
    extern __shared__ __align__(1024) unsigned char smem[];
    float *k_smem = reinterpret_cast<float *>(smem);
    float *v_smem = reinterpret_cast<float *>(smem + kF32Buffers * kF32SubBytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + 2 * kF32Buffers * kF32SubBytes);     // 7 x 8 B
    float (*merge_m)[VT] = reinterpret_cast<float (*)[VT]>(smem + 2 * kF32Buffers * kF32SubBytes + 64);
    float (*merge_l)[VT] = merge_m + kF32Warps;                                               // 2 x 128 B at most
    int *arrival = reinterpret_cast<int *>(smem + 2 * kF32Buffers * kF32SubBytes + kF32TailBytes - 4);

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned int group = p.query_heads / p.kv_heads;
    const unsigned int vectors = p.query_rows * group;
    const unsigned int split = blockIdx.x, kv_head = blockIdx.y, b = blockIdx.z;
    const unsigned int kv_tokens = admitted_kv_tokens(p.kv_tokens, b, p.kv_tokens_uniform, p.kv_tokens_max, p.status);
    long long query_start;
    if (p.query_start)
        query_start = (long long)p.query_start[b];
    else if (p.query_start_from_end)
        query_start = (long long)kv_tokens - (long long)p.query_rows;
    else
        query_start = (long long)p.query_start_uniform;

    const unsigned int t0 = split * p.chunk_tokens;
    if (t0 >= kv_tokens) return;
    unsigned int t1 = min(kv_tokens, t0 + p.chunk_tokens);
    if (p.causal) {
        const long long last = query_start + (long long)p.query_rows;  // exclusive
        if (last < (long long)t1) t1 = last > (long long)t0 ? (unsigned int)last : t0;
    }
    const unsigned int subs = (t1 - t0 + kF32Sub - 1) / kF32Sub;

    // Sub-chunk i lives in buffer i % 6 and is requested by `request`.
    auto request = [&](unsigned int i) {
        const unsigned int buffer = i % kF32Buffers;
        const int token = (int)(t0 + i * kF32Sub);
        const int c1 = head_major ? (int)kv_head : token, c2 = head_major ? token : (int)kv_head;
        mbar_expect_tx(&bars[buffer], 2 * kF32SubBytes);
        tma_load_4d(k_smem + buffer * kF32Sub * kF32HeadDim, &maps.key, &bars[buffer], 0, c1, c2, (int)b);
        tma_load_4d(v_smem + buffer * kF32Sub * kF32HeadDim, &maps.value, &bars[buffer], 0, c1, c2, (int)b);
    };
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.key) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.value) : "memory");
        for (int i = 0; i < kF32Buffers; ++i) mbar_init(&bars[i], 1);
        fence_barrier_init();
    }
    __syncthreads();
    // Every sub-chunk of the CTA is requested now (warp 3 owns a single buffer, so its first lane
    // has the time).
    if (threadIdx.x == 96)
        for (unsigned int i = 0; i < subs; ++i) request(i);

    // Per-vector query (scores in log2 units), visibility limit, running state.
    float4 q[VT];
    long long limit[VT];
    float m[VT], l[VT];
    float4 acc[VT];
#pragma unroll
    for (int v = 0; v < VT; ++v) {
        const bool live = (unsigned int)v < vectors;
        const unsigned int row = live ? v / group : 0u;
        const unsigned int qhead = kv_head * group + (live ? v % group : 0u);
        const float *qp = reinterpret_cast<const float *>(p.query) +
                          (unsigned long long)b * p.query_session_stride +
                          (unsigned long long)row * p.query_row_stride + (unsigned long long)qhead * kF32HeadDim;
        const float scale = p.scale * 1.4426950408889634f;
        float4 value = live ? *reinterpret_cast<const float4 *>(qp + 4u * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
        q[v] = make_float4(value.x * scale, value.y * scale, value.z * scale, value.w * scale);
        limit[v] = !live ? -1 : p.causal ? query_start + (long long)row : (long long)kv_tokens - 1;
        m[v] = -INFINITY;
        l[v] = 0.0f;
        acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

    bool ok = true;
    // A buffer (= a sub-chunk) belongs to one warp (buffer % 4).
    for (unsigned int sb = 0; sb < subs; ++sb) {
        const unsigned int buffer = sb;
        if (buffer % kF32Warps != warp) continue;
        if (ok) ok = mbar_wait(&bars[buffer], 0u);
        float *kb = k_smem + buffer * kF32Sub * kF32HeadDim;
        const float *vb = v_smem + buffer * kF32Sub * kF32HeadDim;
        // the sub-chunk's softmax weights [VT][16] go where its K row 0 was: the rows are in
        // registers by then, and the buffer is this warp's alone
        float (*weights)[kF32Sub] = reinterpret_cast<float (*)[kF32Sub]>(kb);
        const long long base = (long long)t0 + (long long)sb * kF32Sub;
        const unsigned int valid = min((unsigned int)kF32Sub, t1 - (unsigned int)base);
        float4 krow[kF32Sub];
#pragma unroll
        for (int t = 0; t < kF32Sub; ++t) krow[t] = reinterpret_cast<const float4 *>(kb + t * kF32HeadDim)[lane];
        __syncwarp();  // every lane holds its K before any lane stores a weight over row 0
#pragma unroll
        for (int v0 = 0; v0 < VT; v0 += 4) {
            float part[4][kF32Sub], score[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int t = 0; t < kF32Sub; ++t)
                    part[u][t] = fmaf(q[v0 + u].w, krow[t].w,
                                      fmaf(q[v0 + u].z, krow[t].z, fmaf(q[v0 + u].y, krow[t].y, q[v0 + u].x * krow[t].x)));
            reduce16x4(part, lane, score);
            const long long token = base + (long long)(lane >> 1);
            float tile_max[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (token > limit[v0 + u] || (lane >> 1) >= valid) score[u] = -INFINITY;
                tile_max[u] = score[u];
            }
#pragma unroll
            for (int offset = 2; offset < 32; offset <<= 1)
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    tile_max[u] = fmaxf(tile_max[u], __shfl_xor_sync(0xffffffffu, tile_max[u], offset));
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = v0 + u;
                const float fresh = fmaxf(m[v], tile_max[u]);
                const float keep = fresh == -INFINITY ? 1.0f : f32_exp2(m[v] - fresh);
                const float weight = fresh == -INFINITY ? 0.0f : f32_exp2(score[u] - fresh);
                m[v] = fresh;
                l[v] = l[v] * keep + ((lane & 1u) ? 0.0f : weight);
                acc[v] = make_float4(acc[v].x * keep, acc[v].y * keep, acc[v].z * keep, acc[v].w * keep);
                if (!(lane & 1u)) weights[v][lane >> 1] = weight;
            }
        }
        __syncwarp();
#pragma unroll
        for (int t4 = 0; t4 < kF32Sub / 4; ++t4) {
            if (4u * t4 >= valid) break;  // rows past the chunk may hold anything
            float4 vrow[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                vrow[j] = reinterpret_cast<const float4 *>(vb + (4 * t4 + j) * kF32HeadDim)[lane];
#pragma unroll
            for (int v = 0; v < VT; ++v) {
                const float4 w = *reinterpret_cast<const float4 *>(&weights[v][4 * t4]);
                const float ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (4u * t4 + j >= valid) continue;
                    acc[v].x = fmaf(ws[j], vrow[j].x, acc[v].x);
                    acc[v].y = fmaf(ws[j], vrow[j].y, acc[v].y);
                    acc[v].z = fmaf(ws[j], vrow[j].z, acc[v].z);
                    acc[v].w = fmaf(ws[j], vrow[j].w, acc[v].w);
                }
            }
        }
        __syncwarp();
    }
    if (!__all_sync(0xffffffffu, ok) && lane == 0) atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);

    // The main loop is over: let the combine kernel's launch overlap the epilogue.
    pdl_launch_dependents();
    // Merge the four warps through the (now consumed) K region.
    __syncthreads();
    float *merge_acc = k_smem;  // [warp][VT][128]
#pragma unroll
    for (int v = 0; v < VT; ++v) {
        const float total = warp_sum(l[v]);
        if (lane == 0) {
            merge_m[warp][v] = m[v];
            merge_l[warp][v] = total;
        }
        reinterpret_cast<float4 *>(merge_acc + (warp * VT + v) * kF32HeadDim)[lane] = acc[v];
    }
    __syncthreads();
    const bool direct = p.max_splits == 1u;
    const bool fold_here = !direct && p.tickets != nullptr;
    const unsigned int d = threadIdx.x;  // one head dimension per thread
    for (unsigned int v = 0; v < min((unsigned int)VT, vectors); ++v) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kF32Warps; ++w) mm = fmaxf(mm, merge_m[w][v]);
        float ll = 0.0f, o = 0.0f;
#pragma unroll
        for (int w = 0; w < kF32Warps; ++w) {
            const float scale = merge_m[w][v] == -INFINITY ? 0.0f : f32_exp2(merge_m[w][v] - mm);
            ll = fmaf(merge_l[w][v], scale, ll);
            o = fmaf(merge_acc[(w * VT + v) * kF32HeadDim + d], scale, o);
        }
        const unsigned int row = v / group, qhead = kv_head * group + v % group;
        const unsigned long long item = ((unsigned long long)b * p.query_rows + row) * p.query_heads + qhead;
        if (!YVX_CHECKED_INDEX(item < (unsigned long long)p.sessions * p.query_rows * p.query_heads &&
                                   split < p.max_splits && qhead < p.query_heads, p.status))
            continue;
        if (direct) {
            const float value = o / ll;
            if (!isfinite(value)) atomicCAS(p.status, 0, YVX_STATUS_NONFINITE);
            store_output(p.output, p.output_dtype, item * kF32HeadDim + d, value);
        } else {
            float *part = p.partials + (item * p.max_splits + split) * (kF32HeadDim + 2ull);
            part[d] = ll > 0.0f ? o / ll : 0.0f;
            if (d == 0) {
                part[kF32HeadDim] = mm * 0.6931471805599453f;  // natural-log units
                part[kF32HeadDim + 1] = ll;
            }
        }
    }
    if (!fold_here) return;

    // ---- the fold, inside the same launch ---------------------------------------------------
    // Every CTA publishes its partials (fence) and takes a ticket of its (session, KV head).
    // cooperative != 0 (every CTA of the grid is resident): the CTAs with split < vectors wait,
    // bounded, for all the group's tickets and fold one vector each, four warps sharing its
    // splits, so the folds of a KV head run side by side. Otherwise whichever CTA arrives last
    // folds all the group's vectors, and nobody waits for anybody.
    __threadfence();
    __syncthreads();
    const unsigned int live_splits = min((kv_tokens + p.chunk_tokens - 1u) / p.chunk_tokens, p.max_splits);
    int *ticket = p.tickets + 2ull * ((unsigned long long)b * p.kv_heads + kv_head);
    const unsigned int folders = min(min((unsigned int)VT, vectors), live_splits);
    float *fold_scratch = k_smem;                                   // [4][130]: the buffers are consumed
    float *fold_row = fold_scratch + kF32Warps * (kF32HeadDim + 2);
    if (cooperative) {
        if (threadIdx.x == 0) atomicAdd(ticket, 1);
        if (split >= folders) return;
        if (threadIdx.x == 0) {
            const volatile int *counter = ticket;
            int ok = 0;
            for (unsigned int spin = 0; spin < (1u << 22); ++spin) {
                if (*counter >= (int)live_splits) {
                    ok = 1;
                    break;
                }
                __nanosleep(20);
            }
            *arrival = ok;
            // the last folder to have seen the full count leaves both counters at zero
            if (ok && atomicAdd(ticket + 1, 1) == (int)folders - 1) {
                ticket[1] = 0;
                ticket[0] = 0;
            }
        }
        __syncthreads();
        if (!*arrival) {
            if (threadIdx.x == 0) atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
            return;
        }
        __threadfence();
        for (unsigned int v = split; v < min((unsigned int)VT, vectors); v += folders) {
            const unsigned int row = v / group, qhead = kv_head * group + v % group;
            const unsigned long long item = ((unsigned long long)b * p.query_rows + row) * p.query_heads + qhead;
            fold_splits_128<kF32Warps, F32BlockSync>(p.partials + item * p.max_splits * (kF32HeadDim + 2ull), live_splits,
                                                     fold_scratch, fold_row, threadIdx.x);
            const float value = fold_row[d];
            if (!isfinite(value) || !(fold_row[kF32HeadDim + 1] > 0.0f)) atomicCAS(p.status, 0, YVX_STATUS_NONFINITE);
            store_output(p.output, p.output_dtype, item * kF32HeadDim + d, value);
            __syncthreads();
        }
        return;
    }
    if (threadIdx.x == 0) {
        const int taken = atomicAdd(ticket, 1);
        *arrival = taken == (int)live_splits - 1;
        if (*arrival) *ticket = 0;  // left at zero for the next call
    }
    __syncthreads();
    if (!*arrival) return;
    __threadfence();
    for (unsigned int v = 0; v < min((unsigned int)VT, vectors); ++v) {
        const unsigned int row = v / group, qhead = kv_head * group + v % group;
        const unsigned long long item = ((unsigned long long)b * p.query_rows + row) * p.query_heads + qhead;
        fold_splits_128<kF32Warps, F32BlockSync>(p.partials + item * p.max_splits * (kF32HeadDim + 2ull), live_splits,
                                                 fold_scratch, fold_row, threadIdx.x);
        const float value = fold_row[d];
        if (!isfinite(value) || !(fold_row[kF32HeadDim + 1] > 0.0f)) atomicCAS(p.status, 0, YVX_STATUS_NONFINITE);
        store_output(p.output, p.output_dtype, item * kF32HeadDim + d, value);
        __syncthreads();
    }
}

// ---- host side ------------------------------------------------------------------

typedef CUresult (*F32EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                     const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                     const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static F32EncodeTiledFn f32_encode_entry()
{
    static F32EncodeTiledFn entry = nullptr;
    static bool resolved = false;
    if (!resolved) {
        void *symbol = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &query) ==
                cudaSuccess &&
            query == cudaDriverEntryPointSuccess)
            entry = reinterpret_cast<F32EncodeTiledFn>(symbol);
        resolved = true;
    }
    return entry;
}

// 4-D f32 map {128 dims, a, b, session}; the 16-token dimension is whichever of
// the two middle dimensions has the token stride. No swizzle: a row is 512 bytes.
static bool f32_encode(CUtensorMap *map, const void *base, unsigned long long token_stride,
                       unsigned long long head_stride, unsigned long long session_stride,
                       unsigned long long tokens, unsigned long long heads, unsigned long long sessions,
                       bool head_first)
{
    F32EncodeTiledFn encode = f32_encode_entry();
    if (!encode) return false;
    const unsigned long long tb = token_stride * 4ull, hb = head_stride * 4ull;
    unsigned long long sb = session_stride * 4ull;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (tb & 15ull) || (hb & 15ull) || (sb & 15ull) || !tb || !hb)
        return false;
    if (sessions <= 1ull || !sb) {
        if (sessions > 1ull) return false;
        sessions = 1ull;
        sb = ((head_first ? tb * tokens : hb * heads) + 15ull) & ~15ull;
    }
    cuuint64_t dims[4] = {kF32HeadDim, head_first ? heads : tokens, head_first ? tokens : heads, sessions};
    cuuint64_t strides[3] = {head_first ? hb : tb, head_first ? tb : hb, sb};
    cuuint32_t box[4] = {kF32HeadDim, head_first ? 1u : (cuuint32_t)kF32Sub, head_first ? (cuuint32_t)kF32Sub : 1u, 1};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    for (int i = 0; i < 3; ++i)
        if (strides[i] >= (1ull << 40)) return false;
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void *>(base), dims, strides, box,
                  elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Shapes this kernel takes (also used by the split planner).
bool gqa_decode_f32_admits(const yvx_gqa_problem &p)
{
    if (p.head_dim != (unsigned)kF32HeadDim || p.query_dtype != YVEX_DTYPE_F32 || p.kv_dtype != YVEX_DTYPE_F32 ||
        p.block_table || p.partial_output || p.kv_position_base || !p.kv_heads || p.query_heads % p.kv_heads)
        return false;
    if (p.query_head_stride && p.query_head_stride != p.head_dim) return false;
    const unsigned int vectors = p.query_rows * (p.query_heads / p.kv_heads);
    if (vectors == 0u || vectors > 8u) return false;
    if ((reinterpret_cast<uintptr_t>(p.query) & 15u) || (p.query_row_stride & 3ull) || (p.query_session_stride & 3ull))
        return false;
    return p.kv_tokens_max <= kF32MaxSplits * (unsigned)(kF32MaxSubs * kF32Sub);
}

// Chunk that puts two CTAs on every SM in a single wave: a multiple of 16 tokens, at most 112.
void gqa_decode_f32_plan(yvx_gqa_problem *p, int sm_count)
{
    const unsigned long long lanes = (unsigned long long)p->sessions * p->kv_heads;
    const unsigned long long target = 2ull * (unsigned long long)(sm_count > 0 ? sm_count : 148);
    unsigned long long splits = lanes ? target / lanes : 1ull;
    if (splits < 1ull) splits = 1ull;
    unsigned long long chunk = ((unsigned long long)p->kv_tokens_max + splits - 1ull) / splits;
    chunk = ((chunk + kF32Sub - 1ull) / kF32Sub) * kF32Sub;
    if (chunk < (unsigned)kF32Sub) chunk = kF32Sub;
    if (chunk > (unsigned)(kF32MaxSubs * kF32Sub)) chunk = kF32MaxSubs * kF32Sub;
    p->chunk_tokens = (unsigned int)chunk;
    p->max_splits = (p->kv_tokens_max + p->chunk_tokens - 1u) / p->chunk_tokens;
    if (!p->max_splits) p->max_splits = 1u;
}

// Returns 1 when the launch was made (a combine follows when the KV was split),
// 0 when the shape is not this kernel's, negative on a launch error.
int gqa_decode_f32_launch(const yvx_gqa_problem &p, cudaStream_t stream)
{
    if (!gqa_decode_f32_admits(p) || p.chunk_tokens % kF32Sub || p.chunk_tokens > (unsigned)(kF32MaxSubs * kF32Sub))
        return 0;
    const bool head_first = p.key_head_stride < p.key_token_stride;
    if ((p.value_head_stride < p.value_token_stride) != head_first) return 0;
    F32Maps maps;
    if (!f32_encode(&maps.key, p.key, p.key_token_stride, p.key_head_stride, p.key_session_stride,
                    p.kv_tokens_max, p.kv_heads, p.sessions, head_first) ||
        !f32_encode(&maps.value, p.value, p.value_token_stride, p.value_head_stride, p.value_session_stride,
                    p.kv_tokens_max, p.kv_heads, p.sessions, head_first))
        return 0;
    const unsigned int vectors = p.query_rows * (p.query_heads / p.kv_heads);
    const dim3 grid(p.max_splits, p.kv_heads, p.sessions);
    cudaError_t error;
    const bool fold_here = p.tickets && p.max_splits > 1u;
    // per device, once: attributes and resident-CTA capacities of both instantiations
    static int configured_device = -1, resident[2] = {0, 0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return YVEX_ERR_BACKEND;
    if (configured_device != device) {
        int sms = 0, coop = 0, per_sm[2] = {0, 0};
        const void *kernels[2] = {(const void *)gqa_decode_f32_kernel<4>, (const void *)gqa_decode_f32_kernel<8>};
        for (int i = 0; i < 2; ++i) {
            error = cudaFuncSetAttribute(kernels[i], cudaFuncAttributeMaxDynamicSharedMemorySize, kF32SmemBytes);
            if (error == cudaSuccess)
                error = cudaFuncSetAttribute(kernels[i], cudaFuncAttributePreferredSharedMemoryCarveout, 100);
            if (error != cudaSuccess) return yvx_cuda_check(error, "gqa_decode_f32_kernel attribute");
        }
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
            cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm[0], gqa_decode_f32_kernel<4>, kF32Threads, kF32SmemBytes) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm[1], gqa_decode_f32_kernel<8>, kF32Threads, kF32SmemBytes) != cudaSuccess)
            return YVEX_ERR_BACKEND;
        resident[0] = coop ? sms * per_sm[0] : 0;
        resident[1] = coop ? sms * per_sm[1] : 0;
        configured_device = device;
    }
    if (fold_here && (unsigned long long)grid.x * grid.y * grid.z <= (unsigned long long)resident[vectors <= 4u ? 0 : 1]) {
        // every CTA resident at once (the planner's single wave): a cooperative launch lets the
        // group's own CTAs fold side by side; a grid that does not fit folds in its last arrivals
        const void *kernel = vectors <= 4u ? (const void *)gqa_decode_f32_kernel<4> : (const void *)gqa_decode_f32_kernel<8>;
        yvx_gqa_problem problem = p;
        F32Maps tensor_maps = maps;
        int major = head_first ? 1 : 0, cooperative = 1;
        void *args[] = {&problem, &tensor_maps, &major, &cooperative};
        error = cudaLaunchCooperativeKernel(kernel, grid, dim3(kF32Threads, 1, 1), args, kF32SmemBytes, stream);
        if (error != cudaSuccess) return yvx_cuda_check(error, "gqa_decode_f32_kernel (cooperative)");
        return 2;
    }
    if (vectors <= 4u) {
        gqa_decode_f32_kernel<4><<<grid, kF32Threads, kF32SmemBytes, stream>>>(p, maps, head_first ? 1 : 0, 0);
    } else {
        gqa_decode_f32_kernel<8><<<grid, kF32Threads, kF32SmemBytes, stream>>>(p, maps, head_first ? 1 : 0, 0);
    }
    const int rc = yvx_cuda_check(cudaGetLastError(), "gqa_decode_f32_kernel");
    // with tickets the kernel has folded its splits itself: the output is final
    return rc != 0 ? rc : (p.tickets && p.max_splits > 1u ? 2 : 1);
}

}  // namespace yvx
