// General split-KV grouped-query attention for sm_100a: any head_dim <= 256,
// F32 or BF16 operands, contiguous strided KV rows or a block table. This is
// the exact-F32 contract's kernel and the path every shape without a
// specialised kernel takes. It is bandwidth-shaped: one warp streams KV rows
// with coalesced 128-byte loads, lanes own head dimensions, every KV row is
// read once for the whole query-head group and all verify rows, and the
// softmax statistics live in registers.
//
// Replaces yvex_gqa_f32_body (src/backend/cuda/transformer_kernels.cu:137-238
// in the reference), which walks all KV rows serially in one CTA per query
// head with two barriers per row and re-reads each KV head once per query
// head.
#include "combine.cuh"

namespace yvx {

constexpr int kGenericThreads = 128;
constexpr int kGenericWarps = kGenericThreads / 32;

// 2^x, max error 2 ulp over the normal range (ex2.approx), -inf -> 0.
__device__ __forceinline__ float exp2_fast(float x)
{
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct SessionView {
    unsigned int kv_tokens;
    long long query_start_local;  // query_start - kv_position_base (may be negative)
};

__device__ __forceinline__ SessionView session_view(const yvx_gqa_problem &p, unsigned int b)
{
    SessionView s;
    s.kv_tokens = admitted_kv_tokens(p.kv_tokens, b, p.kv_tokens_uniform, p.kv_tokens_max, p.status);
    long long start;
    if (p.query_start)
        start = (long long)p.query_start[b];
    else if (p.query_start_from_end)
        start = (long long)p.kv_position_base + (long long)s.kv_tokens - (long long)p.query_rows;
    else
        start = (long long)p.query_start_uniform;
    s.query_start_local = start - (long long)p.kv_position_base;
    return s;
}

// Address of one KV row of one head. A block-table entry outside the pool is a
// contract failure: it is recorded in the status word and the row reads pool
// block 0 instead of an arbitrary address (the result is discarded by the host).
template <typename KT>
__device__ __forceinline__ const KT *kv_row(const void *base, const yvx_gqa_problem &p,
                                            unsigned int b, unsigned int token,
                                            unsigned int kv_head, bool is_key)
{
    const unsigned long long token_stride = is_key ? p.key_token_stride : p.value_token_stride;
    const unsigned long long head_stride = is_key ? p.key_head_stride : p.value_head_stride;
    unsigned long long offset;
    if (p.block_table) {
        const unsigned int block = token / p.block_tokens;
        const unsigned int within = token - block * p.block_tokens;
        int pool_block = p.block_table[(unsigned long long)b * p.block_table_stride + block];
        if (pool_block < 0 || (unsigned int)pool_block >= p.pool_blocks) {
            atomicCAS(p.status, 0, YVX_STATUS_CONTRACT);
            pool_block = 0;
        }
        offset = (unsigned long long)pool_block * (is_key ? p.key_block_stride : p.value_block_stride) +
                 (unsigned long long)within * token_stride;
    } else {
        offset = (unsigned long long)b * (is_key ? p.key_session_stride : p.value_session_stride) +
                 (unsigned long long)token * token_stride;
    }
    return reinterpret_cast<const KT *>(base) + offset + (unsigned long long)kv_head * head_stride;
}

// grid: x = (kv_head * vector_tiles + tile) * max_splits + split, z = session (a prefill-sized
// call has more (head, tile) pairs than grid.y admits, so they share x with the splits).
// A "vector" is one (query row, query head of the group) pair; a CTA carries
// VT of them so each KV row it loads serves VT dot products.
template <typename QT, typename KT, int SLOTS, int VT>
__global__ void __launch_bounds__(kGenericThreads)
gqa_split_generic_kernel(const yvx_gqa_problem p)
{
    constexpr int HD_CAP = SLOTS * 32;
    if (p.gate && *p.gate != p.gate_value) return;  // the other kernel of the pair owns this problem
    __shared__ float sm_acc[kGenericWarps][VT][HD_CAP];
    __shared__ float sm_m[kGenericWarps][VT];
    __shared__ float sm_l[kGenericWarps][VT];

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned int group = p.query_heads / p.kv_heads;
    const unsigned int vectors = p.query_rows * group;
    const unsigned int tiles = (vectors + VT - 1) / VT;
    const unsigned int head_tile = blockIdx.x / p.max_splits, split = blockIdx.x % p.max_splits;
    const unsigned int kv_head = head_tile / tiles, tile = head_tile % tiles;
    const unsigned int b = blockIdx.z;
    const unsigned int hd = p.head_dim;
    const SessionView s = session_view(p, b);

    const unsigned int t0 = split * p.chunk_tokens;
    if (t0 >= s.kv_tokens) return;
    unsigned int t1 = min(s.kv_tokens, t0 + p.chunk_tokens);

    // Per-vector query registers and visibility limits.
    float q[VT][SLOTS];
    long long limit[VT];
    bool live[VT];
    long long tile_limit = -1;
#pragma unroll
    for (int i = 0; i < VT; ++i) {
        const unsigned int v = tile * VT + i;
        live[i] = v < vectors;
        const unsigned int row = live[i] ? v / group : 0u;
        const unsigned int qhead = kv_head * group + (live[i] ? v % group : 0u);
        limit[i] = !live[i] ? -1
                   : p.causal ? s.query_start_local + (long long)row
                              : (long long)s.kv_tokens - 1;
        tile_limit = limit[i] > tile_limit ? limit[i] : tile_limit;
        const QT *qp = reinterpret_cast<const QT *>(p.query) +
                       (unsigned long long)b * p.query_session_stride +
                       (unsigned long long)row * p.query_row_stride +
                       (unsigned long long)qhead * (p.query_head_stride ? p.query_head_stride : hd);
#pragma unroll
        for (int sl = 0; sl < SLOTS; ++sl) {
            const unsigned int d = lane + 32u * sl;
            // scores are kept in log2 units: q carries scale * log2(e)
            q[i][sl] = (live[i] && d < hd) ? load_as_float(qp + d) * (p.scale * 1.4426950408889634f) : 0.0f;
        }
    }
    if (tile_limit + 1 < (long long)t1) t1 = tile_limit + 1 > 0 ? (unsigned int)(tile_limit + 1) : 0u;

    float m[VT], l[VT], acc[VT][SLOTS];
#pragma unroll
    for (int i = 0; i < VT; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.0f;
#pragma unroll
        for (int sl = 0; sl < SLOTS; ++sl) acc[i][sl] = 0.0f;
    }

    // Each warp takes U consecutive tokens per pass and issues all of their K
    // and V loads before any arithmetic, so 2*U rows per warp are in flight.
    constexpr int U = SLOTS <= 4 ? 4 : 2;
    for (unsigned int base = t0 + warp * U; base < t1; base += kGenericWarps * U) {
        float kc[U][SLOTS], vc[U][SLOTS];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned int t = base + u;
            const bool in_range = t < t1;
            const KT *kp = kv_row<KT>(p.key, p, b, in_range ? t : t0, kv_head, true);
            const KT *vp = kv_row<KT>(p.value, p, b, in_range ? t : t0, kv_head, false);
#pragma unroll
            for (int sl = 0; sl < SLOTS; ++sl) {
                const unsigned int d = lane + 32u * sl;
                kc[u][sl] = (in_range && d < hd) ? load_as_float(kp + d) : 0.0f;
                vc[u][sl] = (in_range && d < hd) ? load_as_float(vp + d) : 0.0f;
            }
        }
        float dot[U][VT];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int i = 0; i < VT; ++i) {
                float partial = 0.0f;
#pragma unroll
                for (int sl = 0; sl < SLOTS; ++sl) partial = fmaf(q[i][sl], kc[u][sl], partial);
                dot[u][i] = partial;
            }
#pragma unroll
        for (int offset = 16; offset; offset >>= 1)
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int i = 0; i < VT; ++i)
                    dot[u][i] += __shfl_xor_sync(0xffffffffu, dot[u][i], offset);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned int t = base + u;
            if (t >= t1) break;
#pragma unroll
            for (int i = 0; i < VT; ++i) {
                if ((long long)t <= limit[i]) {
                    // dot is identical on every lane, so both branches are warp-uniform.
                    if (dot[u][i] <= m[i]) {
                        const float weight = exp2_fast(dot[u][i] - m[i]);
                        l[i] += weight;
#pragma unroll
                        for (int sl = 0; sl < SLOTS; ++sl)
                            acc[i][sl] = fmaf(weight, vc[u][sl], acc[i][sl]);
                    } else {
                        const float keep = exp2_fast(m[i] - dot[u][i]);  // 0 when m is -inf
                        l[i] = fmaf(l[i], keep, 1.0f);
#pragma unroll
                        for (int sl = 0; sl < SLOTS; ++sl)
                            acc[i][sl] = fmaf(acc[i][sl], keep, vc[u][sl]);
                        m[i] = dot[u][i];
                    }
                }
            }
        }
    }

    // Merge the four warps' running states.
#pragma unroll
    for (int i = 0; i < VT; ++i) {
        if (lane == 0) {
            sm_m[warp][i] = m[i];
            sm_l[warp][i] = l[i];
        }
#pragma unroll
        for (int sl = 0; sl < SLOTS; ++sl) sm_acc[warp][i][lane + 32 * sl] = acc[i][sl];
    }
    __syncthreads();

    // The main loop is over: let the combine kernel's launch overlap the epilogue.
    pdl_launch_dependents();
    const bool direct = p.max_splits == 1u;
    for (int i = 0; i < VT; ++i) {
        const unsigned int v = tile * VT + i;
        if (v >= vectors) break;
        const unsigned int row = v / group, qhead = kv_head * group + v % group;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kGenericWarps; ++w) mm = fmaxf(mm, sm_m[w][i]);
        float scale_w[kGenericWarps], ll = 0.0f;
#pragma unroll
        for (int w = 0; w < kGenericWarps; ++w) {
            scale_w[w] = sm_m[w][i] == -INFINITY ? 0.0f : exp2_fast(sm_m[w][i] - mm);
            ll += sm_l[w][i] * scale_w[w];
        }
        const float inverse = ll > 0.0f ? 1.0f / ll : 0.0f;
        const unsigned long long item =
            ((unsigned long long)b * p.query_rows + row) * p.query_heads + qhead;
        if (!YVX_CHECKED_INDEX(item < (unsigned long long)p.sessions * p.query_rows * p.query_heads &&
                                   split < p.max_splits && qhead < p.query_heads && row < p.query_rows, p.status))
            continue;
        for (unsigned int d = threadIdx.x; d < hd; d += kGenericThreads) {
            float o = 0.0f;
#pragma unroll
            for (int w = 0; w < kGenericWarps; ++w) o += sm_acc[w][i][d] * scale_w[w];
            if (direct && !p.partial_output) {
                const float value = o / ll;
                if (!isfinite(value)) atomicCAS(p.status, 0, YVX_STATUS_NONFINITE);
                store_output(p.output, p.output_dtype, item * hd + d, value);
            } else {
                float *part = direct ? p.partial_output + item * (hd + 2ull)
                                     : p.partials + (item * p.max_splits + split) * (hd + 2ull);
                part[d] = o * inverse;
                if (d == 0) {
                    part[hd] = mm * 0.6931471805599453f;  // natural-log units
                    part[hd + 1] = ll;
                }
            }
        }
    }
}

__global__ void __launch_bounds__(kCombineWarps * 32)
gqa_combine_kernel(const yvx_gqa_problem p)
{
    pdl_wait();  // the split kernel's partials must be complete and visible
    if (p.gate && *p.gate != p.gate_value) return;
    const unsigned long long item = blockIdx.x;
    const unsigned int b = (unsigned int)(item / ((unsigned long long)p.query_rows * p.query_heads));
    const unsigned int hd = p.head_dim;
    const SessionView s = session_view(p, b);
    // never more parts than the scratch holds per item, whatever the stored length says
    const unsigned int splits = min((s.kv_tokens + p.chunk_tokens - 1u) / p.chunk_tokens, p.max_splits);
    combine_parts(p.partials + item * p.max_splits * (hd + 2ull), splits, hd + 2u, hd, p.output,
                  p.output_dtype, item * hd,
                  p.partial_output ? p.partial_output + item * (hd + 2ull) : nullptr, p.status);
}

// Combine of externally gathered partials: part j of item i starts at
// parts + i * item_stride + j * part_stride (floats) and holds (o[hd], m, l).
__global__ void __launch_bounds__(kCombineWarps * 32)
lse_combine_kernel(const float *parts, unsigned int part_count, unsigned int hd,
                   unsigned long long item_stride, unsigned long long part_stride, void *output,
                   int output_dtype, int *status)
{
    pdl_wait();
    const unsigned long long item = blockIdx.x;
    combine_parts(parts + item * item_stride, part_count, (unsigned int)part_stride, hd, output,
                  output_dtype, item * hd, nullptr, status);
}

// One WARP per item, for many items with few parts each (latent decode: 8192
// items x 9 parts): no shared memory, no block barrier, parts folded in index
// order, four loaded at a time.
__global__ void __launch_bounds__(kCombineWarps * 32)
lse_combine_warp_kernel(const float *__restrict__ parts, unsigned int items, unsigned int part_count,
                        unsigned int hd, unsigned long long item_stride,
                        unsigned long long part_stride, void *output, int output_dtype, int *status)
{
    pdl_wait();
    const unsigned int lane = threadIdx.x & 31u;
    const unsigned long long item = (unsigned long long)blockIdx.x * kCombineWarps + (threadIdx.x >> 5);
    if (item >= items) return;
    const float *base = parts + item * item_stride;
    float acc[8], run_max = -INFINITY, run_sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    for (unsigned int j0 = 0; j0 < part_count; j0 += kCombineBatch) {
        float mj[kCombineBatch], lj[kCombineBatch], oj[kCombineBatch][8];
#pragma unroll
        for (int u = 0; u < kCombineBatch; ++u) {
            const bool live = j0 + u < part_count;
            const float *part = base + (unsigned long long)(live ? j0 + u : j0) * part_stride;
            mj[u] = live ? part[hd] : -INFINITY;
            lj[u] = part[hd + 1];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const unsigned int d = lane + 32u * i;
                oj[u][i] = d < hd ? part[d] : 0.0f;
            }
        }
#pragma unroll
        for (int u = 0; u < kCombineBatch; ++u) {
            if (mj[u] == -INFINITY) continue;
            const float new_max = fmaxf(run_max, mj[u]);
            const float keep = expf(run_max - new_max);
            const float weight = lj[u] * expf(mj[u] - new_max);
            run_sum = fmaf(run_sum, keep, weight);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(acc[i], keep, oj[u][i] * weight);
            run_max = new_max;
        }
    }
    bool finite = true;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const unsigned int d = lane + 32u * i;
        if (d >= hd) continue;
        const float value = acc[i] / run_sum;
        finite = finite && isfinite(value);
        store_output(output, output_dtype, item * hd + d, value);
    }
    if (!finite) atomicCAS(status, 0, YVX_STATUS_NONFINITE);
}

template <typename QT, typename KT, int SLOTS>
static int launch_generic(const yvx_gqa_problem &p, cudaStream_t stream)
{
    const unsigned int group = p.query_heads / p.kv_heads;
    const unsigned int vectors = p.query_rows * group;
    const unsigned int per_cta = vectors <= 4u ? 4u : 8u;
    const unsigned long long ctas =
        (unsigned long long)p.kv_heads * ((vectors + per_cta - 1u) / per_cta) * p.max_splits;
    if (ctas > 0x7fffffffull || p.sessions > 65535u) {
        yvx_cuda_set_error_text("the attention grid exceeds the launch limits (2^31-1 CTAs per session, 65535 sessions)");
        return YVEX_ERR_BOUNDS;
    }
    const dim3 grid((unsigned int)ctas, 1, p.sessions);
    if (per_cta == 4u)
        gqa_split_generic_kernel<QT, KT, SLOTS, 4><<<grid, kGenericThreads, 0, stream>>>(p);
    else
        gqa_split_generic_kernel<QT, KT, SLOTS, 8><<<grid, kGenericThreads, 0, stream>>>(p);
    return yvx_cuda_check(cudaGetLastError(), "gqa_split_generic_kernel");
}

template <typename QT, typename KT>
static int launch_generic_slots(const yvx_gqa_problem &p, cudaStream_t stream)
{
    if (p.head_dim <= 128u) return launch_generic<QT, KT, 4>(p, stream);
    return launch_generic<QT, KT, 8>(p, stream);
}

// Launches the general attention kernel only (no combine).
int gqa_generic_main_launch(const yvx_gqa_problem &p, cudaStream_t stream)
{
    if (p.head_dim == 0u || p.head_dim > 256u) return YVEX_ERR_UNSUPPORTED;
    if (p.query_dtype == YVEX_DTYPE_F32 && p.kv_dtype == YVEX_DTYPE_F32)
        return launch_generic_slots<float, float>(p, stream);
    if (p.query_dtype == YVEX_DTYPE_BF16 && p.kv_dtype == YVEX_DTYPE_BF16)
        return launch_generic_slots<__nv_bfloat16, __nv_bfloat16>(p, stream);
    if (p.query_dtype == YVEX_DTYPE_F32 && p.kv_dtype == YVEX_DTYPE_BF16)
        return launch_generic_slots<float, __nv_bfloat16>(p, stream);
    return YVEX_ERR_UNSUPPORTED;
}

// Folds the per-split partials; needed whenever max_splits > 1.
int gqa_combine_launch(const yvx_gqa_problem &p, cudaStream_t stream)
{
    const unsigned long long items = (unsigned long long)p.sessions * p.query_rows * p.query_heads;
    // Launched so that its scheduling overlaps the tail of the split kernel
    // before it in the stream; the kernel itself waits for that kernel's results.
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned int)items, 1, 1);
    config.blockDim = dim3(kCombineWarps * 32, 1, 1);
    config.dynamicSmemBytes = 0;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    const cudaError_t launched = cudaLaunchKernelEx(&config, gqa_combine_kernel, p);
    if (launched != cudaSuccess) return yvx_cuda_check(launched, "gqa_combine_kernel");
    return yvx_cuda_check(cudaGetLastError(), "gqa_combine_kernel");
}

}  // namespace yvx

namespace yvx {

// Launches the gathered-partials combine as a programmatic dependent of the
// kernel before it in the stream (the kernels wait for that kernel's results
// themselves). Many items with few parts each go one warp per item.
static int lse_combine_launch(const float *parts, unsigned int items, unsigned int part_count,
                              unsigned int hd, unsigned long long item_stride,
                              unsigned long long part_stride, void *output, int output_dtype,
                              int *status, cudaStream_t stream)
{
    cudaLaunchConfig_t config = {};
    config.blockDim = dim3(kCombineWarps * 32, 1, 1);
    config.dynamicSmemBytes = 0;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    cudaError_t launched;
    if (items >= 1024u && part_count <= 32u && hd <= 256u) {
        config.gridDim = dim3((items + kCombineWarps - 1u) / kCombineWarps, 1, 1);
        launched = cudaLaunchKernelEx(&config, lse_combine_warp_kernel, parts, items, part_count, hd,
                                      item_stride, part_stride, output, output_dtype, status);
    } else {
        config.gridDim = dim3(items, 1, 1);
        launched = cudaLaunchKernelEx(&config, lse_combine_kernel, parts, part_count, hd, item_stride,
                                      part_stride, output, output_dtype, status);
    }
    if (launched != cudaSuccess) return yvx_cuda_check(launched, "lse_combine_kernel");
    return yvx_cuda_check(cudaGetLastError(), "lse_combine_kernel");
}

}  // namespace yvx

extern "C" int yvx_cuda_lse_combine(const float *parts, unsigned int items,
                                    unsigned int part_count, unsigned int head_dim,
                                    void *output, int output_dtype, int *status, void *stream)
{
    if (!parts || !items || !part_count || !head_dim || head_dim > 256u || !output || !status)
        return YVEX_ERR_INVALID_ARG;
    return yvx::lse_combine_launch(parts, items, part_count, head_dim,
                                   (unsigned long long)part_count * (head_dim + 2ull), head_dim + 2ull,
                                   output, output_dtype, status, (cudaStream_t)stream);
}

extern "C" int yvx_cuda_lse_combine_strided(const float *parts, unsigned int items,
                                            unsigned int part_count, unsigned int head_dim,
                                            unsigned long long item_stride,
                                            unsigned long long part_stride, void *output,
                                            int output_dtype, int *status, void *stream)
{
    if (!parts || !items || !part_count || !head_dim || head_dim > 256u || !output || !status ||
        part_stride < head_dim + 2ull || part_stride > 0xffffffffull)
        return YVEX_ERR_INVALID_ARG;
    return yvx::lse_combine_launch(parts, items, part_count, head_dim, item_stride, part_stride, output,
                                   output_dtype, status, (cudaStream_t)stream);
}
