// Sparse index selection for the shared-latent attention stage: the score of every
// compressed row against a token's index queries, and the ranked top-k rows.
//
// Replaces the reference's yvex_attention_csa_select (src/graph/attention.c:369-497)
// and yvex_attention_topk_select (src/graph/numeric.c:1086-1150), which walk the
// candidates serially on the host and rank them with two qsort calls. The scores
// keep the reference's double-precision arithmetic in the reference's order (a
// product of two floats is exact in double, so the lane loop is one rounded add per
// lane; the sum over heads is a rounded multiply and a rounded add per head), which
// makes every float score bit-equal to the CPU result and the ranking a pure integer
// problem: a 64-bit key of (inverted ordered score, row index) sorted ascending. Row
// index order is position order because positions are required to increase.
#include "common.cuh"

namespace yvx {

constexpr int kCsaScoreThreads = 256;
constexpr int kCsaRowsPerBlock = 32;
constexpr int kCsaSortThreads = 1024;
constexpr int kCsaSortKeys = 4096;  // keys one CTA ranks at a time
constexpr unsigned long long kCsaAbsent = ~0ull;

__device__ __forceinline__ bool csa_candidate(unsigned long long position, unsigned long long ratio,
                                              unsigned long long query_position)
{
    return position <= query_position && position <= ~0ull - ratio + 1ull &&
           position + ratio - 1ull <= query_position;
}

// grid: x = block of kCsaRowsPerBlock rows, y = token. threads: heads x (256 / heads) rows.
// smem: query [heads][head_dim + 1] floats, dots [rows in flight][heads] doubles.
__global__ void __launch_bounds__(kCsaScoreThreads)
csa_score_kernel(const yvx_csa_select_args a, const double inv_sqrt_dim, const double inv_sqrt_heads)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const unsigned int heads = a.heads, hd = a.head_dim, pitch = hd + 1u;
    float *q = reinterpret_cast<float *>(smem_raw);
    double *dots = reinterpret_cast<double *>(smem_raw + (((size_t)heads * pitch * 4u + 7u) & ~(size_t)7u));
    const unsigned long long token = blockIdx.y;
    const unsigned long long query_position = a.phase_start_position + token;
    const float *query = a.query + token * heads * hd;
    const float *weights = a.weights + token * heads;
    bool finite = true, query_finite = true, any_candidate = false;
    for (unsigned int i = threadIdx.x; i < heads * hd; i += blockDim.x) {
        const float v = query[i];
        query_finite = query_finite && isfinite(v);
        q[(i / hd) * pitch + i % hd] = v;
    }
    __syncthreads();
    const unsigned int rows_in_flight = blockDim.x / heads;
    const unsigned int slot = threadIdx.x / heads, head = threadIdx.x % heads;
    const unsigned long long first = (unsigned long long)blockIdx.x * kCsaRowsPerBlock;
    for (unsigned int base = 0; base < (unsigned int)kCsaRowsPerBlock; base += rows_in_flight) {
        const unsigned long long row = first + base + slot;
        bool candidate = false;
        if (base + slot < (unsigned int)kCsaRowsPerBlock && row < a.rows) {
            const unsigned long long position = a.positions[row];
            if (row > 0ull && a.positions[row - 1ull] >= position && head == 0u)
                atomicCAS(a.status, 0, YVX_STATUS_CONTRACT);
            candidate = csa_candidate(position, a.ratio, query_position);
        }
        if (candidate) {
            const float *key = a.keys + row * a.key_stride;
            const float *qh = q + head * pitch;
            double dot = 0.0;
            for (unsigned int lane = 0; lane < hd; ++lane) {
                const float k = __ldg(key + lane);
                finite = finite && isfinite(k);
                dot = __dadd_rn(dot, __dmul_rn((double)qh[lane], (double)k));
            }
            dots[slot * heads + head] = dot < 0.0 ? 0.0 : dot;
        }
        any_candidate = __syncthreads_or(candidate) || any_candidate;
        if (candidate && head == 0u) {
            double score = 0.0;
            for (unsigned int h = 0; h < heads; ++h) {
                const float w = weights[h];
                finite = finite && isfinite(w);
                score = __dadd_rn(score, __dmul_rn(dots[slot * heads + h], (double)w));
            }
            score = __dmul_rn(score, inv_sqrt_dim);
            score = __dmul_rn(score, inv_sqrt_heads);
            finite = finite && isfinite(score);
            a.scores[token * a.rows + row] = __double2float_rn(score);
        }
        __syncthreads();
    }
    // the reference inspects the query only while it scores a candidate
    if (!finite || (any_candidate && !query_finite)) atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
}

// Ascending key order = the reference's ranked order: higher score first (+0 and -0
// equal), equal scores by lower row index (= lower position).
__device__ __forceinline__ unsigned long long csa_key(float score, unsigned int row)
{
    unsigned int u = score == 0.0f ? 0u : __float_as_uint(score);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // ascending in score
    return ((unsigned long long)(~u) << 32) | row;
}

__device__ __forceinline__ void csa_sort_4096(unsigned long long *keys)
{
    for (unsigned int size = 2; size <= (unsigned int)kCsaSortKeys; size <<= 1) {
        for (unsigned int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (unsigned int t = threadIdx.x; t < (unsigned int)kCsaSortKeys / 2; t += blockDim.x) {
                const unsigned int low = 2u * t - (t & (stride - 1u));
                const unsigned int high = low + stride;
                const bool ascending = (low & size) == 0u;
                const unsigned long long x = keys[low], y = keys[high];
                if ((x > y) == ascending) {
                    keys[low] = y;
                    keys[high] = x;
                }
            }
        }
    }
    __syncthreads();
}

// First level. grid: x = chunk of 4096 rows, y = token. Ranks the chunk's candidates and
// keeps its best `keep` keys: straight into selected[] when the chunk is the only one,
// else into level storage [token][chunk][keep].
__global__ void __launch_bounds__(kCsaSortThreads)
csa_rank_rows_kernel(const yvx_csa_select_args a, unsigned long long *level, unsigned int chunks)
{
    __shared__ unsigned long long keys[kCsaSortKeys];
    const unsigned long long token = blockIdx.y;
    const unsigned long long query_position = a.phase_start_position + token;
    const unsigned long long first = (unsigned long long)blockIdx.x * kCsaSortKeys;
    for (unsigned int i = threadIdx.x; i < (unsigned int)kCsaSortKeys; i += blockDim.x) {
        const unsigned long long row = first + i;
        unsigned long long key = kCsaAbsent;
        if (row < a.rows && csa_candidate(a.positions[row], a.ratio, query_position))
            key = csa_key(a.scores[token * a.rows + row], (unsigned int)row);
        keys[i] = key;
    }
    csa_sort_4096(keys);
    if (chunks == 1u) {
        int mine = 0;
        for (unsigned int i = threadIdx.x; i < a.topk; i += blockDim.x)
            if (keys[i] != kCsaAbsent) {
                a.selected[token * a.topk_capacity + i] = keys[i] & 0xffffffffull;
                ++mine;
            }
        // topk <= 1024 = blockDim.x: every thread holds at most one key
        const int count = __syncthreads_count(mine);
        if (threadIdx.x == 0) a.selected_count[token] = (unsigned long long)count;
    } else {
        unsigned long long *out = level + (token * chunks + blockIdx.x) * a.topk;
        for (unsigned int i = threadIdx.x; i < a.topk; i += blockDim.x) out[i] = keys[i];
    }
}

// Later levels. grid: x = group of fan_in lists, y = token. Merges up to fan_in ranked
// lists of `topk` keys (fan_in * topk <= 4096) by ranking them together.
__global__ void __launch_bounds__(kCsaSortThreads)
csa_rank_lists_kernel(const yvx_csa_select_args a, const unsigned long long *from, unsigned int lists,
                      unsigned long long *to, unsigned int groups, unsigned int fan_in)
{
    __shared__ unsigned long long keys[kCsaSortKeys];
    const unsigned long long token = blockIdx.y;
    const unsigned int first_list = blockIdx.x * fan_in;
    const unsigned int mine_lists = min(fan_in, lists - first_list);
    const unsigned long long *source = from + (token * lists + first_list) * a.topk;
    for (unsigned int i = threadIdx.x; i < (unsigned int)kCsaSortKeys; i += blockDim.x)
        keys[i] = i < mine_lists * a.topk ? source[i] : kCsaAbsent;
    csa_sort_4096(keys);
    if (groups == 1u) {
        int mine = 0;
        for (unsigned int i = threadIdx.x; i < a.topk; i += blockDim.x)
            if (keys[i] != kCsaAbsent) {
                a.selected[token * a.topk_capacity + i] = keys[i] & 0xffffffffull;
                ++mine;
            }
        const int count = __syncthreads_count(mine);
        if (threadIdx.x == 0) a.selected_count[token] = (unsigned long long)count;
    } else {
        unsigned long long *out = to + (token * groups + blockIdx.x) * a.topk;
        for (unsigned int i = threadIdx.x; i < a.topk; i += blockDim.x) out[i] = keys[i];
    }
}

static unsigned long long csa_chunks(unsigned long long rows)
{
    return (rows + kCsaSortKeys - 1) / kCsaSortKeys;
}

}  // namespace yvx

// Two level buffers (ping-pong), each [token][lists][topk] keys; the first level has
// the most lists.
extern "C" unsigned long long yvx_cuda_csa_select_workspace_bytes(unsigned long long rows,
                                                                  unsigned long long token_count,
                                                                  unsigned int topk)
{
    const unsigned long long chunks = yvx::csa_chunks(rows);
    if (chunks <= 1ull) return 16ull;
    return 2ull * token_count * chunks * topk * sizeof(unsigned long long);
}

extern "C" int yvx_cuda_csa_select(const yvx_csa_select_args *a, void *stream, unsigned int *launches)
{
    if (launches) *launches = 0u;
    if (!a || !a->keys || !a->positions || !a->query || !a->weights || !a->scores || !a->selected ||
        !a->selected_count || !a->status || !a->rows || !a->heads || !a->head_dim || !a->topk ||
        !a->ratio || !a->token_count || a->key_stride < a->head_dim || a->topk_capacity < a->topk)
        return YVEX_ERR_INVALID_ARG;
    if (a->heads > 64u || a->head_dim > 256u || a->topk > 1024u || a->rows >= (1ull << 31) ||
        a->token_count > 65535ull)
        return YVEX_ERR_UNSUPPORTED;
    const unsigned long long chunks = yvx::csa_chunks(a->rows);
    if (chunks > 1ull && !a->workspace) return YVEX_ERR_INVALID_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    unsigned int count = 0u;
    {
        const unsigned int threads = (yvx::kCsaScoreThreads / a->heads) * a->heads;
        const size_t query_bytes = ((size_t)a->heads * (a->head_dim + 1u) * 4u + 7u) & ~(size_t)7u;
        const size_t smem = query_bytes + (size_t)(threads / a->heads) * a->heads * sizeof(double);
        if (smem > 48u * 1024u) {
            cudaError_t e = cudaFuncSetAttribute(yvx::csa_score_kernel,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return yvx_cuda_check(e, "csa_score_kernel attribute");
        }
        const dim3 grid((unsigned int)((a->rows + yvx::kCsaRowsPerBlock - 1) / yvx::kCsaRowsPerBlock),
                        (unsigned int)a->token_count);
        yvx::csa_score_kernel<<<grid, threads, smem, s>>>(*a, 1.0 / sqrt((double)a->head_dim),
                                                          1.0 / sqrt((double)a->heads));
        ++count;
    }
    unsigned long long *ping = (unsigned long long *)a->workspace;
    unsigned long long *pong = ping ? ping + a->token_count * chunks * a->topk : nullptr;
    yvx::csa_rank_rows_kernel<<<dim3((unsigned int)chunks, (unsigned int)a->token_count),
                                yvx::kCsaSortThreads, 0, s>>>(*a, ping, (unsigned int)chunks);
    ++count;
    const unsigned int fan_in = (unsigned int)yvx::kCsaSortKeys / a->topk;  // >= 4
    unsigned int lists = (unsigned int)chunks;
    while (lists > 1u) {
        const unsigned int groups = (lists + fan_in - 1u) / fan_in;
        yvx::csa_rank_lists_kernel<<<dim3(groups, (unsigned int)a->token_count), yvx::kCsaSortThreads, 0, s>>>(
            *a, ping, lists, pong, groups, fan_in);
        ++count;
        unsigned long long *swap = ping;
        ping = pong;
        pong = swap;
        lists = groups;
    }
    if (launches) *launches = count;
    return yvx_cuda_check(cudaGetLastError(), "csa_select");
}
