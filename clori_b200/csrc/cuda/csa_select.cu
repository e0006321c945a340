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
// problem: 64-bit keys of (inverted ordered score, row index), smallest first. Row
// index order is position order because positions are required to increase.
#include "common.cuh"

namespace yvx {

constexpr int kCsaScoreThreads = 256;  // two warps per scheduler hide the fixed FP64 and shared-memory latencies
constexpr unsigned int kCsaHeadSlots = 64;  // heads <= 64; unused slots hold zeros
constexpr int kCsaSortThreads = 1024;
constexpr int kCsaSortKeys = 4096;  // keys one CTA ranks at a time
constexpr unsigned long long kCsaAbsent = ~0ull;

__device__ __forceinline__ bool csa_candidate(unsigned long long position, unsigned long long ratio,
                                              unsigned long long query_position)
{
    return position <= query_position && position <= ~0ull - ratio + 1ull &&
           position + ratio - 1ull <= query_position;
}

// Scores. grid: x = CTAs striding over row tiles, y = token; 8 warps. A warp owns all 64
// head slots x 2*RT rows of the tile: lane = head lane (16) + 16 * row lane (2), a thread
// accumulates heads {hl, hl+16, hl+32, hl+48} x RT rows, so one step of the lane loop costs
// 4 + RT shared-memory reads for 4*RT fused multiply-adds and the FP64 pipe is the limit.
// The query and the tile's keys are widened to double once, in shared memory (pitches
// hd+1 and hd+2 doubles keep the 16 head lanes and the 2 row lanes on distinct banks).
// Arithmetic order is the reference's: per (row, head) the lanes in order (the product of
// two floats is exact in double, so a fused multiply-add rounds once exactly like the
// reference's multiply-then-add), clamp at zero, then per row the heads in order with a
// rounded multiply by the weight and a rounded add, then the two scalings.
template <int RT>
__global__ void __launch_bounds__(kCsaScoreThreads)
csa_score_kernel(const yvx_csa_select_args a, const double inv_sqrt_dim, const double inv_sqrt_heads)
{
    constexpr unsigned int kTileRows = (kCsaScoreThreads / 32) * 2 * RT;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const unsigned int heads = a.heads, hd = a.head_dim;
    const unsigned int qp = hd + 1u, kp = max((hd + 3u) & ~1u, kCsaHeadSlots + 2u), dp = kCsaHeadSlots + 1u;
    double *q = reinterpret_cast<double *>(smem_raw);           // [64][qp]
    double *keys = q + kCsaHeadSlots * qp;                      // [kTileRows][kp]; reused as dots [kTileRows][dp]
    __shared__ unsigned char visible[kTileRows];
    const unsigned long long token = blockIdx.y;
    const unsigned long long query_position = a.phase_start_position + token;
    const float *query = a.query + token * heads * hd;
    const float *weights = a.weights + token * heads;
    bool finite = true, query_finite = true, any_candidate = false;
    for (unsigned int i0 = threadIdx.x; i0 < kCsaHeadSlots * hd; i0 += 8u * blockDim.x) {
        float v[8];  // eight loads in flight per thread
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const unsigned int i = i0 + u * blockDim.x;
            v[u] = i < heads * hd ? query[i] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const unsigned int i = i0 + u * blockDim.x;
            if (i < kCsaHeadSlots * hd) {
                query_finite = query_finite && isfinite(v[u]);
                q[(i / hd) * qp + i % hd] = (double)v[u];
            }
        }
    }
    const unsigned int warp = threadIdx.x >> 5, hl = threadIdx.x & 15u, rl = (threadIdx.x >> 4) & 1u;
    // the two row lanes take alternate rows, one key pitch apart: distinct banks in one read
    const unsigned int row0 = warp * 2u * RT + rl;
    const unsigned long long tiles = (a.rows + kTileRows - 1u) / kTileRows;
    // The tile after the current one travels through registers while the current one is
    // being scored, so its load latency hides behind the FP64 work. kPrefetch float4 per
    // thread cover the tile when hd <= 128 (vector path: hd and key_stride multiples of 4).
    constexpr unsigned int kPrefetch = kTileRows * 128u / 4u / kCsaScoreThreads;
    const bool vector_path = (hd & 3u) == 0u && (a.key_stride & 3ull) == 0ull && hd <= 128u &&
                             (reinterpret_cast<unsigned long long>(a.keys) & 15ull) == 0ull;
    const unsigned int quads = hd >> 2;  // float4 per row
    float4 pre[kPrefetch];
    unsigned long long pre_position = 0ull, pre_before = 0ull;  // positions[row], positions[row - 1]
    // Volatile loads: they must be issued here, ahead of the scoring loop, not sunk to their use.
    auto prefetch = [&](unsigned long long tile) {
        const unsigned long long first = tile * kTileRows;
        if (threadIdx.x < kTileRows && tile < tiles && first + threadIdx.x < a.rows) {
            const unsigned long long *p = a.positions + first + threadIdx.x;
            asm volatile("ld.global.nc.u64 %0, [%1];" : "=l"(pre_position) : "l"(p));
            if (first + threadIdx.x > 0ull) asm volatile("ld.global.nc.u64 %0, [%1];" : "=l"(pre_before) : "l"(p - 1));
        }
        if (!vector_path) return;
#pragma unroll
        for (unsigned int i = 0; i < kPrefetch; ++i) {
            const unsigned int slot = threadIdx.x + i * kCsaScoreThreads;
            const unsigned int r = slot / quads, c = slot % quads;
            pre[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (tile < tiles && r < kTileRows && first + r < a.rows) {
                const float4 *p = reinterpret_cast<const float4 *>(a.keys + (first + r) * a.key_stride) + c;
                asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(pre[i].x), "=f"(pre[i].y), "=f"(pre[i].z), "=f"(pre[i].w) : "l"(p));
            }
        }
    };
    float weight[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const unsigned int h = hl + 16u * j;
        weight[j] = h < heads ? weights[h] : 0.0f;
    }
    prefetch(blockIdx.x);
    for (unsigned long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const unsigned long long first = tile * kTileRows;
        __syncthreads();  // the previous tile's sums are done with the shared region; q is written
        if (threadIdx.x < kTileRows) {
            const unsigned long long row = first + threadIdx.x;
            bool candidate = false;
            if (row < a.rows) {
                if (row > 0ull && pre_before >= pre_position) atomicCAS(a.status, 0, YVX_STATUS_CONTRACT);
                candidate = csa_candidate(pre_position, a.ratio, query_position);
            }
            visible[threadIdx.x] = candidate;
        }
        __syncthreads();
        if (vector_path) {
#pragma unroll
            for (unsigned int i = 0; i < kPrefetch; ++i) {
                const unsigned int slot = threadIdx.x + i * kCsaScoreThreads;
                const unsigned int r = slot / quads, c = slot % quads;
                if (r < kTileRows) {
                    float4 k = pre[i];
                    if (visible[r]) {
                        finite = finite && isfinite(k.x) && isfinite(k.y) && isfinite(k.z) && isfinite(k.w);
                        any_candidate = true;
                    } else {
                        k = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    }
                    double2 *dst = reinterpret_cast<double2 *>(keys + r * kp + 4u * c);  // kp is even
                    dst[0] = make_double2((double)k.x, (double)k.y);
                    dst[1] = make_double2((double)k.z, (double)k.w);
                }
            }
        } else {
            for (unsigned int i = threadIdx.x; i < kTileRows * hd; i += blockDim.x) {
                const unsigned int r = i / hd, lane = i % hd;
                float k = 0.0f;
                if (visible[r]) {
                    k = __ldg(a.keys + (first + r) * a.key_stride + lane);
                    finite = finite && isfinite(k);
                    any_candidate = true;
                }
                keys[r * kp + lane] = (double)k;
            }
        }
        prefetch(tile + gridDim.x);
        __syncthreads();
        double acc[4][RT];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int r = 0; r < RT; ++r) acc[j][r] = 0.0;
        const double *qh = q + hl * qp, *kr = keys + row0 * kp;
#pragma unroll 2
        for (unsigned int lane = 0; lane < hd; ++lane) {
            double qv[4], kv[RT];
#pragma unroll
            for (int j = 0; j < 4; ++j) qv[j] = qh[j * 16u * qp + lane];
#pragma unroll
            for (int r = 0; r < RT; ++r) kv[r] = kr[2u * r * kp + lane];
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int r = 0; r < RT; ++r) acc[j][r] = fma(qv[j], kv[r], acc[j][r]);
        }
        __syncthreads();  // every warp is done with the keys
        double *dots = keys;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const unsigned int h = hl + 16u * j;
            finite = finite && isfinite(weight[j]);
#pragma unroll
            for (int r = 0; r < RT; ++r)
                dots[(row0 + 2u * r) * dp + h] = __dmul_rn(acc[j][r] < 0.0 ? 0.0 : acc[j][r], (double)weight[j]);
        }
        __syncthreads();
        if (threadIdx.x < kTileRows && visible[threadIdx.x]) {
            double score = 0.0;
            for (unsigned int h = 0; h < heads; ++h) score = __dadd_rn(score, dots[threadIdx.x * dp + h]);
            score = __dmul_rn(score, inv_sqrt_dim);
            score = __dmul_rn(score, inv_sqrt_heads);
            finite = finite && isfinite(score);
            a.scores[token * a.rows + first + threadIdx.x] = __double2float_rn(score);
        }
    }
    // the reference inspects the query and the weights only while it scores a candidate
    if (__syncthreads_or(any_candidate) && (!finite || !query_finite)) atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
}

// Ascending key order = the reference's ranked order: higher score first (+0 and -0
// equal), equal scores by lower row index (= lower position).
__device__ __forceinline__ unsigned long long csa_key(float score, unsigned int row)
{
    unsigned int u = score == 0.0f ? 0u : __float_as_uint(score);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // ascending in score
    return ((unsigned long long)(~u) << 32) | row;
}

// Ranking. A CTA of 1024 threads holds 4096 keys, four per thread, in registers.
// The k smallest are found without sorting everything: an 8-bit radix select from the
// top byte down finds the k-th smallest key exactly (keys are unique: the low word is
// the row), the keys up to it are compacted into shared memory, and only those k keys
// are sorted, and only by the launch that publishes (earlier levels pass sets on).
struct csa_rank_shared {
    unsigned long long keys[1024];  // the kept keys
    unsigned int histogram[256];
    unsigned int digit, rank, kept, in_digit;
    unsigned long long found;
};

// The need-th smallest (1-based) of the CTA's keys; need <= number of keys below kCsaAbsent.
__device__ __forceinline__ unsigned long long csa_kth_smallest(const unsigned long long (&e)[4], unsigned int need,
                                                               csa_rank_shared &sh)
{
    const unsigned int lane = threadIdx.x & 31u;
    unsigned long long prefix = 0ull, decided = 0ull;
    for (int shift = 56; shift >= 0; shift -= 8) {
        if (threadIdx.x < 256u) sh.histogram[threadIdx.x] = 0u;
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const bool in = (e[i] & decided) == prefix;
            const unsigned int digit = (unsigned int)(e[i] >> shift) & 255u;
            const unsigned int active = __ballot_sync(0xffffffffu, in);
            if (in) {  // one shared-memory add per distinct digit in the warp
                const unsigned int peers = __match_any_sync(active, digit);
                if (lane == (unsigned int)__ffs(peers) - 1u) atomicAdd(&sh.histogram[digit], (unsigned int)__popc(peers));
            }
        }
        __syncthreads();
        if (threadIdx.x < 32u) {  // lane owns bins [8 lane, 8 lane + 8)
            unsigned int bins[8], sum = 0u;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                bins[j] = sh.histogram[8u * lane + j];
                sum += bins[j];
            }
            unsigned int inclusive = sum;
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1) {
                const unsigned int below = __shfl_up_sync(0xffffffffu, inclusive, offset);
                if (lane >= (unsigned int)offset) inclusive += below;
            }
            unsigned int run = inclusive - sum;
            if (run < need && need <= inclusive) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (need > run && need <= run + bins[j]) {
                        sh.digit = 8u * lane + j;
                        sh.rank = need - run;
                        sh.in_digit = bins[j];
                    }
                    run += bins[j];
                }
            }
        }
        __syncthreads();
        prefix |= (unsigned long long)sh.digit << shift;
        decided |= 0xffull << shift;
        need = sh.rank;
        if (sh.in_digit == 1u && shift > 0) {  // one key left under this prefix: it is the answer
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if ((e[i] & decided) == prefix) sh.found = e[i];
            __syncthreads();
            return sh.found;
        }
    }
    return prefix;
}

// Ascending bitonic sort of sh.keys[0 .. n), n a power of two in [4, 1024]. Thread t < n/4
// keeps four consecutive keys in registers: strides 1 and 2 are exchanges inside the
// thread, strides 4..64 reach a lane of the same warp by shuffle, strides >= 128 go through
// shared memory. Every thread of the CTA calls it (the barriers are CTA-wide).
__device__ __forceinline__ void csa_sort_kept(csa_rank_shared &sh, unsigned int n)
{
    const unsigned int t = threadIdx.x;
    const bool holder = 4u * t < n;
    const bool in_warp = t < max(n >> 2, 32u);  // whole warps take part in the shuffles
    unsigned long long e[4] = {kCsaAbsent, kCsaAbsent, kCsaAbsent, kCsaAbsent};
    if (holder) {
#pragma unroll
        for (int i = 0; i < 4; ++i) e[i] = sh.keys[4u * t + i];
    }
    auto order = [](unsigned long long &x, unsigned long long &y, bool ascending) {
        const unsigned long long small = x < y ? x : y, large = x < y ? y : x;
        x = ascending ? small : large;
        y = ascending ? large : small;
    };
    for (unsigned int size = 2; size <= n; size <<= 1) {
        for (unsigned int stride = size >> 1; stride > 0; stride >>= 1) {
            if (stride >= 128u) {
                __syncthreads();  // partners have read the previous contents
                if (holder) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) sh.keys[4u * t + i] = e[i];
                }
                __syncthreads();
                if (holder) {
                    const unsigned int partner = t ^ (stride >> 2);
                    const bool keep_small = (((4u * t) & stride) == 0u) == (((4u * t) & size) == 0u);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const unsigned long long other = sh.keys[4u * partner + i];
                        e[i] = keep_small == (e[i] < other) ? e[i] : other;
                    }
                }
            } else if (!in_warp) {
                continue;
            } else if (stride >= 4u) {
                const bool keep_small = (((4u * t) & stride) == 0u) == (((4u * t) & size) == 0u);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const unsigned long long other = __shfl_xor_sync(0xffffffffu, e[i], stride >> 2);
                    e[i] = keep_small == (e[i] < other) ? e[i] : other;
                }
            } else if (stride == 2u) {
                const bool ascending = ((4u * t) & size) == 0u;  // size >= 4 here
                order(e[0], e[2], ascending);
                order(e[1], e[3], ascending);
            } else {
                const bool first = size == 2u ? true : ((4u * t) & size) == 0u;
                const bool second = size == 2u ? false : first;
                order(e[0], e[1], first);
                order(e[2], e[3], second);
            }
        }
    }
    __syncthreads();
    if (holder) {
#pragma unroll
        for (int i = 0; i < 4; ++i) sh.keys[4u * t + i] = e[i];
    }
    __syncthreads();
}

// The shared tail of both ranking kernels: keeps the smallest min(topk, present) of the
// CTA's keys. publish: sorts them and writes the token's lists. Otherwise writes the set
// (unsorted, padded with kCsaAbsent to topk keys) to `out`.
__device__ __forceinline__ void csa_keep_smallest(const yvx_csa_select_args &a, const unsigned long long (&e)[4],
                                                  unsigned long long token, bool publish, unsigned long long *out,
                                                  csa_rank_shared &sh)
{
    unsigned int present = 0u;
#pragma unroll
    for (int i = 0; i < 4; ++i) present += (unsigned int)__syncthreads_count(e[i] != kCsaAbsent);
    const unsigned int keep = min(a.topk, present);
    if (threadIdx.x == 0) sh.kept = 0u;
    if (keep == 0u) {  // identical on every thread
        if (publish) {
            if (threadIdx.x == 0) a.selected_count[token] = 0ull;
        } else {
            for (unsigned int i = threadIdx.x; i < a.topk; i += blockDim.x) out[i] = kCsaAbsent;
        }
        return;
    }
    const unsigned long long threshold = csa_kth_smallest(e, keep, sh);  // its barriers also publish sh.kept = 0
    const unsigned int lane = threadIdx.x & 31u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const bool kept = e[i] <= threshold;
        const unsigned int mask = __ballot_sync(0xffffffffu, kept);
        unsigned int base = 0u;
        if (lane == 0u && mask) base = atomicAdd(&sh.kept, (unsigned int)__popc(mask));
        base = __shfl_sync(0xffffffffu, base, 0);
        if (kept) sh.keys[base + __popc(mask & ((1u << lane) - 1u))] = e[i];
    }
    __syncthreads();
    if (!publish) {
        for (unsigned int i = threadIdx.x; i < a.topk; i += blockDim.x) out[i] = i < keep ? sh.keys[i] : kCsaAbsent;
        return;
    }
    unsigned int n = 4u;
    while (n < keep) n <<= 1;
    for (unsigned int i = keep + threadIdx.x; i < n; i += blockDim.x) sh.keys[i] = kCsaAbsent;
    __syncthreads();
    csa_sort_kept(sh, n);
    for (unsigned int i = threadIdx.x; i < keep; i += blockDim.x)
        a.selected[token * a.topk_capacity + i] = sh.keys[i] & 0xffffffffull;
    if (threadIdx.x == 0) a.selected_count[token] = (unsigned long long)keep;
}

// First level. grid: x = chunk of 4096 rows, y = token.
__global__ void __launch_bounds__(kCsaSortThreads)
csa_rank_rows_kernel(const yvx_csa_select_args a, unsigned long long *level, unsigned int chunks)
{
    __shared__ csa_rank_shared sh;
    const unsigned long long token = blockIdx.y;
    const unsigned long long query_position = a.phase_start_position + token;
    const unsigned long long first = (unsigned long long)blockIdx.x * kCsaSortKeys + 4ull * threadIdx.x;
    unsigned long long e[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const unsigned long long row = first + i;
        e[i] = kCsaAbsent;
        if (row < a.rows && csa_candidate(a.positions[row], a.ratio, query_position))
            e[i] = csa_key(a.scores[token * a.rows + row], (unsigned int)row);
    }
    csa_keep_smallest(a, e, token, chunks == 1u,
                      chunks == 1u ? nullptr : level + (token * chunks + blockIdx.x) * a.topk, sh);
}

// Later levels. grid: x = group of fan_in key sets, y = token. Keeps the smallest topk of
// up to fan_in sets of topk keys (fan_in * topk <= 4096).
__global__ void __launch_bounds__(kCsaSortThreads)
csa_rank_lists_kernel(const yvx_csa_select_args a, const unsigned long long *from, unsigned int lists,
                      unsigned long long *to, unsigned int groups, unsigned int fan_in)
{
    __shared__ csa_rank_shared sh;
    const unsigned long long token = blockIdx.y;
    const unsigned int first_list = blockIdx.x * fan_in;
    const unsigned int mine_lists = min(fan_in, lists - first_list);
    const unsigned long long *source = from + (token * lists + first_list) * a.topk;
    unsigned long long e[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const unsigned int slot = 4u * threadIdx.x + i;
        e[i] = slot < mine_lists * a.topk ? source[slot] : kCsaAbsent;
    }
    csa_keep_smallest(a, e, token, groups == 1u,
                      groups == 1u ? nullptr : to + (token * groups + blockIdx.x) * a.topk, sh);
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
        // 8 rows per thread while the widened tile fits beside the widened query, else 2
        const bool wide = a->head_dim <= 128u;
        const unsigned int tile_rows = (yvx::kCsaScoreThreads / 32) * 2 * (wide ? 8 : 2);
        const unsigned int even = (a->head_dim + 3u) & ~1u;  // an even pitch >= head_dim + 2
        const unsigned int kp = even > yvx::kCsaHeadSlots + 2u ? even : yvx::kCsaHeadSlots + 2u;
        const size_t smem = ((size_t)yvx::kCsaHeadSlots * (a->head_dim + 1u) + (size_t)tile_rows * kp) * sizeof(double);
        auto kernel = wide ? yvx::csa_score_kernel<8> : yvx::csa_score_kernel<2>;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return yvx_cuda_check(e, "csa_score_kernel attribute");
        const unsigned long long tiles = (a->rows + tile_rows - 1u) / tile_rows;
        int sms = 148;
        int device = 0;
        if (cudaGetDevice(&device) == cudaSuccess)
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        // a CTA widens the query once and then strides over tiles; spread tokens over the SMs
        unsigned long long per_token = ((unsigned long long)sms + a->token_count - 1ull) / a->token_count;
        if (per_token > tiles) per_token = tiles;
        const dim3 grid((unsigned int)per_token, (unsigned int)a->token_count);
        kernel<<<grid, yvx::kCsaScoreThreads, smem, s>>>(*a, 1.0 / sqrt((double)a->head_dim),
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
