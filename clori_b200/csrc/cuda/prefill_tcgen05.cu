// Causal / full prefill attention on the 5th-generation tensor cores (sm_100a):
// bf16 Q/K/V, head_dim 128, f32 softmax and accumulation. One CTA owns TWO
// 128-row query tiles (A, B: 256 consecutive rows) of one query head: every
// K / V tile brought into shared memory feeds twice the tensor work, and while
// one tile is in its softmax phase the other is in its matrix phase.
//
//   warp 8      TMA producer: both Q tiles once, then 128-token K and V tiles
//               into two-stage rings (128-byte swizzle, full/empty mbarriers)
//   warp 9      allocates tensor memory and issues tcgen05.mma; all 32 lanes run
//               the loop converged and one elected lane issues, which keeps the
//               descriptors in uniform registers:
//               S_x = Q_x K^T (A, B in shared memory, 8 k-steps of 128x128x16)
//               O_x += P_x V  (A = P in tensor memory, B = V tile, MN-major)
//               in the order PV_A(j) QK_A(j+1) PV_B(j) QK_B(j+1)
//   warps 0-3   softmax of tile A, warps 4-7 softmax of tile B: thread r owns
//               query row r == TMEM lane r. It reads its 128 scores with
//               tcgen05.ld, keeps the running max / sum in registers, rescales O
//               in tensor memory only when the max grew by more than 2^8 (the
//               stale max keeps P <= 256, exact in f32/bf16 range), and writes P
//               as packed bf16 back into the score columns with tcgen05.st in two
//               halves of 64 tokens, each handed to the MMA warp as soon as it is
//               stored, so P V starts while the second half is exponentiated.
// Tensor memory map (512 columns): S_A [0,128) S_B [128,256) O_A [256,384)
// O_B [384,512); P_x aliases the first 64 columns of S_x.
//
// Replaces the reference's tiled MHA prefill (src/backend/cuda/transformer.c:
// 493-677: cuBLAS SGEMM QK^T, softmax kernel, SGEMM PV over a materialised
// [H, 512, Tkv] f32 score buffer) and its per-row GQA kernel for prefill shapes.
#include "tcgen05.cuh"

namespace yvx {

constexpr int kPfM = 128;          // query rows per tile (two tiles per CTA)
constexpr int kPfN = 128;          // KV tokens per tile
constexpr int kPfD = 128;          // head_dim
constexpr int kPfStages = 2;
constexpr int kPfThreads = 320;
constexpr int kPfHalfBytes = kPfM * 64 * 2;        // one [128][64] bf16 swizzled half tile
constexpr int kPfTileBytes = 2 * kPfHalfBytes;     // 32 KB
constexpr int kPfSmemBytes = (2 + 2 * kPfStages) * kPfTileBytes + 1024 + 512;
constexpr float kPfRescaleThreshold = 8.0f;        // log2 units
constexpr uint32_t kPfTmemColumns = 512;

struct PrefillMaps {
    CUtensorMap query, key, value;
};

struct PrefillBarriers {
    uint64_t q_full;
    uint64_t k_full[kPfStages], k_empty[kPfStages];
    uint64_t v_full[kPfStages], v_empty[kPfStages];
    uint64_t s_full[2], p_half[2][2], pv_done[2];  // per query tile; P is handed over in halves
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(PrefillBarriers) <= 512, "barrier block outgrew its shared-memory slot");

__device__ __forceinline__ void prefill_fail(const yvx_gqa_problem &p, PrefillBarriers *bars)
{
    atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
    bars->abort_flag = 1;
}

// Number of 128-token KV tiles the rows [row0, row0 + 128) of the query can see.
__device__ __forceinline__ unsigned int prefill_tile_count(const yvx_gqa_problem &p,
                                                           unsigned int row0, long long query_start,
                                                           unsigned int kv_tokens)
{
    if (row0 >= p.query_rows) return 0u;
    long long visible_end = kv_tokens;
    if (p.causal) {
        const long long last = query_start + (long long)min(row0 + kPfM, p.query_rows);
        if (last < visible_end) visible_end = last;
    }
    return visible_end > 0 ? (unsigned int)((visible_end + kPfN - 1) / kPfN) : 0u;
}

// grid: one dimension. The (session, query head) lanes are taken in groups of `lane_group`
// whose K and V streams fit the L2 together (all of them when they do: grouped-query shapes;
// a few heads at a time for long multi-head prefills, where every head has its own K and V).
// Inside a group the pair of query tiles varies slowest, longest first, and the lane fastest,
// so the CTAs left for the tail are the short ones and neighbours share K / V.
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_tcgen05_kernel(const yvx_gqa_problem p, const __grid_constant__ PrefillMaps maps,
                       const int head_major, const unsigned int lane_group)
{
    extern __shared__ unsigned char smem_raw[];
    // uniform over the grid, before any barrier or tensor memory exists
    if (p.gate && *p.gate != p.gate_value) return;
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    unsigned char *q_tiles_smem = smem;                          // tile A, then tile B
    unsigned char *k_tiles = smem + 2 * kPfTileBytes;
    unsigned char *v_tiles = k_tiles + kPfStages * kPfTileBytes;
    PrefillBarriers *bars = reinterpret_cast<PrefillBarriers *>(v_tiles + kPfStages * kPfTileBytes);

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned int pairs = (p.query_rows + 2 * kPfM - 1) / (2 * kPfM);
    const unsigned int lanes_of_work = p.query_heads * p.sessions;
    const unsigned int within = blockIdx.x % (pairs * lane_group);
    const unsigned int work_lane = blockIdx.x / (pairs * lane_group) * lane_group + within % lane_group;
    if (work_lane >= lanes_of_work) return;  // the last group may be short; uniform over the CTA
    const unsigned int q0 = (pairs - 1u - within / lane_group) * 2u * kPfM;
    const unsigned int qhead = work_lane % p.query_heads;
    const unsigned int b = work_lane / p.query_heads;
    const unsigned int kv_head = qhead / (p.query_heads / p.kv_heads);
    const unsigned int kv_tokens = admitted_kv_tokens(p.kv_tokens, b, p.kv_tokens_uniform, p.kv_tokens_max, p.status);
    const long long query_start =
        p.query_start ? (long long)p.query_start[b]
                      : (p.query_start_from_end ? (long long)kv_tokens - (long long)p.query_rows
                                                : (long long)p.query_start_uniform);
    const unsigned int tiles_a = prefill_tile_count(p, q0, query_start, kv_tokens);
    const unsigned int tiles_b = prefill_tile_count(p, q0 + kPfM, query_start, kv_tokens);
    const unsigned int tiles = max(tiles_a, tiles_b);

    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, 1);
        for (int i = 0; i < kPfStages; ++i) {
            mbar_init(&bars->k_full[i], 1);
            mbar_init(&bars->k_empty[i], 1);
            mbar_init(&bars->v_full[i], 1);
            mbar_init(&bars->v_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->s_full[i], 1);
            mbar_init(&bars->p_half[i][0], kPfM);
            mbar_init(&bars->p_half[i][1], kPfM);
            mbar_init(&bars->pv_done[i], 1);
        }
        bars->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 9) {
        tmem_alloc(&bars->tmem_base, kPfTmemColumns);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 8) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0 && tiles) {
            mbar_expect_tx(&bars->q_full, (tiles_b ? 2u : 1u) * kPfTileBytes);
            for (unsigned int x = 0; x < (tiles_b ? 2u : 1u); ++x) {
                unsigned char *qd = q_tiles_smem + x * kPfTileBytes;
                const int row = (int)(q0 + x * kPfM);
                tma_load_4d(qd, &maps.query, &bars->q_full, 0, (int)qhead, row, (int)b);
                tma_load_4d(qd + kPfHalfBytes, &maps.query, &bars->q_full, 64, (int)qhead, row, (int)b);
            }
            for (unsigned int j = 0; j < tiles; ++j) {
                const unsigned int stage = j % kPfStages;
                const uint32_t parity = ((j / kPfStages) - 1u) & 1u;
                const int token = (int)(j * kPfN);
                const int c1 = head_major ? (int)kv_head : token;
                const int c2 = head_major ? token : (int)kv_head;
                if (j >= (unsigned)kPfStages && !mbar_wait(&bars->k_empty[stage], parity)) {
                    prefill_fail(p, bars);
                    break;
                }
                unsigned char *kd = k_tiles + stage * kPfTileBytes;
                mbar_expect_tx(&bars->k_full[stage], kPfTileBytes);
                tma_load_4d(kd, &maps.key, &bars->k_full[stage], 0, c1, c2, (int)b);
                tma_load_4d(kd + kPfHalfBytes, &maps.key, &bars->k_full[stage], 64, c1, c2, (int)b);
                if (j >= (unsigned)kPfStages && !mbar_wait(&bars->v_empty[stage], parity)) {
                    prefill_fail(p, bars);
                    break;
                }
                unsigned char *vd = v_tiles + stage * kPfTileBytes;
                mbar_expect_tx(&bars->v_full[stage], kPfTileBytes);
                tma_load_4d(vd, &maps.value, &bars->v_full[stage], 0, c1, c2, (int)b);
                tma_load_4d(vd + kPfHalfBytes, &maps.value, &bars->v_full[stage], 64, c1, c2, (int)b);
            }
        }
    } else if (warp == 9) {
        // ------------------------------ MMA issuer --------------------------------
        // All 32 lanes run the loop converged; one elected lane issues each instruction.
        if (tiles) {
            constexpr uint32_t idesc_qk = idesc_bf16_f32(kPfM, kPfN, false);
            constexpr uint32_t idesc_pv = idesc_bf16_f32(kPfM, kPfD, true);
            const uint32_t q_addr = smem_u32(q_tiles_smem);
            const unsigned int tiles_x[2] = {tiles_a, tiles_b};
            // S_x(j) = Q_x K(j)^T; the K stage is known to be full.
            auto issue_qk = [&](unsigned int x, unsigned int j) {
                const uint32_t k_addr = smem_u32(k_tiles + (j % kPfStages) * kPfTileBytes);
                const uint32_t qa = q_addr + x * kPfTileBytes;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks >> 2) * kPfHalfBytes + (ks & 3) * 32;
                    tc_mma_ss_elect(tmem + x * kPfN, smem_desc_sw128(qa + off, 16, 1024),
                              smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk, ks ? 1u : 0u);
                }
                tc_commit_elect(&bars->s_full[x]);
            };
            // O_x += P_x(j) V(j); the V stage is known to be full.
            auto issue_pv = [&](unsigned int x, unsigned int j) -> bool {
                const uint32_t v_addr = smem_u32(v_tiles + (j % kPfStages) * kPfTileBytes);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    // The weights of the first 64 tokens arrive while the softmax warps
                    // are still exponentiating the last 64.
                    if (!__all_sync(0xffffffffu, mbar_wait(&bars->p_half[x][h], j & 1u))) return false;
                    tc_fence_after_sync();
#pragma unroll
                    for (int kk = 4 * h; kk < 4 * h + 4; ++kk)
                        tc_mma_ts_elect(tmem + (2 + x) * kPfN, tmem + x * kPfN + kk * 8,
                                        smem_desc_sw128(v_addr + kk * 2048, kPfHalfBytes, 1024),
                                        idesc_pv, (j || kk) ? 1u : 0u);
                }
                tc_commit_elect(&bars->pv_done[x]);
                return true;
            };
            bool ok = __all_sync(0xffffffffu, mbar_wait(&bars->q_full, 0));
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->k_full[0], 0));
            if (ok) {
                tc_fence_after_sync();
#pragma unroll
                for (unsigned int x = 0; x < 2; ++x)
                    if (tiles_x[x]) issue_qk(x, 0);
                tc_commit_elect(&bars->k_empty[0]);
            }
            for (unsigned int j = 0; ok && j < tiles; ++j) {
                const unsigned int stage = j % kPfStages, next = (j + 1) % kPfStages;
                const bool more = j + 1 < tiles;
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->v_full[stage], (j / kPfStages) & 1u));
                if (ok && more)
                    ok = __all_sync(0xffffffffu,
                                    mbar_wait(&bars->k_full[next], ((j + 1) / kPfStages) & 1u));
#pragma unroll
                for (unsigned int x = 0; x < 2; ++x) {
                    if (ok && j < tiles_x[x]) ok = issue_pv(x, j);
                    if (ok && j + 1 < tiles_x[x]) issue_qk(x, j + 1);
                }
                if (!ok) break;
                tc_commit_elect(&bars->v_empty[stage]);
                if (more) tc_commit_elect(&bars->k_empty[next]);
            }
            if (!ok && lane == 0) prefill_fail(p, bars);
        }
    } else {
        // ------------------------------ softmax warps -----------------------------
        const unsigned int x = warp >> 2;                 // 0: tile A, 1: tile B
        const unsigned int row = threadIdx.x & 127u;      // query row in the tile == TMEM lane
        const unsigned int my_tiles = x ? tiles_b : tiles_a;
        const uint32_t lane_base = tmem + (((warp & 3u) * 32u) << 16);
        const uint32_t s_col = lane_base + x * kPfN, o_col = lane_base + (2u + x) * kPfN;
        const long long qi = (long long)q0 + x * kPfM + row;
        long long row_limit = (long long)kv_tokens - 1;
        if (p.causal && query_start + qi < row_limit) row_limit = query_start + qi;
        const float sscale = p.scale * 1.4426950408889634f;
        float m_used = -INFINITY, l = 0.0f;
        bool ok = true;
        for (unsigned int j = 0; j < my_tiles; ++j) {
            if (!mbar_wait(&bars->s_full[x], j & 1u)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            uint32_t s[4][32];
#pragma unroll
            for (int i = 0; i < 4; ++i) tmem_ld32(s_col + 32 * i, s[i]);
            tmem_wait_ld();
            const long long k0 = (long long)j * kPfN;
            // Masked entries become -inf; the maximum runs over four independent
            // chains of three-input max instructions.
            if (k0 + kPfN - 1 > row_limit) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        if (k0 + 32 * i + c > row_limit) s[i][c] = 0xff800000u;
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int c = 0; c < 32; c += 2)
                    mx[(c >> 1) & 3] = max3(mx[(c >> 1) & 3], __uint_as_float(s[i][c]),
                                            __uint_as_float(s[i][c + 1]));
            const float row_max = max3(mx[0], mx[1], fmaxf(mx[2], mx[3]));
            const float m_tile = row_max * sscale;  // -inf stays -inf (sscale > 0)
            const bool grow = m_tile > m_used + kPfRescaleThreshold || m_used == -INFINITY;
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = fmaxf(m_used, m_tile);
                const float factor = m_new == -INFINITY ? 1.0f : exp2_approx(m_used - m_new);
                l *= factor;
                m_used = m_new;
                if (j > 0) {
                    // O may only be touched once the previous tile's P V has landed.
                    if (!mbar_wait(&bars->pv_done[x], (j - 1u) & 1u)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        uint32_t o[16];
                        tmem_ld16(o_col + 16 * i, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * factor);
                        tmem_st16(o_col + 16 * i, o);
                    }
                    tmem_wait_st();
                }
            }
            const float offset = m_used == -INFINITY ? 0.0f : -m_used;
            float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t packed[32];
#pragma unroll
                for (int i = 2 * h; i < 2 * h + 2; ++i)
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        const float p0 = exp2_approx(fmaf(__uint_as_float(s[i][c]), sscale, offset));
                        const float p1 = exp2_approx(fmaf(__uint_as_float(s[i][c + 1]), sscale, offset));
                        sum0 += p0;
                        sum1 += p1;
                        packed[(i & 1) * 16 + (c >> 1)] = pack_bf16(p0, p1);
                    }
                // Hand over the weights of tokens 64 * h .. 64 * h + 63.
                tmem_st32(s_col + 32 * h, packed);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&bars->p_half[x][h]);
            }
            l += sum0 + sum1;
        }
        // ------------------------------ epilogue ------------------------------------
        if (ok && my_tiles) ok = mbar_wait(&bars->pv_done[x], (my_tiles - 1u) & 1u);
        // Every lane takes part in the tensor-memory loads; only rows that exist store.
        const bool all_ok = __all_sync(0xffffffffu, ok);
        if (!all_ok) {
            prefill_fail(p, bars);
        } else {
            tc_fence_after_sync();
            const bool exists = qi < (long long)p.query_rows;
            const float inverse = 1.0f / l;  // l == 0 (nothing visible) publishes a non-finite row
            const unsigned long long item =
                (((unsigned long long)b * p.query_rows + (unsigned long long)(exists ? qi : 0)) *
                     p.query_heads + qhead) * kPfD;
            bool finite = my_tiles != 0u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t o[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) o[c] = 0u;
                if (my_tiles) {
                    tmem_ld32(o_col + 32 * i, o);
                    tmem_wait_ld();
                }
                float v[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    v[c] = __uint_as_float(o[c]) * inverse;
                    finite = finite && isfinite(v[c]);
                }
                if (!exists) continue;
                if (p.output_dtype == YVEX_DTYPE_BF16) {
                    uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<unsigned short *>(p.output) + item + 32 * i);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                        dst[q4] = make_uint4(pack_bf16(v[8 * q4], v[8 * q4 + 1]), pack_bf16(v[8 * q4 + 2], v[8 * q4 + 3]),
                                             pack_bf16(v[8 * q4 + 4], v[8 * q4 + 5]), pack_bf16(v[8 * q4 + 6], v[8 * q4 + 7]));
                } else {
                    float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.output) + item + 32 * i);
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4)
                        dst[q4] = make_float4(v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]);
                }
            }
            if (exists && !finite) atomicCAS(p.status, 0, YVX_STATUS_NONFINITE);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, kPfTmemColumns);
}

// ---- host side ------------------------------------------------------------------

typedef CUresult (*PfEncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                    const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                    const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PfEncodeTiledFn pf_encode_entry()
{
    static PfEncodeTiledFn entry = nullptr;
    static bool resolved = false;
    if (!resolved) {
        void *symbol = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &query) ==
                cudaSuccess &&
            query == cudaDriverEntryPointSuccess)
            entry = reinterpret_cast<PfEncodeTiledFn>(symbol);
        resolved = true;
    }
    return entry;
}

// 4-D bf16 map {128 elems, a, b, outer} with a 64 x (1|128) x (128|1) x 1 box: the
// 128-row dimension is whichever of the two middle dimensions is the token/row one.
static bool pf_encode(CUtensorMap *map, const void *base, unsigned long long row_stride,
                      unsigned long long head_stride, unsigned long long outer_stride,
                      unsigned long long rows, unsigned long long heads, unsigned long long outer,
                      bool head_first)
{
    PfEncodeTiledFn encode = pf_encode_entry();
    if (!encode) return false;
    const unsigned long long rb = row_stride * 2ull, hb = head_stride * 2ull;
    unsigned long long ob = outer_stride * 2ull;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (rb & 15ull) || (hb & 15ull) || (ob & 15ull) ||
        !rb || !hb)
        return false;
    if (outer <= 1ull || !ob) {
        if (outer > 1ull) return false;
        outer = 1ull;
        ob = ((head_first ? rb * rows : hb * heads) + 15ull) & ~15ull;
    }
    cuuint64_t dims[4] = {kPfD, head_first ? heads : rows, head_first ? rows : heads, outer};
    cuuint64_t strides[3] = {head_first ? hb : rb, head_first ? rb : hb, ob};
    cuuint32_t box[4] = {64, head_first ? 1u : (cuuint32_t)kPfM, head_first ? (cuuint32_t)kPfM : 1u, 1};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    for (int i = 0; i < 3; ++i)
        if (strides[i] >= (1ull << 40)) return false;
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides,
                  box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Returns 2 when the launch was made and the output is final (no combine), 0
// when the shape is not this kernel's, negative on a launch error.
int prefill_tcgen05_launch(const yvx_gqa_problem &p, cudaStream_t stream)
{
    if (p.head_dim != (unsigned)kPfD || p.query_dtype != YVEX_DTYPE_BF16 ||
        p.kv_dtype != YVEX_DTYPE_BF16 || p.block_table || p.partial_output || p.kv_position_base ||
        (p.output_dtype != YVEX_DTYPE_BF16 && p.output_dtype != YVEX_DTYPE_F32) ||
        (reinterpret_cast<uintptr_t>(p.output) & 15u) || p.query_heads % p.kv_heads)
        return 0;
    // Q rows are [row][head][dim]: the head dimension (stride head_dim) comes first.
    const bool kv_head_first = p.key_head_stride < p.key_token_stride;
    if ((p.value_head_stride < p.value_token_stride) != kv_head_first) return 0;
    PrefillMaps maps;
    if (!pf_encode(&maps.query, p.query, p.query_row_stride, kPfD, p.query_session_stride,
                   p.query_rows, p.query_heads, p.sessions, true) ||
        !pf_encode(&maps.key, p.key, p.key_token_stride, p.key_head_stride, p.key_session_stride,
                   p.kv_tokens_max, p.kv_heads, p.sessions, kv_head_first) ||
        !pf_encode(&maps.value, p.value, p.value_token_stride, p.value_head_stride,
                   p.value_session_stride, p.kv_tokens_max, p.kv_heads, p.sessions, kv_head_first))
        return 0;
    cudaError_t error = cudaFuncSetAttribute(prefill_tcgen05_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kPfSmemBytes);
    if (error != cudaSuccess) return yvx_cuda_check(error, "prefill_tcgen05_kernel attribute");
    // lanes whose K + V (bf16) fit half of the 126 MB L2 together form a group
    const unsigned long long lanes = (unsigned long long)p.query_heads * p.sessions;
    const unsigned long long group = p.query_heads / p.kv_heads;
    const unsigned long long stream_bytes = (unsigned long long)p.kv_tokens_max * kPfD * 2ull * 2ull;
    unsigned long long streams = stream_bytes ? (64ull << 20) / stream_bytes : lanes;
    if (streams < 1ull) streams = 1ull;
    unsigned long long lane_group = streams * group;
    if (lane_group > lanes) lane_group = lanes;
    const unsigned long long pairs = (p.query_rows + 2 * kPfM - 1) / (2 * kPfM);
    const unsigned long long ctas = (lanes + lane_group - 1ull) / lane_group * lane_group * pairs;
    if (ctas == 0ull || ctas > 0x7fffffffull) return 0;
    const dim3 grid((unsigned int)ctas, 1, 1);
    prefill_tcgen05_kernel<<<grid, kPfThreads, kPfSmemBytes, stream>>>(p, maps, kv_head_first ? 1 : 0,
                                                                       (unsigned int)lane_group);
    const int rc = yvx_cuda_check(cudaGetLastError(), "prefill_tcgen05_kernel");
    return rc != 0 ? rc : 2;
}

}  // namespace yvx
