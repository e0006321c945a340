// Causal / full prefill attention on the 5th-generation tensor cores (sm_100a):
// bf16 Q/K/V, head_dim 128, f32 softmax and accumulation, one 128-row query
// tile of one query head per CTA.
//
//   warp 4      TMA producer: the Q tile once, then 128-token K and V tiles into
//               two-stage rings (128-byte swizzle, full/empty mbarriers)
//   warp 5      allocates tensor memory and issues tcgen05.mma from one lane:
//               S = Q K^T  (A, B in shared memory, 8 k-steps of 128x128x16)
//               O += P V   (A = P in tensor memory, B = V tile, MN-major)
//   warps 0-3   softmax: thread r owns query row r == TMEM lane r. It reads its
//               128 scores with tcgen05.ld, keeps the running max / sum in
//               registers, rescales O in tensor memory only when the max grew by
//               more than 2^8 (the stale max keeps P <= 256, exact in f32/bf16
//               range), writes P as packed bf16 back into the score columns with
//               tcgen05.st, and hands it to the MMA warp.
// Two score buffers let S(j+1) be computed while softmax works on S(j).
// Tensor memory map (512 columns): S0 [0,128) S1 [128,256) O [256,384); P(j)
// aliases the first 64 columns of S(j%2).
//
// Replaces the reference's tiled MHA prefill (src/backend/cuda/transformer.c:
// 493-677: cuBLAS SGEMM QK^T, softmax kernel, SGEMM PV over a materialised
// [H, 512, Tkv] f32 score buffer) and its per-row GQA kernel for prefill shapes.
#include "tcgen05.cuh"

namespace yvx {

constexpr int kPfM = 128;          // query rows per CTA
constexpr int kPfN = 128;          // KV tokens per tile
constexpr int kPfD = 128;          // head_dim
constexpr int kPfStages = 2;
constexpr int kPfThreads = 192;
constexpr int kPfHalfBytes = kPfM * 64 * 2;        // one [128][64] bf16 swizzled half tile
constexpr int kPfTileBytes = 2 * kPfHalfBytes;     // 32 KB
constexpr int kPfSmemBytes = (1 + 2 * kPfStages) * kPfTileBytes + 1024 + 512;
constexpr float kPfRescaleThreshold = 8.0f;        // log2 units
constexpr uint32_t kPfTmemColumns = 512;

struct PrefillMaps {
    CUtensorMap query, key, value;
};

struct PrefillBarriers {
    uint64_t q_full;
    uint64_t k_full[kPfStages], k_empty[kPfStages];
    uint64_t v_full[kPfStages], v_empty[kPfStages];
    uint64_t s_full[2], p_full[2];
    uint64_t pv_done;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void prefill_fail(const yvx_gqa_problem &p, PrefillBarriers *bars)
{
    atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
    bars->abort_flag = 1;
}

// grid: x = query tile (longest first), y = query head, z = session.
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_tcgen05_kernel(const yvx_gqa_problem p, const __grid_constant__ PrefillMaps maps,
                       const int head_major)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    unsigned char *q_tile = smem;
    unsigned char *k_tiles = smem + kPfTileBytes;
    unsigned char *v_tiles = k_tiles + kPfStages * kPfTileBytes;
    PrefillBarriers *bars = reinterpret_cast<PrefillBarriers *>(v_tiles + kPfStages * kPfTileBytes);

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned int q_tiles = (p.query_rows + kPfM - 1) / kPfM;
    const unsigned int q_tile_index = q_tiles - 1u - blockIdx.x;
    const unsigned int q0 = q_tile_index * kPfM;
    const unsigned int qhead = blockIdx.y, b = blockIdx.z;
    const unsigned int kv_head = qhead / (p.query_heads / p.kv_heads);
    const unsigned int kv_tokens = p.kv_tokens ? p.kv_tokens[b] : p.kv_tokens_uniform;
    const long long query_start =
        p.query_start ? (long long)p.query_start[b]
                      : (p.query_start_from_end ? (long long)kv_tokens - (long long)p.query_rows
                                                : (long long)p.query_start_uniform);
    // Tokens any row of this tile can see.
    long long visible_end = kv_tokens;
    if (p.causal) {
        const long long last = query_start + (long long)min(q0 + kPfM, p.query_rows);
        if (last < visible_end) visible_end = last;
    }
    const unsigned int tiles = visible_end > 0 ? (unsigned int)((visible_end + kPfN - 1) / kPfN) : 0u;

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
            mbar_init(&bars->p_full[i], kPfM);
        }
        mbar_init(&bars->pv_done, 1);
        bars->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 5) {
        tmem_alloc(&bars->tmem_base, kPfTmemColumns);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 4) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0 && tiles) {
            mbar_expect_tx(&bars->q_full, kPfTileBytes);
            tma_load_4d(q_tile, &maps.query, &bars->q_full, 0, (int)qhead, (int)q0, (int)b);
            tma_load_4d(q_tile + kPfHalfBytes, &maps.query, &bars->q_full, 64, (int)qhead, (int)q0, (int)b);
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
    } else if (warp == 5) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0 && tiles) {
            constexpr uint32_t idesc_qk = idesc_bf16_f32(kPfM, kPfN, false);
            constexpr uint32_t idesc_pv = idesc_bf16_f32(kPfM, kPfD, true);
            const uint32_t q_addr = smem_u32(q_tile);
            bool ok = mbar_wait(&bars->q_full, 0);
            auto issue_qk = [&](unsigned int j) -> bool {
                const unsigned int stage = j % kPfStages;
                if (!mbar_wait(&bars->k_full[stage], (j / kPfStages) & 1u)) return false;
                tc_fence_after_sync();
                const uint32_t k_addr = smem_u32(k_tiles + stage * kPfTileBytes);
                const uint32_t d = tmem + (j & 1u) * kPfN;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks >> 2) * kPfHalfBytes + (ks & 3) * 32;
                    tc_mma_ss(d, smem_desc_sw128(q_addr + off, 16, 1024),
                              smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk, ks ? 1u : 0u);
                }
                tc_commit(&bars->k_empty[stage]);
                tc_commit(&bars->s_full[j & 1u]);
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (unsigned int j = 0; ok && j < tiles; ++j) {
                if (j + 1 < tiles) ok = issue_qk(j + 1);
                if (!ok) break;
                const unsigned int stage = j % kPfStages;
                if (!mbar_wait(&bars->p_full[j & 1u], (j >> 1) & 1u) ||
                    !mbar_wait(&bars->v_full[stage], (j / kPfStages) & 1u)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t v_addr = smem_u32(v_tiles + stage * kPfTileBytes);
                const uint32_t p_tmem = tmem + (j & 1u) * kPfN;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)
                    tc_mma_ts(tmem + 2 * kPfN, p_tmem + kk * 8,
                              smem_desc_sw128(v_addr + kk * 2048, kPfHalfBytes, 1024), idesc_pv,
                              (j || kk) ? 1u : 0u);
                tc_commit(&bars->v_empty[stage]);
                tc_commit(&bars->pv_done);
            }
            if (!ok) prefill_fail(p, bars);
        }
    } else {
        // ------------------------------ softmax warps -----------------------------
        const unsigned int row = threadIdx.x;  // query row in the tile == TMEM lane
        const uint32_t lane_base = tmem + ((warp * 32u) << 16);
        const long long qi = (long long)q0 + row;
        long long row_limit = (long long)kv_tokens - 1;
        if (p.causal && query_start + qi < row_limit) row_limit = query_start + qi;
        const float sscale = p.scale * 1.4426950408889634f;
        float m_used = -INFINITY, l = 0.0f;
        bool ok = true;
        for (unsigned int j = 0; j < tiles; ++j) {
            const unsigned int buf = j & 1u;
            if (!mbar_wait(&bars->s_full[buf], (j >> 1) & 1u)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            uint32_t s[4][32];
#pragma unroll
            for (int i = 0; i < 4; ++i) tmem_ld32(lane_base + buf * kPfN + 32 * i, s[i]);
            tmem_wait_ld();
            const long long k0 = (long long)j * kPfN;
            float row_max = -INFINITY;
            if (k0 + kPfN - 1 > row_limit) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        if (k0 + 32 * i + c > row_limit) s[i][c] = 0xff800000u;  // -inf
                        row_max = fmaxf(row_max, __uint_as_float(s[i][c]));
                    }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int c = 0; c < 32; ++c) row_max = fmaxf(row_max, __uint_as_float(s[i][c]));
            }
            const float m_tile = row_max * sscale;  // -inf stays -inf (sscale > 0)
            const bool grow = m_tile > m_used + kPfRescaleThreshold || m_used == -INFINITY;
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = fmaxf(m_used, m_tile);
                const float factor = m_new == -INFINITY ? 1.0f : exp2_approx(m_used - m_new);
                l *= factor;
                m_used = m_new;
                if (j > 0) {
                    // O may only be touched once the previous tile's P V has landed.
                    if (!mbar_wait(&bars->pv_done, (j - 1u) & 1u)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t o[32];
                        tmem_ld32(lane_base + 2 * kPfN + 32 * i, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * factor);
                        tmem_st32(lane_base + 2 * kPfN + 32 * i, o);
                    }
                    tmem_wait_st();
                }
            }
            const float offset = m_used == -INFINITY ? 0.0f : -m_used;
            uint32_t packed[2][32];
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    const float p0 = exp2_approx(fmaf(__uint_as_float(s[i][c]), sscale, offset));
                    const float p1 = exp2_approx(fmaf(__uint_as_float(s[i][c + 1]), sscale, offset));
                    // The row sum uses the bf16-rounded weights the MMA will use,
                    // so the normalised weights stay consistent with the value mix.
                    const uint32_t pair = pack_bf16(p0, p1);
                    sum += __uint_as_float(pair << 16) + __uint_as_float(pair & 0xffff0000u);
                    packed[i >> 1][(i & 1) * 16 + (c >> 1)] = pair;
                }
            l += sum;
            tmem_st32(lane_base + buf * kPfN, packed[0]);
            tmem_st32(lane_base + buf * kPfN + 32, packed[1]);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&bars->p_full[buf]);
        }
        // ------------------------------ epilogue ------------------------------------
        if (ok && tiles) ok = mbar_wait(&bars->pv_done, (tiles - 1u) & 1u);
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
            bool finite = tiles != 0u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t o[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) o[c] = 0u;
                if (tiles) {
                    tmem_ld32(lane_base + 2 * kPfN + 32 * i, o);
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
    if (warp == 5) tmem_dealloc(tmem, kPfTmemColumns);
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
    const dim3 grid((p.query_rows + kPfM - 1) / kPfM, p.query_heads, p.sessions);
    prefill_tcgen05_kernel<<<grid, kPfThreads, kPfSmemBytes, stream>>>(p, maps, kv_head_first ? 1 : 0);
    const int rc = yvx_cuda_check(cudaGetLastError(), "prefill_tcgen05_kernel");
    return rc != 0 ? rc : 2;
}

}  // namespace yvx
