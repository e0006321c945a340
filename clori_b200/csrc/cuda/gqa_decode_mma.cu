// Split-KV flash-decoding for decode and speculative verify on sm_100a:
// head_dim 128, bf16 Q/K/V, up to 16 (query row x group head) vectors per KV
// head in one CTA, contiguous or block-tabled KV.
//
// Bandwidth-shaped. A producer warp streams 64-token K and V tiles of one KV
// head into a 3-stage shared-memory ring with TMA (128-byte swizzle, one
// mbarrier pair per stage). Four consumer warps each own 16 tokens of a tile:
// S = Q K^T and O += P V run on the tensor cores (mma.sync m16n8k16 bf16, f32
// accumulate) with the query-head group and the verify rows stacked in the M
// dimension, so every KV byte is fetched once per group. Online softmax lives
// in registers (exp2 domain, quad shuffles for row max). P is split into a
// bf16 head and tail (two MMAs) so the value mix keeps ~16 bits of P. Each CTA
// publishes a normalised (o, m, l) partial per vector; the combine kernel
// folds the splits in order.
//
// Replaces yvex_gqa_f32_body (src/backend/cuda/transformer_kernels.cu:137-238
// in the reference) for the decode/verify shapes.
#include "pipeline.cuh"

namespace yvx {

constexpr int kDecodeStages = 3;
constexpr int kTileTokens = 64;
constexpr int kHeadDim = 128;
constexpr int kConsumerWarps = 4;
constexpr int kDecodeThreads = (kConsumerWarps + 1) * 32;
constexpr int kTileBytes = kTileTokens * kHeadDim * 2;            // one K or V tile (bf16)
constexpr int kStageBytes = 2 * kTileBytes;                       // K + V
constexpr int kQRowBytes = kHeadDim * 2 + 16;                     // padded: conflict-free ldmatrix
constexpr int kMergeRowFloats = kHeadDim + 4;
constexpr int kDecodeSmemBytes = kDecodeStages * kStageBytes + 16 * kQRowBytes + 1024 /*align*/ + 256;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct DecodeMaps {
    CUtensorMap key, value;
};

struct DecodeSession {
    unsigned int kv_tokens;
    long long query_start_local;
};

__device__ __forceinline__ DecodeSession decode_session(const yvx_gqa_problem &p, unsigned int b)
{
    DecodeSession s;
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

// grid: x = split, y = kv_head * row_tiles + row_tile, z = session.
// `head_major`: the tensor maps order their middle dimensions (head, token)
// instead of (token, head); strides decide that on the host.
__global__ void __launch_bounds__(kDecodeThreads, 2)
gqa_decode_mma_kernel(const yvx_gqa_problem p, const __grid_constant__ DecodeMaps maps,
                      const int head_major)
{
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits 4..9.
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    unsigned char *stages = smem;
    unsigned char *q_smem = smem + kDecodeStages * kStageBytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(q_smem + 16 * kQRowBytes);
    uint64_t *empty = full + kDecodeStages;
    int *abort_flag = reinterpret_cast<int *>(empty + kDecodeStages);

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned int group = p.query_heads / p.kv_heads;
    const unsigned int vectors = p.query_rows * group;
    const unsigned int row_tiles = (vectors + 15u) / 16u;
    const unsigned int kv_head = blockIdx.y / row_tiles, row_tile = blockIdx.y % row_tiles;
    const unsigned int b = blockIdx.z, split = blockIdx.x;
    const DecodeSession s = decode_session(p, b);
    const unsigned int t0 = split * p.chunk_tokens;
    if (t0 >= s.kv_tokens) return;

    const unsigned int vector_base = row_tile * 16u;
    const unsigned int live = min(16u, vectors - vector_base);
    // Last visible token over the rows of this CTA.
    long long tile_limit;
    if (p.causal) {
        const unsigned int last_row = (vector_base + live - 1u) / group;
        tile_limit = s.query_start_local + (long long)last_row;
    } else {
        tile_limit = (long long)s.kv_tokens - 1;
    }
    unsigned int t1 = min(s.kv_tokens, t0 + p.chunk_tokens);
    if (tile_limit + 1 < (long long)t1) t1 = tile_limit + 1 > 0 ? (unsigned int)(tile_limit + 1) : 0u;
    const unsigned int tiles = t1 > t0 ? (t1 - t0 + kTileTokens - 1) / kTileTokens : 0u;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kDecodeStages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kConsumerWarps);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    // Query rows of this CTA into padded shared memory (zero rows beyond `live`).
    for (unsigned int i = threadIdx.x; i < 16u * (kHeadDim / 8); i += kDecodeThreads) {
        const unsigned int row = i / (kHeadDim / 8), chunk = i % (kHeadDim / 8);
        uint4 value = make_uint4(0u, 0u, 0u, 0u);
        if (row < live) {
            const unsigned int v = vector_base + row;
            const unsigned int qrow = v / group, qhead = kv_head * group + v % group;
            const __nv_bfloat16 *src = reinterpret_cast<const __nv_bfloat16 *>(p.query) +
                                       (unsigned long long)b * p.query_session_stride +
                                       (unsigned long long)qrow * p.query_row_stride +
                                       (unsigned long long)qhead * kHeadDim + chunk * 8u;
            value = *reinterpret_cast<const uint4 *>(src);
        }
        *reinterpret_cast<uint4 *>(q_smem + row * kQRowBytes + chunk * 16u) = value;
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ---------------- producer: one elected lane issues the TMA loads ----
        if (lane == 0) {
            for (unsigned int i = 0; i < tiles; ++i) {
                const unsigned int stage = i % kDecodeStages;
                if (i >= (unsigned int)kDecodeStages &&
                    !mbar_wait(&empty[stage], ((i / kDecodeStages) - 1u) & 1u)) {
                    atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
                    *abort_flag = 1;
                    break;
                }
                const unsigned int token = t0 + i * kTileTokens;
                int outer, inner_token;
                if (p.block_table) {
                    const unsigned int block = token / p.block_tokens;
                    outer = p.block_table[(unsigned long long)b * p.block_table_stride + block];
                    if (outer < 0 || (unsigned int)outer >= p.pool_blocks) {
                        atomicCAS(p.status, 0, YVX_STATUS_CONTRACT);
                        outer = 0;
                    }
                    inner_token = (int)(token - block * p.block_tokens);
                } else {
                    outer = (int)b;
                    inner_token = (int)token;
                }
                unsigned char *dst = stages + stage * kStageBytes;
                const int c1 = head_major ? (int)kv_head : inner_token;
                const int c2 = head_major ? inner_token : (int)kv_head;
                mbar_expect_tx(&full[stage], kStageBytes);
                tma_load_4d(dst, &maps.key, &full[stage], 0, c1, c2, outer);
                tma_load_4d(dst + kTileBytes / 2, &maps.key, &full[stage], 64, c1, c2, outer);
                tma_load_4d(dst + kTileBytes, &maps.value, &full[stage], 0, c1, c2, outer);
                tma_load_4d(dst + kTileBytes + kTileBytes / 2, &maps.value, &full[stage], 64, c1, c2,
                            outer);
            }
        }
        return;
    }

    // ---------------- consumers ---------------------------------------------
    const unsigned int g = lane >> 2, c = lane & 3u;
    // A fragments of Q for the 8 k-steps, kept in registers for the whole item.
    uint32_t qa[8][4];
    {
        const unsigned int j = lane >> 3, i = lane & 7u;
        const uint32_t base = smem_u32(q_smem) + (8u * (j & 1u) + i) * kQRowBytes + 16u * (j >> 1);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) ldmatrix_x4(qa[ks], base + ks * 32u);
    }
    // Visibility limit of the two rows this thread owns (g and g + 8).
    long long limit[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const unsigned int row = g + 8u * h;
        if (row >= live)
            limit[h] = -1;
        else if (p.causal)
            limit[h] = s.query_start_local + (long long)((vector_base + row) / group);
        else
            limit[h] = (long long)s.kv_tokens - 1;
    }
    const float score_scale = p.scale * kLog2e;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.0f;

    for (unsigned int i = 0; i < tiles; ++i) {
        const unsigned int stage = i % kDecodeStages;
        if (!mbar_wait(&full[stage], (i / kDecodeStages) & 1u)) {
            atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
            break;
        }
        const uint32_t k_base = smem_u32(stages + stage * kStageBytes);
        const uint32_t v_base = k_base + kTileBytes;
        const unsigned int tile_token = t0 + i * kTileTokens + 16u * warp;  // first token of this warp

        // ---- S = Q K^T over this warp's 16 tokens ------------------------
        float sc[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[n][e] = 0.0f;
        {
            const unsigned int j = lane >> 3, r = lane & 7u;
            const unsigned int token = 16u * warp + 8u * (j >> 1) + r;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const unsigned int chunk = 2u * (ks & 3) + (j & 1u);
                const uint32_t addr = k_base + (ks >> 2) * (kTileBytes / 2) + token * 128u +
                                      ((chunk ^ (token & 7u)) << 4);
                uint32_t kb[4];
                ldmatrix_x4(kb, addr);
                mma_bf16(sc[0], qa[ks], kb[0], kb[1]);
                mma_bf16(sc[1], qa[ks], kb[2], kb[3]);
            }
        }
        // ---- masking + online softmax (exp2 domain) ----------------------
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                const long long token = (long long)tile_token + 8 * n + 2 * c + (e & 1);
                const float value = token <= limit[h] ? sc[n][e] * score_scale : -INFINITY;
                sc[n][e] = value;
                tile_max[h] = fmaxf(tile_max[h], value);
            }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
            tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
        }
        float keep[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float fresh = fmaxf(m[h], tile_max[h]);
            keep[h] = fresh == -INFINITY ? 1.0f : exp2_approx(m[h] - fresh);
            m[h] = fresh;
            l[h] *= keep[h];
        }
        const bool rescale = keep[0] != 1.0f || keep[1] != 1.0f;
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int n = 0; n < 16; ++n) {
                o[n][0] *= keep[0];
                o[n][1] *= keep[0];
                o[n][2] *= keep[1];
                o[n][3] *= keep[1];
            }
        }
        uint32_t p_head[4], p_tail[4];
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float base = m[h] == -INFINITY ? 0.0f : m[h];
                const float p0 = exp2_approx(sc[n][2 * h] - base);
                const float p1 = exp2_approx(sc[n][2 * h + 1] - base);
                l[h] += p0 + p1;
                const uint32_t head = pack_bf16(p0, p1);
                const float r0 = p0 - __uint_as_float(head << 16);
                const float r1 = p1 - __uint_as_float(head & 0xffff0000u);
                p_head[2 * n + h] = head;
                p_tail[2 * n + h] = pack_bf16(r0, r1);
            }
        // Rows of the V tile beyond the session's length may hold anything
        // (even NaN patterns); P is zero there, so zero those rows too.
        if (tile_token + 16u > s.kv_tokens) {
            for (unsigned int r = lane; r < 16u * 16u; r += 32u) {
                const unsigned int row = 16u * warp + r / 16u, chunk16 = r % 16u;
                if (tile_token - 16u * warp + row >= s.kv_tokens)
                    *reinterpret_cast<uint4 *>(stages + stage * kStageBytes + kTileBytes +
                                               (chunk16 >> 3) * (kTileBytes / 2) + row * 128u +
                                               (((chunk16 & 7u) ^ (row & 7u)) << 4)) =
                        make_uint4(0u, 0u, 0u, 0u);
            }
            __syncwarp();
        }
        // ---- O += P V ------------------------------------------------------
        {
            const unsigned int j = lane >> 3, r = lane & 7u;
            const unsigned int token = 16u * warp + 8u * (j & 1u) + r;
#pragma unroll
            for (int np = 0; np < 8; ++np) {
                const unsigned int chunk = 2u * (np & 3) + (j >> 1);
                const uint32_t addr = v_base + (np >> 2) * (kTileBytes / 2) + token * 128u +
                                      ((chunk ^ (token & 7u)) << 4);
                uint32_t vb[4];
                ldmatrix_x4_trans(vb, addr);
                mma_bf16(o[2 * np], p_head, vb[0], vb[1]);
                mma_bf16(o[2 * np], p_tail, vb[0], vb[1]);
                mma_bf16(o[2 * np + 1], p_head, vb[2], vb[3]);
                mma_bf16(o[2 * np + 1], p_tail, vb[2], vb[3]);
            }
        }
        __syncwarp();
        if (tile_token + 16u > s.kv_tokens) fence_proxy_async();
        if (lane == 0) mbar_arrive(&empty[stage]);
    }

    // ---- merge the four warps and publish ---------------------------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    named_barrier(1, kConsumerWarps * 32);  // every warp is done reading the stages
    float *merge_o = reinterpret_cast<float *>(stages);                          // [4][16][132]
    float *merge_m = merge_o + kConsumerWarps * 16 * kMergeRowFloats;            // [4][16]
    float *merge_l = merge_m + kConsumerWarps * 16;                              // [4][16]
#pragma unroll
    for (int n = 0; n < 16; ++n) {
        float *row0 = merge_o + (warp * 16 + g) * kMergeRowFloats + 8 * n + 2 * c;
        float *row1 = merge_o + (warp * 16 + g + 8) * kMergeRowFloats + 8 * n + 2 * c;
        *reinterpret_cast<float2 *>(row0) = make_float2(o[n][0], o[n][1]);
        *reinterpret_cast<float2 *>(row1) = make_float2(o[n][2], o[n][3]);
    }
    if (c == 0) {
        merge_m[warp * 16 + g] = m[0];
        merge_m[warp * 16 + g + 8] = m[1];
        merge_l[warp * 16 + g] = l[0];
        merge_l[warp * 16 + g + 8] = l[1];
    }
    named_barrier(1, kConsumerWarps * 32);

    // The main loop is over: let the combine kernel's launch overlap the epilogue.
    pdl_launch_dependents();
    const bool direct = p.max_splits == 1u;
    const unsigned int d = threadIdx.x;  // 0..127: one head dimension per consumer thread
    for (unsigned int row = 0; row < live; ++row) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) mm = fmaxf(mm, merge_m[w * 16 + row]);
        float ll = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
            const float mw = merge_m[w * 16 + row];
            const float weight = mw == -INFINITY ? 0.0f : exp2_approx(mw - mm);
            ll += merge_l[w * 16 + row] * weight;
            acc += merge_o[(w * 16 + row) * kMergeRowFloats + d] * weight;
        }
        const unsigned int v = vector_base + row;
        const unsigned int qrow = v / group, qhead = kv_head * group + v % group;
        const unsigned long long item =
            ((unsigned long long)b * p.query_rows + qrow) * p.query_heads + qhead;
        if (direct && !p.partial_output) {
            const float value = acc / ll;
            if (!isfinite(value)) atomicCAS(p.status, 0, YVX_STATUS_NONFINITE);
            store_output(p.output, p.output_dtype, item * kHeadDim + d, value);
        } else {
            float *part = direct ? p.partial_output + item * (kHeadDim + 2ull)
                                 : p.partials + (item * p.max_splits + split) * (kHeadDim + 2ull);
            part[d] = ll > 0.0f ? acc / ll : 0.0f;
            if (d == 0) {
                part[kHeadDim] = mm == -INFINITY ? -INFINITY : mm * kLn2;  // natural-log units
                part[kHeadDim + 1] = ll;
            }
        }
    }
}

// ---- host side: tensor maps -------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_entry()
{
    static EncodeTiledFn entry = nullptr;
    static bool resolved = false;
    if (!resolved) {
        void *symbol = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &query) ==
                cudaSuccess &&
            query == cudaDriverEntryPointSuccess)
            entry = reinterpret_cast<EncodeTiledFn>(symbol);
        resolved = true;
    }
    return entry;
}

// 4-D map {128 elems, mid0, mid1, outer}; the two middle dimensions are ordered
// by ascending stride. Returns false when TMA cannot describe the layout
// (misaligned base or strides), in which case the caller takes the general kernel.
static bool encode_kv_map(CUtensorMap *map, const void *base, unsigned long long token_stride,
                          unsigned long long head_stride, unsigned long long outer_stride,
                          unsigned long long tokens, unsigned long long heads,
                          unsigned long long outer, bool head_major)
{
    EncodeTiledFn encode = encode_tiled_entry();
    if (!encode) return false;
    const unsigned long long tb = token_stride * 2ull, hb = head_stride * 2ull;
    unsigned long long ob = outer_stride * 2ull;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (tb & 15ull) || (hb & 15ull) || (ob & 15ull))
        return false;
    if (outer <= 1ull) {
        outer = 1ull;
        ob = (head_major ? tb * tokens : hb * heads);
        ob = (ob + 15ull) & ~15ull;
    }
    cuuint64_t dims[4] = {kHeadDim, head_major ? heads : tokens, head_major ? tokens : heads, outer};
    cuuint64_t strides[3] = {head_major ? hb : tb, head_major ? tb : hb, ob};
    cuuint32_t box[4] = {64, head_major ? 1u : (cuuint32_t)kTileTokens,
                         head_major ? (cuuint32_t)kTileTokens : 1u, 1};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    for (int i = 0; i < 3; ++i)
        if (!strides[i] || strides[i] >= (1ull << 40)) return false;
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides,
                  box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Returns 1 when the launch was made, 0 when the shape is not this kernel's,
// negative on a launch error.
int gqa_decode_mma_launch(const yvx_gqa_problem &p, cudaStream_t stream)
{
    if (p.head_dim != (unsigned)kHeadDim || p.query_dtype != YVEX_DTYPE_BF16 ||
        p.kv_dtype != YVEX_DTYPE_BF16 || p.chunk_tokens % kTileTokens ||
        (p.query_row_stride % 8ull) || (p.query_session_stride % 8ull) ||
        (reinterpret_cast<uintptr_t>(p.query) & 15u))
        return 0;
    if (p.block_table && (p.block_tokens % kTileTokens)) return 0;
    const unsigned int group = p.query_heads / p.kv_heads;
    const unsigned int vectors = p.query_rows * group;
    if (vectors > 64u) return 0;  // long query blocks are prefill's shape, not this kernel's
    const bool head_major = p.key_head_stride < p.key_token_stride;
    if ((p.value_head_stride < p.value_token_stride) != head_major) return 0;
    DecodeMaps maps;
    const unsigned long long tokens = p.block_table ? p.block_tokens : p.kv_tokens_max;
    const unsigned long long outer = p.block_table ? p.pool_blocks : p.sessions;
    if (!encode_kv_map(&maps.key, p.key, p.key_token_stride, p.key_head_stride,
                       p.block_table ? p.key_block_stride : p.key_session_stride, tokens,
                       p.kv_heads, outer, head_major) ||
        !encode_kv_map(&maps.value, p.value, p.value_token_stride, p.value_head_stride,
                       p.block_table ? p.value_block_stride : p.value_session_stride, tokens,
                       p.kv_heads, outer, head_major))
        return 0;
    cudaError_t error = cudaFuncSetAttribute(gqa_decode_mma_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kDecodeSmemBytes);
    if (error != cudaSuccess) return yvx_cuda_check(error, "gqa_decode_mma_kernel attribute");
    const dim3 grid(p.max_splits, p.kv_heads * ((vectors + 15u) / 16u), p.sessions);
    gqa_decode_mma_kernel<<<grid, kDecodeThreads, kDecodeSmemBytes, stream>>>(p, maps,
                                                                              head_major ? 1 : 0);
    const int rc = yvx_cuda_check(cudaGetLastError(), "gqa_decode_mma_kernel");
    return rc != 0 ? rc : 1;
}

}  // namespace yvx
