// Split-KV decode / speculative verify over a Q8_0-quantised KV cache on
// sm_100a: head_dim 128, bf16 queries, up to 16 (row x group head) vectors per
// KV head per CTA.
//
// KV layout ("Q8 record"): one contiguous 17408-byte record per (64-token
// block, KV head) holding the block's Q8_0 data in the order the tensor-core
// fragments consume it:
//     [ K lanes 8192 | V lanes 8192 | K scales 512 | V scales 512 ]
// It is a byte permutation of the GGUF Q8_0 rows of the same tokens (34-byte
// blocks, f16 scale + 32 int8 lanes: src/gguf/quant_block.c:160-187 in the
// reference), so the bytes moved per token are exactly Q8_0's 34/32 per lane,
// each record arrives with ONE linear bulk copy, and every shared-memory read
// in the loop is a conflict-free 16-byte load.
//
// Arithmetic: lanes become exact f16 integers (magic-number conversion). For K
// the per-32-lane scale multiplies the f32 partial sum of its block, which is
// the reference's dequantisation x = f16(d) * int8 (quant_block.c:819-832)
// carried out exactly. For V the scale is folded into the f16 operand (one
// rounding, 2^-12 relative). P is f16 (11 significant bits). Softmax and all
// accumulation are f32.
#include "exchange.cuh"
#include "pipeline.cuh"

namespace yvx {

constexpr int kQ8Stages = 5;
constexpr int kQ8TileTokens = 64;
constexpr int kQ8HeadDim = 128;
constexpr int kQ8ConsumerWarps = 4;
constexpr int kQ8Threads = (kQ8ConsumerWarps + 1) * 32;
constexpr int kQ8RecordBytes = 17408;
constexpr int kQ8KLanes = 0, kQ8VLanes = 8192, kQ8KScales = 16384, kQ8VScales = 16896;
constexpr int kQ8QRowBytes = kQ8HeadDim * 2 + 16;
constexpr int kQ8MergeRowFloats = kQ8HeadDim + 4;
constexpr int kQ8SmemBytes = kQ8Stages * kQ8RecordBytes + 16 * kQ8QRowBytes + 1024 + 256;
constexpr float kQ8Log2e = 1.4426950408889634f;

struct Q8Session {
    unsigned int kv_tokens;
    long long query_start_local;
};

__device__ __forceinline__ Q8Session q8_session(const yvx_gqa_problem &p, unsigned int b)
{
    Q8Session s;
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

// Four stored lanes (lane + 128, one byte each) -> two f16x2 registers holding the
// exact integers: a byte u placed under exponent 0x64 reads as 1024 + u; minus 1152.
__device__ __forceinline__ void q8_lanes_to_f16(uint32_t biased, uint32_t &lo, uint32_t &hi)
{
    uint32_t a, b;
    asm("prmt.b32 %0, %1, %2, 0x4140;" : "=r"(a) : "r"(biased), "r"(0x64646464u));
    asm("prmt.b32 %0, %1, %2, 0x4342;" : "=r"(b) : "r"(biased), "r"(0x64646464u));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(a), "r"(0x64806480u));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(b), "r"(0x64806480u));
}

// D = A * B + C with C given separately (so a chain can start from a constant).
__device__ __forceinline__ void mma_f16_from(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                             uint32_t b1, float c0, float c1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%11,%11};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c0), "f"(c1));
}

// Four signed bytes -> two f16x2 registers holding 1152 + lane (no subtraction):
// used where the constant is cancelled through the accumulator's initial value.
__device__ __forceinline__ void q8_lanes_to_f16_biased(uint32_t biased, uint32_t &lo, uint32_t &hi)
{
    asm("prmt.b32 %0, %1, %2, 0x4140;" : "=r"(lo) : "r"(biased), "r"(0x64646464u));
    asm("prmt.b32 %0, %1, %2, 0x4342;" : "=r"(hi) : "r"(biased), "r"(0x64646464u));
}

__device__ __forceinline__ uint32_t mul_f16x2(uint32_t a, uint32_t b)
{
    uint32_t r;
    asm("mul.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

__device__ __forceinline__ float f16_lo(uint32_t pair)
{
    return __half2float(__ushort_as_half((unsigned short)(pair & 0xffffu)));
}
__device__ __forceinline__ float f16_hi(uint32_t pair)
{
    return __half2float(__ushort_as_half((unsigned short)(pair >> 16)));
}

struct Q8ConsumerSync {
    static __device__ __forceinline__ void sync() { named_barrier(1, kQ8ConsumerWarps * 32); }
};

// grid: x = split, y = kv_head * row_tiles + row_tile, z = session.
// With an exchange (x.gather != NULL; cooperative launch, so every CTA is resident) the step
// is ONE launch: after its partial rows a CTA takes a ticket of its (session, KV head, row
// tile); the CTAs with split < live wait (bounded) for all the group's tickets, fold the
// splits of item vector_base + split, and run the cross-GPU exchange of that item.
__global__ void __launch_bounds__(kQ8Threads, 2)
gqa_decode_q8_kernel(const yvx_gqa_problem p, const yvx_lse_exchange x)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    unsigned char *stages = smem;
    unsigned char *q_smem = smem + kQ8Stages * kQ8RecordBytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(q_smem + 16 * kQ8QRowBytes);
    uint64_t *empty = full + kQ8Stages;
    __shared__ float k_bias_smem[64];

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned int group = p.query_heads / p.kv_heads;
    const unsigned int vectors = p.query_rows * group;
    const unsigned int row_tiles = (vectors + 15u) / 16u;
    const unsigned int kv_head = blockIdx.y / row_tiles, row_tile = blockIdx.y % row_tiles;
    const unsigned int b = blockIdx.z, split = blockIdx.x;
    const Q8Session s = q8_session(p, b);
    const unsigned int t0 = split * p.chunk_tokens;
    if (t0 >= s.kv_tokens) return;

    const unsigned int vector_base = row_tile * 16u;
    const unsigned int live = min(16u, vectors - vector_base);
    long long tile_limit;
    if (p.causal)
        tile_limit = s.query_start_local + (long long)((vector_base + live - 1u) / group);
    else
        tile_limit = (long long)s.kv_tokens - 1;
    unsigned int t1 = min(s.kv_tokens, t0 + p.chunk_tokens);
    if (tile_limit + 1 < (long long)t1) t1 = tile_limit + 1 > 0 ? (unsigned int)(tile_limit + 1) : 0u;
    const unsigned int tiles = t1 > t0 ? (t1 - t0 + kQ8TileTokens - 1) / kQ8TileTokens : 0u;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kQ8Stages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kQ8ConsumerWarps);
        }
        fence_barrier_init();
    }
    // Queries: bf16 in global memory -> f16 in padded shared memory. Exact for
    // every bf16 value inside f16's normal range.
    for (unsigned int i = threadIdx.x; i < 16u * (kQ8HeadDim / 8); i += kQ8Threads) {
        const unsigned int row = i / (kQ8HeadDim / 8), chunk = i % (kQ8HeadDim / 8);
        uint4 out = make_uint4(0u, 0u, 0u, 0u);
        if (row < live) {
            const unsigned int v = vector_base + row;
            const unsigned int qrow = v / group, qhead = kv_head * group + v % group;
            const __nv_bfloat16 *src = reinterpret_cast<const __nv_bfloat16 *>(p.query) +
                                       (unsigned long long)b * p.query_session_stride +
                                       (unsigned long long)qrow * p.query_row_stride +
                                       (unsigned long long)qhead * kQ8HeadDim + chunk * 8u;
            const uint4 raw = *reinterpret_cast<const uint4 *>(src);
            const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
            uint32_t packed[4];
#pragma unroll
            for (int w = 0; w < 4; ++w)
                packed[w] = pack_f16(__uint_as_float(words[w] << 16),
                                     __uint_as_float(words[w] & 0xffff0000u));
            out = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
        *reinterpret_cast<uint4 *>(q_smem + row * kQ8QRowBytes + chunk * 16u) = out;
    }
    __syncthreads();
    // K lanes enter the MMA as 1152 + lane; the surplus 1152 * sum_k q[row][k]
    // over each 32-lane block is cancelled by starting that block's accumulator
    // at its negative. One sum per (row, block), computed once per CTA.
    if (threadIdx.x < 64u) {
        const unsigned int row = threadIdx.x >> 2, db = threadIdx.x & 3u;
        const __half *qrow = reinterpret_cast<const __half *>(q_smem + row * kQ8QRowBytes) + 32u * db;
        float sum = 0.0f;
#pragma unroll 8
        for (int k = 0; k < 32; ++k) sum += __half2float(qrow[k]);
        k_bias_smem[row * 4u + db] = -1152.0f * sum;
    }
    __syncthreads();

    if (warp == kQ8ConsumerWarps) {
        if (lane == 0) {
            const unsigned char *records = reinterpret_cast<const unsigned char *>(p.key);
            for (unsigned int i = 0; i < tiles; ++i) {
                const unsigned int stage = i % kQ8Stages;
                if (i >= (unsigned int)kQ8Stages &&
                    !mbar_wait(&empty[stage], ((i / kQ8Stages) - 1u) & 1u)) {
                    atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
                    break;
                }
                const unsigned int block = (t0 + i * kQ8TileTokens) / kQ8TileTokens;
                unsigned long long offset;
                if (p.block_table) {
                    int pool_block = p.block_table[(unsigned long long)b * p.block_table_stride + block];
                    if (pool_block < 0 || (unsigned int)pool_block >= p.pool_blocks) {
                        atomicCAS(p.status, 0, YVX_STATUS_CONTRACT);
                        pool_block = 0;
                    }
                    offset = (unsigned long long)pool_block * p.key_block_stride;
                } else {
                    offset = (unsigned long long)b * p.key_session_stride +
                             (unsigned long long)block * p.key_block_stride;
                }
                offset += (unsigned long long)kv_head * p.key_head_stride;
                mbar_expect_tx(&full[stage], kQ8RecordBytes);
                bulk_load(stages + stage * kQ8RecordBytes, records + offset, kQ8RecordBytes,
                          &full[stage]);
            }
        }
        return;
    }

    const unsigned int g = lane >> 2, c = lane & 3u;
    // ldmatrix address of this lane's row of the Q tile (A operand, k-step 0).
    const uint32_t q_frag_base = smem_u32(q_smem) + (8u * ((lane >> 3) & 1u) + (lane & 7u)) * kQ8QRowBytes +
                                 16u * (lane >> 4);
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
    // Tokens up to `unmasked_until` are visible to every live row of this CTA.
    long long unmasked_until;
    if (p.causal)
        unmasked_until = s.query_start_local + (long long)(vector_base / group);
    else
        unmasked_until = (long long)s.kv_tokens - 1;
    if (unmasked_until > (long long)s.kv_tokens - 1) unmasked_until = (long long)s.kv_tokens - 1;
    const float score_scale = p.scale * kQ8Log2e;
    const float slack = 8.0f / score_scale;  // raw-score distance worth 2^8 in the weights
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};   // m in raw score units
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.0f;

    for (unsigned int i = 0; i < tiles; ++i) {
        const unsigned int stage = i % kQ8Stages;
        if (!mbar_wait(&full[stage], (i / kQ8Stages) & 1u)) {
            atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
            break;
        }
        const unsigned char *record = stages + stage * kQ8RecordBytes;
        const unsigned int tile_token = t0 + i * kQ8TileTokens + 16u * warp;

        // ---- S = Q K^T: per 32-lane block, exact integer dot then scale ----
        // Q fragments are re-read from shared memory per block (registers are the
        // scarcer resource: three CTAs share an SM).
        float sc[2][4];
        uint4 ks[2];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            // scales of tokens (8nt + 2c) and (8nt + 2c + 1): 2 x 4 f16
            ks[n] = *reinterpret_cast<const uint4 *>(record + kQ8KScales + (8u * (2u * warp + n) + 2u * c) * 8u);
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[n][e] = 0.0f;
        }
#pragma unroll
        for (int kg = 0; kg < 2; ++kg) {
            uint4 kq[2];
#pragma unroll
            for (int n = 0; n < 2; ++n)
                kq[n] = *reinterpret_cast<const uint4 *>(
                    record + kQ8KLanes + (((2u * warp + n) * 2u + kg) * 32u + lane) * 16u);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int db = 2 * kg + half;
                uint32_t qa0[4], qa1[4];
                ldmatrix_x4(qa0, q_frag_base + (4 * kg + 2 * half) * 32u);
                ldmatrix_x4(qa1, q_frag_base + (4 * kg + 2 * half + 1) * 32u);
                const float bias0 = k_bias_smem[g * 4u + db], bias1 = k_bias_smem[(g + 8u) * 4u + db];
#pragma unroll
                for (int n = 0; n < 2; ++n) {
                    const uint32_t kq_words[4] = {kq[n].x, kq[n].y, kq[n].z, kq[n].w};
                    const uint32_t ks_words[4] = {ks[n].x, ks[n].y, ks[n].z, ks[n].w};
                    float acc[4];
                    uint32_t b0, b1;
                    q8_lanes_to_f16_biased(kq_words[2 * half], b0, b1);
                    mma_f16_from(acc, qa0, b0, b1, bias0, bias1);
                    q8_lanes_to_f16_biased(kq_words[2 * half + 1], b0, b1);
                    mma_f16(acc, qa1, b0, b1);
                    // token 2c uses ks_words[0..1], token 2c+1 uses ks_words[2..3]
                    const uint32_t pair0 = ks_words[db >> 1], pair1 = ks_words[2 + (db >> 1)];
                    const float d0 = (db & 1) ? f16_hi(pair0) : f16_lo(pair0);
                    const float d1 = (db & 1) ? f16_hi(pair1) : f16_lo(pair1);
                    sc[n][0] = fmaf(acc[0], d0, sc[n][0]);
                    sc[n][1] = fmaf(acc[1], d1, sc[n][1]);
                    sc[n][2] = fmaf(acc[2], d0, sc[n][2]);
                    sc[n][3] = fmaf(acc[3], d1, sc[n][3]);
                }
            }
        }
        // ---- masking (only on tiles that cross a visibility limit) ----------
        if ((long long)tile_token + 15 > unmasked_until) {
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const long long token = (long long)tile_token + 8 * n + 2 * c + (e & 1);
                    if (token > limit[e >> 1]) sc[n][e] = -INFINITY;
                }
        }
        // ---- online softmax: m in raw score units, exponent = (s - m) * scale.
        // The reference maximum is stale by design: it moves (quad shuffles, rescale of O)
        // only when some score of the warp exceeds it by more than 2^8 in the exponent,
        // so the common tile costs one vote instead of four shuffles and a rescale;
        // weights stay <= 256, exact in f16 / f32 range.
        bool grow = false;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float bound = m[h] + slack;  // -inf while the row has seen nothing
#pragma unroll
            for (int n = 0; n < 2; ++n) grow = grow || sc[n][2 * h] > bound || sc[n][2 * h + 1] > bound;
        }
        if (__any_sync(0xffffffffu, grow)) {
            float tile_max[2], keep[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tile_max[h] = fmaxf(fmaxf(sc[0][2 * h], sc[0][2 * h + 1]), fmaxf(sc[1][2 * h], sc[1][2 * h + 1]));
                tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
                tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
                const float fresh = fmaxf(m[h], tile_max[h]);
                keep[h] = fresh == -INFINITY ? 1.0f : exp2_approx((m[h] - fresh) * score_scale);
                m[h] = fresh;
                l[h] *= keep[h];
            }
#pragma unroll
            for (int n = 0; n < 16; ++n) {
                o[n][0] *= keep[0];
                o[n][1] *= keep[0];
                o[n][2] *= keep[1];
                o[n][3] *= keep[1];
            }
        }
        float offset[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) offset[h] = m[h] == -INFINITY ? 0.0f : -m[h] * score_scale;
        uint32_t p_head[4];
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float p0 = exp2_approx(fmaf(sc[n][2 * h], score_scale, offset[h]));
                const float p1 = exp2_approx(fmaf(sc[n][2 * h + 1], score_scale, offset[h]));
                l[h] += p0 + p1;
                p_head[2 * n + h] = pack_f16(p0, p1);
            }
        // ---- O += P V: lanes -> f16, scale folded into the operand ----------
        {
            // V scales of this warp's tokens {2c, 2c+1, 2c+8, 2c+9} for the 4 dim blocks.
            const uint4 va = *reinterpret_cast<const uint4 *>(record + kQ8VScales + ((warp * 4u + c) * 4u) * 8u);
            const uint4 vb = *reinterpret_cast<const uint4 *>(record + kQ8VScales + ((warp * 4u + c) * 4u) * 8u + 16u);
            uint32_t vs01[4] = {va.x, va.z, vb.x, vb.z};  // (d[2c], d[2c+1]) per dim block
            uint32_t vs23[4] = {va.y, va.w, vb.y, vb.w};  // (d[2c+8], d[2c+9]) per dim block
            if (tile_token + 16u > s.kv_tokens) {
                // Slots beyond the session's length may hold any bytes; their P is
                // zero, so zero their scale too (0 * Inf would poison the sum).
                const long long t_a = (long long)tile_token + 2 * c, t_b = t_a + 8;
                const uint32_t mask01 = (t_a < (long long)s.kv_tokens ? 0x0000ffffu : 0u) |
                                        (t_a + 1 < (long long)s.kv_tokens ? 0xffff0000u : 0u);
                const uint32_t mask23 = (t_b < (long long)s.kv_tokens ? 0x0000ffffu : 0u) |
                                        (t_b + 1 < (long long)s.kv_tokens ? 0xffff0000u : 0u);
#pragma unroll
                for (int db = 0; db < 4; ++db) {
                    vs01[db] &= mask01;
                    vs23[db] &= mask23;
                }
            }
#pragma unroll
            for (int db = 0; db < 4; ++db) {
                const uint4 vq = *reinterpret_cast<const uint4 *>(
                    record + kQ8VLanes + ((warp * 4u + db) * 32u + lane) * 16u);
                const uint32_t vq_words[4] = {vq.x, vq.y, vq.z, vq.w};
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    uint32_t b0, b1;
                    q8_lanes_to_f16(vq_words[i4], b0, b1);
                    b0 = mul_f16x2(b0, vs01[db]);
                    b1 = mul_f16x2(b1, vs23[db]);
                    mma_f16(o[4 * db + i4], p_head, b0, b1);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stage]);
    }

    // ---- merge the four warps and publish ---------------------------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    named_barrier(1, kQ8ConsumerWarps * 32);
    float *merge_o = reinterpret_cast<float *>(stages);
    float *merge_m = merge_o + kQ8ConsumerWarps * 16 * kQ8MergeRowFloats;
    float *merge_l = merge_m + kQ8ConsumerWarps * 16;
#pragma unroll
    for (int n = 0; n < 16; ++n) {
        float *row0 = merge_o + (warp * 16 + g) * kQ8MergeRowFloats + 8 * n + 2 * c;
        float *row1 = merge_o + (warp * 16 + g + 8) * kQ8MergeRowFloats + 8 * n + 2 * c;
        *reinterpret_cast<float2 *>(row0) = make_float2(o[n][0], o[n][1]);
        *reinterpret_cast<float2 *>(row1) = make_float2(o[n][2], o[n][3]);
    }
    if (c == 0) {
        merge_m[warp * 16 + g] = m[0];
        merge_m[warp * 16 + g + 8] = m[1];
        merge_l[warp * 16 + g] = l[0];
        merge_l[warp * 16 + g + 8] = l[1];
    }
    named_barrier(1, kQ8ConsumerWarps * 32);

    // The main loop is over: let the combine kernel's launch overlap the epilogue.
    pdl_launch_dependents();
    const bool direct = p.max_splits == 1u;
    const unsigned int d = threadIdx.x;
    for (unsigned int row = 0; row < live; ++row) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kQ8ConsumerWarps; ++w) mm = fmaxf(mm, merge_m[w * 16 + row]);
        float ll = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < kQ8ConsumerWarps; ++w) {
            const float mw = merge_m[w * 16 + row];
            const float weight = mw == -INFINITY ? 0.0f : exp2_approx((mw - mm) * score_scale);
            ll += merge_l[w * 16 + row] * weight;
            acc += merge_o[(w * 16 + row) * kQ8MergeRowFloats + d] * weight;
        }
        const unsigned int v = vector_base + row;
        const unsigned int qrow = v / group, qhead = kv_head * group + v % group;
        const unsigned long long item =
            ((unsigned long long)b * p.query_rows + qrow) * p.query_heads + qhead;
        if (direct && !p.partial_output) {
            const float value = acc / ll;
            if (!isfinite(value)) atomicCAS(p.status, 0, YVX_STATUS_NONFINITE);
            store_output(p.output, p.output_dtype, item * kQ8HeadDim + d, value);
        } else {
            float *part = direct ? p.partial_output + item * (kQ8HeadDim + 2ull)
                                 : p.partials + (item * p.max_splits + split) * (kQ8HeadDim + 2ull);
            part[d] = ll > 0.0f ? acc / ll : 0.0f;
            if (d == 0) {
                part[kQ8HeadDim] = mm == -INFINITY ? -INFINITY : mm * p.scale;  // natural-log units
                part[kQ8HeadDim + 1] = ll;
            }
        }
    }
    if (!x.gather) return;

    // ---- one-launch step: this group's splits are folded and exchanged by its own CTAs -------
    const unsigned int items = p.sessions * p.query_rows * p.query_heads;
    unsigned int *ticket = x.arrivals[x.rank] + items + ((unsigned long long)b * gridDim.y + blockIdx.y);
    __threadfence();  // the partial rows above, before the ticket
    Q8ConsumerSync::sync();
    if (threadIdx.x == 0) atomicAdd(ticket, 1u);
    if (split >= live) return;
    float *fold_scratch = reinterpret_cast<float *>(stages);             // [4][130], the ring is drained
    float *fold_row = fold_scratch + kQ8ConsumerWarps * (kQ8HeadDim + 2);
    int *flag = reinterpret_cast<int *>(fold_row + kQ8HeadDim + 2);
    if (threadIdx.x == 0) {
        // tickets only grow: epoch e is complete at e * splits (the plan is the same every epoch)
        const volatile unsigned int *counter = ticket;
        const unsigned int target = x.epoch * gridDim.x;
        int ok = 0;
        for (unsigned int spin = 0; spin < kExchangeSpinLimit; ++spin) {
            if ((int)(*counter - target) >= 0) {
                ok = 1;
                break;
            }
            __nanosleep(40);
        }
        *flag = ok;
    }
    Q8ConsumerSync::sync();
    if (!*flag) {
        if (threadIdx.x == 0) atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
        return;
    }
    __threadfence();
    for (unsigned int i = split; i < live; i += gridDim.x) {
        const unsigned int v = vector_base + i;
        const unsigned int qrow = v / group, qhead = kv_head * group + v % group;
        const unsigned long long item = ((unsigned long long)b * p.query_rows + qrow) * p.query_heads + qhead;
        if (direct) {
            const float *mine = p.partial_output + item * (kQ8HeadDim + 2ull);
            for (unsigned int e = threadIdx.x; e < (unsigned)kQ8HeadDim + 2u; e += kQ8ConsumerWarps * 32u)
                fold_row[e] = __ldcg(mine + e);
            Q8ConsumerSync::sync();
        } else {
            fold_splits_128<kQ8ConsumerWarps, Q8ConsumerSync>(
                p.partials + item * p.max_splits * (kQ8HeadDim + 2ull), p.max_splits, fold_scratch, fold_row, threadIdx.x);
        }
        const bool came =
            x.tagged_words
                ? exchange_item_tagged<Q8ConsumerSync>(x, x.rank, items, (unsigned int)item, kQ8HeadDim, fold_row,
                                                       fold_scratch, flag, threadIdx.x, kQ8ConsumerWarps * 32u, p.output,
                                                       p.output_dtype, item * kQ8HeadDim, p.status)
                : exchange_item<Q8ConsumerSync>(x, x.rank, items, (unsigned int)item, kQ8HeadDim, fold_row, flag,
                                                threadIdx.x, kQ8ConsumerWarps * 32u, p.output, p.output_dtype,
                                                item * kQ8HeadDim, p.status);
        if (!came) return;
        Q8ConsumerSync::sync();
    }
}

int gqa_decode_q8_launch(const yvx_gqa_problem &p, cudaStream_t stream, const yvx_lse_exchange *exchange)
{
    if (p.kv_dtype != YVEX_DTYPE_Q8_0) return 0;
    if (p.head_dim != (unsigned)kQ8HeadDim || p.query_dtype != YVEX_DTYPE_BF16 ||
        p.chunk_tokens % kQ8TileTokens || (p.query_row_stride % 8ull) ||
        (p.query_session_stride % 8ull) || (reinterpret_cast<uintptr_t>(p.query) & 15u) ||
        (reinterpret_cast<uintptr_t>(p.key) & 15u) || (p.key_head_stride % 16ull) ||
        (p.key_block_stride % 16ull) || (p.key_session_stride % 16ull) ||
        p.key_head_stride < (unsigned long long)kQ8RecordBytes ||
        (p.block_table && p.block_tokens != (unsigned)kQ8TileTokens))
        return YVEX_ERR_UNSUPPORTED;
    const unsigned int group = p.query_heads / p.kv_heads;
    const unsigned int vectors = p.query_rows * group;
    if (vectors > 64u) return YVEX_ERR_UNSUPPORTED;
    // per device, once: the attribute and the resident-CTA capacity (host calls that would
    // otherwise sit in front of every launch of a latency-sized step)
    static int configured_device = -1, resident_ctas = 0;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return YVEX_ERR_BACKEND;
    if (configured_device != device) {
        int sms = 0, per_sm = 0;
        cudaError_t error = cudaFuncSetAttribute(gqa_decode_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 kQ8SmemBytes);
        if (error != cudaSuccess) return yvx_cuda_check(error, "gqa_decode_q8_kernel attribute");
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gqa_decode_q8_kernel, kQ8Threads, kQ8SmemBytes) !=
                cudaSuccess)
            return YVEX_ERR_BACKEND;
        resident_ctas = sms * per_sm;
        configured_device = device;
    }
    const dim3 grid(p.max_splits, p.kv_heads * ((vectors + 15u) / 16u), p.sessions);
    if (exchange) {
        // The one-launch step: CTAs wait on one another's tickets, so all of them must be resident:
        // a cooperative launch, or (when the grid does not fit, or the shape is not the tail's) the
        // caller's two-launch path. Lengths must be uniform so that every CTA of the grid arrives.
        if (p.kv_tokens || !p.output || (p.max_splits == 1u && !p.partial_output) || exchange->ranks > 128u) return 0;
        if ((unsigned long long)grid.x * grid.y * grid.z > (unsigned long long)resident_ctas) return 0;
        yvx_gqa_problem problem = p;
        yvx_lse_exchange x = *exchange;
        void *args[] = {&problem, &x};
        const cudaError_t launched = cudaLaunchCooperativeKernel((const void *)gqa_decode_q8_kernel, grid,
                                                                 dim3(kQ8Threads, 1, 1), args, kQ8SmemBytes, stream);
        if (launched != cudaSuccess) return yvx_cuda_check(launched, "gqa_decode_q8_kernel (cooperative)");
        return 3;  // launched, folded and exchanged: the output is final
    }
    yvx_lse_exchange none = {};
    gqa_decode_q8_kernel<<<grid, kQ8Threads, kQ8SmemBytes, stream>>>(p, none);
    const int rc = yvx_cuda_check(cudaGetLastError(), "gqa_decode_q8_kernel");
    return rc != 0 ? rc : 1;
}

// ---- packing GGUF Q8_0 rows into records ----------------------------------------

// One thread per (token, kv head, 32-lane block) of K and of V. Rows are GGUF
// Q8_0: [token][kv_heads * 4 blocks * 34 bytes].
__global__ void q8_kv_pack_kernel(const unsigned char *k_rows, const unsigned char *v_rows,
                                  unsigned int tokens, unsigned int kv_heads,
                                  unsigned char *records, const int *block_ids,
                                  unsigned long long block_stride, unsigned long long head_stride,
                                  unsigned int first_token)
{
    const unsigned long long index = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned long long total = (unsigned long long)tokens * kv_heads * 4ull;
    if (index >= total) return;
    const unsigned int db = (unsigned int)(index % 4ull);
    const unsigned int head = (unsigned int)((index / 4ull) % kv_heads);
    const unsigned int token = (unsigned int)(index / (4ull * kv_heads));
    const unsigned int absolute = first_token + token;
    const unsigned int block = absolute / 64u, t = absolute % 64u;
    const unsigned long long pool_block = block_ids ? (unsigned long long)block_ids[block] : block;
    unsigned char *record = records + pool_block * block_stride + (unsigned long long)head * head_stride;
    const unsigned long long source = ((unsigned long long)token * kv_heads + head) * 4ull * 34ull + db * 34ull;
    const unsigned char *kb = k_rows + source, *vb = v_rows + source;
    // scales
    record[kQ8KScales + (t * 4u + db) * 2u] = kb[0];
    record[kQ8KScales + (t * 4u + db) * 2u + 1u] = kb[1];
    {
        const unsigned int w = t / 16u, e = t % 16u, c = (e % 8u) / 2u, j = (e % 2u) + 2u * (e / 8u);
        const unsigned int at = kQ8VScales + (((w * 4u + c) * 4u + db) * 4u + j) * 2u;
        record[at] = vb[0];
        record[at + 1u] = vb[1];
    }
    for (unsigned int lane32 = 0; lane32 < 32u; ++lane32) {
        const unsigned int dim = db * 32u + lane32;
        {   // K: fragment order of the QK^T B operand
            const unsigned int nt = t / 8u, g = t % 8u, kg = dim / 64u, ks = (dim % 64u) / 16u;
            const unsigned int e = dim % 16u, c = (e % 8u) / 2u, j = (e % 2u) + 2u * (e / 8u);
            record[kQ8KLanes + ((nt * 2u + kg) * 32u + g * 4u + c) * 16u + ks * 4u + j] = kb[2u + lane32] ^ 0x80u;
        }
        {   // V: fragment order of the PV B operand
            const unsigned int w = t / 16u, e = t % 16u, c = (e % 8u) / 2u, j = (e % 2u) + 2u * (e / 8u);
            const unsigned int nd = dim / 8u, g = dim % 8u;
            record[kQ8VLanes + (((w * 4u + nd / 4u) * 32u + g * 4u + c) * 4u + nd % 4u) * 4u + j] = vb[2u + lane32] ^ 0x80u;
        }
    }
}

}  // namespace yvx

extern "C" {

unsigned long long yvx_cuda_q8_record_bytes(void) { return yvx::kQ8RecordBytes; }

int yvx_cuda_q8_kv_pack(const void *k_rows, const void *v_rows, unsigned int tokens,
                        unsigned int kv_heads, void *records, const int *block_ids,
                        unsigned long long block_stride, unsigned long long head_stride,
                        unsigned int first_token, void *stream)
{
    if (!k_rows || !v_rows || !records || !tokens || !kv_heads ||
        head_stride < (unsigned long long)yvx::kQ8RecordBytes ||
        block_stride < head_stride * kv_heads)
        return YVEX_ERR_INVALID_ARG;
    const unsigned long long total = (unsigned long long)tokens * kv_heads * 4ull;
    yvx::q8_kv_pack_kernel<<<(unsigned int)((total + 127ull) / 128ull), 128, 0, (cudaStream_t)stream>>>(
        (const unsigned char *)k_rows, (const unsigned char *)v_rows, tokens, kv_heads,
        (unsigned char *)records, block_ids, block_stride, head_stride, first_token);
    return yvx_cuda_check(cudaGetLastError(), "q8_kv_pack_kernel");
}

}  // extern "C"
