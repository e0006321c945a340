// Latent-compressed (MLA-style) decode on sm_100a: 128 query heads over one
// shared [latent 512 | rope 64] row per position, bf16, f32 accumulation.
//
// Arithmetic intensity sits at the machine's ridge (about 242 flop per byte),
// so the attention runs on the 5th-generation tensor cores with all 128 heads
// in the M dimension of one tcgen05.mma:
//   S[128 x 64]  = Q_abs[128 x 576] . K_tile^T          (36 k-steps of 128x64x16)
//   O[128 x 256] += P[128 x 64] . latent_tile[64 x 256]  (A = P in tensor memory)
// A 64-token tile is loaded ONCE into shared memory and serves as K (K-major)
// and as V (the same bytes read MN-major). The f32 output of 128 heads x 512
// dims would fill all of tensor memory, so a CTA owns one half of the latent
// dims (256 accumulator columns) and recomputes S; the two CTAs of a pair run
// side by side and share their tile through L2.
//
// Each stage of the two-stage tile ring has two parts with their own full /
// free barriers: the CTA's own latent half (32 KB: K of the last 16 k-steps and
// V of P V, free after P V) and the scores-only part (other half + rope, 40 KB,
// free after the first 20 k-steps). The matching query dims of the own half sit
// in tensor memory (128 columns), the rest in shared memory (80 KB). The score
// buffer is double: the tensor pipe runs S(j+1) part one, P(j) V(j), S(j+1)
// part two, so the softmax of tile j and the tile loads hide under the MMAs.
// Tensor memory map: O [0,256) | S0 [256,320) S1 [320,384), P(j) aliases the
// first 32 columns of S(j % 2) | Q [384,512).
#include <cstdlib>

#include "tcgen05.cuh"

namespace yvx {

constexpr int kMlaHeads = 128, kMlaNope = 128, kMlaLatent = 512, kMlaRope = 64;
constexpr int kMlaWidth = kMlaLatent + kMlaRope;          // 576
constexpr int kMlaN = 64;                                  // tokens per tile
constexpr int kMlaHalf = kMlaLatent / 2;                   // accumulator columns per CTA
constexpr int kMlaStages = 2;
constexpr int kMlaThreads = 320;   // 4 + 4 softmax warps, the TMA warp (4) and the MMA warp (5)
constexpr int kMlaQSubBytes = kMlaHeads * 64 * 2;          // [128][64] bf16 = 16 KB
constexpr int kMlaQTmemDims = kMlaHalf;                   // own-half query dims held in tensor memory                         // query dims held in tensor memory
constexpr int kMlaQSmemSubs = (kMlaWidth - kMlaQTmemDims) / 64;  // 5 sub-tiles stay in shared memory
constexpr int kMlaQBytes = kMlaQSmemSubs * kMlaQSubBytes;
constexpr int kMlaKvSubBytes = kMlaN * 64 * 2;             // [64][64] bf16 = 8 KB
constexpr int kMlaKvBytes = (kMlaWidth / 64) * kMlaKvSubBytes; // 72 KB
constexpr int kMlaVPartBytes = (kMlaHalf / 64) * kMlaKvSubBytes;    // own latent half, first in a stage
constexpr int kMlaKOnlyBytes = kMlaKvBytes - kMlaVPartBytes;       // other half + rope
constexpr int kMlaSmemBytes = kMlaQBytes + kMlaStages * kMlaKvBytes + 1024 + 256 + 1024;  // + the softmax halves' exchange
constexpr uint32_t kMlaTmemColumns = 512;
constexpr float kMlaRescaleThreshold = 8.0f;

#ifdef YVX_MLA_TRACE
// Cycle counters of CTA (0, 0, 0), a development aid compiled out of the library.
__device__ unsigned long long yvx_mla_trace[16];
__device__ unsigned long long yvx_mla_marks[16];
__device__ unsigned long long yvx_mla_spans[1024];
#define MLA_MARK(slot) do { if (traced && warp == 0) yvx_mla_marks[slot] = (unsigned long long)(clock64() - trace_start); } while (0)
#define MLA_TRACE_BEGIN(t) const long long t = clock64()
#define MLA_TRACE_ADD(slot, t) \
    do { if (traced) trace_local[slot] += (unsigned long long)(clock64() - t); } while (0)
#else
#define MLA_TRACE_BEGIN(t) do { } while (0)
#define MLA_MARK(slot) do { } while (0)
#define MLA_TRACE_ADD(slot, t) do { } while (0)
#endif

struct MlaMaps {
    CUtensorMap query, latent, rope;
    CUtensorMap weights;   // the four-CTA form's scratch slots: [slot][128 heads][64 tokens] bf16
};

struct MlaBarriers {
    uint64_t q_full, q_tmem_full;
    uint64_t ka_full[kMlaStages], kb_full[kMlaStages];  // scores-only part / own-half part loaded
    uint64_t ka_done[kMlaStages], v_done[kMlaStages];   // ... and free again
    uint64_t s_full[2], p_full[2];
    uint64_t pv_done;
    uint32_t tmem_base;
};
static_assert(sizeof(MlaBarriers) <= 256, "barrier block outgrew its shared-memory slot");
static_assert(kMlaStages == 2, "score buffers and stages are indexed by tile parity");

// ---- absorb: q_abs[b][h] = [ bf16(q_nope[b][h] . W_uk[h]) | q_rope[b][h] ] ----------
// grid (heads, 4 latent quarters): a CTA stages its [128 k][128 n] block of W_uk[head]
// (32 KB, all loads of a thread issued before its first store, so one round trip),
// then walks the sessions 16 at a time; warp w owns 32 of the quarter's columns.
// 512 small CTAs are all resident at once, so the 16.8 MB of W_uk stream in one wave.
constexpr int kAbsorbPitch = 128 * 2 + 16;  // padded row of 128 bf16
constexpr int kAbsorbSmem = 16 * kAbsorbPitch + 128 * kAbsorbPitch;

__global__ void __launch_bounds__(128)
mla_absorb_kernel(const yvx_mla_problem p)
{
    extern __shared__ unsigned char absorb_smem[];
    unsigned char *a_smem = absorb_smem;                       // [16 sessions][128 nope]
    unsigned char *w_smem = absorb_smem + 16 * kAbsorbPitch;   // [128 k][128 n]
    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned int head = blockIdx.x, quarter = blockIdx.y;
    const __nv_bfloat16 *q_nope = reinterpret_cast<const __nv_bfloat16 *>(p.q_nope);
    const __nv_bfloat16 *w = reinterpret_cast<const __nv_bfloat16 *>(p.w_uk) +
                             (unsigned long long)head * kMlaNope * kMlaLatent + quarter * 128u;
    // A thread's two chunks of the next 16 sessions' query rows (16 rows x 16 chunks of 16 bytes), asked for a
    // tile ahead; the first tile's and the rope chunks travel together with the weights.
    uint4 a_next[2];
    auto load_a = [&](unsigned int session0) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const unsigned int i = threadIdx.x + 128u * u, row = i >> 4, chunk = i & 15u;
            a_next[u] = make_uint4(0u, 0u, 0u, 0u);
            if (session0 + row < p.sessions)
                a_next[u] = *reinterpret_cast<const uint4 *>(
                    q_nope + ((unsigned long long)(session0 + row) * kMlaHeads + head) * kMlaNope + chunk * 8u);
        }
    };
    const unsigned short *q_rope = reinterpret_cast<const unsigned short *>(p.q_rope);
    uint4 rope_first[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
    {
        uint4 staged[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const unsigned int i = threadIdx.x + 128u * u, k = i >> 4, chunk = i & 15u;
            staged[u] = *reinterpret_cast<const uint4 *>(w + (unsigned long long)k * kMlaLatent + chunk * 8u);
        }
        load_a(0u);
        if (quarter == 0u) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const unsigned int i = threadIdx.x + 128u * u;
                if (i < p.sessions * 8u)
                    rope_first[u] = *reinterpret_cast<const uint4 *>(
                        q_rope + ((unsigned long long)(i >> 3) * kMlaHeads + head) * kMlaRope + (i & 7u) * 8u);
            }
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const unsigned int i = threadIdx.x + 128u * u, k = i >> 4, chunk = i & 15u;
            *reinterpret_cast<uint4 *>(w_smem + k * kAbsorbPitch + chunk * 16u) = staged[u];
        }
    }
    unsigned short *out = reinterpret_cast<unsigned short *>(p.q_absorbed);
    const unsigned int g = lane >> 2, c = lane & 3u;
    for (unsigned int session0 = 0; session0 < p.sessions; session0 += 16u) {
        __syncthreads();  // the previous tile's fragments have been read (and W is staged)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const unsigned int i = threadIdx.x + 128u * u, row = i >> 4, chunk = i & 15u;
            *reinterpret_cast<uint4 *>(a_smem + row * kAbsorbPitch + chunk * 16u) = a_next[u];
        }
        if (session0 + 16u < p.sessions) load_a(session0 + 16u);   // in flight under this tile's products
        __syncthreads();
        uint32_t qa[8][4];
        const unsigned int j = lane >> 3, i8 = lane & 7u;
        {
            const uint32_t base = smem_u32(a_smem) + (8u * (j & 1u) + i8) * kAbsorbPitch + 16u * (j >> 1);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) ldmatrix_x4(qa[ks], base + ks * 32u);
        }
        float acc[4][4];
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[n][e] = 0.0f;
        const uint32_t wbase = smem_u32(w_smem) + warp * 64u;  // this warp's 32 columns
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, wbase + (16u * ks + 8u * (j & 1u) + i8) * kAbsorbPitch +
                                         (16u * np + 8u * (j >> 1)) * 2u);
                mma_bf16(acc[2 * np], qa[ks], b[0], b[1]);
                mma_bf16(acc[2 * np + 1], qa[ks], b[2], b[3]);
            }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const unsigned int session = session0 + g + 8u * h;
            if (session >= p.sessions) continue;
            unsigned short *dst = out + ((unsigned long long)session * kMlaHeads + head) * kMlaWidth +
                                  quarter * 128u + warp * 32u;
#pragma unroll
            for (int n = 0; n < 4; ++n)
                *reinterpret_cast<uint32_t *>(dst + 8 * n + 2 * c) = pack_bf16(acc[n][2 * h], acc[n][2 * h + 1]);
        }
    }
    // rope part: copied through by the first quarter's CTA
    if (quarter == 0u) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const unsigned int i = threadIdx.x + 128u * u;
            if (i < p.sessions * 8u)
                *reinterpret_cast<uint4 *>(out + ((unsigned long long)(i >> 3) * kMlaHeads + head) * kMlaWidth + kMlaLatent +
                                           (i & 7u) * 8u) = rope_first[u];
        }
        for (unsigned int i = threadIdx.x + 256u; i < p.sessions * 8u; i += 128u) {
            const unsigned int row = i >> 3, chunk = i & 7u;
            const unsigned long long item = (unsigned long long)row * kMlaHeads + head;
            *reinterpret_cast<uint4 *>(out + item * kMlaWidth + kMlaLatent + chunk * 8u) =
                *reinterpret_cast<const uint4 *>(q_rope + item * kMlaRope + chunk * 8u);
        }
    }
}

// ---- attention: grid (2 latent halves, splits, sessions) -----------------------------
__global__ void __launch_bounds__(kMlaThreads, 1)
mla_decode_tcgen05_kernel(const yvx_mla_problem p, const __grid_constant__ MlaMaps maps)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    unsigned char *q_tile = smem;
    unsigned char *kv_tiles = smem + kMlaQBytes;
    MlaBarriers *bars = reinterpret_cast<MlaBarriers *>(kv_tiles + kMlaStages * kMlaKvBytes);

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned int half = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
#ifdef YVX_MLA_TRACE
    const bool traced = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0;
    unsigned long long trace_local[4] = {0, 0, 0, 0};
    const long long trace_start = clock64();
#endif
    const unsigned int kv_tokens = admitted_kv_tokens(p.kv_tokens, b, p.kv_tokens_uniform, p.kv_tokens_max, p.status);
    const unsigned int t0 = split * p.chunk_tokens;
    const unsigned int t1 = min(kv_tokens, t0 + p.chunk_tokens);
    const unsigned long long part_stride = kMlaHalf + 2;
    if (t0 >= t1) {
        // Nothing of this session falls into the split: publish an empty partial.
        if (threadIdx.x < (unsigned)kMlaHeads) {
            float *part = p.partials +
                          ((((unsigned long long)b * kMlaHeads + threadIdx.x) * 2ull + half) * p.max_splits + split) *
                              part_stride;
            for (int d = 0; d < kMlaHalf; ++d) part[d] = 0.0f;
            part[kMlaHalf] = -INFINITY;
            part[kMlaHalf + 1] = 0.0f;
        }
        return;
    }
    const unsigned int tiles = (t1 - t0 + kMlaN - 1) / kMlaN;
    // Sub-tile (64 dims) indices: this CTA's own latent half, and the other one.
    const int own0 = 4 * (int)half, other0 = 4 * (1 - (int)half);

    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, 1);
        mbar_init(&bars->q_tmem_full, kMlaHeads);
        for (int i = 0; i < kMlaStages; ++i) {
            mbar_init(&bars->ka_full[i], 1);
            mbar_init(&bars->kb_full[i], 1);
            mbar_init(&bars->ka_done[i], 1);
            mbar_init(&bars->v_done[i], 1);
            mbar_init(&bars->s_full[i], 1);
            mbar_init(&bars->p_full[i], 2 * kMlaHeads);
        }
        mbar_init(&bars->pv_done, 1);
        fence_barrier_init();
    }
    if (warp == 5) {
        tmem_alloc(&bars->tmem_base, kMlaTmemColumns);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = bars->tmem_base;
    const uint32_t tmem_o = tmem, tmem_s = tmem + kMlaHalf, tmem_q = tmem + kMlaHalf + 2 * kMlaN;

    if (warp == 4) {
        // ------------------------------ TMA producer ------------------------------
        // Two lanes, one per part of a stage, each with its own free barrier: the scores-only
        // part of tile j + 2 is requested as soon as the first 20 k-steps of tile j have run,
        // without queueing behind the own-half part, which has to wait for P V of tile j.
        if (lane == 0) {
            mbar_expect_tx(&bars->q_full, kMlaQBytes);
            for (int u = 0; u < kMlaQSmemSubs; ++u)
                tma_load_3d(q_tile + u * kMlaQSubBytes, &maps.query, &bars->q_full,
                            u < 4 ? 64 * (other0 + u) : kMlaLatent, 0, (int)b);
            for (unsigned int j = 0; j < tiles; ++j) {
                const unsigned int stage = j % kMlaStages;
                const uint32_t parity = ((j / kMlaStages) - 1u) & 1u;
                unsigned char *dst = kv_tiles + stage * kMlaKvBytes;
                const int token = (int)(t0 + j * kMlaN);
                MLA_TRACE_BEGIN(tp0);
                if (j >= (unsigned)kMlaStages && !mbar_wait(&bars->ka_done[stage], parity)) {
                    atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
                    break;
                }
                MLA_TRACE_ADD(0, tp0);
                mbar_expect_tx(&bars->ka_full[stage], kMlaKOnlyBytes);
                for (int u = 0; u < 4; ++u)
                    tma_load_3d(dst + kMlaVPartBytes + u * kMlaKvSubBytes, &maps.latent,
                                &bars->ka_full[stage], 64 * (other0 + u), token, (int)b);
                tma_load_3d(dst + kMlaVPartBytes + 4 * kMlaKvSubBytes, &maps.rope, &bars->ka_full[stage], 0,
                            token, (int)b);
            }
#ifdef YVX_MLA_TRACE
            if (traced) yvx_mla_trace[0] = trace_local[0];   // producer: waiting for a scores-only part to free
#endif
        } else if (lane == 1) {
            for (unsigned int j = 0; j < tiles; ++j) {
                const unsigned int stage = j % kMlaStages;
                const uint32_t parity = ((j / kMlaStages) - 1u) & 1u;
                unsigned char *dst = kv_tiles + stage * kMlaKvBytes;
                const int token = (int)(t0 + j * kMlaN);
                // Own latent half: K of the last 16 k-steps and V of P V; free after P V.
                if (j >= (unsigned)kMlaStages && !mbar_wait(&bars->v_done[stage], parity)) {
                    atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
                    break;
                }
                mbar_expect_tx(&bars->kb_full[stage], kMlaVPartBytes);
                for (int u = 0; u < 4; ++u)
                    tma_load_3d(dst + u * kMlaKvSubBytes, &maps.latent, &bars->kb_full[stage],
                                64 * (own0 + u), token, (int)b);
            }
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer --------------------------------
        // All 32 lanes run the loop converged; one elected lane issues each instruction.
        constexpr uint32_t idesc_qk = idesc_bf16_f32(kMlaHeads, kMlaN, false);
        constexpr uint32_t idesc_pv = idesc_bf16_f32(kMlaHeads, kMlaHalf, true);
        const uint32_t q_addr = smem_u32(q_tile);
        const uint32_t elected = tc_elect_one() ? 1u : 0u;   // the one lane that issues everything below
        constexpr uint32_t desc_hi = smem_desc_sw128_hi(1024);
        // First 20 k-steps of S(j): the other latent half and the rope dims, both
        // operands in shared memory. Frees the scores-only part of the stage.
        auto qk_a = [&](unsigned int j) -> bool {
            const unsigned int stage = j % kMlaStages;
            MLA_TRACE_BEGIN(tm0);
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->ka_full[stage], (j / kMlaStages) & 1u))) return false;
            MLA_TRACE_ADD(0, tm0);
            tc_fence_after_sync();
            const uint32_t k_addr = smem_u32(kv_tiles + stage * kMlaKvBytes + kMlaVPartBytes);
#ifdef YVX_MLA_TRACE
            const long long issue_start = clock64();
#endif
            {
                const uint32_t a_lo = smem_desc_sw128_lo(q_addr, 16), b_lo = smem_desc_sw128_lo(k_addr, 16);
#pragma unroll
                for (int ks = 0; ks < 4 * kMlaQSmemSubs; ++ks) {
                    const uint32_t off = (ks & 3) * 32;
                    tc_mma_ss_pred(elected, tmem_s + (j & 1u) * kMlaN, a_lo + (((ks >> 2) * kMlaQSubBytes + off) >> 4), desc_hi,
                                   b_lo + (((ks >> 2) * kMlaKvSubBytes + off) >> 4), desc_hi, idesc_qk, ks ? 1u : 0u);
                }
                tc_commit_pred(elected, &bars->ka_done[stage]);
            }
#ifdef YVX_MLA_TRACE
            if (traced && j == 0) yvx_mla_trace[12] = (unsigned long long)(clock64() - issue_start);   // 20 issues, idle pipe
            if (traced && j == 40) yvx_mla_trace[13] = (unsigned long long)(clock64() - issue_start);  // 20 issues, steady state
#endif
            return true;
        };
        // Last 16 k-steps: this CTA's own latent half, query operand in tensor memory.
        auto qk_b = [&](unsigned int j) -> bool {
            const unsigned int stage = j % kMlaStages;
            MLA_TRACE_BEGIN(tm1);
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->kb_full[stage], (j / kMlaStages) & 1u))) return false;
            MLA_TRACE_ADD(1, tm1);
            tc_fence_after_sync();
            const uint32_t k_addr = smem_u32(kv_tiles + stage * kMlaKvBytes);
            {
                const uint32_t b_lo = smem_desc_sw128_lo(k_addr, 16);
#pragma unroll
                for (int ks = 0; ks < kMlaQTmemDims / 16; ++ks)
                    tc_mma_ts_pred(elected, tmem_s + (j & 1u) * kMlaN, tmem_q + ks * 8,
                                   b_lo + (((ks >> 2) * kMlaKvSubBytes + (ks & 3) * 32) >> 4), desc_hi, idesc_qk, 1u);
                tc_commit_pred(elected, &bars->s_full[j & 1u]);
            }
            return true;
        };
        auto pv = [&](unsigned int j) -> bool {
            const unsigned int stage = j % kMlaStages;
            MLA_TRACE_BEGIN(tm2);
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->p_full[j & 1u], (j >> 1) & 1u))) return false;
            MLA_TRACE_ADD(2, tm2);
            tc_fence_after_sync();
            const uint32_t v_addr = smem_u32(kv_tiles + stage * kMlaKvBytes);
            {
                const uint32_t b_lo = smem_desc_sw128_lo(v_addr, kMlaKvSubBytes);
#pragma unroll
                for (int kk = 0; kk < kMlaN / 16; ++kk)
                    tc_mma_ts_pred(elected, tmem_o, tmem_s + (j & 1u) * kMlaN + kk * 8, b_lo + ((kk * 2048) >> 4), desc_hi,
                                   idesc_pv, (j || kk) ? 1u : 0u);
                tc_commit_pred(elected, &bars->v_done[stage]);
                tc_commit_pred(elected, &bars->pv_done);
            }
            return true;
        };
        bool ok = __all_sync(0xffffffffu, mbar_wait(&bars->q_full, 0)) &&
                  __all_sync(0xffffffffu, mbar_wait(&bars->q_tmem_full, 0));
        ok = ok && qk_a(0) && qk_b(0);
        // Tensor-pipe order per tile: S(j+1) first part, then whichever of the two is ready
        // first: S(j+1) second part (its own-half load had to wait for P V of tile j-1) or
        // P(j) V(j) (the softmax of tile j). With the second part first the softmax of tile j
        // has all of S(j+1) to hide under, and that of tile j+1 starts under P(j) V(j).
        for (unsigned int j = 0; ok && j < tiles; ++j) {
            bool scores_first = false;
            if (j + 1 < tiles) {
                ok = qk_a(j + 1);
                const unsigned int next = j + 1u;
                for (uint32_t spin = 0; ok && spin < kWaitSpinLimit; ++spin) {
                    const bool loaded = mbar_test(&bars->kb_full[next % kMlaStages], (next / kMlaStages) & 1u);
                    const bool weights = mbar_test(&bars->p_full[j & 1u], (j >> 1) & 1u);
                    if (__any_sync(0xffffffffu, loaded)) {
                        scores_first = true;
#ifdef YVX_MLA_TRACE
                        trace_local[3] += 1ull;
#endif
                        break;
                    }
                    if (__any_sync(0xffffffffu, weights)) break;
                }
            }
            if (scores_first) ok = ok && qk_b(j + 1) && pv(j);
            else {
                ok = ok && pv(j);
                if (ok && j + 1 < tiles) ok = qk_b(j + 1);
            }
        }
        if (!ok && lane == 0) atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
#ifdef YVX_MLA_TRACE
        if (traced) {
            yvx_mla_trace[2] = trace_local[0];   // issuer: waiting for a scores-only part to land
            yvx_mla_trace[3] = trace_local[1];   // issuer: waiting for an own-half part to land
            yvx_mla_trace[4] = trace_local[2];   // issuer: waiting for the softmax weights
            yvx_mla_trace[5] = trace_local[3];   // tiles whose second score part went first
            yvx_mla_trace[6] = (unsigned long long)(clock64() - trace_start);
            yvx_mla_trace[7] = tiles;
        }
#endif
    } else {
        // ------------------------------ softmax warps -----------------------------
        // Two warps per 32 heads: warps 0-3 take the first 32 tokens of every tile (and the
        // first half of the accumulator columns), warps 6-9 the last 32 (and the second half).
        // A warp reaches the tensor-memory lanes 32 * (warp % 4) ..., so the partner of warp w
        // is the warp of the other group with the same w % 4; the two meet at a named barrier
        // per tile to agree on the row maximum.
        const unsigned int side = warp < 4u ? 0u : 1u, quadrant = warp & 3u;
        const unsigned int head = quadrant * 32u + lane;
        const uint32_t lane_base = ((quadrant * 32u) << 16);
        float *exchange = reinterpret_cast<float *>(bars + 1);    // [2 sides][128 heads]
        if (side == 0u) {
            // This head's absorbed-query dims of the CTA's own latent half go to tensor
            // memory: bf16 pairs are already the 32-bit words the A operand wants.
            const uint4 *src = reinterpret_cast<const uint4 *>(
                reinterpret_cast<const unsigned short *>(p.q_absorbed) +
                ((unsigned long long)b * kMlaHeads + head) * kMlaWidth + (unsigned long long)half * kMlaHalf);
            // All 32 loads are issued before the first store so they share one round trip.
            uint4 v[kMlaQTmemDims / 8];
#pragma unroll
            for (int c = 0; c < kMlaQTmemDims / 8; ++c) v[c] = src[c];
#pragma unroll
            for (int i = 0; i < kMlaQTmemDims / 64; ++i) {
                uint32_t words[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    words[4 * c] = v[8 * i + c].x;
                    words[4 * c + 1] = v[8 * i + c].y;
                    words[4 * c + 2] = v[8 * i + c].z;
                    words[4 * c + 3] = v[8 * i + c].w;
                }
                tmem_st32(tmem_q + lane_base + 32 * i, words);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&bars->q_tmem_full);
        }
        const float sscale = p.scale * 1.4426950408889634f;
        float m_used = -INFINITY, l = 0.0f;
        bool ok = true;
        for (unsigned int j = 0; j < tiles; ++j) {
            const uint32_t s_col = tmem_s + lane_base + (j & 1u) * kMlaN;
            MLA_TRACE_BEGIN(ts0);
            if (!mbar_wait(&bars->s_full[j & 1u], (j >> 1) & 1u)) {
                ok = false;
                break;
            }
            MLA_TRACE_ADD(0, ts0);
            MLA_TRACE_BEGIN(ts1);
            tc_fence_after_sync();
            uint32_t s[32];
            tmem_ld32(s_col + 32u * side, s);
            tmem_wait_ld();
            const unsigned int k0 = t0 + j * kMlaN + 32u * side;
            if (k0 + 32u > t1) {
#pragma unroll
                for (int c = 0; c < 32; ++c)
                    if (k0 + c >= t1) s[c] = 0xff800000u;  // -inf
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 32; c += 2)
                mx[(c >> 1) & 3] = max3(mx[(c >> 1) & 3], __uint_as_float(s[c]), __uint_as_float(s[c + 1]));
            // both halves of the row have been read (the weights of one half overwrite score
            // columns of the other) and the row maximum is the larger of the two halves'
            if (j > 0) named_barrier(2 + (int)quadrant, 64);   // the partner has read the previous tile's maximum
            exchange[side * kMlaHeads + head] = max3(mx[0], mx[1], fmaxf(mx[2], mx[3]));
            named_barrier(2 + (int)quadrant, 64);
            const float row_max = fmaxf(exchange[head], exchange[kMlaHeads + head]);
            const float m_tile = row_max * sscale;
            const bool grow = m_tile > m_used + kMlaRescaleThreshold || m_used == -INFINITY;
            // the same rows on both sides: the partner warp takes the same branch
            if (__any_sync(0xffffffffu, grow)) {
#ifdef YVX_MLA_TRACE
                trace_local[2] += 1ull;
#endif
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
#pragma unroll 1
                    for (int i = 0; i < kMlaHalf / 64; ++i) {
                        uint32_t o[32];
                        const uint32_t column = tmem_o + lane_base + 128u * side + 32u * i;
                        tmem_ld32(column, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * factor);
                        tmem_st32(column, o);
                    }
                    tmem_wait_st();
                }
            }
            const float offset = m_used == -INFINITY ? 0.0f : -m_used;
            uint32_t packed[16];
            float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
                const float p0 = exp2_approx(fmaf(__uint_as_float(s[c]), sscale, offset));
                const float p1 = exp2_approx(fmaf(__uint_as_float(s[c + 1]), sscale, offset));
                sum0 += p0;
                sum1 += p1;
                packed[c >> 1] = pack_bf16(p0, p1);
            }
            l += sum0 + sum1;
            tmem_st16(s_col + 16u * side, packed);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&bars->p_full[j & 1u]);
            MLA_TRACE_ADD(1, ts1);
        }
#ifdef YVX_MLA_TRACE
        if (traced && warp == 0) {
            yvx_mla_trace[8] = trace_local[0];   // softmax warp 0: waiting for scores
            yvx_mla_trace[9] = trace_local[1];   // softmax warp 0: scores to weights
            yvx_mla_trace[10] = trace_local[2];  // tiles that rescaled the accumulator
            yvx_mla_trace[11] = (unsigned long long)(clock64() - trace_start);
        }
#endif
        if (ok) ok = mbar_wait(&bars->pv_done, (tiles - 1u) & 1u);
        // The tile loop is over: let the combine kernel's launch overlap the epilogue.
        pdl_launch_dependents();
        // A wait that gave up is recorded; the rows are still written out so that
        // every softmax thread reaches the named barriers below exactly once.
        if (!__all_sync(0xffffffffu, ok)) atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
        {
            tc_fence_after_sync();
            // the row's denominator is the sum of the two halves'
            named_barrier(2 + (int)quadrant, 64);          // the last tile's maxima have been read
            exchange[side * kMlaHeads + head] = l;
            named_barrier(2 + (int)quadrant, 64);
            l = exchange[head] + exchange[kMlaHeads + head];
            const float inverse = l > 0.0f ? 1.0f / l : 0.0f;
            // Every tile has been consumed, so the tile ring is free: the normalised
            // rows go through it, and each warp then writes whole partial rows with
            // coalesced 8-byte stores (a partial row is 8-byte aligned only).
            float *staged = reinterpret_cast<float *>(kv_tiles);
            float *mine = staged + head * (unsigned)part_stride + 128u * side;
#pragma unroll 1
            for (int i = 0; i < kMlaHalf / 64; ++i) {
                uint32_t o[32];
                tmem_ld32(tmem_o + lane_base + 128u * side + 32 * i, o);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; c += 2)
                    *reinterpret_cast<float2 *>(mine + 32 * i + c) =
                        make_float2(__uint_as_float(o[c]) * inverse, __uint_as_float(o[c + 1]) * inverse);
            }
            if (side == 1u)
                *reinterpret_cast<float2 *>(staged + head * (unsigned)part_stride + kMlaHalf) =
                    make_float2(m_used == -INFINITY ? -INFINITY : m_used * 0.6931471805599453f, l);
            named_barrier(1, 2 * kMlaHeads);
            const unsigned int writer = side * 4u + quadrant;
            for (unsigned int r = writer; r < (unsigned)kMlaHeads; r += 8u) {
                float2 *dst = reinterpret_cast<float2 *>(
                    p.partials +
                    ((((unsigned long long)b * kMlaHeads + r) * 2ull + half) * p.max_splits + split) * part_stride);
                const float2 *src = reinterpret_cast<const float2 *>(staged + r * (unsigned)part_stride);
                for (unsigned int k = lane; k < (unsigned)part_stride / 2u; k += 32u) dst[k] = src[k];
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem, kMlaTmemColumns);
}

// ---- attention, paired form: a cluster of two CTAs computes every score tile ONCE ------------
// The two CTAs of a (session, split) still own one latent half of the output each, but they take
// turns at the score product: CTA r computes S = Q K^T and the softmax of the tiles j with j % 2 == r
// and hands the weights P(j) (bf16, the operand layout of the P V product) to its peer through
// distributed shared memory, with the running row maximum it used. Both run P(j) V(j) of EVERY tile
// on their own 256 accumulator columns, A = P from shared memory. Per pair of tiles a CTA issues
// one score product and two P V products instead of two and two.
//
// Shared memory (one CTA per SM): query dims that do not fit tensor memory (3 sub-tiles, 48 KB);
// for the tiles this CTA scores the scores-only part (other latent half + rope, 40 KB, one buffer)
// and the own-half part (32 KB: K of the last k-steps and V of P V, two buffers); for the peer's
// tiles the own-half part alone (V, 32 KB); P of an own tile and P of a peer tile (16 KB each).
// Tensor memory: O 256 | S 64 | Q 192 (384 query dims: the own half and 128 dims of the other).
//
// The row maximum is one sequence for both CTAs (their accumulators must carry the same scale):
// a CTA processes the peer's message for tile j - 1 (adopting its maximum, rescaling O and l if
// it grew) before it computes the weights of tile j. Every wait is bounded and gives up at once
// when either CTA has recorded a failure; both CTAs always reach the cluster barrier at the end.
constexpr int kPairThreads = 320;   // 4 softmax warps (0-3), three TMA warps (4, 6, 7), two MMA warps (5: scores, 9: P V), the sender (8)
constexpr int kPairQSmemSubs = 3, kPairQTmemCols = 192;
constexpr int kPairOffQ = 0;
constexpr int kPairOffKa = kPairQSmemSubs * kMlaQSubBytes;            // 49152
constexpr int kPairKaBytes = 5 * kMlaKvSubBytes;                       // 40960
constexpr int kPairOffKb = kPairOffKa + kPairKaBytes;                  // 90112
constexpr int kPairOffV = kPairOffKb + kMlaVPartBytes;                 // 122880: two own-half parts as V of P V
constexpr int kPairOffPOwn = kPairOffV + 2 * kMlaVPartBytes;           // 188416
constexpr int kPairPBytes = kMlaHeads * kMlaN * 2;                     // 16384
constexpr int kPairOffPPeer = kPairOffPOwn + kPairPBytes;              // 204800
constexpr int kPairOffTail = kPairOffPPeer + kPairPBytes;              // 221184
constexpr int kPairSmemBytes = kPairOffTail + 256 + 4 * 1024 + 1024;   // barriers, 4 float boxes, alignment

struct PairBarriers {
    uint64_t q_full, q_tmem_full;
    uint64_t ka_full, ka_done;            // scores-only part of an own tile: loaded / free again
    uint64_t kb_full, kb_done;            // own-half part of an own tile, as K of its score product
    uint64_t v_full[2], v_done[2];        // own-half part of ANY tile, as V of its P V (two slots, tile parity)
    uint64_t s_full, s_free;              // scores computed / read out of tensor memory
    uint64_t p_own_full, pv_own_done;     // weights of an own tile written / consumed
    uint64_t p_peer_full, peer_ready;     // the peer's weights have arrived / its message is processed
    uint64_t p_peer_free;                 // the peer has consumed the weights this CTA sent it
    uint64_t p_written, p_own_sent;       // an own tile's weights are written / have left for the peer
    uint64_t pv_done;                     // any P V
    uint64_t ka2_full, ka2_done;          // ... its second piece (two sub-tiles of the other half and the rope keys)
    uint64_t rows_staged;                 // all rows of the result are staged
    uint32_t tmem_base;
    int abort;
};
constexpr unsigned int kPairBarrierCount = 23u;   // the 64-bit barrier words above, from q_full on
static_assert(offsetof(PairBarriers, tmem_base) == kPairBarrierCount * 8u, "barrier count out of step");
static_assert(sizeof(PairBarriers) <= 256, "barrier block outgrew its shared-memory slot");

__device__ __forceinline__ uint32_t cluster_map(uint32_t local_address, uint32_t rank)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_address), "r"(rank));
    return remote;
}
__device__ __forceinline__ void cluster_store_v4(uint32_t address, uint4 v)
{
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ void cluster_store_f32(uint32_t address, float v)
{
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(address), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_store_b32(uint32_t address, uint32_t v)
{
    asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(address), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_arrive_remote(uint32_t barrier_address)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(barrier_address) : "memory");
}
// ... where the arrival publishes nothing of this thread's (a credit): no release to wait for
__device__ __forceinline__ void cluster_arrive_remote_relaxed(uint32_t barrier_address)
{
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(barrier_address) : "memory");
}
// Bulk copy from this CTA's shared memory into the peer's, completion counted in bytes on a barrier of the peer.
__device__ __forceinline__ void cluster_bulk_copy(uint32_t peer_destination, const void *source, uint32_t bytes,
                                                  uint32_t peer_barrier)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(peer_destination), "r"(smem_u32(source)), "r"(bytes), "r"(peer_barrier)
        : "memory");
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Bounded wait that also ends when either CTA has given up; acquire at cluster scope (a peer's
// arrival publishes its stores into this CTA's shared memory).
__device__ __forceinline__ bool pair_wait(uint64_t *bar, uint32_t parity, const volatile int *abort)
{
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < kWaitSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if ((spin & 255u) == 255u && *abort) return false;
    }
    return false;
}
// The same for a barrier that only this CTA's threads, bulk copies and tensor-pipe commits arrive on: acquire at
// CTA scope (the cluster-scope acquire costs every look at a barrier some hundred cycles more).
__device__ __forceinline__ bool local_wait(uint64_t *bar, uint32_t parity, const volatile int *abort)
{
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < kWaitSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if ((spin & 255u) == 255u && *abort) return false;
    }
    return false;
}

// ---- the balanced plan (uniform lengths) --------------------------------------------------------------------
// The sessions' tiles are laid end to end with kMlaItemCostTiles cost units in front of each session (what a
// work item costs besides its tiles: query staging, the first tile's latency, writing its partial rows), and
// the pairs take equal runs of that cost line: pair k the units [k * total / pairs, (k + 1) * total / pairs).
// What a run holds of a session's tiles is one work item; the items of a session are numbered from the pair
// that holds its first tile, and that number is the item's partial slot.
constexpr unsigned int kMlaItemCostTiles = 10u;

struct MlaBalance {
    unsigned long long total, unit;   // cost units: all sessions, one session
    unsigned int pairs;
};

__host__ __device__ inline MlaBalance mla_balance(unsigned int sessions, unsigned int kv_tokens, unsigned int pairs)
{
    MlaBalance g;
    g.unit = kMlaItemCostTiles + (kv_tokens + (unsigned)kMlaN - 1u) / (unsigned)kMlaN;
    g.total = g.unit * sessions;
    g.pairs = pairs;
    return g;
}

__host__ __device__ inline unsigned long long mla_run_begin(const MlaBalance &g, unsigned long long k)
{
    return g.total * k / g.pairs;
}

// What pair k holds of session b: tiles [*tile_lo, *tile_hi), partial slot, whether it ends the session.
__host__ __device__ inline bool mla_balanced_item(const MlaBalance &g, unsigned int k, unsigned int b,
                                                  unsigned int *tile_lo, unsigned int *tile_hi,
                                                  unsigned int *slot, bool *ends_session)
{
    const unsigned long long lo = mla_run_begin(g, k), hi = mla_run_begin(g, k + 1ull);
    const unsigned long long seg_lo = g.unit * b + kMlaItemCostTiles, seg_hi = g.unit * (b + 1ull);
    const unsigned long long a = lo > seg_lo ? lo : seg_lo, e = hi < seg_hi ? hi : seg_hi;
    if (a >= e) return false;
    unsigned long long first = seg_lo * g.pairs / g.total;       // the pair whose run holds the session's first tile
    while (mla_run_begin(g, first + 1ull) <= seg_lo) ++first;
    while (mla_run_begin(g, first) > seg_lo) --first;
    *tile_lo = (unsigned int)(a - seg_lo);
    *tile_hi = (unsigned int)(e - seg_lo);
    *slot = k - (unsigned int)first;
    *ends_session = hi >= seg_hi;
    return true;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
mla_decode_pair_kernel(const yvx_mla_problem p, const __grid_constant__ MlaMaps maps)
{
    extern __shared__ unsigned char pair_smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(pair_smem_raw) + 1023u) & ~uintptr_t(1023));
    PairBarriers *bars = reinterpret_cast<PairBarriers *>(smem + kPairOffTail);
    float *exchange = reinterpret_cast<float *>(smem + kPairOffTail + 256);   // [2 sides][128]: the halves' row maxima
    float *m_box = exchange + 2 * kMlaHeads;                                  // [128]: the peer's maximum after its tile
    float *l_box = m_box + 2 * kMlaHeads;                                     // [2 sides][128]: the peer's denominators
    float *m_out = l_box + 2 * kMlaHeads;                                     // [128]: this CTA's maximum, source of the copy to the peer

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned int half = blockIdx.x;   // half == rank in the cluster
    const unsigned int peer = half ^ 1u;
#ifdef YVX_MLA_TRACE
    const bool traced = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0;
    unsigned long long trace_local[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const long long trace_start = clock64();
    const unsigned int span_index = (blockIdx.z * gridDim.y + blockIdx.y) * 2u + blockIdx.x;
    if (threadIdx.x == 0 && span_index < 512u) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        unsigned int smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        yvx_mla_spans[2u * span_index] = (now << 10) | smid;
    }
#endif
    const unsigned long long part_stride = kMlaHalf + 2;
    const bool balanced = p.balanced_pairs != 0u;
    const MlaBalance balance = mla_balance(p.sessions, p.kv_tokens_uniform, balanced ? p.balanced_pairs : 1u);
    if (!balanced) {
        const unsigned int kv_tokens =
            admitted_kv_tokens(p.kv_tokens, blockIdx.z, p.kv_tokens_uniform, p.kv_tokens_max, p.status);
        if (blockIdx.y * p.chunk_tokens >= kv_tokens) {
            // Nothing of this session falls into the split (true for both CTAs of the pair): an empty partial.
            if (threadIdx.x < (unsigned)kMlaHeads) {
                float *part = p.partials + ((((unsigned long long)blockIdx.z * kMlaHeads + threadIdx.x) * 2ull + half) *
                                                p.max_splits + blockIdx.y) * part_stride;
                for (int d = 0; d < kMlaHalf; ++d) part[d] = 0.0f;
                part[kMlaHalf] = -INFINITY;
                part[kMlaHalf + 1] = 0.0f;
            }
            return;
        }
    }
    volatile int *abort = &bars->abort;
    if (threadIdx.x == 0) bars->abort = 0;
    if (warp == 5) {
        tmem_alloc(&bars->tmem_base, kMlaTmemColumns);
        tmem_relinquish();
    }
    // The work items of this pair: one (its session and split) in the grid of sessions x splits; in the balanced
    // plan what its run of the cost line holds of each session it touches, one after the other.
    const unsigned int session_first =
        balanced ? (unsigned int)(mla_run_begin(balance, blockIdx.y) / balance.unit) : blockIdx.z;
    const unsigned int session_last =
        balanced ? (unsigned int)min((unsigned long long)p.sessions - 1ull,
                                     (mla_run_begin(balance, blockIdx.y + 1ull) + balance.unit - 1ull) / balance.unit)
                 : blockIdx.z;
    bool first_item = true;
    for (unsigned int b = session_first; b <= session_last; ++b) {
    unsigned int split = blockIdx.y, t0, t1;
    bool ends_session = false;
    if (balanced) {
        unsigned int tile_lo, tile_hi;
        if (!mla_balanced_item(balance, blockIdx.y, b, &tile_lo, &tile_hi, &split, &ends_session)) continue;
        t0 = tile_lo * kMlaN;
        t1 = min(p.kv_tokens_uniform, tile_hi * (unsigned)kMlaN);
    } else {
        const unsigned int kv_tokens = admitted_kv_tokens(p.kv_tokens, b, p.kv_tokens_uniform, p.kv_tokens_max, p.status);
        t0 = split * p.chunk_tokens;
        t1 = min(kv_tokens, t0 + p.chunk_tokens);
    }
    if (!first_item) {
        // The item before has ended at a cluster barrier with nothing pending on any barrier of either CTA
        // (every role has waited for the last phase of what it alone would have left open).
        __syncthreads();
        if (*abort) break;
    }
    const bool run_ends_here =
        !balanced || mla_run_begin(balance, blockIdx.y + 1ull) <= balance.unit * (b + 1ull) + kMlaItemCostTiles;
    const unsigned int tiles = (t1 - t0 + kMlaN - 1) / kMlaN;
    const unsigned int own_tiles = (tiles + 1u - half) / 2u;     // tiles j with j % 2 == half
    const unsigned int peer_tiles = tiles - own_tiles;
    const int own0 = 4 * (int)half, other0 = 4 * (1 - (int)half);

    if (threadIdx.x == 0) {
        if (!first_item) {
            uint64_t *all = &bars->q_full;
            for (unsigned int i = 0; i < kPairBarrierCount; ++i) mbar_inval(all + i);
        }
        mbar_init(&bars->q_full, 1);
        mbar_init(&bars->q_tmem_full, kMlaHeads);
        mbar_init(&bars->ka_full, 1);
        mbar_init(&bars->ka_done, 1);
        mbar_init(&bars->kb_full, 1);
        mbar_init(&bars->kb_done, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->v_full[i], 1);
            mbar_init(&bars->v_done[i], 1);
        }
        mbar_init(&bars->s_full, 1);
        mbar_init(&bars->s_free, kMlaHeads);
        mbar_init(&bars->p_own_full, 4);
        mbar_init(&bars->pv_own_done, 1);
        mbar_init(&bars->p_peer_full, 1);
        mbar_init(&bars->peer_ready, 4);
        mbar_init(&bars->p_peer_free, 1);
        mbar_init(&bars->p_written, 4);
        mbar_init(&bars->p_own_sent, 1);
        mbar_init(&bars->pv_done, 1);
        mbar_init(&bars->ka2_full, 1);
        mbar_init(&bars->ka2_done, 1);
        mbar_init(&bars->rows_staged, kMlaHeads);
        fence_barrier_init();
        // the first message of the peer: its weights and its maxima, counted in bytes
        if (peer_tiles) mbar_expect_tx(&bars->p_peer_full, kPairPBytes + kMlaHeads * 4);
    }
    first_item = false;
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();          // the peer's barriers exist before anything arrives on them
    tc_fence_after_sync();
    const uint32_t tmem = bars->tmem_base;
    MLA_MARK(0);
    const uint32_t tmem_o = tmem, tmem_s = tmem + kMlaHalf, tmem_q = tmem + kMlaHalf + kMlaN;
    const uint32_t peer_abort = cluster_map(smem_u32(&bars->abort), peer);
    auto give_up = [&]() {   // records the failure here and at the peer, whose waits then end too
        atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
        bars->abort = 1;
        cluster_store_b32(peer_abort, 1u);
    };

    if (warp == 4 || warp == 6 || warp == 7) {
        // ------------------------------ TMA producers: one warp per kind of part (a lane that spins on
        // a barrier beside other spinning lanes of its warp reacts late) ------------------------------
        if (warp == 4 && lane == 0) {
            mbar_expect_tx(&bars->q_full, kPairQSmemSubs * kMlaQSubBytes);
            tma_load_3d(smem + kPairOffQ, &maps.query, &bars->q_full, 64 * (other0 + 2), 0, (int)b);
            tma_load_3d(smem + kPairOffQ + kMlaQSubBytes, &maps.query, &bars->q_full, 64 * (other0 + 3), 0, (int)b);
            tma_load_3d(smem + kPairOffQ + 2 * kMlaQSubBytes, &maps.query, &bars->q_full, kMlaLatent, 0, (int)b);
            for (unsigned int i = 0; i < own_tiles; ++i) {
                const int token = (int)(t0 + (2u * i + half) * kMlaN);
                // two pieces with their own barriers: the first is free again (and its reload under way) while
                // the score product still reads the second
                if (i > 0 && !local_wait(&bars->ka_done, (i - 1u) & 1u, abort)) {
                    give_up();
                    break;
                }
                unsigned char *dst = smem + kPairOffKa;
                mbar_expect_tx(&bars->ka_full, 2 * kMlaKvSubBytes);
                for (int u = 0; u < 2; ++u)
                    tma_load_3d(dst + u * kMlaKvSubBytes, &maps.latent, &bars->ka_full, 64 * (other0 + u), token, (int)b);
                if (i > 0 && !local_wait(&bars->ka2_done, (i - 1u) & 1u, abort)) {
                    give_up();
                    break;
                }
                mbar_expect_tx(&bars->ka2_full, 3 * kMlaKvSubBytes);
                for (int u = 2; u < 4; ++u)
                    tma_load_3d(dst + u * kMlaKvSubBytes, &maps.latent, &bars->ka2_full, 64 * (other0 + u), token, (int)b);
                tma_load_3d(dst + 4 * kMlaKvSubBytes, &maps.rope, &bars->ka2_full, 0, token, (int)b);
            }
        } else if (warp == 6 && lane == 0) {
            // the own-half part of an own tile as K: one buffer, free again when the score product has read it
            for (unsigned int i = 0; i < own_tiles; ++i) {
                const int token = (int)(t0 + (2u * i + half) * kMlaN);
                if (i > 0 && !local_wait(&bars->kb_done, (i - 1u) & 1u, abort)) {
                    give_up();
                    break;
                }
                unsigned char *dst = smem + kPairOffKb;
                mbar_expect_tx(&bars->kb_full, kMlaVPartBytes);
                for (int u = 0; u < 4; ++u)
                    tma_load_3d(dst + u * kMlaKvSubBytes, &maps.latent, &bars->kb_full, 64 * (own0 + u), token, (int)b);
            }
        } else if (warp == 7 && lane == 0) {
            // the own-half part of EVERY tile as V, two slots: asked for (out of L2, where the score product's
            // load of the tile, this CTA's or the peer's, has just brought it) a whole tile pair ahead of its
            // P V. Holding the K copy of an own tile until its P V instead kept that buffer for one and a half
            // periods, and the score product of the tile after next waited for it.
            for (unsigned int j = 0; j < tiles; ++j) {
                const unsigned int slot = j & 1u;
                const int token = (int)(t0 + j * kMlaN);
                if (j >= 2u && !local_wait(&bars->v_done[slot], ((j >> 1) - 1u) & 1u, abort)) {
                    give_up();
                    break;
                }
                unsigned char *dst = smem + kPairOffV + slot * kMlaVPartBytes;
                mbar_expect_tx(&bars->v_full[slot], kMlaVPartBytes);
                for (int u = 0; u < 4; ++u)
                    tma_load_3d(dst + u * kMlaKvSubBytes, &maps.latent, &bars->v_full[slot], 64 * (own0 + u), token, (int)b);
            }
        }
    } else if (warp == 8) {
        // ------------------------------ sender ------------------------------
        // The weights of an own tile (and the maxima they were scaled with) go to the peer as two bulk
        // copies between the shared memories, counted in bytes on the peer's barrier, as soon as the
        // peer has consumed the tile sent before. The softmax does not wait for that: its buffer is
        // the second of the two tiles in flight (it waits for THIS tile to have left before it writes
        // the next one).
        if (lane == 0) {
            const uint32_t peer_p = cluster_map(smem_u32(smem + kPairOffPPeer), peer);
            const uint32_t peer_m = cluster_map(smem_u32(m_box), peer);
            const uint32_t peer_full = cluster_map(smem_u32(&bars->p_peer_full), peer);
            for (unsigned int i = 0; i < own_tiles; ++i) {
                if (!local_wait(&bars->p_written, i & 1u, abort) ||
                    (i > 0 && !pair_wait(&bars->p_peer_free, (i - 1u) & 1u, abort))) {
                    give_up();
                    break;
                }
                fence_proxy_async();
                cluster_bulk_copy(peer_p, smem + kPairOffPOwn, kPairPBytes, peer_full);
                cluster_bulk_copy(peer_m, m_out, kMlaHeads * 4, peer_full);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                mbar_arrive(&bars->p_own_sent);
                // the last credit is nobody's to wait for otherwise: nothing may be pending when the item ends
                if (i + 1u == own_tiles && !pair_wait(&bars->p_peer_free, i & 1u, abort)) give_up();
            }
        }
    } else if (warp == 5 || warp == 9) {
        // ------------------------------ MMA issuers ------------------------------
        // Two warps, one for the score products and one for the P V products: each blocks on its own operands
        // and the tensor pipe takes whatever either has issued, so neither kind of product waits behind a wait
        // for the other's operands. (Products of one kind stay in one thread, hence in order; the two kinds
        // share no buffer: the score product reads the K copy of a tile's own-half part, P V its V copy.)
        constexpr uint32_t idesc_qk = idesc_bf16_f32(kMlaHeads, kMlaN, false);
        constexpr uint32_t idesc_pv = idesc_bf16_f32(kMlaHeads, kMlaHalf, true);
        constexpr uint32_t desc_hi = smem_desc_sw128_hi(1024);
        const uint32_t elected = tc_elect_one() ? 1u : 0u;
        auto wait_all = [&](uint64_t *bar, uint32_t parity) -> bool {    // every lane waits: the warp stays converged
            return __all_sync(0xffffffffu, local_wait(bar, parity, abort)) != 0;
        };
        bool ok = true;
        if (warp == 9) {
            const uint32_t peer_credit = cluster_map(smem_u32(&bars->p_peer_free), peer);
            // P V of tile j, once its weights (and V) are there, in tile order
            for (unsigned int j = 0; ok && j < tiles; ++j) {
                const unsigned int i = j >> 1;
                const bool own = (j & 1u) == half;
                MLA_TRACE_BEGIN(tw);
                ok = wait_all(own ? &bars->p_own_full : &bars->peer_ready, i & 1u) && wait_all(&bars->v_full[j & 1u], i & 1u);
                if (!ok) break;
                MLA_TRACE_ADD(4, tw);
                MLA_TRACE_BEGIN(tpv);
                tc_fence_after_sync();
                const uint32_t p_lo = smem_desc_sw128_lo(smem_u32(smem + (own ? kPairOffPOwn : kPairOffPPeer)), 16);
                const uint32_t v_lo = smem_desc_sw128_lo(smem_u32(smem + kPairOffV + (j & 1u) * kMlaVPartBytes), kMlaKvSubBytes);
#pragma unroll
                for (int kk = 0; kk < kMlaN / 16; ++kk)
                    tc_mma_ss_pred(elected, tmem_o, p_lo + 2u * kk, desc_hi, v_lo + ((kk * 2048) >> 4), desc_hi, idesc_pv,
                                   (j || kk) ? 1u : 0u);
                tc_commit_pred(elected, &bars->v_done[j & 1u]);
                if (own) {
                    tc_commit_pred(elected, &bars->pv_own_done);
                } else {
                    // ... and tells the peer at once that the weights it sent are consumed
                    asm volatile(
                        "{\n\t.reg .pred pe;\n\t"
                        "setp.ne.b32 pe, %0, 0;\n\t"
                        "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%1];\n\t}"
                        ::"r"(elected), "r"(peer_credit)
                        : "memory");
                }
                tc_commit_pred(elected, &bars->pv_done);
                MLA_TRACE_ADD(1, tpv);
            }
            // nothing may be pending on a barrier when the item ends: the last phases nobody else waits for
            for (unsigned int slot = 0; ok && slot < 2u; ++slot) {
                const unsigned int uses = (tiles + 1u - slot) / 2u;
                if (uses) ok = wait_all(&bars->v_done[slot], (uses - 1u) & 1u);
            }
            if (ok && own_tiles) ok = wait_all(&bars->pv_own_done, (own_tiles - 1u) & 1u);
        } else {
            const uint32_t q_lo = smem_desc_sw128_lo(smem_u32(smem + kPairOffQ), 16);
            const uint32_t ka_lo = smem_desc_sw128_lo(smem_u32(smem + kPairOffKa), 16);
            ok = wait_all(&bars->q_full, 0) && wait_all(&bars->q_tmem_full, 0);
            // the score product of own tile i: 8 + 12 k-steps over the scores-only part, 16 over the own half
            for (unsigned int i = 0; ok && i < own_tiles; ++i) {
                MLA_TRACE_BEGIN(tw);
                if (!(ok = wait_all(&bars->ka_full, i & 1u))) break;
                MLA_TRACE_ADD(5, tw);
                MLA_TRACE_BEGIN(tw3);
                // the score buffer is free once the softmax has read the previous own tile out of it
                if (i > 0u && !(ok = wait_all(&bars->s_free, (i - 1u) & 1u))) break;
                MLA_TRACE_ADD(7, tw3);
                MLA_TRACE_BEGIN(tqa);
                tc_fence_after_sync();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)      // query dims in tensor memory (first two sub-tiles of the other half)
                    tc_mma_ts_pred(elected, tmem_s, tmem_q + 128 + ks * 8,
                                   ka_lo + (((ks >> 2) * kMlaKvSubBytes + (ks & 3) * 32) >> 4), desc_hi, idesc_qk, ks ? 1u : 0u);
                tc_commit_pred(elected, &bars->ka_done);
                if (!(ok = wait_all(&bars->ka2_full, i & 1u))) break;
                tc_fence_after_sync();
#pragma unroll
                for (int ks = 0; ks < 12; ++ks)     // query dims in shared memory (its last two sub-tiles, then the rope dims)
                    tc_mma_ss_pred(elected, tmem_s, q_lo + (((ks >> 2) * kMlaQSubBytes + (ks & 3) * 32) >> 4), desc_hi,
                                   ka_lo + ((((ks >> 2) + 2) * kMlaKvSubBytes + (ks & 3) * 32) >> 4), desc_hi, idesc_qk, 1u);
                tc_commit_pred(elected, &bars->ka2_done);
                MLA_TRACE_ADD(2, tqa);
                MLA_TRACE_BEGIN(tw2);
                if (!(ok = wait_all(&bars->kb_full, i & 1u))) break;
                MLA_TRACE_ADD(6, tw2);
                MLA_TRACE_BEGIN(tqb);
                tc_fence_after_sync();
                const uint32_t kb_lo = smem_desc_sw128_lo(smem_u32(smem + kPairOffKb), 16);
#pragma unroll
                for (int ks = 0; ks < 16; ++ks)
                    tc_mma_ts_pred(elected, tmem_s, tmem_q + ks * 8,
                                   kb_lo + (((ks >> 2) * kMlaKvSubBytes + (ks & 3) * 32) >> 4), desc_hi, idesc_qk, 1u);
                tc_commit_pred(elected, &bars->kb_done);
                tc_commit_pred(elected, &bars->s_full);
                MLA_TRACE_ADD(3, tqb);
            }
            if (ok && own_tiles)   // the last phases of the "free again" barriers (see the P V warp)
                ok = wait_all(&bars->ka_done, (own_tiles - 1u) & 1u) && wait_all(&bars->ka2_done, (own_tiles - 1u) & 1u) &&
                     wait_all(&bars->kb_done, (own_tiles - 1u) & 1u);
        }
        if (!ok && lane == 0) give_up();
#ifdef YVX_MLA_TRACE
        if (traced && warp == 5) {
            yvx_mla_trace[9] = (unsigned long long)(clock64() - trace_start);
            yvx_mla_trace[11] = trace_local[2];
            yvx_mla_trace[12] = trace_local[3];
            yvx_mla_trace[14] = trace_local[5];
            yvx_mla_trace[15] = trace_local[7];
            yvx_mla_trace[8] = trace_local[6];
        }
        if (traced && warp == 9) {
            yvx_mla_trace[10] = trace_local[1];
            yvx_mla_trace[13] = trace_local[4];
        }
#endif
    } else {
        // ------------------------------ softmax warps: a thread owns a head (a row of every tile) ------------------------------
        // (Two warps per 32 heads, each with half of a tile's tokens, were slower here: the two had to agree on
        // the row maximum through shared memory, and those meetings cost more than the exponentials they halved.)
        const unsigned int quadrant = warp;
        const unsigned int head = quadrant * 32u + lane;
        const uint32_t lane_base = ((quadrant * 32u) << 16);
        {
            // 384 query dims of this head into tensor memory: the own latent half, then 128 dims of the other
            const unsigned short *row0 = reinterpret_cast<const unsigned short *>(p.q_absorbed) +
                                         ((unsigned long long)b * kMlaHeads + quadrant * 32u) * kMlaWidth;
            // A warp reads 128-byte pieces of four rows per instruction (a thread reading its own row would touch 32
            // lines per instruction) and turns them through its 4 KB of the (still unused) weights buffer; three
            // 64-dim groups are in flight together.
            unsigned char *turn = smem + kPairOffPOwn + quadrant * 4096u;
            const unsigned int piece_row = lane >> 3, piece = lane & 7u;
#pragma unroll 1
            for (int batch = 0; batch < kPairQTmemCols / 96; ++batch) {
                uint4 v[3][8];
#pragma unroll
                for (int g = 0; g < 3; ++g) {
                    const int i = 3 * batch + g;
                    const unsigned short *group =
                        row0 + (i < 4 ? (unsigned)half * kMlaHalf + 64u * i : (unsigned)(1u - half) * kMlaHalf + 64u * (i - 4));
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        v[g][c] = *reinterpret_cast<const uint4 *>(group + (4u * c + piece_row) * kMlaWidth + piece * 8u);
                }
#pragma unroll
                for (int g = 0; g < 3; ++g) {
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const unsigned int r = 4u * c + piece_row;
                        *reinterpret_cast<uint4 *>(turn + r * 128u + ((piece ^ (r & 7u)) * 16u)) = v[g][c];
                    }
                    __syncwarp();
                    uint32_t words[32];
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const uint4 w = *reinterpret_cast<const uint4 *>(turn + lane * 128u + (((unsigned)c ^ (lane & 7u)) * 16u));
                        words[4 * c] = w.x;
                        words[4 * c + 1] = w.y;
                        words[4 * c + 2] = w.z;
                        words[4 * c + 3] = w.w;
                    }
                    __syncwarp();
                    tmem_st32(tmem_q + lane_base + 32 * (3 * batch + g), words);
                }
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&bars->q_tmem_full);
            MLA_MARK(1);
        }
        const float sscale = p.scale * 1.4426950408889634f;
        // m_used: the maximum this CTA's weights are scaled with (and its l); m_o: the scale its accumulator carries
        float m_used = -INFINITY, l = 0.0f, m_o = -INFINITY, m_heard = -INFINITY;
        bool ok = true;
        auto rescale = [&](float factor) {
#pragma unroll 1
            for (int i = 0; i < kMlaHalf / 32; ++i) {
                uint32_t o[32];
                const uint32_t column = tmem_o + lane_base + 32u * i;
                tmem_ld32(column, o);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * factor);
                tmem_st32(column, o);
            }
            tmem_wait_st();
        };
        // Lets the tensor pipe run P(j) V(j): first brings the accumulator to the scale the weights of
        // tile j were computed with (up or down; rare), in tile order, after every earlier P V has landed.
        auto release = [&](unsigned int j, float m_p, uint64_t *go) -> bool {
            const bool differs = m_p != m_o && m_p != -INFINITY;
            if (__any_sync(0xffffffffu, differs)) {
                if (j > 0) {
                    if (!local_wait(&bars->pv_done, (j - 1u) & 1u, abort)) return false;
                    tc_fence_after_sync();
                    rescale(differs && m_o != -INFINITY ? exp2_approx(m_o - m_p) : 1.0f);
                    tc_fence_before_sync();
                }
                if (differs) m_o = m_p;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(go);
            return true;
        };
        // The peer's message for its tile j: its weights are in place, its maxima in m_box.
        auto receive = [&](unsigned int j) -> bool {
            const unsigned int ip = j >> 1;
            MLA_TRACE_BEGIN(w4);
            if (!pair_wait(&bars->p_peer_full, ip & 1u, abort)) return false;
            MLA_TRACE_ADD(4, w4);
            MLA_TRACE_BEGIN(w5);
            if (warp == 0 && lane == 0 && ip + 1u < peer_tiles)   // the next message may be counted from now on
                mbar_expect_tx(&bars->p_peer_full, kPairPBytes + kMlaHeads * 4);
            const float m_in = m_box[head];
            m_heard = m_in;     // adopted at a fixed point of the program (results must not depend on timing)
            const bool fine = release(j, m_in, &bars->peer_ready);
            MLA_TRACE_ADD(5, w5);
            return fine;
        };
        for (unsigned int i = 0; i < own_tiles && ok; ++i) {
            const unsigned int j = 2u * i + half;
            bool received_early = false;
            {
                // ---- the weights of a tile this CTA scores; nothing here waits for the peer's softmax ----
                MLA_TRACE_BEGIN(w0);
                if (!local_wait(&bars->s_full, i & 1u, abort)) {
                    ok = false;
                    break;
                }
                MLA_TRACE_ADD(0, w0);
                if (i == 0) MLA_MARK(2);
                if (i == 1) MLA_MARK(3);
                MLA_TRACE_BEGIN(w1);
                tc_fence_after_sync();
                uint32_t s[2][32];
                tmem_ld32(tmem_s + lane_base, s[0]);
                tmem_ld32(tmem_s + lane_base + 32u, s[1]);
                tmem_wait_ld();
                tc_fence_before_sync();
                mbar_arrive(&bars->s_free);
                const unsigned int k0 = t0 + j * kMlaN;
                if (k0 + kMlaN > t1) {
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int c = 0; c < 32; ++c)
                            if (k0 + 32 * h + c >= t1) s[h][c] = 0xff800000u;  // -inf
                }
                // Has the peer's message for the tile in front of this one arrived already? Then it is
                // processed now (its P V can run, and the peer gets its buffer back, while this tile's
                // exponentials are computed); otherwise after this tile's weights are out.
                received_early = j > 0 && __shfl_sync(0xffffffffu, (int)mbar_test(&bars->p_peer_full, ((j - 1u) >> 1) & 1u), 0) != 0;
                if (received_early && !receive(j - 1u)) {
                    ok = false;
                    break;
                }
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < 32; c += 2)
                        mx[(c >> 1) & 3] = max3(mx[(c >> 1) & 3], __uint_as_float(s[h][c]), __uint_as_float(s[h][c + 1]));
                const float m_tile = max3(mx[0], mx[1], fmaxf(mx[2], mx[3])) * sscale;
                if (m_tile > m_used + kMlaRescaleThreshold || m_used == -INFINITY) {
                    const float m_new = fmaxf(m_used, m_tile);
                    l *= m_new == -INFINITY || m_used == -INFINITY ? 1.0f : exp2_approx(m_used - m_new);
                    m_used = m_new;
                }
                const float offset = m_used == -INFINITY ? 0.0f : -m_used;
                uint32_t packed[32];
                float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        const float p0 = exp2_approx(fmaf(__uint_as_float(s[h][c]), sscale, offset));
                        const float p1 = exp2_approx(fmaf(__uint_as_float(s[h][c + 1]), sscale, offset));
                        sum0 += p0;
                        sum1 += p1;
                        packed[16 * h + (c >> 1)] = pack_bf16(p0, p1);
                    }
                l += sum0 + sum1;
                MLA_TRACE_ADD(1, w1);
                MLA_TRACE_BEGIN(w2);
                // the previous own tile's weights have been consumed here and have left for the peer
                if (i > 0 && !(local_wait(&bars->pv_own_done, (i - 1u) & 1u, abort) &&
                               local_wait(&bars->p_own_sent, (i - 1u) & 1u, abort))) {
                    ok = false;
                    break;
                }
                MLA_TRACE_ADD(2, w2);
                MLA_TRACE_BEGIN(w3);
                // row `head`: its eight 16-byte chunks under the 128-byte swizzle
                {
                    unsigned char *mine = smem + kPairOffPOwn + head * 128u;
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        *reinterpret_cast<uint4 *>(mine + ((unsigned)c ^ (head & 7u)) * 16u) =
                            make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
                    m_out[head] = m_used;
                }
                fence_proxy_async();   // the tensor pipe and the bulk copy read these bytes through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->p_written);
                MLA_TRACE_ADD(3, w3);
            }
            // ---- P V in tile order: the peer's tile in front of this one, then this one ----
            const float m_own = m_used;
            if (j > 0 && !received_early) ok = receive(j - 1u);
            if (ok) ok = release(j, m_own, &bars->p_own_full);
            // Here, whether the peer's message was processed before or after this tile's exponentials:
            // adopt a larger maximum, so that the two CTAs' references stay together.
            if (m_heard > m_used) {
                l *= m_used == -INFINITY ? 1.0f : exp2_approx(m_used - m_heard);
                m_used = m_heard;
            }
        }
        // the last tile when it is the peer's
        if (ok && ((tiles - 1u) & 1u) != half) ok = receive(tiles - 1u);
#ifdef YVX_MLA_TRACE
        if (traced && warp == 0) {
            for (int i = 0; i < 6; ++i) yvx_mla_trace[i] = trace_local[i];
            yvx_mla_trace[6] = (unsigned long long)(clock64() - trace_start);
            yvx_mla_trace[7] = tiles;
        }
#endif
        MLA_MARK(4);
        if (ok) ok = local_wait(&bars->pv_done, (tiles - 1u) & 1u, abort);
        MLA_MARK(5);
        if (!__all_sync(0xffffffffu, ok) && lane == 0) give_up();
        // this CTA's share of the denominators, and the maximum it is relative to, go to the peer
        cluster_store_f32(cluster_map(smem_u32(l_box + head), peer), l);
        cluster_store_f32(cluster_map(smem_u32(m_box + kMlaHeads + head), peer), m_used);
        if (run_ends_here) pdl_launch_dependents();
        if (balanced && ends_session) {
            // the slots of this session that no item fills read as empty parts in the fold
            for (unsigned int unused = split + 1u; unused < p.max_splits; ++unused)
                *reinterpret_cast<float2 *>(
                    p.partials + ((((unsigned long long)b * kMlaHeads + head) * 2ull + half) * p.max_splits + unused) * part_stride +
                    kMlaHalf) = make_float2(-INFINITY, 0.0f);
        }
        // (the cluster barrier below is reached by every thread of both CTAs)
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        bool fine = ok && !*abort;
        MLA_MARK(6);
        float *staged = reinterpret_cast<float *>(smem);
        if (fine) {
            tc_fence_after_sync();
            // the row's denominator: both CTAs' shares at the accumulator's scale
            const float m_theirs = m_box[kMlaHeads + head];
            const float mine_scaled = m_used == -INFINITY ? 0.0f : l * exp2_approx(m_used - m_o);
            const float theirs_scaled = m_theirs == -INFINITY ? 0.0f : l_box[head] * exp2_approx(m_theirs - m_o);
            l = mine_scaled + theirs_scaled;
            const float inverse = l > 0.0f ? 1.0f / l : 0.0f;
            // every tile has been consumed: the tile buffers are free for the turn of the rows
            float *mine = staged + head * (unsigned)part_stride;
#pragma unroll 1
            for (int i = 0; i < kMlaHalf / 32; ++i) {
                uint32_t o[32];
                tmem_ld32(tmem_o + lane_base + 32 * i, o);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; c += 2)
                    *reinterpret_cast<float2 *>(mine + 32 * i + c) =
                        make_float2(__uint_as_float(o[c]) * inverse, __uint_as_float(o[c + 1]) * inverse);
            }
            *reinterpret_cast<float2 *>(mine + kMlaHalf) =
                make_float2(m_o == -INFINITY ? -INFINITY : m_o * 0.6931471805599453f, l);
            mbar_arrive(&bars->rows_staged);
            MLA_MARK(8);
            fine = local_wait(&bars->rows_staged, 0, abort);
            MLA_MARK(9);
        }
        if (fine) {
            // four rows at a time, all of their loads from shared memory ahead of the stores (a row is 129
            // 8-byte words: four full sweeps of the warp and one word)
            constexpr unsigned int kRowWords = (unsigned)(kMlaHalf + 2) / 2u;
#pragma unroll 1
            for (unsigned int r0 = warp * 32u; r0 < warp * 32u + 32u; r0 += 4u) {
                float2 v[4][5];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 *src = reinterpret_cast<const float2 *>(staged + (r0 + q) * (unsigned)part_stride);
#pragma unroll
                    for (int u = 0; u < 5; ++u)
                        if (lane + 32u * u < kRowWords) v[q][u] = src[lane + 32u * u];
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float2 *dst = reinterpret_cast<float2 *>(
                        p.partials +
                        ((((unsigned long long)b * kMlaHeads + r0 + q) * 2ull + half) * p.max_splits + split) * part_stride);
#pragma unroll
                    for (int u = 0; u < 5; ++u)
                        if (lane + 32u * u < kRowWords) dst[lane + 32u * u] = v[q][u];
                }
            }
        }
        MLA_MARK(7);
    }
    if (warp >= 4u) {
        // the producer, sender and issuer warps meet the softmax warps at the cluster barrier
        __syncwarp();
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    }   // work items
    tc_fence_before_sync();
    __syncthreads();
#ifdef YVX_MLA_TRACE
    if (threadIdx.x == 0 && span_index < 512u) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        yvx_mla_spans[2u * span_index + 1u] = now;
    }
#endif
    if (warp == 5) tmem_dealloc(bars->tmem_base, kMlaTmemColumns);
}

// ---- the form with clusters of FOUR CTAs -------------------------------------------------------------------
// CTA r of a cluster owns a quarter of the latent columns of O (128 tensor-memory columns), so all 576 query dims
// fit tensor memory (288 columns) beside the score buffer: every score instruction reads its A operand there, and
// shared memory holds tile buffers only. Tile j is scored by CTA j % 4, which sends the weights (with the row
// maxima they were scaled with) to the other three; every CTA runs P V of every tile on its own quarter, with V
// (a tile's own quarter, 16 KB) from a ring of four slots. With one cluster per session nothing is split: no
// partial rows and no combine launch.
// The weights travel through L2: the scorer's softmax threads write them (plain rows, coalesced) into one of two
// slots of a scratch area in global memory and tell the peers; each peer's loader pulls them with one tiled TMA
// load, which lays them out swizzled as the tensor pipe reads them. (Three bulk copies between shared memories
// took 2650-3170 cycles per tile out of one SM, in series.) A CTA processes the tiles of a period (its own
// included) one period late, at a fixed point of its program, so the transfer is hidden and results do not
// depend on timing; its own weights are double-buffered for that. Every barrier that can run two phases ahead
// of its waiter exists once per buffer.
// Behind the partial rows of the four-CTA form: two scratch slots per (session, split, rank) for the weights of an own
// tile ([128 heads][64 tokens] bf16) on their way to the peers, then as many slots of 128 maxima.
__host__ __device__ inline unsigned long long mla_quad_rows_bytes(const yvx_mla_problem &p)
{
    const unsigned long long rows = (unsigned long long)p.sessions * kMlaHeads * 4ull * p.max_splits * (kMlaLatent / 4 + 2) * 4ull;
    return (rows + 1023ull) & ~1023ull;
}
__host__ __device__ inline unsigned char *mla_quad_scratch(const yvx_mla_problem &p)
{
    return reinterpret_cast<unsigned char *>(p.partials) + mla_quad_rows_bytes(p);
}

constexpr int kQuadThreads = 320;    // warps 0-3 softmax, 4: K pieces, 5: score issuer, 6: V ring, 7: idle, 8: sender, 9: P V issuer
constexpr int kQuadCols = kMlaLatent / 4;                               // 128 accumulator columns per CTA
constexpr int kQuadQCols = kMlaWidth / 2;                               // 288 columns of query dims
constexpr int kQuadPieceBytes = 3 * kMlaKvSubBytes;                     // a third of a tile: 24 KB, 12 score instructions
constexpr int kQuadOffK = 0;                                            // a whole tile as K: 9 sub-tiles, 72 KB
constexpr int kQuadVSlotBytes = 2 * kMlaKvSubBytes;                     // a tile's own quarter as V: 16 KB
constexpr int kQuadOffV = kMlaKvBytes;                                  // 73728, four slots
constexpr int kQuadOffPOwn = kQuadOffV + 4 * kQuadVSlotBytes;           // 139264
constexpr int kQuadOffPPeer = kQuadOffPOwn + 2 * kPairPBytes;           // 172032: one buffer per source (own weights: two)
constexpr int kQuadOffTail = kQuadOffPPeer + 3 * kPairPBytes;           // 221184
constexpr int kQuadBoxBytes = 3 * kMlaHeads * 4;                        // three sources x 128 floats
constexpr int kQuadSmemBytes = kQuadOffTail + 512 + 3 * kQuadBoxBytes + 2 * kMlaHeads * 4 + 1024;
constexpr unsigned long long kQuadMessageBytes = kPairPBytes + kMlaHeads * 4;   // weights + the maxima they were scaled with

#ifdef YVX_QUAD_TRACE
__device__ unsigned long long yvx_quad_trace[16];
#define QT_BEGIN(t) const long long t = clock64()
#define QT_ADD(slot, t) do { if (qtraced) qt[slot] += (unsigned long long)(clock64() - t); } while (0)
#else
#define QT_BEGIN(t) do { } while (0)
#define QT_ADD(slot, t) do { } while (0)
#endif

struct QuadBarriers {
    uint64_t q_tmem_full;
    uint64_t k_full[3], k_done[3];        // the three pieces of an own tile: loaded / read by their score instructions
    uint64_t v_full[4], v_done[4];        // the own quarter of any tile as V, four slots (tile % 4)
    uint64_t s_full, s_free;
    uint64_t p_own_full[2], pv_own_done[2];   // per buffer of own weights: released to the tensor pipe / consumed
    uint64_t p_peer_full[3], peer_ready[3];   // per source: its weights have landed here / its message is processed
    uint64_t p_avail[3][2];               // per source and scratch slot: its weights are in global memory
    uint64_t peer_consumed[3];            // per source: the P V that read its weights has run
    uint64_t g_free[2];                   // per scratch slot: all three peers have pulled this CTA's weights out of it
    uint64_t p_written[2], p_own_sent[2]; // per buffer of own weights: written by the softmax / stored to the scratch slot
    uint64_t pv_done;
    uint64_t rows_staged;
    uint32_t tmem_base;
    int abort;
};
constexpr unsigned int kQuadBarrierCount = 44u;
static_assert(offsetof(QuadBarriers, tmem_base) == kQuadBarrierCount * 8u, "barrier count out of step");
static_assert(sizeof(QuadBarriers) <= 512, "barrier block outgrew its shared-memory slot");

__global__ void __cluster_dims__(4, 1, 1) __launch_bounds__(kQuadThreads, 1)
mla_decode_quad_kernel(const yvx_mla_problem p, const __grid_constant__ MlaMaps maps)
{
    extern __shared__ unsigned char quad_smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(quad_smem_raw) + 1023u) & ~uintptr_t(1023));
    QuadBarriers *bars = reinterpret_cast<QuadBarriers *>(smem + kQuadOffTail);
    float *m_box = reinterpret_cast<float *>(smem + kQuadOffTail + 512);   // [3 sources][128]: a source's maxima with its tile
    float *l_box = m_box + 3 * kMlaHeads;                                  // [3][128]: the peers' denominators at the end
    float *mfin_box = l_box + 3 * kMlaHeads;                               // [3][128]: ... and the maxima they are relative to
    float *m_out = mfin_box + 3 * kMlaHeads;                               // [2 buffers][128]: the maxima of an own tile, source of its store

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned int rank = blockIdx.x, split = blockIdx.y, b = blockIdx.z;   // rank in the cluster
    const unsigned int kv_tokens = admitted_kv_tokens(p.kv_tokens, b, p.kv_tokens_uniform, p.kv_tokens_max, p.status);
    const unsigned int t0 = split * p.chunk_tokens;
    const unsigned int t1 = min(kv_tokens, t0 + p.chunk_tokens);
    const bool direct = p.max_splits == 1u;    // one item per session: the result itself leaves, no partial rows
    const unsigned long long part_stride = kQuadCols + 2;
    // the scratch slots of this cluster's messages: slot index ((item * 4 + rank) * 2 + buffer), weights then maxima
    const unsigned long long item_slot = ((unsigned long long)b * p.max_splits + split) * 8ull;
    unsigned char *weights_scratch = mla_quad_scratch(p);
    float *maxima_scratch = reinterpret_cast<float *>(weights_scratch +
                                                      (unsigned long long)p.sessions * p.max_splits * 8ull * kPairPBytes);
    if (t0 >= t1) {
        // Nothing of this session falls into the split (true for all four CTAs): an empty partial; a session without
        // any token has no result (0 / 0, reported), as the fold of nothing gives.
        if (threadIdx.x < (unsigned)kMlaHeads) {
            if (direct) {
                float *row = p.output + ((unsigned long long)b * kMlaHeads + threadIdx.x) * kMlaLatent + rank * kQuadCols;
                for (int d = 0; d < kQuadCols; ++d) row[d] = __int_as_float(0x7fc00000);
                atomicCAS(p.status, 0, YVX_STATUS_NONFINITE);
            } else {
                float *part = p.partials +
                              ((((unsigned long long)b * kMlaHeads + threadIdx.x) * 4ull + rank) * p.max_splits + split) * part_stride;
                for (int d = 0; d < kQuadCols; ++d) part[d] = 0.0f;
                part[kQuadCols] = -INFINITY;
                part[kQuadCols + 1] = 0.0f;
            }
        }
        return;
    }
    const unsigned int tiles = (t1 - t0 + kMlaN - 1) / kMlaN;
    const unsigned int own_tiles = (tiles + 3u - rank) / 4u;     // tiles j with j % 4 == rank
    volatile int *abort = &bars->abort;

    if (threadIdx.x == 0) {
        mbar_init(&bars->q_tmem_full, kMlaHeads);
        for (int i = 0; i < 3; ++i) {
            mbar_init(&bars->k_full[i], 1);
            mbar_init(&bars->k_done[i], 1);
            mbar_init(&bars->p_peer_full[i], 1);
            mbar_init(&bars->peer_ready[i], 4);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&bars->v_full[i], 1);
            mbar_init(&bars->v_done[i], 1);
        }
        mbar_init(&bars->s_full, 1);
        mbar_init(&bars->s_free, kMlaHeads);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->p_own_full[i], 4);
            mbar_init(&bars->pv_own_done[i], 1);
            mbar_init(&bars->g_free[i], 3);
            mbar_init(&bars->p_written[i], 4);
            mbar_init(&bars->p_own_sent[i], 1);
            for (int q = 0; q < 3; ++q) mbar_init(&bars->p_avail[q][i], 1);
        }
        for (int q = 0; q < 3; ++q) mbar_init(&bars->peer_consumed[q], 1);
        mbar_init(&bars->pv_done, 1);
        mbar_init(&bars->rows_staged, kMlaHeads);
        bars->abort = 0;
        fence_barrier_init();
    }
    if (warp == 5) {
        tmem_alloc(&bars->tmem_base, kMlaTmemColumns);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();          // the peers' barriers exist before anything arrives on them
    tc_fence_after_sync();
    const uint32_t tmem = bars->tmem_base;
    const uint32_t tmem_o = tmem, tmem_s = tmem + kQuadCols, tmem_q = tmem + kQuadCols + kMlaN;
    auto give_up = [&]() {   // records the failure here and at the peers, whose waits then end too
        atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
        bars->abort = 1;
        for (unsigned int d = 1; d < 4u; ++d) cluster_store_b32(cluster_map(smem_u32(&bars->abort), (rank + d) & 3u), 1u);
    };

    if (warp == 4 || warp == 6 || warp == 7) {
        if (warp == 4 && lane == 0) {
            // an own tile as K, in three pieces with their own barriers (a piece is asked for again as soon as its
            // twelve score instructions have read it)
            for (unsigned int i = 0; i < own_tiles; ++i) {
                const int token = (int)(t0 + (4u * i + rank) * kMlaN);
                bool fine = true;
                for (int piece = 0; piece < 3 && fine; ++piece) {
                    if (i > 0 && !local_wait(&bars->k_done[piece], (i - 1u) & 1u, abort)) {
                        give_up();
                        fine = false;
                        break;
                    }
                    mbar_expect_tx(&bars->k_full[piece], kQuadPieceBytes);
                    for (int u = 3 * piece; u < 3 * piece + 3; ++u) {
                        unsigned char *dst = smem + kQuadOffK + u * kMlaKvSubBytes;
                        if (u < 8)
                            tma_load_3d(dst, &maps.latent, &bars->k_full[piece], 64 * u, token, (int)b);
                        else
                            tma_load_3d(dst, &maps.rope, &bars->k_full[piece], 0, token, (int)b);
                    }
                }
                if (!fine) break;
            }
        } else if (warp == 6 && lane == 0) {
            // the own quarter of EVERY tile as V (out of L2 for the most part: a score product's load of the tile has
            // brought it there), four slots
            for (unsigned int j = 0; j < tiles; ++j) {
                const unsigned int slot = j & 3u;
                const int token = (int)(t0 + j * kMlaN);
                if (j >= 4u && !local_wait(&bars->v_done[slot], ((j >> 2) - 1u) & 1u, abort)) {
                    give_up();
                    break;
                }
                unsigned char *dst = smem + kQuadOffV + slot * kQuadVSlotBytes;
                mbar_expect_tx(&bars->v_full[slot], kQuadVSlotBytes);
                for (int u = 0; u < 2; ++u)
                    tma_load_3d(dst + u * kMlaKvSubBytes, &maps.latent, &bars->v_full[slot], 64 * (2 * (int)rank + u), token, (int)b);
            }
        } else if (warp == 7 && lane == 0) {
            // the peers' messages, pulled out of their scratch slots in tile order: once the source has said that the
            // weights are in global memory and the P V that read its previous weights here has run
            for (unsigned int j = 0; j < tiles; ++j) {
                const unsigned int source = j & 3u, ii = j >> 2;
                if (source == rank) continue;
                const unsigned int q = (source - rank - 1u) & 3u;
                if (!pair_wait(&bars->p_avail[q][ii & 1u], (ii >> 1) & 1u, abort) ||
                    (ii > 0 && !local_wait(&bars->peer_consumed[q], (ii - 1u) & 1u, abort))) {
                    give_up();
                    break;
                }
                const unsigned long long slot = item_slot + source * 2ull + (ii & 1u);
                mbar_expect_tx(&bars->p_peer_full[q], (uint32_t)kQuadMessageBytes);
                tma_load_3d(smem + kQuadOffPPeer + q * kPairPBytes, &maps.weights, &bars->p_peer_full[q], 0, 0, (int)slot);
                bulk_load(m_box + q * kMlaHeads, maxima_scratch + slot * kMlaHeads, kMlaHeads * 4, &bars->p_peer_full[q]);
            }
        }
    } else if (warp == 8) {
        // ------------------------------ sender ------------------------------
        // An own tile's weights (and the maxima they were scaled with) leave for this CTA's scratch slot as bulk
        // stores (the tiled one undoes the swizzle), and when those are complete the peers are told.
        if (lane == 0) {
            for (unsigned int i = 0; i < own_tiles; ++i) {
                const unsigned int buffer = i & 1u;
                if (!local_wait(&bars->p_written[buffer], (i >> 1) & 1u, abort) ||
                    (i >= 2u && !pair_wait(&bars->g_free[buffer], ((i >> 1) - 1u) & 1u, abort))) {
                    give_up();
                    break;
                }
                const unsigned long long slot = item_slot + rank * 2ull + buffer;
                asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                             ::"l"(&maps.weights), "r"(0), "r"(0), "r"((int)slot),
                               "r"(smem_u32(smem + kQuadOffPOwn + buffer * kPairPBytes))
                             : "memory");
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                             ::"l"(maxima_scratch + slot * kMlaHeads), "r"(smem_u32(m_out + buffer * kMlaHeads)), "r"(kMlaHeads * 4)
                             : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                mbar_arrive(&bars->p_own_sent[buffer]);
                // one fence (the peers are in this cluster) orders the completed stores before the three arrivals: a
                // releasing arrival each costs more, and so does a device-wide fence
                asm volatile("fence.acq_rel.cluster;" ::: "memory");
                for (unsigned int d = 1; d < 4u; ++d)
                    cluster_arrive_remote_relaxed(cluster_map(smem_u32(&bars->p_avail[(3u - d) & 3u][buffer]), (rank + d) & 3u));
            }
        }
    } else if (warp == 5 || warp == 9) {
        // ------------------------------ MMA issuers: one for the score products, one for the P V products ------
        constexpr uint32_t idesc_qk = idesc_bf16_f32(kMlaHeads, kMlaN, false);
        constexpr uint32_t idesc_pv = idesc_bf16_f32(kMlaHeads, kQuadCols, true);
        constexpr uint32_t desc_hi = smem_desc_sw128_hi(1024);
        const uint32_t elected = tc_elect_one() ? 1u : 0u;
        auto wait_all = [&](uint64_t *bar, uint32_t parity) -> bool {    // every lane waits: the warp stays converged
            return __all_sync(0xffffffffu, local_wait(bar, parity, abort)) != 0;
        };
        bool ok = true;
        if (warp == 9) {
            for (unsigned int j = 0; ok && j < tiles; ++j) {
                const unsigned int i = j >> 2, source = j & 3u, slot = j & 3u;
                const bool own = source == rank;
                const unsigned int q = (source - rank - 1u) & 3u;
                ok = (own ? wait_all(&bars->p_own_full[i & 1u], (i >> 1) & 1u) : wait_all(&bars->peer_ready[q], i & 1u)) &&
                     wait_all(&bars->v_full[slot], i & 1u);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t p_lo = smem_desc_sw128_lo(
                    smem_u32(smem + (own ? kQuadOffPOwn + (int)(i & 1u) * kPairPBytes : kQuadOffPPeer + (int)q * kPairPBytes)), 16);
                const uint32_t v_lo = smem_desc_sw128_lo(smem_u32(smem + kQuadOffV + slot * kQuadVSlotBytes), kMlaKvSubBytes);
#pragma unroll
                for (int kk = 0; kk < kMlaN / 16; ++kk)
                    tc_mma_ss_pred(elected, tmem_o, p_lo + 2u * kk, desc_hi, v_lo + ((kk * 2048) >> 4), desc_hi, idesc_pv,
                                   (j || kk) ? 1u : 0u);
                tc_commit_pred(elected, &bars->v_done[slot]);
                tc_commit_pred(elected, own ? &bars->pv_own_done[i & 1u] : &bars->peer_consumed[q]);
                tc_commit_pred(elected, &bars->pv_done);
            }
            // nothing may be pending on a barrier when the kernel ends: the last phases nobody else waits for
            for (unsigned int slot = 0; ok && slot < 4u; ++slot) {
                const unsigned int uses = (tiles + 3u - slot) / 4u;
                if (uses) ok = wait_all(&bars->v_done[slot], (uses - 1u) & 1u);
            }
            (void)own_tiles;
        } else {
            const uint32_t k_lo = smem_desc_sw128_lo(smem_u32(smem + kQuadOffK), 16);
            ok = wait_all(&bars->q_tmem_full, 0);
            for (unsigned int i = 0; ok && i < own_tiles; ++i) {
#pragma unroll
                for (int piece = 0; piece < 3; ++piece) {
                    if (!(ok = wait_all(&bars->k_full[piece], i & 1u))) break;
                    // the score buffer is free once the softmax has read the previous own tile out of it
                    if (piece == 0 && i > 0u && !(ok = wait_all(&bars->s_free, (i - 1u) & 1u))) break;
                    tc_fence_after_sync();
#pragma unroll
                    for (int ks = 12 * piece; ks < 12 * piece + 12; ++ks)
                        tc_mma_ts_pred(elected, tmem_s, tmem_q + ks * 8,
                                       k_lo + (((ks >> 2) * kMlaKvSubBytes + (ks & 3) * 32) >> 4), desc_hi, idesc_qk, ks ? 1u : 0u);
                    tc_commit_pred(elected, &bars->k_done[piece]);
                }
                if (!ok) break;
                tc_commit_pred(elected, &bars->s_full);
            }
            for (int piece = 0; ok && own_tiles && piece < 3; ++piece) ok = wait_all(&bars->k_done[piece], (own_tiles - 1u) & 1u);
        }
        if (!ok && lane == 0) give_up();
    } else {
        // ------------------------------ softmax warps: a thread owns a head (a row of every tile) ------------------
        const unsigned int quadrant = warp;
        const unsigned int head = quadrant * 32u + lane;
        const uint32_t lane_base = ((quadrant * 32u) << 16);
        {
            // all 576 query dims of this head into tensor memory. A warp reads 128-byte pieces of four rows per
            // instruction and turns them through its 4 KB of the (still unused) weights buffer.
            const unsigned short *row0 = reinterpret_cast<const unsigned short *>(p.q_absorbed) +
                                         ((unsigned long long)b * kMlaHeads + quadrant * 32u) * kMlaWidth;
            unsigned char *turn = smem + kQuadOffPOwn + quadrant * 4096u;
            const unsigned int piece_row = lane >> 3, piece = lane & 7u;
#pragma unroll 1
            for (int batch = 0; batch < kQuadQCols / 96; ++batch) {
                uint4 v[3][8];
#pragma unroll
                for (int g = 0; g < 3; ++g) {
                    const unsigned short *group = row0 + 64u * (3 * batch + g);
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        v[g][c] = *reinterpret_cast<const uint4 *>(group + (4u * c + piece_row) * kMlaWidth + piece * 8u);
                }
#pragma unroll
                for (int g = 0; g < 3; ++g) {
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const unsigned int r = 4u * c + piece_row;
                        *reinterpret_cast<uint4 *>(turn + r * 128u + ((piece ^ (r & 7u)) * 16u)) = v[g][c];
                    }
                    __syncwarp();
                    uint32_t words[32];
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const uint4 w = *reinterpret_cast<const uint4 *>(turn + lane * 128u + (((unsigned)c ^ (lane & 7u)) * 16u));
                        words[4 * c] = w.x;
                        words[4 * c + 1] = w.y;
                        words[4 * c + 2] = w.z;
                        words[4 * c + 3] = w.w;
                    }
                    __syncwarp();
                    tmem_st32(tmem_q + lane_base + 32 * (3 * batch + g), words);
                }
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&bars->q_tmem_full);
        }
#ifdef YVX_QUAD_TRACE
        const bool qtraced = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0;
        unsigned long long qt[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const long long qt_start = clock64();
#endif
        const float sscale = p.scale * 1.4426950408889634f;
        // m_used: the maximum this CTA's weights are scaled with (and its l); m_o: the scale its accumulator carries
        float m_used = -INFINITY, l = 0.0f, m_o = -INFINITY, m_heard = -INFINITY;
        bool ok = true;
        auto rescale = [&](float factor) {
#pragma unroll 1
            for (int i = 0; i < kQuadCols / 32; ++i) {
                uint32_t o[32];
                const uint32_t column = tmem_o + lane_base + 32u * i;
                tmem_ld32(column, o);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * factor);
                tmem_st32(column, o);
            }
            tmem_wait_st();
        };
        // Lets the tensor pipe run P(j) V(j): first brings the accumulator to the scale the weights of tile j were
        // computed with (up or down; rare), in tile order, after every earlier P V has landed.
        auto release = [&](unsigned int j, float m_p, uint64_t *go) -> bool {
            const bool differs = m_p != m_o && m_p != -INFINITY;
            if (__any_sync(0xffffffffu, differs)) {
                if (j > 0) {
                    QT_BEGIN(qr);
                    if (!local_wait(&bars->pv_done, (j - 1u) & 1u, abort)) return false;
                    tc_fence_after_sync();
#ifdef YVX_QUAD_TRACE
                    if (qtraced) qt[6] += 1;
#endif
                    rescale(differs && m_o != -INFINITY ? exp2_approx(m_o - m_p) : 1.0f);
                    QT_ADD(7, qr);
                    tc_fence_before_sync();
                }
                if (differs) m_o = m_p;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(go);
            return true;
        };
        // A peer's message for its tile j: its weights are in place, its maxima in its box.
        auto receive = [&](unsigned int j) -> bool {
            const unsigned int source = j & 3u, q = (source - rank - 1u) & 3u, ip = j >> 2;
            QT_BEGIN(qw);
            if (!local_wait(&bars->p_peer_full[q], ip & 1u, abort)) return false;   // completed by this CTA's own loads
            QT_ADD(5, qw);
            if (warp == q && lane == 0)   // the message has been pulled: the source may write that scratch slot again
                cluster_arrive_remote_relaxed(cluster_map(smem_u32(&bars->g_free[ip & 1u]), source));
            const float m_in = m_box[q * kMlaHeads + head];
            m_heard = fmaxf(m_heard, m_in);   // adopted at a fixed point of the program (results must not depend on timing)
            return release(j, m_in, &bars->peer_ready[q]);
        };
        // Tiles are processed (a peer's message received, an own tile released to the tensor pipe) in tile order and
        // one period late: after the weights of own tile 4 i + rank are out, every tile below 4 i is processed,
        // blocking; those messages were written a whole period ago. Nothing here depends on when a message arrives.
        unsigned int next_tile = 0;
        float m_own_saved[2] = {-INFINITY, -INFINITY};   // the maxima the weights of the own tiles not yet released were scaled with
        auto process_until = [&](unsigned int limit) -> bool {
            for (; next_tile < limit; ++next_tile) {
                const bool fine = (next_tile & 3u) == rank
                                      ? release(next_tile, m_own_saved[(next_tile >> 2) & 1u], &bars->p_own_full[(next_tile >> 2) & 1u])
                                      : receive(next_tile);
                if (!fine) return false;
            }
            return true;
        };
        for (unsigned int i = 0; i < own_tiles && ok; ++i) {
            const unsigned int j = 4u * i + rank;
            QT_BEGIN(q0);
            if (!local_wait(&bars->s_full, i & 1u, abort)) {
                ok = false;
                break;
            }
            QT_ADD(0, q0);
            tc_fence_after_sync();
            uint32_t s[2][32];
            tmem_ld32(tmem_s + lane_base, s[0]);
            tmem_ld32(tmem_s + lane_base + 32u, s[1]);
            tmem_wait_ld();
            tc_fence_before_sync();
            mbar_arrive(&bars->s_free);
            const unsigned int k0 = t0 + j * kMlaN;
            if (k0 + kMlaN > t1) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        if (k0 + 32 * h + c >= t1) s[h][c] = 0xff800000u;  // -inf
            }
            QT_BEGIN(q2);
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int c = 0; c < 32; c += 2)
                    mx[(c >> 1) & 3] = max3(mx[(c >> 1) & 3], __uint_as_float(s[h][c]), __uint_as_float(s[h][c + 1]));
            const float m_tile = max3(mx[0], mx[1], fmaxf(mx[2], mx[3])) * sscale;
            if (m_tile > m_used + kMlaRescaleThreshold || m_used == -INFINITY) {
                const float m_new = fmaxf(m_used, m_tile);
                l *= m_new == -INFINITY || m_used == -INFINITY ? 1.0f : exp2_approx(m_used - m_new);
                m_used = m_new;
            }
            const float offset = m_used == -INFINITY ? 0.0f : -m_used;
            uint32_t packed[32];
            float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    const float p0 = exp2_approx(fmaf(__uint_as_float(s[h][c]), sscale, offset));
                    const float p1 = exp2_approx(fmaf(__uint_as_float(s[h][c + 1]), sscale, offset));
                    sum0 += p0;
                    sum1 += p1;
                    packed[16 * h + (c >> 1)] = pack_bf16(p0, p1);
                }
            l += sum0 + sum1;
            QT_ADD(2, q2);
            QT_BEGIN(q3);
            // this buffer's last weights (own tile i - 2) have been consumed here and stored to the scratch slot
            if (i >= 2u && !(local_wait(&bars->pv_own_done[i & 1u], ((i >> 1) - 1u) & 1u, abort) &&
                             local_wait(&bars->p_own_sent[i & 1u], ((i >> 1) - 1u) & 1u, abort))) {
                ok = false;
                break;
            }
            QT_ADD(3, q3);
            QT_BEGIN(q4);
            {
                // row `head`: its eight 16-byte chunks under the 128-byte swizzle
                unsigned char *mine = smem + kQuadOffPOwn + (i & 1u) * kPairPBytes + head * 128u;
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<uint4 *>(mine + ((unsigned)c ^ (head & 7u)) * 16u) =
                        make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
                m_out[(i & 1u) * kMlaHeads + head] = m_used;
            }
            m_own_saved[i & 1u] = m_used;
            fence_proxy_async();   // the tensor pipe and the bulk stores read these bytes through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->p_written[i & 1u]);
            QT_ADD(4, q4);
            // the tiles of the period before this one: their messages were written a whole period ago
            QT_BEGIN(q1);
            if (!(ok = process_until(4u * i))) break;
            QT_ADD(1, q1);
            // adopt a larger maximum heard from the peers (all of the periods before this one: a fixed set)
            if (m_heard > m_used) {
                l *= m_used == -INFINITY ? 1.0f : exp2_approx(m_used - m_heard);
                m_used = m_heard;
            }
        }
#ifdef YVX_QUAD_TRACE
        if (qtraced) {
            for (int k = 0; k < 5; ++k) yvx_quad_trace[k] = qt[k];
            yvx_quad_trace[5] = (unsigned long long)(clock64() - qt_start);
            yvx_quad_trace[6] = own_tiles;
            yvx_quad_trace[7] = qt[5];
            yvx_quad_trace[8] = qt[6];
            yvx_quad_trace[9] = qt[7];
        }
#endif
        // what is left: the last period's tiles, the peers' tiles behind this CTA's last one
        if (ok) ok = process_until(tiles);
        if (ok) ok = local_wait(&bars->pv_done, (tiles - 1u) & 1u, abort);
        if (!__all_sync(0xffffffffu, ok) && lane == 0) give_up();
        // this CTA's share of the denominators, and the maximum it is relative to, go to the peers
        for (unsigned int d = 1; d < 4u; ++d) {
            const unsigned int destination = (rank + d) & 3u, q = (3u - d) & 3u;
            cluster_store_f32(cluster_map(smem_u32(l_box + q * kMlaHeads + head), destination), l);
            cluster_store_f32(cluster_map(smem_u32(mfin_box + q * kMlaHeads + head), destination), m_used);
        }
        pdl_launch_dependents();
        // (the cluster barrier below is reached by every thread of all four CTAs)
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        bool fine = ok && !*abort;
        float *staged = reinterpret_cast<float *>(smem);
        if (fine) {
            tc_fence_after_sync();
            // the row's denominator: all four shares at the accumulator's scale
            float total = m_used == -INFINITY ? 0.0f : l * exp2_approx(m_used - m_o);
#pragma unroll
            for (int q = 0; q < 3; ++q) {
                const float m_theirs = mfin_box[q * kMlaHeads + head];
                total += m_theirs == -INFINITY ? 0.0f : l_box[q * kMlaHeads + head] * exp2_approx(m_theirs - m_o);
            }
            l = total;
            const float inverse = direct ? 1.0f / l : (l > 0.0f ? 1.0f / l : 0.0f);
            // every tile has been consumed: the tile buffers are free for the turn of the rows
            float *mine = staged + head * (unsigned)part_stride;
            bool finite = true;
#pragma unroll 1
            for (int i = 0; i < kQuadCols / 32; ++i) {
                uint32_t o[32];
                tmem_ld32(tmem_o + lane_base + 32 * i, o);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    const float2 value = make_float2(__uint_as_float(o[c]) * inverse, __uint_as_float(o[c + 1]) * inverse);
                    finite = finite && isfinite(value.x) && isfinite(value.y);
                    *reinterpret_cast<float2 *>(mine + 32 * i + c) = value;
                }
            }
            if (direct && !finite) atomicCAS(p.status, 0, YVX_STATUS_NONFINITE);
            *reinterpret_cast<float2 *>(mine + kQuadCols) =
                make_float2(m_o == -INFINITY ? -INFINITY : m_o * 0.6931471805599453f, l);
            mbar_arrive(&bars->rows_staged);
            fine = local_wait(&bars->rows_staged, 0, abort);
        }
        if (fine) {
            // four rows at a time, all of their loads from shared memory ahead of the stores
            const unsigned int row_words = direct ? (unsigned)kQuadCols / 2u : (unsigned)(kQuadCols + 2) / 2u;
#pragma unroll 1
            for (unsigned int r0 = warp * 32u; r0 < warp * 32u + 32u; r0 += 4u) {
                float2 v[4][3];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 *src = reinterpret_cast<const float2 *>(staged + (r0 + q) * (unsigned)part_stride);
#pragma unroll
                    for (int u = 0; u < 3; ++u)
                        if (lane + 32u * u < row_words) v[q][u] = src[lane + 32u * u];
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float2 *dst = reinterpret_cast<float2 *>(
                        direct ? p.output + ((unsigned long long)b * kMlaHeads + r0 + q) * kMlaLatent + rank * kQuadCols
                               : p.partials + ((((unsigned long long)b * kMlaHeads + r0 + q) * 4ull + rank) * p.max_splits + split) *
                                                  part_stride);
#pragma unroll
                    for (int u = 0; u < 3; ++u)
                        if (lane + 32u * u < row_words) dst[lane + 32u * u] = v[q][u];
                }
            }
        }
    }
    if (warp >= 4u) {
        // the producer, sender and issuer warps meet the softmax warps at the cluster barrier
        __syncwarp();
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem, kMlaTmemColumns);
}

// ---- host side ------------------------------------------------------------------------

typedef CUresult (*MlaEncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                     const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                     const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static MlaEncodeTiledFn mla_encode_entry()
{
    static MlaEncodeTiledFn entry = nullptr;
    static bool resolved = false;
    if (!resolved) {
        void *symbol = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &query) ==
                cudaSuccess &&
            query == cudaDriverEntryPointSuccess)
            entry = reinterpret_cast<MlaEncodeTiledFn>(symbol);
        resolved = true;
    }
    return entry;
}

// 3-D bf16 map {width, rows, outer}, box 64 x box_rows x 1, 128-byte swizzle.
static bool mla_encode(CUtensorMap *map, const void *base, unsigned long long width,
                       unsigned long long rows, unsigned long long outer,
                       unsigned long long outer_stride, unsigned int box_rows)
{
    MlaEncodeTiledFn encode = mla_encode_entry();
    if (!encode || (reinterpret_cast<uintptr_t>(base) & 15u)) return false;
    unsigned long long ob = outer_stride * 2ull;
    if (outer <= 1ull || !ob) {
        if (outer > 1ull) return false;
        outer = 1ull;
        ob = rows * width * 2ull;
    }
    if (ob & 15ull) return false;
    cuuint64_t dims[3] = {width, rows, outer};
    cuuint64_t strides[2] = {width * 2ull, ob};
    cuuint32_t box[3] = {64, box_rows, 1};
    cuuint32_t elem[3] = {1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides,
                  box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace yvx

extern "C" {

// One CTA per SM is resident (shared memory), so a wave is sm_count work items:
// sessions x 2 halves x splits. Every work item pays a fixed cost (query staging,
// first tile latency, writing its partial rows) worth about ten 64-token tiles,
// so the chunk minimises waves x (tiles per chunk + 10): a single wave that
// leaves a few SMs idle beats four full waves of short chunks.
void yvx_cuda_mla_plan(yvx_mla_problem *p, int sm_count)
{
    if (!p) return;
    const unsigned long long wave = (unsigned long long)(sm_count > 0 ? sm_count : 148);
    const unsigned long long lanes = 2ull * p->sessions;
    const unsigned int longest = ((p->kv_tokens_max + 63u) / 64u) * 64u;
    const unsigned long long fixed_tiles = 10ull;
    unsigned int best = 64u;
    unsigned long long best_cost = ~0ull;
    for (unsigned int chunk = longest ? longest : 64u; chunk >= 64u; chunk -= 64u) {
        const unsigned long long splits = ((unsigned long long)p->kv_tokens_max + chunk - 1ull) / chunk;
        const unsigned long long items = lanes * (splits ? splits : 1ull);
        const unsigned long long waves = (items + wave - 1ull) / wave;
        const unsigned long long cost = waves * (chunk / 64ull + fixed_tiles);
        if (cost < best_cost) {  // ties keep the larger chunk (fewer partial rows)
            best_cost = cost;
            best = chunk;
        }
    }
    p->chunk_tokens = best;
    p->max_splits = (p->kv_tokens_max + p->chunk_tokens - 1u) / p->chunk_tokens;
    if (!p->max_splits) p->max_splits = 1u;
    p->balanced_pairs = 0u;
    p->cluster_ctas = 2u;
    // Clusters of four CTAs (YVEX_B200_MLA_FORM=quad): one cluster per session and split, as many splits as keep
    // the clusters within one wave (seven eighths of sm_count / 4: a cluster needs four free SMs of one GPC).
    const char *shape = getenv("YVEX_B200_MLA_FORM");
    if (shape && shape[0] == 'q' && p->sessions) {
        const unsigned long long cap = wave / 4ull * 7ull / 8ull ? wave / 4ull * 7ull / 8ull : 1ull;
        const unsigned long long tiles_max = (unsigned long long)(longest ? longest : 64u) / 64ull;
        unsigned long long splits = cap / p->sessions;
        if (splits < 1ull) splits = 1ull;
        if (splits > tiles_max) splits = tiles_max;
        p->chunk_tokens = (unsigned int)(((tiles_max + splits - 1ull) / splits) * 64ull);
        p->max_splits = (p->kv_tokens_max + p->chunk_tokens - 1u) / p->chunk_tokens;
        if (!p->max_splits) p->max_splits = 1u;
        p->cluster_ctas = 4u;
        return;
    }
    // Uniform lengths (the host knows every session's tiles): equal runs of the sessions' tiles laid end to end,
    // one per pair of SMs, when that costs less than the grid of sessions x splits (which leaves SMs idle
    // whenever sessions x splits x 2 is not a multiple of them). YVEX_B200_MLA_PLAN=grid|balanced forces one.
    const char *form = getenv("YVEX_B200_MLA_INDEPENDENT");
    const char *forced = getenv("YVEX_B200_MLA_PLAN");
    const bool uniform = !p->kv_tokens && p->kv_tokens_uniform > 0u && p->kv_tokens_uniform <= p->kv_tokens_max;
    if (!uniform || !p->sessions || (form && form[0] == '1') || (forced && forced[0] == 'g')) return;
    const unsigned int pairs = (unsigned int)(wave / 2ull ? wave / 2ull : 1ull);
    const yvx::MlaBalance g = yvx::mla_balance(p->sessions, p->kv_tokens_uniform, pairs);
    // every run must hold at least one cost unit: the items of a session are numbered by the pairs between the
    // one that holds its first tile and the one at hand, which only counts them if none of those runs is empty
    if (g.total < pairs) return;
    const unsigned long long balanced_cost = (g.total + pairs - 1ull) / pairs + yvx::kMlaItemCostTiles;
    // (by an eighth at least: a run that crosses sessions pays the item cost twice, and measured on 32 x 16384
    // tokens, where the model promises a tenth, the two plans take the same time)
    if (!(forced && forced[0] == 'b') && balanced_cost * 8ull >= best_cost * 7ull) return;
    unsigned int pieces = 1u;
    for (unsigned int k = 0; k < pairs; ++k) {
        const unsigned long long lo = yvx::mla_run_begin(g, k), hi = yvx::mla_run_begin(g, k + 1ull);
        if (hi <= lo) continue;
        for (unsigned long long b = lo / g.unit; b <= (hi - 1ull) / g.unit && b < p->sessions; ++b) {
            unsigned int tile_lo, tile_hi, slot;
            bool ends;
            if (yvx::mla_balanced_item(g, k, (unsigned int)b, &tile_lo, &tile_hi, &slot, &ends) && slot + 1u > pieces)
                pieces = slot + 1u;
        }
    }
    p->balanced_pairs = pairs;
    p->max_splits = pieces;
    p->chunk_tokens = ((p->kv_tokens_uniform + 63u) / 64u) * 64u;   // not used by the balanced plan; kept a tile multiple
}

#ifdef YVX_QUAD_TRACE
int yvx_cuda_quad_trace_read(unsigned long long out[16])
{
    return cudaMemcpyFromSymbol(out, yvx::yvx_quad_trace, 16 * sizeof(unsigned long long)) == cudaSuccess ? 0 : 1;
}
#endif
#ifdef YVX_MLA_TRACE
int yvx_cuda_mla_trace_read(unsigned long long out[16])
{
    return cudaMemcpyFromSymbol(out, yvx::yvx_mla_trace, 16 * sizeof(unsigned long long)) == cudaSuccess ? 0 : 1;
}
int yvx_cuda_mla_spans_read(unsigned long long out[1024])
{
    return cudaMemcpyFromSymbol(out, yvx::yvx_mla_spans, 1024 * sizeof(unsigned long long)) == cudaSuccess ? 0 : 1;
}
int yvx_cuda_mla_marks_read(unsigned long long out[16])
{
    return cudaMemcpyFromSymbol(out, yvx::yvx_mla_marks, 16 * sizeof(unsigned long long)) == cudaSuccess ? 0 : 1;
}
#endif

unsigned long long yvx_cuda_mla_absorbed_bytes(const yvx_mla_problem *p)
{
    return p ? (unsigned long long)p->sessions * p->heads * (p->latent_dim + p->rope_dim) * 2ull : 0ull;
}

unsigned long long yvx_cuda_mla_partials_bytes(const yvx_mla_problem *p)
{
    if (!p) return 0ull;
    if (p->cluster_ctas == 4u)   // (o[latent_dim / 4], m, l) per session, head, quarter and split, then the messages' scratch slots
        return yvx::mla_quad_rows_bytes(*p) + (unsigned long long)p->sessions * p->max_splits * 8ull * yvx::kQuadMessageBytes;
    return (unsigned long long)p->sessions * p->heads * 2ull * p->max_splits * (p->latent_dim / 2ull + 2ull) * sizeof(float);
}

int yvx_cuda_mla_decode(const yvx_mla_problem *p, void *stream, void *events[4], unsigned int *launches)
{
    using namespace yvx;
    if (launches) *launches = 0;
    if (!p || !p->q_nope || !p->q_rope || !p->w_uk || !p->latent || !p->rope_key || !p->q_absorbed ||
        !p->partials || !p->output || !p->status || !p->sessions || !p->kv_tokens_max ||
        !p->chunk_tokens || !p->max_splits)
        return YVEX_ERR_INVALID_ARG;
    if (p->heads != (unsigned)kMlaHeads || p->nope_dim != (unsigned)kMlaNope ||
        p->latent_dim != (unsigned)kMlaLatent || p->rope_dim != (unsigned)kMlaRope)
        return YVEX_ERR_UNSUPPORTED;
    if (p->chunk_tokens % kMlaN) return YVEX_ERR_INVALID_ARG;
    if (p->balanced_pairs && (p->kv_tokens || !p->kv_tokens_uniform || p->balanced_pairs > 65535u))
        return YVEX_ERR_INVALID_ARG;   // the balanced plan is for uniform lengths
    cudaStream_t s = (cudaStream_t)stream;
    MlaMaps maps;
    if (!mla_encode(&maps.query, p->q_absorbed, kMlaWidth, kMlaHeads, p->sessions,
                    (unsigned long long)kMlaHeads * kMlaWidth, kMlaHeads) ||
        !mla_encode(&maps.latent, p->latent, kMlaLatent, p->kv_tokens_max, p->sessions,
                    p->latent_session_stride, kMlaN) ||
        !mla_encode(&maps.rope, p->rope_key, kMlaRope, p->kv_tokens_max, p->sessions,
                    p->rope_session_stride, kMlaN))
        return YVEX_ERR_UNSUPPORTED;
    cudaError_t error = cudaFuncSetAttribute(mla_absorb_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, kAbsorbSmem);
    if (error == cudaSuccess)
        error = cudaFuncSetAttribute(mla_decode_tcgen05_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmemBytes);
    if (error != cudaSuccess) return yvx_cuda_check(error, "mla kernel attributes");
    if (events) cudaEventRecord((cudaEvent_t)events[0], s);
    mla_absorb_kernel<<<dim3(kMlaHeads, 4), 128, kAbsorbSmem, s>>>(*p);
    if (events) cudaEventRecord((cudaEvent_t)events[1], s);
    // The paired form (one score product per tile for the two CTAs of a pair) is taken unless the
    // environment asks for the independent form (YVEX_B200_MLA_INDEPENDENT=1: comparisons and tests).
    static int pair_configured = -1;
    if (pair_configured < 0) {
        pair_configured = cudaFuncSetAttribute(mla_decode_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               kPairSmemBytes) == cudaSuccess;
        if (!pair_configured) cudaGetLastError();
    }
    const char *choice = getenv("YVEX_B200_MLA_INDEPENDENT");
    const bool paired = pair_configured && !(choice && choice[0] == '1');
    if (p->cluster_ctas == 4u) {
        static int quad_configured = -1;
        if (quad_configured < 0) {
            quad_configured = cudaFuncSetAttribute(mla_decode_quad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   kQuadSmemBytes) == cudaSuccess;
            if (!quad_configured) cudaGetLastError();
        }
        if (!quad_configured || p->balanced_pairs ||
            !mla_encode(&maps.weights, mla_quad_scratch(*p), 64, kMlaHeads, (unsigned long long)p->sessions * p->max_splits * 8ull,
                        (unsigned long long)kMlaHeads * 64ull, kMlaHeads)) {
            yvx_cuda_set_error_text("the four-CTA form of the latent decode kernel is not available for this plan");
            return YVEX_ERR_UNSUPPORTED;
        }
        mla_decode_quad_kernel<<<dim3(4, p->max_splits, p->sessions), kQuadThreads, kQuadSmemBytes, s>>>(*p, maps);
        if (events) cudaEventRecord((cudaEvent_t)events[2], s);
        int quad_rc = yvx_cuda_check(cudaGetLastError(), "mla kernels");
        if (quad_rc != 0) return quad_rc;
        if (p->max_splits > 1u)
            quad_rc = yvx_cuda_lse_combine(p->partials, p->sessions * kMlaHeads * 4u, p->max_splits, kQuadCols, p->output,
                                           YVEX_DTYPE_F32, p->status, stream);
        if (events) cudaEventRecord((cudaEvent_t)events[3], s);
        if (quad_rc != 0) return quad_rc;
        if (launches) *launches = p->max_splits > 1u ? 3u : 2u;
        return 0;
    }
    if (!paired && p->balanced_pairs) {
        yvx_cuda_set_error_text("the balanced plan needs the paired form of the latent decode kernel");
        return YVEX_ERR_UNSUPPORTED;
    }
    if (paired)
        mla_decode_pair_kernel<<<p->balanced_pairs ? dim3(2, p->balanced_pairs, 1) : dim3(2, p->max_splits, p->sessions),
                                 kPairThreads, kPairSmemBytes, s>>>(*p, maps);
    else
        mla_decode_tcgen05_kernel<<<dim3(2, p->max_splits, p->sessions), kMlaThreads, kMlaSmemBytes, s>>>(*p, maps);
    if (events) cudaEventRecord((cudaEvent_t)events[2], s);
    int rc = yvx_cuda_check(cudaGetLastError(), "mla kernels");
    if (rc != 0) return rc;
    rc = yvx_cuda_lse_combine(p->partials, p->sessions * kMlaHeads * 2u, p->max_splits, kMlaHalf,
                              p->output, YVEX_DTYPE_F32, p->status, stream);
    if (events) cudaEventRecord((cudaEvent_t)events[3], s);
    if (rc != 0) return rc;
    if (launches) *launches = 3u;
    return 0;
}

}  // extern "C"
