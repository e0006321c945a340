// The cross-GPU exchange of (o, m, l) rows over NVLink peer memory, shared by the exchange
// kernel and by the attention kernels that fold it into their own tail.
//
// Every rank owns an exchange area [2 epochs][ranks][items][head_dim + 2] floats, [items]
// arrival counters and (behind them) split tickets, and maps its peers' areas (CUDA IPC).
// For one item a group of threads
//   1. stores this rank's row into slot `rank` of the item in EVERY rank's area (peer stores),
//      fences system-wide and adds 1 to the item's arrival counter on every rank;
//   2. waits, bounded, until its own counter shows all ranks' rows of this epoch;
//   3. folds the ranks' rows in rank order (deterministic) and writes the output.
// Counters only grow (epoch * ranks is the target) and the area is double-buffered by epoch
// parity, so nothing is reset and a rank cannot overwrite rows a peer still reads: finishing
// an epoch needs every peer's row of that epoch. Plain peer loads and stores only.
#pragma once

#include "combine.cuh"

namespace yvx {

constexpr unsigned int kExchangeSpinLimit = 1u << 23;  // about a second of 100 ns polls, then status 3

// Release / acquire at system scope (peers are other GPUs).
__device__ __forceinline__ void fence_acq_rel_system()
{
    asm volatile("fence.acq_rel.sys;" ::: "memory");
}

// Steps 1-3 for one item. `row` [hd + 2] and `flag` live in shared memory; the `threads`
// participants (tid 0 .. threads-1, at least x.ranks of them) meet at Sync::sync(). Returns
// false, with status 3 recorded, when the wait ran out.
template <typename Sync>
__device__ __forceinline__ bool exchange_item(const yvx_lse_exchange &x, unsigned int rank, unsigned int items,
                                              unsigned int item, unsigned int hd, const float *row, int *flag,
                                              unsigned int tid, unsigned int threads, void *output,
                                              int output_dtype, unsigned long long output_index, int *status)
{
    const unsigned int stride = hd + 2u;
    const unsigned long long slot = ((unsigned long long)(x.epoch & 1u) * x.ranks + rank) * items + item;
    for (unsigned int r = 0; r < x.ranks; ++r) {
        float *dst = x.gather[r] + slot * stride;
        for (unsigned int d = tid; d < stride; d += threads) dst[d] = row[d];
    }
    Sync::sync();
    // Thread r tells rank r. Its system-wide fence after the barrier orders every thread's peer
    // stores (they happen before it through the barrier) ahead of the count.
    if (tid < x.ranks) {
        fence_acq_rel_system();
        atomicAdd_system(x.arrivals[tid] + item, 1u);
    }
    if (tid == 0) {
        const volatile unsigned int *counter = x.arrivals[rank] + item;
        const unsigned int target = x.epoch * x.ranks;
        int ok = 0;
        for (unsigned int spin = 0; spin < kExchangeSpinLimit; ++spin) {
            if ((int)(*counter - target) >= 0) {
                ok = 1;
                break;
            }
            __nanosleep(100);
        }
        // Acquire side: this fence, then the barrier, order every thread's reads of the peers'
        // rows after the observation of the counter.
        fence_acq_rel_system();
        *flag = ok;
    }
    Sync::sync();
    if (!*flag) {
        if (tid == 0) atomicCAS(status, 0, YVX_STATUS_TIMEOUT);
        return false;
    }
    // Peers wrote the rows, so bypass L1; the loads of up to eight ranks are issued before the
    // first use (one trip to L2 per batch).
    const float *base = x.gather[rank] + ((unsigned long long)(x.epoch & 1u) * x.ranks * items + item) * stride;
    const unsigned long long rank_stride = (unsigned long long)items * stride;
    for (unsigned int d = tid; d < hd; d += threads) {
        float run_max = -INFINITY, run_sum = 0.0f, acc = 0.0f;
        for (unsigned int r0 = 0; r0 < x.ranks; r0 += 8u) {
            float mr[8], lr[8], orow[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const bool live = r0 + u < x.ranks;
                const float *part = base + (unsigned long long)(live ? r0 + u : r0) * rank_stride;
                mr[u] = live ? __ldcg(part + hd) : -INFINITY;
                lr[u] = __ldcg(part + hd + 1u);
                orow[u] = __ldcg(part + d);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (mr[u] == -INFINITY) continue;  // empty shard or past the last rank
                const float new_max = fmaxf(run_max, mr[u]);
                const float keep = expf(run_max - new_max);
                const float weight = lr[u] * expf(mr[u] - new_max);
                run_sum = fmaf(run_sum, keep, weight);
                acc = fmaf(acc, keep, orow[u] * weight);
                run_max = new_max;
            }
        }
        const float value = acc / run_sum;
        if (!isfinite(value)) atomicCAS(status, 0, YVX_STATUS_NONFINITE);
        store_output(output, output_dtype, output_index + d, value);
    }
    return true;
}


// ---- the same exchange without fences or counters ------------------------------------------
// Every 32-bit lane of a row travels in its own 8-byte word (value, epoch): an aligned 8-byte
// store is indivisible, so a receiver that reads the epoch of this step in a word has its value
// too, and nothing has to be ordered: no system-wide fence, no arrival counter, one NVLink store
// latency from the sender's last store to the receiver's fold. The area is [2 epochs][ranks]
// [items][head_dim + 2] words of 8 bytes, zero-filled once; epochs count from 1 and only grow,
// and the parity double buffer keeps a fast rank from overwriting words a slow one still reads
// (finishing an epoch needs every peer's words of that epoch). Waits are bounded.
__device__ __forceinline__ void store_word_system(uint2 *address, uint32_t value, uint32_t tag)
{
    asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(address), "r"(value), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 load_word_system(const uint2 *address)
{
    uint2 word;
    asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(word.x), "=r"(word.y) : "l"(address) : "memory");
    return word;
}

// Bounded wait for one tagged word; returns false when the tag did not come (or when another
// thread of the group has already given up: `alive` in shared memory turns 0).
__device__ __forceinline__ bool wait_word_system(const uint2 *address, uint32_t tag, float *value,
                                                 const volatile int *alive)
{
    for (unsigned int spin = 0; spin < kExchangeSpinLimit; ++spin) {
        const uint2 word = load_word_system(address);
        if (word.y == tag) {
            *value = __uint_as_float(word.x);
            return true;
        }
        if (spin > 64u) {
            __nanosleep(100);
            if ((spin & 1023u) == 0u && !*alive) break;
        }
    }
    *value = 0.0f;
    return false;
}

// `row` [hd + 2], `scales` [2 * ranks floats] and `flag` live in shared memory; `threads`
// participants (at least x.ranks) meet at Sync::sync().
template <typename Sync>
__device__ __forceinline__ bool exchange_item_tagged(const yvx_lse_exchange &x, unsigned int rank, unsigned int items,
                                                     unsigned int item, unsigned int hd, const float *row,
                                                     float *scales, int *flag, unsigned int tid, unsigned int threads,
                                                     void *output, int output_dtype, unsigned long long output_index,
                                                     int *status, bool publish = true)
{
    const unsigned int stride = hd + 2u;
    const unsigned long long slot = ((unsigned long long)(x.epoch & 1u) * x.ranks + rank) * items + item;
    for (unsigned int r = 0; publish && r < x.ranks; ++r) {   // (publish = false: a rank that never comes, for tests)
        uint2 *dst = reinterpret_cast<uint2 *>(x.gather[r]) + slot * stride;
        for (unsigned int d = tid; d < stride; d += threads) store_word_system(dst + d, __float_as_uint(row[d]), x.epoch);
    }
    if (tid == 0) *flag = 1;
    Sync::sync();
    const uint2 *base = reinterpret_cast<const uint2 *>(x.gather[rank]) +
                        ((unsigned long long)(x.epoch & 1u) * x.ranks * items + item) * stride;
    const unsigned long long rank_stride = (unsigned long long)items * stride;
    // The (m, l) words of rank r are polled by thread threads - 1 - r (the high threads, which
    // have no lane when there are more threads than lanes) into shared memory.
    bool mine_came = true;
    for (unsigned int r = threads - 1u - tid; r < x.ranks; r += threads) {
        float m, l;
        const bool came = wait_word_system(base + r * rank_stride + hd, x.epoch, &m, flag) &&
                          wait_word_system(base + r * rank_stride + hd + 1u, x.epoch, &l, flag);
        if (!came) {
            *flag = 0;
            mine_came = false;
        }
        scales[2u * r] = came ? m : -INFINITY;
        scales[2u * r + 1u] = came ? l : 0.0f;
    }
    Sync::sync();
    // A thread polls its lane of up to eight ranks with all loads in flight at once (one trip to
    // L2 per round, not one per rank); what has not come is polled again.
    for (unsigned int d = tid; d < hd && *flag; d += threads) {
        float run_max = -INFINITY, run_sum = 0.0f, acc = 0.0f;
        for (unsigned int r0 = 0; r0 < x.ranks && mine_came; r0 += 8u) {
            float value[8];
            unsigned int missing = 0u;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (r0 + u < x.ranks) missing |= 1u << u;
            for (unsigned int spin = 0; missing && spin < kExchangeSpinLimit; ++spin) {
                uint2 word[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (missing >> u & 1u) word[u] = load_word_system(base + (r0 + u) * rank_stride + d);
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if ((missing >> u & 1u) && word[u].y == x.epoch) {
                        value[u] = __uint_as_float(word[u].x);
                        missing &= ~(1u << u);
                    }
                if (missing && spin > 64u) {
                    __nanosleep(100);
                    if ((spin & 1023u) == 0u && !*flag) break;
                }
            }
            if (missing) {
                mine_came = false;
                *flag = 0;
                break;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (r0 + u >= x.ranks) break;
                const float mr = scales[2u * (r0 + u)], lr = scales[2u * (r0 + u) + 1u];
                if (mr == -INFINITY) continue;  // empty shard
                const float new_max = fmaxf(run_max, mr);
                const float keep = expf(run_max - new_max);
                const float weight = lr * expf(mr - new_max);
                run_sum = fmaf(run_sum, keep, weight);
                acc = fmaf(acc, keep, value[u] * weight);
                run_max = new_max;
            }
        }
        const float result = acc / run_sum;
        if (mine_came) {
            if (!isfinite(result)) atomicCAS(status, 0, YVX_STATUS_NONFINITE);
            store_output(output, output_dtype, output_index + d, result);
        }
    }
    if (!mine_came) atomicCAS(status, 0, YVX_STATUS_TIMEOUT);
    Sync::sync();   // the caller reuses `row`; and one thread's verdict becomes the group's
    return *flag != 0;
}

// The fold of one item's split partials by `WARPS` warps that meet at Sync::sync(): warp w takes
// splits w, w + WARPS, ...; a lane owns four dimensions (head_dim 128); the warps' running states
// are merged in warp order through `scratch` ([WARPS][head_dim + 2] floats of shared memory) into
// `row` [head_dim + 2] = (o normalised, m, l). Deterministic.
template <int WARPS, typename Sync>
__device__ __forceinline__ void fold_splits_128(const float *parts, unsigned int count, float *scratch, float *row,
                                                unsigned int tid)
{
    constexpr unsigned int kHd = 128u, kStride = kHd + 2u;
    const unsigned int warp = tid >> 5, lane = tid & 31u;
    float run_max = -INFINITY, run_sum = 0.0f;
    float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
    for (unsigned int j0 = warp; j0 < count; j0 += WARPS * 4u) {
        float2 lo[4], hi[4];
        float mj[4], lj[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const unsigned int j = j0 + u * WARPS;
            const bool live = j < count;
            const float *part = parts + (unsigned long long)(live ? j : j0) * kStride;
            lo[u] = __ldcg(reinterpret_cast<const float2 *>(part + 4u * lane));
            hi[u] = __ldcg(reinterpret_cast<const float2 *>(part + 4u * lane + 2u));
            mj[u] = live ? __ldcg(part + kHd) : -INFINITY;
            lj[u] = __ldcg(part + kHd + 1u);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (mj[u] == -INFINITY) continue;
            const float fresh = fmaxf(run_max, mj[u]);
            const float keep = expf(run_max - fresh);
            const float weight = lj[u] * expf(mj[u] - fresh);
            run_sum = fmaf(run_sum, keep, weight);
            total.x = fmaf(total.x, keep, lo[u].x * weight);
            total.y = fmaf(total.y, keep, lo[u].y * weight);
            total.z = fmaf(total.z, keep, hi[u].x * weight);
            total.w = fmaf(total.w, keep, hi[u].y * weight);
            run_max = fresh;
        }
    }
    float *mine = scratch + warp * kStride;
    mine[4u * lane] = total.x;
    mine[4u * lane + 1u] = total.y;
    mine[4u * lane + 2u] = total.z;
    mine[4u * lane + 3u] = total.w;
    if (lane == 0) {
        mine[kHd] = run_max;
        mine[kHd + 1u] = run_sum;
    }
    Sync::sync();
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, scratch[w * kStride + kHd]);
    float ll = 0.0f, scale_w[WARPS];
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
        const float mw = scratch[w * kStride + kHd];
        scale_w[w] = mw == -INFINITY ? 0.0f : expf(mw - mm);
        ll = fmaf(scratch[w * kStride + kHd + 1u], scale_w[w], ll);
    }
    for (unsigned int d = tid; d < kHd; d += WARPS * 32u) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) o = fmaf(scratch[w * kStride + d], scale_w[w], o);
        row[d] = ll > 0.0f ? o / ll : 0.0f;
    }
    if (tid == 0) {
        row[kHd] = mm;
        row[kHd + 1u] = ll;
    }
    Sync::sync();
}

}  // namespace yvx
