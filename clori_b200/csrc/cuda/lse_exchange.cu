// Cross-GPU fold of split-attention partials over NVLink peer memory, fused with
// the rank's own split fold: one kernel where the plain path runs a local
// combine, an NCCL all-gather and a second combine.
//
// Every rank owns an exchange area [2 epochs][ranks][items][head_dim + 2] floats
// and [items] arrival counters, and maps its peers' areas (CUDA IPC). CTA i:
//   1. folds this rank's splits of item i into one row (o normalised, m, l);
//   2. stores the row into slot `rank` of item i in EVERY rank's area (peer
//      stores over NVLink), fences system-wide, and adds 1 to item i's arrival
//      counter on every rank;
//   3. waits (bounded) until its own counter shows all ranks' rows of this epoch;
//   4. folds the ranks' rows in rank order (deterministic) and writes the output.
// Counters only grow (epoch * ranks is the target), the area is double-buffered by
// epoch parity, so no reset and no reuse hazard: a rank cannot be two epochs ahead
// of a peer, because finishing an epoch needs that peer's row of the same epoch.
// Plain peer loads and stores only; no multicast, no TMA.
#include "combine.cuh"

namespace yvx {

constexpr int kExchangeThreads = kCombineWarps * 32;
constexpr unsigned int kExchangeSpinLimit = 1u << 23;  // about a second of 100 ns polls, then status 3

// Release / acquire at system scope (peers are other GPUs); lighter than the
// sequentially consistent fence and all this protocol needs.
__device__ __forceinline__ void fence_acq_rel_system()
{
    asm volatile("fence.acq_rel.sys;" ::: "memory");
}

__global__ void __launch_bounds__(kExchangeThreads)
lse_exchange_kernel(const yvx_gqa_problem p, const yvx_lse_exchange x, const unsigned int items,
                    const int emulated)
{
    pdl_wait();  // the split kernel's partials must be complete and visible
    __shared__ float row[258];
    __shared__ int arrived;
    const unsigned int item = blockIdx.x;
    const unsigned int rank = emulated ? blockIdx.y : x.rank;
    const unsigned int hd = p.head_dim, stride = hd + 2u;
    // 1. this rank's row
    if (p.max_splits > 1u && !emulated) {
        const unsigned int b = (unsigned int)(item / ((unsigned long long)p.query_rows * p.query_heads));
        const unsigned int kv_tokens = admitted_kv_tokens(p.kv_tokens, b, p.kv_tokens_uniform, p.kv_tokens_max, p.status);
        const unsigned int splits = min((kv_tokens + p.chunk_tokens - 1u) / p.chunk_tokens, p.max_splits);
        combine_parts(p.partials + (unsigned long long)item * p.max_splits * stride, splits, stride, hd, nullptr,
                      0, 0ull, row, p.status);
    } else {
        const float *mine = p.partial_output + ((unsigned long long)(emulated ? rank * items : 0u) + item) * stride;
        for (unsigned int d = threadIdx.x; d < stride; d += kExchangeThreads) row[d] = mine[d];
    }
    __syncthreads();
    // 2. publish to every rank, then count
    const unsigned long long slot = ((unsigned long long)(x.epoch & 1u) * x.ranks + rank) * items + item;
    for (unsigned int r = 0; r < x.ranks; ++r) {
        float *dst = x.gather[r] + slot * stride;
        for (unsigned int d = threadIdx.x; d < stride; d += kExchangeThreads) dst[d] = row[d];
    }
    __syncthreads();
    // Thread r tells rank r. Its system-wide fence after the barrier orders every
    // thread's peer stores (they happen before it through the barrier) ahead of the count.
    if (threadIdx.x < x.ranks) {
        fence_acq_rel_system();
        atomicAdd_system(x.arrivals[threadIdx.x] + item, 1u);
    }
    if (threadIdx.x == 0) {
        // 3. bounded wait for the rows of all ranks
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
        // Acquire side: this fence, then the barrier, order every thread's reads of the
        // peers' rows after the observation of the counter.
        fence_acq_rel_system();
        arrived = ok;
    }
    __syncthreads();
    if (!arrived) {
        if (threadIdx.x == 0) atomicCAS(p.status, 0, YVX_STATUS_TIMEOUT);
        return;
    }
    // 4. fold the ranks' rows in rank order; peers wrote them, so bypass L1. All loads
    // of up to eight ranks are issued before the first use (one trip to L2 per batch).
    const float *base = x.gather[rank] + ((unsigned long long)(x.epoch & 1u) * x.ranks * items + item) * stride;
    const unsigned long long rank_stride = (unsigned long long)items * stride;
    for (unsigned int d = threadIdx.x; d < hd; d += kExchangeThreads) {
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
        if (!isfinite(value)) atomicCAS(p.status, 0, YVX_STATUS_NONFINITE);
        store_output(emulated ? (void *)((float *)p.output + (unsigned long long)rank * items * hd) : p.output,
                     p.output_dtype, (unsigned long long)item * hd + d, value);
    }
}

int lse_exchange_launch(const yvx_gqa_problem &p, const yvx_lse_exchange &x, cudaStream_t stream)
{
    const unsigned long long items = (unsigned long long)p.sessions * p.query_rows * p.query_heads;
    if (!x.ranks || x.ranks > 64u || x.rank >= x.ranks || !x.epoch || !x.gather || !x.arrivals ||
        p.head_dim > 256u || !items || items > 0x7fffffffull || !p.partial_output || !p.output)
        return YVEX_ERR_INVALID_ARG;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned int)items, 1, 1);
    config.blockDim = dim3(kExchangeThreads, 1, 1);
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    const cudaError_t launched =
        cudaLaunchKernelEx(&config, lse_exchange_kernel, p, x, (unsigned int)items, 0);
    if (launched != cudaSuccess) return yvx_cuda_check(launched, "lse_exchange_kernel");
    return yvx_cuda_check(cudaGetLastError(), "lse_exchange_kernel");
}

}  // namespace yvx

// All ranks of the exchange emulated by ONE cooperative launch on one GPU (the
// blocks wait on one another, so they must be co-resident): block (item, rank)
// plays `rank` with its row taken from rows[rank][item][head_dim + 2] and its
// output written to output[rank][item][head_dim]. For tests without several GPUs.
extern "C" int yvx_cuda_lse_exchange_emulated(const float *rows, unsigned int ranks, unsigned int items,
                                              unsigned int head_dim, float *const *gather,
                                              unsigned int *const *arrivals, unsigned int epoch,
                                              float *output, int *status, void *stream)
{
    using namespace yvx;
    if (!rows || !ranks || ranks > 64u || !items || !head_dim || head_dim > 256u || !gather || !arrivals ||
        !epoch || !output || !status)
        return YVEX_ERR_INVALID_ARG;
    int device = 0, sms = 0, per_sm = 0;
    YVX_CUDA_TRY(cudaGetDevice(&device));
    YVX_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    YVX_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lse_exchange_kernel, kExchangeThreads, 0));
    if ((unsigned long long)items * ranks > (unsigned long long)sms * per_sm) return YVEX_ERR_BOUNDS;
    yvx_gqa_problem p = {};
    p.sessions = 1;
    p.query_rows = 1;
    p.query_heads = items;
    p.head_dim = head_dim;
    p.max_splits = 1;
    p.partial_output = const_cast<float *>(rows);
    p.output = output;
    p.output_dtype = YVEX_DTYPE_F32;
    p.status = status;
    yvx_lse_exchange x = {};
    x.ranks = ranks;
    x.epoch = epoch;
    x.gather = gather;
    x.arrivals = arrivals;
    int emulated = 1;
    void *args[] = {&p, &x, &items, &emulated};
    YVX_CUDA_TRY(cudaLaunchCooperativeKernel((const void *)lse_exchange_kernel, dim3(items, ranks, 1),
                                             dim3(kExchangeThreads, 1, 1), args, 0, (cudaStream_t)stream));
    return 0;
}
