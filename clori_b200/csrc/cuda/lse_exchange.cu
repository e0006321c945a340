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
#include "exchange.cuh"

namespace yvx {

constexpr int kExchangeThreads = kCombineWarps * 32;

struct BlockSync {
    static __device__ __forceinline__ void sync() { __syncthreads(); }
};

// four CTAs per SM: the emulation of all ranks on one GPU needs ranks x items of them resident
__global__ void __launch_bounds__(kExchangeThreads, 4)
lse_exchange_kernel(const yvx_gqa_problem p, const yvx_lse_exchange x, const unsigned int items,
                    const int emulated)
{
    pdl_wait();  // the split kernel's partials must be complete and visible
    __shared__ float row[258];
    __shared__ float scales[2 * 64];
    __shared__ int arrived;
    const unsigned int rank = emulated ? blockIdx.y : x.rank;
    const unsigned int hd = p.head_dim, stride = hd + 2u;
    // The grid is never larger than what is resident at once; a CTA walks items blockIdx.x,
    // blockIdx.x + gridDim.x, ... in the same order on every rank, so a CTA that waits for a
    // peer's item waits for a CTA that is running.
    for (unsigned int item = blockIdx.x; item < items; item += gridDim.x) {
        __syncthreads();   // the previous item's row has been read by every thread
        // this rank's row
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
        void *out = emulated ? (void *)((float *)p.output + (unsigned long long)rank * items * hd) : p.output;
        if (x.tagged_words)   // emulated >= 2: rank (emulated - 2) never publishes
            exchange_item_tagged<BlockSync>(x, rank, items, item, hd, row, scales, &arrived, threadIdx.x, kExchangeThreads,
                                            out, p.output_dtype, (unsigned long long)item * hd, p.status,
                                            emulated < 2 || rank != (unsigned)(emulated - 2));
        else
            exchange_item<BlockSync>(x, rank, items, item, hd, row, &arrived, threadIdx.x, kExchangeThreads, out,
                                     p.output_dtype, (unsigned long long)item * hd, p.status);
    }
}

int lse_exchange_launch(const yvx_gqa_problem &p, const yvx_lse_exchange &x, cudaStream_t stream)
{
    const unsigned long long items = (unsigned long long)p.sessions * p.query_rows * p.query_heads;
    if (!x.ranks || x.ranks > 64u || x.rank >= x.ranks || !x.epoch || !x.gather || !x.arrivals ||
        p.head_dim > 256u || !items || items > 0x7fffffffull || !p.partial_output || !p.output)
        return YVEX_ERR_INVALID_ARG;
    // CTAs of this launch wait for CTAs of the peers' launches: only as many as are resident at once
    static int configured_device = -1, resident = 0;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return YVEX_ERR_BACKEND;
    if (configured_device != device) {
        int sms = 0, per_sm = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lse_exchange_kernel, kExchangeThreads, 0) != cudaSuccess ||
            sms * per_sm < 1)
            return YVEX_ERR_BACKEND;
        resident = sms * per_sm;
        configured_device = device;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned int)min(items, (unsigned long long)resident), 1, 1);
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
    return yvx_cuda_lse_exchange_emulated_form(rows, ranks, items, head_dim, gather, arrivals, epoch, output, status,
                                               stream, 0, -1);
}

extern "C" int yvx_cuda_lse_exchange_emulated_form(const float *rows, unsigned int ranks, unsigned int items,
                                                   unsigned int head_dim, float *const *gather,
                                                   unsigned int *const *arrivals, unsigned int epoch,
                                                   float *output, int *status, void *stream, int tagged_words,
                                                   int absent_rank)
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
    x.tagged_words = tagged_words;
    int emulated = tagged_words && absent_rank >= 0 ? 2 + absent_rank : 1;
    void *args[] = {&p, &x, &items, &emulated};
    YVX_CUDA_TRY(cudaLaunchCooperativeKernel((const void *)lse_exchange_kernel, dim3(items, ranks, 1),
                                             dim3(kExchangeThreads, 1, 1), args, 0, (cudaStream_t)stream));
    return 0;
}
