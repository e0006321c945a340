// Kernel selection and split planning for grouped-query attention.
#include "common.cuh"

namespace yvx {
int gqa_generic_main_launch(const yvx_gqa_problem &p, cudaStream_t stream);
int gqa_combine_launch(const yvx_gqa_problem &p, cudaStream_t stream);
int gqa_decode_mma_launch(const yvx_gqa_problem &p, cudaStream_t stream);
int gqa_decode_q8_launch(const yvx_gqa_problem &p, cudaStream_t stream);
}

extern "C" {

// Splits exist to fill the machine: the chunk is the smallest multiple of 64
// tokens that keeps the number of (session, kv head, split) work items near
// eight CTAs per SM, bounded to [64, 1024]. It depends only on the problem's
// shape, so repeated calls split identically and results repeat bit for bit.
void yvx_cuda_gqa_plan_splits(yvx_gqa_problem *p, int sm_count)
{
    if (!p) return;
    const unsigned long long target = (unsigned long long)(sm_count > 0 ? sm_count : 148) * 8ull;
    const unsigned long long rows_total =
        (unsigned long long)p->kv_tokens_max * p->sessions * p->kv_heads;
    unsigned long long chunk = (rows_total + target - 1ull) / target;
    chunk = (chunk + 63ull) / 64ull * 64ull;
    if (chunk < 64ull) chunk = 64ull;
    if (chunk > 1024ull) chunk = 1024ull;
    p->chunk_tokens = (unsigned int)chunk;
    p->max_splits = (p->kv_tokens_max + p->chunk_tokens - 1u) / p->chunk_tokens;
    if (!p->max_splits) p->max_splits = 1u;
}

unsigned long long yvx_cuda_gqa_partials_bytes(const yvx_gqa_problem *p)
{
    if (!p || p->max_splits <= 1u) return 0ull;
    return (unsigned long long)p->sessions * p->query_rows * p->query_heads * p->max_splits *
           (p->head_dim + 2ull) * sizeof(float);
}

static int gqa_launch(const yvx_gqa_problem *p, void *stream, cudaEvent_t *events,
                      unsigned int *launches)
{
    unsigned int count = 0;
    if (launches) *launches = 0;
    if (!p || !p->query || !p->key || (!p->value && p->kv_dtype != YVEX_DTYPE_Q8_0) ||
        (!p->output && !p->partial_output) ||
        !p->status || !p->sessions || !p->query_rows || !p->query_heads || !p->kv_heads ||
        p->query_heads % p->kv_heads || !p->head_dim || !p->chunk_tokens || !p->max_splits ||
        (p->max_splits > 1u && !p->partials) || (p->block_table && !p->block_tokens))
        return YVEX_ERR_INVALID_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (events) cudaEventRecord(events[0], s);
    // Specialised kernels return 1 when they took the problem, 0 when its shape
    // is not theirs; the general kernel takes everything else.
    int rc = yvx::gqa_decode_q8_launch(*p, s);
    if (rc == 0 && !p->force_general) rc = yvx::gqa_decode_mma_launch(*p, s);
    if (rc == 0) rc = yvx::gqa_generic_main_launch(*p, s);
    else if (rc == 1) rc = 0;
    if (rc != 0) return rc;
    count = 1u;
    if (events) cudaEventRecord(events[1], s);
    if (p->max_splits > 1u) {
        rc = yvx::gqa_combine_launch(*p, s);
        if (rc != 0) return rc;
        count = 2u;
    }
    if (events) cudaEventRecord(events[2], s);
    if (launches) *launches = count;
    return 0;
}

int yvx_cuda_gqa_attention(const yvx_gqa_problem *p, void *stream, unsigned int *launches)
{
    return gqa_launch(p, stream, nullptr, launches);
}

int yvx_cuda_gqa_attention_profiled(const yvx_gqa_problem *p, void *stream, void *events[3],
                                    unsigned int *launches)
{
    if (!events || !events[0] || !events[1] || !events[2]) return YVEX_ERR_INVALID_ARG;
    cudaEvent_t typed[3] = {(cudaEvent_t)events[0], (cudaEvent_t)events[1], (cudaEvent_t)events[2]};
    return gqa_launch(p, stream, typed, launches);
}

}  // extern "C"
