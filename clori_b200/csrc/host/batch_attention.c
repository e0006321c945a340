/* Batched attention over session KV caches: decode (1 row per session) and
 * speculative verify (2..8 rows), contiguous or block-tabled KV, F32 or BF16
 * operands. An extension: the reference operator has no batch dimension, no
 * 16-bit KV and no block table (src/backend/cuda/exact_attention.c:35-49
 * refuses them). Per-session semantics are the exact operator's. */
#include "private.h"

#include <math.h>
#include <string.h>

static int batch_view(const yvex_backend *backend, const yvex_device_tensor *tensor,
                      yvex_dtype dtype, unsigned long long min_elements)
{
    unsigned long long bytes;
    return yvx_tensor_owned(backend, tensor) && tensor->dtype == dtype &&
           yvx_u64_mul(min_elements, yvx_dtype_bytes(dtype), &bytes) && tensor->bytes >= bytes;
}

int yvex_b200_attention_batch_execute(yvex_backend *backend,
                                      const yvex_b200_attention_batch_request *request,
                                      yvex_backend_operation_facts *facts, yvex_error *err)
{
    const char *where = "b200.attention.batch";
    const yvex_transformer_attention_requirement *r;
    unsigned long long query_width, kv_width, kv_token_stride, value_token_stride, head_stride;
    unsigned long long query_elements, output_elements, kv_elements, block_stride = 0ull;
    unsigned long long session_stride = 0ull, pool_blocks = 0ull, table_elements = 0ull;
    yvx_gqa_problem problem;
    unsigned int launches = 0;
    void *scratch = NULL;
    int rc;
    int q8;
    if (!request || !facts || !request->query || !request->key ||
        (!request->value &&
         request->requirement.numeric_contract !=
             YVEX_TRANSFORMER_ATTENTION_NUMERIC_Q8_0_KV_F32_ACCUMULATE) ||
        !request->output || !request->kv_tokens)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where,
                        "complete batch tensors and result facts are required");
    r = &request->requirement;
    if (!request->session_count || request->session_count > 0xffffull || !r->query_tokens ||
        r->query_tokens > 0xffffffffull || !r->key_value_tokens ||
        r->key_value_tokens > 0xffffffffull - 1024ull || r->query_tokens > r->key_value_tokens ||
        !r->query_heads || !r->key_value_heads || r->query_heads % r->key_value_heads ||
        !r->head_dimension || !yvx_u64_mul(r->query_heads, r->head_dimension, &query_width) ||
        !yvx_u64_mul(r->key_value_heads, r->head_dimension, &kv_width) ||
        (r->query_token_stride && r->query_token_stride < query_width))
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where,
                        "complete batched attention geometry is required");
    if (r->layout != YVEX_TRANSFORMER_ATTENTION_LAYOUT_TOKEN_HEAD_DIM ||
        r->mask < YVEX_TRANSFORMER_ATTENTION_MASK_FULL ||
        r->mask > YVEX_TRANSFORMER_ATTENTION_MASK_CAUSAL || r->head_dimension > 256ull ||
        !r->deterministic || r->key_dtype != r->value_dtype ||
        !((r->numeric_contract == YVEX_TRANSFORMER_ATTENTION_NUMERIC_EXACT_F32 &&
           r->query_dtype == YVEX_DTYPE_F32 && r->key_dtype == YVEX_DTYPE_F32 &&
           r->output_dtype == YVEX_DTYPE_F32) ||
          (r->numeric_contract == YVEX_TRANSFORMER_ATTENTION_NUMERIC_BF16_F32_ACCUMULATE &&
           (r->query_dtype == YVEX_DTYPE_BF16 || r->query_dtype == YVEX_DTYPE_F32) &&
           r->key_dtype == YVEX_DTYPE_BF16 &&
           (r->output_dtype == YVEX_DTYPE_F32 || r->output_dtype == YVEX_DTYPE_BF16)) ||
          (r->numeric_contract == YVEX_TRANSFORMER_ATTENTION_NUMERIC_Q8_0_KV_F32_ACCUMULATE &&
           r->query_dtype == YVEX_DTYPE_BF16 && r->key_dtype == YVEX_DTYPE_Q8_0 &&
           r->head_dimension == 128ull && !r->key_token_stride && !r->value_token_stride &&
           (r->output_dtype == YVEX_DTYPE_F32 || r->output_dtype == YVEX_DTYPE_BF16))))
        return yvx_fail(err, YVEX_ERR_UNSUPPORTED, where,
                        "unsupported layout, mask, numeric contract or dtype combination");
    memset(facts, 0, sizeof(*facts));
    rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;

    q8 = r->key_dtype == YVEX_DTYPE_Q8_0;
    kv_token_stride = r->key_token_stride ? r->key_token_stride : kv_width;
    value_token_stride = r->value_token_stride ? r->value_token_stride : kv_width;
    head_stride = request->kv_head_stride ? request->kv_head_stride : r->head_dimension;
    query_elements = request->session_count * r->query_tokens *
                     (r->query_token_stride ? r->query_token_stride : query_width);
    output_elements = request->session_count * r->query_tokens * query_width;
    if (q8) {
        /* Records: strides are bytes; one record per (64-token block, kv head). */
        const unsigned long long record = yvx_cuda_q8_record_bytes();
        unsigned long long blocks_per_session = (r->key_value_tokens + 63ull) / 64ull;
        head_stride = request->kv_head_stride ? request->kv_head_stride : record;
        block_stride = request->kv_block_stride ? request->kv_block_stride
                                                : head_stride * r->key_value_heads;
        if (head_stride < record || block_stride < head_stride * r->key_value_heads)
            return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "Q8 record strides are too small");
        if (request->kv_layout == YVEX_B200_KV_BLOCK_TABLE) {
            if (!request->block_table || request->block_tokens != 64ull ||
                request->max_blocks_per_session < blocks_per_session)
                return yvx_fail(err, YVEX_ERR_INVALID_ARG, where,
                                "a 64-token block table covering the longest session is required");
            pool_blocks = request->key->bytes / block_stride;
            table_elements = request->session_count * request->max_blocks_per_session;
            if (!pool_blocks || pool_blocks > 0x7fffffffull ||
                !batch_view(backend, request->block_table, YVEX_DTYPE_I32, table_elements))
                return yvx_fail(err, YVEX_ERR_FORMAT, where,
                                "block table and record pool do not match the declared geometry");
            kv_elements = block_stride;
        } else if (request->kv_layout == YVEX_B200_KV_CONTIGUOUS) {
            session_stride = request->kv_session_stride ? request->kv_session_stride
                                                        : blocks_per_session * block_stride;
            kv_elements = (request->session_count - 1ull) * session_stride +
                          blocks_per_session * block_stride;
        } else {
            return yvx_fail(err, YVEX_ERR_UNSUPPORTED, where, "unknown KV layout");
        }
        if (!yvx_tensor_owned(backend, request->key) || request->key->bytes < kv_elements)
            return yvx_fail(err, YVEX_ERR_FORMAT, where,
                            "the Q8 record tensor is smaller than the declared geometry");
    } else if (request->kv_layout == YVEX_B200_KV_BLOCK_TABLE) {
        if (!request->block_table || !request->block_tokens || request->block_tokens % 64ull ||
            !request->max_blocks_per_session ||
            request->max_blocks_per_session * request->block_tokens < r->key_value_tokens)
            return yvx_fail(err, YVEX_ERR_INVALID_ARG, where,
                            "a block table covering the longest session is required "
                            "(block_tokens a multiple of 64)");
        block_stride = request->kv_block_stride
                           ? request->kv_block_stride
                           : request->block_tokens * kv_token_stride;
        pool_blocks = request->key->bytes / yvx_dtype_bytes(r->key_dtype) / block_stride;
        table_elements = request->session_count * request->max_blocks_per_session;
        kv_elements = block_stride; /* at least one block */
        if (!pool_blocks || pool_blocks > 0x7fffffffull ||
            !batch_view(backend, request->block_table, YVEX_DTYPE_I32, table_elements))
            return yvx_fail(err, YVEX_ERR_FORMAT, where,
                            "block table and pool tensors do not match the declared geometry");
    } else if (request->kv_layout == YVEX_B200_KV_CONTIGUOUS) {
        session_stride = request->kv_session_stride;
        if (request->session_count > 1ull && !session_stride)
            return yvx_fail(err, YVEX_ERR_INVALID_ARG, where,
                            "kv_session_stride is required for more than one contiguous session");
        kv_elements = (request->session_count - 1ull) * session_stride +
                      (r->key_value_tokens - 1ull) * kv_token_stride + kv_width;
    } else {
        return yvx_fail(err, YVEX_ERR_UNSUPPORTED, where, "unknown KV layout");
    }
    if (!batch_view(backend, request->query, r->query_dtype, query_elements) ||
        !request->query->is_written ||
        (!q8 && (!batch_view(backend, request->key, r->key_dtype, kv_elements) ||
                 !batch_view(backend, request->value, r->value_dtype, kv_elements))) ||
        !batch_view(backend, request->output, r->output_dtype, output_elements) ||
        !batch_view(backend, request->kv_tokens, YVEX_DTYPE_I32, request->session_count))
        return yvx_fail(err, YVEX_ERR_FORMAT, where,
                        "bounded Q/K/V/output views matching the declared geometry are required");

    memset(&problem, 0, sizeof(problem));
    problem.sessions = (unsigned int)request->session_count;
    problem.query_rows = (unsigned int)r->query_tokens;
    problem.query_heads = (unsigned int)r->query_heads;
    problem.kv_heads = (unsigned int)r->key_value_heads;
    problem.head_dim = (unsigned int)r->head_dimension;
    problem.causal = r->mask == YVEX_TRANSFORMER_ATTENTION_MASK_CAUSAL;
    problem.scale = 1.0f / sqrtf((float)r->head_dimension);
    problem.query_dtype = r->query_dtype;
    problem.kv_dtype = r->key_dtype;
    problem.output_dtype = r->output_dtype;
    problem.query = request->query->data;
    problem.query_row_stride = r->query_token_stride ? r->query_token_stride : query_width;
    problem.query_session_stride = problem.query_row_stride * r->query_tokens;
    problem.output = request->output->data;
    problem.key = request->key->data;
    problem.value = q8 ? request->key->data : request->value->data;
    problem.key_token_stride = kv_token_stride;
    problem.value_token_stride = value_token_stride;
    problem.key_head_stride = problem.value_head_stride = head_stride;
    problem.key_session_stride = problem.value_session_stride = session_stride;
    if (q8) problem.key_block_stride = problem.value_block_stride = block_stride;
    if (request->kv_layout == YVEX_B200_KV_BLOCK_TABLE) {
        problem.block_table = (const int *)request->block_table->data;
        problem.block_tokens = (unsigned int)request->block_tokens;
        problem.block_table_stride = (unsigned int)request->max_blocks_per_session;
        problem.pool_blocks = (unsigned int)pool_blocks;
        problem.key_block_stride = problem.value_block_stride = block_stride;
    }
    problem.kv_tokens = (const unsigned int *)request->kv_tokens->data;
    problem.kv_tokens_max = (unsigned int)r->key_value_tokens;
    problem.query_start_from_end = 1u;
    problem.status = backend->status_device;
    yvx_cuda_gqa_plan_splits(&problem, backend->sm_count);
    rc = yvx_backend_scratch(backend, yvx_cuda_gqa_partials_bytes(&problem), &scratch, where, err);
    if (rc != YVEX_OK) return rc;
    problem.partials = scratch;
    rc = yvx_backend_status_arm(backend, where, err);
    if (rc != YVEX_OK) return rc;
    rc = yvx_cuda_gqa_attention(&problem, backend->stream, &launches);
    if (rc != 0) return yvx_backend_device_fail(backend, rc, where, err);
    facts->kernel_launches = launches;
    facts->temporary_bytes = yvx_cuda_gqa_partials_bytes(&problem);
    facts->activation_bytes = query_elements * yvx_dtype_bytes(r->query_dtype) +
                              output_elements * yvx_dtype_bytes(r->output_dtype);
    facts->compulsory_memory_facts_available = 1;
    if (backend->synchronous) {
        rc = yvx_backend_status_collect(backend, facts, where, err);
        if (rc != YVEX_OK) return rc;
    } else {
        backend->status_pending = 1;
    }
    request->output->is_written = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}
