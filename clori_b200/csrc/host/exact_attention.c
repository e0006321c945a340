/* The exact-attention operator: admission, tensor-view checks, launch and
 * facts. Admission and refusal codes follow the reference operator
 * (src/backend/cuda/exact_attention.c:8-108) and its tensor-view check
 * (src/backend/cuda/transformer.c:725-773). What differs is documented here:
 *
 *  - No score workspace exists on this path (scores never leave the SM), so
 *    attention_workspace_required reports 0 bytes for every admitted geometry,
 *    including packed MHA, where the reference reports its tiled score buffer.
 *  - facts.kernel_launches is the real count: 1 when one KV split covers the
 *    sequence, 2 (attention + combine) otherwise.
 *  - Non-finite outputs are detected on every path and refused with
 *    YVEX_ERR_FORMAT; the reference checks them on its tiled MHA path only.
 */
#include "private.h"

#include <math.h>
#include <string.h>

enum { YVX_EXACT_ATTENTION_HEAD_MAX = 256 };

static int exact_attention_validate(const yvex_transformer_attention_requirement *r,
                                    const char *stage, yvex_error *err)
{
    unsigned long long query_end, query_width, kv_width;
    if (!r || !r->query_tokens || !r->key_value_tokens ||
        !yvx_u64_add(r->query_start, r->query_tokens, &query_end) ||
        query_end > r->key_value_tokens || !r->query_heads || !r->key_value_heads ||
        r->query_heads % r->key_value_heads || !r->head_dimension ||
        !yvx_u64_mul(r->query_heads, r->head_dimension, &query_width) ||
        !yvx_u64_mul(r->key_value_heads, r->head_dimension, &kv_width) ||
        (r->query_token_stride && r->query_token_stride < query_width) ||
        (r->key_token_stride && r->key_token_stride < kv_width) ||
        (r->value_token_stride && r->value_token_stride < kv_width))
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, stage,
                        "complete exact-attention geometry is required");
    if (r->layout != YVEX_TRANSFORMER_ATTENTION_LAYOUT_TOKEN_HEAD_DIM ||
        r->mask < YVEX_TRANSFORMER_ATTENTION_MASK_FULL ||
        r->mask > YVEX_TRANSFORMER_ATTENTION_MASK_CAUSAL ||
        r->numeric_contract != YVEX_TRANSFORMER_ATTENTION_NUMERIC_EXACT_F32 ||
        r->head_dimension > YVX_EXACT_ATTENTION_HEAD_MAX ||
        r->query_dtype != YVEX_DTYPE_F32 || r->key_dtype != YVEX_DTYPE_F32 ||
        r->value_dtype != YVEX_DTYPE_F32 || r->output_dtype != YVEX_DTYPE_F32 ||
        !r->deterministic)
        return yvx_fail(err, YVEX_ERR_UNSUPPORTED, stage,
                        "CUDA requires deterministic token/head/dimension exact F32 attention");
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_b200_transformer_attention_workspace_required(
    const yvex_transformer_attention_requirement *requirement, unsigned long long *bytes,
    yvex_error *err)
{
    int rc;
    if (bytes) *bytes = 0ull;
    rc = exact_attention_validate(requirement, "cuda.transformer.attention.workspace", err);
    if (rc != YVEX_OK) return rc;
    if (!bytes)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, "cuda.transformer.attention.workspace",
                        "a byte-count destination is required");
    return YVEX_OK;
}

static int f32_view(const yvex_backend *backend, const yvex_device_tensor *tensor,
                    unsigned long long elements, int require_written)
{
    return yvx_tensor_owned(backend, tensor) && (!require_written || tensor->is_written) &&
           tensor->dtype == YVEX_DTYPE_F32 && elements <= ULLONG_MAX / sizeof(float) &&
           tensor->bytes == elements * sizeof(float);
}

int yvex_b200_transformer_attention_execute(yvex_backend *backend,
                                            const yvex_transformer_attention_request *request,
                                            yvex_backend_operation_facts *facts,
                                            yvex_error *err)
{
    const char *where = "cuda.transformer.gqa";
    const yvex_transformer_attention_requirement *r;
    unsigned long long query_width, kv_width, query_stride, key_stride, value_stride;
    unsigned long long query_elements, key_elements, value_elements, output_elements;
    yvx_gqa_problem problem;
    unsigned int launches = 0;
    void *scratch = NULL;
    int rc;
    if (!request || !request->query || !request->key || !request->value || !request->output ||
        !facts)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, "cuda.transformer.attention",
                        "complete exact-attention tensors and result facts are required");
    rc = exact_attention_validate(&request->requirement, "cuda.transformer.attention", err);
    if (rc != YVEX_OK) return rc;
    memset(facts, 0, sizeof(*facts));
    rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    r = &request->requirement;
    query_width = r->query_heads * r->head_dimension;
    kv_width = r->key_value_heads * r->head_dimension;
    query_stride = r->query_token_stride ? r->query_token_stride : query_width;
    key_stride = r->key_token_stride ? r->key_token_stride : kv_width;
    value_stride = r->value_token_stride ? r->value_token_stride : kv_width;
    if (r->key_value_tokens > 0xffffffffull - 1024ull || r->query_tokens > 0xffffffffull ||
        !yvx_u64_mul(r->query_tokens - 1ull, query_stride, &query_elements) ||
        !yvx_u64_add(query_elements, query_width, &query_elements) ||
        !yvx_u64_mul(r->query_tokens, query_width, &output_elements) ||
        !yvx_u64_mul(r->key_value_tokens - 1ull, key_stride, &key_elements) ||
        !yvx_u64_add(key_elements, kv_width, &key_elements) ||
        !yvx_u64_mul(r->key_value_tokens - 1ull, value_stride, &value_elements) ||
        !yvx_u64_add(value_elements, kv_width, &value_elements) ||
        !f32_view(backend, request->query, query_elements, 1) ||
        !f32_view(backend, request->key, key_elements, 1) ||
        !f32_view(backend, request->value, value_elements, 1) ||
        !f32_view(backend, request->output, output_elements, 0))
        return yvx_fail(err, YVEX_ERR_FORMAT, where,
                        "bounded Q/K/V views matching the declared token strides are required");

    memset(&problem, 0, sizeof(problem));
    problem.sessions = 1u;
    problem.query_rows = (unsigned int)r->query_tokens;
    problem.query_heads = (unsigned int)r->query_heads;
    problem.kv_heads = (unsigned int)r->key_value_heads;
    problem.head_dim = (unsigned int)r->head_dimension;
    problem.causal = r->mask == YVEX_TRANSFORMER_ATTENTION_MASK_CAUSAL;
    problem.scale = 1.0f / sqrtf((float)r->head_dimension);
    problem.query_dtype = problem.kv_dtype = problem.output_dtype = YVEX_DTYPE_F32;
    problem.query = request->query->data;
    problem.query_row_stride = query_stride;
    problem.output = request->output->data;
    problem.key = request->key->data;
    problem.value = request->value->data;
    problem.key_token_stride = key_stride;
    problem.value_token_stride = value_stride;
    problem.key_head_stride = problem.value_head_stride = r->head_dimension;
    problem.kv_tokens_uniform = problem.kv_tokens_max = (unsigned int)r->key_value_tokens;
    problem.query_start_uniform = (unsigned int)r->query_start;
    problem.status = backend->status_device;
    if (2ull * problem.sessions * problem.kv_heads <= (unsigned long long)YVX_BACKEND_TICKETS)
        problem.tickets = backend->tickets;
    yvx_cuda_gqa_plan_splits(&problem, backend->sm_count);
    {
        /* one arena: the split partials, then (prefill-sized problems) the bf16 staging of the
         * tensor-core path */
        const unsigned long long partial_bytes = (yvx_cuda_gqa_partials_bytes(&problem) + 255ull) & ~255ull;
        const unsigned long long staging_bytes = yvx_cuda_gqa_f32_staging_bytes(&problem);
        rc = yvx_backend_scratch(backend, partial_bytes + staging_bytes, &scratch, where, err);
        if (rc != YVEX_OK) return rc;
        problem.partials = partial_bytes ? scratch : NULL;
        if (staging_bytes) problem.f32_staging = (unsigned char *)scratch + partial_bytes;
    }
    rc = yvx_backend_status_arm(backend, where, err);
    if (rc != YVEX_OK) return rc;
    rc = yvx_cuda_gqa_attention(&problem, backend->stream, &launches);
    if (rc != 0) return yvx_backend_device_fail(backend, rc, where, err);
    facts->kernel_launches = launches;
    facts->temporary_bytes = yvx_cuda_gqa_partials_bytes(&problem) + yvx_cuda_gqa_f32_staging_bytes(&problem);
    facts->state_bytes = (key_elements + value_elements) * sizeof(float);
    facts->activation_bytes = (query_elements + output_elements) * sizeof(float);
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

static const yvex_b200_transformer_operations yvx_operations = {
    yvex_b200_transformer_attention_workspace_required,
    yvex_b200_transformer_attention_execute,
};

/* The reference returns NULL for backends without the table (its CPU backend);
 * callers then refuse (src/runtime/stateful_attention.c:294-298). */
const yvex_b200_transformer_operations *yvex_b200_transformer_operations_get(
    const yvex_backend *backend)
{
    return backend && !backend->failed ? &yvx_operations : NULL;
}
