/* Operator-level entry points for the latent attention stages and the KV
 * append: borrowed yvex_device_tensor arguments, ownership and extent checks,
 * the reference's refusal codes, the backend's status word, facts.
 *
 * yvex_b200_attention_reduce_execute is the reduce stage of the encoded
 * attention job (yvex_backend_attention_execute, include/yvex/internal/
 * backend.h:193-195; stage in src/backend/cuda/attention.c:1386-1422), with
 * the reference's typed failure {code, stage, expected, actual}
 * (include/yvex/internal/backend.h:144-161).
 * yvex_b200_kv_append_rotary_execute stands where src/runtime/decoder.c:
 * 1112-1131 and src/runtime/stateful_attention.c:183-243 rotate and copy.
 * yvex_b200_attention_select_execute is the sparse index selection in front of
 * that stage (CPU reference src/graph/attention.c:369-497).
 * yvex_b200_attention_compress_execute is the rolling compressor that feeds both
 * (CPU reference src/graph/attention.c:745-836, attention_execute.c:730-832).
 * yvex_b200_mla_decode_execute has no counterpart in the reference. */
#include "private.h"

#include <math.h>
#include <string.h>

static int view_ok(const yvex_backend *backend, const yvex_device_tensor *tensor, yvex_dtype dtype,
                   unsigned long long elements)
{
    unsigned long long bytes;
    return yvx_tensor_owned(backend, tensor) && tensor->dtype == dtype &&
           yvx_u64_mul(elements, yvx_dtype_bytes(dtype), &bytes) && tensor->bytes >= bytes;
}

static int reduce_refuse(yvex_b200_attention_failure *failure, yvex_b200_attention_failure_code code,
                         unsigned long long expected, unsigned long long actual, yvex_error *err,
                         yvex_status status, const char *message)
{
    if (failure) {
        failure->code = code;
        failure->stage = "reduce";
        failure->expected = expected;
        failure->actual = actual;
    }
    return yvx_fail(err, status, "b200.attention.reduce", message);
}

static int finish(yvex_backend *backend, yvex_backend_operation_facts *facts, unsigned int launches,
                  unsigned long long temporary, const char *where, yvex_error *err)
{
    facts->kernel_launches = launches;
    facts->temporary_bytes = temporary;
    facts->compulsory_memory_facts_available = 1;
    if (backend->synchronous) return yvx_backend_status_collect(backend, facts, where, err);
    backend->status_pending = 1;
    return YVEX_OK;
}

int yvex_b200_attention_reduce_execute(yvex_backend *backend,
                                       const yvex_b200_attention_reduce_request *r,
                                       yvex_b200_attention_failure *failure,
                                       yvex_backend_operation_facts *facts, yvex_error *err)
{
    const char *where = "b200.attention.reduce";
    unsigned long long width, local_rows, elements = 0ull, workspace;
    unsigned int launches = 0u;
    void *scratch = NULL;
    yvx_latent_reduce_args a;
    int rc;
    if (failure) memset(failure, 0, sizeof(*failure));
    if (!r || !facts || !r->query || !r->local || !r->local_positions || !r->sinks || !r->output)
        return reduce_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, 1ull, 0ull, err,
                             YVEX_ERR_INVALID_ARG, "query, local rows, positions, sinks and output are required");
    memset(facts, 0, sizeof(*facts));
    rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (!r->token_count || !r->query_heads || !r->head_dimension || !r->sliding_window ||
        !yvx_u64_mul(r->query_heads, r->head_dimension, &width) ||
        !yvx_u64_add(r->local_count, r->token_count, &local_rows) || r->local_stride < r->head_dimension)
        return reduce_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, r->head_dimension,
                             r->local_stride, err, YVEX_ERR_INVALID_ARG,
                             "token count, heads, head dimension, window and local stride must be consistent");
    if (r->head_dimension > 512ull || r->attention_class > YVEX_B200_ATTENTION_HCA)
        return reduce_refuse(failure, YVEX_B200_ATTENTION_FAILURE_CAPABILITY, 512ull, r->head_dimension, err,
                             YVEX_ERR_UNSUPPORTED, "head dimension above 512 or unknown attention class");
    if (r->attention_class != YVEX_B200_ATTENTION_SWA) {
        if (!r->compressed || !r->compressed_positions || !r->compression_ratio ||
            r->compressed_stride < r->head_dimension)
            return reduce_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, r->head_dimension,
                                 r->compressed_stride, err, YVEX_ERR_INVALID_ARG,
                                 "compressed rows, positions and ratio are required for this class");
        if (r->attention_class == YVEX_B200_ATTENTION_CSA && (!r->selected || !r->selected_count || !r->indexer_topk))
            return reduce_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, 1ull, 0ull, err,
                                 YVEX_ERR_INVALID_ARG, "selected rows and counts are required for sparse attention");
    }
    if (!yvx_u64_mul(r->token_count, width, &elements) || !view_ok(backend, r->query, YVEX_DTYPE_F32, elements) ||
        !view_ok(backend, r->output, YVEX_DTYPE_F32, elements) ||
        !view_ok(backend, r->sinks, YVEX_DTYPE_F32, r->query_heads) ||
        !yvx_u64_mul(local_rows, r->local_stride, &elements) || !view_ok(backend, r->local, YVEX_DTYPE_F32, elements) ||
        !view_ok(backend, r->local_positions, YVEX_DTYPE_I64, local_rows))
        return reduce_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, elements,
                             r->local ? r->local->bytes : 0ull, err, YVEX_ERR_FORMAT,
                             "tensor views do not cover the stated geometry");
    if (r->attention_class != YVEX_B200_ATTENTION_SWA) {
        if (!yvx_u64_mul(r->compressed_count ? r->compressed_count : 1ull, r->compressed_stride, &elements) ||
            !view_ok(backend, r->compressed, YVEX_DTYPE_F32, elements) ||
            !view_ok(backend, r->compressed_positions, YVEX_DTYPE_I64, r->compressed_count ? r->compressed_count : 1ull))
            return reduce_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, elements,
                                 r->compressed->bytes, err, YVEX_ERR_FORMAT,
                                 "compressed views do not cover the stated geometry");
        if (r->attention_class == YVEX_B200_ATTENTION_CSA &&
            (!yvx_u64_mul(r->token_count, r->indexer_topk, &elements) ||
             !view_ok(backend, r->selected, YVEX_DTYPE_I64, elements) ||
             !view_ok(backend, r->selected_count, YVEX_DTYPE_I64, r->token_count)))
            return reduce_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, elements,
                                 r->selected->bytes, err, YVEX_ERR_FORMAT,
                                 "selected views do not cover the stated geometry");
    }
    memset(&a, 0, sizeof(a));
    a.query = (const float *)r->query->data;
    a.local = (const float *)r->local->data;
    a.local_positions = (const unsigned long long *)r->local_positions->data;
    a.initial_local_count = r->local_count;
    a.local_stride = r->local_stride;
    if (r->attention_class != YVEX_B200_ATTENTION_SWA) {
        a.compressed = (const float *)r->compressed->data;
        a.compressed_positions = (const unsigned long long *)r->compressed_positions->data;
        a.compressed_stride = r->compressed_stride;
        a.ratio = r->compression_ratio;
    }
    if (r->attention_class == YVEX_B200_ATTENTION_CSA) {
        a.selected = (const unsigned long long *)r->selected->data;
        a.selected_count = (const unsigned long long *)r->selected_count->data;
        a.topk_capacity = r->indexer_topk;
    }
    a.sinks = (const float *)r->sinks->data;
    a.query_heads = r->query_heads;
    a.head_dim = r->head_dimension;
    a.sliding_window = r->sliding_window;
    a.attention_class = (unsigned int)r->attention_class;
    a.phase_start_position = r->token_position;
    a.token_count = r->token_count;
    a.candidate_block_visible = r->candidate_block_visible;
    a.out = (float *)r->output->data;
    a.status = backend->status_device;
    if (r->rope_frequency) {
        if (r->rope_dimension < 2ull || (r->rope_dimension & 1ull) || r->rope_dimension > r->head_dimension ||
            ((r->head_dimension - r->rope_dimension) & 1ull))
            return reduce_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, r->head_dimension,
                                 r->rope_dimension, err, YVEX_ERR_INVALID_ARG,
                                 "rotated width must be even, at least 2 and leave an even unrotated width");
        if (!view_ok(backend, r->rope_frequency, YVEX_DTYPE_F64, r->rope_dimension / 2ull))
            return reduce_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, r->rope_dimension / 2ull,
                                 r->rope_frequency->bytes, err, YVEX_ERR_FORMAT,
                                 "frequency view does not cover the rotated pairs");
        a.rope_dims = r->rope_dimension;
        a.rope_frequency = (const double *)r->rope_frequency->data;
    }
    workspace = yvx_cuda_latent_reduce_workspace_bytes(&a);
    rc = yvx_backend_scratch(backend, workspace, &scratch, where, err);
    if (rc != YVEX_OK) {
        if (failure) {
            failure->code = YVEX_B200_ATTENTION_FAILURE_ALLOCATION;
            failure->stage = "reduce";
            failure->expected = workspace;
        }
        return rc;
    }
    a.workspace = scratch;
    rc = yvx_backend_status_arm(backend, where, err);
    if (rc != YVEX_OK) return rc;
    rc = yvx_cuda_latent_reduce_launches(&a, backend->stream, &launches);
    if (rc != 0) {
        if (failure) {
            failure->code = YVEX_B200_ATTENTION_FAILURE_LAUNCH;
            failure->stage = "reduce";
        }
        return yvx_backend_device_fail(backend, rc, where, err);
    }
    rc = finish(backend, facts, launches, workspace, where, err);
    if (rc != YVEX_OK) {
        if (failure) {
            failure->code = rc == YVEX_ERR_FORMAT ? YVEX_B200_ATTENTION_FAILURE_NUMERIC
                                                  : YVEX_B200_ATTENTION_FAILURE_SYNCHRONIZE;
            failure->stage = "reduce";
        }
        return rc;
    }
    r->output->is_written = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_b200_rope_frequencies(const yvex_b200_position_policy *policy,
                               unsigned long long rope_dimension, double *frequency)
{
    static const double pi = 3.14159265358979323846;
    unsigned long long pair;
    if (!policy || !frequency || rope_dimension < 2ull || policy->theta <= 1ull) return YVEX_ERR_INVALID_ARG;
    rope_dimension &= ~1ull;
    for (pair = 0; pair < rope_dimension / 2ull; ++pair) {
        double value = 1.0 / pow((double)policy->theta, (double)(pair * 2ull) / (double)rope_dimension);
        if (policy->original_context && policy->scaling_factor) {
            const double span = 2.0 * log((double)policy->theta);
            double low = floor((double)rope_dimension *
                               log((double)policy->original_context / ((double)policy->beta_fast * 2.0 * pi)) / span);
            double high = ceil((double)rope_dimension *
                               log((double)policy->original_context / ((double)policy->beta_slow * 2.0 * pi)) / span);
            double ramp, keep;
            if (low < 0.0) low = 0.0;
            if (high > (double)rope_dimension - 1.0) high = (double)rope_dimension - 1.0;
            if (low == high) high += 0.001;
            ramp = ((double)pair - low) / (high - low);
            ramp = ramp < 0.0 ? 0.0 : ramp > 1.0 ? 1.0 : ramp;
            keep = 1.0 - ramp;
            value = value / (double)policy->scaling_factor * (1.0 - keep) + value * keep;
        }
        frequency[pair] = value;
    }
    return YVEX_OK;
}

static int select_refuse(yvex_b200_attention_failure *failure, yvex_b200_attention_failure_code code,
                         unsigned long long expected, unsigned long long actual, yvex_error *err,
                         yvex_status status, const char *message)
{
    if (failure) {
        failure->code = code;
        failure->stage = "select";
        failure->expected = expected;
        failure->actual = actual;
    }
    return yvx_fail(err, status, "b200.attention.select", message);
}

int yvex_b200_attention_select_execute(yvex_backend *backend, const yvex_b200_attention_select_request *r,
                                       yvex_b200_attention_failure *failure,
                                       yvex_backend_operation_facts *facts, yvex_error *err)
{
    const char *where = "b200.attention.select";
    unsigned long long width, elements = 0ull, workspace;
    unsigned int launches = 0u;
    void *scratch = NULL;
    yvx_csa_select_args a;
    int rc;
    if (failure) memset(failure, 0, sizeof(*failure));
    if (!r || !facts || !r->index_keys || !r->positions || !r->index_query || !r->index_weights || !r->scores ||
        !r->selected || !r->selected_count)
        return select_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, 1ull, 0ull, err,
                             YVEX_ERR_INVALID_ARG, "index keys, positions, queries, weights and outputs are required");
    memset(facts, 0, sizeof(*facts));
    rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (!r->token_count || !r->count || !r->indexer_heads || !r->indexer_head_dimension || !r->indexer_topk ||
        !r->compression_ratio || r->key_stride < r->indexer_head_dimension ||
        !yvx_u64_mul(r->indexer_heads, r->indexer_head_dimension, &width))
        return select_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, r->indexer_head_dimension,
                             r->key_stride, err, YVEX_ERR_INVALID_ARG,
                             "token count, row count, heads, width, top-k, ratio and key stride must be consistent");
    if (r->indexer_heads > 64ull || r->indexer_head_dimension > 256ull || r->indexer_topk > 1024ull ||
        r->count >= (1ull << 31) || r->token_count > 65535ull)
        return select_refuse(failure, YVEX_B200_ATTENTION_FAILURE_CAPABILITY, 64ull, r->indexer_heads, err,
                             YVEX_ERR_UNSUPPORTED, "at most 64 index heads of width 256, top-k 1024");
    if (!yvx_u64_mul(r->count, r->key_stride, &elements) || !view_ok(backend, r->index_keys, YVEX_DTYPE_F32, elements) ||
        !view_ok(backend, r->positions, YVEX_DTYPE_I64, r->count) ||
        !yvx_u64_mul(r->token_count, width, &elements) || !view_ok(backend, r->index_query, YVEX_DTYPE_F32, elements) ||
        !yvx_u64_mul(r->token_count, r->indexer_heads, &elements) ||
        !view_ok(backend, r->index_weights, YVEX_DTYPE_F32, elements) ||
        !yvx_u64_mul(r->token_count, r->count, &elements) || !view_ok(backend, r->scores, YVEX_DTYPE_F32, elements) ||
        !yvx_u64_mul(r->token_count, r->indexer_topk, &elements) ||
        !view_ok(backend, r->selected, YVEX_DTYPE_I64, elements) ||
        !view_ok(backend, r->selected_count, YVEX_DTYPE_I64, r->token_count))
        return select_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, elements, 0ull, err,
                             YVEX_ERR_FORMAT, "tensor views do not cover the stated geometry");
    workspace = yvx_cuda_csa_select_workspace_bytes(r->count, r->token_count, (unsigned int)r->indexer_topk);
    rc = yvx_backend_scratch(backend, workspace, &scratch, where, err);
    if (rc != YVEX_OK) {
        if (failure) {
            failure->code = YVEX_B200_ATTENTION_FAILURE_ALLOCATION;
            failure->stage = "select";
            failure->expected = workspace;
        }
        return rc;
    }
    memset(&a, 0, sizeof(a));
    a.keys = (const float *)r->index_keys->data;
    a.positions = (const unsigned long long *)r->positions->data;
    a.rows = r->count;
    a.key_stride = r->key_stride;
    a.query = (const float *)r->index_query->data;
    a.weights = (const float *)r->index_weights->data;
    a.heads = (unsigned int)r->indexer_heads;
    a.head_dim = (unsigned int)r->indexer_head_dimension;
    a.topk = (unsigned int)r->indexer_topk;
    a.ratio = r->compression_ratio;
    a.phase_start_position = r->token_position;
    a.token_count = r->token_count;
    a.scores = (float *)r->scores->data;
    a.selected = (unsigned long long *)r->selected->data;
    a.selected_count = (unsigned long long *)r->selected_count->data;
    a.topk_capacity = r->indexer_topk;
    a.workspace = scratch;
    a.status = backend->status_device;
    rc = yvx_backend_status_arm(backend, where, err);
    if (rc != YVEX_OK) return rc;
    rc = yvx_cuda_csa_select(&a, backend->stream, &launches);
    if (rc != 0) {
        if (failure) {
            failure->code = YVEX_B200_ATTENTION_FAILURE_LAUNCH;
            failure->stage = "select";
        }
        return yvx_backend_device_fail(backend, rc, where, err);
    }
    rc = finish(backend, facts, launches, workspace, where, err);
    if (rc != YVEX_OK) {
        if (failure) {
            failure->code = rc == YVEX_ERR_FORMAT ? YVEX_B200_ATTENTION_FAILURE_NUMERIC
                                                  : YVEX_B200_ATTENTION_FAILURE_SYNCHRONIZE;
            failure->stage = "select";
        }
        return rc;
    }
    r->scores->is_written = r->selected->is_written = r->selected_count->is_written = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}

static int compress_refuse(yvex_b200_attention_failure *failure, yvex_b200_attention_failure_code code,
                           unsigned long long expected, unsigned long long actual, yvex_error *err,
                           yvex_status status, const char *message)
{
    if (failure) {
        failure->code = code;
        failure->stage = "compress";
        failure->expected = expected;
        failure->actual = actual;
    }
    return yvx_fail(err, status, "b200.attention.compress", message);
}

int yvex_b200_attention_compress_execute(yvex_backend *backend, yvex_b200_attention_compress_request *r,
                                         yvex_b200_attention_failure *failure,
                                         yvex_backend_operation_facts *facts, yvex_error *err)
{
    const char *where = "b200.attention.compress";
    unsigned long long width = 0ull, slots = 0ull, elements = 0ull, emitted, launched = 0ull;
    yvx_compressor_args a;
    unsigned int activation_launches = 0u;
    int overlap, rc, separate_activation = 0;
    if (failure) memset(failure, 0, sizeof(*failure));
    if (!r || !facts || !r->position_rows || !r->state_kv || !r->state_score || !r->next_state_kv ||
        !r->next_state_score || (r->token_count && (!r->token_kv || !r->token_score)))
        return compress_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, 1ull, 0ull, err,
                               YVEX_ERR_INVALID_ARG, "token rows, position rows and both states are required");
    r->emitted = 0ull;
    memset(facts, 0, sizeof(*facts));
    rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    /* yvex_attention_rolling_geometry: index rows exist for the sparse class only */
    if ((r->kind != YVEX_B200_ROLLING_MAIN && r->kind != YVEX_B200_ROLLING_INDEXER) ||
        (r->attention_class != YVEX_B200_ATTENTION_CSA && r->attention_class != YVEX_B200_ATTENTION_HCA) ||
        (r->kind == YVEX_B200_ROLLING_INDEXER && r->attention_class != YVEX_B200_ATTENTION_CSA))
        return compress_refuse(failure, YVEX_B200_ATTENTION_FAILURE_CAPABILITY, 1ull, 0ull, err,
                               YVEX_ERR_UNSUPPORTED, "this class keeps no rolling state of this kind");
    overlap = r->attention_class == YVEX_B200_ATTENTION_CSA;
    if (!r->compression_ratio || !r->head_dimension ||
        !yvx_u64_mul(r->head_dimension, overlap ? 2ull : 1ull, &width) ||
        !yvx_u64_mul(r->compression_ratio, overlap ? 2ull : 1ull, &slots) ||
        (r->token_count && r->token_stride < width) || r->token_position > ~0ull - r->token_count)
        return compress_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, width, r->token_stride, err,
                               YVEX_ERR_INVALID_ARG, "ratio, head dimension, token stride and position must be consistent");
    if (r->head_dimension > 1024ull || (r->head_dimension & 1ull) || (r->rope_dimension & 1ull) ||
        r->rope_dimension > r->head_dimension)
        return compress_refuse(failure, YVEX_B200_ATTENTION_FAILURE_CAPABILITY, 1024ull, r->head_dimension, err,
                               YVEX_ERR_UNSUPPORTED, "even head dimension up to 1024 and an even rotated width");
    if (r->next_state_kv->data == r->state_kv->data || r->next_state_score->data == r->state_score->data)
        return compress_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, 0ull, 1ull, err,
                               YVEX_ERR_INVALID_ARG, "the next state must not alias the current state");
    emitted = (r->token_position % r->compression_ratio + r->token_count) / r->compression_ratio;
    if (!yvx_u64_mul(slots, width, &elements) || !view_ok(backend, r->state_kv, YVEX_DTYPE_F32, elements) ||
        !view_ok(backend, r->state_score, YVEX_DTYPE_F32, elements) ||
        !view_ok(backend, r->next_state_kv, YVEX_DTYPE_F32, elements) ||
        !view_ok(backend, r->next_state_score, YVEX_DTYPE_F32, elements) ||
        !yvx_u64_mul(r->compression_ratio, width, &elements) ||
        !view_ok(backend, r->position_rows, YVEX_DTYPE_F32, elements) ||
        (r->token_count &&
         (!yvx_u64_mul(r->token_count, r->token_stride, &elements) ||
          !view_ok(backend, r->token_kv, YVEX_DTYPE_F32, elements) ||
          !view_ok(backend, r->token_score, YVEX_DTYPE_F32, elements))) ||
        (emitted &&
         (!r->compressed || !yvx_u64_mul(emitted, r->head_dimension, &elements) ||
          !view_ok(backend, r->compressed, YVEX_DTYPE_F32, elements) ||
          (r->compressed_positions && !view_ok(backend, r->compressed_positions, YVEX_DTYPE_I64, emitted)))) ||
        (r->norm_weights && !view_ok(backend, r->norm_weights, YVEX_DTYPE_F32, r->head_dimension)) ||
        (r->norm_weights && r->rope_dimension &&
         (!r->rope_frequency || !view_ok(backend, r->rope_frequency, YVEX_DTYPE_F64, r->rope_dimension / 2ull))))
        return compress_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, elements, 0ull, err,
                               YVEX_ERR_FORMAT, "tensor views do not cover the stated geometry");
    if (r->activation_quantization) {
        unsigned long long active = r->kind == YVEX_B200_ROLLING_MAIN ? r->head_dimension - r->rope_dimension
                                                                      : r->head_dimension;
        if (r->activation_quantization != 8u && r->activation_quantization != 4u)
            return compress_refuse(failure, YVEX_B200_ATTENTION_FAILURE_NUMERIC, 8ull, r->activation_quantization,
                                   err, YVEX_ERR_FORMAT, "activation quantisation is unsupported");
        if (!r->activation_block_width || r->activation_block_width > 1024ull || active % r->activation_block_width)
            return compress_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, r->activation_block_width,
                                   active, err, YVEX_ERR_BOUNDS,
                                   "activation requires exact block divisibility");
    }
    if (r->norm_weights && !(isfinite(r->rms_norm_epsilon) && r->rms_norm_epsilon > 0.0))
        return compress_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, 1ull, 0ull, err,
                               YVEX_ERR_INVALID_ARG, "the norm epsilon must be positive and finite");
    memset(&a, 0, sizeof(a));
    a.ratio = r->compression_ratio;
    a.head_dim = r->head_dimension;
    a.overlap = overlap;
    a.start_position = r->token_position;
    a.token_count = r->token_count;
    a.token_kv = r->token_count ? (const float *)r->token_kv->data : NULL;
    a.token_score = r->token_count ? (const float *)r->token_score->data : NULL;
    a.token_stride = r->token_stride;
    a.ape = (const float *)r->position_rows->data;
    a.state_kv = (const float *)r->state_kv->data;
    a.state_score = (const float *)r->state_score->data;
    a.after_kv = (float *)r->next_state_kv->data;
    a.after_score = (float *)r->next_state_score->data;
    a.compressed = emitted ? (float *)r->compressed->data : NULL;
    a.compressed_stride = r->head_dimension;
    a.positions = emitted && r->compressed_positions ? (unsigned long long *)r->compressed_positions->data : NULL;
    if (r->norm_weights) {
        a.norm_weights = (const float *)r->norm_weights->data;
        a.epsilon = r->rms_norm_epsilon;
        a.rope_dims = r->rope_dimension;
        a.rope_frequency = r->rope_dimension ? (const double *)r->rope_frequency->data : NULL;
    }
    a.status = backend->status_device;
    rc = yvx_backend_status_arm(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (r->activation_quantization && emitted) {
        /* main rows keep their rotated lanes; index rows are quantised whole
         * (src/graph/attention_execute.c:807-818). Fused into the compressor's launch where its
         * row geometry allows, else a launch of its own behind it. */
        a.activation_quantization = r->activation_quantization;
        a.activation_count = r->kind == YVEX_B200_ROLLING_MAIN ? r->head_dimension - r->rope_dimension
                                                                : r->head_dimension;
        a.activation_block_width = r->activation_block_width;
        a.activation_hadamard = r->activation_hadamard;
        if (!a.activation_count) a.activation_quantization = 0u;
    }
    rc = yvx_cuda_compressor_chunk(&a, backend->stream, &launched);
    if (rc == YVEX_ERR_UNSUPPORTED && a.activation_quantization) {
        a.activation_quantization = 0u;
        separate_activation = 1;
        rc = yvx_cuda_compressor_chunk(&a, backend->stream, &launched);
    }
    if (rc != 0) {
        if (failure) {
            failure->code = YVEX_B200_ATTENTION_FAILURE_LAUNCH;
            failure->stage = "compress";
        }
        return yvx_backend_device_fail(backend, rc, where, err);
    }
    if (separate_activation) {
        yvx_activation_args q;
        memset(&q, 0, sizeof(q));
        q.values = a.compressed;
        q.rows = emitted;
        q.row_stride = r->head_dimension;
        q.count = r->kind == YVEX_B200_ROLLING_MAIN ? r->head_dimension - r->rope_dimension : r->head_dimension;
        q.quantization = r->activation_quantization;
        q.block_width = (unsigned int)r->activation_block_width;
        q.hadamard = r->activation_hadamard;
        q.hadamard_scale = 1.0f / sqrtf((float)q.count);
        q.status = backend->status_device;
        rc = q.count ? yvx_cuda_activation_quant(&q, backend->stream) : 0;
        if (rc != 0) {
            if (failure) {
                failure->code = YVEX_B200_ATTENTION_FAILURE_LAUNCH;
                failure->stage = "compress";
            }
            return yvx_backend_device_fail(backend, rc, where, err);
        }
        activation_launches = q.count ? 1u : 0u;
    }
    rc = finish(backend, facts, 1u + activation_launches, 0ull, where, err);
    if (rc != YVEX_OK) {
        if (failure) {
            failure->code = rc == YVEX_ERR_FORMAT ? YVEX_B200_ATTENTION_FAILURE_NUMERIC
                                                  : YVEX_B200_ATTENTION_FAILURE_SYNCHRONIZE;
            failure->stage = "compress";
        }
        return rc;
    }
    r->emitted = launched;
    r->next_state_kv->is_written = r->next_state_score->is_written = 1;
    if (emitted) {
        r->compressed->is_written = 1;
        if (r->compressed_positions) r->compressed_positions->is_written = 1;
    }
    yvex_error_clear(err);
    return YVEX_OK;
}

static int activation_refuse(yvex_b200_attention_failure *failure, yvex_b200_attention_failure_code code,
                             unsigned long long expected, unsigned long long actual, yvex_error *err,
                             yvex_status status, const char *message)
{
    if (failure) {
        failure->code = code;
        failure->stage = "activation";
        failure->expected = expected;
        failure->actual = actual;
    }
    return yvx_fail(err, status, "b200.attention.activation", message);
}

int yvex_b200_attention_activation_execute(yvex_backend *backend,
                                           const yvex_b200_attention_activation_request *r,
                                           yvex_b200_attention_failure *failure,
                                           yvex_backend_operation_facts *facts, yvex_error *err)
{
    const char *where = "b200.attention.activation";
    unsigned long long elements = 0ull;
    yvx_activation_args q;
    int rc;
    if (failure) memset(failure, 0, sizeof(*failure));
    if (!r || !facts || !r->values || !r->count || !r->block_width)
        return activation_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, 1ull, 0ull, err,
                                 YVEX_ERR_INVALID_ARG, "activation requires values and a block width");
    memset(facts, 0, sizeof(*facts));
    rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (r->quantization != 8u && r->quantization != 4u)
        return activation_refuse(failure, YVEX_B200_ATTENTION_FAILURE_NUMERIC, 8ull, r->quantization, err,
                                 YVEX_ERR_FORMAT, "activation quantisation is unsupported");
    if (r->count % r->block_width)
        return activation_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, r->block_width, r->count,
                                 err, YVEX_ERR_BOUNDS, "activation requires exact block divisibility");
    if (r->count > 8192ull || r->block_width > 1024ull)
        return activation_refuse(failure, YVEX_B200_ATTENTION_FAILURE_CAPABILITY, 8192ull, r->count, err,
                                 YVEX_ERR_UNSUPPORTED, "rows of at most 8192 lanes, blocks of at most 1024");
    if (r->row_stride < r->count || !yvx_u64_mul(r->rows ? r->rows : 1ull, r->row_stride, &elements) ||
        !view_ok(backend, r->values, YVEX_DTYPE_F32, elements - (r->row_stride - r->count)))
        return activation_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, elements, r->values->bytes,
                                 err, YVEX_ERR_FORMAT, "tensor view does not cover the stated rows");
    memset(&q, 0, sizeof(q));
    q.values = (float *)r->values->data;
    q.rows = r->rows;
    q.row_stride = r->row_stride;
    q.count = r->count;
    q.quantization = r->quantization;
    q.block_width = (unsigned int)r->block_width;
    q.hadamard = r->hadamard;
    q.hadamard_scale = 1.0f / sqrtf((float)r->count);
    q.status = backend->status_device;
    rc = yvx_backend_status_arm(backend, where, err);
    if (rc != YVEX_OK) return rc;
    rc = yvx_cuda_activation_quant(&q, backend->stream);
    if (rc != 0) {
        if (failure) {
            failure->code = YVEX_B200_ATTENTION_FAILURE_LAUNCH;
            failure->stage = "activation";
        }
        return yvx_backend_device_fail(backend, rc, where, err);
    }
    rc = finish(backend, facts, r->rows ? 1u : 0u, 0ull, where, err);
    if (rc != YVEX_OK) {
        if (failure) {
            failure->code = rc == YVEX_ERR_FORMAT ? YVEX_B200_ATTENTION_FAILURE_NUMERIC
                                                  : YVEX_B200_ATTENTION_FAILURE_SYNCHRONIZE;
            failure->stage = "activation";
        }
        return rc;
    }
    r->values->is_written = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}

static int publish_refuse(yvex_b200_attention_failure *failure, yvex_b200_attention_failure_code code,
                          unsigned long long expected, unsigned long long actual, yvex_error *err,
                          yvex_status status, const char *message)
{
    if (failure) {
        failure->code = code;
        failure->stage = "publish";
        failure->expected = expected;
        failure->actual = actual;
    }
    return yvx_fail(err, status, "b200.attention.publish", message);
}

int yvex_b200_attention_publish_execute(yvex_backend *backend, const yvex_b200_attention_publish_request *r,
                                        yvex_b200_attention_failure *failure,
                                        yvex_backend_operation_facts *facts, yvex_error *err)
{
    const char *where = "b200.attention.publish";
    unsigned long long elements = 0ull;
    yvx_rows_publish_args a;
    int rc;
    if (failure) memset(failure, 0, sizeof(*failure));
    if (!r || !facts || !r->values || !r->width || !r->rows_per_token)
        return publish_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, 1ull, 0ull, err,
                              YVEX_ERR_INVALID_ARG, "publication requires rows, a width and rows per token");
    memset(facts, 0, sizeof(*facts));
    rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (r->row_stride < r->width || !yvx_u64_mul(r->rows ? r->rows : 1ull, r->row_stride, &elements) ||
        !view_ok(backend, r->values, YVEX_DTYPE_F32, elements - (r->row_stride - r->width)) ||
        (r->norm_mode == 2 && (!r->norm_weights || !view_ok(backend, r->norm_weights, YVEX_DTYPE_F32, r->width))) ||
        (r->rope_dimension &&
         (!r->rope_frequency || !view_ok(backend, r->rope_frequency, YVEX_DTYPE_F64, r->rope_dimension / 2ull))))
        return publish_refuse(failure, YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT, elements, r->values->bytes, err,
                              YVEX_ERR_FORMAT, "tensor views do not cover the stated geometry");
    memset(&a, 0, sizeof(a));
    a.values = (float *)r->values->data;
    a.rows = r->rows;
    a.rows_per_token = r->rows_per_token;
    a.row_stride = r->row_stride;
    a.width = r->width;
    a.norm_mode = r->norm_mode;
    a.norm_weights = r->norm_mode == 2 ? (const float *)r->norm_weights->data : NULL;
    a.epsilon = r->rms_norm_epsilon;
    a.rope_dims = r->rope_dimension;
    a.rope_frequency = r->rope_dimension ? (const double *)r->rope_frequency->data : NULL;
    a.start_position = r->token_position;
    a.quantization = r->activation_quantization;
    a.activation_count = r->activation_count;
    a.block_width = r->activation_block_width;
    a.hadamard = r->activation_hadamard;
    a.status = backend->status_device;
    rc = yvx_backend_status_arm(backend, where, err);
    if (rc != YVEX_OK) return rc;
    rc = yvx_cuda_rows_publish(&a, backend->stream);
    if (rc != 0) {
        /* the shim's refusals are argument refusals, not device failures */
        if (rc == YVEX_ERR_INVALID_ARG || rc == YVEX_ERR_UNSUPPORTED || rc == YVEX_ERR_BOUNDS || rc == YVEX_ERR_FORMAT)
            return publish_refuse(failure, rc == YVEX_ERR_UNSUPPORTED ? YVEX_B200_ATTENTION_FAILURE_CAPABILITY
                                                                      : YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT,
                                  0ull, 0ull, err, (yvex_status)rc, "publication chain refused its arguments");
        if (failure) {
            failure->code = YVEX_B200_ATTENTION_FAILURE_LAUNCH;
            failure->stage = "publish";
        }
        return yvx_backend_device_fail(backend, rc, where, err);
    }
    rc = finish(backend, facts, r->rows ? 1u : 0u, 0ull, where, err);
    if (rc != YVEX_OK) {
        if (failure) {
            failure->code = rc == YVEX_ERR_FORMAT ? YVEX_B200_ATTENTION_FAILURE_NUMERIC
                                                  : YVEX_B200_ATTENTION_FAILURE_SYNCHRONIZE;
            failure->stage = "publish";
        }
        return rc;
    }
    r->values->is_written = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_b200_kv_append_rotary_execute(yvex_backend *backend, const yvex_b200_kv_append_request *r,
                                       yvex_backend_operation_facts *facts, yvex_error *err)
{
    const char *where = "b200.kv.append_rotary";
    unsigned long long rows, query_width, kv_width, elements;
    yvx_kv_append_args a;
    int rc;
    if (!r || !facts || !r->key || !r->value || !r->cosines || !r->sines)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "new key and value rows and rotary tables are required");
    memset(facts, 0, sizeof(*facts));
    rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (!r->session_count || !r->token_count || !r->key_value_heads || !r->head_dimension ||
        !r->rotary_dimension || (r->rotary_dimension & 1ull) || r->rotary_dimension > r->head_dimension ||
        (r->query && !r->query_heads) || r->session_count > 65535ull || r->token_count > 0x7fffffffull ||
        !yvx_u64_mul(r->session_count, r->token_count, &rows) ||
        !yvx_u64_mul(r->query_heads, r->head_dimension, &query_width) ||
        !yvx_u64_mul(r->key_value_heads, r->head_dimension, &kv_width))
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "sessions, rows, heads and rotary width must be consistent");
    if (!r->state_values && !r->key_pool)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "a state bank or a block-table pool is required");
    if ((r->query && (!yvx_u64_mul(rows, query_width, &elements) || !view_ok(backend, r->query, YVEX_DTYPE_F32, elements))) ||
        !yvx_u64_mul(rows, kv_width, &elements) || !view_ok(backend, r->key, YVEX_DTYPE_F32, elements) ||
        !view_ok(backend, r->value, YVEX_DTYPE_F32, elements) ||
        !yvx_u64_mul(rows, r->rotary_dimension, &elements) || !view_ok(backend, r->cosines, YVEX_DTYPE_F32, elements) ||
        !view_ok(backend, r->sines, YVEX_DTYPE_F32, elements) ||
        (r->kv_tokens && !view_ok(backend, r->kv_tokens, YVEX_DTYPE_I32, r->session_count)) ||
        (r->token_position && !view_ok(backend, r->token_position, YVEX_DTYPE_I64, r->session_count)))
        return yvx_fail(err, YVEX_ERR_FORMAT, where, "packed F32 rows and explicit rotary tables are required");
    memset(&a, 0, sizeof(a));
    if (r->state_values) {
        /* the caller bounds the bank: rows [0, state_capacity) of state_row_stride floats per session */
        if (r->state_row_stride < 2ull * kv_width || !r->state_capacity ||
            !yvx_u64_mul(r->state_capacity, r->state_row_stride, &elements) ||
            !yvx_u64_mul(elements, r->session_count, &elements) ||
            !view_ok(backend, r->state_values, YVEX_DTYPE_F32, elements) ||
            (r->state_positions &&
             (!yvx_u64_mul(r->state_capacity, r->session_count, &elements) ||
              !view_ok(backend, r->state_positions, YVEX_DTYPE_I64, elements))) ||
            r->max_kv_tokens > r->state_capacity || r->token_count > r->state_capacity - r->max_kv_tokens)
            return yvx_fail(err, YVEX_ERR_BOUNDS, where, "new rows exceed the admitted state view");
        a.state_values = (float *)r->state_values->data;
        a.state_row_stride = r->state_row_stride;
        a.state_session_stride = r->state_capacity * r->state_row_stride;
        if (r->state_positions) {
            a.state_positions = (unsigned long long *)r->state_positions->data;
            a.state_position_stride = r->state_capacity;
        }
    }
    if (r->key_pool) {
        unsigned long long blocks_needed, block_elements;
        if (!r->value_pool || !r->block_table || !r->block_tokens || !r->max_blocks_per_session ||
            !yvx_u64_mul(r->block_tokens, kv_width, &block_elements) || !r->pool_blocks ||
            !yvx_u64_mul(r->pool_blocks, block_elements, &elements) ||
            !view_ok(backend, r->key_pool, YVEX_DTYPE_BF16, elements) ||
            !view_ok(backend, r->value_pool, YVEX_DTYPE_BF16, elements) ||
            !yvx_u64_mul(r->session_count, r->max_blocks_per_session, &elements) ||
            !view_ok(backend, r->block_table, YVEX_DTYPE_I32, elements))
            return yvx_fail(err, YVEX_ERR_FORMAT, where, "bf16 pools and an int32 block table are required");
        blocks_needed = (r->max_kv_tokens + r->token_count + r->block_tokens - 1ull) / r->block_tokens;
        if (blocks_needed > r->max_blocks_per_session)
            return yvx_fail(err, YVEX_ERR_BOUNDS, where, "new rows exceed the block table");
        a.key_pool = r->key_pool->data;
        a.value_pool = r->value_pool->data;
        a.block_table = (const int *)r->block_table->data;
        a.block_tokens = (unsigned int)r->block_tokens;
        a.block_table_stride = (unsigned int)r->max_blocks_per_session;
        a.pool_blocks = (unsigned int)r->pool_blocks;
        a.pool_token_stride = kv_width;
        a.pool_head_stride = r->head_dimension;
        a.pool_block_stride = block_elements;
    }
    a.sessions = (unsigned int)r->session_count;
    a.tokens = (unsigned int)r->token_count;
    a.query_heads = (unsigned int)r->query_heads;
    a.kv_heads = (unsigned int)r->key_value_heads;
    a.head_dim = (unsigned int)r->head_dimension;
    a.rotary_dim = (unsigned int)r->rotary_dimension;
    a.staged_bf16 = r->bf16_staged_products;
    a.query = r->query ? (float *)r->query->data : NULL;
    a.key = (const float *)r->key->data;
    a.value = (const float *)r->value->data;
    a.cosines = (const float *)r->cosines->data;
    a.sines = (const float *)r->sines->data;
    a.kv_tokens = r->kv_tokens ? (const int *)r->kv_tokens->data : NULL;
    a.kv_tokens_uniform = (unsigned int)r->max_kv_tokens;
    a.token_position = r->token_position ? (const unsigned long long *)r->token_position->data : NULL;
    a.status = backend->status_device;
    if (r->state_values)
        a.row_capacity = r->state_capacity > 0xffffffffull ? 0xffffffffu : (unsigned int)r->state_capacity;
    rc = yvx_backend_status_arm(backend, where, err);
    if (rc != YVEX_OK) return rc;
    rc = yvx_cuda_kv_append_rotary(&a, backend->stream);
    if (rc != 0) return yvx_backend_device_fail(backend, rc, where, err);
    facts->d2d_bytes = rows * 2ull * kv_width * (r->state_values ? 4ull : 0ull) +
                       rows * 2ull * kv_width * (r->key_pool ? 2ull : 0ull);
    rc = finish(backend, facts, 1u, 0ull, where, err);
    if (rc != YVEX_OK) return rc;
    if (r->query) r->query->is_written = 1;
    if (r->state_values) r->state_values->is_written = 1;
    if (r->state_positions) r->state_positions->is_written = 1;
    if (r->key_pool) r->key_pool->is_written = r->value_pool->is_written = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_b200_mla_decode_execute(yvex_backend *backend, const yvex_b200_mla_decode_request *r,
                                 yvex_backend_operation_facts *facts, yvex_error *err)
{
    const char *where = "b200.attention.mla_decode";
    unsigned long long items, elements, absorbed, partials;
    yvx_mla_problem p;
    unsigned int launches = 0;
    void *scratch = NULL;
    int rc;
    if (!r || !facts || !r->q_nope || !r->q_rope || !r->w_uk || !r->latent || !r->rope_key || !r->output)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "queries, up-projection, caches and output are required");
    memset(facts, 0, sizeof(*facts));
    rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (!r->session_count || !r->context_capacity || !r->max_kv_tokens || r->max_kv_tokens > r->context_capacity ||
        r->session_count > 65535ull || r->context_capacity > 0x7fffffffull || !(r->scale > 0.0f) || !isfinite(r->scale))
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "sessions, context and a positive finite scale are required");
    if (r->heads != 128ull || r->nope_dimension != 128ull || r->latent_dimension != 512ull || r->rope_dimension != 64ull)
        return yvx_fail(err, YVEX_ERR_UNSUPPORTED, where, "128 heads, 128 nope, 512 latent and 64 rope dims are supported");
    items = r->session_count * r->heads;
    if (!view_ok(backend, r->q_nope, YVEX_DTYPE_BF16, items * r->nope_dimension) ||
        !view_ok(backend, r->q_rope, YVEX_DTYPE_BF16, items * r->rope_dimension) ||
        !view_ok(backend, r->w_uk, YVEX_DTYPE_BF16, r->heads * r->nope_dimension * r->latent_dimension) ||
        !yvx_u64_mul(r->session_count * r->context_capacity, r->latent_dimension, &elements) ||
        !view_ok(backend, r->latent, YVEX_DTYPE_BF16, elements) ||
        !view_ok(backend, r->rope_key, YVEX_DTYPE_BF16, r->session_count * r->context_capacity * r->rope_dimension) ||
        !view_ok(backend, r->output, YVEX_DTYPE_F32, items * r->latent_dimension) ||
        (r->kv_tokens && !view_ok(backend, r->kv_tokens, YVEX_DTYPE_I32, r->session_count)))
        return yvx_fail(err, YVEX_ERR_FORMAT, where, "bf16 queries and caches, F32 output and I32 lengths are required");
    memset(&p, 0, sizeof(p));
    p.sessions = (unsigned int)r->session_count;
    p.heads = 128u;
    p.nope_dim = 128u;
    p.latent_dim = 512u;
    p.rope_dim = 64u;
    p.scale = r->scale;
    p.q_nope = r->q_nope->data;
    p.q_rope = r->q_rope->data;
    p.w_uk = r->w_uk->data;
    p.latent = r->latent->data;
    p.rope_key = r->rope_key->data;
    p.latent_session_stride = r->context_capacity * r->latent_dimension;
    p.rope_session_stride = r->context_capacity * r->rope_dimension;
    p.kv_tokens = r->kv_tokens ? (const unsigned int *)r->kv_tokens->data : NULL;
    p.kv_tokens_uniform = (unsigned int)r->max_kv_tokens;
    p.kv_tokens_max = (unsigned int)r->max_kv_tokens;
    yvx_cuda_mla_plan(&p, backend->sm_count);
    absorbed = (yvx_cuda_mla_absorbed_bytes(&p) + 255ull) & ~255ull;
    partials = yvx_cuda_mla_partials_bytes(&p);
    rc = yvx_backend_scratch(backend, absorbed + partials, &scratch, where, err);
    if (rc != YVEX_OK) return rc;
    p.q_absorbed = scratch;
    p.partials = (float *)((unsigned char *)scratch + absorbed);
    p.output = (float *)r->output->data;
    p.status = backend->status_device;
    rc = yvx_backend_status_arm(backend, where, err);
    if (rc != YVEX_OK) return rc;
    rc = yvx_cuda_mla_decode(&p, backend->stream, NULL, &launches);
    if (rc != 0) return yvx_backend_device_fail(backend, rc, where, err);
    rc = finish(backend, facts, launches, absorbed + partials, where, err);
    if (rc != YVEX_OK) return rc;
    r->output->is_written = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}
