/* TEST INFRASTRUCTURE ONLY.
 *
 * Flat C entry points over the YVEX reference's own CPU code, compiled
 * together with the reference's sources into oracle/_ref/libyvex_ref.so (see
 * the Makefile beside this file). The bridge contains no arithmetic of its
 * own: every number comes out of the reference's public functions
 * (yvex_backend_op_attention on its CPU backend, the gguf scalar and Q8_0
 * codecs). It validates the restatement in yvx_oracle.c and serves as the
 * "reference" CPU baseline of the benchmark.
 */
#ifndef _GNU_SOURCE
#define _GNU_SOURCE
#endif
#include <yvex/backend.h>
#include <yvex/core.h>
#include <yvex/internal/quant_numeric.h>
#include <yvex/qtype.h>

#include <pthread.h>
#include <stdlib.h>
#include <string.h>

float yvx_ref_bf16_decode(unsigned short bits) { return yvex_quant_bf16_decode(bits); }
unsigned short yvx_ref_bf16_encode(float value) { return yvex_quant_bf16_encode(value); }
float yvx_ref_f16_decode(unsigned short bits) { return yvex_quant_f16_decode(bits); }
unsigned short yvx_ref_f16_encode(float value) { return yvex_quant_f16_encode(value); }

int yvx_ref_q8_0_encode_block(const float *source, unsigned char *encoded)
{
    yvex_error err;
    size_t written = 0;
    return yvex_quant_encode_block(YVEX_GGUF_QTYPE_Q8_0, source, 32ull, encoded, 34u,
                                   &written, NULL, &err) == YVEX_OK &&
           written == 34u;
}

int yvx_ref_q8_0_decode_block(const unsigned char *encoded, float *out)
{
    yvex_error err;
    return yvex_quant_decode_block(YVEX_GGUF_QTYPE_Q8_0, encoded, 34u, out, 32ull,
                                   NULL, &err) == YVEX_OK;
}

typedef struct {
    yvex_backend *backend;
    yvex_device_tensor *query, *keys, *values, *scores, *probabilities, *out;
    unsigned long long seq, hd;
} ref_head_tensors;

static int ref_tensor(yvex_backend *backend, const char *name, unsigned int rank,
                      unsigned long long d0, unsigned long long d1,
                      yvex_device_tensor **out)
{
    yvex_backend_tensor_desc desc;
    yvex_error err;
    memset(&desc, 0, sizeof(desc));
    desc.name = name;
    desc.dtype = YVEX_DTYPE_F32;
    desc.rank = rank;
    desc.dims[0] = d0;
    desc.dims[1] = d1;
    desc.bytes = d0 * (rank > 1 ? d1 : 1ull) * sizeof(float);
    return yvex_backend_tensor_alloc(backend, &desc, out, &err) == YVEX_OK;
}

static void ref_head_release(ref_head_tensors *t)
{
    if (!t->backend) return;
    yvex_backend_tensor_free(t->backend, t->query);
    yvex_backend_tensor_free(t->backend, t->keys);
    yvex_backend_tensor_free(t->backend, t->values);
    yvex_backend_tensor_free(t->backend, t->scores);
    yvex_backend_tensor_free(t->backend, t->probabilities);
    yvex_backend_tensor_free(t->backend, t->out);
    yvex_backend_close(t->backend);
    memset(t, 0, sizeof(*t));
}

static int ref_head_prepare(ref_head_tensors *t, unsigned long long seq,
                            unsigned long long hd)
{
    yvex_error err;
    memset(t, 0, sizeof(*t));
    t->seq = seq;
    t->hd = hd;
    if (yvex_backend_open_cpu(&t->backend, &err) != YVEX_OK) return 0;
    if (ref_tensor(t->backend, "q", 1, hd, 0, &t->query) &&
        ref_tensor(t->backend, "k", 2, seq, hd, &t->keys) &&
        ref_tensor(t->backend, "v", 2, seq, hd, &t->values) &&
        ref_tensor(t->backend, "s", 1, seq, 0, &t->scores) &&
        ref_tensor(t->backend, "p", 1, seq, 0, &t->probabilities) &&
        ref_tensor(t->backend, "o", 1, hd, 0, &t->out))
        return 1;
    ref_head_release(t);
    return 0;
}

/* One head, one query vector, through yvex_backend_op_attention on the
 * reference's CPU backend. Returns the reference's status code. */
int yvx_ref_op_attention(const float *query, const float *keys, const float *values,
                         unsigned long long seq_len, unsigned long long position,
                         float scale, int causal, unsigned long long head_dim,
                         float *score_scratch, float *probability_scratch, float *out)
{
    ref_head_tensors t;
    yvex_error err;
    int rc;
    if (!ref_head_prepare(&t, seq_len, head_dim)) return YVEX_ERR_NOMEM;
    rc = yvex_backend_tensor_write(t.backend, t.query, query, head_dim * 4ull, &err);
    if (rc == YVEX_OK)
        rc = yvex_backend_tensor_write(t.backend, t.keys, keys, seq_len * head_dim * 4ull, &err);
    if (rc == YVEX_OK)
        rc = yvex_backend_tensor_write(t.backend, t.values, values, seq_len * head_dim * 4ull, &err);
    if (rc == YVEX_OK)
        rc = yvex_backend_op_attention(t.backend, t.query, t.keys, t.values, seq_len,
                                       position, scale, causal, t.scores,
                                       t.probabilities, t.out, &err);
    if (rc == YVEX_OK) {
        yvex_backend_tensor_read(t.backend, t.out, out, head_dim * 4ull, &err);
        if (score_scratch)
            yvex_backend_tensor_read(t.backend, t.scores, score_scratch, seq_len * 4ull, &err);
        if (probability_scratch)
            yvex_backend_tensor_read(t.backend, t.probabilities, probability_scratch,
                                     seq_len * 4ull, &err);
    }
    ref_head_release(&t);
    return rc;
}

typedef struct {
    const float *query, *key, *value;
    float *output;
    unsigned long long query_tokens, key_value_tokens, query_start;
    unsigned long long query_heads, key_value_heads, head_dimension;
    unsigned long long query_stride, key_stride, value_stride;
    float scale;
    int causal;
    unsigned int worker, workers;
    int status;
} ref_gqa_job;

static void *ref_gqa_worker(void *argument)
{
    ref_gqa_job *job = (ref_gqa_job *)argument;
    const unsigned long long hd = job->head_dimension, seq = job->key_value_tokens;
    const unsigned long long group = job->query_heads / job->key_value_heads;
    const unsigned long long items = job->key_value_heads * job->query_tokens * group;
    float *packed = malloc((size_t)(seq * hd) * sizeof(float));
    unsigned long long gathered_head = ~0ull, item, row;
    ref_head_tensors t;
    yvex_error err;
    job->status = YVEX_OK;
    if (!packed || !ref_head_prepare(&t, seq, hd)) {
        free(packed);
        job->status = YVEX_ERR_NOMEM;
        return NULL;
    }
    for (item = job->worker; item < items; item += job->workers) {
        unsigned long long kv_head = item / (job->query_tokens * group);
        unsigned long long rest = item % (job->query_tokens * group);
        unsigned long long token = rest / group;
        unsigned long long query_head = kv_head * group + rest % group;
        int rc;
        if (kv_head != gathered_head) {
            for (row = 0; row < seq; ++row)
                memcpy(packed + row * hd, job->key + row * job->key_stride + kv_head * hd,
                       (size_t)hd * sizeof(float));
            yvex_backend_tensor_write(t.backend, t.keys, packed, seq * hd * 4ull, &err);
            for (row = 0; row < seq; ++row)
                memcpy(packed + row * hd, job->value + row * job->value_stride + kv_head * hd,
                       (size_t)hd * sizeof(float));
            yvex_backend_tensor_write(t.backend, t.values, packed, seq * hd * 4ull, &err);
            gathered_head = kv_head;
        }
        yvex_backend_tensor_write(t.backend, t.query,
                                  job->query + token * job->query_stride + query_head * hd,
                                  hd * 4ull, &err);
        rc = yvex_backend_op_attention(
            t.backend, t.query, t.keys, t.values, seq,
            job->causal ? job->query_start + token : 0ull, job->scale, job->causal,
            t.scores, t.probabilities, t.out, &err);
        if (rc != YVEX_OK) {
            job->status = rc;
            break;
        }
        yvex_backend_tensor_read(t.backend, t.out,
                                 job->output + (token * job->query_heads + query_head) * hd,
                                 hd * 4ull, &err);
    }
    ref_head_release(&t);
    free(packed);
    return NULL;
}

/* Grouped-query attention as a loop of the reference primitive; argument
 * meaning matches yvx_oracle_gqa_attention. */
int yvx_ref_gqa_attention(const float *query, const float *key, const float *value,
                          float *output, unsigned long long query_tokens,
                          unsigned long long key_value_tokens,
                          unsigned long long query_start,
                          unsigned long long query_heads,
                          unsigned long long key_value_heads,
                          unsigned long long head_dimension,
                          unsigned long long query_stride,
                          unsigned long long key_stride,
                          unsigned long long value_stride, float scale, int causal,
                          unsigned int threads)
{
    enum { MAX_THREADS = 256 };
    pthread_t handles[MAX_THREADS];
    ref_gqa_job jobs[MAX_THREADS];
    int created[MAX_THREADS];
    unsigned int t;
    int status = YVEX_OK;
    if (!threads) threads = 1;
    if (threads > MAX_THREADS) threads = MAX_THREADS;
    for (t = 0; t < threads; ++t) {
        ref_gqa_job *job = &jobs[t];
        job->query = query;
        job->key = key;
        job->value = value;
        job->output = output;
        job->query_tokens = query_tokens;
        job->key_value_tokens = key_value_tokens;
        job->query_start = query_start;
        job->query_heads = query_heads;
        job->key_value_heads = key_value_heads;
        job->head_dimension = head_dimension;
        job->query_stride = query_stride ? query_stride : query_heads * head_dimension;
        job->key_stride = key_stride ? key_stride : key_value_heads * head_dimension;
        job->value_stride = value_stride ? value_stride : key_value_heads * head_dimension;
        job->scale = scale;
        job->causal = causal;
        job->worker = t;
        job->workers = threads;
        job->status = YVEX_OK;
        created[t] = threads > 1 &&
                     pthread_create(&handles[t], NULL, ref_gqa_worker, job) == 0;
        if (!created[t]) ref_gqa_worker(job);
    }
    for (t = 0; t < threads; ++t)
        if (created[t]) pthread_join(handles[t], NULL);
    for (t = 0; t < threads; ++t)
        if (jobs[t].status != YVEX_OK) status = jobs[t].status;
    return status;
}

/* ---- graph-level latent attention: reduce, index selection, top-k, rotation ----
 * Flat entry points over the reference's CPU functions in src/graph/core.c,
 * attention.c and numeric.c. The structs come from the checker's header so one
 * set of Python structures serves both libraries; every number is computed by
 * the reference. */
/* the header the reference's own focused tests include for these functions */
#include <src/graph/private.h>
#include "yvx_oracle.h"

static void ref_position(const yvx_oracle_position_policy *policy, unsigned long long rope_dims,
                         yvex_attention_position_policy *out)
{
    memset(out, 0, sizeof(*out));
    out->rope_dimension = rope_dims;
    out->theta = policy->theta;
    out->scaling_factor = policy->scaling_factor;
    out->original_context = policy->original_context;
    out->beta_fast = policy->beta_fast;
    out->beta_slow = policy->beta_slow;
    out->partial_rope = 1;
    out->inverse_output_rotation = 1;
}

int yvx_ref_rope_apply(float *values, unsigned long long count, unsigned long long rope_dims,
                       unsigned long long token_position,
                       const yvx_oracle_position_policy *policy, int inverse)
{
    yvex_attention_position_policy position;
    ref_position(policy, rope_dims, &position);
    return yvex_attention_rope_apply(values, count, rope_dims, token_position, &position, inverse);
}

int yvx_ref_topk_select(const float *scores, const unsigned long long *ordinals,
                        unsigned long long count, unsigned long long k,
                        unsigned long long *selected, unsigned long long *selected_count)
{
    yvex_attention_scratch_budget scratch;
    yvex_attention_failure failure;
    yvex_error err;
    memset(&scratch, 0, sizeof(scratch));
    memset(&failure, 0, sizeof(failure));
    return yvex_attention_topk_select(scores, ordinals, count, k, selected, selected_count,
                                      &scratch, &failure, &err) == YVEX_OK;
}

static void ref_indexer_layer(const yvx_oracle_indexer *indexer, yvex_attention_layer_plan *layer,
                              yvex_attention_history_view *history)
{
    layer->attention_class = YVEX_ATTENTION_CLASS_CSA;
    layer->compression_ratio = indexer->ratio;
    layer->indexer_required = 1;
    layer->indexer_heads = indexer->heads;
    layer->indexer_head_dimension = indexer->head_dim;
    layer->indexer_topk = indexer->topk;
    layer->sparse_topk.required = 1;
    layer->sparse_topk.k = indexer->topk;
    history->indexer_entry_count = indexer->rows;
    history->indexer_kv = indexer->keys;
    history->indexer_kv_stride = indexer->key_stride;
    history->indexer_positions = indexer->positions;
}

int yvx_ref_csa_select(const yvx_oracle_indexer *indexer, unsigned long long token,
                       unsigned long long query_position, unsigned long long *selected,
                       unsigned long long *selected_count, unsigned long long *valid_count)
{
    yvex_attention_layer_plan layer;
    yvex_attention_history_view history;
    yvex_attention_scratch_budget scratch;
    yvex_attention_failure failure;
    yvex_error err;
    memset(&layer, 0, sizeof(layer));
    memset(&history, 0, sizeof(history));
    memset(&scratch, 0, sizeof(scratch));
    memset(&failure, 0, sizeof(failure));
    ref_indexer_layer(indexer, &layer, &history);
    return yvex_attention_csa_select(&layer, &history, NULL, 0ull, 0ull, NULL,
                                     indexer->query + token * indexer->heads * indexer->head_dim,
                                     indexer->weights + token * indexer->heads, query_position,
                                     selected, selected_count, valid_count, &scratch, &failure,
                                     &err) == YVEX_OK;
}

/* The whole CPU reduce of a phase: selection (class 1), both passes, the bf16
 * publication, the inverse output rotation and the second publication. Every
 * row is handed over as history except the phase's own local rows.
 * trace_counts / trace_positions (class 1, may be NULL): per token the number of
 * selected rows and their positions in ranked order, [token][indexer->topk]. */
int yvx_ref_latent_reduce_chunk(const yvx_oracle_latent_args *a,
                                unsigned long long compressed_rows,
                                const yvx_oracle_position_policy *policy,
                                const yvx_oracle_indexer *indexer, float *out,
                                unsigned long long *trace_counts,
                                unsigned long long *trace_positions)
{
    yvex_attention_layer_plan layer;
    yvex_attention_history_view history;
    yvex_attention_scratch_budget scratch;
    yvex_attention_failure failure;
    yvex_attention_cpu_result result;
    yvex_error err;
    memset(&layer, 0, sizeof(layer));
    memset(&history, 0, sizeof(history));
    memset(&scratch, 0, sizeof(scratch));
    memset(&failure, 0, sizeof(failure));
    memset(&result, 0, sizeof(result));
    if (a->attention_class == 1u) {
        if (!indexer || indexer->rows != compressed_rows) return 0;
        ref_indexer_layer(indexer, &layer, &history);
    }
    layer.attention_class = a->attention_class == 0u   ? YVEX_ATTENTION_CLASS_SWA
                            : a->attention_class == 1u ? YVEX_ATTENTION_CLASS_CSA
                                                       : YVEX_ATTENTION_CLASS_HCA;
    layer.compression_ratio = a->ratio;
    layer.sliding_window = a->sliding_window;
    layer.query_heads = a->query_heads;
    layer.kv_heads = 1ull;
    layer.head_dimension = a->head_dim;
    layer.rope_head_dimension = a->rope_dims;
    layer.compute_contract = YVEX_ATTENTION_COMPUTE_BF16_F32_RNE_V1;
    ref_position(policy, a->rope_dims, &layer.position);
    history.local_tail_count = a->initial_local_count;
    history.local_kv = a->local;
    history.local_kv_stride = a->local_stride;
    history.local_positions = a->local_positions;
    history.compressed_entry_count = a->attention_class ? compressed_rows : 0ull;
    history.compressed_kv = a->compressed;
    history.compressed_kv_stride = a->compressed_stride;
    history.compressed_positions = a->compressed_positions;
    history.immutable = 1;
    return yvex_attention_reduce_chunk(
               &layer, a->query, &history, a->local + a->initial_local_count * a->local_stride,
               a->local_stride, NULL, 0ull, 0ull, NULL, NULL, 0ull, 0ull, NULL,
               indexer ? indexer->query : NULL, indexer ? indexer->heads * indexer->head_dim : 0ull,
               indexer ? indexer->weights : NULL, indexer ? indexer->heads : 0ull, a->sinks,
               a->token_count, a->phase_start_position, out, a->candidate_block_visible,
               trace_counts, trace_positions, indexer ? indexer->topk : 0ull, &scratch, &result,
               &failure, &err) == YVEX_OK;
}

/* The reference's rolling compressor over a chunk of tokens: its own state
 * transition once per token, and on each emission the publication chain of its
 * chunk executor (round, RMS norm, round, rotation, round), each step the
 * reference's own function. kind: 1 the main rows, 2 the index rows. */
int yvx_ref_compressor_chunk(const yvx_oracle_compressor_args *a, unsigned int kind,
                             const yvx_oracle_position_policy *policy,
                             unsigned long long *emitted)
{
    yvex_attention_layer_plan layer;
    yvex_attention_rolling_state_view current;
    yvex_attention_rolling_state_output after;
    yvex_attention_failure failure;
    yvex_error err;
    unsigned long long width = a->head_dim * (a->overlap ? 2ull : 1ull);
    unsigned long long slots = a->ratio * (a->overlap ? 2ull : 1ull);
    unsigned long long extent = width * slots, token, count = 0;
    float *bank[2] = {NULL, NULL}, *scratch_row = NULL;
    int ok = 0, which = 0;
    if (emitted) *emitted = 0;
    memset(&layer, 0, sizeof(layer));
    memset(&current, 0, sizeof(current));
    memset(&failure, 0, sizeof(failure));
    layer.attention_class = (kind == 2u || a->overlap) ? YVEX_ATTENTION_CLASS_CSA
                                                       : YVEX_ATTENTION_CLASS_HCA;
    layer.compression_ratio = a->ratio;
    layer.head_dimension = kind == 1u ? a->head_dim : 4ull * a->head_dim;
    layer.indexer_head_dimension = kind == 2u ? a->head_dim : 0ull;
    layer.rope_head_dimension = a->rope_dims;
    layer.rms_norm_epsilon = a->epsilon;
    layer.compute_contract = YVEX_ATTENTION_COMPUTE_BF16_F32_RNE_V1;
    if (policy) ref_position(policy, a->rope_dims, &layer.position);
    bank[0] = malloc((size_t)extent * 2u * sizeof(float));
    bank[1] = malloc((size_t)extent * 2u * sizeof(float));
    scratch_row = malloc((size_t)a->head_dim * sizeof(float));
    if (!bank[0] || !bank[1] || !scratch_row) goto done;
    memcpy(bank[0], a->state_kv, (size_t)extent * sizeof(float));
    memcpy(bank[0] + extent, a->state_score, (size_t)extent * sizeof(float));
    current.present = 1;
    current.schema_version = YVEX_ATTENTION_ROLLING_STATE_SCHEMA_V1;
    current.kind = kind == 1u ? YVEX_ATTENTION_ROLLING_MAIN : YVEX_ATTENTION_ROLLING_INDEXER;
    current.attention_class = layer.attention_class;
    current.next_token_position = a->start_position;
    current.ratio = a->ratio;
    current.head_dimension = a->head_dim;
    current.state_width = width;
    current.state_slots = slots;
    current.cursor = current.current_fill = a->start_position % a->ratio;
    current.previous_fill = a->overlap && a->start_position >= a->ratio ? a->ratio : 0ull;
    current.kv_state_stride = current.score_state_stride = width;
    current.kv_state_extent = current.score_state_extent = extent;
    current.kv_state = bank[0];
    current.score_state = bank[0] + extent;
    current.overlap = a->overlap;
    current.rotated = kind == 2u;
    for (token = 0; token < a->token_count; ++token) {
        unsigned long long position = a->start_position + token;
        float *out = a->compressed ? a->compressed + count * a->compressed_stride : scratch_row;
        int emitted_now = 0;
        memset(&after, 0, sizeof(after));
        after.kv_state = bank[which ^ 1];
        after.score_state = bank[which ^ 1] + extent;
        after.kv_state_stride = after.score_state_stride = width;
        after.kv_state_extent = after.score_state_extent = extent;
        if (yvex_attention_rolling_state_step_cpu(
                &layer, &current, a->token_kv + token * a->token_stride,
                a->token_score + token * a->token_stride, a->ape + (position % a->ratio) * width,
                &after, out, a->head_dim, &emitted_now, &failure, &err) != YVEX_OK)
            goto done;
        if (emitted_now) {
            if (a->norm_weights) {
                if (!yvex_attention_compute_round(layer.compute_contract, out, a->head_dim) ||
                    !yvex_attention_rms_norm(out, a->head_dim, a->norm_weights, a->epsilon) ||
                    !yvex_attention_compute_round(layer.compute_contract, out, a->head_dim))
                    goto done;
                if (a->rope_dims &&
                    (!yvex_attention_rope_apply(out, a->head_dim, a->rope_dims,
                                                position + 1ull - a->ratio, &layer.position, 0) ||
                     !yvex_attention_compute_round(layer.compute_contract, out, a->head_dim)))
                    goto done;
            }
            if (a->positions) a->positions[count] = position + 1ull - a->ratio;
            ++count;
        }
        memcpy(&current, &after, sizeof(current));
        which ^= 1;
    }
    memcpy(a->after_kv, bank[which], (size_t)extent * sizeof(float));
    memcpy(a->after_score, bank[which] + extent, (size_t)extent * sizeof(float));
    if (emitted) *emitted = count;
    ok = 1;
done:
    free(bank[0]);
    free(bank[1]);
    free(scratch_row);
    return ok;
}

/* The reference's activation fake quantisation of one row in place (its policy record
 * filled as the model family fills it: final-dimension blocks, 8-bit exponent scales). */
int yvx_ref_activation_quant(float *values, unsigned long long count, unsigned int quantization,
                             unsigned long long block_width, int hadamard)
{
    yvex_attention_activation_policy policy;
    yvex_attention_scratch_budget scratch;
    yvex_attention_failure failure;
    yvex_error err;
    memset(&policy, 0, sizeof(policy));
    memset(&scratch, 0, sizeof(scratch));
    memset(&failure, 0, sizeof(failure));
    policy.required = 1;
    policy.quantization = quantization == 8u ? YVEX_ATTENTION_QUANT_FP8_E4M3_UE8M0_FAKE_DEQUANT
                                             : YVEX_ATTENTION_QUANT_FP4_E2M1_UE8M0_FAKE_DEQUANT;
    policy.block_axis = YVEX_ATTENTION_AXIS_FINAL_DIMENSION;
    policy.block_width = block_width;
    policy.scale_format = YVEX_ATTENTION_SCALE_UE8M0;
    policy.pre_transform = hadamard ? YVEX_ATTENTION_TRANSFORM_DAO_FHT_V1_1_0_POST2
                                    : YVEX_ATTENTION_TRANSFORM_NONE;
    policy.fake_quant_inplace = 1;
    return yvex_attention_activation_apply(&policy, values, count, 0ull, YVEX_TENSOR_ROLE_UNKNOWN,
                                           &scratch, &failure, &err) == YVEX_OK;
}

/* The reference's publication chain of projected rows, step by step with its own
 * functions, in the order its chunk executor applies them. */
int yvx_ref_rows_publish(const yvx_oracle_publish_args *a, const yvx_oracle_position_policy *policy)
{
    yvex_attention_position_policy position;
    unsigned long long r;
    if (policy) ref_position(policy, a->rope_dims, &position);
    for (r = 0; r < a->rows; ++r) {
        float *row = a->values + r * a->row_stride;
        if (a->norm_mode) {
            int ok = a->norm_mode == 2 ? yvex_attention_rms_norm(row, a->width, a->norm_weights, a->epsilon)
                                       : yvex_attention_unit_rms_norm(row, a->width, a->epsilon);
            if (!ok || !yvex_attention_compute_round(YVEX_ATTENTION_COMPUTE_BF16_F32_RNE_V1, row, a->width))
                return 0;
        }
        if (a->rope_dims &&
            (!policy ||
             !yvex_attention_rope_apply(row, a->width, a->rope_dims, a->start_position + r / a->rows_per_token,
                                        &position, 0) ||
             !yvex_attention_compute_round(YVEX_ATTENTION_COMPUTE_BF16_F32_RNE_V1, row, a->width)))
            return 0;
        if (a->quantization && a->activation_count &&
            !yvx_ref_activation_quant(row, a->activation_count, a->quantization, a->block_width, a->hadamard))
            return 0;
    }
    return 1;
}

/* The reference's own encoded-row dot and decode (src/gguf/quant_compute.c:116-181,
 * src/gguf/quant_block.c:780-832) for one row of `width` lanes. */
int yvx_ref_qtype_dot(unsigned int qtype, const unsigned char *encoded, unsigned long long row_bytes,
                      const float *vector, unsigned long long width, float *out)
{
    yvex_quant_failure failure;
    yvex_error err;
    return yvex_quant_cpu_dot(qtype, encoded, (size_t)row_bytes, vector, width, out, &failure, &err) == YVEX_OK;
}

int yvx_ref_qtype_decode_row(unsigned int qtype, const unsigned char *encoded, unsigned long long width,
                             float *out)
{
    const yvex_gguf_qtype_geometry *geometry = yvex_gguf_qtype_geometry_find(qtype);
    unsigned long long block, blocks;
    if (!geometry || !geometry->block_size || width % geometry->block_size) return 0;
    blocks = width / geometry->block_size;
    for (block = 0; block < blocks; ++block) {
        yvex_quant_failure failure;
        yvex_error err;
        if (yvex_quant_decode_block(qtype, encoded + block * geometry->bytes_per_block,
                                    geometry->bytes_per_block, out + block * geometry->block_size,
                                    geometry->block_size, &failure, &err) != YVEX_OK)
            return 0;
    }
    return 1;
}
