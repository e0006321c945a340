/* The encoded (latent) attention job: yvex_backend_attention_execute and
 * yvex_backend_attention_complete under the reference's names and job schema 3
 * (include/yvex/internal/backend.h:94-198), the entry point its graph layer calls once per
 * phase (src/graph/attention_execute.c:1632).
 *
 * Replaces src/backend/cuda/attention.c:776-1990. The reference runs five kernel stages
 * (:1484): envelope_pre, project (:1162-1236), compress (:1237-1385, one launch chain per
 * token), reduce with the output projections (:1386-1452) and envelope_post, inside a
 * transaction of five phases (:1918-1923) with a cancellation poll between them. Here the
 * same stages run over the whole phase at once:
 *
 *   project   input bf16 publication, q_a, weighted norm, q_b, kv, kv norm, unit norm of
 *             the query heads, rotation of queries and new local rows, activation of the
 *             local rows, sinks            -> 3 projections + 1 batched publication launch
 *   compress  compressor projections for every token, the rolling compressor of the whole
 *             chunk (main rows; index rows for the sparse class), index queries and
 *             weights, ranked top-k        -> yvx_cuda_compressor_chunk, yvx_cuda_csa_select
 *   reduce    shared-latent reduce with the inverse rotation fused, grouped out_a, out_b
 *
 * Numerics follow the CPU twin (src/graph/attention_execute.c:452-1122, src/graph/core.c:
 * 608-829, 1107-1215), which the reference itself compares its device path against.
 *
 * What is refused, with the reference's typed failure: the residual-mixing envelope
 * (operation_scope ENVELOPE: FAILURE_CAPABILITY at "cuda.attention.mhc_pre"), weight
 * encodings other than F32 / F16 / BF16 / Q8_0 (FAILURE_CAPABILITY at the weight's stage),
 * deferred completion and retained prefix checkpoints (FAILURE_CAPABILITY).
 * There is no host fallback for any of them. */
#include "private.h"

#include "yvex_b200/attention_job.h"

#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { JOB_BUFFERS = 64 };

typedef struct {
    void **target;
    unsigned long long bytes;
} job_buffer;

typedef struct {
    yvex_backend *backend;
    const yvex_backend_attention_job *job;
    yvex_backend_attention_output *out;
    yvex_backend_attention_failure *failure;
    yvex_error *err;
    int work_pending;
    /* geometry */
    unsigned long long tokens, query_width, low_width, index_query_width, input_stride;
    unsigned long long local_rows, compressed_new, compressed_rows, compressed_stride;
    unsigned long long indexer_rows, indexer_stride, topk_capacity;
    unsigned long long select_bytes, reduce_bytes;
    /* device buffers, carved from the backend's arena */
    job_buffer buffers[JOB_BUFFERS];
    unsigned int buffer_count;
    float *input, *q_low, *query, *sinks, *attention, *low, *output;
    float *q_norm, *kv_norm;
    float *local, *compressed, *indexer;
    unsigned long long *local_positions, *compressed_positions, *indexer_positions;
    struct job_rolling {
        float *before_kv, *before_score, *after_kv, *after_score;
        float *token_kv, *token_score, *ape, *norm;
    } rolling[2];
    float *index_query, *index_weights, *scores;
    unsigned long long *selected, *selected_count;
    double *rope_frequency;
    void *select_workspace, *reduce_workspace;
    /* accounting */
    unsigned long long launches, h2d, d2h, d2d, device_bytes, staged_state;
} job_run;

static int job_fail(job_run *run, yvex_backend_attention_failure_code code, const char *stage,
                    unsigned long long expected, unsigned long long actual, yvex_status status,
                    const char *message)
{
    if (run->failure) {
        run->failure->code = code;
        run->failure->stage = stage;
        run->failure->expected = expected;
        run->failure->actual = actual;
    }
    return yvx_fail(run->err, status, stage, message);
}

/* A failed shim call: typed by what it was doing. YVEX_ERR_BACKEND is sticky. */
static int job_device_fail(job_run *run, yvex_backend_attention_failure_code code, const char *stage, int rc)
{
    if (run->failure) {
        run->failure->code = rc == YVEX_ERR_UNSUPPORTED ? YVEX_BACKEND_ATTENTION_FAILURE_CAPABILITY : code;
        run->failure->stage = stage;
        run->failure->expected = 0ull;
        run->failure->actual = (unsigned long long)(unsigned int)-rc;
    }
    return yvx_backend_device_fail(run->backend, rc, stage, run->err);
}

/* The cooperative cancellation predicate of the job, polled between the phases of the
 * transaction (include/yvex/internal/backend.h:82-83,118; src/backend/cuda/attention.c:
 * 147-151). Work already enqueued is drained first so that nothing reads the arena after
 * the refusal. */
static int job_cancelled(job_run *run, const char *stage)
{
    const yvex_backend_cancellation *c = run->job->cancellation;
    if (!c || !c->requested || !c->requested(c->context)) return YVEX_OK;
    if (run->work_pending) (void)yvx_cuda_stream_synchronize(run->backend->stream);
    run->work_pending = 0;
    run->backend->status_pending = 0;
    return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_CANCELLED, stage, 0ull, 1ull, YVEX_ERR_CANCELLED,
                    "attention job cancelled by its caller");
}

static int job_take(job_run *run, void **target, unsigned long long elements, unsigned long long width)
{
    unsigned long long bytes;
    *target = NULL;
    if (!elements) return 1;
    if (run->buffer_count >= JOB_BUFFERS || !yvx_u64_mul(elements, width, &bytes) || bytes > ULLONG_MAX - 255ull)
        return 0;
    run->buffers[run->buffer_count].target = target;
    run->buffers[run->buffer_count].bytes = (bytes + 255ull) & ~255ull;
    run->buffer_count++;
    return 1;
}
#define TAKE(field, elements, type) job_take(run, (void **)&run->field, (elements), sizeof(type))

static int qtype_admitted(unsigned int qtype)
{
    return qtype == YVX_QTYPE_F32 || qtype == YVX_QTYPE_F16 || qtype == YVX_QTYPE_BF16 || qtype == YVX_QTYPE_Q8_0;
}

static const char *const weight_stage[YVEX_BACKEND_ATTENTION_WEIGHT_COUNT] = {
    "cuda.attention.q_a", "cuda.attention.q_norm", "cuda.attention.q_b", "cuda.attention.kv",
    "cuda.attention.kv_norm", "cuda.attention.sinks", "cuda.attention.output_a", "cuda.attention.output_b",
    "cuda.attention.main_rolling", "cuda.attention.main_rolling", "cuda.attention.main_rolling",
    "cuda.attention.main_rolling", "cuda.attention.index_rolling", "cuda.attention.index_rolling",
    "cuda.attention.index_rolling", "cuda.attention.index_rolling", "cuda.attention.index_query",
    "cuda.attention.index_weights", "cuda.attention.mhc_function", "cuda.attention.mhc_base",
    "cuda.attention.mhc_scale", "cuda.attention.input_norm"};

/* One weight slot against the geometry the job implies for it. */
static int job_weight_check(job_run *run, unsigned int slot, unsigned long long rows, unsigned long long width)
{
    const yvex_backend_attention_weight *w = &run->job->weights[slot];
    unsigned long long row_bytes, bytes;
    if (!w->present || !w->encoded)
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT, weight_stage[slot], 1ull, 0ull,
                        YVEX_ERR_INVALID_ARG, "an encoded weight of the attention job is missing");
    if (!qtype_admitted(w->qtype))
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_CAPABILITY, weight_stage[slot], YVX_QTYPE_BF16,
                        w->qtype, YVEX_ERR_UNSUPPORTED,
                        "weight encoding has no device projection here (F32, F16, BF16 and Q8_0 do)");
    row_bytes = yvx_cuda_qtype_row_bytes(w->qtype, width);
    if (w->row_width != width || w->row_count != rows || !row_bytes || w->row_bytes != row_bytes ||
        !yvx_u64_mul(rows, row_bytes, &bytes) || (unsigned long long)w->encoded_bytes != bytes)
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT, weight_stage[slot], rows * width,
                        w->row_count * w->row_width, YVEX_ERR_FORMAT,
                        "encoded weight geometry does not match the attention job");
    return YVEX_OK;
}

/* A cheap content fingerprint of an encoded weight: its size, its first and last 4 KiB and
 * 256 samples of 16 bytes spread over it (FNV-1a). Host memory that was freed and handed
 * out again with other weights at the same address is told apart by it; a caller that
 * rewrites weights in place calls yvex_b200_backend_weights_forget. */
static unsigned long long weight_fingerprint(const unsigned char *bytes, unsigned long long count)
{
    unsigned long long h = 1469598103934665603ull ^ count, i, k;
    const unsigned long long edge = count < 4096ull ? count : 4096ull;
#define MIX(byte) (h = (h ^ (unsigned long long)(byte)) * 1099511628211ull)
    for (i = 0; i < edge; ++i) MIX(bytes[i]);
    for (i = count - edge; i < count; ++i) MIX(bytes[i]);
    if (count > 8192ull)
        for (k = 0; k < 256ull; ++k) {
            const unsigned long long at = 4096ull + (count - 8192ull) / 256ull * k;
            for (i = 0; i < 16ull && at + i < count; ++i) MIX(bytes[at + i]);
        }
#undef MIX
    return h;
}

/* Device residence of an encoded weight: uploaded on first use, found again by host address,
 * size and fingerprint (the reference resolves resident weights by host address:
 * src/backend/cuda/attention.c:560-580). An address whose content changed is uploaded anew
 * into the same slot. */
static int job_weight_resident(job_run *run, unsigned int slot, const void **device)
{
    yvex_backend *b = run->backend;
    const yvex_backend_attention_weight *w = &run->job->weights[slot];
    unsigned long long address = 0ull, fingerprint;
    unsigned int i;
    void *memory = NULL;
    int rc;
    /* the runtime's resident arena first: read in place, nothing is copied */
    rc = yvex_backend_resident_resolve(b, w->encoded, w->encoded_bytes, &address);
    if (rc == YVEX_BACKEND_RESIDENT_INVALID)
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, weight_stage[slot], w->encoded_bytes, 0ull,
                        YVEX_ERR_STATE, "resident weight mapping is invalid");
    if (rc == YVEX_BACKEND_RESIDENT_HIT) {
        *device = (const void *)(uintptr_t)address;
        return YVEX_OK;
    }
    fingerprint = weight_fingerprint(w->encoded, w->encoded_bytes);
    for (i = 0; i < b->weight_count; ++i)
        if (b->weights[i].host == w->encoded && b->weights[i].bytes == w->encoded_bytes) {
            if (b->weights[i].fingerprint != fingerprint) {
                rc = yvx_cuda_upload_async(b->weights[i].device, w->encoded, w->encoded_bytes, b->stream);
                if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, weight_stage[slot], rc);
                b->weights[i].fingerprint = fingerprint;
                run->h2d += w->encoded_bytes;
                run->work_pending = 1;
            }
            *device = b->weights[i].device;
            return YVEX_OK;
        }
    if (b->weight_count == b->weight_capacity) {
        unsigned int capacity = b->weight_capacity ? b->weight_capacity * 2u : 32u;
        struct yvx_resident_weight *grown = realloc(b->weights, capacity * sizeof(*grown));
        if (!grown)
            return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_ALLOCATION, weight_stage[slot], capacity, 0ull,
                            YVEX_ERR_NOMEM, "weight residency table allocation failed");
        b->weights = grown;
        b->weight_capacity = capacity;
    }
    rc = yvx_cuda_malloc(&memory, w->encoded_bytes);
    if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_ALLOCATION, weight_stage[slot], rc);
    rc = yvx_cuda_upload_async(memory, w->encoded, w->encoded_bytes, b->stream);
    if (rc != 0) {
        (void)yvx_cuda_free(memory);
        return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, weight_stage[slot], rc);
    }
    run->h2d += w->encoded_bytes;
    run->work_pending = 1;
    b->weights[b->weight_count].host = w->encoded;
    b->weights[b->weight_count].bytes = w->encoded_bytes;
    b->weights[b->weight_count].fingerprint = fingerprint;
    b->weights[b->weight_count].device = memory;
    b->weight_count++;
    *device = memory;
    return YVEX_OK;
}

/* Session state (histories, positions, rolling states): a copy on the device when the runtime's
 * state residency knows the range, an upload otherwise. */
static int job_state(job_run *run, void *device, const void *host, unsigned long long bytes, const char *stage)
{
    unsigned long long address = 0ull;
    int rc;
    if (!bytes) return YVEX_OK;
    rc = yvex_backend_state_residency_resolve(run->backend, host, bytes, &address);
    if (rc == YVEX_BACKEND_RESIDENT_INVALID)
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, stage, bytes, 0ull, YVEX_ERR_STATE,
                        "persistent device state mapping is invalid");
    if (rc != YVEX_BACKEND_RESIDENT_HIT) {
        rc = yvx_cuda_upload_async(device, host, bytes, run->backend->stream);
        if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, stage, rc);
        run->h2d += bytes;
    } else {
        rc = yvx_cuda_copy_async(device, (const void *)(uintptr_t)address, bytes, run->backend->stream);
        if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, stage, rc);
        run->d2d += bytes;
        run->staged_state += bytes;
    }
    run->work_pending = 1;
    return YVEX_OK;
}

static int job_upload(job_run *run, void *device, const void *host, unsigned long long bytes, const char *stage)
{
    int rc;
    if (!bytes) return YVEX_OK;
    rc = yvx_cuda_upload_async(device, host, bytes, run->backend->stream);
    if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, stage, rc);
    run->h2d += bytes;
    run->work_pending = 1;
    return YVEX_OK;
}

/* The five row projections around the attention with BF16 weights; never the rolling state
 * (bit-exact by contract) nor the index projections (a flipped lane there can change which
 * rows are selected). */
static int job_gemm_admits(const job_run *run, unsigned int slot, const yvex_backend_attention_weight *w,
                           unsigned long long width, const float *input, unsigned long long input_stride,
                           int round_bf16)
{
    const yvex_backend *b = run->backend;
    const int row_projection = slot == YVEX_BACKEND_ATTENTION_WEIGHT_Q_A || slot == YVEX_BACKEND_ATTENTION_WEIGHT_Q_B ||
                               slot == YVEX_BACKEND_ATTENTION_WEIGHT_KV || slot == YVEX_BACKEND_ATTENTION_WEIGHT_OUT_A ||
                               slot == YVEX_BACKEND_ATTENTION_WEIGHT_OUT_B;
    return row_projection && round_bf16 && b->projection_gemm_tokens && run->tokens >= b->projection_gemm_tokens &&
           w->qtype == YVX_QTYPE_BF16 && width % 8ull == 0ull && input_stride % 2ull == 0ull &&
           ((uintptr_t)input & 7u) == 0u;
}

static int job_matvec(job_run *run, unsigned int slot, unsigned long long rows, unsigned long long width,
                      unsigned long long groups, const float *input, unsigned long long input_stride,
                      float *output, unsigned long long output_stride, int round_bf16)
{
    const yvex_backend_attention_weight *w = &run->job->weights[slot];
    yvx_matvec_args a;
    const void *device = NULL;
    int rc = job_weight_resident(run, slot, &device);
    if (rc != YVEX_OK) return rc;
    if (job_gemm_admits(run, slot, w, width, input, input_stride, round_bf16)) {
        /* prefill-sized token counts: the tensor-core projection (published values within one
         * bf16 step of the exact sum; opted into with yvex_b200_backend_projection_gemm) */
        yvex_backend *b = run->backend;
        yvx_gemm_args g;
        const unsigned long long need = yvx_cuda_bf16_gemm_staging_bytes(run->tokens, groups, width);
        if (need > b->gemm_staging_bytes) {
            rc = yvx_cuda_device_synchronize();
            if (rc == 0) rc = yvx_cuda_free(b->gemm_staging);
            b->gemm_staging = NULL;
            b->gemm_staging_bytes = 0ull;
            if (rc == 0) rc = yvx_cuda_malloc(&b->gemm_staging, need + need / 4ull);
            if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_ALLOCATION, weight_stage[slot], rc);
            b->gemm_staging_bytes = need + need / 4ull;
        }
        memset(&g, 0, sizeof(g));
        g.weights = device;
        g.rows = rows;
        g.width = width;
        g.input = input;
        g.tokens = run->tokens;
        g.input_stride = input_stride;
        g.output = output;
        g.output_stride = output_stride;
        g.groups = groups;
        g.round_bf16 = round_bf16;
        g.staging = b->gemm_staging;
        g.status = b->status_device;
        rc = yvx_cuda_bf16_gemm(&g, b->stream);
        if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_LAUNCH, weight_stage[slot], rc);
        run->launches += 2u;
        run->work_pending = 1;
        return YVEX_OK;
    }
    memset(&a, 0, sizeof(a));
    a.weights = device;
    a.qtype = w->qtype;
    a.rows = rows;
    a.width = width;
    a.row_bytes = w->row_bytes;
    a.input = input;
    a.tokens = run->tokens;
    a.input_stride = input_stride;
    a.output = output;
    a.output_stride = output_stride;
    a.groups = groups;
    a.round_bf16 = round_bf16;
    a.status = run->backend->status_device;
    rc = yvx_cuda_qtype_matvec(&a, run->backend->stream);
    if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_LAUNCH, weight_stage[slot], rc);
    run->launches++;
    run->work_pending = 1;
    return YVEX_OK;
}

static int job_decode(job_run *run, unsigned int slot, unsigned long long rows, unsigned long long width, float *out)
{
    const yvex_backend_attention_weight *w = &run->job->weights[slot];
    const void *device = NULL;
    int rc = job_weight_resident(run, slot, &device);
    if (rc != YVEX_OK) return rc;
    rc = yvx_cuda_qtype_decode_rows(device, w->qtype, 0ull, rows, width, out, run->backend->status_device,
                                    run->backend->stream);
    if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_LAUNCH, weight_stage[slot], rc);
    run->launches++;
    run->work_pending = 1;
    return YVEX_OK;
}

static unsigned int activation_bits(const yvex_backend_attention_activation *a)
{
    return a->required ? a->quantization : 0u;
}

/* ---- admission ------------------------------------------------------------------ */

static int rolling_check(job_run *run, const yvex_backend_attention_rolling *r, unsigned long long head_dimension,
                         const char *stage)
{
    const yvex_backend_attention_job *job = run->job;
    const unsigned long long factor = r->overlap ? 2ull : 1ull, ratio = job->compression_ratio;
    unsigned long long elements;
    if (!r->present || !r->kv_state || !r->score_state)
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT, stage, 1ull, 0ull, YVEX_ERR_INVALID_ARG,
                        "the rolling compressor state of this attention class is missing");
    if (r->ratio != ratio || r->head_dimension != head_dimension || r->state_width != head_dimension * factor ||
        r->state_slots != ratio * factor || !yvx_u64_mul(r->state_slots, r->state_width, &elements) ||
        r->kv_state_capacity < elements || r->score_state_capacity < elements)
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT, stage, head_dimension * factor,
                        r->state_width, YVEX_ERR_FORMAT, "rolling compressor state geometry mismatch");
    /* the record's cursor and fills follow from its position (src/graph/attention.c:598-605) */
    if (r->next_token_position != job->token_position || r->cursor != job->token_position % ratio ||
        r->current_fill != r->cursor ||
        r->previous_fill != (r->overlap && job->token_position >= ratio ? ratio : 0ull))
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT, stage, job->token_position % ratio,
                        r->cursor, YVEX_ERR_STATE, "rolling compressor state does not match its token position");
    return YVEX_OK;
}

static int job_admit(job_run *run)
{
    const yvex_backend_attention_job *job = run->job;
    const char *stage = "cuda.attention.prepare";
    const int compressed = job->attention_class != YVEX_BACKEND_ATTENTION_SWA;
    const int sparse = job->attention_class == YVEX_BACKEND_ATTENTION_CSA;
    unsigned long long end, rope = job->position.rope_dimensions;
    int rc;
#define BAD(expected, actual, message) \
    return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT, stage, (expected), (actual), \
                    YVEX_ERR_INVALID_ARG, (message))
#define UNSUPPORTED(where, expected, actual, message) \
    return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_CAPABILITY, (where), (expected), (actual), \
                    YVEX_ERR_UNSUPPORTED, (message))
    if (job->schema != YVEX_BACKEND_ATTENTION_JOB_SCHEMA)
        BAD(YVEX_BACKEND_ATTENTION_JOB_SCHEMA, job->schema, "attention job schema mismatch");
    if ((int)job->phase < 0 || job->phase >= YVEX_BACKEND_ATTENTION_PHASE_COUNT ||
        job->phase == 4 || job->phase == 5)
        BAD(YVEX_BACKEND_ATTENTION_PHASE_DECODE, job->phase, "attention job phase is not a backend phase");
    if ((unsigned int)job->attention_class > YVEX_BACKEND_ATTENTION_HCA)
        BAD(YVEX_BACKEND_ATTENTION_HCA, job->attention_class, "unknown attention class");
    if (job->compute_contract != YVEX_BACKEND_ATTENTION_COMPUTE_BF16_F32_RNE_V1)
        UNSUPPORTED(stage, YVEX_BACKEND_ATTENTION_COMPUTE_BF16_F32_RNE_V1, job->compute_contract,
                    "attention compute contract has no device projection");
    if (job->operation_scope != YVEX_BACKEND_ATTENTION_SCOPE_CORE)
        UNSUPPORTED("cuda.attention.mhc_pre", YVEX_BACKEND_ATTENTION_SCOPE_CORE, job->operation_scope,
                    "the residual-mixing envelope is not built: only the core scope runs");
    if (job->device_completion && job->device_completion->defer)
        UNSUPPORTED("cuda.attention.complete.prepare", 0ull, 1ull, "deferred completion is not built");
    if (job->retain_prefix_checkpoints)
        UNSUPPORTED("cuda.attention.alloc.main_kv_state", 0ull, 1ull, "retained prefix checkpoints are not built");
    if (!job->token_count || !job->hidden_width || !job->q_rank || !job->query_heads || !job->head_dimension ||
        !job->sliding_window || !job->output_groups || !job->output_group_input_width || !job->output_rank ||
        job->input_stride < job->hidden_width || (!job->input && !job->device_input) ||
        job->kv_width != job->head_dimension || !(job->rms_epsilon > 0.0) ||
        !yvx_u64_mul(job->query_heads, job->head_dimension, &run->query_width) ||
        !yvx_u64_mul(job->output_groups, job->output_rank, &run->low_width) ||
        !yvx_u64_add(job->token_position, job->token_count, &end))
        BAD(1ull, 0ull, "complete attention job geometry is required");
    if (job->output_groups * job->output_group_input_width != run->query_width)
        BAD(run->query_width, job->output_groups * job->output_group_input_width,
            "output groups do not tile the attention width");
    /* contracts of the device stages (publication: rows of at most 1024 lanes in 16-byte
     * steps; reduce: head dimension at most 512) */
    if (job->head_dimension > 512ull || job->head_dimension % 4ull || job->q_rank > 1024ull || job->q_rank % 4ull ||
        job->token_count > 0x7fffffffull || rope < 2ull || (rope & 1ull) || rope > job->head_dimension ||
        (job->head_dimension - rope) % 4ull || job->position.theta <= 1ull)
        UNSUPPORTED(stage, 512ull, job->head_dimension, "attention geometry is outside the device stages' contracts");
    run->tokens = job->token_count;
    run->input_stride = job->device_input ? job->hidden_width : job->input_stride;
    if (job->local_count && (!job->local_kv || !job->local_positions || job->local_stride < job->head_dimension))
        BAD(job->head_dimension, job->local_stride, "local history rows, positions and stride are required");
    if (!yvx_u64_add(job->local_count, job->token_count, &run->local_rows)) BAD(1ull, 0ull, "local rows overflow");
    rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_Q_A, job->q_rank, job->hidden_width);
    if (rc == YVEX_OK) rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_Q_A_NORM, 1ull, job->q_rank);
    if (rc == YVEX_OK) rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_Q_B, run->query_width, job->q_rank);
    if (rc == YVEX_OK) rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_KV, job->kv_width, job->hidden_width);
    if (rc == YVEX_OK) rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_KV_NORM, 1ull, job->kv_width);
    if (rc == YVEX_OK) {
        /* sinks: query_heads values in one row or one value per row */
        const yvex_backend_attention_weight *w = &job->weights[YVEX_BACKEND_ATTENTION_WEIGHT_SINKS];
        rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_SINKS, w->row_count,
                              w->row_count ? job->query_heads / w->row_count : 0ull);
        if (rc == YVEX_OK && w->row_count * w->row_width != job->query_heads)
            BAD(job->query_heads, w->row_count * w->row_width, "one sink per query head is required");
    }
    if (rc == YVEX_OK)
        rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_OUT_A, run->low_width, job->output_group_input_width);
    if (rc == YVEX_OK) rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_OUT_B, job->hidden_width, run->low_width);
    if (rc != YVEX_OK) return rc;
    run->topk_capacity = 1ull;
    if (job->token_count > 65535ull ||
        (job->attention_class == YVEX_BACKEND_ATTENTION_CSA && job->compression_ratio != 4ull) ||
        (job->attention_class == YVEX_BACKEND_ATTENTION_HCA && job->compression_ratio != 128ull))
        UNSUPPORTED("cuda.attention.reduce", 4ull, job->compression_ratio,
                    "the reduce stage takes at most 65535 tokens, ratio 4 for the sparse and 128 for the dense class");
    if (compressed) {
        const unsigned long long ratio = job->compression_ratio;
        const yvex_backend_attention_rolling *m = &job->main_rolling;
        if (!ratio) BAD(1ull, 0ull, "a compression ratio is required for this attention class");
        rc = rolling_check(run, m, job->head_dimension, "cuda.attention.main_rolling");
        if (rc != YVEX_OK) return rc;
        run->compressed_new = end / ratio - job->token_position / ratio;
        run->compressed_stride = job->compressed_stride ? job->compressed_stride : job->head_dimension;
        if (run->compressed_stride < job->head_dimension ||
            (job->compressed_count && (!job->compressed_kv || !job->compressed_positions)) ||
            !yvx_u64_add(job->compressed_count, run->compressed_new, &run->compressed_rows))
            BAD(job->head_dimension, run->compressed_stride, "compressed history rows, positions and stride are required");
        rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_MAIN_KV, m->state_width, job->hidden_width);
        if (rc == YVEX_OK) rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_MAIN_GATE, m->state_width, job->hidden_width);
        if (rc == YVEX_OK) rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_MAIN_APE, ratio, m->state_width);
        if (rc == YVEX_OK) rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_MAIN_NORM, 1ull, job->head_dimension);
        if (rc != YVEX_OK) return rc;
    }
    if (sparse) {
        const yvex_backend_attention_rolling *x = &job->indexer_rolling;
        const unsigned long long id = job->indexer_head_dimension;
        if (!job->indexer_heads || !id || !job->indexer_topk ||
            !yvx_u64_mul(job->indexer_heads, id, &run->index_query_width))
            BAD(1ull, 0ull, "indexer heads, head dimension and top-k are required for sparse attention");
        if (job->indexer_heads > 64ull || id > 256ull || id % 4ull || job->indexer_topk > 1024ull || rope > id ||
            (id - rope) % 4ull)
            UNSUPPORTED("cuda.attention.topk", 64ull, job->indexer_heads, "indexer geometry is outside the selection stage's contract");
        rc = rolling_check(run, x, id, "cuda.attention.index_rolling");
        if (rc != YVEX_OK) return rc;
        run->indexer_stride = job->indexer_stride ? job->indexer_stride : id;
        if (job->indexer_count != job->compressed_count || run->indexer_stride < id ||
            (job->indexer_count && (!job->indexer_kv || !job->indexer_positions)))
            return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT, "cuda.attention.topk",
                            job->compressed_count, job->indexer_count, YVEX_ERR_FORMAT,
                            "compressed and indexer entries are not paired");
        run->indexer_rows = run->compressed_rows;
        run->topk_capacity = job->indexer_topk;
        rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_KV, x->state_width, job->hidden_width);
        if (rc == YVEX_OK) rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_GATE, x->state_width, job->hidden_width);
        if (rc == YVEX_OK) rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_APE, job->compression_ratio, x->state_width);
        if (rc == YVEX_OK) rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_NORM, 1ull, id);
        if (rc == YVEX_OK) rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_Q, run->index_query_width, job->q_rank);
        if (rc == YVEX_OK) rc = job_weight_check(run, YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_PROJECTION, job->indexer_heads, job->hidden_width);
        if (rc != YVEX_OK) return rc;
    }
#undef BAD
#undef UNSUPPORTED
    return YVEX_OK;
}

/* ---- arena ---------------------------------------------------------------------- */

static int job_layout(job_run *run)
{
    const yvex_backend_attention_job *job = run->job;
    const unsigned long long t = run->tokens;
    const int compressed = job->attention_class != YVEX_BACKEND_ATTENTION_SWA;
    const int sparse = job->attention_class == YVEX_BACKEND_ATTENTION_CSA;
    unsigned long long total = 0ull;
    unsigned int i;
    unsigned char *base = NULL;
    void *arena = NULL;
    int ok, rc;
    ok = TAKE(input, t * run->input_stride, float) && TAKE(q_low, t * job->q_rank, float) &&
         TAKE(query, t * run->query_width, float) && TAKE(sinks, job->query_heads, float) &&
         TAKE(attention, t * run->query_width, float) && TAKE(low, t * run->low_width, float) &&
         TAKE(output, t * job->hidden_width, float) && TAKE(q_norm, job->q_rank, float) &&
         TAKE(kv_norm, job->kv_width, float) && TAKE(rope_frequency, job->position.rope_dimensions / 2ull, double) &&
         TAKE(local, run->local_rows * (job->local_stride ? job->local_stride : job->head_dimension), float) &&
         TAKE(local_positions, run->local_rows, unsigned long long);
    if (ok && compressed) {
        const yvex_backend_attention_rolling *m = &job->main_rolling;
        const unsigned long long state = m->state_slots * m->state_width;
        ok = TAKE(compressed, (run->compressed_rows ? run->compressed_rows : 1ull) * run->compressed_stride, float) &&
             TAKE(compressed_positions, run->compressed_rows ? run->compressed_rows : 1ull, unsigned long long) &&
             TAKE(rolling[0].before_kv, state, float) && TAKE(rolling[0].before_score, state, float) &&
             TAKE(rolling[0].after_kv, state, float) && TAKE(rolling[0].after_score, state, float) &&
             TAKE(rolling[0].token_kv, t * m->state_width, float) && TAKE(rolling[0].token_score, t * m->state_width, float) &&
             TAKE(rolling[0].ape, job->compression_ratio * m->state_width, float) &&
             TAKE(rolling[0].norm, job->head_dimension, float);
    }
    if (ok && sparse) {
        const yvex_backend_attention_rolling *x = &job->indexer_rolling;
        const unsigned long long state = x->state_slots * x->state_width;
        const unsigned long long rows = run->indexer_rows ? run->indexer_rows : 1ull;
        run->select_bytes = yvx_cuda_csa_select_workspace_bytes(rows, t, (unsigned int)job->indexer_topk);
        ok = TAKE(indexer, rows * run->indexer_stride, float) && TAKE(indexer_positions, rows, unsigned long long) &&
             TAKE(rolling[1].before_kv, state, float) && TAKE(rolling[1].before_score, state, float) &&
             TAKE(rolling[1].after_kv, state, float) && TAKE(rolling[1].after_score, state, float) &&
             TAKE(rolling[1].token_kv, t * x->state_width, float) && TAKE(rolling[1].token_score, t * x->state_width, float) &&
             TAKE(rolling[1].ape, job->compression_ratio * x->state_width, float) &&
             TAKE(rolling[1].norm, job->indexer_head_dimension, float) &&
             TAKE(index_query, t * run->index_query_width, float) && TAKE(index_weights, t * job->indexer_heads, float) &&
             TAKE(scores, t * rows, float) && TAKE(selected, t * run->topk_capacity, unsigned long long) &&
             TAKE(selected_count, t, unsigned long long) && TAKE(select_workspace, run->select_bytes, unsigned char);
    }
    /* the reduce workspace is sized once the arguments are known: an upper bound here */
    if (ok) {
        run->reduce_bytes = t * job->query_heads * 64ull * (job->head_dimension + 2ull) * sizeof(float);
        if (run->reduce_bytes > (256ull << 20)) run->reduce_bytes = 256ull << 20;
        ok = TAKE(reduce_workspace, run->reduce_bytes, unsigned char);
    }
    for (i = 0; ok && i < run->buffer_count; ++i) ok = yvx_u64_add(total, run->buffers[i].bytes, &total);
    if (!ok)
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_BUDGET, "cuda.attention.alloc.extent", ULLONG_MAX, 0ull,
                        YVEX_ERR_BOUNDS, "attention request arena extent overflowed");
    if (job->max_device_bytes && total > job->max_device_bytes)
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_BUDGET, "cuda.attention.alloc.budget", job->max_device_bytes,
                        total, YVEX_ERR_BOUNDS, "attention request exceeds its device byte budget");
    rc = yvx_backend_scratch(run->backend, total, &arena, "cuda.attention.alloc", run->err);
    if (rc != YVEX_OK) {
        if (run->failure) {
            run->failure->code = YVEX_BACKEND_ATTENTION_FAILURE_ALLOCATION;
            run->failure->stage = "cuda.attention.alloc";
            run->failure->expected = total;
            run->failure->actual = 0ull;
        }
        return rc;
    }
    base = (unsigned char *)arena;
    for (i = 0; i < run->buffer_count; ++i) {
        *run->buffers[i].target = base;
        base += run->buffers[i].bytes;
    }
    run->device_bytes = total;
    return YVEX_OK;
}

/* ---- staging of the inputs ------------------------------------------------------- */

static int job_stage_inputs(job_run *run)
{
    const yvex_backend_attention_job *job = run->job;
    yvex_backend *b = run->backend;
    const unsigned long long t = run->tokens, local_stride = job->local_stride ? job->local_stride : job->head_dimension;
    unsigned long long *positions;
    double *frequency;
    yvex_b200_position_policy policy;
    unsigned long long i;
    int rc;
    if (job->device_input) {
        const yvex_device_tensor *in = job->device_input;
        unsigned long long elements = t * job->hidden_width;
        if (!yvx_tensor_owned(b, in) || in->dtype != YVEX_DTYPE_F32 || in->bytes < elements * sizeof(float) || !in->is_written)
            return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT, "cuda.attention.alloc.input",
                            elements * sizeof(float), in->bytes, YVEX_ERR_FORMAT,
                            "device input must be a written F32 tensor of this backend");
        rc = yvx_cuda_copy_async(run->input, in->data, elements * sizeof(float), b->stream);
        if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, "cuda.attention.alloc.input", rc);
        run->d2d += elements * sizeof(float);
        run->work_pending = 1;
    } else {
        rc = job_upload(run, run->input, job->input, ((t - 1ull) * job->input_stride + job->hidden_width) * sizeof(float),
                        "cuda.attention.alloc.input");
        if (rc != YVEX_OK) return rc;
    }
    /* local rows: the history, then room for the phase's own rows; positions of both */
    positions = malloc((size_t)run->local_rows * sizeof(*positions));
    if (!positions)
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_ALLOCATION, "cuda.attention.alloc.local_positions",
                        run->local_rows, 0ull, YVEX_ERR_NOMEM, "host staging allocation failed");
    for (i = 0; i < job->local_count; ++i) positions[i] = job->local_positions[i];
    for (i = 0; i < t; ++i) positions[job->local_count + i] = job->token_position + i;
    rc = job_upload(run, run->local_positions, positions, run->local_rows * sizeof(*positions),
                    "cuda.attention.alloc.local_positions");
    if (rc == YVEX_OK) rc = yvx_cuda_stream_synchronize(b->stream) ? YVEX_ERR_BACKEND : YVEX_OK;
    free(positions);
    if (rc != YVEX_OK) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, "cuda.attention.alloc.local_positions", rc);
    rc = job_state(run, run->local, job->local_kv, job->local_count * local_stride * sizeof(float),
                    "cuda.attention.alloc.local_history");
    if (rc != YVEX_OK) return rc;
    if (job->attention_class != YVEX_BACKEND_ATTENTION_SWA) {
        const yvex_backend_attention_rolling *m = &job->main_rolling;
        rc = job_state(run, run->compressed, job->compressed_kv,
                        job->compressed_count * run->compressed_stride * sizeof(float), "cuda.attention.alloc.compressed_history");
        if (rc == YVEX_OK)
            rc = job_state(run, run->compressed_positions, job->compressed_positions,
                            job->compressed_count * sizeof(unsigned long long), "cuda.attention.alloc.compressed_positions");
        if (rc == YVEX_OK)
            rc = job_state(run, run->rolling[0].before_kv, m->kv_state, m->state_slots * m->state_width * sizeof(float),
                            "cuda.attention.alloc.main_kv_state");
        if (rc == YVEX_OK)
            rc = job_state(run, run->rolling[0].before_score, m->score_state, m->state_slots * m->state_width * sizeof(float),
                            "cuda.attention.alloc.main_score_state");
        if (rc != YVEX_OK) return rc;
    }
    if (job->attention_class == YVEX_BACKEND_ATTENTION_CSA) {
        const yvex_backend_attention_rolling *x = &job->indexer_rolling;
        rc = job_state(run, run->indexer, job->indexer_kv, job->indexer_count * run->indexer_stride * sizeof(float),
                        "cuda.attention.alloc.indexer_history");
        if (rc == YVEX_OK)
            rc = job_state(run, run->indexer_positions, job->indexer_positions,
                            job->indexer_count * sizeof(unsigned long long), "cuda.attention.alloc.indexer_positions");
        if (rc == YVEX_OK)
            rc = job_state(run, run->rolling[1].before_kv, x->kv_state, x->state_slots * x->state_width * sizeof(float),
                            "cuda.attention.alloc.index_kv_state");
        if (rc == YVEX_OK)
            rc = job_state(run, run->rolling[1].before_score, x->score_state, x->state_slots * x->state_width * sizeof(float),
                            "cuda.attention.alloc.index_score_state");
        if (rc != YVEX_OK) return rc;
    }
    /* rotation frequencies of the position policy, computed on the host in double */
    frequency = malloc((size_t)(job->position.rope_dimensions / 2ull) * sizeof(*frequency));
    if (!frequency)
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_ALLOCATION, "cuda.attention.query_rope", 1ull, 0ull,
                        YVEX_ERR_NOMEM, "host staging allocation failed");
    policy.theta = job->position.theta;
    policy.scaling_factor = job->position.scaling_factor;
    policy.original_context = job->position.original_context;
    policy.beta_fast = job->position.beta_fast;
    policy.beta_slow = job->position.beta_slow;
    if (yvex_b200_rope_frequencies(&policy, job->position.rope_dimensions, frequency) != YVEX_OK) {
        free(frequency);
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT, "cuda.attention.query_rope",
                        job->position.rope_dimensions, 0ull, YVEX_ERR_INVALID_ARG, "position policy has no rotation frequencies");
    }
    rc = job_upload(run, run->rope_frequency, frequency, job->position.rope_dimensions / 2ull * sizeof(*frequency),
                    "cuda.attention.query_rope");
    if (rc == YVEX_OK && yvx_cuda_stream_synchronize(b->stream) != 0)
        rc = job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, "cuda.attention.query_rope", YVEX_ERR_BACKEND);
    free(frequency);
    return rc;
}

/* ---- the stages ------------------------------------------------------------------ */

static void publish_set(yvx_rows_publish_args *p, job_run *run, float *values, unsigned long long rows,
                        unsigned long long rows_per_token, unsigned long long row_stride, unsigned long long width,
                        int norm_mode, const float *norm_weights, unsigned long long rope_dims,
                        const yvex_backend_attention_activation *activation, unsigned long long activation_count)
{
    memset(p, 0, sizeof(*p));
    p->values = values;
    p->rows = rows;
    p->rows_per_token = rows_per_token;
    p->row_stride = row_stride;
    p->width = width;
    p->norm_mode = norm_mode;
    p->norm_weights = norm_weights;
    p->epsilon = run->job->rms_epsilon;
    p->rope_dims = rope_dims;
    p->rope_frequency = rope_dims ? run->rope_frequency : NULL;
    p->start_position = run->job->token_position;
    if (activation && activation_bits(activation) && activation_count) {
        p->quantization = activation_bits(activation);
        p->activation_count = activation_count;
        p->block_width = activation->block_width;
        p->hadamard = activation->hadamard;
    }
    p->status = run->backend->status_device;
}

static int job_publish(job_run *run, const yvx_rows_publish_args *sets, unsigned int count, const char *stage)
{
    int rc = count == 1u ? yvx_cuda_rows_publish(&sets[0], run->backend->stream)
                         : yvx_cuda_rows_publish_batch(sets, count, run->backend->stream);
    if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_LAUNCH, stage, rc);
    run->launches++;
    run->work_pending = 1;
    return YVEX_OK;
}

static int job_project(job_run *run)
{
    const yvex_backend_attention_job *job = run->job;
    yvex_backend *b = run->backend;
    const unsigned long long t = run->tokens, local_stride = job->local_stride ? job->local_stride : job->head_dimension;
    const unsigned long long rope = job->position.rope_dimensions;
    float *raw_kv = run->local + job->local_count * local_stride;
    yvx_rows_publish_args sets[2];
    int rc;
    /* core scope: the input is published as bf16 before the first projection */
    rc = yvx_cuda_round_bf16_rows(run->input, t, job->hidden_width, run->input_stride, b->status_device, b->stream);
    if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_LAUNCH, "cuda.attention.input_round", rc);
    run->launches++;
    rc = job_matvec(run, YVEX_BACKEND_ATTENTION_WEIGHT_Q_A, job->q_rank, job->hidden_width, 1ull, run->input,
                    run->input_stride, run->q_low, job->q_rank, 1);
    if (rc == YVEX_OK) rc = job_decode(run, YVEX_BACKEND_ATTENTION_WEIGHT_Q_A_NORM, 1ull, job->q_rank, run->q_norm);
    if (rc != YVEX_OK) return rc;
    publish_set(&sets[0], run, run->q_low, t, 1ull, job->q_rank, job->q_rank, 2, run->q_norm, 0ull, NULL, 0ull);
    rc = job_publish(run, sets, 1u, "cuda.attention.q_norm");
    if (rc == YVEX_OK)
        rc = job_matvec(run, YVEX_BACKEND_ATTENTION_WEIGHT_Q_B, run->query_width, job->q_rank, 1ull, run->q_low,
                        job->q_rank, run->query, run->query_width, 1);
    if (rc == YVEX_OK)
        rc = job_matvec(run, YVEX_BACKEND_ATTENTION_WEIGHT_KV, job->kv_width, job->hidden_width, 1ull, run->input,
                        run->input_stride, raw_kv, local_stride, 1);
    if (rc == YVEX_OK) rc = job_decode(run, YVEX_BACKEND_ATTENTION_WEIGHT_KV_NORM, 1ull, job->kv_width, run->kv_norm);
    if (rc != YVEX_OK) return rc;
    /* query heads: unit norm, rotation; new local rows: weighted norm, rotation, activation of
     * the lanes in front of the rotated ones; one launch for both */
    publish_set(&sets[0], run, run->query, t * job->query_heads, job->query_heads, job->head_dimension,
                job->head_dimension, 1, NULL, rope, NULL, 0ull);
    publish_set(&sets[1], run, raw_kv, t, 1ull, local_stride, job->kv_width, 2, run->kv_norm, rope,
                &job->attention_kv_activation, job->kv_width - rope);
    rc = job_publish(run, sets, 2u, "cuda.attention.query_rope");
    if (rc != YVEX_OK) return rc;
    return job_decode(run, YVEX_BACKEND_ATTENTION_WEIGHT_SINKS,
                      job->weights[YVEX_BACKEND_ATTENTION_WEIGHT_SINKS].row_count,
                      job->weights[YVEX_BACKEND_ATTENTION_WEIGHT_SINKS].row_width, run->sinks);
}

static int job_rolling(job_run *run, unsigned int kind)
{
    const yvex_backend_attention_job *job = run->job;
    yvex_backend *b = run->backend;
    const int index = kind == 1u;
    const yvex_backend_attention_rolling *r = index ? &job->indexer_rolling : &job->main_rolling;
    struct job_rolling *d = &run->rolling[kind];
    const unsigned int base = index ? YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_KV : YVEX_BACKEND_ATTENTION_WEIGHT_MAIN_KV;
    const yvex_backend_attention_activation *activation =
        index ? &job->compressor_rotated_activation : &job->compressor_activation;
    const char *stage = index ? "cuda.attention.index_rolling" : "cuda.attention.main_rolling";
    const unsigned long long rope = job->position.rope_dimensions;
    unsigned long long emitted = 0ull, rows_before = index ? job->indexer_count : job->compressed_count;
    yvx_compressor_args a;
    int rc;
    rc = job_matvec(run, base, r->state_width, job->hidden_width, 1ull, run->input, run->input_stride, d->token_kv,
                    r->state_width, 0);
    if (rc == YVEX_OK)
        rc = job_matvec(run, base + 1u, r->state_width, job->hidden_width, 1ull, run->input, run->input_stride,
                        d->token_score, r->state_width, 0);
    if (rc == YVEX_OK) rc = job_decode(run, base + 2u, job->compression_ratio, r->state_width, d->ape);
    if (rc == YVEX_OK) rc = job_decode(run, base + 3u, 1ull, r->head_dimension, d->norm);
    if (rc != YVEX_OK) return rc;
    memset(&a, 0, sizeof(a));
    a.ratio = job->compression_ratio;
    a.head_dim = r->head_dimension;
    a.overlap = r->overlap;
    a.start_position = job->token_position;
    a.token_count = run->tokens;
    a.token_kv = d->token_kv;
    a.token_score = d->token_score;
    a.token_stride = r->state_width;
    a.ape = d->ape;
    a.state_kv = d->before_kv;
    a.state_score = d->before_score;
    a.after_kv = d->after_kv;
    a.after_score = d->after_score;
    a.compressed = index ? run->indexer + rows_before * run->indexer_stride
                         : run->compressed + rows_before * run->compressed_stride;
    a.compressed_stride = index ? run->indexer_stride : run->compressed_stride;
    a.positions = (index ? run->indexer_positions : run->compressed_positions) + rows_before;
    a.norm_weights = d->norm;
    a.epsilon = job->rms_epsilon;
    a.rope_dims = rope;
    a.rope_frequency = run->rope_frequency;
    a.status = b->status_device;
    if (!index && r->head_dimension <= rope)
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT, stage, rope + 1ull, r->head_dimension,
                        YVEX_ERR_FORMAT, "the main compressor requires lanes in front of the rotated ones");
    if (activation_bits(activation)) {
        a.activation_quantization = activation_bits(activation);
        a.activation_count = index ? r->head_dimension : r->head_dimension - rope;
        a.activation_block_width = activation->block_width;
        a.activation_hadamard = activation->hadamard;
    }
    rc = yvx_cuda_compressor_chunk(&a, b->stream, &emitted);
    if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_LAUNCH, stage, rc);
    run->launches++;
    run->work_pending = 1;
    if (emitted != run->compressed_new)
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT, stage, run->compressed_new, emitted,
                        YVEX_ERR_STATE, "the compressor emitted a different number of rows than the phase holds");
    return YVEX_OK;
}

static int job_compress(job_run *run)
{
    const yvex_backend_attention_job *job = run->job;
    yvex_backend *b = run->backend;
    yvx_rows_publish_args set;
    yvx_csa_select_args s;
    unsigned int launches = 0u;
    int rc;
    if (job->attention_class == YVEX_BACKEND_ATTENTION_SWA) return YVEX_OK;
    rc = job_rolling(run, 0u);
    if (rc != YVEX_OK || job->attention_class != YVEX_BACKEND_ATTENTION_CSA) return rc;
    rc = job_rolling(run, 1u);
    if (rc != YVEX_OK) return rc;
    /* index queries from the normalised low-rank query, head weights from the input */
    rc = job_matvec(run, YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_Q, run->index_query_width, job->q_rank, 1ull, run->q_low,
                    job->q_rank, run->index_query, run->index_query_width, 1);
    if (rc == YVEX_OK)
        rc = job_matvec(run, YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_PROJECTION, job->indexer_heads, job->hidden_width, 1ull,
                        run->input, run->input_stride, run->index_weights, job->indexer_heads, 1);
    if (rc != YVEX_OK) return rc;
    publish_set(&set, run, run->index_query, run->tokens * job->indexer_heads, job->indexer_heads,
                job->indexer_head_dimension, job->indexer_head_dimension, 0, NULL, job->position.rope_dimensions,
                &job->indexer_query_activation, job->indexer_head_dimension);
    rc = job_publish(run, &set, 1u, "cuda.attention.index_query_rope");
    if (rc != YVEX_OK) return rc;
    if (!run->indexer_rows) {
        /* nothing to rank: every token selects no row */
        rc = yvx_cuda_memset_async(run->selected_count, 0, run->tokens * sizeof(unsigned long long), b->stream);
        if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_LAUNCH, "cuda.attention.topk", rc);
        return YVEX_OK;
    }
    memset(&s, 0, sizeof(s));
    s.keys = run->indexer;
    s.positions = run->indexer_positions;
    s.rows = run->indexer_rows;
    s.key_stride = run->indexer_stride;
    s.query = run->index_query;
    s.weights = run->index_weights;
    s.heads = (unsigned int)job->indexer_heads;
    s.head_dim = (unsigned int)job->indexer_head_dimension;
    s.topk = (unsigned int)job->indexer_topk;
    s.ratio = job->compression_ratio;
    s.phase_start_position = job->token_position;
    s.token_count = run->tokens;
    s.scores = run->scores;
    s.selected = run->selected;
    s.selected_count = run->selected_count;
    s.topk_capacity = run->topk_capacity;
    s.workspace = run->select_workspace;
    s.status = b->status_device;
    rc = yvx_cuda_csa_select(&s, b->stream, &launches);
    if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_LAUNCH, "cuda.attention.topk", rc);
    run->launches += launches;
    run->work_pending = 1;
    return YVEX_OK;
}

static int job_reduce(job_run *run)
{
    const yvex_backend_attention_job *job = run->job;
    yvex_backend *b = run->backend;
    yvx_latent_reduce_args a;
    unsigned int launches = 0u;
    int rc;
    memset(&a, 0, sizeof(a));
    a.query = run->query;
    a.local = run->local;
    a.local_positions = run->local_positions;
    a.initial_local_count = job->local_count;
    a.local_stride = job->local_stride ? job->local_stride : job->head_dimension;
    a.compressed = run->compressed;
    a.compressed_positions = run->compressed_positions;
    a.compressed_stride = run->compressed_stride;
    a.selected = run->selected;
    a.selected_count = run->selected_count;
    a.topk_capacity = run->topk_capacity;
    a.sinks = run->sinks;
    a.query_heads = job->query_heads;
    a.head_dim = job->head_dimension;
    a.sliding_window = job->sliding_window;
    a.ratio = job->attention_class == YVEX_BACKEND_ATTENTION_SWA ? 0ull : job->compression_ratio;
    a.attention_class = (unsigned int)job->attention_class;
    a.phase_start_position = job->token_position;
    a.token_count = run->tokens;
    a.candidate_block_visible = job->candidate_block_visible;
    a.out = run->attention;
    a.status = b->status_device;
    a.rope_dims = job->position.rope_dimensions;
    a.rope_frequency = run->rope_frequency;
    if (job->attention_class == YVEX_BACKEND_ATTENTION_HCA) {
        /* the dense class walks every compressed row of the history and of this phase */
        a.selected = NULL;
        a.selected_count = NULL;
    }
    /* HCA's candidate count travels with compressed_positions: rows beyond the visible ones
     * are masked by position; the row count is what the arena holds */
    a.workspace = yvx_cuda_latent_reduce_workspace_bytes(&a) <= run->reduce_bytes ? run->reduce_workspace : NULL;
    rc = yvx_cuda_latent_reduce_launches(&a, b->stream, &launches);
    if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_LAUNCH, "cuda.attention.reduce", rc);
    run->launches += launches;
    run->work_pending = 1;
    /* grouped low-rank output projection, then the projection back to the hidden width */
    rc = job_matvec(run, YVEX_BACKEND_ATTENTION_WEIGHT_OUT_A, job->output_rank, job->output_group_input_width,
                    job->output_groups, run->attention, run->query_width, run->low, run->low_width, 1);
    if (rc == YVEX_OK)
        rc = job_matvec(run, YVEX_BACKEND_ATTENTION_WEIGHT_OUT_B, job->hidden_width, run->low_width, 1ull, run->low,
                        run->low_width, run->output, job->hidden_width, 1);
    return rc;
}

/* ---- publication of the results --------------------------------------------------- */

static int job_download(job_run *run, void *host, unsigned long long capacity, const void *device,
                        unsigned long long rows, unsigned long long width, unsigned long long device_stride,
                        size_t element, const char *stage)
{
    unsigned long long r;
    int rc = 0;
    if (!host || !rows || !width) return YVEX_OK;
    if (capacity < rows * width)
        return job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, stage, rows * width, capacity, YVEX_ERR_BOUNDS,
                        "attention output span is smaller than the published extent");
    if (device_stride == width) {
        rc = yvx_cuda_download_async(host, device, rows * width * element, run->backend->stream);
    } else {
        for (r = 0; rc == 0 && r < rows; ++r)
            rc = yvx_cuda_download_async((unsigned char *)host + r * width * element,
                                         (const unsigned char *)device + r * device_stride * element, width * element,
                                         run->backend->stream);
    }
    if (rc != 0) return job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, stage, rc);
    run->d2h += rows * width * element;
    return YVEX_OK;
}

static int job_publish_outputs(job_run *run)
{
    const yvex_backend_attention_job *job = run->job;
    yvex_backend_attention_output *o = run->out;
    yvex_backend *b = run->backend;
    const unsigned long long t = run->tokens, local_stride = job->local_stride ? job->local_stride : job->head_dimension;
    const int compressed = job->attention_class != YVEX_BACKEND_ATTENTION_SWA;
    const int sparse = job->attention_class == YVEX_BACKEND_ATTENTION_CSA;
    unsigned long long *selected = NULL, *counts = NULL;
    unsigned long long token, i;
    int rc;
#define FLOATS(span, device, rows, width, stride, stage) \
    job_download(run, o->span.data, o->span.capacity, (device), (rows), (width), (stride), sizeof(float), (stage))
    rc = FLOATS(core_input, run->input, t, job->hidden_width, run->input_stride, "cuda.attention.copy.core_input");
    if (rc == YVEX_OK) rc = FLOATS(q_low, run->q_low, t, job->q_rank, job->q_rank, "cuda.attention.copy.q_low");
    if (rc == YVEX_OK) rc = FLOATS(query, run->query, t, run->query_width, run->query_width, "cuda.attention.copy.query");
    if (rc == YVEX_OK)
        rc = FLOATS(raw_kv, run->local + job->local_count * local_stride, t, job->kv_width, local_stride,
                    "cuda.attention.copy.raw_kv");
    if (rc == YVEX_OK)
        rc = FLOATS(attention_values, run->attention, t, run->query_width, run->query_width, "cuda.attention.copy.attention");
    if (rc == YVEX_OK) rc = FLOATS(output, run->output, t, job->hidden_width, job->hidden_width, "cuda.attention.copy.output");
    if (rc == YVEX_OK && compressed) {
        const yvex_backend_attention_rolling *m = &job->main_rolling;
        rc = FLOATS(compressed_kv, run->compressed + job->compressed_count * run->compressed_stride, run->compressed_new,
                    job->head_dimension, run->compressed_stride, "cuda.attention.copy.compressed");
        if (rc == YVEX_OK)
            rc = job_download(run, o->compressed_positions.data, o->compressed_positions.capacity,
                              run->compressed_positions + job->compressed_count, run->compressed_new, 1ull, 1ull,
                              sizeof(unsigned long long), "cuda.attention.copy.compressed_positions");
        if (rc == YVEX_OK)
            rc = FLOATS(main_kv_state, run->rolling[0].after_kv, 1ull, m->state_slots * m->state_width,
                        m->state_slots * m->state_width, "cuda.attention.copy.main_kv_state");
        if (rc == YVEX_OK)
            rc = FLOATS(main_score_state, run->rolling[0].after_score, 1ull, m->state_slots * m->state_width,
                        m->state_slots * m->state_width, "cuda.attention.copy.main_score_state");
    }
    if (rc == YVEX_OK && sparse) {
        const yvex_backend_attention_rolling *x = &job->indexer_rolling;
        rc = FLOATS(indexer_kv, run->indexer + job->indexer_count * run->indexer_stride, run->compressed_new,
                    job->indexer_head_dimension, run->indexer_stride, "cuda.attention.copy.indexer");
        if (rc == YVEX_OK)
            rc = job_download(run, o->indexer_positions.data, o->indexer_positions.capacity,
                              run->indexer_positions + job->indexer_count, run->compressed_new, 1ull, 1ull,
                              sizeof(unsigned long long), "cuda.attention.copy.indexer_positions");
        if (rc == YVEX_OK)
            rc = FLOATS(index_query, run->index_query, t, run->index_query_width, run->index_query_width,
                        "cuda.attention.copy.index_query");
        if (rc == YVEX_OK)
            rc = FLOATS(index_weights, run->index_weights, t, job->indexer_heads, job->indexer_heads,
                        "cuda.attention.copy.index_weights");
        if (rc == YVEX_OK)
            rc = FLOATS(indexer_kv_state, run->rolling[1].after_kv, 1ull, x->state_slots * x->state_width,
                        x->state_slots * x->state_width, "cuda.attention.copy.index_kv_state");
        if (rc == YVEX_OK)
            rc = FLOATS(indexer_score_state, run->rolling[1].after_score, 1ull, x->state_slots * x->state_width,
                        x->state_slots * x->state_width, "cuda.attention.copy.index_score_state");
        /* selection counts always come back (the counters need them); lists on request */
        counts = malloc((size_t)t * sizeof(*counts));
        selected = o->topk_positions.data ? malloc((size_t)(t * run->topk_capacity) * sizeof(*selected)) : NULL;
        if (rc == YVEX_OK && (!counts || (o->topk_positions.data && !selected)))
            rc = job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_ALLOCATION, "cuda.attention.copy.selected_count", t, 0ull,
                          YVEX_ERR_NOMEM, "host staging allocation failed");
        if (rc == YVEX_OK)
            rc = job_download(run, counts, t, run->selected_count, t, 1ull, 1ull, sizeof(unsigned long long),
                              "cuda.attention.copy.selected_count");
        if (rc == YVEX_OK && selected)
            rc = job_download(run, selected, t * run->topk_capacity, run->selected, t, run->topk_capacity,
                              run->topk_capacity, sizeof(unsigned long long), "cuda.attention.copy.selected");
    }
#undef FLOATS
    if (rc == YVEX_OK && job->device_output) {
        yvex_device_tensor *out = job->device_output;
        const unsigned long long bytes = t * job->hidden_width * sizeof(float);
        if (!yvx_tensor_owned(b, out) || out->dtype != YVEX_DTYPE_F32 || out->bytes < bytes)
            rc = job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT, "cuda.attention.copy.device_output", bytes,
                          out ? out->bytes : 0ull, YVEX_ERR_FORMAT, "device output must be an F32 tensor of this backend");
        else if (yvx_cuda_copy_async(out->data, run->output, bytes, b->stream) != 0)
            rc = job_device_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, "cuda.attention.copy.device_output", YVEX_ERR_BACKEND);
        else {
            out->is_written = 1;
            run->d2d += bytes;
        }
    }
    /* the status word and every copy above: one synchronisation */
    if (rc == YVEX_OK) {
        yvex_backend_operation_facts facts;
        memset(&facts, 0, sizeof(facts));
        rc = yvx_backend_status_collect(b, &facts, "cuda.attention.copy.status", run->err);
        run->work_pending = 0;
        run->d2h += facts.d2h_bytes;
        if (rc != YVEX_OK && run->failure) {
            run->failure->code = rc == YVEX_ERR_BACKEND ? YVEX_BACKEND_ATTENTION_FAILURE_SYNCHRONIZE
                                                       : YVEX_BACKEND_ATTENTION_FAILURE_NUMERIC;
            run->failure->stage = "cuda.attention.copy.status";
            run->failure->expected = 0ull;
            run->failure->actual = (unsigned long long)*b->status_host;
        }
    } else if (run->work_pending) {
        (void)yvx_cuda_stream_synchronize(b->stream);
        run->work_pending = 0;
        b->status_pending = 0;
    }
    if (rc == YVEX_OK) {
        o->tokens_executed = t;
        o->compressed_count = compressed ? run->compressed_new : 0ull;
        o->indexer_count = sparse ? run->compressed_new : 0ull;
    }
    if (rc == YVEX_OK && sparse) {
        /* per token: how many rows were visible, how many were selected, and where they lie */
        const unsigned long long ratio = job->compression_ratio;
        for (token = 0; token < t; ++token) {
            const unsigned long long position = job->token_position + token;
            const unsigned long long visible_new = (position + 1ull) / ratio - job->token_position / ratio;
            unsigned long long valid = 0ull;
            for (i = 0; i < job->compressed_count; ++i)
                if (job->compressed_positions[i] + ratio - 1ull <= position) valid++;
            valid += visible_new < run->compressed_new ? visible_new : run->compressed_new;
            if (o->valid_candidate_counts.data && token < o->valid_candidate_counts.capacity)
                o->valid_candidate_counts.data[token] = valid;
            if (o->topk_counts.data && token < o->topk_counts.capacity) o->topk_counts.data[token] = counts[token];
            if (valid > o->valid_candidate_count) o->valid_candidate_count = valid;
            if (counts[token] > o->topk_count) o->topk_count = counts[token];
            if (selected) {
                if (o->topk_positions.capacity < (token + 1ull) * run->topk_capacity) {
                    rc = job_fail(run, YVEX_BACKEND_ATTENTION_FAILURE_COPY, "cuda.attention.copy.selected",
                                  t * run->topk_capacity, o->topk_positions.capacity, YVEX_ERR_BOUNDS,
                                  "attention output span is smaller than the published extent");
                    break;
                }
                for (i = 0; i < counts[token]; ++i) {
                    const unsigned long long row = selected[token * run->topk_capacity + i];
                    o->topk_positions.data[token * run->topk_capacity + i] =
                        row < job->compressed_count
                            ? job->compressed_positions[row]
                            : (job->token_position / ratio + (row - job->compressed_count)) * ratio;
                }
            }
        }
    }
    free(counts);
    free(selected);
    return rc;
}

/* ---- entry points ----------------------------------------------------------------- */

int yvex_backend_attention_execute(yvex_backend *backend, const yvex_backend_attention_job *job,
                                   yvex_backend_attention_output *output,
                                   yvex_backend_attention_failure *failure, yvex_error *err)
{
    const char *where = "cuda.attention";
    job_run *run;
    int rc;
    if (failure) memset(failure, 0, sizeof(*failure));
    if (!backend || !job || !output) {
        if (failure) {
            failure->code = YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT;
            failure->stage = "cuda.attention.prepare";
            failure->expected = 1ull;
        }
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "backend, job and output are required");
    }
    rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) {
        if (failure) {
            failure->code = YVEX_BACKEND_ATTENTION_FAILURE_CAPABILITY;
            failure->stage = "cuda.attention.capability";
            failure->expected = 1ull;
        }
        return rc;
    }
    run = calloc(1, sizeof(*run));
    if (!run) return yvx_fail(err, YVEX_ERR_NOMEM, where, "attention job bookkeeping allocation failed");
    run->backend = backend;
    run->job = job;
    run->out = output;
    run->failure = failure;
    run->err = err;
    rc = job_admit(run);
    if (rc == YVEX_OK) rc = job_cancelled(run, "cuda.attention.cancel.before_dispatch");
    if (rc == YVEX_OK) rc = job_layout(run);
    if (rc == YVEX_OK) {
        rc = yvx_backend_status_arm(backend, where, err);
        if (rc != YVEX_OK && failure) {
            failure->code = YVEX_BACKEND_ATTENTION_FAILURE_LAUNCH;
            failure->stage = "cuda.attention.status";
            failure->expected = 1ull;
        }
    }
    if (rc == YVEX_OK) {
        run->work_pending = 1;
        rc = job_stage_inputs(run);
    }
    if (rc == YVEX_OK) rc = job_cancelled(run, "cuda.attention.cancel.after_allocation");
    if (rc == YVEX_OK) rc = job_project(run);
    if (rc == YVEX_OK) rc = job_cancelled(run, "cuda.attention.cancel.after_request");
    if (rc == YVEX_OK) rc = job_compress(run);
    if (rc == YVEX_OK) rc = job_cancelled(run, "cuda.attention.cancel.after_request");
    if (rc == YVEX_OK) rc = job_reduce(run);
    if (rc == YVEX_OK) rc = job_cancelled(run, "cuda.attention.cancel.before_commit");
    if (rc == YVEX_OK) rc = job_publish_outputs(run);
    if (rc != YVEX_OK && run->work_pending) {
        /* nothing may still read the arena when the caller sees the refusal */
        (void)yvx_cuda_stream_synchronize(backend->stream);
        backend->status_pending = 0;
    }
    if (rc == YVEX_OK) rc = job_cancelled(run, "cuda.attention.cancel.publish");
    output->kernel_launches = run->launches;
    output->accelerated_matrix_launches = 0ull;
    output->h2d_bytes = run->h2d;
    output->d2h_bytes = run->d2h;
    output->d2d_bytes = run->d2d;
    output->device_bytes = output->peak_device_bytes = run->device_bytes;
    output->device_state_staged_bytes = run->staged_state;
    output->device_state_staged = run->staged_state != 0ull;
    output->device_synchronizations = rc == YVEX_OK ? 1ull : 0ull;
    if (job->device_completion) {
        job->device_completion->pending = 0;
        job->device_completion->output = *output;
        if (failure) job->device_completion->failure = *failure;
    }
    free(run);
    if (rc == YVEX_OK) yvex_error_clear(err);
    return rc;
}

/* ---- residency mappings (src/backend/residency.c:24-207) ------------------------------- */

int yvex_backend_resident_attach(yvex_backend *backend, const unsigned char *host_base, unsigned long long bytes,
                                 const yvex_device_tensor *device_tensor, unsigned long long generation,
                                 yvex_error *err)
{
    const char *where = "backend.residency.attach";
    if (!backend || backend->failed || !host_base || !bytes || !device_tensor || !yvx_tensor_owned(backend, device_tensor) ||
        !device_tensor->bytes || !generation)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "a CUDA tensor of this backend covering the host range is required");
    if (backend->resident_host_base)
        return yvx_fail(err, YVEX_ERR_STATE, where, "backend residency mapping is already attached");
    if (device_tensor->bytes < bytes)
        return yvx_fail(err, YVEX_ERR_STATE, where, "the device tensor is smaller than the host range");
    backend->resident_host_base = host_base;
    backend->resident_host_bytes = bytes;
    backend->resident_device_address = (unsigned long long)(uintptr_t)device_tensor->data;
    backend->resident_generation = generation;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_resident_detach(yvex_backend *backend, yvex_error *err)
{
    if (backend) {
        backend->resident_host_base = NULL;
        backend->resident_host_bytes = backend->resident_device_address = backend->resident_generation = 0ull;
    }
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_resident_resolve(const yvex_backend *backend, const unsigned char *host, unsigned long long bytes,
                                  unsigned long long *device_address)
{
    unsigned long long offset;
    if (device_address) *device_address = 0ull;
    if (!backend || backend->failed || !host || !bytes || !device_address || !backend->resident_host_base ||
        (uintptr_t)host < (uintptr_t)backend->resident_host_base)
        return YVEX_BACKEND_RESIDENT_MISS;
    offset = (unsigned long long)((uintptr_t)host - (uintptr_t)backend->resident_host_base);
    if (offset > backend->resident_host_bytes || bytes > backend->resident_host_bytes - offset)
        return YVEX_BACKEND_RESIDENT_MISS;
    if (backend->resident_device_address > ULLONG_MAX - offset) return YVEX_BACKEND_RESIDENT_INVALID;
    *device_address = backend->resident_device_address + offset;
    return YVEX_BACKEND_RESIDENT_HIT;
}

int yvex_backend_state_residency_attach(yvex_backend *backend, const void *context,
                                        yvex_backend_state_resolve_fn resolve, unsigned long long generation,
                                        yvex_error *err)
{
    if (!backend || !context || !resolve || !generation)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, "backend.state.attach", "CUDA backend and complete state resolver are required");
    if (backend->state_residency_context)
        return yvx_fail(err, YVEX_ERR_STATE, "backend.state.attach", "backend state residency is already attached");
    backend->state_residency_context = context;
    backend->state_residency_resolve = resolve;
    backend->state_residency_generation = generation;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_state_residency_validate_generation(yvex_backend *backend, unsigned long long generation,
                                                     yvex_error *err)
{
    if (!backend || backend->failed || !generation)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, "backend.state.publish", "attached state owner and generation are required");
    if ((backend->state_residency_context == NULL) != (backend->state_residency_resolve == NULL))
        return yvx_fail(err, YVEX_ERR_STATE, "backend.state.publish", "state generation owner is partially attached");
    if (generation < backend->state_residency_generation)
        return yvx_fail(err, YVEX_ERR_STATE, "backend.state.publish", "state generation cannot regress");
    yvex_error_clear(err);
    return YVEX_OK;
}

void yvex_backend_state_residency_publish_generation(yvex_backend *backend, unsigned long long generation)
{
    if (backend) backend->state_residency_generation = generation;
}

void yvex_backend_state_residency_detach(yvex_backend *backend)
{
    if (!backend) return;
    backend->state_residency_context = NULL;
    backend->state_residency_resolve = NULL;
    backend->state_residency_generation = 0ull;
}

int yvex_backend_state_residency_resolve(const yvex_backend *backend, const void *host, unsigned long long bytes,
                                         unsigned long long *device_address)
{
    int result;
    if (device_address) *device_address = 0ull;
    if (!backend || !host || !bytes || !device_address || !backend->state_residency_context ||
        !backend->state_residency_resolve)
        return YVEX_BACKEND_RESIDENT_MISS;
    result = backend->state_residency_resolve(backend->state_residency_context, host, bytes, device_address);
    return result == YVEX_BACKEND_RESIDENT_HIT && !*device_address ? YVEX_BACKEND_RESIDENT_INVALID : result;
}

/* Drops every resident weight (a caller that rewrites or unloads weights calls this; nothing
 * may be in flight on the backend's stream). No counterpart in the reference. */
int yvex_b200_backend_weights_forget(yvex_backend *backend, yvex_error *err)
{
    unsigned int i;
    int rc = yvx_backend_admit(backend, "b200.weights.forget", err);
    if (rc != YVEX_OK) return rc;
    rc = yvx_cuda_device_synchronize();
    if (rc != 0) return yvx_backend_device_fail(backend, rc, "b200.weights.forget", err);
    for (i = 0; i < backend->weight_count; ++i) (void)yvx_cuda_free(backend->weights[i].device);
    backend->weight_count = 0u;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_b200_backend_projection_gemm(yvex_backend *backend, unsigned long long min_tokens, yvex_error *err)
{
    int rc = yvx_backend_admit(backend, "b200.projection.gemm", err);
    if (rc != YVEX_OK) return rc;
    backend->projection_gemm_tokens = min_tokens;
    yvex_error_clear(err);
    return YVEX_OK;
}

/* Deferred completion is refused at execute, so a completion object never has work
 * pending here: the call checks its arguments and reports that state. */
int yvex_backend_attention_complete(yvex_backend *backend, yvex_backend_attention_completion *completion,
                                    int barrier_observed, yvex_error *err)
{
    const char *where = "cuda.attention.complete";
    if (!backend || !completion) return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "backend and completion are required");
    if (completion->pending)
        return yvx_fail(err, YVEX_ERR_STATE, where, "no deferred attention work was issued by this backend");
    completion->barrier_observed = barrier_observed != 0;
    yvex_error_clear(err);
    return YVEX_OK;
}

/* ---- capability query --------------------------------------------------------------- */

static const char *const variant_names[YVEX_BACKEND_VARIANT_COUNT] = {
    "tensor-alloc", "tensor-zero", "tensor-write", "tensor-read", "tensor-copy", "embed-f32-to-f32",
    "embed-f16-to-f32", "rms-norm-f32-weight-f32", "rms-norm-f32-weight-f16", "rope-f32", "matmul-f32",
    "mlp-dense-f32", "mlp-routed-f32", "attention-causal-f32", "attention-noncausal-f32", "qtype-row-dot",
    "encoded-attention"};
static const char *const state_names[] = {"unsupported", "supported", "failed"};
static const char *const reason_names[] = {
    "none", "driver-unavailable", "device-unavailable", "context-unavailable", "kernel-bundle-absent",
    "kernel-bundle-rejected", "required-function-missing", "variant-unsupported", "launch-failed",
    "synchronization-failed", "cleanup-failed"};

const char *yvex_backend_operation_variant_name(yvex_backend_operation_variant variant)
{
    return (unsigned int)variant < YVEX_BACKEND_VARIANT_COUNT ? variant_names[variant] : "unknown";
}

const char *yvex_backend_capability_state_name(yvex_backend_capability_state state)
{
    return (unsigned int)state < sizeof(state_names) / sizeof(state_names[0]) ? state_names[state] : "unknown";
}

const char *yvex_backend_capability_reason_name(yvex_backend_capability_reason reason)
{
    return (unsigned int)reason < sizeof(reason_names) / sizeof(reason_names[0]) ? reason_names[reason] : "unknown";
}

int yvex_backend_query_capability(const yvex_backend *backend, yvex_backend_operation_variant variant,
                                  yvex_backend_capability_result *out, yvex_error *err)
{
    const char *where = "yvex_backend_query_capability";
    int built;
    if (!backend || !out) return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "backend and out are required");
    if ((int)variant < 0 || variant >= YVEX_BACKEND_VARIANT_COUNT)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "operation variant is out of range");
    memset(out, 0, sizeof(*out));
    out->backend_kind = YVEX_BACKEND_KIND_CUDA;
    out->variant = variant;
    out->context_available = 1;
    out->kernel_bundle_available = 1; /* the kernels are linked into the library */
    /* dtype projection of the reference's table (src/backend/core.c:48-73) */
    out->output_dtype = variant >= YVEX_BACKEND_VARIANT_EMBED_F32_TO_F32 ? YVEX_DTYPE_F32 : YVEX_DTYPE_UNKNOWN;
    if (variant >= YVEX_BACKEND_VARIANT_EMBED_F32_TO_F32 && variant <= YVEX_BACKEND_VARIANT_ATTENTION_NONCAUSAL_F32) {
        out->input_dtype = variant == YVEX_BACKEND_VARIANT_EMBED_F16_TO_F32 ? YVEX_DTYPE_F16 : YVEX_DTYPE_F32;
        out->weight_dtype = variant == YVEX_BACKEND_VARIANT_EMBED_F16_TO_F32 ||
                                    variant == YVEX_BACKEND_VARIANT_RMS_NORM_F32_WEIGHT_F16
                                ? YVEX_DTYPE_F16
                                : YVEX_DTYPE_F32;
    }
    built = variant <= YVEX_BACKEND_VARIANT_TENSOR_COPY || variant == YVEX_BACKEND_VARIANT_ATTENTION_CAUSAL_F32 ||
            variant == YVEX_BACKEND_VARIANT_ATTENTION_NONCAUSAL_F32 || variant == YVEX_BACKEND_VARIANT_QTYPE_ROW_DOT ||
            variant == YVEX_BACKEND_VARIANT_ATTENTION_ENCODED;
    if (backend->failed) {
        /* sticky: a failed launch or synchronisation closes every variant */
        out->state = YVEX_BACKEND_CAPABILITY_FAILED;
        out->reason = backend->failure_reason == 9 ? YVEX_BACKEND_CAPABILITY_REASON_SYNCHRONIZATION_FAILED
                                                   : YVEX_BACKEND_CAPABILITY_REASON_LAUNCH_FAILED;
    } else if (built) {
        out->state = YVEX_BACKEND_CAPABILITY_SUPPORTED;
        out->reason = YVEX_BACKEND_CAPABILITY_REASON_NONE;
        out->function_available = 1;
    } else {
        out->state = YVEX_BACKEND_CAPABILITY_UNSUPPORTED;
        out->reason = YVEX_BACKEND_CAPABILITY_REASON_VARIANT_UNSUPPORTED;
    }
    yvex_error_clear(err);
    return YVEX_OK;
}
