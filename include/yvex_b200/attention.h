/* Operator-level C-ABI of the B200 attention drop-in (libyvex_b200.so).
 *
 * These are the entry points the YVEX reference runtime binds for its
 * attention hot path, with the reference's names, argument meaning and error
 * behaviour; the citation beside each names the reference declaration it
 * replaces. Functions without a counterpart in the reference say so.
 *
 * There is no CPU backend behind this library and no fallback of any kind: if
 * no sm_100 device is usable, opening a backend fails and every operator
 * refuses with YVEX_ERR_UNSUPPORTED or YVEX_ERR_BACKEND.
 */
#ifndef YVEX_B200_ATTENTION_H
#define YVEX_B200_ATTENTION_H

#include "yvex_b200/abi.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- error helpers: include/yvex/core.h:42-48 ---------------------------- */
void yvex_error_clear(yvex_error *err);
void yvex_error_set(yvex_error *err, yvex_status code, const char *where, const char *message);
const char *yvex_status_name(yvex_status status);

/* ---- backend lifecycle and tensors: include/yvex/backend.h:148-206 -------- */
typedef enum {
    YVEX_BACKEND_KIND_CPU = 0,
    YVEX_BACKEND_KIND_CUDA,
    YVEX_BACKEND_KIND_METAL,
    YVEX_BACKEND_KIND_ROCM
} yvex_backend_kind;

typedef struct {
    yvex_backend_kind kind;
    const char *device;                 /* decimal device index, NULL = "0" */
    unsigned long long memory_limit_bytes;
} yvex_backend_options;

/* Only YVEX_BACKEND_KIND_CUDA opens; every other kind is refused with
 * YVEX_ERR_UNSUPPORTED (the reference's CPU backend has no exact-attention
 * table either: src/runtime/stateful_attention.c:294-298). */
int yvex_backend_open(yvex_backend **out, const yvex_backend_options *options, yvex_error *err);
int yvex_backend_close_checked(yvex_backend **backend, yvex_error *err);
void yvex_backend_close(yvex_backend *backend);
int yvex_backend_cuda_available(void);
int yvex_backend_sync(yvex_backend *backend, yvex_error *err);

int yvex_backend_tensor_alloc(yvex_backend *backend, const yvex_backend_tensor_desc *desc,
                              yvex_device_tensor **out, yvex_error *err);
int yvex_backend_tensor_release(yvex_backend *backend, yvex_device_tensor **tensor,
                                yvex_error *err);
void yvex_backend_tensor_free(yvex_backend *backend, yvex_device_tensor *tensor);
int yvex_backend_tensor_write(yvex_backend *backend, yvex_device_tensor *tensor,
                              const void *src, unsigned long long len, yvex_error *err);
int yvex_backend_tensor_read(yvex_backend *backend, const yvex_device_tensor *tensor,
                             void *dst, unsigned long long len, yvex_error *err);
int yvex_backend_tensor_zero(yvex_backend *backend, yvex_device_tensor *tensor, yvex_error *err);
/* include/yvex/internal/backend.h:258-260: an F32 window [offset, offset+count)
 * of a tensor, sharing its storage. Returns 1 on success, 0 on refusal. */
int yvex_backend_tensor_f32_subview(const yvex_device_tensor *source, unsigned long long offset,
                                    unsigned long long count, yvex_device_tensor *view);
/* No counterpart in the reference: wraps device memory the caller owns (for
 * instance a KV bank of the reference's state residency, or a framework
 * allocation) as a borrowed tensor of this backend. The wrapper is released
 * with yvex_backend_tensor_release; the memory is never freed by the library. */
int yvex_b200_tensor_wrap(yvex_backend *backend, const yvex_backend_tensor_desc *desc,
                          void *device_pointer, yvex_device_tensor **out, yvex_error *err);
/* No counterpart in the reference: binds the backend's operations to a CUDA
 * stream the caller owns (cudaStream_t as void*); NULL restores the backend's
 * own stream. `synchronous` = 0 makes operators return after enqueueing (the
 * status word is then checked by yvex_backend_sync). */
int yvex_b200_backend_bind_stream(yvex_backend *backend, void *stream, int synchronous,
                                  yvex_error *err);
void *yvex_b200_backend_stream(const yvex_backend *backend);
int yvex_b200_backend_sm_count(const yvex_backend *backend);

/* ---- exact attention operator: include/yvex/internal/transformer.h:291-294,
 * reached through yvex_backend_transformer_operations_get() in the reference
 * (src/backend/core.c:118; CUDA table src/backend/cuda/capability.c:21-42).
 * Implementation replaced: src/backend/cuda/exact_attention.c:55-108. ------- */
typedef struct yvex_b200_transformer_operations {
    int (*attention_workspace_required)(const yvex_transformer_attention_requirement *,
                                        unsigned long long *, yvex_error *);
    int (*attention_execute)(yvex_backend *, const yvex_transformer_attention_request *,
                             yvex_backend_operation_facts *, yvex_error *);
} yvex_b200_transformer_operations;

const yvex_b200_transformer_operations *yvex_b200_transformer_operations_get(
    const yvex_backend *backend);
int yvex_b200_transformer_attention_workspace_required(
    const yvex_transformer_attention_requirement *requirement, unsigned long long *bytes,
    yvex_error *err);
int yvex_b200_transformer_attention_execute(yvex_backend *backend,
                                            const yvex_transformer_attention_request *request,
                                            yvex_backend_operation_facts *facts,
                                            yvex_error *err);

/* ---- single-head primitive: include/yvex/backend.h:249-260 ---------------- */
int yvex_backend_op_attention(yvex_backend *backend, const yvex_device_tensor *query,
                              const yvex_device_tensor *keys, const yvex_device_tensor *values,
                              unsigned long long seq_len, unsigned long long position,
                              float scale, int causal, yvex_device_tensor *score_scratch,
                              yvex_device_tensor *probability_scratch, yvex_device_tensor *out,
                              yvex_error *err);

/* ---- batched attention over session KV caches (extension) ------------------
 * No counterpart in the reference, whose operator has no batch dimension, no
 * bf16 or Q8_0 KV and no block table. Per session the semantics are exactly
 * those of the exact attention operator above with query_start = kv length -
 * query rows (decode: 1 row; speculative verify: 2..8 rows, causal among
 * themselves). Unknown combinations are refused with YVEX_ERR_UNSUPPORTED. */
typedef enum {
    YVEX_B200_KV_CONTIGUOUS = 0, /* [session][token][kv_head*head_dim], strided */
    YVEX_B200_KV_BLOCK_TABLE = 1 /* pool of fixed-size token blocks + int32 table */
} yvex_b200_kv_layout;

typedef struct yvex_b200_attention_batch_request {
    /* heads, head_dimension, dtypes, mask, numeric_contract, deterministic are
     * read from here; query_tokens = rows per session; key_value_tokens = the
     * largest session length; query_start is ignored (taken from the end). */
    yvex_transformer_attention_requirement requirement;
    unsigned long long session_count;
    yvex_b200_kv_layout kv_layout;
    const yvex_device_tensor *query;   /* [session][row][query_heads*head_dim] */
    const yvex_device_tensor *key, *value; /* contiguous sessions or the pools */
    const yvex_device_tensor *kv_tokens;   /* I32 [session]: length of each session */
    const yvex_device_tensor *block_table; /* I32 [session][max_blocks]; block layout only */
    unsigned long long block_tokens;       /* tokens per pool block (64) */
    unsigned long long max_blocks_per_session;
    /* element strides; zero selects the packed default of the layout */
    unsigned long long kv_session_stride;  /* contiguous: elements between sessions */
    unsigned long long kv_block_stride;    /* block layout: elements between pool blocks */
    unsigned long long kv_head_stride;     /* elements between kv heads (default head_dim) */
    yvex_device_tensor *output;            /* [session][row][query_heads*head_dim] */
} yvex_b200_attention_batch_request;

int yvex_b200_attention_batch_execute(yvex_backend *backend,
                                      const yvex_b200_attention_batch_request *request,
                                      yvex_backend_operation_facts *facts, yvex_error *err);

/* ---- latent attention: the reduce stage of the encoded attention job ---------
 * The reference reaches this stage inside yvex_backend_attention_execute
 * (include/yvex/internal/backend.h:193-195; src/backend/cuda/attention.c:1386-1422).
 * The request names the job fields that stage consumes (include/yvex/internal/
 * backend.h:94-124): phase geometry, the phase's query, local window rows with
 * positions, compressed rows with positions, the selected lists of sparse
 * attention, and the per-head sinks. The failure record is the reference's
 * {code, stage, expected, actual} (include/yvex/internal/backend.h:144-161). */
typedef enum {
    YVEX_B200_ATTENTION_SWA = 0, /* window only */
    YVEX_B200_ATTENTION_CSA,     /* window + selected compressed rows */
    YVEX_B200_ATTENTION_HCA      /* window + every visible compressed row */
} yvex_b200_attention_class;
typedef enum {
    YVEX_B200_ATTENTION_FAILURE_NONE = 0,
    YVEX_B200_ATTENTION_FAILURE_INVALID_ARGUMENT,
    YVEX_B200_ATTENTION_FAILURE_CAPABILITY,
    YVEX_B200_ATTENTION_FAILURE_BUDGET,
    YVEX_B200_ATTENTION_FAILURE_ALLOCATION,
    YVEX_B200_ATTENTION_FAILURE_COPY,
    YVEX_B200_ATTENTION_FAILURE_LAUNCH,
    YVEX_B200_ATTENTION_FAILURE_SYNCHRONIZE,
    YVEX_B200_ATTENTION_FAILURE_NUMERIC
} yvex_b200_attention_failure_code;
typedef struct {
    yvex_b200_attention_failure_code code;
    const char *stage;
    unsigned long long expected, actual;
} yvex_b200_attention_failure;
typedef struct yvex_b200_attention_reduce_request {
    yvex_b200_attention_class attention_class;
    unsigned long long token_position, token_count;   /* first position and rows of this phase */
    unsigned long long query_heads, head_dimension;
    unsigned long long sliding_window, compression_ratio, indexer_topk;
    int candidate_block_visible;
    const yvex_device_tensor *query;                  /* F32 [token][heads*head_dim] */
    const yvex_device_tensor *local, *local_positions; /* F32 [local_count+token_count][local_stride], I64 */
    unsigned long long local_count, local_stride;     /* rows before this phase's own */
    const yvex_device_tensor *compressed, *compressed_positions; /* F32 [count][stride], I64 */
    unsigned long long compressed_count, compressed_stride;
    const yvex_device_tensor *selected, *selected_count; /* I64 [token][indexer_topk], I64 [token] */
    const yvex_device_tensor *sinks;                  /* F32 [heads] */
    yvex_device_tensor *output;                       /* F32 [token][heads*head_dim], bf16-rounded values */
    /* rope_frequency != NULL: the reference's inverse output rotation and second bf16
     * publication (src/graph/core.c:498-507) run in the same launch. */
    unsigned long long rope_dimension;
    const yvex_device_tensor *rope_frequency;         /* F64 [rope_dimension/2], radians per position */
} yvex_b200_attention_reduce_request;
/* The rotation frequencies of the reference's position policy
 * (attention_yarn_frequency, src/graph/numeric.c:877-917), computed on the host in
 * double precision: theta^(-2p/rope_dimension), blended with frequency/scaling_factor
 * over the ramp between the beta_fast and beta_slow correction dims when
 * original_context and scaling_factor are non-zero. frequency[rope_dimension/2]. */
typedef struct {
    unsigned long long theta, scaling_factor, original_context, beta_fast, beta_slow;
} yvex_b200_position_policy;
int yvex_b200_rope_frequencies(const yvex_b200_position_policy *policy,
                               unsigned long long rope_dimension, double *frequency);

/* The sparse index selection that feeds the reduce stage of class CSA: scores of
 * every compressed row against the phase's index queries and the ranked top-k rows
 * (CPU reference: yvex_attention_csa_select src/graph/attention.c:369-497,
 * yvex_attention_topk_select src/graph/numeric.c:1086-1150). selected /
 * selected_count are the tensors the reduce request takes. */
typedef struct yvex_b200_attention_select_request {
    unsigned long long token_position, token_count;
    unsigned long long indexer_heads, indexer_head_dimension, indexer_topk, compression_ratio;
    const yvex_device_tensor *index_keys;             /* F32 [count][key_stride], row i = compressed row i */
    const yvex_device_tensor *positions;              /* I64 [count], strictly increasing */
    unsigned long long count, key_stride;
    const yvex_device_tensor *index_query;            /* F32 [token][heads*head_dim] */
    const yvex_device_tensor *index_weights;          /* F32 [token][heads] */
    yvex_device_tensor *scores;                       /* F32 [token][count] */
    yvex_device_tensor *selected, *selected_count;    /* I64 [token][indexer_topk], I64 [token] */
} yvex_b200_attention_select_request;
int yvex_b200_attention_select_execute(yvex_backend *backend,
                                       const yvex_b200_attention_select_request *request,
                                       yvex_b200_attention_failure *failure,
                                       yvex_backend_operation_facts *facts, yvex_error *err);

/* The rolling compressor that produces the compressed rows (and, for the sparse
 * class, the index rows) the two stages above read: the state transition of every
 * token of a phase and the rows emitted on the way, published as the reference
 * publishes them (CPU reference: yvex_attention_rolling_state_step_cpu
 * src/graph/attention.c:745-836 driven by cpu_chunk_rolling_step
 * src/graph/attention_execute.c:730-832; CUDA: yvex_attention_rolling_state
 * src/backend/cuda/kernels.cu:1536-1631). kind and class decide the geometry as
 * yvex_attention_rolling_geometry does (src/graph/attention.c:500-528): main rows
 * have two halves for the sparse class only, index rows always. The projected token
 * rows (kv, score) and the additive position rows come from the caller's projection
 * stage; the quantising activation after the publication is the caller's too. */
typedef enum yvex_b200_rolling_kind {
    YVEX_B200_ROLLING_MAIN = 1,
    YVEX_B200_ROLLING_INDEXER = 2
} yvex_b200_rolling_kind;
typedef struct yvex_b200_attention_compress_request {
    yvex_b200_rolling_kind kind;
    yvex_b200_attention_class attention_class;        /* CSA or HCA */
    unsigned long long token_position, token_count;   /* the state has consumed token_position tokens */
    unsigned long long compression_ratio, head_dimension;  /* head dimension of this kind's rows */
    const yvex_device_tensor *token_kv, *token_score; /* F32 [token][token_stride] */
    unsigned long long token_stride;
    const yvex_device_tensor *position_rows;          /* F32 [ratio][state_width] */
    const yvex_device_tensor *state_kv, *state_score; /* F32 [state_slots][state_width] */
    yvex_device_tensor *next_state_kv, *next_state_score;
    const yvex_device_tensor *norm_weights;           /* F32 [head_dimension] */
    double rms_norm_epsilon;
    unsigned long long rope_dimension;                /* 0: no rotation */
    const yvex_device_tensor *rope_frequency;         /* F64 [rope_dimension/2] */
    yvex_device_tensor *compressed;                   /* F32 [emitted][head_dimension] */
    yvex_device_tensor *compressed_positions;         /* I64 [emitted] */
    unsigned long long emitted;                       /* out: rows written */
    /* The quantising activation the reference applies to each emitted row after the chain
     * (src/graph/attention_execute.c:807-818): 0 none, 8 FP8 E4M3, 4 FP4 E2M1; main rows
     * leave their rotated lanes alone, index rows are transformed and quantised whole. */
    unsigned int activation_quantization;
    unsigned long long activation_block_width;
    int activation_hadamard;
} yvex_b200_attention_compress_request;
int yvex_b200_attention_compress_execute(yvex_backend *backend,
                                         yvex_b200_attention_compress_request *request,
                                         yvex_b200_attention_failure *failure,
                                         yvex_backend_operation_facts *facts, yvex_error *err);

/* Activation fake quantisation in place over the first `count` lanes of `rows` rows of an
 * F32 tensor (yvex_attention_activation_apply, src/graph/core.c:829-945): what the
 * reference applies to new local rows, emitted compressed rows and index queries.
 * Refusals follow the reference: a count that is not a multiple of the block width is
 * YVEX_ERR_BOUNDS, an unknown quantisation YVEX_ERR_FORMAT, a non-finite lane YVEX_ERR_FORMAT. */
typedef struct yvex_b200_attention_activation_request {
    yvex_device_tensor *values;                       /* F32 [rows][row_stride] */
    unsigned long long rows, row_stride, count;
    unsigned int quantization;                        /* 8: FP8 E4M3, 4: FP4 E2M1 */
    unsigned long long block_width;
    int hadamard;
} yvex_b200_attention_activation_request;
int yvex_b200_attention_activation_execute(yvex_backend *backend,
                                           const yvex_b200_attention_activation_request *request,
                                           yvex_b200_attention_failure *failure,
                                           yvex_backend_operation_facts *facts, yvex_error *err);

/* The publication chain of projected rows (query heads, new local rows, index queries):
 * optional RMS norm -> bf16 -> optional rotation -> bf16 -> optional activation fake
 * quantisation, in one launch (CPU reference: src/graph/attention_execute.c:527-612 and
 * :970-1003; on the reference's device path a launch per step, src/backend/cuda/
 * attention.c:1162-1236). norm_mode: 0 none, 1 unit RMS norm, 2 learned weights. */
typedef struct yvex_b200_attention_publish_request {
    yvex_device_tensor *values;                       /* F32 [rows][row_stride] */
    unsigned long long rows, rows_per_token, row_stride, width;
    unsigned long long token_position;                /* position of the first token */
    int norm_mode;
    const yvex_device_tensor *norm_weights;           /* F32 [width] */
    double rms_norm_epsilon;
    unsigned long long rope_dimension;
    const yvex_device_tensor *rope_frequency;         /* F64 [rope_dimension/2] */
    unsigned int activation_quantization;             /* 0 none, 8, 4 */
    unsigned long long activation_count, activation_block_width;
    int activation_hadamard;
} yvex_b200_attention_publish_request;
int yvex_b200_attention_publish_execute(yvex_backend *backend,
                                        const yvex_b200_attention_publish_request *request,
                                        yvex_b200_attention_failure *failure,
                                        yvex_backend_operation_facts *facts, yvex_error *err);

int yvex_b200_attention_reduce_execute(yvex_backend *backend,
                                       const yvex_b200_attention_reduce_request *request,
                                       yvex_b200_attention_failure *failure,
                                       yvex_backend_operation_facts *facts, yvex_error *err);

/* ---- KV append + rotary for the new rows of a step ----------------------------
 * One call where the reference makes two rotate-half launches
 * (yvex_cuda_transformer_rotary_half, src/backend/cuda/transformer.c:449-457, from
 * src/runtime/decoder.c:1112-1131), two device copies per new token and a position
 * upload (src/runtime/stateful_attention.c:183-243). Refusals: geometry ->
 * YVEX_ERR_INVALID_ARG; views that are not packed F32 rows / explicit tables ->
 * YVEX_ERR_FORMAT (as src/backend/cuda/transformer.c:431-433); rows beyond the
 * admitted state view or block table -> YVEX_ERR_BOUNDS (as stateful_attention.c:
 * 203-206). */
typedef struct yvex_b200_kv_append_request {
    unsigned long long session_count, token_count;    /* new rows per session */
    unsigned long long query_heads, key_value_heads, head_dimension, rotary_dimension;
    int bf16_staged_products;                         /* 1: the decoder's rotary arithmetic */
    yvex_device_tensor *query;                        /* F32 [session][token][heads*hd], in place; may be NULL */
    const yvex_device_tensor *key, *value;            /* F32 [session][token][kv_heads*hd] */
    const yvex_device_tensor *cosines, *sines;        /* F32 [session][token][rotary_dimension] */
    const yvex_device_tensor *kv_tokens;              /* I32 [session] rows present; NULL: max_kv_tokens for all */
    unsigned long long max_kv_tokens;                 /* upper bound of every session's rows present */
    const yvex_device_tensor *token_position;         /* I64 [session]; NULL: position = row index */
    yvex_device_tensor *state_values;                 /* F32 [session][state_capacity][state_row_stride] or NULL */
    yvex_device_tensor *state_positions;              /* I64 [session][state_capacity] or NULL */
    unsigned long long state_capacity, state_row_stride;
    yvex_device_tensor *key_pool, *value_pool;        /* BF16 [block][block_tokens][kv_heads*hd] or NULL */
    const yvex_device_tensor *block_table;            /* I32 [session][max_blocks_per_session] */
    unsigned long long block_tokens, max_blocks_per_session, pool_blocks;
} yvex_b200_kv_append_request;
int yvex_b200_kv_append_rotary_execute(yvex_backend *backend, const yvex_b200_kv_append_request *request,
                                       yvex_backend_operation_facts *facts, yvex_error *err);

/* ---- latent decode with a separate rope key and an absorbed up-projection -------
 * No counterpart in the reference (its latent rows carry the rope dims inside the
 * 512 and serve as key and value). 128 heads, 128 nope, 512 latent, 64 rope dims;
 * any other geometry is refused with YVEX_ERR_UNSUPPORTED. */
typedef struct yvex_b200_mla_decode_request {
    unsigned long long session_count, heads, nope_dimension, latent_dimension, rope_dimension;
    unsigned long long context_capacity, max_kv_tokens;
    float scale;
    const yvex_device_tensor *q_nope, *q_rope;        /* BF16 [session][head][nope | rope] */
    const yvex_device_tensor *w_uk;                   /* BF16 [head][nope][latent] */
    const yvex_device_tensor *latent, *rope_key;      /* BF16 [session][context_capacity][latent | rope] */
    const yvex_device_tensor *kv_tokens;              /* I32 [session]; NULL: max_kv_tokens for all */
    yvex_device_tensor *output;                       /* F32 [session][head][latent] */
} yvex_b200_mla_decode_request;
int yvex_b200_mla_decode_execute(yvex_backend *backend, const yvex_b200_mla_decode_request *request,
                                 yvex_backend_operation_facts *facts, yvex_error *err);

/* ---- KV block and page indexing (integer, bit-exact) ------------------------
 * Page geometry follows include/yvex/internal/deployment.h:112-132 and
 * src/deployment/plan.c:208-283; page touch follows
 * src/graph/state_pages.c:660-669. The block-row map is this library's
 * extension (the reference keeps KV contiguous in virtual address space). */
typedef struct {
    unsigned long long logical_block_tokens, kernel_tile_tokens;
    unsigned long long promotion_granularity_tokens, alignment_bytes;
    unsigned long long bytes_per_block, page_table_entry_bytes;
    unsigned long long device_page_bytes, logical_tokens;
    int copy_on_write, candidate_extent;
} yvex_b200_page_request;
int yvex_b200_kv_page_tokens(const yvex_b200_page_request *request,
                             unsigned long long *page_tokens, unsigned long long *page_bytes);
int yvex_b200_kv_page_touch(unsigned long long element_start, unsigned long long element_count,
                            unsigned long long page_elements, unsigned long long *first_page,
                            unsigned long long *last_page);
/* KV-sequence sharding of one long session over `shards` GPUs (extension; the
 * reference is single-device): shard `index` owns the contiguous token range
 * [*begin, *end), boundaries aligned to `block_tokens`, sizes differing by at
 * most one block, empty ranges allowed when there are more shards than blocks.
 * Returns 1 on success, 0 on bad arguments. */
int yvex_b200_kv_sequence_shard(unsigned long long tokens, unsigned int shards, unsigned int index,
                                unsigned long long block_tokens, unsigned long long *begin,
                                unsigned long long *end);
/* The byte layout of one layer's state bank in the reference: per component the spans
 * [values, positions, auxiliary], each at the next 8-byte boundary of a running cursor
 * (src/runtime/state_residency.c:44-54, 346-395). A history component (history != 0) holds
 * capacity * value_width floats and capacity u64 positions; a rolling-compressor component
 * holds its kv-state floats as values and its score-state floats as auxiliary. This is the
 * payload layout the reference's checkpoints carry (src/runtime/state_store.c:1-9);
 * yvx_cuda_kv_bank_transfer moves a pooled session into it and back. Returns 1, or 0 on
 * overflow / bad arguments. */
typedef struct {
    int history;
    unsigned long long capacity, value_width;            /* history */
    unsigned long long kv_state_extent, score_state_extent; /* rolling */
} yvex_b200_kv_bank_component;
typedef struct {
    unsigned long long offset[3], bytes[3];              /* values, positions, auxiliary */
} yvex_b200_kv_bank_span;
int yvex_b200_kv_bank_layout(const yvex_b200_kv_bank_component *components, unsigned int count,
                             yvex_b200_kv_bank_span *spans, unsigned long long *bank_bytes);
/* ---- block pool bookkeeping (host side; extension) ----------------------------
 * Which pool blocks a session owns in the pooled KV layout, with shared prefixes
 * (fork), copy-on-write of a shared partial block, and the committed / candidate
 * split of speculative decoding. Stands where the reference keeps two banks per
 * layer and commits pages lazily (src/runtime/state_residency.c:346-483,
 * :678-776; candidate rows become visible through select_prefix,
 * src/graph/state.c:1329-1413). Rows [0, committed) are visible; reserve(n) makes
 * rows [committed, committed + n) writable (the session's own verify step may
 * read them: pass committed + n as its length); commit(accepted) moves the
 * boundary and forgets the rest. Status codes: YVEX_ERR_INVALID_ARG,
 * YVEX_ERR_BOUNDS (table or session slots exhausted), YVEX_ERR_NOMEM (pool full). */
typedef struct yvex_b200_kv_pool yvex_b200_kv_pool;
typedef struct {
    int needed;                       /* 1: copy rows [0, rows) of source into destination, K and V */
    int source_block, destination_block;
    unsigned int rows;
} yvex_b200_kv_copy;
yvex_b200_kv_pool *yvex_b200_kv_pool_create(unsigned int blocks, unsigned int block_tokens,
                                            unsigned int max_sessions, unsigned int max_blocks_per_session);
void yvex_b200_kv_pool_destroy(yvex_b200_kv_pool *pool);
int yvex_b200_kv_pool_session_open(yvex_b200_kv_pool *pool, unsigned int *session);
int yvex_b200_kv_pool_session_fork(yvex_b200_kv_pool *pool, unsigned int parent, unsigned int *child);
int yvex_b200_kv_pool_session_close(yvex_b200_kv_pool *pool, unsigned int session);
int yvex_b200_kv_pool_reserve(yvex_b200_kv_pool *pool, unsigned int session, unsigned int new_rows,
                              yvex_b200_kv_copy *copy);
int yvex_b200_kv_pool_commit(yvex_b200_kv_pool *pool, unsigned int session, unsigned int accepted_rows);
const int *yvex_b200_kv_pool_table(const yvex_b200_kv_pool *pool, unsigned int session);
unsigned long long yvex_b200_kv_pool_committed(const yvex_b200_kv_pool *pool, unsigned int session);
unsigned long long yvex_b200_kv_pool_reserved(const yvex_b200_kv_pool *pool, unsigned int session);
unsigned int yvex_b200_kv_pool_free_blocks(const yvex_b200_kv_pool *pool);
unsigned int yvex_b200_kv_pool_block_refcount(const yvex_b200_kv_pool *pool, unsigned int block);
unsigned long long yvex_b200_kv_block_row(const int *block_table,
                                          unsigned long long block_tokens,
                                          unsigned long long row);

#ifdef __cplusplus
}
#endif
#endif /* YVEX_B200_ATTENTION_H */
