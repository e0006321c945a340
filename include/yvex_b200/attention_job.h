/* The encoded (latent) attention job of the YVEX backend ABI, and the capability query.
 *
 * Every type here mirrors, field for field and value for value, the type of the same
 * name in the reference tree, so that a job built by the reference's graph layer
 * (src/graph/attention_execute.c:1440-1648) can be handed to this library unchanged:
 *   job schema 3, weights, position, activation, rolling state, spans, output, typed
 *   failure, deferred completion      include/yvex/internal/backend.h:17-180
 *   yvex_backend_attention_execute / _complete       include/yvex/internal/backend.h:193-198
 *   operation variants, capability state / reason / result, yvex_backend_query_capability
 *                                                    include/yvex/backend.h:77-129, 205-211
 * The two entry points and the query are exported under the reference's own names.
 */
#ifndef YVEX_B200_ATTENTION_JOB_H
#define YVEX_B200_ATTENTION_JOB_H

#include <stddef.h>

#include "yvex_b200/attention.h"

#ifdef __cplusplus
extern "C" {
#endif

#define YVEX_BACKEND_ATTENTION_JOB_SCHEMA 3u

typedef enum {
    YVEX_BACKEND_ATTENTION_WEIGHT_Q_A = 0,
    YVEX_BACKEND_ATTENTION_WEIGHT_Q_A_NORM,
    YVEX_BACKEND_ATTENTION_WEIGHT_Q_B,
    YVEX_BACKEND_ATTENTION_WEIGHT_KV,
    YVEX_BACKEND_ATTENTION_WEIGHT_KV_NORM,
    YVEX_BACKEND_ATTENTION_WEIGHT_SINKS,
    YVEX_BACKEND_ATTENTION_WEIGHT_OUT_A,
    YVEX_BACKEND_ATTENTION_WEIGHT_OUT_B,
    YVEX_BACKEND_ATTENTION_WEIGHT_MAIN_KV,
    YVEX_BACKEND_ATTENTION_WEIGHT_MAIN_GATE,
    YVEX_BACKEND_ATTENTION_WEIGHT_MAIN_APE,
    YVEX_BACKEND_ATTENTION_WEIGHT_MAIN_NORM,
    YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_KV,
    YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_GATE,
    YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_APE,
    YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_NORM,
    YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_Q,
    YVEX_BACKEND_ATTENTION_WEIGHT_INDEX_PROJECTION,
    YVEX_BACKEND_ATTENTION_WEIGHT_MHC_FUNCTION,
    YVEX_BACKEND_ATTENTION_WEIGHT_MHC_BASE,
    YVEX_BACKEND_ATTENTION_WEIGHT_MHC_SCALE,
    YVEX_BACKEND_ATTENTION_WEIGHT_INPUT_NORM,
    YVEX_BACKEND_ATTENTION_WEIGHT_COUNT
} yvex_backend_attention_weight_slot;

typedef struct {
    const unsigned char *encoded;
    size_t encoded_bytes;
    unsigned long long row_bytes, row_width, row_count;
    unsigned int qtype;
    int present;
} yvex_backend_attention_weight;

typedef struct {
    unsigned long long theta, scaling_factor, original_context;
    unsigned long long beta_fast, beta_slow, rope_dimensions;
} yvex_backend_attention_position;

typedef struct {
    int required;
    unsigned long long block_width;
    unsigned int quantization;
    int hadamard;
} yvex_backend_attention_activation;

typedef enum {
    YVEX_BACKEND_ATTENTION_SWA = 0,
    YVEX_BACKEND_ATTENTION_CSA,
    YVEX_BACKEND_ATTENTION_HCA
} yvex_backend_attention_class;

typedef enum {
    YVEX_BACKEND_ATTENTION_COMPUTE_UNKNOWN = 0,
    YVEX_BACKEND_ATTENTION_COMPUTE_BF16_F32_RNE_V1
} yvex_backend_attention_compute;

typedef enum {
    YVEX_BACKEND_ATTENTION_SCOPE_CORE = 0,
    YVEX_BACKEND_ATTENTION_SCOPE_ENVELOPE
} yvex_backend_attention_scope;

typedef enum {
    YVEX_BACKEND_ATTENTION_PHASE_PREFILL = 0,
    YVEX_BACKEND_ATTENTION_PHASE_DECODE = 1,
    YVEX_BACKEND_ATTENTION_PHASE_SPECULATIVE_DRAFT = 2,
    YVEX_BACKEND_ATTENTION_PHASE_SPECULATIVE_VERIFY = 3,
    YVEX_BACKEND_ATTENTION_PHASE_MIXED = 6,
    YVEX_BACKEND_ATTENTION_PHASE_COUNT = 7
} yvex_backend_attention_phase;

typedef int (*yvex_backend_cancelled_fn)(void *context);
typedef struct {
    yvex_backend_cancelled_fn requested;
    void *context;
} yvex_backend_cancellation;
typedef struct {
    float *data;
    unsigned long long capacity;
} yvex_backend_float_span;
typedef struct {
    unsigned long long *data, capacity;
} yvex_backend_u64_span;
typedef struct yvex_backend_attention_completion yvex_backend_attention_completion;

typedef struct {
    int present, overlap;
    unsigned long long next_token_position, ratio, head_dimension, state_width, state_slots;
    unsigned long long cursor, previous_fill, current_fill;
    const float *kv_state, *score_state;
    unsigned long long kv_state_capacity, score_state_capacity;
} yvex_backend_attention_rolling;

typedef struct {
    unsigned int schema;
    yvex_backend_attention_phase phase;
    yvex_backend_attention_class attention_class;
    yvex_backend_attention_compute compute_contract;
    yvex_backend_attention_scope operation_scope;
    unsigned long long token_position, token_count, input_stride;
    unsigned long long hidden_width, q_rank, query_heads, head_dimension, kv_width;
    unsigned long long sliding_window, compression_ratio;
    unsigned long long output_groups, output_group_input_width, output_rank;
    unsigned long long indexer_heads, indexer_head_dimension, indexer_topk;
    unsigned long long residual_stream_count, residual_stream_width, residual_expanded_width;
    unsigned long long mhc_mixing_rows, mhc_sinkhorn_iterations;
    double rms_epsilon, mhc_epsilon, mhc_residual_post_multiplier;
    yvex_backend_attention_position position;
    yvex_backend_attention_activation attention_kv_activation, compressor_activation;
    yvex_backend_attention_activation compressor_rotated_activation, indexer_query_activation;
    yvex_backend_attention_weight weights[YVEX_BACKEND_ATTENTION_WEIGHT_COUNT];
    const float *input, *local_kv, *compressed_kv, *indexer_kv;
    const yvex_device_tensor *device_input;
    yvex_device_tensor *device_output;
    const unsigned long long *local_positions, *compressed_positions, *indexer_positions;
    unsigned long long local_count, local_stride, compressed_count, compressed_stride;
    unsigned long long indexer_count, indexer_stride;
    yvex_backend_attention_rolling main_rolling, indexer_rolling;
    const yvex_backend_cancellation *cancellation;
    yvex_backend_attention_completion *device_completion;
    unsigned int evidence_level;
    int measure_device_time;
    int candidate_block_visible, retain_prefix_checkpoints, native_execution;
    unsigned long long max_host_bytes, max_device_bytes;
} yvex_backend_attention_job;

typedef struct {
    yvex_backend_float_span core_input, q_low, query, raw_kv;
    yvex_backend_float_span compressed_kv, indexer_kv, index_query, index_weights;
    yvex_backend_float_span attention_values, output, envelope_output;
    yvex_backend_u64_span compressed_positions, indexer_positions, topk_positions;
    yvex_backend_u64_span topk_counts, valid_candidate_counts;
    yvex_backend_float_span main_kv_state, main_score_state;
    yvex_backend_float_span indexer_kv_state, indexer_score_state;
    unsigned long long tokens_executed, compressed_count, indexer_count;
    unsigned long long topk_count, valid_candidate_count;
    unsigned long long host_bytes, peak_host_bytes, device_bytes, peak_device_bytes;
    unsigned long long kernel_launches, accelerated_matrix_launches;
    unsigned long long h2d_bytes, d2h_bytes, d2d_bytes;
    unsigned long long device_state_staged_bytes;
    unsigned long long queue_synchronizations, device_synchronizations;
    unsigned long long device_execution_elapsed_ns, host_workspace_capacity;
    unsigned long long host_workspace_used, host_workspace_peak, host_workspace_allocation_count;
    int host_workspace_reused, device_state_staged;
} yvex_backend_attention_output;

typedef enum {
    YVEX_BACKEND_ATTENTION_FAILURE_NONE = 0,
    YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT,
    YVEX_BACKEND_ATTENTION_FAILURE_CAPABILITY,
    YVEX_BACKEND_ATTENTION_FAILURE_BUDGET,
    YVEX_BACKEND_ATTENTION_FAILURE_ALLOCATION,
    YVEX_BACKEND_ATTENTION_FAILURE_COPY,
    YVEX_BACKEND_ATTENTION_FAILURE_LAUNCH,
    YVEX_BACKEND_ATTENTION_FAILURE_SYNCHRONIZE,
    YVEX_BACKEND_ATTENTION_FAILURE_NUMERIC,
    YVEX_BACKEND_ATTENTION_FAILURE_CANCELLED,
    YVEX_BACKEND_ATTENTION_FAILURE_CLEANUP
} yvex_backend_attention_failure_code;

typedef struct {
    yvex_backend_attention_failure_code code;
    const char *stage;
    unsigned long long expected, actual;
} yvex_backend_attention_failure;

#define YVEX_BACKEND_ATTENTION_COMPLETION_TRANSFER_CAP 20u
typedef struct {
    void *output, *staged;
    unsigned long long capacity, output_capacity, used;
    size_t width;
    const char *stage;
} yvex_backend_attention_completion_transfer;

struct yvex_backend_attention_completion {
    int defer, stack_start, pending, barrier_observed;
    yvex_backend_attention_output output;
    yvex_backend_attention_failure failure;
    int *host_status;
    unsigned long long *host_selected_counts, *host_candidate_counts;
    unsigned int attention_class;
    unsigned long long token_count, indexer_topk, candidate_capacity;
    unsigned int transfer_count;
    yvex_backend_attention_completion_transfer transfers[YVEX_BACKEND_ATTENTION_COMPLETION_TRANSFER_CAP];
};

/* One encoded attention operation: projections, compression, selection, the shared-latent
 * reduce and the output projections of job->token_count tokens. Every span of `output`
 * whose data pointer is set receives that intermediate (capacity in elements is checked);
 * the counters are always filled. On a refusal `failure` names the stage in the
 * reference's vocabulary ("cuda.attention.<stage>"). */
int yvex_backend_attention_execute(yvex_backend *backend, const yvex_backend_attention_job *job,
                                   yvex_backend_attention_output *output,
                                   yvex_backend_attention_failure *failure, yvex_error *err);
/* Finishes a job that was executed with a deferred completion object. */
int yvex_backend_attention_complete(yvex_backend *backend,
                                    yvex_backend_attention_completion *completion,
                                    int barrier_observed, yvex_error *err);

/* ---- residency: the runtime's device copies of weights and of session state -------------
 * include/yvex/internal/backend.h:200-202, 275-283, 315-322; src/backend/residency.c:24-207.
 * The reference's runtime owns a device arena of weights and device banks of session state
 * and tells the backend how host addresses map into them. With these attached, a job's
 * weights are read where they lie (no upload) and its histories and rolling states are
 * copied on the device instead of over PCIe. resolve returns HIT, MISS (outside every
 * mapping: the job uploads) or INVALID. The backend owns none of the memory. */
typedef int (*yvex_backend_state_resolve_fn)(const void *context, const void *host, unsigned long long bytes,
                                             unsigned long long *device_address);
typedef enum {
    YVEX_BACKEND_RESIDENT_INVALID = -1,
    YVEX_BACKEND_RESIDENT_MISS = 0,
    YVEX_BACKEND_RESIDENT_HIT = 1
} yvex_backend_resident_result;
int yvex_backend_resident_attach(yvex_backend *backend, const unsigned char *host_base, unsigned long long bytes,
                                 const yvex_device_tensor *device_tensor, unsigned long long generation,
                                 yvex_error *err);
int yvex_backend_resident_detach(yvex_backend *backend, yvex_error *err);
int yvex_backend_resident_resolve(const yvex_backend *backend, const unsigned char *host, unsigned long long bytes,
                                  unsigned long long *device_address);
int yvex_backend_state_residency_attach(yvex_backend *backend, const void *context,
                                        yvex_backend_state_resolve_fn resolve, unsigned long long generation,
                                        yvex_error *err);
int yvex_backend_state_residency_validate_generation(yvex_backend *backend, unsigned long long generation,
                                                     yvex_error *err);
void yvex_backend_state_residency_publish_generation(yvex_backend *backend, unsigned long long generation);
void yvex_backend_state_residency_detach(yvex_backend *backend);
int yvex_backend_state_residency_resolve(const yvex_backend *backend, const void *host, unsigned long long bytes,
                                         unsigned long long *device_address);

/* No counterpart in the reference. The job keeps encoded weights resident on the device,
 * found again by host address, size and a sampled content fingerprint; a caller that
 * rewrites weights in place, or unloads a model, drops them with this call. */
int yvex_b200_backend_weights_forget(yvex_backend *backend, yvex_error *err);
/* Jobs of at least `min_tokens` tokens run their published row projections (q_a, q_b, kv,
 * out_a, out_b) with BF16 weights on the tensor cores (yvx_cuda_bf16_gemm): a published value
 * is then within one bf16 step of the exact sum instead of equal to it. 0 (the default): never.
 * No reference counterpart (its CUDA projections are one matvec launch per token tile). */
int yvex_b200_backend_projection_gemm(yvex_backend *backend, unsigned long long min_tokens, yvex_error *err);

/* ---- capability query ----------------------------------------------------------- */
typedef enum {
    YVEX_BACKEND_VARIANT_TENSOR_ALLOC = 0,
    YVEX_BACKEND_VARIANT_TENSOR_ZERO,
    YVEX_BACKEND_VARIANT_TENSOR_WRITE,
    YVEX_BACKEND_VARIANT_TENSOR_READ,
    YVEX_BACKEND_VARIANT_TENSOR_COPY,
    YVEX_BACKEND_VARIANT_EMBED_F32_TO_F32,
    YVEX_BACKEND_VARIANT_EMBED_F16_TO_F32,
    YVEX_BACKEND_VARIANT_RMS_NORM_F32_WEIGHT_F32,
    YVEX_BACKEND_VARIANT_RMS_NORM_F32_WEIGHT_F16,
    YVEX_BACKEND_VARIANT_ROPE_F32,
    YVEX_BACKEND_VARIANT_MATMUL_F32,
    YVEX_BACKEND_VARIANT_MLP_DENSE_F32,
    YVEX_BACKEND_VARIANT_MLP_ROUTED_F32,
    YVEX_BACKEND_VARIANT_ATTENTION_CAUSAL_F32,
    YVEX_BACKEND_VARIANT_ATTENTION_NONCAUSAL_F32,
    YVEX_BACKEND_VARIANT_QTYPE_ROW_DOT,
    YVEX_BACKEND_VARIANT_ATTENTION_ENCODED,
    YVEX_BACKEND_VARIANT_COUNT
} yvex_backend_operation_variant;

typedef enum {
    YVEX_BACKEND_CAPABILITY_UNSUPPORTED = 0,
    YVEX_BACKEND_CAPABILITY_SUPPORTED,
    YVEX_BACKEND_CAPABILITY_FAILED
} yvex_backend_capability_state;

typedef enum {
    YVEX_BACKEND_CAPABILITY_REASON_NONE = 0,
    YVEX_BACKEND_CAPABILITY_REASON_DRIVER_UNAVAILABLE,
    YVEX_BACKEND_CAPABILITY_REASON_DEVICE_UNAVAILABLE,
    YVEX_BACKEND_CAPABILITY_REASON_CONTEXT_UNAVAILABLE,
    YVEX_BACKEND_CAPABILITY_REASON_KERNEL_BUNDLE_ABSENT,
    YVEX_BACKEND_CAPABILITY_REASON_KERNEL_BUNDLE_REJECTED,
    YVEX_BACKEND_CAPABILITY_REASON_FUNCTION_MISSING,
    YVEX_BACKEND_CAPABILITY_REASON_VARIANT_UNSUPPORTED,
    YVEX_BACKEND_CAPABILITY_REASON_LAUNCH_FAILED,
    YVEX_BACKEND_CAPABILITY_REASON_SYNCHRONIZATION_FAILED,
    YVEX_BACKEND_CAPABILITY_REASON_CLEANUP_FAILED
} yvex_backend_capability_reason;

typedef struct {
    yvex_backend_kind backend_kind;
    yvex_backend_operation_variant variant;
    yvex_backend_capability_state state;
    yvex_backend_capability_reason reason;
    yvex_dtype input_dtype;
    yvex_dtype weight_dtype;
    yvex_dtype output_dtype;
    int context_available;
    int kernel_bundle_available;
    int function_available;
} yvex_backend_capability_result;

/* Truthful per-variant capability (fail-closed logic of the reference:
 * src/backend/core.c:905-945, src/backend/cuda/capability.c:662-713). SUPPORTED only for
 * what this library implements on the device: the tensor variants, the single-head
 * attention primitive (causal and non-causal), the encoded row dot and the encoded
 * attention job; every other variant is UNSUPPORTED with reason VARIANT_UNSUPPORTED, and
 * after a failed launch or synchronisation every variant reads FAILED with that reason. */
int yvex_backend_query_capability(const yvex_backend *backend, yvex_backend_operation_variant variant,
                                  yvex_backend_capability_result *out, yvex_error *err);
const char *yvex_backend_operation_variant_name(yvex_backend_operation_variant variant);
const char *yvex_backend_capability_state_name(yvex_backend_capability_state state);
const char *yvex_backend_capability_reason_name(yvex_backend_capability_reason reason);

#ifdef __cplusplus
}
#endif
#endif /* YVEX_B200_ATTENTION_JOB_H */
