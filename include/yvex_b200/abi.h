/* Shared ABI vocabulary of the B200 attention drop-in.
 *
 * Every type in this file mirrors, field for field, the type of the same name
 * in the YVEX reference tree so that a request built by the reference runtime
 * can be handed to this library unchanged. The citation beside each type names
 * the reference declaration it must stay layout-compatible with.
 */
#ifndef YVEX_B200_ABI_H
#define YVEX_B200_ABI_H

#ifdef __cplusplus
extern "C" {
#endif

/* Status vocabulary: include/yvex/core.h:13-26 in the reference. */
typedef enum {
    YVEX_OK = 0,
    YVEX_ERR = -1,
    YVEX_ERR_NOMEM = -2,
    YVEX_ERR_IO = -3,
    YVEX_ERR_FORMAT = -4,
    YVEX_ERR_UNSUPPORTED = -5,
    YVEX_ERR_BACKEND = -6,
    YVEX_ERR_BOUNDS = -7,
    YVEX_ERR_STATE = -8,
    YVEX_ERR_CANCELLED = -9,
    YVEX_ERR_INVALID_ARG = -10,
    YVEX_ERR_TIMEOUT = -11
} yvex_status;

/* Structured error: include/yvex/core.h:33-40. */
#define YVEX_ERROR_WHERE_CAP 96
#define YVEX_ERROR_MESSAGE_CAP 256
typedef struct {
    yvex_status code;
    char where[YVEX_ERROR_WHERE_CAP];
    char message[YVEX_ERROR_MESSAGE_CAP];
} yvex_error;

/* Dtype ids: include/yvex/model.h:19-36 (only the ids this path touches are
 * named; the numeric values are the reference's). */
typedef enum {
    YVEX_DTYPE_UNKNOWN = 0,
    YVEX_DTYPE_F32 = 1,
    YVEX_DTYPE_F16 = 2,
    YVEX_DTYPE_BF16 = 3,
    YVEX_DTYPE_F64 = 4,
    YVEX_DTYPE_I8 = 5,
    YVEX_DTYPE_I16 = 6,
    YVEX_DTYPE_I32 = 7,
    YVEX_DTYPE_I64 = 8,
    YVEX_DTYPE_Q8_0 = 13
} yvex_dtype;

#define YVEX_TENSOR_MAX_DIMS 4u /* include/yvex/model.h:85 */

typedef struct yvex_backend yvex_backend;

/* Borrowed device tensor: include/yvex/internal/backend.h:215-228. */
typedef struct yvex_device_tensor {
    yvex_backend *owner;
    unsigned long long owner_id;
    char *name;
    yvex_dtype dtype;
    unsigned int rank;
    unsigned long long dims[YVEX_TENSOR_MAX_DIMS];
    unsigned long long bytes;
    unsigned char *data, *host_data;
    void *backend_allocation;
    unsigned long long resident_bytes;
    int virtual_reserved;
    int is_written, host_accessible, borrowed_host;
} yvex_device_tensor;

/* Tensor descriptor: include/yvex/backend.h:46-52. */
typedef struct {
    const char *name;
    yvex_dtype dtype;
    unsigned int rank;
    unsigned long long dims[YVEX_TENSOR_MAX_DIMS];
    unsigned long long bytes;
} yvex_backend_tensor_desc;

/* Per-operation facts: include/yvex/internal/backend.h:284-290. */
typedef struct yvex_backend_operation_facts {
    unsigned long long h2d_bytes, d2h_bytes, d2d_bytes, kernel_launches, upload_count;
    unsigned long long download_count, queue_synchronizations, device_synchronizations;
    unsigned long long active_weight_bytes, state_bytes;
    unsigned long long activation_bytes, temporary_bytes, accelerated_matrix_launches;
    int compulsory_memory_facts_available;
} yvex_backend_operation_facts;

/* Exact-attention contract: include/yvex/internal/transformer.h:245-275. */
typedef enum {
    YVEX_TRANSFORMER_ATTENTION_LAYOUT_UNKNOWN = 0,
    YVEX_TRANSFORMER_ATTENTION_LAYOUT_TOKEN_HEAD_DIM
} yvex_transformer_attention_layout;

typedef enum {
    YVEX_TRANSFORMER_ATTENTION_MASK_UNKNOWN = 0,
    YVEX_TRANSFORMER_ATTENTION_MASK_FULL,
    YVEX_TRANSFORMER_ATTENTION_MASK_CAUSAL
} yvex_transformer_attention_mask;

/* The reference admits EXACT_F32 only. The two enumerators after it are
 * extensions of this library: they are refused by the reference and admitted
 * here only through the extension entry points in attention.h. */
typedef enum {
    YVEX_TRANSFORMER_ATTENTION_NUMERIC_UNKNOWN = 0,
    YVEX_TRANSFORMER_ATTENTION_NUMERIC_EXACT_F32 = 1,
    YVEX_TRANSFORMER_ATTENTION_NUMERIC_BF16_F32_ACCUMULATE = 2,
    YVEX_TRANSFORMER_ATTENTION_NUMERIC_Q8_0_KV_F32_ACCUMULATE = 3
} yvex_transformer_attention_numeric_contract;

typedef struct yvex_transformer_attention_requirement {
    unsigned long long query_tokens, key_value_tokens, query_start;
    unsigned long long query_heads, key_value_heads, head_dimension;
    /* Zero selects the packed row width; non-zero strides are elements per token. */
    unsigned long long query_token_stride, key_token_stride, value_token_stride;
    yvex_dtype query_dtype, key_dtype, value_dtype, output_dtype;
    yvex_transformer_attention_layout layout;
    yvex_transformer_attention_mask mask;
    yvex_transformer_attention_numeric_contract numeric_contract;
    int deterministic;
} yvex_transformer_attention_requirement;

typedef struct yvex_transformer_attention_request {
    yvex_transformer_attention_requirement requirement;
    const yvex_device_tensor *query, *key, *value;
    yvex_device_tensor *output;
} yvex_transformer_attention_request;

#ifdef __cplusplus
}
#endif
#endif /* YVEX_B200_ABI_H */
