"""ctypes mirror of include/yvex_b200/*.h: the C-ABI of libyvex_b200.so.

Loading fails loudly when the shared library has not been built; nothing in
this package can compute on the host.
"""
import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# YVEX_B200_LIBRARY=checked selects the build with index checks compiled in (clori_b200/_build.py).
LIB_PATH = os.path.join(PKG, "libyvex_b200_checked.so" if os.environ.get("YVEX_B200_LIBRARY") == "checked"
                        else "libyvex_b200.so")

# yvex_status (include/yvex_b200/abi.h)
YVEX_OK = 0
YVEX_ERR = -1
YVEX_ERR_NOMEM = -2
YVEX_ERR_IO = -3
YVEX_ERR_FORMAT = -4
YVEX_ERR_UNSUPPORTED = -5
YVEX_ERR_BACKEND = -6
YVEX_ERR_BOUNDS = -7
YVEX_ERR_STATE = -8
YVEX_ERR_CANCELLED = -9
YVEX_ERR_INVALID_ARG = -10
YVEX_ERR_TIMEOUT = -11

# yvex_dtype
DTYPE_F32, DTYPE_F16, DTYPE_BF16, DTYPE_F64 = 1, 2, 3, 4
DTYPE_I8, DTYPE_I16, DTYPE_I32, DTYPE_I64 = 5, 6, 7, 8
DTYPE_Q8_0 = 13
DTYPE_BYTES = {DTYPE_F32: 4, DTYPE_F16: 2, DTYPE_BF16: 2, DTYPE_F64: 8, DTYPE_I8: 1,
               DTYPE_I16: 2, DTYPE_I32: 4, DTYPE_I64: 8}

LAYOUT_TOKEN_HEAD_DIM = 1
MASK_FULL, MASK_CAUSAL = 1, 2
NUMERIC_EXACT_F32 = 1
NUMERIC_BF16_F32_ACCUMULATE = 2
NUMERIC_Q8_0_KV_F32_ACCUMULATE = 3
BACKEND_KIND_CPU, BACKEND_KIND_CUDA = 0, 1
KV_CONTIGUOUS, KV_BLOCK_TABLE = 0, 1
MAX_DIMS = 4
u64 = C.c_ulonglong


class Error(C.Structure):
    _fields_ = [("code", C.c_int), ("where", C.c_char * 96), ("message", C.c_char * 256)]


class DeviceTensor(C.Structure):
    _fields_ = [
        ("owner", C.c_void_p), ("owner_id", u64), ("name", C.c_char_p), ("dtype", C.c_int),
        ("rank", C.c_uint), ("dims", u64 * MAX_DIMS), ("bytes", u64), ("data", C.c_void_p),
        ("host_data", C.c_void_p), ("backend_allocation", C.c_void_p), ("resident_bytes", u64),
        ("virtual_reserved", C.c_int), ("is_written", C.c_int), ("host_accessible", C.c_int),
        ("borrowed_host", C.c_int),
    ]


class TensorDesc(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_int), ("rank", C.c_uint),
                ("dims", u64 * MAX_DIMS), ("bytes", u64)]


class OperationFacts(C.Structure):
    _fields_ = [(n, u64) for n in (
        "h2d_bytes", "d2h_bytes", "d2d_bytes", "kernel_launches", "upload_count",
        "download_count", "queue_synchronizations", "device_synchronizations",
        "active_weight_bytes", "state_bytes", "activation_bytes", "temporary_bytes",
        "accelerated_matrix_launches")] + [("compulsory_memory_facts_available", C.c_int)]


class AttentionRequirement(C.Structure):
    _fields_ = [(n, u64) for n in (
        "query_tokens", "key_value_tokens", "query_start", "query_heads", "key_value_heads",
        "head_dimension", "query_token_stride", "key_token_stride", "value_token_stride")] + [
        ("query_dtype", C.c_int), ("key_dtype", C.c_int), ("value_dtype", C.c_int),
        ("output_dtype", C.c_int), ("layout", C.c_int), ("mask", C.c_int),
        ("numeric_contract", C.c_int), ("deterministic", C.c_int)]


class AttentionRequest(C.Structure):
    _fields_ = [("requirement", AttentionRequirement), ("query", C.POINTER(DeviceTensor)),
                ("key", C.POINTER(DeviceTensor)), ("value", C.POINTER(DeviceTensor)),
                ("output", C.POINTER(DeviceTensor))]


class BackendOptions(C.Structure):
    _fields_ = [("kind", C.c_int), ("device", C.c_char_p), ("memory_limit_bytes", u64)]


WORKSPACE_FN = C.CFUNCTYPE(C.c_int, C.POINTER(AttentionRequirement), C.POINTER(u64),
                           C.POINTER(Error))
EXECUTE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(AttentionRequest),
                         C.POINTER(OperationFacts), C.POINTER(Error))


class TransformerOperations(C.Structure):
    _fields_ = [("attention_workspace_required", WORKSPACE_FN),
                ("attention_execute", EXECUTE_FN)]


class BatchRequest(C.Structure):
    _fields_ = [("requirement", AttentionRequirement), ("session_count", u64),
                ("kv_layout", C.c_int), ("query", C.POINTER(DeviceTensor)),
                ("key", C.POINTER(DeviceTensor)), ("value", C.POINTER(DeviceTensor)),
                ("kv_tokens", C.POINTER(DeviceTensor)), ("block_table", C.POINTER(DeviceTensor)),
                ("block_tokens", u64), ("max_blocks_per_session", u64),
                ("kv_session_stride", u64), ("kv_block_stride", u64), ("kv_head_stride", u64),
                ("output", C.POINTER(DeviceTensor))]


class PageRequest(C.Structure):
    _fields_ = [(n, u64) for n in (
        "logical_block_tokens", "kernel_tile_tokens", "promotion_granularity_tokens",
        "alignment_bytes", "bytes_per_block", "page_table_entry_bytes", "device_page_bytes",
        "logical_tokens")] + [("copy_on_write", C.c_int), ("candidate_extent", C.c_int)]


class GqaProblem(C.Structure):
    """yvx_gqa_problem (include/yvex_b200/cuda_shim.h)."""
    _fields_ = [
        ("sessions", C.c_uint), ("query_rows", C.c_uint), ("query_heads", C.c_uint),
        ("kv_heads", C.c_uint), ("head_dim", C.c_uint), ("causal", C.c_uint),
        ("scale", C.c_float), ("query_dtype", C.c_int), ("kv_dtype", C.c_int),
        ("output_dtype", C.c_int),
        ("query", C.c_void_p), ("query_row_stride", u64), ("query_session_stride", u64),
        ("output", C.c_void_p),
        ("key", C.c_void_p), ("value", C.c_void_p),
        ("key_token_stride", u64), ("value_token_stride", u64),
        ("key_head_stride", u64), ("value_head_stride", u64),
        ("key_session_stride", u64), ("value_session_stride", u64),
        ("block_table", C.c_void_p), ("block_tokens", C.c_uint), ("block_table_stride", C.c_uint),
        ("pool_blocks", C.c_uint),
        ("key_block_stride", u64), ("value_block_stride", u64),
        ("kv_tokens", C.c_void_p), ("kv_tokens_uniform", C.c_uint), ("kv_tokens_max", C.c_uint),
        ("query_start", C.c_void_p), ("query_start_uniform", C.c_uint),
        ("query_start_from_end", C.c_uint), ("kv_position_base", C.c_uint),
        ("chunk_tokens", C.c_uint), ("max_splits", C.c_uint),
        ("partials", C.c_void_p), ("partial_output", C.c_void_p), ("status", C.c_void_p),
        ("force_general", C.c_int), ("query_head_stride", u64),
        ("f32_staging", C.c_void_p), ("gate", C.c_void_p), ("gate_value", C.c_int), ("tickets", C.c_void_p),
    ]


class LatentReduceArgs(C.Structure):
    """yvx_latent_reduce_args (include/yvex_b200/cuda_shim.h); the CPU checker's argument
    struct has the same layout."""
    _fields_ = [
        ("query", C.c_void_p), ("local", C.c_void_p), ("local_positions", C.c_void_p),
        ("initial_local_count", u64), ("local_stride", u64),
        ("compressed", C.c_void_p), ("compressed_positions", C.c_void_p), ("compressed_stride", u64),
        ("selected", C.c_void_p), ("selected_count", C.c_void_p), ("topk_capacity", u64),
        ("sinks", C.c_void_p), ("query_heads", u64), ("head_dim", u64), ("sliding_window", u64),
        ("ratio", u64), ("attention_class", C.c_uint), ("phase_start_position", u64),
        ("token_count", u64), ("candidate_block_visible", C.c_int),
        ("out", C.c_void_p), ("status", C.c_void_p),
        ("rope_dims", u64), ("rope_frequency", C.c_void_p), ("workspace", C.c_void_p),
    ]


class LseExchange(C.Structure):
    """yvx_lse_exchange (include/yvex_b200/cuda_shim.h)."""
    _fields_ = [("ranks", C.c_uint), ("rank", C.c_uint), ("epoch", C.c_uint),
                ("gather", C.c_void_p), ("arrivals", C.c_void_p), ("one_launch", C.c_int),
                ("tagged_words", C.c_int)]


class KvCopy(C.Structure):
    """yvex_b200_kv_copy (include/yvex_b200/attention.h)."""
    _fields_ = [("needed", C.c_int), ("source_block", C.c_int), ("destination_block", C.c_int),
                ("rows", C.c_uint)]


class AttentionFailure(C.Structure):
    """yvex_b200_attention_failure (include/yvex_b200/attention.h)."""
    _fields_ = [("code", C.c_int), ("stage", C.c_char_p), ("expected", u64), ("actual", u64)]


class AttentionReduceRequest(C.Structure):
    """yvex_b200_attention_reduce_request (include/yvex_b200/attention.h)."""
    _fields_ = [
        ("attention_class", C.c_int), ("token_position", u64), ("token_count", u64),
        ("query_heads", u64), ("head_dimension", u64),
        ("sliding_window", u64), ("compression_ratio", u64), ("indexer_topk", u64),
        ("candidate_block_visible", C.c_int),
        ("query", C.c_void_p), ("local", C.c_void_p), ("local_positions", C.c_void_p),
        ("local_count", u64), ("local_stride", u64),
        ("compressed", C.c_void_p), ("compressed_positions", C.c_void_p),
        ("compressed_count", u64), ("compressed_stride", u64),
        ("selected", C.c_void_p), ("selected_count", C.c_void_p),
        ("sinks", C.c_void_p), ("output", C.c_void_p),
        ("rope_dimension", u64), ("rope_frequency", C.c_void_p),
    ]


class PositionPolicy(C.Structure):
    """yvex_b200_position_policy (include/yvex_b200/attention.h)."""
    _fields_ = [(name, u64) for name in ("theta", "scaling_factor", "original_context", "beta_fast", "beta_slow")]


class AttentionSelectRequest(C.Structure):
    """yvex_b200_attention_select_request (include/yvex_b200/attention.h)."""
    _fields_ = [
        ("token_position", u64), ("token_count", u64),
        ("indexer_heads", u64), ("indexer_head_dimension", u64), ("indexer_topk", u64), ("compression_ratio", u64),
        ("index_keys", C.c_void_p), ("positions", C.c_void_p), ("count", u64), ("key_stride", u64),
        ("index_query", C.c_void_p), ("index_weights", C.c_void_p),
        ("scores", C.c_void_p), ("selected", C.c_void_p), ("selected_count", C.c_void_p),
    ]


class AttentionCompressRequest(C.Structure):
    """yvex_b200_attention_compress_request (include/yvex_b200/attention.h)."""
    _fields_ = [
        ("kind", C.c_int), ("attention_class", C.c_int), ("token_position", u64), ("token_count", u64),
        ("compression_ratio", u64), ("head_dimension", u64),
        ("token_kv", C.c_void_p), ("token_score", C.c_void_p), ("token_stride", u64),
        ("position_rows", C.c_void_p), ("state_kv", C.c_void_p), ("state_score", C.c_void_p),
        ("next_state_kv", C.c_void_p), ("next_state_score", C.c_void_p),
        ("norm_weights", C.c_void_p), ("rms_norm_epsilon", C.c_double),
        ("rope_dimension", u64), ("rope_frequency", C.c_void_p),
        ("compressed", C.c_void_p), ("compressed_positions", C.c_void_p), ("emitted", u64),
        ("activation_quantization", C.c_uint), ("activation_block_width", u64), ("activation_hadamard", C.c_int),
    ]


class AttentionActivationRequest(C.Structure):
    """yvex_b200_attention_activation_request (include/yvex_b200/attention.h)."""
    _fields_ = [("values", C.c_void_p), ("rows", u64), ("row_stride", u64), ("count", u64),
                ("quantization", C.c_uint), ("block_width", u64), ("hadamard", C.c_int)]


class AttentionPublishRequest(C.Structure):
    """yvex_b200_attention_publish_request (include/yvex_b200/attention.h)."""
    _fields_ = [("values", C.c_void_p), ("rows", u64), ("rows_per_token", u64), ("row_stride", u64), ("width", u64),
                ("token_position", u64), ("norm_mode", C.c_int), ("norm_weights", C.c_void_p),
                ("rms_norm_epsilon", C.c_double), ("rope_dimension", u64), ("rope_frequency", C.c_void_p),
                ("activation_quantization", C.c_uint), ("activation_count", u64), ("activation_block_width", u64),
                ("activation_hadamard", C.c_int)]


class RowsPublishArgs(C.Structure):
    """yvx_rows_publish_args (include/yvex_b200/cuda_shim.h)."""
    _fields_ = [("values", C.c_void_p), ("rows", u64), ("rows_per_token", u64), ("row_stride", u64), ("width", u64),
                ("norm_mode", C.c_int), ("norm_weights", C.c_void_p), ("epsilon", C.c_double),
                ("rope_dims", u64), ("rope_frequency", C.c_void_p), ("start_position", u64),
                ("quantization", C.c_uint), ("activation_count", u64), ("block_width", u64),
                ("hadamard", C.c_int), ("status", C.c_void_p)]


class ActivationArgs(C.Structure):
    """yvx_activation_args (include/yvex_b200/cuda_shim.h)."""
    _fields_ = [("values", C.c_void_p), ("rows", u64), ("row_stride", u64), ("count", u64),
                ("quantization", C.c_uint), ("block_width", C.c_uint), ("hadamard", C.c_int),
                ("hadamard_scale", C.c_float), ("status", C.c_void_p)]


class CompressorArgs(C.Structure):
    """yvx_compressor_args (include/yvex_b200/cuda_shim.h)."""
    _fields_ = [
        ("ratio", u64), ("head_dim", u64), ("overlap", C.c_int), ("start_position", u64), ("token_count", u64),
        ("token_kv", C.c_void_p), ("token_score", C.c_void_p), ("token_stride", u64), ("ape", C.c_void_p),
        ("state_kv", C.c_void_p), ("state_score", C.c_void_p), ("after_kv", C.c_void_p), ("after_score", C.c_void_p),
        ("compressed", C.c_void_p), ("compressed_stride", u64), ("positions", C.c_void_p),
        ("norm_weights", C.c_void_p), ("epsilon", C.c_double), ("rope_dims", u64), ("rope_frequency", C.c_void_p),
        ("status", C.c_void_p),
        ("activation_quantization", C.c_uint), ("activation_count", u64), ("activation_block_width", u64),
        ("activation_hadamard", C.c_int),
    ]


class CsaSelectArgs(C.Structure):
    """yvx_csa_select_args (include/yvex_b200/cuda_shim.h)."""
    _fields_ = [
        ("keys", C.c_void_p), ("positions", C.c_void_p), ("rows", u64), ("key_stride", u64),
        ("query", C.c_void_p), ("weights", C.c_void_p),
        ("heads", C.c_uint), ("head_dim", C.c_uint), ("topk", C.c_uint),
        ("ratio", u64), ("phase_start_position", u64), ("token_count", u64),
        ("scores", C.c_void_p), ("selected", C.c_void_p), ("selected_count", C.c_void_p),
        ("topk_capacity", u64), ("workspace", C.c_void_p), ("status", C.c_void_p),
    ]


class KvAppendRequest(C.Structure):
    """yvex_b200_kv_append_request (include/yvex_b200/attention.h)."""
    _fields_ = [
        ("session_count", u64), ("token_count", u64),
        ("query_heads", u64), ("key_value_heads", u64), ("head_dimension", u64), ("rotary_dimension", u64),
        ("bf16_staged_products", C.c_int),
        ("query", C.c_void_p), ("key", C.c_void_p), ("value", C.c_void_p),
        ("cosines", C.c_void_p), ("sines", C.c_void_p),
        ("kv_tokens", C.c_void_p), ("max_kv_tokens", u64), ("token_position", C.c_void_p),
        ("state_values", C.c_void_p), ("state_positions", C.c_void_p),
        ("state_capacity", u64), ("state_row_stride", u64),
        ("key_pool", C.c_void_p), ("value_pool", C.c_void_p), ("block_table", C.c_void_p),
        ("block_tokens", u64), ("max_blocks_per_session", u64), ("pool_blocks", u64),
    ]


class MlaDecodeRequest(C.Structure):
    """yvex_b200_mla_decode_request (include/yvex_b200/attention.h)."""
    _fields_ = [
        ("session_count", u64), ("heads", u64), ("nope_dimension", u64), ("latent_dimension", u64),
        ("rope_dimension", u64), ("context_capacity", u64), ("max_kv_tokens", u64), ("scale", C.c_float),
        ("q_nope", C.c_void_p), ("q_rope", C.c_void_p), ("w_uk", C.c_void_p),
        ("latent", C.c_void_p), ("rope_key", C.c_void_p), ("kv_tokens", C.c_void_p), ("output", C.c_void_p),
    ]


class KvAppendArgs(C.Structure):
    """yvx_kv_append_args (include/yvex_b200/cuda_shim.h)."""
    _fields_ = [
        ("sessions", C.c_uint), ("tokens", C.c_uint),
        ("query_heads", C.c_uint), ("kv_heads", C.c_uint), ("head_dim", C.c_uint), ("rotary_dim", C.c_uint),
        ("staged_bf16", C.c_int),
        ("query", C.c_void_p), ("key", C.c_void_p), ("value", C.c_void_p),
        ("cosines", C.c_void_p), ("sines", C.c_void_p),
        ("kv_tokens", C.c_void_p), ("kv_tokens_uniform", C.c_uint),
        ("state_values", C.c_void_p), ("state_session_stride", u64), ("state_row_stride", u64),
        ("state_positions", C.c_void_p), ("state_position_stride", u64),
        ("token_position", C.c_void_p),
        ("key_pool", C.c_void_p), ("value_pool", C.c_void_p), ("block_table", C.c_void_p),
        ("block_tokens", C.c_uint), ("block_table_stride", C.c_uint), ("pool_blocks", C.c_uint),
        ("pool_token_stride", u64), ("pool_head_stride", u64), ("pool_block_stride", u64),
        ("status", C.c_void_p), ("row_capacity", C.c_uint),
    ]


class MlaProblem(C.Structure):
    """yvx_mla_problem (include/yvex_b200/cuda_shim.h)."""
    _fields_ = [
        ("sessions", C.c_uint), ("heads", C.c_uint), ("nope_dim", C.c_uint), ("latent_dim", C.c_uint),
        ("rope_dim", C.c_uint), ("scale", C.c_float),
        ("q_nope", C.c_void_p), ("q_rope", C.c_void_p), ("w_uk", C.c_void_p), ("latent", C.c_void_p),
        ("rope_key", C.c_void_p), ("latent_session_stride", u64), ("rope_session_stride", u64),
        ("kv_tokens", C.c_void_p), ("kv_tokens_uniform", C.c_uint), ("kv_tokens_max", C.c_uint),
        ("chunk_tokens", C.c_uint), ("max_splits", C.c_uint),
        ("balanced_pairs", C.c_uint), ("cluster_ctas", C.c_uint),
        ("q_absorbed", C.c_void_p), ("partials", C.c_void_p), ("output", C.c_void_p),
        ("status", C.c_void_p),
    ]

# ---- the encoded attention job (include/yvex_b200/attention_job.h) -----------------------
ATTENTION_JOB_SCHEMA = 3
(WEIGHT_Q_A, WEIGHT_Q_A_NORM, WEIGHT_Q_B, WEIGHT_KV, WEIGHT_KV_NORM, WEIGHT_SINKS, WEIGHT_OUT_A, WEIGHT_OUT_B,
 WEIGHT_MAIN_KV, WEIGHT_MAIN_GATE, WEIGHT_MAIN_APE, WEIGHT_MAIN_NORM, WEIGHT_INDEX_KV, WEIGHT_INDEX_GATE,
 WEIGHT_INDEX_APE, WEIGHT_INDEX_NORM, WEIGHT_INDEX_Q, WEIGHT_INDEX_PROJECTION, WEIGHT_MHC_FUNCTION,
 WEIGHT_MHC_BASE, WEIGHT_MHC_SCALE, WEIGHT_INPUT_NORM, WEIGHT_COUNT) = range(23)
QTYPE_F32, QTYPE_F16, QTYPE_Q8_0, QTYPE_BF16 = 0, 1, 8, 30
ATTENTION_SWA, ATTENTION_CSA, ATTENTION_HCA = 0, 1, 2
ATTENTION_COMPUTE_BF16_F32_RNE_V1 = 1
ATTENTION_SCOPE_CORE, ATTENTION_SCOPE_ENVELOPE = 0, 1
ATTENTION_PHASE_PREFILL, ATTENTION_PHASE_DECODE = 0, 1
(JOB_FAILURE_NONE, JOB_FAILURE_INVALID_ARGUMENT, JOB_FAILURE_CAPABILITY, JOB_FAILURE_BUDGET,
 JOB_FAILURE_ALLOCATION, JOB_FAILURE_COPY, JOB_FAILURE_LAUNCH, JOB_FAILURE_SYNCHRONIZE, JOB_FAILURE_NUMERIC,
 JOB_FAILURE_CANCELLED, JOB_FAILURE_CLEANUP) = range(11)
(VARIANT_TENSOR_ALLOC, VARIANT_TENSOR_ZERO, VARIANT_TENSOR_WRITE, VARIANT_TENSOR_READ, VARIANT_TENSOR_COPY,
 VARIANT_EMBED_F32_TO_F32, VARIANT_EMBED_F16_TO_F32, VARIANT_RMS_NORM_F32_WEIGHT_F32,
 VARIANT_RMS_NORM_F32_WEIGHT_F16, VARIANT_ROPE_F32, VARIANT_MATMUL_F32, VARIANT_MLP_DENSE_F32,
 VARIANT_MLP_ROUTED_F32, VARIANT_ATTENTION_CAUSAL_F32, VARIANT_ATTENTION_NONCAUSAL_F32, VARIANT_QTYPE_ROW_DOT,
 VARIANT_ATTENTION_ENCODED, VARIANT_COUNT) = range(18)
CAPABILITY_UNSUPPORTED, CAPABILITY_SUPPORTED, CAPABILITY_FAILED = 0, 1, 2
CANCELLED_FN = C.CFUNCTYPE(C.c_int, C.c_void_p)
STATE_RESOLVE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, u64, C.POINTER(u64))


class JobWeight(C.Structure):
    _fields_ = [("encoded", C.c_void_p), ("encoded_bytes", C.c_size_t), ("row_bytes", u64), ("row_width", u64),
                ("row_count", u64), ("qtype", C.c_uint), ("present", C.c_int)]


class JobPosition(C.Structure):
    _fields_ = [(n, u64) for n in ("theta", "scaling_factor", "original_context", "beta_fast", "beta_slow",
                                   "rope_dimensions")]


class JobActivation(C.Structure):
    _fields_ = [("required", C.c_int), ("block_width", u64), ("quantization", C.c_uint), ("hadamard", C.c_int)]


class JobCancellation(C.Structure):
    _fields_ = [("requested", CANCELLED_FN), ("context", C.c_void_p)]


class FloatSpan(C.Structure):
    _fields_ = [("data", C.c_void_p), ("capacity", u64)]


class U64Span(C.Structure):
    _fields_ = [("data", C.c_void_p), ("capacity", u64)]


class JobRolling(C.Structure):
    _fields_ = [("present", C.c_int), ("overlap", C.c_int), ("next_token_position", u64), ("ratio", u64),
                ("head_dimension", u64), ("state_width", u64), ("state_slots", u64), ("cursor", u64),
                ("previous_fill", u64), ("current_fill", u64), ("kv_state", C.c_void_p), ("score_state", C.c_void_p),
                ("kv_state_capacity", u64), ("score_state_capacity", u64)]


class AttentionJob(C.Structure):
    _fields_ = [
        ("schema", C.c_uint), ("phase", C.c_int), ("attention_class", C.c_int), ("compute_contract", C.c_int),
        ("operation_scope", C.c_int),
        ("token_position", u64), ("token_count", u64), ("input_stride", u64),
        ("hidden_width", u64), ("q_rank", u64), ("query_heads", u64), ("head_dimension", u64), ("kv_width", u64),
        ("sliding_window", u64), ("compression_ratio", u64),
        ("output_groups", u64), ("output_group_input_width", u64), ("output_rank", u64),
        ("indexer_heads", u64), ("indexer_head_dimension", u64), ("indexer_topk", u64),
        ("residual_stream_count", u64), ("residual_stream_width", u64), ("residual_expanded_width", u64),
        ("mhc_mixing_rows", u64), ("mhc_sinkhorn_iterations", u64),
        ("rms_epsilon", C.c_double), ("mhc_epsilon", C.c_double), ("mhc_residual_post_multiplier", C.c_double),
        ("position", JobPosition),
        ("attention_kv_activation", JobActivation), ("compressor_activation", JobActivation),
        ("compressor_rotated_activation", JobActivation), ("indexer_query_activation", JobActivation),
        ("weights", JobWeight * WEIGHT_COUNT),
        ("input", C.c_void_p), ("local_kv", C.c_void_p), ("compressed_kv", C.c_void_p), ("indexer_kv", C.c_void_p),
        ("device_input", C.POINTER(DeviceTensor)), ("device_output", C.POINTER(DeviceTensor)),
        ("local_positions", C.c_void_p), ("compressed_positions", C.c_void_p), ("indexer_positions", C.c_void_p),
        ("local_count", u64), ("local_stride", u64), ("compressed_count", u64), ("compressed_stride", u64),
        ("indexer_count", u64), ("indexer_stride", u64),
        ("main_rolling", JobRolling), ("indexer_rolling", JobRolling),
        ("cancellation", C.POINTER(JobCancellation)), ("device_completion", C.c_void_p),
        ("evidence_level", C.c_uint), ("measure_device_time", C.c_int),
        ("candidate_block_visible", C.c_int), ("retain_prefix_checkpoints", C.c_int), ("native_execution", C.c_int),
        ("max_host_bytes", u64), ("max_device_bytes", u64),
    ]


class AttentionJobOutput(C.Structure):
    _fields_ = (
        [(n, FloatSpan) for n in ("core_input", "q_low", "query", "raw_kv", "compressed_kv", "indexer_kv",
                                  "index_query", "index_weights", "attention_values", "output", "envelope_output")] +
        [(n, U64Span) for n in ("compressed_positions", "indexer_positions", "topk_positions", "topk_counts",
                                "valid_candidate_counts")] +
        [(n, FloatSpan) for n in ("main_kv_state", "main_score_state", "indexer_kv_state", "indexer_score_state")] +
        [(n, u64) for n in ("tokens_executed", "compressed_count", "indexer_count", "topk_count",
                            "valid_candidate_count", "host_bytes", "peak_host_bytes", "device_bytes",
                            "peak_device_bytes", "kernel_launches", "accelerated_matrix_launches", "h2d_bytes",
                            "d2h_bytes", "d2d_bytes", "device_state_staged_bytes", "queue_synchronizations",
                            "device_synchronizations", "device_execution_elapsed_ns", "host_workspace_capacity",
                            "host_workspace_used", "host_workspace_peak", "host_workspace_allocation_count")] +
        [("host_workspace_reused", C.c_int), ("device_state_staged", C.c_int)])


class AttentionJobFailure(C.Structure):
    _fields_ = [("code", C.c_int), ("stage", C.c_char_p), ("expected", u64), ("actual", u64)]


class CompletionTransfer(C.Structure):
    _fields_ = [("output", C.c_void_p), ("staged", C.c_void_p), ("capacity", u64), ("output_capacity", u64),
                ("used", u64), ("width", C.c_size_t), ("stage", C.c_char_p)]


class AttentionCompletion(C.Structure):
    _fields_ = [("defer", C.c_int), ("stack_start", C.c_int), ("pending", C.c_int), ("barrier_observed", C.c_int),
                ("output", AttentionJobOutput), ("failure", AttentionJobFailure), ("host_status", C.c_void_p),
                ("host_selected_counts", C.c_void_p), ("host_candidate_counts", C.c_void_p),
                ("attention_class", C.c_uint), ("token_count", u64), ("indexer_topk", u64),
                ("candidate_capacity", u64), ("transfer_count", C.c_uint), ("transfers", CompletionTransfer * 20)]


class CapabilityResult(C.Structure):
    _fields_ = [("backend_kind", C.c_int), ("variant", C.c_int), ("state", C.c_int), ("reason", C.c_int),
                ("input_dtype", C.c_int), ("weight_dtype", C.c_int), ("output_dtype", C.c_int),
                ("context_available", C.c_int), ("kernel_bundle_available", C.c_int),
                ("function_available", C.c_int)]


class KvBankComponent(C.Structure):
    _fields_ = [("history", C.c_int), ("capacity", u64), ("value_width", u64), ("kv_state_extent", u64),
                ("score_state_extent", u64)]


class KvBankSpan(C.Structure):
    _fields_ = [("offset", u64 * 3), ("bytes", u64 * 3)]


class KvBankArgs(C.Structure):
    """yvx_kv_bank_args (include/yvex_b200/cuda_shim.h)."""
    _fields_ = [("sessions", C.c_uint), ("kv_heads", C.c_uint), ("head_dim", C.c_uint), ("kv_tokens", C.c_void_p),
                ("kv_tokens_uniform", C.c_uint), ("row_capacity", C.c_uint), ("bank", C.c_void_p),
                ("bank_session_bytes", u64), ("values_offset", u64), ("positions_offset", u64), ("value_width", u64),
                ("position_base", u64), ("key_pool", C.c_void_p), ("value_pool", C.c_void_p),
                ("block_table", C.c_void_p), ("block_tokens", C.c_uint), ("block_table_stride", C.c_uint),
                ("pool_blocks", C.c_uint), ("pool_token_stride", u64), ("pool_head_stride", u64),
                ("pool_block_stride", u64), ("status", C.c_void_p)]


class MatvecArgs(C.Structure):
    """yvx_matvec_args (include/yvex_b200/cuda_shim.h)."""
    _fields_ = [("weights", C.c_void_p), ("qtype", C.c_uint), ("first_row", u64), ("rows", u64), ("width", u64),
                ("row_bytes", u64), ("input", C.c_void_p), ("tokens", u64), ("input_stride", u64),
                ("output", C.c_void_p), ("output_stride", u64), ("groups", u64), ("round_bf16", C.c_int),
                ("status", C.c_void_p)]


class GemmArgs(C.Structure):
    """yvx_gemm_args (include/yvex_b200/cuda_shim.h)."""
    _fields_ = [("weights", C.c_void_p), ("first_row", u64), ("rows", u64), ("width", u64), ("input", C.c_void_p),
                ("tokens", u64), ("input_stride", u64), ("output", C.c_void_p), ("output_stride", u64),
                ("groups", u64), ("round_bf16", C.c_int), ("staging", C.c_void_p), ("status", C.c_void_p)]


# Every symbol the headers declare; tests check the library exports each one.
EXPORTED_SYMBOLS = [
    # attention_job.h
    "yvex_backend_attention_execute", "yvex_backend_attention_complete", "yvex_backend_query_capability",
    "yvex_b200_backend_weights_forget", "yvex_b200_backend_projection_gemm", "yvex_b200_kv_bank_layout",
    "yvex_backend_resident_attach", "yvex_backend_resident_detach", "yvex_backend_resident_resolve",
    "yvex_backend_state_residency_attach", "yvex_backend_state_residency_validate_generation",
    "yvex_backend_state_residency_publish_generation", "yvex_backend_state_residency_detach",
    "yvex_backend_state_residency_resolve",
    "yvex_backend_operation_variant_name", "yvex_backend_capability_state_name",
    "yvex_backend_capability_reason_name",
    # attention.h
    "yvex_error_clear", "yvex_error_set", "yvex_status_name",
    "yvex_backend_open", "yvex_backend_close_checked", "yvex_backend_close",
    "yvex_backend_cuda_available", "yvex_backend_sync",
    "yvex_backend_tensor_alloc", "yvex_backend_tensor_release", "yvex_backend_tensor_free",
    "yvex_backend_tensor_write", "yvex_backend_tensor_read", "yvex_backend_tensor_zero",
    "yvex_backend_tensor_f32_subview", "yvex_b200_tensor_wrap",
    "yvex_b200_backend_bind_stream", "yvex_b200_backend_stream", "yvex_b200_backend_sm_count",
    "yvex_b200_transformer_operations_get",
    "yvex_b200_transformer_attention_workspace_required",
    "yvex_b200_transformer_attention_execute",
    "yvex_backend_op_attention", "yvex_b200_attention_batch_execute",
    "yvex_b200_attention_reduce_execute", "yvex_b200_kv_append_rotary_execute", "yvex_b200_mla_decode_execute",
    "yvex_b200_attention_select_execute", "yvex_b200_rope_frequencies",
    "yvex_b200_attention_compress_execute", "yvex_b200_attention_activation_execute",
    "yvex_b200_attention_publish_execute",
    "yvex_b200_kv_pool_create", "yvex_b200_kv_pool_destroy", "yvex_b200_kv_pool_session_open",
    "yvex_b200_kv_pool_session_fork", "yvex_b200_kv_pool_session_close", "yvex_b200_kv_pool_reserve",
    "yvex_b200_kv_pool_commit", "yvex_b200_kv_pool_table", "yvex_b200_kv_pool_committed",
    "yvex_b200_kv_pool_reserved", "yvex_b200_kv_pool_free_blocks", "yvex_b200_kv_pool_block_refcount",
    "yvex_b200_kv_page_tokens", "yvex_b200_kv_page_touch", "yvex_b200_kv_block_row",
    "yvex_b200_kv_sequence_shard",
    # cuda_shim.h
    "yvx_cuda_device_count", "yvx_cuda_device_select", "yvx_cuda_device_properties",
    "yvx_cuda_malloc", "yvx_cuda_free", "yvx_cuda_host_alloc", "yvx_cuda_host_free",
    "yvx_cuda_memset_async", "yvx_cuda_upload_async", "yvx_cuda_download_async",
    "yvx_cuda_copy_async", "yvx_cuda_stream_create", "yvx_cuda_stream_destroy",
    "yvx_cuda_stream_synchronize", "yvx_cuda_device_synchronize", "yvx_cuda_event_create", "yvx_cuda_event_destroy",
    "yvx_cuda_event_record", "yvx_cuda_stream_wait_event", "yvx_cuda_event_elapsed_ms", "yvx_cuda_last_error_text",
    "yvx_cuda_lse_exchange_bytes", "yvx_cuda_lse_exchange_counter_offset", "yvx_cuda_gqa_attention_exchange",
    "yvx_cuda_lse_exchange_emulated", "yvx_cuda_lse_exchange_emulated_form", "yvx_cuda_bf16_gemm",
    "yvx_cuda_bf16_gemm_staging_bytes", "yvx_cuda_ipc_export", "yvx_cuda_ipc_open", "yvx_cuda_ipc_close",
    "yvx_cuda_graph_capture_begin", "yvx_cuda_graph_capture_end", "yvx_cuda_graph_launch", "yvx_cuda_graph_destroy",
    "yvx_cuda_gqa_partials_bytes", "yvx_cuda_gqa_f32_staging_bytes", "yvx_cuda_gqa_plan_splits", "yvx_cuda_gqa_attention",
    "yvx_cuda_lse_combine", "yvx_cuda_lse_combine_strided", "yvx_cuda_op_attention_f32",
    "yvx_cuda_gqa_attention_profiled",
    "yvx_cuda_fill_normal", "yvx_cuda_fill_normal_rope_bf16", "yvx_cuda_fill_q8_lanes", "yvx_cuda_fill_f16_uniform",
    "yvx_cuda_gqa_static_scratch_capacity", "yvx_cuda_gqa_attention_static_scratch",
    "yvx_cuda_q8_record_bytes", "yvx_cuda_q8_kv_pack", "yvx_cuda_fill_q8_records",
    "yvx_cuda_latent_reduce", "yvx_cuda_latent_reduce_launches", "yvx_cuda_latent_reduce_workspace_bytes",
    "yvx_cuda_csa_select", "yvx_cuda_csa_select_workspace_bytes", "yvx_cuda_kv_append_rotary", "yvx_cuda_mla_plan", "yvx_cuda_mla_absorbed_bytes", "yvx_cuda_mla_partials_bytes",
    "yvx_cuda_kv_bank_transfer", "yvx_cuda_qtype_row_bytes", "yvx_cuda_qtype_matvec", "yvx_cuda_qtype_decode_rows", "yvx_cuda_round_bf16_rows",
    "yvx_cuda_mla_decode", "yvx_cuda_compressor_chunk", "yvx_cuda_activation_quant", "yvx_cuda_rows_publish", "yvx_cuda_rows_publish_batch",
]

_lib = None


def load():
    """Load libyvex_b200.so; raise if it is missing (there is no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is not built; run `python -m clori_b200._build` "
            "(the attention path has no CPU or library fallback)")
    lib = C.CDLL(LIB_PATH)
    P = C.POINTER
    vp = C.c_void_p
    lib.yvex_status_name.restype = C.c_char_p
    lib.yvex_status_name.argtypes = [C.c_int]
    lib.yvex_backend_open.argtypes = [P(vp), P(BackendOptions), P(Error)]
    lib.yvex_backend_close_checked.argtypes = [P(vp), P(Error)]
    lib.yvex_backend_close.restype = None
    lib.yvex_backend_close.argtypes = [vp]
    lib.yvex_backend_sync.argtypes = [vp, P(Error)]
    lib.yvex_backend_tensor_alloc.argtypes = [vp, P(TensorDesc), P(P(DeviceTensor)), P(Error)]
    lib.yvex_b200_tensor_wrap.argtypes = [vp, P(TensorDesc), vp, P(P(DeviceTensor)), P(Error)]
    lib.yvex_backend_tensor_release.argtypes = [vp, P(P(DeviceTensor)), P(Error)]
    lib.yvex_backend_tensor_write.argtypes = [vp, P(DeviceTensor), vp, u64, P(Error)]
    lib.yvex_backend_tensor_read.argtypes = [vp, P(DeviceTensor), vp, u64, P(Error)]
    lib.yvex_backend_tensor_zero.argtypes = [vp, P(DeviceTensor), P(Error)]
    lib.yvex_backend_tensor_f32_subview.argtypes = [P(DeviceTensor), u64, u64, P(DeviceTensor)]
    lib.yvex_b200_backend_bind_stream.argtypes = [vp, vp, C.c_int, P(Error)]
    lib.yvex_b200_backend_stream.restype = vp
    lib.yvex_b200_backend_stream.argtypes = [vp]
    lib.yvex_b200_backend_sm_count.argtypes = [vp]
    lib.yvex_b200_transformer_operations_get.restype = P(TransformerOperations)
    lib.yvex_b200_transformer_operations_get.argtypes = [vp]
    lib.yvex_b200_transformer_attention_workspace_required.argtypes = [
        P(AttentionRequirement), P(u64), P(Error)]
    lib.yvex_b200_transformer_attention_execute.argtypes = [
        vp, P(AttentionRequest), P(OperationFacts), P(Error)]
    lib.yvex_backend_op_attention.argtypes = [
        vp, P(DeviceTensor), P(DeviceTensor), P(DeviceTensor), u64, u64, C.c_float, C.c_int,
        P(DeviceTensor), P(DeviceTensor), P(DeviceTensor), P(Error)]
    lib.yvex_b200_attention_batch_execute.argtypes = [
        vp, P(BatchRequest), P(OperationFacts), P(Error)]
    lib.yvex_b200_attention_reduce_execute.argtypes = [
        vp, P(AttentionReduceRequest), P(AttentionFailure), P(OperationFacts), P(Error)]
    lib.yvex_b200_attention_select_execute.argtypes = [
        vp, P(AttentionSelectRequest), P(AttentionFailure), P(OperationFacts), P(Error)]
    lib.yvex_b200_rope_frequencies.argtypes = [P(PositionPolicy), u64, vp]
    lib.yvex_b200_attention_compress_execute.argtypes = [
        vp, P(AttentionCompressRequest), P(AttentionFailure), P(OperationFacts), P(Error)]
    lib.yvx_cuda_compressor_chunk.argtypes = [P(CompressorArgs), vp, P(u64)]
    lib.yvex_backend_attention_execute.argtypes = [vp, P(AttentionJob), P(AttentionJobOutput),
                                                   P(AttentionJobFailure), P(Error)]
    lib.yvex_backend_attention_complete.argtypes = [vp, P(AttentionCompletion), C.c_int, P(Error)]
    lib.yvex_b200_backend_weights_forget.argtypes = [vp, P(Error)]
    lib.yvex_backend_resident_attach.argtypes = [vp, vp, u64, P(DeviceTensor), u64, P(Error)]
    lib.yvex_backend_resident_detach.argtypes = [vp, P(Error)]
    lib.yvex_backend_resident_resolve.argtypes = [vp, vp, u64, P(u64)]
    lib.yvex_backend_state_residency_attach.argtypes = [vp, vp, STATE_RESOLVE_FN, u64, P(Error)]
    lib.yvex_backend_state_residency_validate_generation.argtypes = [vp, u64, P(Error)]
    lib.yvex_backend_state_residency_publish_generation.restype = None
    lib.yvex_backend_state_residency_publish_generation.argtypes = [vp, u64]
    lib.yvex_backend_state_residency_detach.restype = None
    lib.yvex_backend_state_residency_detach.argtypes = [vp]
    lib.yvex_backend_state_residency_resolve.argtypes = [vp, vp, u64, P(u64)]
    lib.yvex_backend_query_capability.argtypes = [vp, C.c_int, P(CapabilityResult), P(Error)]
    for name in ("yvex_backend_operation_variant_name", "yvex_backend_capability_state_name",
                 "yvex_backend_capability_reason_name"):
        getattr(lib, name).restype = C.c_char_p
        getattr(lib, name).argtypes = [C.c_int]
    lib.yvx_cuda_kv_bank_transfer.argtypes = [P(KvBankArgs), C.c_int, vp]
    lib.yvex_b200_kv_bank_layout.argtypes = [P(KvBankComponent), C.c_uint, P(KvBankSpan), P(u64)]
    lib.yvx_cuda_gqa_f32_staging_bytes.restype = u64
    lib.yvx_cuda_gqa_f32_staging_bytes.argtypes = [P(GqaProblem)]
    lib.yvx_cuda_qtype_row_bytes.restype = u64
    lib.yvx_cuda_qtype_row_bytes.argtypes = [C.c_uint, u64]
    lib.yvx_cuda_qtype_matvec.argtypes = [P(MatvecArgs), vp]
    lib.yvx_cuda_qtype_decode_rows.argtypes = [vp, C.c_uint, u64, u64, u64, vp, vp, vp]
    lib.yvx_cuda_round_bf16_rows.argtypes = [vp, u64, u64, u64, vp, vp]
    lib.yvex_b200_attention_activation_execute.argtypes = [
        vp, P(AttentionActivationRequest), P(AttentionFailure), P(OperationFacts), P(Error)]
    lib.yvx_cuda_activation_quant.argtypes = [P(ActivationArgs), vp]
    lib.yvex_b200_attention_publish_execute.argtypes = [
        vp, P(AttentionPublishRequest), P(AttentionFailure), P(OperationFacts), P(Error)]
    lib.yvx_cuda_rows_publish.argtypes = [P(RowsPublishArgs), vp]
    lib.yvx_cuda_rows_publish_batch.argtypes = [P(RowsPublishArgs), C.c_uint, vp]
    lib.yvex_b200_kv_append_rotary_execute.argtypes = [vp, P(KvAppendRequest), P(OperationFacts), P(Error)]
    lib.yvex_b200_mla_decode_execute.argtypes = [vp, P(MlaDecodeRequest), P(OperationFacts), P(Error)]
    lib.yvex_b200_kv_pool_create.restype = vp
    lib.yvex_b200_kv_pool_create.argtypes = [C.c_uint, C.c_uint, C.c_uint, C.c_uint]
    lib.yvex_b200_kv_pool_destroy.restype = None
    lib.yvex_b200_kv_pool_destroy.argtypes = [vp]
    lib.yvex_b200_kv_pool_session_open.argtypes = [vp, P(C.c_uint)]
    lib.yvex_b200_kv_pool_session_fork.argtypes = [vp, C.c_uint, P(C.c_uint)]
    lib.yvex_b200_kv_pool_session_close.argtypes = [vp, C.c_uint]
    lib.yvex_b200_kv_pool_reserve.argtypes = [vp, C.c_uint, C.c_uint, P(KvCopy)]
    lib.yvex_b200_kv_pool_commit.argtypes = [vp, C.c_uint, C.c_uint]
    lib.yvex_b200_kv_pool_table.restype = P(C.c_int)
    lib.yvex_b200_kv_pool_table.argtypes = [vp, C.c_uint]
    lib.yvex_b200_kv_pool_committed.restype = u64
    lib.yvex_b200_kv_pool_committed.argtypes = [vp, C.c_uint]
    lib.yvex_b200_kv_pool_reserved.restype = u64
    lib.yvex_b200_kv_pool_reserved.argtypes = [vp, C.c_uint]
    lib.yvex_b200_kv_pool_free_blocks.restype = C.c_uint
    lib.yvex_b200_kv_pool_free_blocks.argtypes = [vp]
    lib.yvex_b200_kv_pool_block_refcount.restype = C.c_uint
    lib.yvex_b200_kv_pool_block_refcount.argtypes = [vp, C.c_uint]
    lib.yvex_b200_kv_page_tokens.argtypes = [P(PageRequest), P(u64), P(u64)]
    lib.yvex_b200_kv_page_touch.argtypes = [u64, u64, u64, P(u64), P(u64)]
    lib.yvex_b200_kv_block_row.restype = u64
    lib.yvex_b200_kv_block_row.argtypes = [P(C.c_int), u64, u64]
    lib.yvx_cuda_last_error_text.restype = C.c_char_p
    lib.yvx_cuda_device_count.argtypes = [P(C.c_int)]
    lib.yvx_cuda_malloc.argtypes = [P(vp), u64]
    lib.yvx_cuda_free.argtypes = [vp]
    lib.yvx_cuda_host_alloc.argtypes = [P(vp), u64]
    lib.yvx_cuda_host_free.argtypes = [vp]
    lib.yvx_cuda_memset_async.argtypes = [vp, C.c_int, u64, vp]
    lib.yvx_cuda_upload_async.argtypes = [vp, vp, u64, vp]
    lib.yvx_cuda_download_async.argtypes = [vp, vp, u64, vp]
    lib.yvx_cuda_copy_async.argtypes = [vp, vp, u64, vp]
    lib.yvx_cuda_stream_create.argtypes = [P(vp)]
    lib.yvx_cuda_stream_destroy.argtypes = [vp]
    lib.yvx_cuda_stream_synchronize.argtypes = [vp]
    lib.yvx_cuda_event_create.argtypes = [P(vp)]
    lib.yvx_cuda_event_destroy.argtypes = [vp]
    lib.yvx_cuda_event_record.argtypes = [vp, vp]
    lib.yvx_cuda_stream_wait_event.argtypes = [vp, vp]
    lib.yvx_cuda_lse_exchange_bytes.restype = u64
    lib.yvx_cuda_lse_exchange_bytes.argtypes = [C.c_uint, C.c_uint, C.c_uint]
    lib.yvx_cuda_lse_exchange_counter_offset.restype = u64
    lib.yvx_cuda_lse_exchange_counter_offset.argtypes = [C.c_uint, C.c_uint, C.c_uint]
    lib.yvx_cuda_gqa_attention_exchange.argtypes = [P(GqaProblem), P(LseExchange), vp, P(C.c_uint)]
    lib.yvx_cuda_lse_exchange_emulated.argtypes = [vp, C.c_uint, C.c_uint, C.c_uint, vp, vp, C.c_uint, vp, vp, vp]
    lib.yvx_cuda_bf16_gemm.argtypes = [P(GemmArgs), vp]
    lib.yvx_cuda_bf16_gemm_staging_bytes.restype = u64
    lib.yvx_cuda_bf16_gemm_staging_bytes.argtypes = [u64, u64, u64]
    lib.yvx_cuda_lse_exchange_emulated_form.argtypes = [vp, C.c_uint, C.c_uint, C.c_uint, vp, vp, C.c_uint, vp, vp, vp,
                                                        C.c_int, C.c_int]
    lib.yvx_cuda_ipc_export.argtypes = [vp, vp]
    lib.yvx_cuda_ipc_open.argtypes = [vp, P(vp)]
    lib.yvx_cuda_ipc_close.argtypes = [vp]
    lib.yvx_cuda_graph_capture_begin.argtypes = [vp]
    lib.yvx_cuda_graph_capture_end.argtypes = [vp, P(vp)]
    lib.yvx_cuda_graph_launch.argtypes = [vp, vp]
    lib.yvx_cuda_graph_destroy.argtypes = [vp]
    lib.yvx_cuda_event_elapsed_ms.argtypes = [vp, vp, P(C.c_float)]
    lib.yvx_cuda_gqa_partials_bytes.restype = u64
    lib.yvx_cuda_gqa_partials_bytes.argtypes = [P(GqaProblem)]
    lib.yvx_cuda_gqa_plan_splits.restype = None
    lib.yvx_cuda_gqa_plan_splits.argtypes = [P(GqaProblem), C.c_int]
    lib.yvx_cuda_gqa_attention.argtypes = [P(GqaProblem), vp, P(C.c_uint)]
    lib.yvx_cuda_gqa_attention_profiled.argtypes = [P(GqaProblem), vp, vp * 3, P(C.c_uint)]
    lib.yvx_cuda_fill_normal.argtypes = [vp, C.c_int, u64, u64, C.c_float, vp]
    lib.yvx_cuda_fill_normal_rope_bf16.argtypes = [vp, u64, C.c_uint, C.c_uint, C.c_uint, u64, C.c_float, C.c_double, vp]
    lib.yvx_cuda_fill_q8_lanes.argtypes = [vp, u64, u64, vp]
    lib.yvx_cuda_fill_f16_uniform.argtypes = [vp, u64, u64, C.c_float, C.c_float, vp]
    lib.yvx_cuda_gqa_static_scratch_capacity.restype = u64
    lib.yvx_cuda_gqa_static_scratch_capacity.argtypes = []
    lib.yvx_cuda_gqa_attention_static_scratch.argtypes = [P(GqaProblem), vp, P(C.c_uint)]
    lib.yvx_cuda_latent_reduce.argtypes = [P(LatentReduceArgs), vp]
    lib.yvx_cuda_latent_reduce_launches.argtypes = [P(LatentReduceArgs), vp, P(C.c_uint)]
    lib.yvx_cuda_latent_reduce_workspace_bytes.restype = u64
    lib.yvx_cuda_latent_reduce_workspace_bytes.argtypes = [P(LatentReduceArgs)]
    lib.yvx_cuda_csa_select_workspace_bytes.restype = u64
    lib.yvx_cuda_csa_select_workspace_bytes.argtypes = [u64, u64, C.c_uint]
    lib.yvx_cuda_csa_select.argtypes = [P(CsaSelectArgs), vp, P(C.c_uint)]
    lib.yvx_cuda_kv_append_rotary.argtypes = [P(KvAppendArgs), vp]
    lib.yvx_cuda_mla_plan.restype = None
    lib.yvx_cuda_mla_plan.argtypes = [P(MlaProblem), C.c_int]
    lib.yvx_cuda_mla_absorbed_bytes.restype = u64
    lib.yvx_cuda_mla_absorbed_bytes.argtypes = [P(MlaProblem)]
    lib.yvx_cuda_mla_partials_bytes.restype = u64
    lib.yvx_cuda_mla_partials_bytes.argtypes = [P(MlaProblem)]
    lib.yvx_cuda_mla_decode.argtypes = [P(MlaProblem), vp, vp, P(C.c_uint)]
    lib.yvx_cuda_fill_q8_records.argtypes = [vp, u64, u64, C.c_float, C.c_float, vp]
    lib.yvx_cuda_q8_record_bytes.restype = u64
    lib.yvx_cuda_q8_record_bytes.argtypes = []
    lib.yvx_cuda_q8_kv_pack.argtypes = [vp, vp, C.c_uint, C.c_uint, vp, vp, u64, u64, C.c_uint, vp]
    lib.yvex_b200_kv_sequence_shard.argtypes = [u64, C.c_uint, C.c_uint, u64, P(u64), P(u64)]
    lib.yvx_cuda_lse_combine_strided.argtypes = [vp, C.c_uint, C.c_uint, C.c_uint, u64, u64, vp, C.c_int, vp, vp]
    lib.yvx_cuda_lse_combine.argtypes = [vp, C.c_uint, C.c_uint, C.c_uint, vp, C.c_int, vp, vp]
    _lib = lib
    return lib
