/* Thin C-ABI over the sm_100a attention kernels.
 *
 * Plain pointers and sizes only. Host code (C11) includes this header and never
 * a CUDA header, the same rule the reference keeps between its host code and
 * its driver shim (src/backend/cuda/private.h:16-21). Every function returns 0
 * on success or a negative yvex_status; device pointers are raw addresses and
 * `stream` is a cudaStream_t passed as void* (NULL = the default stream).
 *
 * Each launch entry replaces one launch site of the reference, named beside it.
 */
#ifndef YVEX_B200_CUDA_SHIM_H
#define YVEX_B200_CUDA_SHIM_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- device runtime plumbing (reference: src/backend/cuda/backend.c open,
 * alloc, copy and synchronize paths) ------------------------------------- */
int yvx_cuda_device_count(int *count);
int yvx_cuda_device_select(int device);
int yvx_cuda_device_properties(int device, int *sm_count, int *cc_major, int *cc_minor,
                               unsigned long long *global_bytes, char *name, size_t name_cap);
int yvx_cuda_malloc(void **out, unsigned long long bytes);
int yvx_cuda_free(void *pointer);
int yvx_cuda_host_alloc(void **out, unsigned long long bytes);
int yvx_cuda_host_free(void *pointer);
int yvx_cuda_memset_async(void *device, int value, unsigned long long bytes, void *stream);
int yvx_cuda_upload_async(void *device, const void *host, unsigned long long bytes, void *stream);
int yvx_cuda_download_async(void *host, const void *device, unsigned long long bytes, void *stream);
int yvx_cuda_copy_async(void *destination, const void *source, unsigned long long bytes, void *stream);
int yvx_cuda_stream_create(void **stream);
int yvx_cuda_stream_destroy(void *stream);
int yvx_cuda_stream_synchronize(void *stream);
int yvx_cuda_event_create(void **event);
int yvx_cuda_event_destroy(void *event);
int yvx_cuda_event_record(void *event, void *stream);
/* Work enqueued on `stream` after this call waits for the work `event` recorded (another
 * stream's, as a rule). Inside a stream capture it forks / joins the captured graph. */
int yvx_cuda_stream_wait_event(void *stream, void *event);
int yvx_cuda_event_elapsed_ms(void *start, void *stop, float *milliseconds);
/* Capture of the calls made on `stream` into a replayable graph (no reference entry
 * point of this name; the reference's operators are capture-aware, src/backend/cuda/
 * capability.c:802-805). The yvx_cuda_gqa_attention, _mla_decode, _latent_reduce,
 * _kv_append_rotary, _lse_combine, _rows_publish, _compressor_chunk and _activation_quant
 * entries may be called between begin and end. */
int yvx_cuda_graph_capture_begin(void *stream);
int yvx_cuda_graph_capture_end(void *stream, void **executable);
int yvx_cuda_graph_launch(void *executable, void *stream);
int yvx_cuda_graph_destroy(void *executable);
const char *yvx_cuda_last_error_text(void);
/* Waits for every stream of the current device (used before an arena that enqueued work on
 * any stream may still read is released). */
int yvx_cuda_device_synchronize(void);

/* ---- grouped-query attention over a KV cache ------------------------------
 * Replaces the launch of yvex_gqa_f32 / yvex_gqa_wide_f32
 * (src/backend/cuda/transformer.c:787-806, kernels in
 * src/backend/cuda/transformer_kernels.cu:137-238) and the tiled MHA sequence
 * (src/backend/cuda/transformer.c:493-677). One description covers decode
 * (1 row), speculative verify (2..8 rows) and general causal/full attention,
 * over one session or a batch, with contiguous strided KV rows or a block
 * table over a shared pool.
 *
 *   O[b,t,h,:] = softmax_s( scale * Q[b,t,h,:] . K[b,s,h/g,:] ) V[b,s,h/g,:]
 *   causal: s visible iff  kv_position_base + s <= query_start[b] + t
 *
 * All strides are in ELEMENTS of the tensor's dtype.
 *
 * kv_dtype = YVEX_DTYPE_Q8_0 selects the quantised cache: `key` points at Q8
 * records (see yvx_cuda_q8_kv_pack), `value` is unused, head_dim must be 128,
 * block_tokens 64, and key_head_stride / key_block_stride / key_session_stride
 * are in BYTES (record of head h of block j: key + j*key_block_stride +
 * h*key_head_stride; without a block table, block j of session b is
 * b*key_session_stride/key_block_stride + j). */
typedef struct yvx_gqa_problem {
    unsigned int sessions;        /* batch of independent sessions */
    unsigned int query_rows;      /* query rows per session (uniform) */
    unsigned int query_heads, kv_heads, head_dim;
    unsigned int causal;          /* 0 = full, 1 = causal */
    float scale;
    int query_dtype, kv_dtype, output_dtype; /* yvex_dtype ids */

    const void *query;            /* [session][row][query_heads*head_dim] */
    unsigned long long query_row_stride, query_session_stride;
    void *output;                 /* packed [session][row][query_heads*head_dim] */

    const void *key, *value;      /* session 0 / pool block 0, token 0, head 0 */
    unsigned long long key_token_stride, value_token_stride;
    unsigned long long key_head_stride, value_head_stride;
    unsigned long long key_session_stride, value_session_stride; /* contiguous layout */
    const int *block_table;       /* device [sessions][block_table_stride]; NULL = contiguous */
    unsigned int block_tokens, block_table_stride;
    unsigned int pool_blocks;     /* table entries outside [0, pool_blocks) are a contract failure */
    unsigned long long key_block_stride, value_block_stride;

    const unsigned int *kv_tokens;   /* device [sessions]; NULL = uniform */
    unsigned int kv_tokens_uniform;
    unsigned int kv_tokens_max;      /* host-side upper bound of every length */
    const unsigned int *query_start; /* device [sessions]; NULL = uniform / from end */
    unsigned int query_start_uniform;
    unsigned int query_start_from_end; /* 1: query_start = kv length - query_rows */
    unsigned int kv_position_base;   /* absolute position of local KV token 0 */

    unsigned int chunk_tokens;       /* KV tokens per split: a multiple of 64 (the short F32
                                        decode plan uses multiples of 16, at most 112) */
    unsigned int max_splits;         /* ceil(kv_tokens_max / chunk_tokens) */
    float *partials;                 /* scratch [session][row][qhead][split][head_dim+2] */
    float *partial_output;           /* non-NULL: emit (o, m, l) per (session,row,qhead)
                                        instead of the final output: [..][head_dim+2] */
    int *status;                     /* device status word; 0 ok, 1 non-finite, 2 contract,
                                        3 a bounded device-side wait gave up */
    int force_general;               /* 1: take the general kernel even when a specialised
                                        one admits the shape (cross-checks in tests) */
    unsigned long long query_head_stride; /* elements between query heads of a row; 0 = head_dim.
                                        Anything else (interleaved [head][Q|K|V][dim] rows,
                                        src/graph/numeric.c:1771-1826) takes the general kernel */
    void *f32_staging;               /* optional, F32 problems only: yvx_cuda_gqa_f32_staging_bytes()
                                        bytes of scratch. With it a prefill-sized F32 problem
                                        (head_dim 128, more than 64 vectors per KV head, contiguous
                                        KV) whose Q, K and V lanes are all representable in bf16 runs
                                        on the tensor-core prefill kernel (bf16 operands staged here,
                                        F32 accumulation and output; the reference's tiled path and
                                        its tolerance: src/backend/cuda/transformer.c:493-677,
                                        tests/unit/cuda/quant_qtype.c:2717-2866); any other lane value
                                        is found on the device and the exact general kernel runs
                                        instead, with no host round trip (three launches either way) */
    const int *gate;                 /* kernels of this problem run only while *gate == gate_value;
                                        NULL: always (set by the launcher for the path above) */
    int gate_value;
    int *tickets;                    /* optional: 2 * sessions * kv_heads device counters, zero before the
                                        first call (the kernels leave them at zero). With them the short
                                        F32 decode kernel folds its own splits: the CTA that arrives last
                                        for a KV head reads every split's partial, in split order, and
                                        writes the output: one launch instead of two. Calls that overlap
                                        on the GPU must not share tickets */
} yvx_gqa_problem;

/* Scratch the tensor-core path of an F32 problem needs (0 when the shape never takes it). */
unsigned long long yvx_cuda_gqa_f32_staging_bytes(const yvx_gqa_problem *problem);

/* Scratch bytes `partials` must hold for a problem (0 when one split suffices). */
unsigned long long yvx_cuda_gqa_partials_bytes(const yvx_gqa_problem *problem);
/* Picks chunk_tokens/max_splits for a device with `sm_count` SMs. Deterministic
 * in the problem's shape, dtypes, layout flags and pointer alignment only; call it
 * after every other field is set (short F32 decode shapes get their own plan). */
void yvx_cuda_gqa_plan_splits(yvx_gqa_problem *problem, int sm_count);
/* Launches the attention (1 launch) and, when max_splits > 1, the combine
 * (1 more). `launches` receives the number of kernels enqueued. */
int yvx_cuda_gqa_attention(const yvx_gqa_problem *problem, void *stream,
                           unsigned int *launches);
/* Same launches with three events (cudaEvent_t as void*) recorded on `stream`:
 * before the attention kernel, between it and the combine, after the combine.
 * For measuring the dominant kernel alone; no counterpart in the reference. */
int yvx_cuda_gqa_attention_profiled(const yvx_gqa_problem *problem, void *stream,
                                    void *events[3], unsigned int *launches);

/* ---- split attention + cross-GPU fold over NVLink peer memory -------------------
 * For one session whose KV sequence is sharded over `ranks` GPUs (one process per
 * GPU): the attention kernel, then ONE kernel that folds this rank's splits, stores
 * the resulting (o, m, l) row of every item into every rank's exchange area with
 * peer stores, counts arrivals, waits (bounded, status 3 on expiry) for the rows of
 * all ranks and folds them in rank order into `problem->output`. No reference
 * counterpart (the reference is single-device); it replaces the sequence local
 * combine -> NCCL all-gather -> yvx_cuda_lse_combine_strided.
 * Each rank allocates an area of yvx_cuda_lse_exchange_bytes(ranks, items, head_dim)
 * bytes: room for [2][ranks][items][head_dim + 2] 8-byte words (the float form uses the
 * first half) followed by [items] 32-bit arrival counters and [items] tickets, zero-filled once; exports it with yvx_cuda_ipc_export, opens its peers'
 * handles with yvx_cuda_ipc_open, and passes device arrays of the `ranks` area
 * pointers and counter pointers (own entries are the local addresses). `epoch`
 * counts calls from 1 and must be the same on every rank for the same step.
 * problem->partial_output (a local [items][head_dim + 2] row buffer) must be set. */
typedef struct yvx_lse_exchange {
    unsigned int ranks, rank, epoch;
    float *const *gather;            /* device array [ranks]: base of rank r's area */
    unsigned int *const *arrivals;   /* device array [ranks]: rank r's arrival counters */
    int one_launch;                  /* 1: fold the splits and run the exchange in the tail of the
                                        attention kernel itself (one cooperative launch per step:
                                        Q8_0 KV, uniform lengths, a grid that is resident at once,
                                        and the same split plan every epoch of an area; otherwise
                                        the two-launch path is taken silently) */
    int tagged_words;                /* 1: every 32-bit lane of a row travels as an 8-byte (value, epoch)
                                        word and receivers poll the words themselves: no system-wide fence
                                        and no arrival counter on the path. The area is then laid out as
                                        [2][ranks][items][head_dim + 2] 8-byte words; an area serves one
                                        of the two forms for its whole life */
} yvx_lse_exchange;
unsigned long long yvx_cuda_lse_exchange_bytes(unsigned int ranks, unsigned int items, unsigned int head_dim);
unsigned long long yvx_cuda_lse_exchange_counter_offset(unsigned int ranks, unsigned int items,
                                                        unsigned int head_dim);
int yvx_cuda_gqa_attention_exchange(const yvx_gqa_problem *problem, const yvx_lse_exchange *exchange,
                                    void *stream, unsigned int *launches);
/* The same exchange with every rank played by one cooperative launch on one GPU
 * (rows[rank][item][head_dim + 2] in, output[rank][item][head_dim] out): for tests. */
int yvx_cuda_lse_exchange_emulated(const float *rows, unsigned int ranks, unsigned int items,
                                   unsigned int head_dim, float *const *gather,
                                   unsigned int *const *arrivals, unsigned int epoch, float *output,
                                   int *status, void *stream);
/* The same with the form of the area chosen (tagged_words as in yvx_lse_exchange) and, in the
 * tagged form, one rank that never publishes (absent_rank >= 0): the others' bounded waits run out. */
int yvx_cuda_lse_exchange_emulated_form(const float *rows, unsigned int ranks, unsigned int items,
                                        unsigned int head_dim, float *const *gather,
                                        unsigned int *const *arrivals, unsigned int epoch, float *output,
                                        int *status, void *stream, int tagged_words, int absent_rank);
/* CUDA IPC for the exchange areas: a 64-byte handle of a yvx_cuda_malloc allocation,
 * and the mapping of a peer's handle into this process (peer access is enabled). */
int yvx_cuda_ipc_export(void *device_pointer, void *handle_64_bytes);
int yvx_cuda_ipc_open(const void *handle_64_bytes, void **device_pointer);
int yvx_cuda_ipc_close(void *device_pointer);

/* The same attention for callers that cannot allocate device memory on this
 * path (a host that gave the whole GPU to its own pool, a latency-critical step
 * that cannot afford an allocation's synchronisation, a plug-in handed only its
 * inputs and outputs). It has no counterpart in the reference. `problem->partials`
 * is ignored: the split scratch is a fixed 16 MiB array inside the library's
 * device image (held by every GPU that loads the library until the process
 * exits). Problems whose yvx_cuda_gqa_partials_bytes() exceeds
 * yvx_cuda_gqa_static_scratch_capacity() are refused with YVEX_ERR_BOUNDS and a
 * message in yvx_cuda_last_error_text(). The call itself performs no device or
 * host allocation. The first call on each device looks the array's address up
 * once (with that device current); make that first call before any stream
 * capture begins. All calls on a device share the one array and it keeps the
 * previous call's bytes: nothing in it has to start at zero, because every
 * partial the combine reads is written by the attention kernel of the same call,
 * but two calls that overlap on the GPU (different streams, or graphs replayed
 * concurrently) race on it. Serialise them. */
unsigned long long yvx_cuda_gqa_static_scratch_capacity(void);
int yvx_cuda_gqa_attention_static_scratch(const yvx_gqa_problem *problem, void *stream,
                                          unsigned int *launches);

/* ---- log-sum-exp combine of partial results ---------------------------------
 * parts: [items][part_count][head_dim + 2] holding (o normalised, m, l).
 * Used after the cross-GPU all-gather of sequence-sharded partials. No
 * counterpart in the reference (it has no split or sharded attention). */
int yvx_cuda_lse_combine(const float *parts, unsigned int items, unsigned int part_count,
                         unsigned int head_dim, void *output, int output_dtype,
                         int *status, void *stream);
/* The same with explicit strides (in floats): part j of item i starts at
 * parts + i*item_stride + j*part_stride. An all-gather of per-rank
 * [items][head_dim+2] buffers is [rank][items][head_dim+2], i.e. item_stride =
 * head_dim+2 and part_stride = items*(head_dim+2): no transpose is needed. */
int yvx_cuda_lse_combine_strided(const float *parts, unsigned int items, unsigned int part_count,
                                 unsigned int head_dim, unsigned long long item_stride,
                                 unsigned long long part_stride, void *output, int output_dtype,
                                 int *status, void *stream);

/* ---- single-head primitive (reference: yvex_attention_f32,
 * src/backend/cuda/kernels.cu:362-434, launched from
 * src/backend/cuda/ops.c:1717-1808) ----------------------------------------- */
int yvx_cuda_op_attention_f32(const float *query, const float *keys, const float *values,
                              unsigned long long seq_len, unsigned long long position,
                              float scale, int causal, unsigned long long head_dim,
                              float *scores, float *probabilities, float *out,
                              void *stream);

/* ---- shared-latent attention reduce ------------------------------------------------
 * Replaces the launch of yvex_attention_reduce_native
 * (src/backend/cuda/attention.c:1386-1422, kernel src/backend/cuda/attention_kernels.cu:
 * 259-406); the fields are that kernel's parameters with the same meaning. All heads
 * share one row per position (the row is key and value); sinks[head] seeds the softmax
 * maximum and adds exp(sink - max) to the denominator; pass 0 = local window rows
 * (positions in [pos+1-W, pos], or every local row when candidate_block_visible),
 * pass 1 = compressed rows (class 1: selected[token][0..selected_count), ratio 4;
 * class 2: all rows with position + ratio - 1 <= pos, ratio 128; class 0: none).
 * out = quotient rounded to bf16 (nearest even), stored as F32. status: 1 non-finite,
 * 2 contract. head_dim <= 512.
 * rope_frequency != NULL fuses what the reference runs after the reduce on every
 * published row (CPU: src/graph/core.c:498-507, yvex_attention_rope_apply
 * src/graph/numeric.c:919-949 with inverse = 1; CUDA: the yarn-rope launch of
 * src/backend/cuda/attention.c:1424-1451): the last rope_dims lanes, taken as adjacent
 * (x, y) pairs, are rotated by -position * rope_frequency[pair] in double precision,
 * narrowed to float and rounded to bf16 again. rope_frequency is a device array of
 * rope_dims / 2 doubles, radians per position (yvex_b200_rope_frequencies computes the
 * reference's values on the host); rope_dims and head_dim - rope_dims must be even. */
typedef struct yvx_latent_reduce_args {
    const float *query;                       /* [token][heads*head_dim] */
    const float *local;                       /* [initial_local_count + token_count][local_stride] */
    const unsigned long long *local_positions;
    unsigned long long initial_local_count, local_stride;
    const float *compressed;
    const unsigned long long *compressed_positions;
    unsigned long long compressed_stride;
    const unsigned long long *selected;
    const unsigned long long *selected_count;
    unsigned long long topk_capacity;
    const float *sinks;
    unsigned long long query_heads, head_dim, sliding_window, ratio;
    unsigned int attention_class;
    unsigned long long phase_start_position, token_count;
    int candidate_block_visible;
    float *out;                               /* [token][heads*head_dim] */
    int *status;
    unsigned long long rope_dims;             /* used when rope_frequency != NULL */
    const double *rope_frequency;             /* [rope_dims/2] or NULL */
    void *workspace;                          /* yvx_cuda_latent_reduce_workspace_bytes() bytes, or NULL */
} yvx_latent_reduce_args;
/* With a workspace the candidate list of a (token, head) is split over several CTAs when
 * the phase alone cannot fill the GPU (decode, short verify phases) and a second launch
 * folds the partial states and publishes; the split plan depends only on the arguments
 * and the SM count. workspace == NULL: one launch, one CTA per (token, 8 heads).
 * _workspace_bytes returns 0 when the plan has a single split (or the arguments are
 * refused). _launches is yvx_cuda_latent_reduce that also reports the launch count. */
unsigned long long yvx_cuda_latent_reduce_workspace_bytes(const yvx_latent_reduce_args *args);
int yvx_cuda_latent_reduce(const yvx_latent_reduce_args *args, void *stream);
int yvx_cuda_latent_reduce_launches(const yvx_latent_reduce_args *args, void *stream,
                                    unsigned int *launches);

/* ---- sparse index selection: scores + ranked top-k ---------------------------------
 * Replaces, for one phase, the reference's index scoring and top-k
 * (CPU: yvex_attention_csa_select src/graph/attention.c:369-497 and
 * yvex_attention_topk_select src/graph/numeric.c:1086-1150; CUDA stage: the compress /
 * indexer / topk launches of src/backend/cuda/attention.c:1237-1385). Row i of `keys`
 * belongs to compressed row i. For token t at position p = phase_start_position + t a
 * row is a candidate when positions[i] + ratio - 1 <= p; its score is
 *   (float)( 1/sqrt(heads) * 1/sqrt(head_dim) * sum_h weights[t][h] * max(0, q[t][h] . key_i) )
 * with the dot, the sum over heads and the two scalings in double precision in the
 * reference's order, so scores are bit-equal to the CPU reference. The candidates are
 * ranked by score descending (+0 equals -0), equal scores by ascending position, and
 * selected[t][0 .. selected_count[t]) receives the first min(candidates, topk) row
 * indices in ranked order: the lists yvx_cuda_latent_reduce reads for class 1.
 * Contract: positions strictly increasing (the reference refuses duplicate positions;
 * here unordered ones are refused as well), heads <= 64, head_dim <= 256, topk <= 1024,
 * rows < 2^31. scores [token][rows] receives every candidate's score. workspace:
 * yvx_cuda_csa_select_workspace_bytes() bytes. status: 1 non-finite, 2 contract.
 * Launches: 2 when rows <= 4096, else 3 or more. */
typedef struct yvx_csa_select_args {
    const float *keys;                        /* [rows][key_stride] */
    const unsigned long long *positions;      /* [rows] */
    unsigned long long rows, key_stride;
    const float *query;                       /* [token][heads*head_dim] */
    const float *weights;                     /* [token][heads] */
    unsigned int heads, head_dim, topk;
    unsigned long long ratio;
    unsigned long long phase_start_position, token_count;
    float *scores;                            /* [token][rows] */
    unsigned long long *selected;             /* [token][topk_capacity] */
    unsigned long long *selected_count;       /* [token] */
    unsigned long long topk_capacity;         /* >= topk */
    void *workspace;
    int *status;
} yvx_csa_select_args;
unsigned long long yvx_cuda_csa_select_workspace_bytes(unsigned long long rows,
                                                       unsigned long long token_count,
                                                       unsigned int topk);
int yvx_cuda_csa_select(const yvx_csa_select_args *args, void *stream, unsigned int *launches);

/* ---- rolling compressor over a chunk of tokens (one launch) -------------------------
 * Replaces the per-token state transition of the reference
 * (CPU: yvex_attention_rolling_state_step_cpu src/graph/attention.c:745-836; CUDA:
 * yvex_attention_rolling_state src/backend/cuda/kernels.cu:1536-1631, one launch of one
 * CTA per token) and, with norm_weights set, the publication chain that follows each
 * emission (src/graph/attention_execute.c:776-806: bf16 round, RMS norm with learned
 * weights, bf16 round, position rotation of the last rope_dims lanes at the group's first
 * position, bf16 round). The quantising activation step after the chain is not part of it.
 * A token row has state_width = head_dim * (overlap ? 2 : 1) lanes; the state has
 * state_slots = ratio * (overlap ? 2 : 1) rows of state_width lanes, packed. The token at
 * position p is stored with score token_score + ape[p % ratio]; each time p % ratio ==
 * ratio - 1 one row is emitted: per lane the softmax-weighted mean over the group's ratio
 * rows (lanes [head_dim, 2 head_dim) with overlap) and, with overlap, the previous group's
 * rows (lanes [0, head_dim)), in double precision in the reference's order. The cursor
 * and fills of the reference's state record follow from start_position. Every emission of
 * the chunk is computed in parallel; after_kv / after_score receive the state the
 * reference would hold after the last token, slot for slot, and must not alias the input
 * state. compressed [emitted][compressed_stride], positions [emitted] = first position of
 * each emitted group; the emitted count = (start_position % ratio + token_count) / ratio is
 * returned through *emitted. Contract: head_dim <= 1024 and even, rope_dims even and
 * <= head_dim. status: 1 non-finite input or emission. */
typedef struct yvx_compressor_args {
    unsigned long long ratio, head_dim;
    int overlap;
    unsigned long long start_position;
    unsigned long long token_count;
    const float *token_kv, *token_score;      /* [token][token_stride] */
    unsigned long long token_stride;
    const float *ape;                         /* [ratio][state_width] */
    const float *state_kv, *state_score;      /* [state_slots][state_width] */
    float *after_kv, *after_score;
    float *compressed;
    unsigned long long compressed_stride;
    unsigned long long *positions;            /* may be NULL */
    const float *norm_weights;                /* [head_dim]; NULL: raw emission */
    double epsilon;
    unsigned long long rope_dims;             /* 0: no rotation */
    const double *rope_frequency;             /* [rope_dims/2] radians per position */
    int *status;
    /* optional, behind the publication chain and in the same launch: the activation fake
     * quantisation of yvx_cuda_activation_quant over the first activation_count lanes of every
     * emitted row (0: none; needs the 16-byte row geometry, blocks of 4 << k <= 128 lanes, and
     * with the transform activation_count in (64, 128]; otherwise YVEX_ERR_UNSUPPORTED) */
    unsigned int activation_quantization;
    unsigned long long activation_count, activation_block_width;
    int activation_hadamard;
} yvx_compressor_args;
int yvx_cuda_compressor_chunk(const yvx_compressor_args *args, void *stream,
                              unsigned long long *emitted);

/* ---- activation fake quantisation of rows in place (one launch) -----------------------
 * Replaces yvex_attention_activation_apply (src/graph/core.c:829-945; CUDA stage:
 * yvex_attention_activation_quantize, src/backend/cuda/kernels.cu:1136). Applied by the reference to the non-rotated lanes
 * of new local rows and of emitted compressed rows (FP8, blocks of 64) and to index
 * queries and emitted index rows (Hadamard transform, then FP4, blocks of 32).
 * Per row of `count` lanes: with hadamard != 0 the row, zero-padded to a power of two, goes
 * through single-precision butterflies of growing stride and its first count lanes are
 * multiplied by hadamard_scale (the caller passes 1.0f / sqrtf((float)count)); then per
 * block of block_width lanes: amax = max(|x|, floor) with floor 1e-4 (FP8) or 6 * 2^-126
 * (FP4), scale = amax / 448 (FP8) or amax / 6 (FP4) rounded up to a power of two, each
 * lane replaced by bf16(nearest(x / scale) * scale), nearest = the closest FP8 E4M3 (FP4
 * E2M1) value, exact ties to the even code. Every step is exact or a single rounding, so
 * results are bit-equal to the reference's. quantization: 8 or 4. Contract: count a
 * multiple of block_width (else YVEX_ERR_BOUNDS), count <= 8192, block_width <= 1024.
 * status: 1 when a lane is not finite. */
typedef struct yvx_activation_args {
    float *values;                            /* [rows][row_stride], first count lanes of each row */
    unsigned long long rows, row_stride, count;
    unsigned int quantization, block_width;
    int hadamard;
    float hadamard_scale;
    int *status;
} yvx_activation_args;
int yvx_cuda_activation_quant(const yvx_activation_args *args, void *stream);

/* ---- publication chain of projected rows of the latent attention (one launch) ---------
 * Replaces, for the rows a projection has produced, the per-row sequence of the reference
 * (CPU: src/graph/attention_execute.c:527-612 and :970-1003; CUDA: the weighted_norm /
 * unit norm, rope and activation launches of src/backend/cuda/attention.c:1162-1236):
 *   norm_mode 1: RMS norm without weights, 2: with learned weights; then bf16 publication
 *   rope_dims > 0: rotation of the last rope_dims lanes (adjacent pairs) at the row's token
 *     position, then bf16 publication of the row
 *   quantization 8 / 4: the activation fake quantisation of yvx_cuda_activation_quant over the
 *     first activation_count lanes
 * Query heads take (1, rope, none); new local rows (2, rope, FP8 on the lanes in front of the
 * rotated ones); index queries (0, rope, transform + FP4 on the whole head). Row r belongs to
 * the token at start_position + r / rows_per_token. Sums of squares and the scaling run in
 * double precision, the rotation as in yvx_cuda_latent_reduce. Contract: width a multiple of 4
 * and at most 1024, rows 16-byte aligned, rope_dims even, activation blocks of 4 << k <= 128
 * lanes; with the transform activation_count in (64, 128]. status: 1 non-finite. */
typedef struct yvx_rows_publish_args {
    float *values;                            /* [rows][row_stride] */
    unsigned long long rows, rows_per_token, row_stride, width;
    int norm_mode;
    const float *norm_weights;                /* [width] */
    double epsilon;
    unsigned long long rope_dims;
    const double *rope_frequency;             /* [rope_dims/2] */
    unsigned long long start_position;
    unsigned int quantization;
    unsigned long long activation_count, block_width;
    int hadamard;
    int *status;
} yvx_rows_publish_args;
int yvx_cuda_rows_publish(const yvx_rows_publish_args *args, void *stream);
/* Up to four row sets in ONE launch (a decode step publishes its query heads, its new local
 * row and its index queries); each set as in yvx_cuda_rows_publish, results identical. */
int yvx_cuda_rows_publish_batch(const yvx_rows_publish_args *sets, unsigned int count, void *stream);

/* ---- a session's KV history between the block pool and the reference's state bank ------
 * The reference keeps a layer's state in one byte buffer per bank with the components
 * [values, positions, auxiliary] at 8-byte aligned offsets (src/runtime/state_residency.c:
 * 346-395; yvex_b200_kv_bank_layout restates the offsets), values = F32 rows
 * [row][K heads | V heads], positions = u64 per row; that bank is what its checkpoints carry
 * (src/runtime/state_store.c:1-9). export: rows [0, kv_tokens[b]) of every session go from the
 * bf16 pools behind the block table into the bank (positions[row] = position_base + row);
 * import: the other way. Exact both ways for the bf16-representable values the reference
 * stores; importing a value bf16 cannot hold is status 2. */
typedef struct yvx_kv_bank_args {
    unsigned int sessions, kv_heads, head_dim;
    const int *kv_tokens;                     /* device [session] rows held; NULL: uniform */
    unsigned int kv_tokens_uniform;
    unsigned int row_capacity;                /* rows a session's bank holds */
    void *bank;                               /* [session] banks, bank_session_bytes apart */
    unsigned long long bank_session_bytes, values_offset, positions_offset, value_width;
    unsigned long long position_base;
    void *key_pool, *value_pool;              /* bf16 */
    const int *block_table;
    unsigned int block_tokens, block_table_stride, pool_blocks;
    unsigned long long pool_token_stride, pool_head_stride, pool_block_stride;
    int *status;
} yvx_kv_bank_args;
int yvx_cuda_kv_bank_transfer(const yvx_kv_bank_args *args, int export_direction, void *stream);

/* ---- projections of the encoded attention operator ---------------------------------
 * Encoded weight rows times activation rows. Replaces, for the admitted encodings, the
 * reference's yvex_qtype_matvec / yvex_qtype_grouped_rows launches
 * (src/backend/cuda/kernels.cu:436-866) as src/backend/cuda/attention.c:1162-1236 and
 * :1424-1451 use them; CPU twin yvex_attention_dot_batch (src/graph/core.c:1107-1215):
 * every lane decoded to float, products and sum in double, narrowed to float, and with
 * round_bf16 published as bf16 (nearest even). qtype: the GGUF type ids of the reference
 * (include/yvex/qtype.h:20-50); F32, F16, BF16 and Q8_0 are admitted, every other id is
 * YVEX_ERR_UNSUPPORTED. output[t][g * rows + r] = weights row (first_row + g * rows + r)
 * . input[t][g * width .. (g + 1) * width); groups 0 or 1 is the plain product.
 * status: 1 when a result is not finite. */
#define YVX_QTYPE_F32 0u
#define YVX_QTYPE_F16 1u
#define YVX_QTYPE_Q8_0 8u
#define YVX_QTYPE_BF16 30u
typedef struct yvx_matvec_args {
    const void *weights;                      /* encoded rows, row_bytes apart */
    unsigned int qtype;
    unsigned long long first_row, rows, width, row_bytes;
    const float *input;                       /* [tokens][input_stride] */
    unsigned long long tokens, input_stride;
    float *output;                            /* [tokens][output_stride] */
    unsigned long long output_stride;
    unsigned long long groups;
    int round_bf16;
    int *status;
} yvx_matvec_args;
unsigned long long yvx_cuda_qtype_row_bytes(unsigned int qtype, unsigned long long width);
int yvx_cuda_qtype_matvec(const yvx_matvec_args *args, void *stream);
/* The same projection at prefill-sized token counts on the tensor cores (tcgen05, F32
 * accumulation in tensor memory): BF16-encoded weight rows, activation rows that bf16 holds
 * exactly (anything else raises status 2 and the output is not to be used), the bf16
 * publication fused into the epilogue (round_bf16). A published value differs from
 * yvx_cuda_qtype_matvec's (the CPU twin's exact sum) by at most one bf16 step. Groups as
 * above. `staging` holds the activations as bf16: yvx_cuda_bf16_gemm_staging_bytes(). Two
 * launches. width a multiple of 8, input 8-byte aligned with an even stride. */
typedef struct yvx_gemm_args {
    const void *weights;                      /* BF16 rows, 2 * width bytes apart, 16-byte aligned */
    unsigned long long first_row, rows, width;
    const float *input;                       /* [tokens][input_stride] */
    unsigned long long tokens, input_stride;
    float *output;                            /* [tokens][output_stride] */
    unsigned long long output_stride;
    unsigned long long groups;
    int round_bf16;
    void *staging;
    int *status;
} yvx_gemm_args;
unsigned long long yvx_cuda_bf16_gemm_staging_bytes(unsigned long long tokens, unsigned long long groups,
                                                    unsigned long long width);
int yvx_cuda_bf16_gemm(const yvx_gemm_args *args, void *stream);
/* Encoded rows [first_row, first_row + rows) decoded to F32 [rows][width] (norm weights,
 * sinks, position biases: yvex_attention_decode_row, src/graph/core.c:1029-1105). */
int yvx_cuda_qtype_decode_rows(const void *weights, unsigned int qtype, unsigned long long first_row,
                               unsigned long long rows, unsigned long long width, float *out, int *status,
                               void *stream);
/* bf16 publication in place of the first `width` lanes of F32 rows (yvex_attention_compute_round,
 * src/graph/numeric.c:614-628). status: 1 when a lane is not finite. */
int yvx_cuda_round_bf16_rows(float *values, unsigned long long rows, unsigned long long width,
                             unsigned long long row_stride, int *status, void *stream);

/* ---- KV append with rotary embedding (one launch per step) ---------------------------
 * Replaces, for the new rows of a step, the two rotate-half launches on Q and K
 * (yvex_cuda_transformer_rotary_half / _rotary_half_f32, src/backend/cuda/transformer.c:
 * 413-469; kernels src/backend/cuda/transformer_kernels.cu:78-134; called from
 * src/runtime/decoder.c:1112-1131) and the per-token device copies of K and V into the
 * state bank with the position upload (stateful_copy_projection,
 * src/runtime/stateful_attention.c:183-243).
 * Q is rotated in place; K is rotated on its way into the history; V is copied.
 * cosines / sines are the explicit tables the reference passes, [session][token][rotary_dim];
 * pair p of a head is (p, p + rotary_dim/2), dims >= rotary_dim are left alone.
 * staged_bf16 != 0: products and sum rounded to bf16 (yvex_rotary_half_f32 kernel, the
 * decoder's variant); 0: plain single precision, no fused multiply-add.
 * Row of session b's token t: kv_tokens[b] + t. Destination A (state_values != NULL): F32
 * rows [row][K heads | V heads] with state_row_stride floats between rows, and
 * state_positions[b][row] = token_position[b] + t (NULL: kv_tokens[b] + t).
 * Destination B (key_pool != NULL): bf16 pools behind a block table, strides in
 * elements, values rounded to nearest even. Either or both may be given.
 * status: 2 when a block-table entry lies outside the pool (the row is skipped). */
typedef struct yvx_kv_append_args {
    unsigned int sessions, tokens;            /* new rows per session */
    unsigned int query_heads, kv_heads, head_dim, rotary_dim;
    int staged_bf16;
    float *query;                             /* [session][token][query_heads*head_dim] or NULL */
    const float *key, *value;                 /* [session][token][kv_heads*head_dim] */
    const float *cosines, *sines;             /* [session][token][rotary_dim] */
    const int *kv_tokens;                     /* [session] rows already present; NULL: uniform */
    unsigned int kv_tokens_uniform;
    float *state_values;
    unsigned long long state_session_stride, state_row_stride;
    unsigned long long *state_positions;
    unsigned long long state_position_stride;
    const unsigned long long *token_position;
    void *key_pool, *value_pool;
    const int *block_table;
    unsigned int block_tokens, block_table_stride, pool_blocks;
    unsigned long long pool_token_stride, pool_head_stride, pool_block_stride;
    int *status;
    /* Rows a session's state bank can hold (0: unbounded). A row at or beyond it, or beyond
     * block_table_stride * block_tokens for the pools, is refused on the device: status 2,
     * nothing of that row written. */
    unsigned int row_capacity;
} yvx_kv_append_args;
int yvx_cuda_kv_append_rotary(const yvx_kv_append_args *args, void *stream);

/* ---- latent-compressed (MLA-style) decode -----------------------------------------
 * One query token per session; every query head attends over ONE shared row per
 * position: score = scale * (q_lat[h] . latent[t] + q_rope[h] . rope_key[t]),
 * out[h] = sum_t softmax_t(score) * latent[t]. The up-projection is absorbed into
 * the query first: q_lat[h] = bf16(q_nope[h] . W_uk[h]) (f32 accumulation).
 * The reference's latent path (yvex_attention_reduce_native,
 * src/backend/cuda/attention_kernels.cu:259-406) keeps its rope dimensions inside
 * the shared row and has no absorbed projection; this variant is an extension.
 * Shapes: heads 128, nope 128, latent 512, rope 64, all bf16; output f32.
 * Strides are elements. */
typedef struct yvx_mla_problem {
    unsigned int sessions, heads, nope_dim, latent_dim, rope_dim;
    float scale;
    const void *q_nope;    /* bf16 [session][head][nope_dim] */
    const void *q_rope;    /* bf16 [session][head][rope_dim] */
    const void *w_uk;      /* bf16 [head][nope_dim][latent_dim] */
    const void *latent;    /* bf16 [session][token][latent_dim] */
    const void *rope_key;  /* bf16 [session][token][rope_dim] */
    unsigned long long latent_session_stride, rope_session_stride;
    const unsigned int *kv_tokens; /* device [sessions]; NULL = uniform */
    unsigned int kv_tokens_uniform, kv_tokens_max;
    unsigned int chunk_tokens, max_splits; /* filled by yvx_cuda_mla_plan */
    /* Filled by yvx_cuda_mla_plan. Nonzero (uniform lengths only): the sessions' tiles are laid end to end and
     * cut into this many equal runs, one per pair of CTAs, so a pair may finish one session and start the next
     * and every SM has work; max_splits is then the largest number of runs a session is cut into. Zero: a
     * grid of sessions x splits of chunk_tokens. */
    unsigned int balanced_pairs;
    /* Filled by yvx_cuda_mla_plan: 4 = the attention kernel runs as clusters of four CTAs, each with a quarter of the
     * latent columns (grid 4 x splits x sessions; with max_splits == 1 the result is written by the kernel itself:
     * no partial rows, no combine launch); 0 or 2 = pairs of CTAs with half of the columns each. */
    unsigned int cluster_ctas;
    void *q_absorbed;      /* scratch bf16 [session][head][latent_dim + rope_dim] */
    float *partials;       /* scratch [session][head][2][max_splits][latent_dim/2 + 2] ([4][..][latent_dim/4 + 2] with cluster_ctas 4) */
    float *output;         /* f32 [session][head][latent_dim] */
    int *status;
} yvx_mla_problem;
void yvx_cuda_mla_plan(yvx_mla_problem *problem, int sm_count);
unsigned long long yvx_cuda_mla_absorbed_bytes(const yvx_mla_problem *problem);
unsigned long long yvx_cuda_mla_partials_bytes(const yvx_mla_problem *problem);
/* Absorb, attention, combine: 3 launches. events (optional, 4 cudaEvent_t as
 * void*): before absorb, after absorb, after attention, after combine. */
int yvx_cuda_mla_decode(const yvx_mla_problem *problem, void *stream, void *events[4],
                        unsigned int *launches);

/* ---- Q8_0 KV records -----------------------------------------------------------
 * No counterpart in the reference (its KV state is F32; Q8_0 exists there as a
 * weight qtype only: src/gguf/quant_block.c:160-187,819-832). A record is the
 * Q8_0 data of 64 tokens of one KV head (head_dim 128) as 17408 contiguous
 * bytes, a byte permutation of the tokens' GGUF Q8_0 rows in which every lane byte
 * has its top bit flipped (a stored lane is int8 + 128, the operand form of the
 * kernel's byte-to-f16 placement; scales are the GGUF f16 bits unchanged):
 *   [K lanes 8192][V lanes 8192][K scales 512][V scales 512]
 * K lane of (token t, dim d): ((t/8*2 + d/64)*32 + (t%8)*4 + (d%16%8)/2)*16
 *                              + (d%64/16)*4 + (d%2) + 2*(d%16/8)
 * V lane of (t, d): 8192 + (((t/16*4 + d/32)*32 + (d%8)*4 + (t%16%8)/2)*4 + d/8%4)*4
 *                              + (t%2) + 2*(t%16/8)
 * K scale of (t, 32-lane block q): 16384 + (t*4 + q)*2
 * V scale of (t, q): 16896 + (((t/16*4 + (t%16%8)/2)*4 + q)*4 + (t%2) + 2*(t%16/8))*2
 * yvx_cuda_q8_kv_pack scatters `tokens` GGUF Q8_0 rows ([token][kv_heads*4*34]
 * bytes, K and V) starting at absolute token `first_token` of a session into
 * its records; block_ids maps the session's block index to a pool block (NULL =
 * identity). Records must be zero-filled before their first token is packed. */
unsigned long long yvx_cuda_q8_record_bytes(void);
int yvx_cuda_q8_kv_pack(const void *k_rows, const void *v_rows, unsigned int tokens,
                        unsigned int kv_heads, void *records, const int *block_ids,
                        unsigned long long block_stride, unsigned long long head_stride,
                        unsigned int first_token, void *stream);

/* ---- seeded device-side fills for benchmark workloads ------------------------
 * No counterpart in the reference. Counter-based (splitmix64 of seed and
 * element index): N(0, sigma^2) as F32 or BF16 (dtype = -YVEX_DTYPE_F32: F32 storage of
 * values rounded to bf16, what the reference's linears publish), int8 lanes uniform in
 * [-127, 127], f16 values uniform in [lo, hi). */
int yvx_cuda_fill_normal(void *dst, int dtype, unsigned long long count,
                         unsigned long long seed, float sigma, void *stream);
/* The F32 values yvx_cuda_fill_normal draws for the same seed, rotated before the bf16
 * rounding: rows [session][token][head][dim], position = token index, rotate-half pairs
 * (lane, lane + dim/2), frequency theta^(-2 pair/dim), cosine / sine rounded to bf16 (the
 * convention of the reference's rotary tables, src/runtime/decoder.c:1080-1094). */
int yvx_cuda_fill_normal_rope_bf16(void *dst, unsigned long long rows, unsigned int tokens,
                                   unsigned int heads, unsigned int dim, unsigned long long seed,
                                   float sigma, double theta, void *stream);
int yvx_cuda_fill_q8_lanes(void *dst, unsigned long long count, unsigned long long seed,
                           void *stream);
int yvx_cuda_fill_f16_uniform(void *dst, unsigned long long count, unsigned long long seed,
                              float lo, float hi, void *stream);
/* Whole Q8 records: uniform lanes in the lane regions, f16 scales uniform in
 * [lo, hi) in the scale regions. */
int yvx_cuda_fill_q8_records(void *records, unsigned long long record_count,
                             unsigned long long seed, float lo, float hi, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* YVEX_B200_CUDA_SHIM_H */
