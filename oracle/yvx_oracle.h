/* TEST INFRASTRUCTURE ONLY.
 *
 * CPU restatement of the YVEX reference's attention arithmetic. It is the
 * checker for the CUDA path: only the test-suite, the smoke check and the
 * benchmark's CPU-baseline leg may build, load or call it. Nothing in the
 * shipped library links against it and it is never a fallback.
 *
 * Parity status: pinned. Each function is checked against the reference's own
 * golden vectors (tests/golden/) and, where the reference's CPU sources are
 * available at build time, against the reference's compiled code
 * (oracle/_ref/libyvex_ref.so) on random inputs.
 */
#ifndef YVX_ORACLE_H
#define YVX_ORACLE_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Scalar codecs. */
float yvx_oracle_bf16_decode(unsigned short bits);
unsigned short yvx_oracle_bf16_encode(float value);
float yvx_oracle_f16_decode(unsigned short bits);
unsigned short yvx_oracle_f16_encode(float value);
void yvx_oracle_bf16_decode_array(const unsigned short *bits, float *out, size_t count);
void yvx_oracle_bf16_encode_array(const float *values, unsigned short *out, size_t count);

/* Q8_0 block codec over GGUF rows: 34-byte blocks, [f16 scale][32 x int8]. */
int yvx_oracle_q8_0_encode_block(const float *source, unsigned char *encoded);
int yvx_oracle_q8_0_decode_block(const unsigned char *encoded, float *out);
int yvx_oracle_q8_0_decode_rows(const unsigned char *encoded, float *out,
                                size_t elements);

/* The reference CPU exponential and the single-head attention primitive. */
double yvx_oracle_exp(double x);
int yvx_oracle_op_attention(const float *query, const float *keys,
                            const float *values, unsigned long long seq_len,
                            unsigned long long position, float scale, int causal,
                            unsigned long long head_dim, float *score_scratch,
                            float *probability_scratch, float *out);

/* Grouped-query attention assembled from the primitive, one call per
 * (query row, query head). Strides are in elements; zero means packed. */
int yvx_oracle_gqa_attention(const float *query, const float *key,
                             const float *value, float *output,
                             unsigned long long query_tokens,
                             unsigned long long key_value_tokens,
                             unsigned long long query_start,
                             unsigned long long query_heads,
                             unsigned long long key_value_heads,
                             unsigned long long head_dimension,
                             unsigned long long query_stride,
                             unsigned long long key_stride,
                             unsigned long long value_stride, float scale,
                             int causal, unsigned int threads);

/* The single-precision scalar oracle the reference's CUDA tests compare with. */
void yvx_oracle_gqa_f32_reference(const float *query, const float *key,
                                  const float *value, float *output,
                                  unsigned long long query_tokens,
                                  unsigned long long key_value_tokens,
                                  unsigned long long query_start,
                                  unsigned long long query_heads,
                                  unsigned long long key_value_heads,
                                  unsigned long long head_dimension, int causal);

/* Block-table addressing: logical row -> pool row. */
unsigned long long yvx_oracle_block_row(const int *block_table,
                                        unsigned long long block_tokens,
                                        unsigned long long row);
void yvx_oracle_block_gather_u16(const unsigned short *pool, const int *block_table,
                                 unsigned long long block_tokens,
                                 unsigned long long rows,
                                 unsigned long long row_elements,
                                 unsigned short *out);

/* KV page geometry (integer, bit-exact). */
typedef struct {
    unsigned long long logical_block_tokens, kernel_tile_tokens;
    unsigned long long promotion_granularity_tokens, alignment_bytes;
    unsigned long long bytes_per_block, page_table_entry_bytes;
    unsigned long long device_page_bytes, logical_tokens;
    int copy_on_write, candidate_extent;
} yvx_oracle_page_request;
int yvx_oracle_page_tokens(const yvx_oracle_page_request *request,
                           unsigned long long *page_tokens,
                           unsigned long long *page_bytes);
int yvx_oracle_page_touch(unsigned long long element_start,
                          unsigned long long element_count,
                          unsigned long long page_elements,
                          unsigned long long *first_page,
                          unsigned long long *last_page);

/* Shared-latent (K == V) reduction with a per-head sink logit. */
int yvx_oracle_latent_reduce(const float *query, const float *rows,
                             const float *sinks, float *out,
                             unsigned long long query_tokens,
                             unsigned long long row_count,
                             unsigned long long query_start,
                             unsigned long long query_heads,
                             unsigned long long head_dimension,
                             unsigned long long row_stride, int round_bf16);

/* The reduce stage's full argument set (window + compressed rows, sink). */
typedef struct {
    const float *query;                       /* [token][heads*head_dim] */
    const float *local;                       /* [initial_local_count + token_count][local_stride] */
    const unsigned long long *local_positions;
    unsigned long long initial_local_count, local_stride;
    const float *compressed;                  /* [rows][compressed_stride] */
    const unsigned long long *compressed_positions;
    unsigned long long compressed_stride;
    const unsigned long long *selected;       /* [token][topk_capacity] (class 1) */
    const unsigned long long *selected_count; /* [token] (class 1) */
    unsigned long long topk_capacity;
    const float *sinks;                       /* [heads] */
    unsigned long long query_heads, head_dim, sliding_window, ratio;
    unsigned int attention_class;             /* 0 window only, 1 selected rows, 2 all rows */
    unsigned long long phase_start_position, token_count;
    int candidate_block_visible;
    float *device_out;                        /* unused here: keeps the device library's layout */
    int *device_status;                       /* unused here */
    unsigned long long rope_dims;             /* 0: publish without the output rotation */
    const double *rope_frequency;             /* [rope_dims/2] radians per position */
    void *device_workspace;                   /* unused here */
} yvx_oracle_latent_args;
int yvx_oracle_latent_reduce_full(const yvx_oracle_latent_args *args, float *out);

/* Position rotation of the last rope_dims lanes (adjacent pairs), the frequencies
 * behind it, the sparse index scores and the ranked top-k selection. */
typedef struct {
    unsigned long long theta, scaling_factor, original_context, beta_fast, beta_slow;
} yvx_oracle_position_policy;
int yvx_oracle_rope_frequencies(const yvx_oracle_position_policy *policy,
                                unsigned long long rope_dims, double *frequency);
int yvx_oracle_rope_apply(float *values, unsigned long long count, unsigned long long rope_dims,
                          unsigned long long token_position, const double *frequency, int inverse);
typedef struct {
    const float *keys;                        /* [rows][key_stride], one per compressed row */
    const unsigned long long *positions;      /* [rows] */
    unsigned long long rows, key_stride;
    const float *query;                       /* [token][heads*head_dim] */
    const float *weights;                     /* [token][heads] */
    unsigned long long heads, head_dim, topk, ratio;
} yvx_oracle_indexer;
int yvx_oracle_topk_select(const float *scores, const unsigned long long *ordinals,
                           unsigned long long count, unsigned long long k,
                           unsigned long long *selected, unsigned long long *selected_count);
int yvx_oracle_csa_select(const yvx_oracle_indexer *indexer, unsigned long long token,
                          unsigned long long query_position, unsigned long long *selected,
                          unsigned long long *selected_count, unsigned long long *valid_count,
                          float *scores_out);

/* Rolling compressor: the per-token state transition that turns every `ratio`
 * projected rows into one compressed row (softmax-weighted mean per lane), run
 * over a chunk of tokens, with the publication chain that follows an emission
 * (bf16 round, RMS norm, bf16 round, position rotation, bf16 round). */
typedef struct {
    unsigned long long ratio, head_dim;
    int overlap;                              /* 1: two halves (sparse class, main and indexer rows) */
    unsigned long long start_position;        /* tokens already consumed by the state */
    unsigned long long token_count;
    const float *token_kv, *token_score;      /* [token][token_stride], state_width lanes used */
    unsigned long long token_stride;
    const float *ape;                         /* [ratio][state_width], row = position % ratio */
    const float *state_kv, *state_score;      /* [state_slots][state_width] before the chunk */
    float *after_kv, *after_score;            /* [state_slots][state_width] after it */
    float *compressed;                        /* [emitted][compressed_stride] */
    unsigned long long compressed_stride;
    unsigned long long *positions;            /* [emitted] first token of each emitted group */
    const float *norm_weights;                /* [head_dim]; NULL: raw emission, no publication chain */
    double epsilon;
    unsigned long long rope_dims;             /* with norm_weights: 0 skips the rotation */
    const double *rope_frequency;             /* [rope_dims/2] */
    int *device_status;                       /* unused here: keeps the device library's layout */
} yvx_oracle_compressor_args;
/* state_width = head_dim * (overlap ? 2 : 1), state_slots = ratio * (overlap ? 2 : 1).
 * Returns 1 and the number of emitted rows, 0 on a refusal. */
int yvx_oracle_compressor_chunk(const yvx_oracle_compressor_args *args,
                                unsigned long long *emitted);

/* Activation fake quantisation of a row in place: an optional Hadamard transform over the
 * whole row (zero-padded to a power of two, scaled by 1/sqrt(count)), then per block of
 * block_width lanes a power-of-two scale, the nearest FP8 E4M3 (quantization 8) or FP4
 * E2M1 (quantization 4) value with ties to the even code, and the product rounded to bf16. */
int yvx_oracle_activation_quant(float *values, unsigned long long count, unsigned int quantization,
                                unsigned long long block_width, int hadamard);

/* The chain the reference runs on every projected row of the latent attention before it is
 * attended or stored (query heads, new local rows, index queries): an optional RMS norm
 * (norm_mode 1: unit, 2: learned weights) with bf16 publication, an optional position
 * rotation of the last rope_dims lanes with bf16 publication, an optional activation fake
 * quantisation of the first activation_count lanes. Row r belongs to the token at
 * start_position + r / rows_per_token. Returns 1, or 0 on a refusal. */
typedef struct {
    float *values;                            /* [rows][row_stride], width lanes used */
    unsigned long long rows, rows_per_token, row_stride, width;
    int norm_mode;
    const float *norm_weights;                /* [width] for norm_mode 2 */
    double epsilon;
    unsigned long long rope_dims;             /* 0: no rotation */
    const double *rope_frequency;             /* [rope_dims/2] */
    unsigned long long start_position;
    unsigned int quantization;                /* 0 none, 8, 4 */
    unsigned long long activation_count, block_width;
    int hadamard;
    int *device_status;                       /* unused here */
} yvx_oracle_publish_args;
int yvx_oracle_rows_publish(const yvx_oracle_publish_args *args);

/* Latent decode with a separate rope key and an absorbed up-projection. */
int yvx_oracle_mla_decode(const unsigned short *q_nope_bf16,
                          const unsigned short *q_rope_bf16,
                          const unsigned short *w_uk_bf16,
                          const unsigned short *latent_bf16,
                          const unsigned short *rope_key_bf16, float *out,
                          unsigned long long heads, unsigned long long nope_dim,
                          unsigned long long latent_dim,
                          unsigned long long rope_dim,
                          unsigned long long context, float scale,
                          float *absorbed_query_out);

/* Rotate-half with explicit tables (bf16-staged or plain) and the decoder's tables. */
int yvx_oracle_rotary_half(float *values, const float *cosines, const float *sines,
                           unsigned long long tokens, unsigned long long heads,
                           unsigned long long head_dim, unsigned long long rotary_dim, int staged);
int yvx_oracle_rope_tables(unsigned long long token_start, unsigned long long tokens,
                           unsigned long long width, double theta, float *cosines, float *sines);

/* Full attention over interleaved [row][head][Q|K|V][width] rows, single precision. */
int yvx_oracle_full_attention_f32(const float *qkv, unsigned long long rows,
                                  unsigned long long heads, unsigned long long head_width,
                                  float *output, float *scratch);

/* Encoded weight rows (GGUF ids F32 0, F16 1, Q8_0 8, BF16 30): decode, row dot in double,
 * and the batch product the projections of the encoded attention operator are made of. */
unsigned long long yvx_oracle_qtype_row_bytes(unsigned int qtype, unsigned long long width);
int yvx_oracle_qtype_decode_row(unsigned int qtype, const unsigned char *encoded,
                                unsigned long long width, float *out);
int yvx_oracle_qtype_dot(unsigned int qtype, const unsigned char *encoded, unsigned long long width,
                         const float *vector, float *out);
int yvx_oracle_qtype_matvec(unsigned int qtype, const unsigned char *encoded,
                            unsigned long long first_row, unsigned long long rows,
                            unsigned long long width, const float *input, unsigned long long tokens,
                            unsigned long long input_stride, float *output,
                            unsigned long long output_stride, int round_bf16);

#ifdef __cplusplus
}
#endif
#endif /* YVX_ORACLE_H */
