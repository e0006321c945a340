/* TEST INFRASTRUCTURE ONLY: CPU restatement of the YVEX reference's attention
 * arithmetic, used as the checker for the CUDA path. Never shipped, never a
 * fallback. Parity status: pinned (see yvx_oracle.h).
 *
 * Citations name the reference file and lines each function follows.
 */
#ifndef _GNU_SOURCE
#define _GNU_SOURCE
#endif
#include "yvx_oracle.h"

#include <limits.h>
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- scalar codecs ------------------------------------------------------ */

/* src/gguf/quant_scalar.c:123-128: bf16 is the upper half of binary32. */
float yvx_oracle_bf16_decode(unsigned short bits)
{
    uint32_t wide = (uint32_t)bits << 16;
    float out;
    memcpy(&out, &wide, sizeof(out));
    return out;
}

/* src/gguf/quant_scalar.c:130-143: round to nearest even; NaNs are quieted by
 * setting the top mantissa bit of the truncated pattern. */
unsigned short yvx_oracle_bf16_encode(float value)
{
    uint32_t bits, high, low;
    memcpy(&bits, &value, sizeof(bits));
    high = bits >> 16;
    low = bits & 0xffffu;
    if ((bits & 0x7f800000u) == 0x7f800000u && (bits & 0x007fffffu))
        return (unsigned short)(high | 0x0040u);
    if (low > 0x8000u || (low == 0x8000u && (high & 1u))) high += 1u;
    return (unsigned short)high;
}

/* src/gguf/quant_scalar.c:40-68: binary16 widening, subnormals normalised. */
float yvx_oracle_f16_decode(unsigned short bits)
{
    uint32_t sign = ((uint32_t)bits & 0x8000u) << 16;
    uint32_t exponent = ((uint32_t)bits >> 10) & 0x1fu;
    uint32_t mantissa = (uint32_t)bits & 0x3ffu;
    uint32_t wide;
    float out;
    if (exponent == 0u) {
        if (!mantissa) {
            wide = sign;
        } else {
            uint32_t shift = 0u;
            while (!(mantissa & 0x400u)) {
                mantissa <<= 1;
                ++shift;
            }
            wide = sign | ((113u - shift) << 23) | ((mantissa & 0x3ffu) << 13);
        }
    } else if (exponent == 0x1fu) {
        wide = sign | 0x7f800000u | (mantissa << 13);
        if (mantissa) wide |= 0x00400000u;
    } else {
        wide = sign | ((exponent + 112u) << 23) | (mantissa << 13);
    }
    memcpy(&out, &wide, sizeof(out));
    return out;
}

/* src/gguf/quant_scalar.c:75-121: binary32 -> binary16, nearest even,
 * overflow to infinity, canonical quiet NaN payload. */
unsigned short yvx_oracle_f16_encode(float value)
{
    uint32_t bits, sign, exponent, mantissa, packed, tail;
    memcpy(&bits, &value, sizeof(bits));
    sign = (bits >> 16) & 0x8000u;
    exponent = (bits >> 23) & 0xffu;
    mantissa = bits & 0x007fffffu;
    if (exponent == 0xffu) {
        if (!mantissa) return (unsigned short)(sign | 0x7c00u);
        return (unsigned short)(sign | 0x7e00u | ((mantissa >> 13) & 0x1ffu));
    }
    if (exponent > 142u) return (unsigned short)(sign | 0x7c00u);
    if (exponent < 113u) {
        uint32_t significand, shift, quotient, rest, half;
        if (exponent < 102u) return (unsigned short)sign;
        significand = mantissa | 0x00800000u;
        shift = 126u - exponent;
        quotient = significand >> shift;
        rest = significand & ((1u << shift) - 1u);
        half = 1u << (shift - 1u);
        if (rest > half || (rest == half && (quotient & 1u))) quotient += 1u;
        return (unsigned short)(sign | quotient);
    }
    packed = ((exponent - 112u) << 10) | (mantissa >> 13);
    tail = mantissa & 0x1fffu;
    if (tail > 0x1000u || (tail == 0x1000u && (packed & 1u))) packed += 1u;
    if ((packed & 0x7c00u) == 0x7c00u) packed &= 0x7c00u;
    return (unsigned short)(sign | packed);
}

void yvx_oracle_bf16_decode_array(const unsigned short *bits, float *out, size_t count)
{
    size_t i;
    for (i = 0; i < count; ++i) out[i] = yvx_oracle_bf16_decode(bits[i]);
}

void yvx_oracle_bf16_encode_array(const float *values, unsigned short *out, size_t count)
{
    size_t i;
    for (i = 0; i < count; ++i) out[i] = yvx_oracle_bf16_encode(values[i]);
}

/* ---- Q8_0 --------------------------------------------------------------- */

enum { Q8_0_ELEMENTS = 32, Q8_0_BYTES = 34 };

static unsigned short load_u16le(const unsigned char *p)
{
    return (unsigned short)((unsigned int)p[0] | ((unsigned int)p[1] << 8));
}

/* src/gguf/quant_block.c:160-187: scale = amax/127 stored as f16 and re-read,
 * lanes = roundf(x / scale) clamped to [-127, 127]. */
int yvx_oracle_q8_0_encode_block(const float *source, unsigned char *encoded)
{
    float amax = 0.0f, scale, inverse;
    unsigned short packed;
    unsigned int i;
    for (i = 0; i < Q8_0_ELEMENTS; ++i) {
        float magnitude = fabsf(source[i]);
        if (magnitude > amax) amax = magnitude;
    }
    packed = yvx_oracle_f16_encode(amax / 127.0f);
    encoded[0] = (unsigned char)(packed & 0xffu);
    encoded[1] = (unsigned char)(packed >> 8);
    scale = yvx_oracle_f16_decode(packed);
    if (!isfinite(scale) || scale < 0.0f || (amax > 0.0f && scale == 0.0f)) return 0;
    inverse = scale != 0.0f ? 1.0f / scale : 0.0f;
    for (i = 0; i < Q8_0_ELEMENTS; ++i) {
        int lane = (int)roundf(source[i] * inverse);
        if (lane < -127) lane = -127;
        if (lane > 127) lane = 127;
        encoded[2 + i] = (unsigned char)(lane < 0 ? 256 + lane : lane);
    }
    return 1;
}

/* src/gguf/quant_block.c:819-832: x = f16(scale) * (float)int8; a negative or
 * non-finite scale is a format error. */
int yvx_oracle_q8_0_decode_block(const unsigned char *encoded, float *out)
{
    float scale = yvx_oracle_f16_decode(load_u16le(encoded));
    unsigned int i;
    if (!isfinite(scale) || scale < 0.0f) return 0;
    for (i = 0; i < Q8_0_ELEMENTS; ++i) {
        int lane = encoded[2 + i] <= 127u ? (int)encoded[2 + i]
                                          : (int)encoded[2 + i] - 256;
        out[i] = scale * (float)lane;
    }
    return 1;
}

int yvx_oracle_q8_0_decode_rows(const unsigned char *encoded, float *out, size_t elements)
{
    size_t block, blocks = elements / Q8_0_ELEMENTS;
    if (elements % Q8_0_ELEMENTS) return 0;
    for (block = 0; block < blocks; ++block)
        if (!yvx_oracle_q8_0_decode_block(encoded + block * Q8_0_BYTES,
                                          out + block * Q8_0_ELEMENTS))
            return 0;
    return 1;
}

/* ---- encoded weight rows: decode and row dot ------------------------------------
 * yvex_quant_decode_block for the F32, F16, BF16 and Q8_0 encodings
 * (src/gguf/quant_block.c:805-832) and yvex_quant_cpu_dot over it
 * (src/gguf/quant_compute.c:116-181): every lane decoded to float, the products and
 * the running sum in double in lane order, the sum narrowed to float; a term or a
 * partial sum that is not finite is refused. qtype: the GGUF ids (F32 0, F16 1,
 * Q8_0 8, BF16 30). */
unsigned long long yvx_oracle_qtype_row_bytes(unsigned int qtype, unsigned long long width)
{
    switch (qtype) {
    case 0u: return width * 4ull;
    case 1u:
    case 30u: return width * 2ull;
    case 8u: return width % Q8_0_ELEMENTS ? 0ull : width / Q8_0_ELEMENTS * Q8_0_BYTES;
    default: return 0ull;
    }
}

int yvx_oracle_qtype_decode_row(unsigned int qtype, const unsigned char *encoded,
                                unsigned long long width, float *out)
{
    unsigned long long i;
    if (!encoded || !out || !yvx_oracle_qtype_row_bytes(qtype, width)) return 0;
    if (qtype == 8u) return yvx_oracle_q8_0_decode_rows(encoded, out, (size_t)width);
    for (i = 0; i < width; ++i) {
        if (qtype == 0u) memcpy(&out[i], encoded + 4ull * i, 4u);
        else if (qtype == 1u) out[i] = yvx_oracle_f16_decode(load_u16le(encoded + 2ull * i));
        else out[i] = yvx_oracle_bf16_decode(load_u16le(encoded + 2ull * i));
    }
    return 1;
}

int yvx_oracle_qtype_dot(unsigned int qtype, const unsigned char *encoded, unsigned long long width,
                         const float *vector, float *out)
{
    float *row = malloc((size_t)width * sizeof(float));
    double sum = 0.0;
    unsigned long long i;
    int ok = row && yvx_oracle_qtype_decode_row(qtype, encoded, width, row);
    for (i = 0; ok && i < width; ++i) {
        double term = (double)row[i] * vector[i];
        if (!isfinite(term) || !isfinite(sum + term)) ok = 0;
        sum += term;
    }
    free(row);
    if (!ok) return 0;
    *out = (float)sum;
    return isfinite(*out);
}

/* yvex_attention_dot_batch (src/graph/core.c:1107-1215) with the publication that follows
 * it where the caller rounds (src/graph/attention_execute.c:461-522): output[t][r] =
 * row (first_row + r) . input[t], optionally rounded to bf16. */
int yvx_oracle_qtype_matvec(unsigned int qtype, const unsigned char *encoded,
                            unsigned long long first_row, unsigned long long rows,
                            unsigned long long width, const float *input, unsigned long long tokens,
                            unsigned long long input_stride, float *output,
                            unsigned long long output_stride, int round_bf16)
{
    const unsigned long long row_bytes = yvx_oracle_qtype_row_bytes(qtype, width);
    float *row = malloc((size_t)width * sizeof(float));
    unsigned long long r, t, i;
    int ok = row && row_bytes;
    for (r = 0; ok && r < rows; ++r) {
        ok = yvx_oracle_qtype_decode_row(qtype, encoded + (first_row + r) * row_bytes, width, row);
        for (t = 0; ok && t < tokens; ++t) {
            const float *vector = input + t * input_stride;
            double sum = 0.0;
            float value;
            for (i = 0; i < width; ++i) {
                double term = (double)row[i] * vector[i];
                if (!isfinite(term) || !isfinite(sum + term)) ok = 0;
                sum += term;
            }
            value = (float)sum;
            if (!isfinite(value)) ok = 0;
            if (round_bf16) value = yvx_oracle_bf16_decode(yvx_oracle_bf16_encode(value));
            output[t * output_stride + r] = value;
        }
    }
    free(row);
    return ok;
}

/* ---- the CPU attention primitive --------------------------------------- */

/* src/backend/cpu.c:217-255: range reduction by ln2 into [-0.5, 0.5], an
 * 18-term Taylor sum, then scaling by repeated doubling or halving. */
double yvx_oracle_exp(double x)
{
    const double ln2 = 0.69314718055994530942;
    double term = 1.0, sum = 1.0;
    int halvings = 0;
    unsigned int i;
    if (x < -60.0) return 0.0;
    if (x > 60.0) x = 60.0;
    while (x > 0.5) {
        x -= ln2;
        ++halvings;
    }
    while (x < -0.5) {
        x += ln2;
        --halvings;
    }
    for (i = 1u; i <= 18u; ++i) {
        term *= x / (double)i;
        sum += term;
    }
    for (; halvings > 0; --halvings) sum *= 2.0;
    for (; halvings < 0; ++halvings) sum *= 0.5;
    return sum;
}

/* src/backend/cpu.c:307-399: scores in double rounded to float, running
 * maximum in double, probabilities rounded to float before and after the
 * division, value mix in double rounded to float. Returns 0 on success, -8
 * (state error) when the exponent sum is not positive, -7 on a bad position. */
int yvx_oracle_op_attention(const float *query, const float *keys,
                            const float *values, unsigned long long seq_len,
                            unsigned long long position, float scale, int causal,
                            unsigned long long head_dim, float *score_scratch,
                            float *probability_scratch, float *out)
{
    unsigned long long visible, i, d;
    double maximum = 0.0, sum = 0.0;
    if (!seq_len || !head_dim || !isfinite(scale) || scale <= 0.0f) return -10;
    if (position >= seq_len) return -7;
    visible = causal ? position + 1ull : seq_len;
    for (i = 0; i < seq_len; ++i) {
        double score = 0.0;
        if (causal && i > position) {
            score_scratch[i] = 0.0f;
            probability_scratch[i] = 0.0f;
            continue;
        }
        for (d = 0; d < head_dim; ++d)
            score += (double)query[d] * (double)keys[i * head_dim + d];
        score *= (double)scale;
        score_scratch[i] = (float)score;
        if (i == 0 || score > maximum) maximum = score;
    }
    for (i = 0; i < visible; ++i) {
        double e = yvx_oracle_exp((double)score_scratch[i] - maximum);
        probability_scratch[i] = (float)e;
        sum += e;
    }
    if (sum <= 0.0) return -8;
    for (i = 0; i < visible; ++i)
        probability_scratch[i] = (float)((double)probability_scratch[i] / sum);
    for (d = 0; d < head_dim; ++d) {
        double mixed = 0.0;
        for (i = 0; i < visible; ++i)
            mixed += (double)probability_scratch[i] * (double)values[i * head_dim + d];
        out[d] = (float)mixed;
    }
    return 0;
}

/* ---- grouped-query attention from the primitive ------------------------- */

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
} gqa_job;

/* One worker owns whole KV heads: it gathers the head's K and V rows into
 * packed [seq, head_dim] arrays (the shape the primitive admits) once, then
 * runs the primitive for every query row and every query head of the group.
 * Work is split by (kv head, query row) pairs so that one long session still
 * spreads over all workers. */
static void *gqa_worker(void *argument)
{
    gqa_job *job = (gqa_job *)argument;
    const unsigned long long hd = job->head_dimension, seq = job->key_value_tokens;
    const unsigned long long group = job->query_heads / job->key_value_heads;
    const unsigned long long items = job->key_value_heads * job->query_tokens * group;
    float *keys = malloc((size_t)(seq * hd) * sizeof(float));
    float *values = malloc((size_t)(seq * hd) * sizeof(float));
    float *scores = malloc((size_t)seq * sizeof(float));
    float *probabilities = malloc((size_t)seq * sizeof(float));
    unsigned long long gathered_head = ULLONG_MAX, item;
    job->status = 0;
    if (!keys || !values || !scores || !probabilities) {
        job->status = -2;
        goto done;
    }
    for (item = job->worker; item < items; item += job->workers) {
        /* item order: kv head slowest so a worker rarely re-gathers. */
        unsigned long long kv_head = item / (job->query_tokens * group);
        unsigned long long rest = item % (job->query_tokens * group);
        unsigned long long token = rest / group;
        unsigned long long query_head = kv_head * group + rest % group;
        unsigned long long row;
        int rc;
        if (kv_head != gathered_head) {
            for (row = 0; row < seq; ++row) {
                memcpy(keys + row * hd,
                       job->key + row * job->key_stride + kv_head * hd,
                       (size_t)hd * sizeof(float));
                memcpy(values + row * hd,
                       job->value + row * job->value_stride + kv_head * hd,
                       (size_t)hd * sizeof(float));
            }
            gathered_head = kv_head;
        }
        rc = yvx_oracle_op_attention(
            job->query + token * job->query_stride + query_head * hd, keys, values,
            seq, job->causal ? job->query_start + token : 0ull, job->scale,
            job->causal, hd, scores, probabilities,
            job->output + (token * job->query_heads + query_head) * hd);
        if (rc != 0) {
            job->status = rc;
            break;
        }
    }
done:
    free(keys);
    free(values);
    free(scores);
    free(probabilities);
    return NULL;
}

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
                             int causal, unsigned int threads)
{
    enum { MAX_THREADS = 256 };
    pthread_t handles[MAX_THREADS];
    gqa_job jobs[MAX_THREADS];
    unsigned int t, started = 0;
    int status = 0;
    if (!query || !key || !value || !output || !query_tokens || !key_value_tokens ||
        !query_heads || !key_value_heads || query_heads % key_value_heads ||
        !head_dimension || query_start + query_tokens > key_value_tokens)
        return -10;
    if (!threads) threads = 1;
    if (threads > MAX_THREADS) threads = MAX_THREADS;
    for (t = 0; t < threads; ++t) {
        gqa_job *job = &jobs[t];
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
        job->status = 0;
        if (threads == 1) {
            gqa_worker(job);
            started = 0;
        } else if (pthread_create(&handles[t], NULL, gqa_worker, job) == 0) {
            ++started;
        } else {
            gqa_worker(job);
        }
    }
    if (threads > 1)
        for (t = 0; t < started; ++t) pthread_join(handles[t], NULL);
    for (t = 0; t < threads; ++t)
        if (jobs[t].status) status = jobs[t].status;
    return status;
}

/* tests/unit/cuda/quant_qtype.c:2343-2391: the float scalar oracle the
 * reference's CUDA tests compare the operator with (two passes, expf). */
void yvx_oracle_gqa_f32_reference(const float *query, const float *key,
                                  const float *value, float *output,
                                  unsigned long long query_tokens,
                                  unsigned long long key_value_tokens,
                                  unsigned long long query_start,
                                  unsigned long long query_heads,
                                  unsigned long long key_value_heads,
                                  unsigned long long head_dimension, int causal)
{
    const float scale = 1.0f / sqrtf((float)head_dimension);
    const unsigned long long group = query_heads / key_value_heads;
    unsigned long long token, head, source, lane;
    for (token = 0; token < query_tokens; ++token)
        for (head = 0; head < query_heads; ++head) {
            const float *q = query + (token * query_heads + head) * head_dimension;
            float *o = output + (token * query_heads + head) * head_dimension;
            unsigned long long kv_head = head / group;
            unsigned long long visible = causal ? query_start + token + 1ull
                                                : key_value_tokens;
            float maximum = -INFINITY, denominator = 0.0f;
            for (source = 0; source < visible; ++source) {
                const float *k = key + (source * key_value_heads + kv_head) * head_dimension;
                float score = 0.0f;
                for (lane = 0; lane < head_dimension; ++lane) score += q[lane] * k[lane];
                if (score * scale > maximum) maximum = score * scale;
            }
            for (lane = 0; lane < head_dimension; ++lane) o[lane] = 0.0f;
            for (source = 0; source < visible; ++source) {
                const float *k = key + (source * key_value_heads + kv_head) * head_dimension;
                const float *v = value + (source * key_value_heads + kv_head) * head_dimension;
                float score = 0.0f, probability;
                for (lane = 0; lane < head_dimension; ++lane) score += q[lane] * k[lane];
                probability = expf(score * scale - maximum);
                denominator += probability;
                for (lane = 0; lane < head_dimension; ++lane) o[lane] += probability * v[lane];
            }
            for (lane = 0; lane < head_dimension; ++lane) o[lane] /= denominator;
        }
}

/* ---- block-table addressing --------------------------------------------- */

/* The reference keeps session KV rows contiguous in virtual address space
 * (src/runtime/state_residency.c:958-1028); a block table is this library's
 * extension. Row r of a session lives in pool row table[r / B] * B + r % B. */
unsigned long long yvx_oracle_block_row(const int *block_table,
                                        unsigned long long block_tokens,
                                        unsigned long long row)
{
    return (unsigned long long)block_table[row / block_tokens] * block_tokens +
           row % block_tokens;
}

void yvx_oracle_block_gather_u16(const unsigned short *pool, const int *block_table,
                                 unsigned long long block_tokens,
                                 unsigned long long rows,
                                 unsigned long long row_elements,
                                 unsigned short *out)
{
    unsigned long long row;
    for (row = 0; row < rows; ++row)
        memcpy(out + row * row_elements,
               pool + yvx_oracle_block_row(block_table, block_tokens, row) * row_elements,
               (size_t)row_elements * sizeof(*out));
}

/* ---- page geometry -------------------------------------------------------- */

static unsigned long long gcd_u64(unsigned long long a, unsigned long long b)
{
    while (b) {
        unsigned long long r = a % b;
        a = b;
        b = r;
    }
    return a;
}

static int mul_u64(unsigned long long a, unsigned long long b, unsigned long long *out)
{
    if (a && b > ULLONG_MAX / a) return 0;
    *out = a * b;
    return 1;
}

static int lcm_u64(unsigned long long a, unsigned long long b, unsigned long long *out)
{
    unsigned long long g;
    if (!a || !b) return 0;
    g = gcd_u64(a, b);
    return mul_u64(a / g, b, out);
}

/* src/deployment/plan.c:208-283: page_tokens is the multiple of
 * lcm(logical block, kernel tile, promotion granularity, alignment-in-tokens)
 * that minimises table + fragmentation + copy-on-write + promotion bytes,
 * bounded by the device page size; ties go to the smaller page. */
int yvx_oracle_page_tokens(const yvx_oracle_page_request *r,
                           unsigned long long *page_tokens,
                           unsigned long long *page_bytes)
{
    unsigned long long base, alignment_blocks, alignment_tokens, maximum, candidate;
    unsigned long long best_score = ULLONG_MAX, best = 0ull;
    if (!r || !r->logical_block_tokens || !r->kernel_tile_tokens ||
        !r->promotion_granularity_tokens || !r->alignment_bytes || !r->bytes_per_block)
        return 0;
    if (!lcm_u64(r->logical_block_tokens, r->kernel_tile_tokens, &base) ||
        !lcm_u64(base, r->promotion_granularity_tokens, &base))
        return 0;
    alignment_blocks = r->alignment_bytes / gcd_u64(r->bytes_per_block, r->alignment_bytes);
    if (!mul_u64(r->logical_block_tokens, alignment_blocks, &alignment_tokens) ||
        !lcm_u64(base, alignment_tokens, &base))
        return 0;
    maximum = r->device_page_bytes / r->bytes_per_block;
    if (!mul_u64(maximum, r->logical_block_tokens, &maximum)) return 0;
    maximum -= maximum % base;
    if (maximum < base) maximum = base;
    for (candidate = base; candidate <= maximum;) {
        unsigned long long pages, rounded, blocks, bytes, table, waste, score;
        pages = r->logical_tokens / candidate + (r->logical_tokens % candidate != 0ull);
        if (!mul_u64(pages, candidate, &rounded) || candidate % r->logical_block_tokens)
            return 0;
        blocks = candidate / r->logical_block_tokens;
        if (!blocks || !mul_u64(blocks, r->bytes_per_block, &bytes)) return 0;
        if (bytes % r->alignment_bytes == 0ull) {
            unsigned long long spare = rounded - r->logical_tokens;
            if (!mul_u64(pages, r->page_table_entry_bytes, &table)) return 0;
            blocks = spare / r->logical_block_tokens + (spare % r->logical_block_tokens != 0ull);
            if (!mul_u64(blocks, r->bytes_per_block, &waste)) return 0;
            score = table + waste + (r->copy_on_write ? bytes : 0ull) +
                    (r->candidate_extent ? waste : 0ull);
            if (score < best_score || (score == best_score && candidate < best)) {
                best_score = score;
                best = candidate;
            }
        }
        if (maximum - candidate < base) break;
        candidate += base;
    }
    if (!best) return 0;
    *page_tokens = best;
    return mul_u64(best / r->logical_block_tokens, r->bytes_per_block, page_bytes);
}

/* src/graph/state_pages.c:660-669: first and last page of an element range. */
int yvx_oracle_page_touch(unsigned long long element_start,
                          unsigned long long element_count,
                          unsigned long long page_elements,
                          unsigned long long *first_page,
                          unsigned long long *last_page)
{
    if (!element_count || !page_elements ||
        element_start > ULLONG_MAX - element_count)
        return 0;
    *first_page = element_start / page_elements;
    *last_page = (element_start + element_count - 1ull) / page_elements;
    return 1;
}

/* ---- shared-latent reduction -------------------------------------------- */

/* src/graph/core.c:361-390 (row visit), :466-508 (head reduce). All query
 * heads share one row per position and the row is both key and value. The
 * sink logit seeds the maximum and contributes exp(sink - max) to the
 * denominator only. Two passes in double; the value accumulator is float as
 * in the reference; the quotient is optionally rounded to bf16. Row r is
 * visible to query row t when r <= query_start + t. */
int yvx_oracle_latent_reduce(const float *query, const float *rows,
                             const float *sinks, float *out,
                             unsigned long long query_tokens,
                             unsigned long long row_count,
                             unsigned long long query_start,
                             unsigned long long query_heads,
                             unsigned long long head_dimension,
                             unsigned long long row_stride, int round_bf16)
{
    const double scale = 1.0 / sqrt((double)head_dimension);
    unsigned long long token, head, r, lane;
    if (!row_stride) row_stride = head_dimension;
    for (token = 0; token < query_tokens; ++token)
        for (head = 0; head < query_heads; ++head) {
            const float *q = query + (token * query_heads + head) * head_dimension;
            float *o = out + (token * query_heads + head) * head_dimension;
            unsigned long long visible = query_start + token + 1ull;
            double maximum = (double)sinks[head], denominator;
            if (visible > row_count) visible = row_count;
            if (!isfinite(maximum)) return 0;
            for (r = 0; r < visible; ++r) {
                const float *row = rows + r * row_stride;
                double score = 0.0;
                for (lane = 0; lane < head_dimension; ++lane)
                    score += (double)q[lane] * (double)row[lane];
                score *= scale;
                if (!isfinite(score)) return 0;
                if (score > maximum) maximum = score;
            }
            denominator = exp((double)sinks[head] - maximum);
            memset(o, 0, (size_t)head_dimension * sizeof(*o));
            for (r = 0; r < visible; ++r) {
                const float *row = rows + r * row_stride;
                double score = 0.0;
                for (lane = 0; lane < head_dimension; ++lane)
                    score += (double)q[lane] * (double)row[lane];
                score = exp(score * scale - maximum);
                denominator += score;
                for (lane = 0; lane < head_dimension; ++lane)
                    o[lane] += (float)(score * row[lane]);
            }
            if (!isfinite(denominator) || denominator <= 0.0) return 0;
            for (lane = 0; lane < head_dimension; ++lane) {
                o[lane] = (float)((double)o[lane] / denominator);
                if (round_bf16)
                    o[lane] = yvx_oracle_bf16_decode(yvx_oracle_bf16_encode(o[lane]));
            }
        }
    return 1;
}

/* ---- latent decode with a split rope key -------------------------------- */

/* The reference has no counterpart for this variant (its rope dimensions live
 * inside the shared latent row). The restatement keeps the reference's
 * ordering and precision rules for the reduce (src/graph/core.c:361-508: two
 * passes, double scores, libm exp) and its bf16 publication rule for the
 * projected query (src/graph/numeric.c bf16 rounding of linear outputs):
 *   q_lat[h,c] = bf16( sum_i q_nope[h,i] * W_uk[h,i,c] )        (double sum)
 *   s[h,t]     = scale * ( q_lat[h,:].latent[t,:] + q_rope[h,:].k_rope[t,:] )
 *   out[h,:]   = sum_t softmax_t(s[h,t]) * latent[t,:]            (float32)
 */
int yvx_oracle_mla_decode(const unsigned short *q_nope_bf16,
                          const unsigned short *q_rope_bf16,
                          const unsigned short *w_uk_bf16,
                          const unsigned short *latent_bf16,
                          const unsigned short *rope_key_bf16, float *out,
                          unsigned long long heads, unsigned long long nope_dim,
                          unsigned long long latent_dim,
                          unsigned long long rope_dim,
                          unsigned long long context, float scale,
                          float *absorbed_query_out)
{
    float *latent = malloc((size_t)(context * latent_dim) * sizeof(float));
    float *rope = malloc((size_t)(context * rope_dim) * sizeof(float));
    float *q_lat = malloc((size_t)latent_dim * sizeof(float));
    double *scores = malloc((size_t)context * sizeof(double));
    double *mixed = malloc((size_t)latent_dim * sizeof(double));
    unsigned long long h, t, c, i;
    int ok = 0;
    if (!latent || !rope || !q_lat || !scores || !mixed) goto done;
    yvx_oracle_bf16_decode_array(latent_bf16, latent, (size_t)(context * latent_dim));
    yvx_oracle_bf16_decode_array(rope_key_bf16, rope, (size_t)(context * rope_dim));
    for (h = 0; h < heads; ++h) {
        double maximum = -INFINITY, denominator = 0.0;
        for (c = 0; c < latent_dim; ++c) {
            double sum = 0.0;
            for (i = 0; i < nope_dim; ++i)
                sum += (double)yvx_oracle_bf16_decode(q_nope_bf16[h * nope_dim + i]) *
                       (double)yvx_oracle_bf16_decode(
                           w_uk_bf16[(h * nope_dim + i) * latent_dim + c]);
            q_lat[c] = yvx_oracle_bf16_decode(yvx_oracle_bf16_encode((float)sum));
            if (absorbed_query_out) absorbed_query_out[h * latent_dim + c] = q_lat[c];
        }
        for (t = 0; t < context; ++t) {
            double score = 0.0;
            for (c = 0; c < latent_dim; ++c)
                score += (double)q_lat[c] * (double)latent[t * latent_dim + c];
            for (i = 0; i < rope_dim; ++i)
                score += (double)yvx_oracle_bf16_decode(q_rope_bf16[h * rope_dim + i]) *
                         (double)rope[t * rope_dim + i];
            scores[t] = score * (double)scale;
            if (scores[t] > maximum) maximum = scores[t];
        }
        for (c = 0; c < latent_dim; ++c) mixed[c] = 0.0;
        for (t = 0; t < context; ++t) {
            double weight = exp(scores[t] - maximum);
            denominator += weight;
            for (c = 0; c < latent_dim; ++c)
                mixed[c] += weight * (double)latent[t * latent_dim + c];
        }
        if (!isfinite(denominator) || denominator <= 0.0) goto done;
        for (c = 0; c < latent_dim; ++c)
            out[h * latent_dim + c] = (float)(mixed[c] / denominator);
    }
    ok = 1;
done:
    free(latent);
    free(rope);
    free(q_lat);
    free(scores);
    free(mixed);
    return ok;
}

/* ---- shared-latent reduce over window + compressed rows ------------------- */

/* Row visibility as the reference's reduce stage defines it
 * (src/backend/cuda/attention_kernels.cu:69-100, CPU twin src/graph/core.c:392-464).
 * Pass 0 walks the local rows [history tail | current tokens]: without
 * candidate_block_visible only the last `sliding_window` rows up to the token are
 * candidates and a row counts when its position lies in [pos+1-W, pos]; with it
 * every local row counts. Pass 1 walks compressed rows (class 1: the token's
 * selected indices; class 2: all rows up to pos/ratio), a row counts when
 * position + ratio - 1 <= pos. Returns the row or NULL. */
static const float *latent_row(const yvx_oracle_latent_args *a, unsigned long long pass,
                               unsigned long long ordinal, unsigned long long candidate,
                               unsigned long long local_offset)
{
    const unsigned long long token_position = a->phase_start_position + ordinal;
    if (pass == 0ull) {
        unsigned long long position, first;
        candidate += local_offset;
        position = a->local_positions[candidate];
        if (!a->candidate_block_visible) {
            first = token_position + 1ull > a->sliding_window
                        ? token_position + 1ull - a->sliding_window : 0ull;
            if (position < first || position > token_position) return NULL;
        }
        return a->local + candidate * a->local_stride;
    } else {
        unsigned long long index = a->attention_class == 2u
                                       ? candidate
                                       : a->selected[ordinal * a->topk_capacity + candidate];
        unsigned long long position = a->compressed_positions[index];
        if (position > token_position || position > ~0ull - a->ratio + 1ull ||
            position + a->ratio - 1ull > token_position)
            return NULL;
        return a->compressed + index * a->compressed_stride;
    }
}

/* src/graph/core.c:466-508 (reduce_head): the sink logit seeds the maximum and
 * adds exp(sink - max) to the denominator; two passes in double; float value
 * accumulator; quotient rounded to bf16 (the reduce stage's publication). */
int yvx_oracle_latent_reduce_full(const yvx_oracle_latent_args *a, float *out)
{
    const double scale = 1.0 / sqrt((double)a->head_dim);
    unsigned long long ordinal, head, pass, candidate, lane;
    for (ordinal = 0; ordinal < a->token_count; ++ordinal) {
        const unsigned long long token_position = a->phase_start_position + ordinal;
        unsigned long long local_offset, local_count, compressed_count;
        if (a->candidate_block_visible) {
            local_offset = 0ull;
            local_count = a->initial_local_count + a->token_count;
        } else {
            unsigned long long before = a->initial_local_count + ordinal;
            unsigned long long history = token_position < a->sliding_window - 1ull
                                             ? token_position : a->sliding_window - 1ull;
            if (history > before) return 0;
            local_offset = before - history;
            local_count = history + 1ull;
        }
        compressed_count = a->attention_class == 0u ? 0ull
                           : a->attention_class == 1u
                               ? a->selected_count[ordinal]
                               : token_position / a->ratio + ((token_position + 1ull) % a->ratio == 0ull);
        for (head = 0; head < a->query_heads; ++head) {
            const float *q = a->query + (ordinal * a->query_heads + head) * a->head_dim;
            float *o = out + (ordinal * a->query_heads + head) * a->head_dim;
            double maximum = (double)a->sinks[head], denominator;
            int phase;
            if (!isfinite(maximum)) return 0;
            memset(o, 0, (size_t)a->head_dim * sizeof(*o));
            denominator = 0.0;
            for (phase = 0; phase < 2; ++phase) {
                if (phase == 1) denominator = exp((double)a->sinks[head] - maximum);
                for (pass = 0; pass < 2ull; ++pass) {
                    unsigned long long count = pass == 0ull ? local_count : compressed_count;
                    for (candidate = 0; candidate < count; ++candidate) {
                        const float *row = latent_row(a, pass, ordinal, candidate, local_offset);
                        double score = 0.0;
                        if (!row) continue;
                        for (lane = 0; lane < a->head_dim; ++lane)
                            score += (double)q[lane] * (double)row[lane];
                        score *= scale;
                        if (!isfinite(score)) return 0;
                        if (phase == 0) {
                            if (score > maximum) maximum = score;
                        } else {
                            score = exp(score - maximum);
                            denominator += score;
                            for (lane = 0; lane < a->head_dim; ++lane)
                                o[lane] += (float)(score * row[lane]);
                        }
                    }
                }
            }
            if (!isfinite(denominator) || denominator <= 0.0) return 0;
            for (lane = 0; lane < a->head_dim; ++lane)
                o[lane] = yvx_oracle_bf16_decode(
                    yvx_oracle_bf16_encode((float)((double)o[lane] / denominator)));
            /* :498-507: the published row is rotated back and published again */
            if (a->rope_dims) {
                if (!yvx_oracle_rope_apply(o, a->head_dim, a->rope_dims, token_position,
                                           a->rope_frequency, 1))
                    return 0;
                for (lane = 0; lane < a->head_dim; ++lane)
                    o[lane] = yvx_oracle_bf16_decode(yvx_oracle_bf16_encode(o[lane]));
            }
        }
    }
    return 1;
}

/* ---- position rotation, sparse index scores, ranked top-k ------------------ */

/* attention_yarn_frequency (src/graph/numeric.c:877-917): theta^(-2p/rope_dims),
 * and with an original context and a scaling factor the ramp between the
 * beta_fast and beta_slow correction dims blends in frequency / factor. */
int yvx_oracle_rope_frequencies(const yvx_oracle_position_policy *policy,
                                unsigned long long rope_dims, double *frequency)
{
    static const double pi = 3.14159265358979323846;
    unsigned long long pair;
    if (!policy || !frequency || rope_dims < 2ull || policy->theta <= 1ull) return 0;
    if (rope_dims & 1ull) rope_dims--;  /* the rotation drops an odd last lane first (:933) */
    for (pair = 0; pair < rope_dims / 2ull; ++pair) {
        double exponent = (double)(pair * 2ull) / (double)rope_dims;
        double f = 1.0 / pow((double)policy->theta, exponent);
        if (policy->original_context && policy->scaling_factor) {
            double denominator = 2.0 * log((double)policy->theta);
            double low = floor((double)rope_dims *
                               log((double)policy->original_context /
                                   ((double)policy->beta_fast * 2.0 * pi)) / denominator);
            double high = ceil((double)rope_dims *
                               log((double)policy->original_context /
                                   ((double)policy->beta_slow * 2.0 * pi)) / denominator);
            double ramp, smooth;
            if (low < 0.0) low = 0.0;
            if (high > (double)rope_dims - 1.0) high = (double)rope_dims - 1.0;
            if (low == high) high += 0.001;
            ramp = ((double)pair - low) / (high - low);
            if (ramp < 0.0) ramp = 0.0;
            if (ramp > 1.0) ramp = 1.0;
            smooth = 1.0 - ramp;
            f = f / (double)policy->scaling_factor * (1.0 - smooth) + f * smooth;
        }
        frequency[pair] = f;
    }
    return 1;
}

/* yvex_attention_rope_apply (src/graph/numeric.c:919-949): the last rope_dims
 * lanes as adjacent (x, y) pairs, angle = position * frequency, double
 * arithmetic, results narrowed to float. Known answer:
 * tests/reference/deepseek_attention.c:2690-2695. */
int yvx_oracle_rope_apply(float *values, unsigned long long count, unsigned long long rope_dims,
                          unsigned long long token_position, const double *frequency, int inverse)
{
    unsigned long long start, i;
    if (!values || !count || !frequency || rope_dims < 2ull || rope_dims > count) return 0;
    if (rope_dims & 1ull) rope_dims--;
    start = count - rope_dims;
    for (i = 0; i < rope_dims; i += 2ull) {
        double angle = (double)token_position * frequency[i / 2ull];
        double c = cos(angle);
        double sn = inverse ? -sin(angle) : sin(angle);
        double x = values[start + i], y = values[start + i + 1ull];
        if (!isfinite(x) || !isfinite(y) || !isfinite(c) || !isfinite(sn)) return 0;
        values[start + i] = (float)(x * c - y * sn);
        values[start + i + 1ull] = (float)(x * sn + y * c);
    }
    return 1;
}

typedef struct {
    float score;
    unsigned long long ordinal, index;
} topk_entry;

/* Ranking of yvex_attention_topk_select (src/graph/numeric.c:957-1000): higher
 * score first, +0 and -0 equal, equal scores by ascending ordinal. */
static int topk_before(const void *left, const void *right)
{
    const topk_entry *a = (const topk_entry *)left, *b = (const topk_entry *)right;
    if (a->score != b->score) return a->score > b->score ? -1 : 1;
    if (a->ordinal != b->ordinal) return a->ordinal < b->ordinal ? -1 : 1;
    return 0;
}

static int topk_by_ordinal(const void *left, const void *right)
{
    const topk_entry *a = (const topk_entry *)left, *b = (const topk_entry *)right;
    return a->ordinal < b->ordinal ? -1 : a->ordinal > b->ordinal;
}

/* yvex_attention_topk_select (src/graph/numeric.c:1086-1150): refuses non-finite
 * scores and duplicate ordinals; the first min(count, k) ranked candidates, as
 * indices into the input, in ranked order. */
int yvx_oracle_topk_select(const float *scores, const unsigned long long *ordinals,
                           unsigned long long count, unsigned long long k,
                           unsigned long long *selected, unsigned long long *selected_count)
{
    topk_entry *entries;
    unsigned long long i, keep;
    if (!scores || !ordinals || !selected || !selected_count) return 0;
    *selected_count = 0ull;
    if (!count || !k) return 1;
    entries = (topk_entry *)malloc((size_t)count * sizeof(*entries));
    if (!entries) return 0;
    for (i = 0; i < count; ++i) {
        if (!isfinite(scores[i])) {
            free(entries);
            return 0;
        }
        entries[i].score = scores[i];
        entries[i].ordinal = ordinals[i];
        entries[i].index = i;
    }
    qsort(entries, (size_t)count, sizeof(*entries), topk_by_ordinal);
    for (i = 1; i < count; ++i)
        if (entries[i - 1ull].ordinal == entries[i].ordinal) {
            free(entries);
            return 0;
        }
    qsort(entries, (size_t)count, sizeof(*entries), topk_before);
    keep = count < k ? count : k;
    for (i = 0; i < keep; ++i) selected[i] = entries[i].index;
    *selected_count = keep;
    free(entries);
    return 1;
}

/* yvex_attention_csa_select (src/graph/attention.c:369-497): a compressed row is
 * a candidate when position + ratio - 1 <= query position; its score is
 * sum_h weight[h] * max(0, q_h . key) in double, scaled by 1/sqrt(head_dim) and
 * 1/sqrt(heads), narrowed to float; candidates are ranked by (score, position).
 * selected[] holds row indices in ranked order. scores_out (may be NULL) gets the
 * float score of every row, NaN for rows that are not candidates. */
int yvx_oracle_csa_select(const yvx_oracle_indexer *ix, unsigned long long token,
                          unsigned long long query_position, unsigned long long *selected,
                          unsigned long long *selected_count, unsigned long long *valid_count,
                          float *scores_out)
{
    const float *query, *weights;
    float *scores;
    unsigned long long *ordinals, *rows, *ranked;
    unsigned long long candidate, head, lane, valid = 0ull, ranked_count = 0ull, i;
    int ok = 0;
    if (!ix || !selected || !selected_count || !valid_count) return 0;
    *selected_count = *valid_count = 0ull;
    if (!ix->rows) return 1;
    query = ix->query + token * ix->heads * ix->head_dim;
    weights = ix->weights + token * ix->heads;
    scores = (float *)malloc((size_t)ix->rows * sizeof(*scores));
    ordinals = (unsigned long long *)malloc((size_t)ix->rows * sizeof(*ordinals));
    rows = (unsigned long long *)malloc((size_t)ix->rows * sizeof(*rows));
    ranked = (unsigned long long *)malloc((size_t)ix->rows * sizeof(*ranked));
    if (!scores || !ordinals || !rows || !ranked) goto done;
    for (candidate = 0; candidate < ix->rows; ++candidate) {
        const float *key = ix->keys + candidate * ix->key_stride;
        const unsigned long long position = ix->positions[candidate];
        double score = 0.0;
        if (scores_out) scores_out[candidate] = NAN;
        if (position > query_position || position > ~0ull - ix->ratio + 1ull ||
            position + ix->ratio - 1ull > query_position)
            continue;
        for (head = 0; head < ix->heads; ++head) {
            const float *q = query + head * ix->head_dim;
            double dot = 0.0;
            for (lane = 0; lane < ix->head_dim; ++lane) {
                if (!isfinite(q[lane]) || !isfinite(key[lane])) goto done;
                dot += (double)q[lane] * (double)key[lane];
            }
            if (dot < 0.0) dot = 0.0;
            if (!isfinite(weights[head])) goto done;
            score += dot * (double)weights[head];
        }
        score *= 1.0 / sqrt((double)ix->head_dim);
        score *= 1.0 / sqrt((double)ix->heads);
        if (!isfinite(score)) goto done;
        scores[valid] = (float)score;
        if (scores_out) scores_out[candidate] = (float)score;
        ordinals[valid] = position;
        rows[valid] = candidate;
        valid++;
    }
    if (valid) {
        if (!yvx_oracle_topk_select(scores, ordinals, valid, ix->topk, ranked, &ranked_count))
            goto done;
        for (i = 0; i < ranked_count; ++i) selected[i] = rows[ranked[i]];
        *selected_count = ranked_count;
    }
    *valid_count = valid;
    ok = 1;
done:
    free(scores);
    free(ordinals);
    free(rows);
    free(ranked);
    return ok;
}

/* Rotate-half applied in place to packed [token][head][head_dim] vectors with
 * explicit tables [token][rotary_dim]; dims >= rotary_dim are left alone.
 * staged != 0: every product and the sum are rounded to bf16, as
 * yvex_rotary_half_f32 does (src/backend/cuda/transformer_kernels.cu:78-108);
 * staged == 0: plain single-precision multiply and add without contraction,
 * yvex_rotary_half_plain_f32 (:110-134). Known answers:
 * tests/unit/cuda/quant_qtype.c:1989-2062 and :3057-3104. */
int yvx_oracle_rotary_half(float *values, const float *cosines, const float *sines,
                           unsigned long long tokens, unsigned long long heads,
                           unsigned long long head_dim, unsigned long long rotary_dim, int staged)
{
    const unsigned long long half = rotary_dim / 2ull;
    unsigned long long token, head, lane;
    if (!values || !cosines || !sines || !tokens || !heads || !half || (rotary_dim & 1ull) ||
        rotary_dim > head_dim)
        return 0;
    for (token = 0; token < tokens; ++token)
        for (head = 0; head < heads; ++head) {
            float *v = values + (token * heads + head) * head_dim;
            for (lane = 0; lane < half; ++lane) {
                const float cosine = cosines[token * rotary_dim + lane];
                const float sine = sines[token * rotary_dim + lane];
                const float first = v[lane], second = v[half + lane];
                if (staged) {
                    volatile float a = yvx_oracle_bf16_decode(yvx_oracle_bf16_encode(first * cosine));
                    volatile float b = yvx_oracle_bf16_decode(yvx_oracle_bf16_encode(second * sine));
                    volatile float c = yvx_oracle_bf16_decode(yvx_oracle_bf16_encode(second * cosine));
                    volatile float d = yvx_oracle_bf16_decode(yvx_oracle_bf16_encode(first * sine));
                    v[lane] = yvx_oracle_bf16_decode(yvx_oracle_bf16_encode(a - b));
                    v[half + lane] = yvx_oracle_bf16_decode(yvx_oracle_bf16_encode(c + d));
                } else {
                    volatile float a = first * cosine, b = second * sine;
                    volatile float c = second * cosine, d = first * sine;
                    v[lane] = a - b;
                    v[half + lane] = c + d;
                }
            }
        }
    return 1;
}

/* Rotary tables of the decoder (src/runtime/decoder.c:1060-1095): for position
 * p and coordinate c, pair = c mod (width/2), angle = p * theta^(-2 pair / width)
 * in double; cosine and sine narrowed to float and rounded to bf16. */
int yvx_oracle_rope_tables(unsigned long long token_start, unsigned long long tokens,
                           unsigned long long width, double theta, float *cosines, float *sines)
{
    unsigned long long token, coordinate;
    if (!width || (width & 1ull) || !cosines || !sines) return 0;
    for (token = 0; token < tokens; ++token)
        for (coordinate = 0; coordinate < width; ++coordinate) {
            const unsigned long long pair = coordinate % (width / 2ull);
            const double frequency = pow(theta, -(double)(2ull * pair) / (double)width);
            const double angle = (double)(token_start + token) * frequency;
            cosines[token * width + coordinate] =
                yvx_oracle_bf16_decode(yvx_oracle_bf16_encode((float)cos(angle)));
            sines[token * width + coordinate] =
                yvx_oracle_bf16_decode(yvx_oracle_bf16_encode((float)sin(angle)));
        }
    return 1;
}

/* Full (non-causal) attention over interleaved [row][head][Q | K | V][width] rows in
 * single precision, three passes (scores and maximum, exponentials and sum, weighted
 * values), restating yvex_graph_full_attention_f32 (src/graph/numeric.c:1771-1826).
 * Known answer: tests/unit/minimax_h3.c:641-681. scratch holds `rows` floats. */
int yvx_oracle_full_attention_f32(const float *qkv, unsigned long long rows,
                                  unsigned long long heads, unsigned long long head_width,
                                  float *output, float *scratch)
{
    const unsigned long long hidden = heads * head_width, qkv_width = hidden * 3ull;
    const float scale = 1.0f / sqrtf((float)head_width);
    unsigned long long query, head, key, coordinate;
    if (!qkv || !rows || !heads || !head_width || !output || !scratch) return 0;
    memset(output, 0, (size_t)(rows * hidden) * sizeof(*output));
    for (query = 0; query < rows; ++query)
        for (head = 0; head < heads; ++head) {
            const float *q = qkv + query * qkv_width + head * head_width * 3ull;
            float maximum = -INFINITY, sum = 0.0f;
            for (key = 0; key < rows; ++key) {
                const float *k = qkv + key * qkv_width + head * head_width * 3ull + head_width;
                float score = 0.0f;
                for (coordinate = 0; coordinate < head_width; ++coordinate)
                    score += q[coordinate] * k[coordinate];
                scratch[key] = score * scale;
                if (scratch[key] > maximum) maximum = scratch[key];
            }
            for (key = 0; key < rows; ++key) {
                scratch[key] = expf(scratch[key] - maximum);
                sum += scratch[key];
            }
            if (!isfinite(sum) || sum <= 0.0f) return 0;
            for (key = 0; key < rows; ++key) {
                const float *value = qkv + key * qkv_width + head * head_width * 3ull + head_width * 2ull;
                const float probability = scratch[key] / sum;
                float *destination = output + query * hidden + head * head_width;
                for (coordinate = 0; coordinate < head_width; ++coordinate)
                    destination[coordinate] += probability * value[coordinate];
            }
        }
    return 1;
}

/* ---- rolling compressor ----------------------------------------------------- */

/* attention_rolling_emit (src/graph/attention.c:697-743): per lane a softmax over
 * the group's scores in double, libm exp, previous half (lane) before current half
 * (lane + head_dim) slot by slot, quotient narrowed to float. */
static int compressor_emit(const float *kv, const float *score, unsigned long long width,
                           unsigned long long head_dim, unsigned long long ratio, int overlap,
                           float *out)
{
    unsigned long long lane, slot;
    for (lane = 0; lane < head_dim; ++lane) {
        double maximum = -HUGE_VAL, denominator = 0.0, value = 0.0;
        for (slot = 0; slot < ratio; ++slot) {
            double s = score[slot * width + lane];
            if (overlap) {
                double s2 = score[(ratio + slot) * width + lane + head_dim];
                if (s2 > maximum) maximum = s2;
            }
            if (s > maximum) maximum = s;
        }
        for (slot = 0; slot < ratio; ++slot) {
            double w = exp((double)score[slot * width + lane] - maximum);
            denominator += w;
            value += w * (double)kv[slot * width + lane];
            if (overlap) {
                double w2 = exp((double)score[(ratio + slot) * width + lane + head_dim] - maximum);
                denominator += w2;
                value += w2 * (double)kv[(ratio + slot) * width + lane + head_dim];
            }
        }
        if (!isfinite(denominator) || denominator <= 0.0 || !isfinite(value)) return 0;
        out[lane] = (float)(value / denominator);
    }
    return 1;
}

static int compressor_round(float *values, unsigned long long count)
{
    unsigned long long i;
    for (i = 0; i < count; ++i) {
        if (!isfinite(values[i])) return 0;
        values[i] = yvx_oracle_bf16_decode(yvx_oracle_bf16_encode(values[i]));
    }
    return 1;
}

/* attention_rms_norm_apply (src/graph/numeric.c:630-654): mean of squares and the
 * scaling in double, lanes in order, narrowed to float. */
static int compressor_rms_norm(float *values, unsigned long long count, const float *weights,
                               double epsilon)
{
    unsigned long long i;
    double mean = 0.0, inverse;
    if (!isfinite(epsilon) || epsilon <= 0.0) return 0;
    for (i = 0; i < count; ++i) {
        double v = values[i];
        if (!isfinite(v) || !isfinite(weights[i])) return 0;
        mean += v * v;
    }
    mean /= (double)count;
    inverse = 1.0 / sqrt(mean + epsilon);
    if (!isfinite(inverse)) return 0;
    for (i = 0; i < count; ++i) {
        double v = (double)values[i] * inverse;
        v *= (double)weights[i];
        if (!isfinite(v)) return 0;
        values[i] = (float)v;
    }
    return 1;
}

/* yvex_attention_rolling_state_step_cpu (src/graph/attention.c:745-836) once per
 * token, followed on an emission by the chain of cpu_chunk_rolling_step
 * (src/graph/attention_execute.c:776-806): round, RMS norm, round, rotation at the
 * group's first position, round. The state's cursor and fills follow from the
 * number of consumed tokens (attention_rolling_state_validate, :569-626). */
int yvx_oracle_compressor_chunk(const yvx_oracle_compressor_args *a, unsigned long long *emitted)
{
    unsigned long long width, slots, token, lane, slot, count = 0;
    if (emitted) *emitted = 0;
    if (!a || !a->ratio || !a->head_dim || !a->ape || !a->state_kv || !a->state_score ||
        !a->after_kv || !a->after_score || (a->token_count && (!a->token_kv || !a->token_score)))
        return 0;
    width = a->head_dim * (a->overlap ? 2ull : 1ull);
    slots = a->ratio * (a->overlap ? 2ull : 1ull);
    if (a->token_count && a->token_stride < width) return 0;
    if (a->after_kv != a->state_kv)
        memcpy(a->after_kv, a->state_kv, (size_t)(slots * width) * sizeof(float));
    if (a->after_score != a->state_score)
        memcpy(a->after_score, a->state_score, (size_t)(slots * width) * sizeof(float));
    for (token = 0; token < a->token_count; ++token) {
        unsigned long long position = a->start_position + token;
        unsigned long long cursor = position % a->ratio;
        const float *kv = a->token_kv + token * a->token_stride;
        const float *score = a->token_score + token * a->token_stride;
        const float *ape = a->ape + cursor * width;
        slot = a->overlap ? a->ratio + cursor : cursor;
        for (lane = 0; lane < width; ++lane)
            if (!isfinite(kv[lane]) || !isfinite(score[lane]) || !isfinite(ape[lane])) return 0;
        for (lane = 0; lane < width; ++lane) {
            a->after_kv[slot * width + lane] = kv[lane];
            a->after_score[slot * width + lane] = score[lane] + ape[lane];
        }
        if (cursor + 1ull != a->ratio) continue;
        if (a->compressed) {
            float *out = a->compressed + count * a->compressed_stride;
            if (a->compressed_stride < a->head_dim ||
                !compressor_emit(a->after_kv, a->after_score, width, a->head_dim, a->ratio,
                                 a->overlap, out))
                return 0;
            if (a->norm_weights) {
                if (!compressor_round(out, a->head_dim) ||
                    !compressor_rms_norm(out, a->head_dim, a->norm_weights, a->epsilon) ||
                    !compressor_round(out, a->head_dim))
                    return 0;
                if (a->rope_dims &&
                    (!yvx_oracle_rope_apply(out, a->head_dim, a->rope_dims,
                                            position + 1ull - a->ratio, a->rope_frequency, 0) ||
                     !compressor_round(out, a->head_dim)))
                    return 0;
            }
        }
        if (a->positions) a->positions[count] = position + 1ull - a->ratio;
        ++count;
        if (a->overlap) {
            memcpy(a->after_kv, a->after_kv + a->ratio * width,
                   (size_t)(a->ratio * width) * sizeof(float));
            memcpy(a->after_score, a->after_score + a->ratio * width,
                   (size_t)(a->ratio * width) * sizeof(float));
        }
    }
    if (emitted) *emitted = count;
    return 1;
}

/* ---- activation fake quantisation --------------------------------------------- */

/* yvex_quant_fp8_e4m3fn_decode (src/gguf/quant_scalar.c:145-161) */
static float activation_fp8_decode(unsigned int code)
{
    unsigned int exponent = (code >> 3) & 0x0fu, mantissa = code & 0x07u;
    if (!(code & 0x7fu)) return 0.0f;
    return exponent == 0u ? ldexpf((float)mantissa, -9)
                          : ldexpf(1.0f + (float)mantissa / 8.0f, (int)exponent - 7);
}

static const float activation_fp4_values[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* attention_fp8_e4m3fn_encode / attention_fp4_e2m1_encode (src/graph/numeric.c:1178-1200,
 * 1277-1299): the code whose value is nearest to the clamped magnitude, an exact tie going to
 * the even code; the value of that code with the input's sign. */
static float activation_nearest(float value, unsigned int quantization)
{
    const unsigned int codes = quantization == 8u ? 0x7fu : 8u;
    const float limit = quantization == 8u ? 448.0f : 6.0f;
    float magnitude = fabsf(value), best_error = INFINITY, decoded;
    unsigned int code, best = 0u;
    if (magnitude > limit) magnitude = limit;
    for (code = 0u; code < codes; ++code) {
        float candidate = quantization == 8u ? activation_fp8_decode(code) : activation_fp4_values[code];
        float error = fabsf(candidate - magnitude);
        if (error < best_error || (error == best_error && !(code & 1u) && (best & 1u))) {
            best_error = error;
            best = code;
        }
    }
    decoded = quantization == 8u ? activation_fp8_decode(best) : activation_fp4_values[best];
    return signbit(value) ? -decoded : decoded;
}

/* attention_fake_quant_block (src/graph/numeric.c:1210-1258): the block's largest magnitude
 * (at least 1e-4 for FP8, 6 * 2^-126 for FP4) over the format's largest value, rounded up to a
 * power of two and stored as an 8-bit exponent (:990-1000, :1157-1171). */
static int activation_block(float *values, unsigned long long count, unsigned int quantization)
{
    const float limit = quantization == 8u ? 448.0f : 6.0f;
    float amax = quantization == 8u ? 1.0e-4f : 6.0f * ldexpf(1.0f, -126), scale, mantissa;
    unsigned long long i;
    int exponent;
    for (i = 0; i < count; ++i) {
        if (!isfinite(values[i])) return 0;
        if (fabsf(values[i]) > amax) amax = fabsf(values[i]);
    }
    mantissa = frexpf(amax / limit, &exponent);
    if (mantissa > 0.5f) exponent++;
    exponent += 126;                 /* scale = 2^(exponent - 127) */
    if (exponent < 0) exponent = 0;
    if (exponent > 254) exponent = 254;
    scale = exponent ? ldexpf(1.0f, exponent - 127) : ldexpf(1.0f, -127);
    for (i = 0; i < count; ++i) {
        float normalized = values[i] / scale;
        if (quantization == 8u && normalized > limit) normalized = limit;
        if (quantization == 8u && normalized < -limit) normalized = -limit;
        values[i] = yvx_oracle_bf16_decode(
            yvx_oracle_bf16_encode(activation_nearest(normalized, quantization) * scale));
    }
    return 1;
}

/* yvex_attention_activation_apply (src/graph/core.c:829-945) with the transform of
 * yvex_attention_hadamard_cpu (src/graph/numeric.c:1008-1078): butterflies of growing stride
 * in single precision over the zero-padded row, the first count lanes scaled by 1/sqrtf(count). */
int yvx_oracle_activation_quant(float *values, unsigned long long count, unsigned int quantization,
                                unsigned long long block_width, int hadamard)
{
    unsigned long long offset;
    if (!values || !count || !block_width || (quantization != 8u && quantization != 4u)) return 0;
    if (hadamard) {
        unsigned long long padded = 1ull, step, block, lane, i;
        float scale = 1.0f / sqrtf((float)count), *scratch;
        while (padded < count) padded *= 2ull;
        scratch = calloc((size_t)padded, sizeof(*scratch));
        if (!scratch) return 0;
        for (i = 0; i < count; ++i) {
            if (!isfinite(values[i])) {
                free(scratch);
                return 0;
            }
            scratch[i] = values[i];
        }
        for (step = 1ull; step < padded; step *= 2ull)
            for (block = 0; block < padded; block += step * 2ull)
                for (lane = 0; lane < step; ++lane) {
                    float left = scratch[block + lane], right = scratch[block + lane + step];
                    scratch[block + lane] = left + right;
                    scratch[block + lane + step] = left - right;
                }
        for (i = 0; i < count; ++i) values[i] = scratch[i] * scale;
        free(scratch);
    }
    if (count % block_width) return 0;
    for (offset = 0; offset < count; offset += block_width)
        if (!activation_block(values + offset, block_width, quantization)) return 0;
    return 1;
}

/* ---- publication chain of projected rows -------------------------------------- */

/* src/graph/attention_execute.c:527-612 (query heads: unit norm, round, rotation, round; new
 * local rows: weighted norm, round, rotation, round, activation of the lanes in front of the
 * rotated ones) and :970-1003 (index queries: rotation, round, activation of the whole head). */
int yvx_oracle_rows_publish(const yvx_oracle_publish_args *a)
{
    unsigned long long r, i;
    if (!a || !a->values || !a->width || a->row_stride < a->width || !a->rows_per_token) return 0;
    for (r = 0; r < a->rows; ++r) {
        float *row = a->values + r * a->row_stride;
        if (a->norm_mode) {
            double mean = 0.0, inverse;
            if (!isfinite(a->epsilon) || a->epsilon <= 0.0) return 0;
            if (a->norm_mode == 2) {
                if (!a->norm_weights || !compressor_rms_norm(row, a->width, a->norm_weights, a->epsilon)) return 0;
            } else {
                /* attention_rms_norm_apply without weights (src/graph/numeric.c:630-654) */
                for (i = 0; i < a->width; ++i) {
                    double v = row[i];
                    if (!isfinite(v)) return 0;
                    mean += v * v;
                }
                mean /= (double)a->width;
                inverse = 1.0 / sqrt(mean + a->epsilon);
                if (!isfinite(inverse)) return 0;
                for (i = 0; i < a->width; ++i) {
                    double v = (double)row[i] * inverse;
                    if (!isfinite(v)) return 0;
                    row[i] = (float)v;
                }
            }
            if (!compressor_round(row, a->width)) return 0;
        }
        if (a->rope_dims) {
            if (!yvx_oracle_rope_apply(row, a->width, a->rope_dims, a->start_position + r / a->rows_per_token,
                                       a->rope_frequency, 0) ||
                !compressor_round(row, a->width))
                return 0;
        }
        if (a->quantization && a->activation_count &&
            !yvx_oracle_activation_quant(row, a->activation_count, a->quantization, a->block_width, a->hadamard))
            return 0;
    }
    return 1;
}
