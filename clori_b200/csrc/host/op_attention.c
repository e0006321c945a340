/* The single-head attention primitive with the reference's admission order
 * (src/backend/core.c:1095-1141 pre-validation, :1547-1616 shared shape
 * validation, src/backend/cuda/ops.c:1717-1808 launch). */
#include "private.h"

#include <math.h>

static int op_f32(const yvex_device_tensor *tensor, unsigned long long elements)
{
    return tensor && elements <= ULLONG_MAX / sizeof(float) &&
           tensor->bytes == elements * sizeof(float);
}

int yvex_backend_op_attention(yvex_backend *backend, const yvex_device_tensor *query,
                              const yvex_device_tensor *keys, const yvex_device_tensor *values,
                              unsigned long long seq_len, unsigned long long position,
                              float scale, int causal, yvex_device_tensor *scores,
                              yvex_device_tensor *probabilities, yvex_device_tensor *out,
                              yvex_error *err)
{
    const char *where = "yvex_backend_op_attention";
    const yvex_device_tensor *tensors[6];
    unsigned long long head_dim, kv_elements;
    unsigned int i;
    int rc;
    if (!backend || !query || !keys || !values || !scores || !probabilities || !out)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where,
                        "backend, Q/K/V, scratches, and output are required");
    rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (!seq_len) return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "seq_len must be positive");
    if (position >= seq_len) return yvx_fail(err, YVEX_ERR_BOUNDS, where, "position-out-of-range");
    if (!isfinite(scale) || scale <= 0.0f)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "scale must be finite and positive");
    tensors[0] = query; tensors[1] = keys; tensors[2] = values;
    tensors[3] = scores; tensors[4] = probabilities; tensors[5] = out;
    for (i = 0; i < 6u; ++i)
        if (!yvx_tensor_owned(backend, tensors[i]))
            return yvx_fail(err, YVEX_ERR_INVALID_ARG, where,
                            "Q/K/V, scratches, and output tensors must belong to this backend");
    for (i = 0; i < 6u; ++i)
        if (tensors[i]->dtype != YVEX_DTYPE_F32)
            return yvx_fail(err, YVEX_ERR_UNSUPPORTED, where,
                            "attention primitive supports F32 Q/K/V, scratches, and output");
    if (query->rank != 1 || !query->dims[0])
        return yvx_fail(err, YVEX_ERR_FORMAT, where,
                        "attention query must be rank 1 with non-zero head_dim");
    head_dim = query->dims[0];
    if (!yvx_u64_mul(seq_len, head_dim, &kv_elements))
        return yvx_fail(err, YVEX_ERR_BOUNDS, where, "attention-element-count-overflow");
    if (keys->rank != 2 || keys->dims[0] != seq_len || keys->dims[1] != head_dim ||
        values->rank != 2 || values->dims[0] != seq_len || values->dims[1] != head_dim)
        return yvx_fail(err, YVEX_ERR_FORMAT, where,
                        "attention keys and values must have dims [seq_len, head_dim]");
    if (scores->rank != 1 || scores->dims[0] != seq_len || probabilities->rank != 1 ||
        probabilities->dims[0] != seq_len || out->rank != 1 || out->dims[0] != head_dim)
        return yvx_fail(err, YVEX_ERR_FORMAT, where,
                        out->rank != 1 || out->dims[0] != head_dim
                            ? "attention output must have dims [head_dim]"
                            : "attention score/probability scratches must have dims [seq_len]");
    if (!op_f32(query, head_dim) || !op_f32(keys, kv_elements) || !op_f32(values, kv_elements) ||
        !op_f32(scores, seq_len) || !op_f32(probabilities, seq_len) || !op_f32(out, head_dim))
        return yvx_fail(err, YVEX_ERR_BOUNDS, where,
                        "attention tensor bytes must match F32 shape accounting");
    rc = yvx_cuda_op_attention_f32((const float *)query->data, (const float *)keys->data,
                                   (const float *)values->data, seq_len, position, scale,
                                   causal != 0, head_dim, (float *)scores->data,
                                   (float *)probabilities->data, (float *)out->data,
                                   backend->stream);
    if (rc == 0) rc = yvx_cuda_stream_synchronize(backend->stream);
    if (rc != 0) return yvx_backend_device_fail(backend, rc, where, err);
    scores->is_written = 1;
    probabilities->is_written = 1;
    out->is_written = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}
