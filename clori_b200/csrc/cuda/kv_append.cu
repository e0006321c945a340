// KV append with rotary embedding, one launch per step.
//
// For the new rows of a step the reference runs a rotate-half kernel on Q and
// another on K (src/backend/cuda/transformer_kernels.cu:78-134, launched from
// src/runtime/decoder.c:1112-1131), then copies every new K row and V row into
// the session's state bank with one device copy each per token and uploads the
// positions (src/runtime/stateful_attention.c:183-243). Here one kernel rotates
// Q in place, rotates K on its way into the history, copies V, and writes the
// positions. Destinations: the reference's F32 state rows [row][K heads | V heads]
// and / or bf16 pools behind a block table (the batched decode layout).
//
// The arithmetic is the reference's, bit for bit: with staged_bf16 every product
// and the sum are rounded to bf16 (RNE, NaN quieted); without it the products
// and the sum are separate single-precision operations (no fused multiply-add).
#include "common.cuh"

namespace yvx {

constexpr int kAppendThreads = 256;

__device__ __forceinline__ float bf16_round(float x)
{
    return __bfloat162float(__float2bfloat16_rn(x));
}

template <bool STAGED>
__device__ __forceinline__ void rotate_pair(float first, float second, float cosine, float sine,
                                            float &out_first, float &out_second)
{
    if (STAGED) {
        const float a = bf16_round(__fmul_rn(first, cosine)), b = bf16_round(__fmul_rn(second, sine));
        const float c = bf16_round(__fmul_rn(second, cosine)), d = bf16_round(__fmul_rn(first, sine));
        out_first = bf16_round(__fsub_rn(a, b));
        out_second = bf16_round(__fadd_rn(c, d));
    } else {
        out_first = __fsub_rn(__fmul_rn(first, cosine), __fmul_rn(second, sine));
        out_second = __fadd_rn(__fmul_rn(second, cosine), __fmul_rn(first, sine));
    }
}

// Rows a session can hold: the caller's row_capacity, and never more than its block-table row
// addresses.
__device__ __forceinline__ unsigned long long append_row_capacity(const yvx_kv_append_args &a)
{
    unsigned long long capacity = a.row_capacity ? a.row_capacity : ~0ull;
    if (a.key_pool) {
        const unsigned long long table_rows = (unsigned long long)a.block_table_stride * a.block_tokens;
        capacity = table_rows < capacity ? table_rows : capacity;
    }
    return capacity;
}

// grid: x = token, y = session; one CTA moves the whole new row of a session:
// query heads in place, then key heads and value heads into the history.
template <bool STAGED>
__global__ void __launch_bounds__(kAppendThreads)
kv_append_rotary_kernel(const yvx_kv_append_args a)
{
    const unsigned int token = blockIdx.x, b = blockIdx.y;
    const unsigned int hd = a.head_dim, half = a.rotary_dim / 2u;
    const unsigned long long vector = (unsigned long long)b * a.tokens + token;
    const float *cosines = a.cosines + vector * a.rotary_dim;
    const float *sines = a.sines + vector * a.rotary_dim;
    // The row this CTA appends. Stored lengths live in device memory; a row at or beyond the
    // capacity the caller admitted (a negative length read as unsigned included) would land in
    // another session's rows or table entries: recorded as a contract failure, nothing written.
    const unsigned long long row =
        (unsigned long long)(a.kv_tokens ? (unsigned int)a.kv_tokens[b] : a.kv_tokens_uniform) + token;
    if (row >= append_row_capacity(a)) {
        if (threadIdx.x == 0) atomicCAS(a.status, 0, YVX_STATUS_CONTRACT);
        return;
    }
    if (a.query) {
        float *q = a.query + vector * a.query_heads * hd;
        for (unsigned int i = threadIdx.x; i < a.query_heads * half; i += kAppendThreads) {
            const unsigned int head = i / half, lane = i % half;
            float *v = q + (unsigned long long)head * hd;
            float first, second;
            rotate_pair<STAGED>(v[lane], v[half + lane], cosines[lane], sines[lane], first, second);
            v[lane] = first;
            v[half + lane] = second;
        }
    }
    // destination A: F32 state row, K heads then V heads
    float *state = nullptr;
    if (a.state_values)
        state = a.state_values + (unsigned long long)b * a.state_session_stride + row * a.state_row_stride;
    // destination B: bf16 pool rows behind the block table
    long long pool_row = -1;
    if (a.key_pool) {
        const int entry = a.block_table[(unsigned long long)b * a.block_table_stride + row / a.block_tokens];
        if (entry < 0 || (unsigned int)entry >= a.pool_blocks) {
            if (threadIdx.x == 0) atomicCAS(a.status, 0, YVX_STATUS_CONTRACT);
        } else {
            pool_row = (long long)((unsigned long long)entry * a.pool_block_stride +
                                   (row % a.block_tokens) * a.pool_token_stride);
        }
    }
    if (threadIdx.x == 0 && a.state_positions)
        a.state_positions[(unsigned long long)b * a.state_position_stride + row] =
            (a.token_position ? a.token_position[b] : row - token) + token;

    const unsigned int kv_width = a.kv_heads * hd;
    const float *key = a.key + vector * kv_width, *value_row = a.value + vector * kv_width;
    for (unsigned int i = threadIdx.x; i < 2u * kv_width; i += kAppendThreads) {
        const bool is_key = i < kv_width;
        const unsigned int column = is_key ? i : i - kv_width;
        const unsigned int head = column / hd, lane = column % hd;
        float value;
        if (is_key && lane < 2u * half) {
            // element `lane` of a rotated pair: which output it is depends on its half
            const float *src = key + (unsigned long long)head * hd;
            const unsigned int pair = lane < half ? lane : lane - half;
            float first, second;
            rotate_pair<STAGED>(src[pair], src[half + pair], cosines[pair], sines[pair], first, second);
            value = lane < half ? first : second;
        } else {
            value = is_key ? key[column] : value_row[column];
        }
        if (state) state[i] = value;
        if (pool_row >= 0) {
            __nv_bfloat16 *pool = reinterpret_cast<__nv_bfloat16 *>(is_key ? a.key_pool : a.value_pool);
            pool[(unsigned long long)pool_row + (unsigned long long)head * a.pool_head_stride + lane] =
                __float2bfloat16_rn(value);
        }
    }
}

// Same work with 16-byte accesses: every thread owns four neighbouring pairs.
// Needs head_dim % 4 == 0, rotary_dim % 8 == 0 and 16-byte aligned rows.
template <bool STAGED>
__global__ void __launch_bounds__(kAppendThreads)
kv_append_rotary_vec4_kernel(const yvx_kv_append_args a)
{
    const unsigned int token = blockIdx.x, b = blockIdx.y;
    const unsigned int hd = a.head_dim, half = a.rotary_dim / 2u, quads = half / 4u;
    const unsigned long long vector = (unsigned long long)b * a.tokens + token;
    const float4 *cosines = reinterpret_cast<const float4 *>(a.cosines + vector * a.rotary_dim);
    const float4 *sines = reinterpret_cast<const float4 *>(a.sines + vector * a.rotary_dim);
    auto rotate4 = [&](const float4 &x, const float4 &y, const float4 &c, const float4 &s, float4 &first,
                       float4 &second) {
        rotate_pair<STAGED>(x.x, y.x, c.x, s.x, first.x, second.x);
        rotate_pair<STAGED>(x.y, y.y, c.y, s.y, first.y, second.y);
        rotate_pair<STAGED>(x.z, y.z, c.z, s.z, first.z, second.z);
        rotate_pair<STAGED>(x.w, y.w, c.w, s.w, first.w, second.w);
    };
    // The row this CTA appends. Stored lengths live in device memory; a row at or beyond the
    // capacity the caller admitted (a negative length read as unsigned included) would land in
    // another session's rows or table entries: recorded as a contract failure, nothing written.
    const unsigned long long row =
        (unsigned long long)(a.kv_tokens ? (unsigned int)a.kv_tokens[b] : a.kv_tokens_uniform) + token;
    if (row >= append_row_capacity(a)) {
        if (threadIdx.x == 0) atomicCAS(a.status, 0, YVX_STATUS_CONTRACT);
        return;
    }
    if (a.query) {
        float *q = a.query + vector * a.query_heads * hd;
        for (unsigned int i = threadIdx.x; i < a.query_heads * quads; i += kAppendThreads) {
            const unsigned int head = i / quads, quad = i % quads;
            float4 *lo = reinterpret_cast<float4 *>(q + (unsigned long long)head * hd) + quad;
            float4 *hi = reinterpret_cast<float4 *>(q + (unsigned long long)head * hd + half) + quad;
            float4 first, second;
            rotate4(*lo, *hi, cosines[quad], sines[quad], first, second);
            *lo = first;
            *hi = second;
        }
    }
    float *state = nullptr;
    if (a.state_values)
        state = a.state_values + (unsigned long long)b * a.state_session_stride + row * a.state_row_stride;
    long long pool_row = -1;
    if (a.key_pool) {
        const int entry = a.block_table[(unsigned long long)b * a.block_table_stride + row / a.block_tokens];
        if (entry < 0 || (unsigned int)entry >= a.pool_blocks) {
            if (threadIdx.x == 0) atomicCAS(a.status, 0, YVX_STATUS_CONTRACT);
        } else {
            pool_row = (long long)((unsigned long long)entry * a.pool_block_stride +
                                   (row % a.block_tokens) * a.pool_token_stride);
        }
    }
    if (threadIdx.x == 0 && a.state_positions)
        a.state_positions[(unsigned long long)b * a.state_position_stride + row] =
            (a.token_position ? a.token_position[b] : row - token) + token;

    const unsigned int kv_width = a.kv_heads * hd;
    auto publish = [&](bool is_key, unsigned int head, unsigned int lane, const float4 &v) {
        if (state)
            *reinterpret_cast<float4 *>(state + (is_key ? 0u : kv_width) + head * hd + lane) = v;
        if (pool_row >= 0) {
            __nv_bfloat16 *pool = reinterpret_cast<__nv_bfloat16 *>(is_key ? a.key_pool : a.value_pool) +
                                  (unsigned long long)pool_row + (unsigned long long)head * a.pool_head_stride + lane;
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
            uint2 packed;
            packed.x = *reinterpret_cast<const unsigned int *>(&lo);
            packed.y = *reinterpret_cast<const unsigned int *>(&hi);
            *reinterpret_cast<uint2 *>(pool) = packed;
        }
    };
    const float *key = a.key + vector * kv_width, *value_row = a.value + vector * kv_width;
    // rotated part of K
    for (unsigned int i = threadIdx.x; i < a.kv_heads * quads; i += kAppendThreads) {
        const unsigned int head = i / quads, quad = i % quads;
        const float4 x = reinterpret_cast<const float4 *>(key + head * hd)[quad];
        const float4 y = reinterpret_cast<const float4 *>(key + head * hd + half)[quad];
        float4 first, second;
        rotate4(x, y, cosines[quad], sines[quad], first, second);
        publish(true, head, 4u * quad, first);
        publish(true, head, half + 4u * quad, second);
    }
    // unrotated suffix of K, then V
    const unsigned int suffix_quads = (hd - 2u * half) / 4u, head_quads = hd / 4u;
    for (unsigned int i = threadIdx.x; i < a.kv_heads * suffix_quads; i += kAppendThreads) {
        const unsigned int head = i / suffix_quads, lane = 2u * half + 4u * (i % suffix_quads);
        publish(true, head, lane, *reinterpret_cast<const float4 *>(key + head * hd + lane));
    }
    for (unsigned int i = threadIdx.x; i < a.kv_heads * head_quads; i += kAppendThreads) {
        const unsigned int head = i / head_quads, lane = 4u * (i % head_quads);
        publish(false, head, lane, *reinterpret_cast<const float4 *>(value_row + head * hd + lane));
    }
}

}  // namespace yvx

extern "C" int yvx_cuda_kv_append_rotary(const yvx_kv_append_args *args, void *stream)
{
    using namespace yvx;
    if (!args || !args->key || !args->value || !args->cosines || !args->sines || !args->status ||
        !args->sessions || !args->tokens || !args->kv_heads || !args->head_dim)
        return YVEX_ERR_INVALID_ARG;
    if (!args->rotary_dim || (args->rotary_dim & 1u) || args->rotary_dim > args->head_dim)
        return YVEX_ERR_INVALID_ARG;
    if (!args->state_values && !args->key_pool) return YVEX_ERR_INVALID_ARG;
    if (args->state_values && (!args->state_row_stride ||
                               args->state_row_stride < 2ull * args->kv_heads * args->head_dim))
        return YVEX_ERR_INVALID_ARG;
    if (args->key_pool && (!args->value_pool || !args->block_table || !args->block_tokens ||
                           !args->pool_blocks || !args->pool_token_stride || !args->pool_head_stride ||
                           !args->pool_block_stride))
        return YVEX_ERR_INVALID_ARG;
    if (args->query && !args->query_heads) return YVEX_ERR_INVALID_ARG;
    if (args->sessions > 65535u) return YVEX_ERR_UNSUPPORTED;
    const dim3 grid(args->tokens, args->sessions, 1);
    cudaStream_t s = (cudaStream_t)stream;
    auto aligned16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0u; };
    const bool vec4 =
        args->head_dim % 4u == 0u && args->rotary_dim % 8u == 0u && aligned16(args->query) &&
        aligned16(args->key) && aligned16(args->value) && aligned16(args->cosines) && aligned16(args->sines) &&
        aligned16(args->state_values) && args->state_row_stride % 4ull == 0ull &&
        args->state_session_stride % 4ull == 0ull && aligned16(args->key_pool) && aligned16(args->value_pool) &&
        args->pool_token_stride % 4ull == 0ull && args->pool_head_stride % 4ull == 0ull &&
        args->pool_block_stride % 4ull == 0ull;
    if (vec4 && args->staged_bf16)
        kv_append_rotary_vec4_kernel<true><<<grid, kAppendThreads, 0, s>>>(*args);
    else if (vec4)
        kv_append_rotary_vec4_kernel<false><<<grid, kAppendThreads, 0, s>>>(*args);
    else if (args->staged_bf16)
        kv_append_rotary_kernel<true><<<grid, kAppendThreads, 0, s>>>(*args);
    else
        kv_append_rotary_kernel<false><<<grid, kAppendThreads, 0, s>>>(*args);
    return yvx_cuda_check(cudaGetLastError(), "kv_append_rotary_kernel");
}
