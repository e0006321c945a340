// Single-head attention primitive: scores, probabilities and the mixed value
// for one query vector, with both scratch vectors published as the reference's
// primitive does (src/backend/cuda/kernels.cu:362-434 runs it in one CTA with
// a serial softmax on thread 0; here the scores are spread over the grid and
// the softmax is a block reduction).
#include "common.cuh"

namespace yvx {

// One warp per KV row: score[i] = scale * q . k_i, masked rows publish 0.
__global__ void __launch_bounds__(256)
op_scores_kernel(const float *query, const float *keys, unsigned long long seq_len,
                 unsigned long long visible, float scale, unsigned long long head_dim,
                 float *scores, float *probabilities)
{
    const unsigned long long row = (unsigned long long)blockIdx.x * 8ull + (threadIdx.x >> 5);
    const unsigned int lane = threadIdx.x & 31u;
    if (row >= seq_len) return;
    if (row >= visible) {
        if (lane == 0) {
            scores[row] = 0.0f;
            probabilities[row] = 0.0f;
        }
        return;
    }
    float partial = 0.0f;
    for (unsigned long long d = lane; d < head_dim; d += 32ull)
        partial = fmaf(query[d], keys[row * head_dim + d], partial);
    partial = warp_sum(partial);
    if (lane == 0) scores[row] = partial * scale;
}

// One CTA: maximum, exponent sum, normalised probabilities.
__global__ void __launch_bounds__(1024)
op_softmax_kernel(const float *scores, unsigned long long visible, float *probabilities)
{
    __shared__ float reduce[32];
    __shared__ float shared_max, shared_sum;
    const unsigned int lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    float maximum = -INFINITY, sum = 0.0f;
    for (unsigned long long i = threadIdx.x; i < visible; i += blockDim.x)
        maximum = fmaxf(maximum, scores[i]);
    maximum = warp_max(maximum);
    if (lane == 0) reduce[warp] = maximum;
    __syncthreads();
    if (warp == 0) {
        maximum = lane < (blockDim.x >> 5) ? reduce[lane] : -INFINITY;
        maximum = warp_max(maximum);
        if (lane == 0) shared_max = maximum;
    }
    __syncthreads();
    maximum = shared_max;
    for (unsigned long long i = threadIdx.x; i < visible; i += blockDim.x)
        sum += expf(scores[i] - maximum);
    sum = warp_sum(sum);
    __syncthreads();
    if (lane == 0) reduce[warp] = sum;
    __syncthreads();
    if (warp == 0) {
        sum = lane < (blockDim.x >> 5) ? reduce[lane] : 0.0f;
        sum = warp_sum(sum);
        if (lane == 0) shared_sum = sum;
    }
    __syncthreads();
    sum = shared_sum;
    for (unsigned long long i = threadIdx.x; i < visible; i += blockDim.x)
        probabilities[i] = expf(scores[i] - maximum) / sum;
}

// out[d] = sum_i p_i v[i][d]; one thread per dimension, coalesced over d.
__global__ void __launch_bounds__(128)
op_mix_kernel(const float *probabilities, const float *values, unsigned long long visible,
              unsigned long long head_dim, float *out)
{
    const unsigned long long d = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= head_dim) return;
    float mixed = 0.0f;
    for (unsigned long long i = 0; i < visible; ++i)
        mixed = fmaf(probabilities[i], values[i * head_dim + d], mixed);
    out[d] = mixed;
}

}  // namespace yvx

extern "C" int yvx_cuda_op_attention_f32(const float *query, const float *keys,
                                         const float *values, unsigned long long seq_len,
                                         unsigned long long position, float scale, int causal,
                                         unsigned long long head_dim, float *scores,
                                         float *probabilities, float *out, void *stream)
{
    if (!query || !keys || !values || !scores || !probabilities || !out || !seq_len || !head_dim)
        return YVEX_ERR_INVALID_ARG;
    if (position >= seq_len) return YVEX_ERR_BOUNDS;
    const unsigned long long visible = causal ? position + 1ull : seq_len;
    cudaStream_t s = (cudaStream_t)stream;
    yvx::op_scores_kernel<<<(unsigned int)((seq_len + 7ull) / 8ull), 256, 0, s>>>(
        query, keys, seq_len, visible, scale, head_dim, scores, probabilities);
    yvx::op_softmax_kernel<<<1, 1024, 0, s>>>(scores, visible, probabilities);
    yvx::op_mix_kernel<<<(unsigned int)((head_dim + 127ull) / 128ull), 128, 0, s>>>(
        probabilities, values, visible, head_dim, out);
    return yvx_cuda_check(cudaGetLastError(), "yvx_cuda_op_attention_f32");
}
