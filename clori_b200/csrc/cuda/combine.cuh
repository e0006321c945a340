// The fold of split-attention partials shared by the combine kernels.
#pragma once

#include "common.cuh"

namespace yvx {

// One CTA per (session, row, query head): folds the per-split (o, m, l)
// triples in a single pass over global memory. Eight warps share the splits
// (warp w takes splits w, w+8, ...) and keep a running (max, sum, weighted
// value) each; lanes own head dimensions. The loads of four splits are issued
// together, so a warp's whole share is usually one round trip. Per-warp
// results are merged in warp order: the result is a fixed function of the
// inputs and does not depend on scheduling.
constexpr int kCombineWarps = 8;
constexpr int kCombineBatch = 4;

__device__ __forceinline__ void combine_parts(const float *__restrict__ parts, unsigned int count,
                                              unsigned int stride, unsigned int hd, void *output,
                                              int output_dtype, unsigned long long out_index,
                                              float *partial_out, int *status)
{
    __shared__ float sm_max[kCombineWarps];
    __shared__ float sm_sum[kCombineWarps];
    __shared__ float sm_acc[kCombineWarps][256];
    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    float acc[8], run_max = -INFINITY, run_sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    for (unsigned int j0 = warp; j0 < count; j0 += kCombineWarps * kCombineBatch) {
        float mj[kCombineBatch], lj[kCombineBatch], oj[kCombineBatch][8];
#pragma unroll
        for (int u = 0; u < kCombineBatch; ++u) {
            const unsigned int j = j0 + u * kCombineWarps;
            const bool live = j < count;
            const float *part = parts + (unsigned long long)(live ? j : j0) * stride;
            mj[u] = live ? part[hd] : -INFINITY;
            lj[u] = part[hd + 1];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const unsigned int d = lane + 32u * i;
                oj[u][i] = d < hd ? part[d] : 0.0f;
            }
        }
#pragma unroll
        for (int u = 0; u < kCombineBatch; ++u) {
            if (mj[u] == -INFINITY) continue;  // empty split or past the end (warp-uniform)
            const float new_max = fmaxf(run_max, mj[u]);
            const float keep = expf(run_max - new_max);  // exp(-inf) = 0 on the first live split
            const float weight = lj[u] * expf(mj[u] - new_max);
            run_sum = fmaf(run_sum, keep, weight);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(acc[i], keep, oj[u][i] * weight);
            run_max = new_max;
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sm_acc[warp][lane + 32 * i] = acc[i];
    if (lane == 0) {
        sm_max[warp] = run_max;
        sm_sum[warp] = run_sum;
    }
    __syncthreads();
    float mm = sm_max[0];
#pragma unroll
    for (int w = 1; w < kCombineWarps; ++w) mm = fmaxf(mm, sm_max[w]);
    float scale_w[kCombineWarps], ll = 0.0f;
#pragma unroll
    for (int w = 0; w < kCombineWarps; ++w) {
        scale_w[w] = sm_max[w] == -INFINITY ? 0.0f : expf(sm_max[w] - mm);
        ll = fmaf(sm_sum[w], scale_w[w], ll);
    }
    for (unsigned int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < kCombineWarps; ++w) o = fmaf(sm_acc[w][d], scale_w[w], o);
        if (partial_out) {
            partial_out[d] = ll > 0.0f ? o / ll : 0.0f;
            if (d == 0) {
                partial_out[hd] = mm;
                partial_out[hd + 1] = ll;
            }
        } else {
            const float value = o / ll;
            if (!isfinite(value)) atomicCAS(status, 0, YVX_STATUS_NONFINITE);
            store_output(output, output_dtype, out_index + d, value);
        }
    }
}

}  // namespace yvx
