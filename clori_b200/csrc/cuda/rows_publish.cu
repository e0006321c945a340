// Publication chain of projected rows of the latent attention, one warp per row:
// RMS norm (unit or learned weights) -> bf16 -> rotation of the last lanes -> bf16 ->
// activation fake quantisation of the leading lanes, the row staying in registers.
//
// Replaces the per-row sequence of the reference's chunk executor
// (src/graph/attention_execute.c:527-612 for query heads and new local rows, :970-1003 for
// index queries; functions attention_rms_norm_apply src/graph/numeric.c:630-654,
// yvex_attention_rope_apply :919-949, yvex_attention_compute_round :614-628,
// yvex_attention_activation_apply src/graph/core.c:829-945), which on the device is a launch
// per step (src/backend/cuda/attention.c:1162-1236). A thread holds four adjacent lanes of
// each 128-lane segment, so rotated pairs and 16-byte accesses stay inside a thread and the
// activation's blocks are groups of neighbouring threads.
#include "activation.cuh"

namespace yvx {

constexpr int kPublishThreads = 128;
constexpr int kPublishSegments = 8;  // width <= 1024
constexpr int kPublishBatch = 4;     // row sets per batched launch

// round to nearest even; only finite values are ever published (a non-finite lane sets the status
// word and the row is not written), so the reference's NaN quieting does not come into it
__device__ __forceinline__ float publish_bf16(float v)
{
    return __bfloat162float(__float2bfloat16_rn(v));
}

// SEGMENTS = 128-lane segments a thread holds (the smallest of 1, 2, 4, 8 that covers the width).
template <int SEGMENTS>
__device__ __forceinline__ void publish_row(const yvx_rows_publish_args &a, unsigned long long r, unsigned int lane)
{
    float *row = a.values + r * a.row_stride;
    const unsigned int width = (unsigned int)a.width;
    const unsigned int segments = (width + 127u) / 128u;
    float v[SEGMENTS][4];
    bool finite = true;
#pragma unroll
    for (int s = 0; s < SEGMENTS; ++s) {
        const unsigned int base = (unsigned int)s * 128u + lane * 4u;
        v[s][0] = v[s][1] = v[s][2] = v[s][3] = 0.0f;
        if (s < (int)segments && base < width) {
            const float4 x = *reinterpret_cast<const float4 *>(row + base);
            v[s][0] = x.x, v[s][1] = x.y, v[s][2] = x.z, v[s][3] = x.w;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) finite = finite && isfinite(v[s][k]);
    }
    if (a.norm_mode) {
        double squares = 0.0;
#pragma unroll
        for (int s = 0; s < SEGMENTS; ++s)
#pragma unroll
            for (int k = 0; k < 4; ++k) squares = __dadd_rn(squares, __dmul_rn((double)v[s][k], (double)v[s][k]));
#pragma unroll
        for (int offset = 16; offset; offset >>= 1)
            squares = __dadd_rn(squares, __shfl_xor_sync(0xffffffffu, squares, offset));
        const double inverse = __ddiv_rn(1.0, sqrt(__dadd_rn(__ddiv_rn(squares, (double)width), a.epsilon)));
        finite = finite && isfinite(inverse);
#pragma unroll
        for (int s = 0; s < SEGMENTS; ++s) {
            const unsigned int base = (unsigned int)s * 128u + lane * 4u;
            if (s >= (int)segments || base >= width) continue;
            float weight[4] = {1.0f, 1.0f, 1.0f, 1.0f};
            if (a.norm_mode == 2) {
                const float4 w = __ldg(reinterpret_cast<const float4 *>(a.norm_weights + base));
                weight[0] = w.x, weight[1] = w.y, weight[2] = w.z, weight[3] = w.w;
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                double scaled = __dmul_rn((double)v[s][k], inverse);
                if (a.norm_mode == 2) scaled = __dmul_rn(scaled, (double)weight[k]);
                const float narrowed = __double2float_rn(scaled);
                finite = finite && isfinite(weight[k]) && isfinite(narrowed);
                v[s][k] = publish_bf16(narrowed);
            }
        }
    }
    if (a.rope_dims) {
        // Pair p (lanes rope_start + 2p, + 2p + 1) is rotated by the thread that holds it, but its sine and
        // cosine are computed by thread p % 32, so the 32 threads share the work; up to two pairs per thread
        // this way (rope_dims <= 128), beyond that each holder computes its own.
        const unsigned int rope_start = width - (unsigned int)a.rope_dims, pairs = (unsigned int)a.rope_dims / 2u;
        const unsigned long long position = a.start_position + r / a.rows_per_token;
        const bool shared = pairs <= 64u;
        double cs[2] = {1.0, 1.0}, sn[2] = {0.0, 0.0};
        if (shared) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const unsigned int p = lane + 32u * j;
                if (p < pairs) sincos(__dmul_rn((double)position, a.rope_frequency[p]), &sn[j], &cs[j]);
                finite = finite && isfinite(cs[j]) && isfinite(sn[j]);
            }
        }
#pragma unroll
        for (int s = 0; s < SEGMENTS; ++s) {
            if ((unsigned int)(s + 1) * 128u <= rope_start || s >= (int)segments) continue;   // uniform over the warp
            const unsigned int base = (unsigned int)s * 128u + lane * 4u;
#pragma unroll
            for (int k = 0; k < 4; k += 2) {
                const bool rotated = base + k >= rope_start && base < width;
                const unsigned int p = rotated ? (base + k - rope_start) >> 1 : 0u;
                double c, sine;
                if (shared) {
                    const int source = (int)(p & 31u);
                    const double c0 = __shfl_sync(0xffffffffu, cs[0], source), c1 = __shfl_sync(0xffffffffu, cs[1], source);
                    const double s0 = __shfl_sync(0xffffffffu, sn[0], source), s1 = __shfl_sync(0xffffffffu, sn[1], source);
                    c = p < 32u ? c0 : c1;
                    sine = p < 32u ? s0 : s1;
                } else if (rotated) {
                    sincos(__dmul_rn((double)position, a.rope_frequency[p]), &sine, &c);
                    finite = finite && isfinite(c) && isfinite(sine);
                }
                if (rotated) {
                    const double x = (double)v[s][k], y = (double)v[s][k + 1];
                    const float rx = __double2float_rn(__dsub_rn(__dmul_rn(x, c), __dmul_rn(y, sine)));
                    const float ry = __double2float_rn(__dadd_rn(__dmul_rn(x, sine), __dmul_rn(y, c)));
                    finite = finite && isfinite(rx) && isfinite(ry);
                    v[s][k] = rx, v[s][k + 1] = ry;
                }
            }
        }
        if (finite) {
#pragma unroll
            for (int s = 0; s < SEGMENTS; ++s)
#pragma unroll
                for (int k = 0; k < 4; ++k) v[s][k] = publish_bf16(v[s][k]);
        }
    }
    if (a.quantization) {
        const unsigned int count = (unsigned int)a.activation_count;
        const unsigned int group = (unsigned int)a.block_width / 4u;
        const bool fp8 = a.quantization == 8u;
        const float hadamard_scale = a.hadamard ? __fdiv_rn(1.0f, sqrtf((float)count)) : 1.0f;
#pragma unroll
        for (int s = 0; s < SEGMENTS; ++s) {
            if ((unsigned int)s * 128u >= count) continue;       // uniform over the warp
            const unsigned int base = (unsigned int)s * 128u + lane * 4u;
            const bool active = base < count;
            float q[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) q[k] = active ? v[s][k] : 0.0f;
            if (a.hadamard) activation_segment<true>(q, lane, group, fp8, hadamard_scale);
            else activation_segment<false>(q, lane, group, fp8, 1.0f);
            if (active) {
#pragma unroll
                for (int k = 0; k < 4; ++k) v[s][k] = q[k];
            }
        }
    }
    if (!finite) {
        atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
        return;
    }
#pragma unroll
    for (int s = 0; s < SEGMENTS; ++s) {
        const unsigned int base = (unsigned int)s * 128u + lane * 4u;
        if (s < (int)segments && base < width)
            *reinterpret_cast<float4 *>(row + base) = make_float4(v[s][0], v[s][1], v[s][2], v[s][3]);
    }
}

template <int SEGMENTS>
__global__ void __launch_bounds__(kPublishThreads, SEGMENTS <= 4 ? 6 : 3)
rows_publish_kernel(const yvx_rows_publish_args a)
{
    const unsigned long long r = (unsigned long long)blockIdx.x * (kPublishThreads / 32) + (threadIdx.x >> 5);
    if (r < a.rows) publish_row<SEGMENTS>(a, r, threadIdx.x & 31u);
}

// Several row sets in one launch (a decode step publishes its query heads, its new local
// row and its index queries): CTAs [first[i], first[i + 1]) belong to set i.
struct publish_batch {
    yvx_rows_publish_args set[kPublishBatch];
    unsigned int first[kPublishBatch + 1];
};

template <int SEGMENTS>
__global__ void __launch_bounds__(kPublishThreads, SEGMENTS <= 4 ? 6 : 3)
rows_publish_batch_kernel(const __grid_constant__ publish_batch batch)
{
    int i = 0;
#pragma unroll
    for (int k = 1; k < kPublishBatch; ++k)
        if (blockIdx.x >= batch.first[k]) i = k;
    const yvx_rows_publish_args &a = batch.set[i];
    const unsigned long long r =
        (unsigned long long)(blockIdx.x - batch.first[i]) * (kPublishThreads / 32) + (threadIdx.x >> 5);
    if (r < a.rows) publish_row<SEGMENTS>(a, r, threadIdx.x & 31u);
}

}  // namespace yvx

static int rows_publish_admit(const yvx_rows_publish_args *a);

extern "C" int yvx_cuda_rows_publish_batch(const yvx_rows_publish_args *sets, unsigned int count, void *stream)
{
    if (!sets || !count || count > (unsigned int)yvx::kPublishBatch) return YVEX_ERR_INVALID_ARG;
    yvx::publish_batch batch;
    unsigned long long widest = 0ull, ctas = 0ull;
    for (unsigned int i = 0; i < (unsigned int)yvx::kPublishBatch; ++i) {
        batch.first[i] = (unsigned int)ctas;
        if (i < count) {
            const int rc = rows_publish_admit(&sets[i]);
            if (rc != 0) return rc;
            batch.set[i] = sets[i];
            widest = sets[i].width > widest ? sets[i].width : widest;
            ctas += (sets[i].rows + 3ull) / 4ull;
        } else {
            batch.set[i] = sets[0];
            batch.set[i].rows = 0ull;
        }
    }
    batch.first[yvx::kPublishBatch] = (unsigned int)ctas;
    if (ctas > 0x7fffffffull) return YVEX_ERR_UNSUPPORTED;
    if (!ctas) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (widest <= 128ull) yvx::rows_publish_batch_kernel<1><<<(unsigned int)ctas, yvx::kPublishThreads, 0, s>>>(batch);
    else if (widest <= 256ull) yvx::rows_publish_batch_kernel<2><<<(unsigned int)ctas, yvx::kPublishThreads, 0, s>>>(batch);
    else if (widest <= 512ull) yvx::rows_publish_batch_kernel<4><<<(unsigned int)ctas, yvx::kPublishThreads, 0, s>>>(batch);
    else yvx::rows_publish_batch_kernel<8><<<(unsigned int)ctas, yvx::kPublishThreads, 0, s>>>(batch);
    return yvx_cuda_check(cudaGetLastError(), "rows_publish_batch_kernel");
}

static int rows_publish_admit(const yvx_rows_publish_args *a)
{
    if (!a || !a->values || !a->status || !a->width || !a->rows_per_token || a->row_stride < a->width)
        return YVEX_ERR_INVALID_ARG;
    if ((a->width & 3ull) || a->width > 128ull * yvx::kPublishSegments || (a->row_stride & 3ull) ||
        ((unsigned long long)a->values & 15ull) || a->rows > 0x1fffffffull)
        return YVEX_ERR_UNSUPPORTED;
    if (a->norm_mode < 0 || a->norm_mode > 2 || (a->norm_mode == 2 && !a->norm_weights) ||
        (a->norm_mode && (!(a->epsilon > 0.0) || a->epsilon > 1.0e300)))
        return YVEX_ERR_INVALID_ARG;
    if (a->norm_mode == 2 && ((unsigned long long)a->norm_weights & 15ull)) return YVEX_ERR_UNSUPPORTED;
    if (a->rope_dims && (!a->rope_frequency || (a->rope_dims & 1ull) || a->rope_dims > a->width))
        return YVEX_ERR_INVALID_ARG;
    if (a->quantization) {
        if (a->quantization != 8u && a->quantization != 4u) return YVEX_ERR_FORMAT;
        if (!a->activation_count || a->activation_count > a->width || !a->block_width) return YVEX_ERR_INVALID_ARG;
        if (a->activation_count % a->block_width) return YVEX_ERR_BOUNDS;
        if (a->block_width < 4ull || a->block_width > 128ull || (a->block_width & (a->block_width - 1ull)) ||
            (a->hadamard && (a->activation_count <= 64ull || a->activation_count > 128ull)))
            return YVEX_ERR_UNSUPPORTED;
    }
    return 0;
}

extern "C" int yvx_cuda_rows_publish(const yvx_rows_publish_args *a, void *stream)
{
    const int rc = rows_publish_admit(a);
    if (rc != 0) return rc;
    if (!a->rows) return 0;
    const unsigned int grid = (unsigned int)((a->rows + 3ull) / 4ull);
    cudaStream_t s = (cudaStream_t)stream;
    if (a->width <= 128ull) yvx::rows_publish_kernel<1><<<grid, yvx::kPublishThreads, 0, s>>>(*a);
    else if (a->width <= 256ull) yvx::rows_publish_kernel<2><<<grid, yvx::kPublishThreads, 0, s>>>(*a);
    else if (a->width <= 512ull) yvx::rows_publish_kernel<4><<<grid, yvx::kPublishThreads, 0, s>>>(*a);
    else yvx::rows_publish_kernel<8><<<grid, yvx::kPublishThreads, 0, s>>>(*a);
    return yvx_cuda_check(cudaGetLastError(), "rows_publish_kernel");
}
