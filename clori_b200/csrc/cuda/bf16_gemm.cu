// Projections at prefill-sized token counts on the 5th-generation tensor cores:
//   output[token][row] = sum_k input[token][k] * weight[row][k]
// for BF16-encoded weight rows and activation rows that bf16 holds exactly (what the
// encoded attention operator publishes between its stages), F32 accumulation in tensor
// memory, the bf16 publication of the result fused into the epilogue.
//
// Replaces, for token counts where one weight byte should serve many tokens, the
// reference's yvex_qtype_matvec / yvex_qtype_grouped_rows launched once per token tile
// (src/backend/cuda/kernels.cu:436-866, stages of src/backend/cuda/attention.c:1162-1236
// and :1424-1451). The CPU twin sums exact products in double (src/gguf/quant_compute.c:
// 116-181); here the products are exact too (two 8-bit mantissas) and the sum runs in the
// tensor core's F32 accumulator, so a published value differs from the twin's by at most
// one bf16 step, and only where the exact sum sits within an F32 rounding of a bf16 tie.
//
// One CTA per 128 tokens x 256 weight rows (x group), two CTAs per SM (half of tensor memory
// and 96 KB of shared memory each), so one CTA's epilogue runs under the other's main loop.
// Operand bytes per flop from L2, not HBM, bound this shape (both operands of a layer fit L2):
// measured, 128 x 128 tiles and 256 x 256 tiles (one CTA per SM, epilogue exposed) both stop
// at 860 TFLOP/s on the widest projection. A TMA warp streams [128][64] and [256][64] bf16
// tiles (128-byte swizzle, K-major) through a two-stage ring, one lane of the MMA warp issues
// four tcgen05.mma (128 x 256 x 16) per stage and frees the stage with a commit, four epilogue
// warps read the accumulator back with tcgen05.ld (a lane owns a token), round to bf16, turn
// 32 x 32 blocks through the (now idle) ring and store whole 128-byte runs of the F32 output
// rows, one row per warp instruction. Activations are
// staged F32 -> bf16 by a small kernel that also raises the status word when a lane is not
// exactly representable (the operator's contract for this path). Every wait is bounded.
#include "tcgen05.cuh"

namespace yvx {

constexpr int kGemmM = 128, kGemmN = 256, kGemmK = 64, kGemmStages = 2, kGemmThreads = 192;
constexpr int kGemmATile = kGemmM * kGemmK * 2, kGemmBTile = kGemmN * kGemmK * 2;   // 16 KB + 32 KB per stage
constexpr int kGemmStageBytes = kGemmATile + kGemmBTile;
constexpr int kGemmSmemBytes = kGemmStages * kGemmStageBytes + 1024 + 256;

struct GemmMaps {
    CUtensorMap activations, weights;
};

struct GemmBarriers {
    uint64_t full[kGemmStages], empty[kGemmStages], accumulated;
    uint32_t tmem_base;
};
static_assert(sizeof(GemmBarriers) <= 256, "barrier block outgrew its shared-memory slot");

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

// F32 [tokens][stride] -> bf16 [tokens][lanes] (lanes = groups * width); a lane that bf16
// cannot hold exactly, or that is not finite, raises the contract status.
__global__ void gemm_stage_rows_kernel(const float *source, unsigned long long tokens, unsigned long long lanes,
                                       unsigned long long stride, unsigned short *packed, int *status)
{
    const unsigned long long pairs = lanes / 2ull, total = tokens * pairs;
    const unsigned long long step = (unsigned long long)gridDim.x * blockDim.x;
    bool exact = true;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const unsigned long long row = i / pairs, pair = i % pairs;
        const float2 v = *reinterpret_cast<const float2 *>(source + row * stride + 2ull * pair);
        const uint32_t lo = __float_as_uint(v.x), hi = __float_as_uint(v.y);
        exact = exact && !((lo | hi) & 0xffffu) && (lo & 0x7f800000u) != 0x7f800000u && (hi & 0x7f800000u) != 0x7f800000u;
        *reinterpret_cast<uint32_t *>(packed + row * lanes + 2ull * pair) = (lo >> 16) | (hi & 0xffff0000u);
    }
    if (!exact) atomicCAS(status, 0, YVX_STATUS_CONTRACT);
}

// grid: x = token tile, y = weight-row tile, z = group.
__global__ void __launch_bounds__(kGemmThreads, 1)
bf16_gemm_tcgen05_kernel(const yvx_gemm_args a, const __grid_constant__ GemmMaps maps)
{
    extern __shared__ unsigned char gemm_smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023u) & ~uintptr_t(1023));
    GemmBarriers *bars = reinterpret_cast<GemmBarriers *>(smem + kGemmStages * kGemmStageBytes);
    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned int token0 = blockIdx.x * kGemmM, row0 = blockIdx.y * kGemmN, group = blockIdx.z;
    const unsigned int k_tiles = (unsigned int)((a.width + kGemmK - 1ull) / kGemmK);

    if (threadIdx.x == 0) {
        for (int i = 0; i < kGemmStages; ++i) {
            mbar_init(&bars->full[i], 1);
            mbar_init(&bars->empty[i], 1);
        }
        mbar_init(&bars->accumulated, 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(&bars->tmem_base, kGemmN);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            const int lane_x = (int)(group * a.width), weight_row = (int)(a.first_row + group * a.rows + row0);
            for (unsigned int kt = 0; kt < k_tiles; ++kt) {
                const unsigned int stage = kt % kGemmStages;
                if (kt >= (unsigned)kGemmStages && !mbar_wait(&bars->empty[stage], ((kt / kGemmStages) - 1u) & 1u)) {
                    atomicCAS(a.status, 0, YVX_STATUS_TIMEOUT);
                    break;
                }
                unsigned char *dst = smem + stage * kGemmStageBytes;
                mbar_expect_tx(&bars->full[stage], kGemmStageBytes);
                // lanes past the width and tokens past the last one are filled with zeros by the copy
                tma_load_2d(dst, &maps.activations, &bars->full[stage], lane_x + (int)(kt * kGemmK), (int)token0);
                tma_load_2d(dst + kGemmATile, &maps.weights, &bars->full[stage], (int)(kt * kGemmK), weight_row);
            }
        }
    } else if (warp == 1) {
        constexpr uint32_t idesc = idesc_bf16_f32(128, kGemmN, false);
        constexpr uint32_t desc_hi = smem_desc_sw128_hi(1024);
        const uint32_t elected = tc_elect_one() ? 1u : 0u;
        bool ok = true;
        for (unsigned int kt = 0; kt < k_tiles && ok; ++kt) {
            const unsigned int stage = kt % kGemmStages;
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->full[stage], (kt / kGemmStages) & 1u));
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t a_lo = smem_desc_sw128_lo(smem_u32(smem + stage * kGemmStageBytes), 16);
            const uint32_t b_lo = smem_desc_sw128_lo(smem_u32(smem + stage * kGemmStageBytes + kGemmATile), 16);
#pragma unroll
            for (int ks = 0; ks < kGemmK / 16; ++ks)
                tc_mma_ss_pred(elected, tmem, a_lo + 2u * ks, desc_hi, b_lo + 2u * ks, desc_hi, idesc, (kt || ks) ? 1u : 0u);
            tc_commit_pred(elected, &bars->empty[stage]);
        }
        if (ok) tc_commit_pred(elected, &bars->accumulated);
        else if (lane == 0) atomicCAS(a.status, 0, YVX_STATUS_TIMEOUT);
    } else {
        // ------------------------------ epilogue: a lane owns a token ------------------------------
        const unsigned int quadrant = warp & 3u;
        if (mbar_wait(&bars->accumulated, 0)) {
            tc_fence_after_sync();
            // every copy has landed and every MMA has read it: the ring is free for the turn
            float *turn = reinterpret_cast<float *>(smem) + quadrant * (32 * 33);
            bool finite = true;
            {
                const unsigned long long first_token = (unsigned long long)token0 + quadrant * 32u;
#pragma unroll 1
                for (int c = 0; c < kGemmN / 32; ++c) {
                    if ((unsigned long long)row0 + 32u * c >= a.rows) break;
                    uint32_t acc[32];
                    tmem_ld32(tmem + ((quadrant * 32u) << 16) + 32u * c, acc);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float value = __uint_as_float(acc[i]);
                        finite = finite && isfinite(value);
                        if (a.round_bf16) value = __uint_as_float((uint32_t)bf16_bits_rne(value) << 16);
                        turn[lane * 33 + i] = value;
                    }
                    __syncwarp();
                    const unsigned long long row = (unsigned long long)row0 + 32u * c + lane;   // this lane's weight row
                    for (unsigned int t = 0; t < 32u; ++t) {
                        const unsigned long long token_t = first_token + t;
                        if (token_t >= a.tokens) break;
                        if (row < a.rows && YVX_CHECKED_INDEX(group * a.rows + row < a.output_stride, a.status))
                            a.output[token_t * a.output_stride + group * a.rows + row] = turn[t * 33 + lane];
                    }
                    __syncwarp();
                }
            }
            // sums of tokens past the last one are sums of zeros: finite
            if (!finite) atomicCAS(a.status, 0, YVX_STATUS_NONFINITE);
        } else {
            atomicCAS(a.status, 0, YVX_STATUS_TIMEOUT);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kGemmN);
}

typedef CUresult (*GemmEncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                      const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 2-D bf16 map {lanes, rows}, box 64 x box_rows, 128-byte swizzle, zeros outside.
static bool gemm_encode(CUtensorMap *map, const void *base, unsigned long long lanes, unsigned long long rows,
                        unsigned long long row_lanes, unsigned int box_rows)
{
    static GemmEncodeTiledFn encode = nullptr;
    static bool resolved = false;
    if (!resolved) {
        void *symbol = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &query) == cudaSuccess &&
            query == cudaDriverEntryPointSuccess)
            encode = reinterpret_cast<GemmEncodeTiledFn>(symbol);
        resolved = true;
    }
    if (!encode || (reinterpret_cast<uintptr_t>(base) & 15u) || (row_lanes * 2ull) & 15ull) return false;
    cuuint64_t dims[2] = {lanes, rows};
    cuuint64_t strides[1] = {row_lanes * 2ull};
    cuuint32_t box[2] = {(cuuint32_t)kGemmK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace yvx

extern "C" {

unsigned long long yvx_cuda_bf16_gemm_staging_bytes(unsigned long long tokens, unsigned long long groups,
                                                    unsigned long long width)
{
    return tokens * (groups ? groups : 1ull) * width * 2ull;
}

int yvx_cuda_bf16_gemm(const yvx_gemm_args *args, void *stream)
{
    using namespace yvx;
    if (!args || !args->weights || !args->input || !args->output || !args->status || !args->staging || !args->rows ||
        !args->width || !args->tokens)
        return YVEX_ERR_INVALID_ARG;
    const unsigned long long groups = args->groups ? args->groups : 1ull;
    const unsigned long long lanes = groups * args->width;
    if (args->width % 8ull || args->input_stride < lanes || args->input_stride % 2ull ||
        (reinterpret_cast<uintptr_t>(args->input) & 7u) || args->output_stride < groups * args->rows)
        return YVEX_ERR_BOUNDS;
    const unsigned long long token_tiles = (args->tokens + kGemmM - 1ull) / kGemmM;
    const unsigned long long row_tiles = (args->rows + kGemmN - 1ull) / kGemmN;
    if (token_tiles > 0x7fffffffull || row_tiles > 65535ull || groups > 65535ull ||
        args->first_row + groups * args->rows > 0x7fffffffull || lanes > 0x7fffffffull) {
        yvx_cuda_set_error_text("the projection grid exceeds the launch limits");
        return YVEX_ERR_BOUNDS;
    }
    cudaStream_t s = (cudaStream_t)stream;
    GemmMaps maps;
    // the weight map ends at the last row of the last group, so a row tile that hangs over reads zeros there
    if (!gemm_encode(&maps.activations, args->staging, lanes, args->tokens, lanes, kGemmM) ||
        !gemm_encode(&maps.weights, args->weights, args->width, args->first_row + groups * args->rows, args->width, kGemmN))
        return YVEX_ERR_UNSUPPORTED;
    static int configured_device = -1;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return YVEX_ERR_BACKEND;
    if (configured_device != device) {
        const cudaError_t error = cudaFuncSetAttribute(bf16_gemm_tcgen05_kernel,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
        if (error != cudaSuccess) return yvx_cuda_check(error, "bf16_gemm_tcgen05_kernel attribute");
        configured_device = device;
    }
    const unsigned long long pairs = args->tokens * (lanes / 2ull);
    const unsigned int blocks = (unsigned int)((pairs + 255ull) / 256ull < 148ull * 16ull ? (pairs + 255ull) / 256ull
                                                                                     : 148ull * 16ull);
    gemm_stage_rows_kernel<<<blocks ? blocks : 1u, 256, 0, s>>>(args->input, args->tokens, lanes, args->input_stride,
                                                                reinterpret_cast<unsigned short *>(args->staging),
                                                                args->status);
    int rc = yvx_cuda_check(cudaGetLastError(), "gemm_stage_rows_kernel");
    if (rc != 0) return rc;
    const dim3 grid((unsigned int)token_tiles, (unsigned int)row_tiles, (unsigned int)groups);
    bf16_gemm_tcgen05_kernel<<<grid, kGemmThreads, kGemmSmemBytes, s>>>(*args, maps);
    return yvx_cuda_check(cudaGetLastError(), "bf16_gemm_tcgen05_kernel");
}

}  // extern "C"
