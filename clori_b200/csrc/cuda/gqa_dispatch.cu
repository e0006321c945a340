// Kernel selection and split planning for grouped-query attention.
#include "common.cuh"

namespace yvx {
int gqa_generic_main_launch(const yvx_gqa_problem &p, cudaStream_t stream);
int gqa_combine_launch(const yvx_gqa_problem &p, cudaStream_t stream);
bool gqa_decode_f32_admits(const yvx_gqa_problem &p);
void gqa_decode_f32_plan(yvx_gqa_problem *p, int sm_count);
int gqa_decode_f32_launch(const yvx_gqa_problem &p, cudaStream_t stream);
int gqa_decode_mma_launch(const yvx_gqa_problem &p, cudaStream_t stream);
int gqa_decode_q8_launch(const yvx_gqa_problem &p, cudaStream_t stream, const yvx_lse_exchange *exchange = nullptr);
int prefill_tcgen05_launch(const yvx_gqa_problem &p, cudaStream_t stream);
int lse_exchange_launch(const yvx_gqa_problem &p, const yvx_lse_exchange &x, cudaStream_t stream);

// ---- F32 problems on the tensor-core prefill kernel ---------------------------------------
// Staging layout: [flag, 256 bytes][Q bf16 packed rows][K bf16 packed rows][V bf16 packed rows].
constexpr unsigned long long kStageFlagBytes = 256ull;

static bool f32_tensor_path_shape(const yvx_gqa_problem &p)
{
    if (p.query_dtype != YVEX_DTYPE_F32 || p.kv_dtype != YVEX_DTYPE_F32 || p.output_dtype != YVEX_DTYPE_F32 ||
        p.head_dim != 128u || p.block_table || p.partial_output || p.kv_position_base || p.kv_tokens ||
        p.query_start || p.force_general || !p.kv_heads || p.query_heads % p.kv_heads ||
        (p.query_head_stride && p.query_head_stride != p.head_dim) || p.sessions != 1u)
        return false;
    return (unsigned long long)p.query_rows * (p.query_heads / p.kv_heads) > 64ull;
}

// One row per CTA-iteration: F32 [rows][stride] -> bf16 packed [rows][width]; a lane that bf16
// cannot hold exactly (or that is not finite) raises the flag.
__global__ void f32_stage_rows_kernel(const float *source, unsigned long long rows, unsigned long long width,
                                      unsigned long long stride, unsigned short *packed, int *flag)
{
    const unsigned long long quads = width / 4ull, total = rows * quads;
    const unsigned long long step = (unsigned long long)gridDim.x * blockDim.x;
    bool exact = true;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const unsigned long long row = i / quads, quad = i % quads;
        const float4 v = *reinterpret_cast<const float4 *>(source + row * stride + 4ull * quad);
        const uint32_t bits[4] = {__float_as_uint(v.x), __float_as_uint(v.y), __float_as_uint(v.z), __float_as_uint(v.w)};
#pragma unroll
        for (int j = 0; j < 4; ++j)
            exact = exact && !(bits[j] & 0xffffu) && (bits[j] & 0x7f800000u) != 0x7f800000u;
        uint2 out;
        out.x = (bits[0] >> 16) | (bits[1] & 0xffff0000u);
        out.y = (bits[2] >> 16) | (bits[3] & 0xffff0000u);
        *reinterpret_cast<uint2 *>(packed + row * width + 4ull * quad) = out;
    }
    if (!exact) atomicExch(flag, 1);
}

static int f32_stage_launch(const float *source, unsigned long long rows, unsigned long long width,
                            unsigned long long stride, unsigned short *packed, int *flag, cudaStream_t s)
{
    const unsigned long long total = rows * (width / 4ull);
    const unsigned int blocks = (unsigned int)((total + 255ull) / 256ull < 148ull * 16ull ? (total + 255ull) / 256ull
                                                                                      : 148ull * 16ull);
    f32_stage_rows_kernel<<<blocks ? blocks : 1u, 256, 0, s>>>(source, rows, width, stride, packed, flag);
    return yvx_cuda_check(cudaGetLastError(), "f32_stage_rows_kernel");
}
}

extern "C" {

// Splits exist to fill the machine. Two CTAs of the attention kernels are
// resident per SM, so one "wave" is 2 * sm_count work items. The chunk is the
// largest multiple of 64 tokens, at most 4096, for which the work items
// (sessions x kv heads x row tiles x splits, counted with the longest session)
// make at least one wave and fill their last wave to 90 %; failing that, the
// best-filled choice with at least one wave; failing that, 64. It depends on the
// problem's shape only, so repeated calls split identically and results repeat
// bit for bit.
void yvx_cuda_gqa_plan_splits(yvx_gqa_problem *p, int sm_count)
{
    if (!p) return;
    // Short F32 decode launches have their own kernel and their own chunk (16..112 tokens).
    if (!p->force_general && yvx::gqa_decode_f32_admits(*p)) {
        yvx::gqa_decode_f32_plan(p, sm_count);
        return;
    }
    const unsigned long long wave = 2ull * (unsigned long long)(sm_count > 0 ? sm_count : 148);
    const unsigned int group = p->kv_heads ? p->query_heads / p->kv_heads : 1u;
    const unsigned long long row_tiles = ((unsigned long long)p->query_rows * group + 15ull) / 16ull;
    const unsigned long long lanes =
        (unsigned long long)p->sessions * p->kv_heads * (row_tiles ? row_tiles : 1ull);
    unsigned int chosen = 64u, best = 0u;
    double best_fill = -1.0;
    for (unsigned int chunk = 4096u; chunk >= 64u; chunk -= 64u) {
        const unsigned long long splits = ((unsigned long long)p->kv_tokens_max + chunk - 1ull) / chunk;
        const unsigned long long items = lanes * splits;
        if (items < wave) continue;
        const unsigned long long waves = (items + wave - 1ull) / wave;
        const double fill = (double)items / (double)(waves * wave);
        if (fill >= 0.9) {
            best = chunk;
            break;
        }
        if (fill > best_fill) {
            best_fill = fill;
            best = chunk;
        }
    }
    if (best) chosen = best;
    p->chunk_tokens = chosen;
    p->max_splits = (p->kv_tokens_max + p->chunk_tokens - 1u) / p->chunk_tokens;
    if (!p->max_splits) p->max_splits = 1u;
}

unsigned long long yvx_cuda_gqa_partials_bytes(const yvx_gqa_problem *p)
{
    if (!p || p->max_splits <= 1u) return 0ull;
    return (unsigned long long)p->sessions * p->query_rows * p->query_heads * p->max_splits *
           (p->head_dim + 2ull) * sizeof(float);
}

unsigned long long yvx_cuda_gqa_f32_staging_bytes(const yvx_gqa_problem *p)
{
    if (!p || !yvx::f32_tensor_path_shape(*p)) return 0ull;
    const unsigned long long q = (unsigned long long)p->query_rows * p->query_heads * p->head_dim;
    const unsigned long long kv = (unsigned long long)p->kv_tokens_max * p->kv_heads * p->head_dim;
    return yvx::kStageFlagBytes + (q + 2ull * kv) * 2ull;
}

// The F32 problem on the tensor cores: stage (1 launch per tensor, 3 in all), the tensor-core
// kernel gated on "every lane was bf16", the general kernel (and its combine) gated on the opposite.
static int gqa_launch_f32_tensor(const yvx_gqa_problem *p, cudaStream_t s, unsigned int *count)
{
    const unsigned long long qw = (unsigned long long)p->query_heads * p->head_dim;
    const unsigned long long kw = (unsigned long long)p->kv_heads * p->head_dim;
    unsigned char *base = reinterpret_cast<unsigned char *>(p->f32_staging);
    int *flag = reinterpret_cast<int *>(base);
    unsigned short *q16 = reinterpret_cast<unsigned short *>(base + yvx::kStageFlagBytes);
    unsigned short *k16 = q16 + (unsigned long long)p->query_rows * qw;
    unsigned short *v16 = k16 + (unsigned long long)p->kv_tokens_max * kw;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (p->query_row_stride & 3ull) || (p->key_token_stride & 3ull) ||
        (p->value_token_stride & 3ull) || (reinterpret_cast<uintptr_t>(p->query) & 15u) ||
        (reinterpret_cast<uintptr_t>(p->key) & 15u) || (reinterpret_cast<uintptr_t>(p->value) & 15u) ||
        p->key_head_stride != p->head_dim || p->value_head_stride != p->head_dim)
        return 0;
    int rc = yvx_cuda_check(cudaMemsetAsync(flag, 0, sizeof(int), s), "f32 staging flag");
    if (rc == 0) rc = yvx::f32_stage_launch((const float *)p->query, p->query_rows, qw, p->query_row_stride, q16, flag, s);
    if (rc == 0) rc = yvx::f32_stage_launch((const float *)p->key, p->kv_tokens_max, kw, p->key_token_stride, k16, flag, s);
    if (rc == 0) rc = yvx::f32_stage_launch((const float *)p->value, p->kv_tokens_max, kw, p->value_token_stride, v16, flag, s);
    if (rc != 0) return rc;
    yvx_gqa_problem staged = *p;
    staged.query_dtype = staged.kv_dtype = YVEX_DTYPE_BF16;
    staged.query = q16;
    staged.key = k16;
    staged.value = v16;
    staged.query_row_stride = qw;
    staged.key_token_stride = staged.value_token_stride = kw;
    staged.gate = flag;
    staged.gate_value = 0;
    rc = yvx::prefill_tcgen05_launch(staged, s);
    if (rc == 0) return YVEX_ERR_UNSUPPORTED;  // the staged shape is the prefill kernel's by construction
    if (rc < 0) return rc;
    yvx_gqa_problem exact = *p;
    exact.gate = flag;
    exact.gate_value = 1;
    rc = yvx::gqa_generic_main_launch(exact, s);
    if (rc != 0) return rc;
    *count = 5u;
    if (exact.max_splits > 1u) {
        rc = yvx::gqa_combine_launch(exact, s);
        if (rc != 0) return rc;
        *count = 6u;
    }
    return 1;
}

static int gqa_launch(const yvx_gqa_problem *p, void *stream, cudaEvent_t *events,
                      unsigned int *launches, const yvx_lse_exchange *exchange = nullptr)
{
    unsigned int count = 0;
    if (launches) *launches = 0;
    if (!p || !p->query || !p->key || (!p->value && p->kv_dtype != YVEX_DTYPE_Q8_0) ||
        (!p->output && !p->partial_output) ||
        !p->status || !p->sessions || !p->query_rows || !p->query_heads || !p->kv_heads ||
        p->query_heads % p->kv_heads || !p->head_dim || !p->chunk_tokens || !p->max_splits ||
        (p->max_splits > 1u && !p->partials) || (p->block_table && !p->block_tokens))
        return YVEX_ERR_INVALID_ARG;
    // Launch limits, refused with a typed error before anything is enqueued: sessions ride in
    // grid.z and the decode kernels' (kv head, row tile) pairs in grid.y, both at most 65535.
    {
        const unsigned long long decode_vectors = (unsigned long long)p->query_rows * (p->query_heads / p->kv_heads);
        if (p->sessions > 65535u || p->max_splits > 0x7fffffffu ||
            (decode_vectors <= 64ull && (unsigned long long)p->kv_heads * ((decode_vectors + 15ull) / 16ull) > 65535ull)) {
            yvx_cuda_set_error_text("the attention grid exceeds the launch limits (65535 sessions, 65535 (kv head, row tile) pairs)");
            return YVEX_ERR_BOUNDS;
        }
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (events) cudaEventRecord(events[0], s);
    // Specialised kernels return 1 when they took the problem, 0 when its shape
    // is not theirs; the general kernel takes everything else.
    // 1 = attention launched (a combine follows when the KV was split), 2 = launched and
    // final, 0 = not this kernel's shape, negative = error.
    // Query heads that are not packed at head_dim are the general kernel's alone.
    const bool packed_heads = !p->query_head_stride || p->query_head_stride == p->head_dim;
    int rc = 0;
    if (exchange && exchange->one_launch && packed_heads && p->kv_dtype == YVEX_DTYPE_Q8_0) {
        // the whole step in one cooperative launch when the shape allows; else the two-launch path
        rc = yvx::gqa_decode_q8_launch(*p, s, exchange);
        if (rc == 3) {
            if (events) {
                cudaEventRecord(events[1], s);
                cudaEventRecord(events[2], s);
            }
            if (launches) *launches = 1u;
            return 0;
        }
        if (rc < 0) return rc;
    }
    rc = packed_heads ? yvx::gqa_decode_q8_launch(*p, s)
                      : (p->kv_dtype == YVEX_DTYPE_Q8_0 ? YVEX_ERR_UNSUPPORTED : 0);
    const unsigned int vectors = p->query_rows * (p->query_heads / p->kv_heads);
    if (rc == 0 && !p->force_general && packed_heads) rc = yvx::gqa_decode_f32_launch(*p, s);
    if (rc == 0 && !p->force_general && packed_heads)
        rc = vectors <= 64u ? yvx::gqa_decode_mma_launch(*p, s) : yvx::prefill_tcgen05_launch(*p, s);
    bool final_output = rc == 2;
    if (rc == 0 && p->f32_staging && yvx::f32_tensor_path_shape(*p)) {
        unsigned int staged_launches = 0u;
        rc = gqa_launch_f32_tensor(p, s, &staged_launches);
        if (rc == 1) {
            if (events) {
                cudaEventRecord(events[1], s);
                cudaEventRecord(events[2], s);
            }
            if (launches) *launches = staged_launches;
            return 0;
        }
        if (rc < 0) return rc;
    }
    if (rc == 0) rc = yvx::gqa_generic_main_launch(*p, s);
    else if (rc == 1 || rc == 2) rc = 0;
    if (rc != 0) return rc;
    count = 1u;
    if (events) cudaEventRecord(events[1], s);
    if (exchange) {
        // the fold of this rank's splits happens inside the exchange kernel
        if (final_output || !p->partial_output) return YVEX_ERR_UNSUPPORTED;
        rc = yvx::lse_exchange_launch(*p, *exchange, s);
        if (rc != 0) return rc;
        count = 2u;
    } else if (p->max_splits > 1u && !final_output) {
        rc = yvx::gqa_combine_launch(*p, s);
        if (rc != 0) return rc;
        count = 2u;
    }
    if (events) cudaEventRecord(events[2], s);
    if (launches) *launches = count;
    return 0;
}

int yvx_cuda_gqa_attention(const yvx_gqa_problem *p, void *stream, unsigned int *launches)
{
    return gqa_launch(p, stream, nullptr, launches);
}

int yvx_cuda_gqa_attention_exchange(const yvx_gqa_problem *p, const yvx_lse_exchange *exchange,
                                    void *stream, unsigned int *launches)
{
    if (!exchange) return YVEX_ERR_INVALID_ARG;
    return gqa_launch(p, stream, nullptr, launches, exchange);
}

unsigned long long yvx_cuda_lse_exchange_counter_offset(unsigned int ranks, unsigned int items,
                                                        unsigned int head_dim)
{
    // sized for the tagged-word form (8 bytes per lane); the float form uses the first half
    const unsigned long long bytes = 2ull * ranks * items * (head_dim + 2ull) * 8ull;
    return (bytes + 255ull) & ~255ull;
}

unsigned long long yvx_cuda_lse_exchange_bytes(unsigned int ranks, unsigned int items, unsigned int head_dim)
{
    // [items] arrival counters, then [items] split tickets of the one-launch step
    return yvx_cuda_lse_exchange_counter_offset(ranks, items, head_dim) + (unsigned long long)items * 8ull;
}

int yvx_cuda_gqa_attention_profiled(const yvx_gqa_problem *p, void *stream, void *events[3],
                                    unsigned int *launches)
{
    if (!events || !events[0] || !events[1] || !events[2]) return YVEX_ERR_INVALID_ARG;
    cudaEvent_t typed[3] = {(cudaEvent_t)events[0], (cudaEvent_t)events[1], (cudaEvent_t)events[2]};
    return gqa_launch(p, stream, typed, launches);
}

}  // extern "C"
