// A session's KV history between the two layouts it lives in: the bf16 block pool behind a
// block table that the batched attention kernels read, and the reference's per-layer state
// bank, one byte buffer with the components [values, positions, auxiliary] packed at 8-byte
// aligned offsets (src/runtime/state_residency.c:346-395), whose values are F32 rows
// [row][K heads | V heads] of width 2 * kv_heads * head_dim (src/graph/plan.c:27-56) and
// whose positions are one u64 per row (src/runtime/stateful_attention.c:183-243). The bank
// is what the reference checkpoints and restores (src/runtime/state_store.c:1-9), so a
// session kept in the pool can be handed back in the layout the checkpoint carries, and a
// restored bank can be put into the pool. bf16 -> F32 is exact and every value the
// reference stores in a bank is bf16-representable, so the round trip is bit-exact.
#include "common.cuh"

namespace yvx {

// grid: x = row, y = session. export_direction != 0: pool -> bank, else bank -> pool.
__global__ void __launch_bounds__(256)
kv_bank_transfer_kernel(const yvx_kv_bank_args a, const int export_direction)
{
    const unsigned int row = blockIdx.x, b = blockIdx.y;
    const unsigned int rows = a.kv_tokens ? (unsigned int)a.kv_tokens[b] : a.kv_tokens_uniform;
    if (row >= rows) return;
    if (rows > a.row_capacity || (unsigned long long)rows > (unsigned long long)a.block_table_stride * a.block_tokens) {
        if (threadIdx.x == 0) atomicCAS(a.status, 0, YVX_STATUS_CONTRACT);
        return;
    }
    const int entry = a.block_table[(unsigned long long)b * a.block_table_stride + row / a.block_tokens];
    if (entry < 0 || (unsigned int)entry >= a.pool_blocks) {
        if (threadIdx.x == 0) atomicCAS(a.status, 0, YVX_STATUS_CONTRACT);
        return;
    }
    const unsigned long long pool_row =
        (unsigned long long)entry * a.pool_block_stride + (unsigned long long)(row % a.block_tokens) * a.pool_token_stride;
    const unsigned int kv_width = a.kv_heads * a.head_dim;
    if (!YVX_CHECKED_INDEX(row < a.row_capacity && 2ull * kv_width <= a.value_width, a.status)) return;
    unsigned char *bank = reinterpret_cast<unsigned char *>(a.bank) + (unsigned long long)b * a.bank_session_bytes;
    float *values = reinterpret_cast<float *>(bank + a.values_offset) + (unsigned long long)row * a.value_width;
    unsigned long long *positions = reinterpret_cast<unsigned long long *>(bank + a.positions_offset);
    __nv_bfloat16 *key_pool = reinterpret_cast<__nv_bfloat16 *>(a.key_pool);
    __nv_bfloat16 *value_pool = reinterpret_cast<__nv_bfloat16 *>(a.value_pool);
    for (unsigned int i = threadIdx.x; i < 2u * kv_width; i += blockDim.x) {
        const bool is_key = i < kv_width;
        const unsigned int column = is_key ? i : i - kv_width;
        const unsigned int head = column / a.head_dim, lane = column % a.head_dim;
        __nv_bfloat16 *cell = (is_key ? key_pool : value_pool) + pool_row + (unsigned long long)head * a.pool_head_stride + lane;
        if (export_direction) {
            values[i] = __bfloat162float(*cell);
        } else {
            const float value = values[i];
            // a bank restored from elsewhere may hold values bf16 cannot: recorded, not hidden
            if (__bfloat162float(__float2bfloat16_rn(value)) != value && value == value)
                atomicCAS(a.status, 0, YVX_STATUS_CONTRACT);
            *cell = __float2bfloat16_rn(value);
        }
    }
    if (threadIdx.x == 0 && export_direction) positions[row] = a.position_base + row;
}

}  // namespace yvx

extern "C" {

int yvx_cuda_kv_bank_transfer(const yvx_kv_bank_args *args, int export_direction, void *stream)
{
    if (!args || !args->bank || !args->key_pool || !args->value_pool || !args->block_table || !args->status ||
        !args->sessions || !args->kv_heads || !args->head_dim || !args->block_tokens || !args->pool_blocks ||
        !args->row_capacity || args->value_width < 2ull * args->kv_heads * args->head_dim ||
        (args->values_offset & 7ull) || (args->positions_offset & 7ull))
        return YVEX_ERR_INVALID_ARG;
    if (args->sessions > 65535u) return YVEX_ERR_BOUNDS;
    const unsigned int rows = args->kv_tokens ? args->row_capacity : args->kv_tokens_uniform;
    if (!rows) return 0;
    const dim3 grid(rows, args->sessions, 1);
    yvx::kv_bank_transfer_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(*args, export_direction ? 1 : 0);
    return yvx_cuda_check(cudaGetLastError(), "kv_bank_transfer_kernel");
}

}  // extern "C"
