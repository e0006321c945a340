// Device-side helpers shared by the attention kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "yvex_b200/abi.h"
#include "yvex_b200/cuda_shim.h"

#define YVX_STATUS_OK 0
#define YVX_STATUS_NONFINITE 1
#define YVX_STATUS_CONTRACT 2
#define YVX_STATUS_CHECKED 4 /* an index check of a checked build (-DYVX_CHECKED) failed */
#define YVX_STATUS_TIMEOUT 3

// Maps a CUDA runtime error to the yvex_status the reference reports for
// launch and copy failures (YVEX_ERR_BACKEND) and remembers the text.
int yvx_cuda_check(cudaError_t error, const char *what);
void yvx_cuda_set_error_text(const char *text);

#define YVX_CUDA_TRY(call)                                 \
    do {                                                   \
        int yvx_rc_ = yvx_cuda_check((call), #call);       \
        if (yvx_rc_ != 0) return yvx_rc_;                  \
    } while (0)

namespace yvx {

// Programmatic dependent launch: a kernel launched with the programmatic stream
// serialization attribute may be scheduled once every CTA of the kernel before
// it has called pdl_launch_dependents() (or exited); it must call pdl_wait()
// before touching that kernel's results. Both are no-ops in a plain launch.
__device__ __forceinline__ void pdl_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int offset = 16; offset; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int offset = 16; offset; offset >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

__device__ __forceinline__ float load_as_float(const float *p) { return *p; }
__device__ __forceinline__ float load_as_float(const __nv_bfloat16 *p)
{
    return __bfloat162float(*p);
}

// Round-to-nearest-even bf16 publication with the reference's NaN quieting
// (src/gguf/quant_scalar.c:130-143; CUDA twin kernel_primitives.h:89).
__device__ __forceinline__ unsigned short bf16_bits_rne(float value)
{
    uint32_t bits = __float_as_uint(value);
    uint32_t high = bits >> 16, low = bits & 0xffffu;
    if ((bits & 0x7f800000u) == 0x7f800000u && (bits & 0x007fffffu))
        return (unsigned short)(high | 0x0040u);
    if (low > 0x8000u || (low == 0x8000u && (high & 1u))) high += 1u;
    return (unsigned short)high;
}

// Checked builds (-DYVX_CHECKED; the stand-in for a memory checker where none can be run):
// index and extent checks in front of the kernels' global stores. A failing check records
// status 4 and the store is skipped; nothing traps. Compiled out of the product build.
#ifdef YVX_CHECKED
#define YVX_CHECKED_INDEX(condition, status) ((condition) ? true : (atomicCAS((status), 0, YVX_STATUS_CHECKED), false))
#else
#define YVX_CHECKED_INDEX(condition, status) (true)
#endif

// A session's length as the kernels use it. Lengths live in device memory, where the
// host cannot check them; the host admitted `maximum` (it sized the split scratch, the
// block-table row and the tensor maps for it). A stored length beyond it (a negative
// value read as unsigned included) is a contract failure: it is recorded in the status
// word and the session is treated as empty, so that no row, table entry or partial
// outside the admitted range is ever addressed.
__device__ __forceinline__ unsigned int admitted_kv_tokens(const unsigned int *lengths, unsigned int b,
                                                           unsigned int uniform, unsigned int maximum,
                                                           int *status)
{
    const unsigned int n = lengths ? lengths[b] : uniform;
    if (n > maximum) {
        atomicCAS(status, 0, YVX_STATUS_CONTRACT);
        return 0u;
    }
    return n;
}

__device__ __forceinline__ void store_output(void *base, int dtype, unsigned long long index,
                                             float value)
{
    if (dtype == YVEX_DTYPE_BF16)
        reinterpret_cast<unsigned short *>(base)[index] = bf16_bits_rne(value);
    else
        reinterpret_cast<float *>(base)[index] = value;
}

}  // namespace yvx
