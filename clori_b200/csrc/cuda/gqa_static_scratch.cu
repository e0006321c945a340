// Grouped-query attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc on the path that runs
// attention: a serving loop that has handed the whole device to its own pool
// allocator and forbids further driver allocations, a real-time step where an
// allocation's implicit synchronisation is unacceptable, or a plug-in that is
// only given the tensors it reads and writes. The split-KV attention needs
// scratch for its per-split (o, m, l) partials; the regular entry point takes
// that scratch from the caller. This entry point takes it from a fixed array
// that lives in the library's device image instead.
#include <stdio.h>

#include <mutex>

#include "common.cuh"

namespace {

// 16 MiB per GPU that loads the library, held until the process exits.
constexpr unsigned long long kStaticScratchBytes = 16ull << 20;
static __device__ __align__(256) unsigned char yvx_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void *g_scratch_address[kMaxDevices];  // device address of the array, per device ordinal

// In host code the array's name is only a handle for the runtime, not a device
// address; the address is asked for once per device, with that device current.
int static_scratch_address(void **out)
{
    int device = -1;
    YVX_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return YVEX_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> guard(g_setup_mutex);
    if (!g_scratch_address[device]) {
        void *address = nullptr;
        YVX_CUDA_TRY(cudaGetSymbolAddress(&address, yvx_static_scratch));
        g_scratch_address[device] = address;
    }
    *out = g_scratch_address[device];
    return 0;
}

}  // namespace

extern "C" {

unsigned long long yvx_cuda_gqa_static_scratch_capacity(void) { return kStaticScratchBytes; }

int yvx_cuda_gqa_attention_static_scratch(const yvx_gqa_problem *problem, void *stream,
                                          unsigned int *launches)
{
    if (launches) *launches = 0;
    if (!problem) return YVEX_ERR_INVALID_ARG;
    const unsigned long long needed = yvx_cuda_gqa_partials_bytes(problem);
    if (needed > kStaticScratchBytes) {
        char text[160];
        snprintf(text, sizeof(text),
                 "needs %llu bytes of split scratch but the built-in array holds %llu",
                 needed, kStaticScratchBytes);
        // Recorded where yvx_cuda_last_error_text() reads it.
        (void)yvx_cuda_check(cudaErrorInvalidValue, text);
        return YVEX_ERR_BOUNDS;
    }
    void *scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != 0) return rc;
    yvx_gqa_problem bound = *problem;
    bound.partials = reinterpret_cast<float *>(scratch);
    return yvx_cuda_gqa_attention(&bound, stream, launches);
}

}  // extern "C"
