// Device runtime plumbing behind the C-ABI: allocation, copies, streams and
// events. Host C11 code reaches CUDA only through these functions.
#include "common.cuh"

#include <stdio.h>
#include <string.h>

static thread_local char yvx_error_text[256] = "";

int yvx_cuda_check(cudaError_t error, const char *what)
{
    if (error == cudaSuccess) return 0;
    snprintf(yvx_error_text, sizeof(yvx_error_text), "%s: %s", what, cudaGetErrorString(error));
    return error == cudaErrorMemoryAllocation ? YVEX_ERR_NOMEM : YVEX_ERR_BACKEND;
}

// Records a refusal that no CUDA call made (a shape beyond a launch limit, a full scratch).
void yvx_cuda_set_error_text(const char *text)
{
    snprintf(yvx_error_text, sizeof(yvx_error_text), "%s", text ? text : "");
}

extern "C" {

const char *yvx_cuda_last_error_text(void) { return yvx_error_text; }

int yvx_cuda_device_synchronize(void)
{
    YVX_CUDA_TRY(cudaDeviceSynchronize());
    return 0;
}

int yvx_cuda_device_count(int *count)
{
    if (!count) return YVEX_ERR_INVALID_ARG;
    *count = 0;
    cudaError_t error = cudaGetDeviceCount(count);
    if (error != cudaSuccess) {
        *count = 0;
        (void)cudaGetLastError();
        return yvx_cuda_check(error, "cudaGetDeviceCount");
    }
    return 0;
}

int yvx_cuda_device_select(int device)
{
    YVX_CUDA_TRY(cudaSetDevice(device));
    return 0;
}

int yvx_cuda_device_properties(int device, int *sm_count, int *cc_major, int *cc_minor,
                               unsigned long long *global_bytes, char *name, size_t name_cap)
{
    cudaDeviceProp properties;
    YVX_CUDA_TRY(cudaGetDeviceProperties(&properties, device));
    if (sm_count) *sm_count = properties.multiProcessorCount;
    if (cc_major) *cc_major = properties.major;
    if (cc_minor) *cc_minor = properties.minor;
    if (global_bytes) *global_bytes = (unsigned long long)properties.totalGlobalMem;
    if (name && name_cap) {
        strncpy(name, properties.name, name_cap - 1);
        name[name_cap - 1] = '\0';
    }
    return 0;
}

int yvx_cuda_malloc(void **out, unsigned long long bytes)
{
    if (!out) return YVEX_ERR_INVALID_ARG;
    *out = NULL;
    YVX_CUDA_TRY(cudaMalloc(out, bytes ? (size_t)bytes : 1u));
    return 0;
}

int yvx_cuda_free(void *pointer)
{
    if (!pointer) return 0;
    YVX_CUDA_TRY(cudaFree(pointer));
    return 0;
}

int yvx_cuda_host_alloc(void **out, unsigned long long bytes)
{
    if (!out) return YVEX_ERR_INVALID_ARG;
    *out = NULL;
    YVX_CUDA_TRY(cudaMallocHost(out, bytes ? (size_t)bytes : 1u));
    return 0;
}

int yvx_cuda_host_free(void *pointer)
{
    if (!pointer) return 0;
    YVX_CUDA_TRY(cudaFreeHost(pointer));
    return 0;
}

int yvx_cuda_memset_async(void *device, int value, unsigned long long bytes, void *stream)
{
    YVX_CUDA_TRY(cudaMemsetAsync(device, value, (size_t)bytes, (cudaStream_t)stream));
    return 0;
}

int yvx_cuda_upload_async(void *device, const void *host, unsigned long long bytes, void *stream)
{
    YVX_CUDA_TRY(cudaMemcpyAsync(device, host, (size_t)bytes, cudaMemcpyHostToDevice,
                                 (cudaStream_t)stream));
    return 0;
}

int yvx_cuda_download_async(void *host, const void *device, unsigned long long bytes, void *stream)
{
    YVX_CUDA_TRY(cudaMemcpyAsync(host, device, (size_t)bytes, cudaMemcpyDeviceToHost,
                                 (cudaStream_t)stream));
    return 0;
}

int yvx_cuda_copy_async(void *destination, const void *source, unsigned long long bytes,
                        void *stream)
{
    YVX_CUDA_TRY(cudaMemcpyAsync(destination, source, (size_t)bytes, cudaMemcpyDeviceToDevice,
                                 (cudaStream_t)stream));
    return 0;
}

int yvx_cuda_stream_create(void **stream)
{
    cudaStream_t created;
    if (!stream) return YVEX_ERR_INVALID_ARG;
    YVX_CUDA_TRY(cudaStreamCreateWithFlags(&created, cudaStreamNonBlocking));
    *stream = (void *)created;
    return 0;
}

int yvx_cuda_stream_destroy(void *stream)
{
    if (!stream) return 0;
    YVX_CUDA_TRY(cudaStreamDestroy((cudaStream_t)stream));
    return 0;
}

int yvx_cuda_stream_synchronize(void *stream)
{
    YVX_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return 0;
}

// Stream capture into a CUDA graph: the attention entry points enqueue kernels
// only (no allocation, no synchronisation), so a decode step's calls can be
// captured once and replayed. The reference's operators are capture-aware for
// the same reason (yvex_cuda_capture_active, src/backend/cuda/capability.c:802-805).
int yvx_cuda_graph_capture_begin(void *stream)
{
    if (!stream) return YVEX_ERR_INVALID_ARG;  // the legacy default stream cannot be captured
    YVX_CUDA_TRY(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
    return 0;
}

int yvx_cuda_graph_capture_end(void *stream, void **executable)
{
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    if (!stream || !executable) return YVEX_ERR_INVALID_ARG;
    YVX_CUDA_TRY(cudaStreamEndCapture((cudaStream_t)stream, &graph));
    const cudaError_t error = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (error != cudaSuccess) return yvx_cuda_check(error, "cudaGraphInstantiate");
    *executable = (void *)exec;
    return 0;
}

int yvx_cuda_graph_launch(void *executable, void *stream)
{
    if (!executable) return YVEX_ERR_INVALID_ARG;
    YVX_CUDA_TRY(cudaGraphLaunch((cudaGraphExec_t)executable, (cudaStream_t)stream));
    return 0;
}

int yvx_cuda_graph_destroy(void *executable)
{
    if (!executable) return 0;
    YVX_CUDA_TRY(cudaGraphExecDestroy((cudaGraphExec_t)executable));
    return 0;
}

int yvx_cuda_ipc_export(void *device_pointer, void *handle_64_bytes)
{
    cudaIpcMemHandle_t handle;
    static_assert(sizeof(handle) == 64, "IPC handle size");
    if (!device_pointer || !handle_64_bytes) return YVEX_ERR_INVALID_ARG;
    YVX_CUDA_TRY(cudaIpcGetMemHandle(&handle, device_pointer));
    memcpy(handle_64_bytes, &handle, sizeof(handle));
    return 0;
}

int yvx_cuda_ipc_open(const void *handle_64_bytes, void **device_pointer)
{
    cudaIpcMemHandle_t handle;
    if (!device_pointer || !handle_64_bytes) return YVEX_ERR_INVALID_ARG;
    memcpy(&handle, handle_64_bytes, sizeof(handle));
    YVX_CUDA_TRY(cudaIpcOpenMemHandle(device_pointer, handle, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}

int yvx_cuda_ipc_close(void *device_pointer)
{
    if (!device_pointer) return 0;
    YVX_CUDA_TRY(cudaIpcCloseMemHandle(device_pointer));
    return 0;
}

int yvx_cuda_event_create(void **event)
{
    cudaEvent_t created;
    if (!event) return YVEX_ERR_INVALID_ARG;
    YVX_CUDA_TRY(cudaEventCreate(&created));
    *event = (void *)created;
    return 0;
}

int yvx_cuda_event_destroy(void *event)
{
    if (!event) return 0;
    YVX_CUDA_TRY(cudaEventDestroy((cudaEvent_t)event));
    return 0;
}

int yvx_cuda_event_record(void *event, void *stream)
{
    YVX_CUDA_TRY(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
    return 0;
}

int yvx_cuda_stream_wait_event(void *stream, void *event)
{
    if (!event) return YVEX_ERR_INVALID_ARG;
    YVX_CUDA_TRY(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0));
    return 0;
}

int yvx_cuda_event_elapsed_ms(void *start, void *stop, float *milliseconds)
{
    YVX_CUDA_TRY(cudaEventSynchronize((cudaEvent_t)stop));
    YVX_CUDA_TRY(cudaEventElapsedTime(milliseconds, (cudaEvent_t)start, (cudaEvent_t)stop));
    return 0;
}

}  // extern "C"
