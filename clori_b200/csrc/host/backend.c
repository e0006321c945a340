/* Backend lifecycle, tensors and the status-word transaction. Mirrors the
 * subset of the reference's backend surface the attention path touches
 * (include/yvex/backend.h:148-206, src/backend/core.c). The only backend kind
 * is CUDA on an sm_100 device; nothing here can execute on the host. */
#include "private.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

int yvex_backend_cuda_available(void)
{
    int count = 0;
    return yvx_cuda_device_count(&count) == 0 && count > 0;
}

int yvx_backend_device_fail(yvex_backend *backend, int rc, const char *where, yvex_error *err)
{
    if (backend && rc == YVEX_ERR_BACKEND) {
        backend->failed = 1;
        if (!backend->failure_reason) backend->failure_reason = 8; /* launch failed */
    }
    yvex_error_set(err, (yvex_status)rc, where, yvx_cuda_last_error_text());
    return rc;
}

int yvx_backend_admit(yvex_backend *backend, const char *where, yvex_error *err)
{
    int rc;
    if (!backend) return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "backend is required");
    if (backend->failed)
        return yvx_fail(err, YVEX_ERR_BACKEND, where,
                        "backend failed earlier and refuses further operations");
    rc = yvx_cuda_device_select(backend->device);
    if (rc != 0) return yvx_backend_device_fail(backend, rc, where, err);
    return YVEX_OK;
}

int yvex_backend_open(yvex_backend **out, const yvex_backend_options *options, yvex_error *err)
{
    const char *where = "yvex_backend_open";
    yvex_backend *backend;
    unsigned long long global_bytes = 0ull;
    int count = 0, device = 0, rc;
    if (out) *out = NULL;
    if (!out || !options) return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "out and options are required");
    if (options->kind != YVEX_BACKEND_KIND_CUDA)
        return yvx_fail(err, YVEX_ERR_UNSUPPORTED, where,
                        "only the CUDA backend exists here; there is no CPU fallback");
    if (options->device && options->device[0]) {
        char *end = NULL;
        long parsed = strtol(options->device, &end, 10);
        if (!end || *end || parsed < 0 || parsed > 1023)
            return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "device must be a decimal index");
        device = (int)parsed;
    }
    if (yvx_cuda_device_count(&count) != 0 || count <= 0)
        return yvx_fail(err, YVEX_ERR_UNSUPPORTED, where, "no CUDA device is available");
    if (device >= count) return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "device index out of range");
    backend = calloc(1, sizeof(*backend));
    if (!backend) return yvx_fail(err, YVEX_ERR_NOMEM, where, "backend allocation failed");
    backend->device = device;
    backend->memory_limit_bytes = options->memory_limit_bytes;
    backend->synchronous = 1;
    backend->tensor_id_next = 1ull;
    rc = yvx_cuda_device_select(device);
    if (rc == 0)
        rc = yvx_cuda_device_properties(device, &backend->sm_count, &backend->cc_major,
                                        &backend->cc_minor, &global_bytes,
                                        backend->device_name, sizeof(backend->device_name));
    if (rc == 0 && backend->cc_major != 10) {
        free(backend);
        return yvx_fail(err, YVEX_ERR_UNSUPPORTED, where,
                        "kernels are built for sm_100a only; this device is not compute capability 10.x");
    }
    if (rc == 0) rc = yvx_cuda_stream_create(&backend->own_stream);
    /* the status word, and behind it (256 bytes on) the arrival tickets of the single-launch
     * split kernels: zero once here, every kernel that uses one leaves it at zero again */
    if (rc == 0) rc = yvx_cuda_malloc((void **)&backend->status_device, 256u + YVX_BACKEND_TICKETS * sizeof(int));
    if (rc == 0) rc = yvx_cuda_memset_async(backend->status_device, 0, 256u + YVX_BACKEND_TICKETS * sizeof(int), backend->own_stream);
    if (rc == 0) rc = yvx_cuda_stream_synchronize(backend->own_stream);
    if (rc == 0) backend->tickets = backend->status_device + 64;
    if (rc == 0) rc = yvx_cuda_host_alloc((void **)&backend->status_host, sizeof(int));
    if (rc != 0) {
        yvex_error_set(err, (yvex_status)rc, where, yvx_cuda_last_error_text());
        yvx_cuda_free(backend->status_device);
        yvx_cuda_host_free(backend->status_host);
        yvx_cuda_stream_destroy(backend->own_stream);
        free(backend);
        return rc;
    }
    backend->stream = backend->own_stream;
    *out = backend;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_close_checked(yvex_backend **handle, yvex_error *err)
{
    const char *where = "yvex_backend_close_checked";
    yvex_backend *backend;
    if (!handle || !*handle) return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "backend is required");
    backend = *handle;
    if (backend->live_tensors)
        return yvx_fail(err, YVEX_ERR_STATE, where, "tensors of this backend are still alive");
    yvx_cuda_device_select(backend->device);
    yvx_cuda_stream_synchronize(backend->stream);
    yvx_cuda_free(backend->scratch);
    yvx_cuda_free(backend->gemm_staging);
    {
        unsigned int i;
        for (i = 0; i < backend->weight_count; ++i) yvx_cuda_free(backend->weights[i].device);
        free(backend->weights);
    }
    yvx_cuda_free(backend->status_device);
    yvx_cuda_host_free(backend->status_host);
    yvx_cuda_stream_destroy(backend->own_stream);
    free(backend);
    *handle = NULL;
    yvex_error_clear(err);
    return YVEX_OK;
}

void yvex_backend_close(yvex_backend *backend)
{
    yvex_error err;
    if (!backend) return;
    backend->live_tensors = 0ull;
    (void)yvex_backend_close_checked(&backend, &err);
}

int yvex_b200_backend_bind_stream(yvex_backend *backend, void *stream, int synchronous,
                                  yvex_error *err)
{
    if (!backend) return yvx_fail(err, YVEX_ERR_INVALID_ARG, "yvex_b200_backend_bind_stream", "backend is required");
    backend->stream = stream ? stream : backend->own_stream;
    backend->synchronous = synchronous != 0;
    yvex_error_clear(err);
    return YVEX_OK;
}

void *yvex_b200_backend_stream(const yvex_backend *backend) { return backend ? backend->stream : NULL; }
int yvex_b200_backend_sm_count(const yvex_backend *backend) { return backend ? backend->sm_count : 0; }

int yvex_backend_sync(yvex_backend *backend, yvex_error *err)
{
    const char *where = "yvex_backend_sync";
    int rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (backend->status_pending) return yvx_backend_status_collect(backend, NULL, where, err);
    rc = yvx_cuda_stream_synchronize(backend->stream);
    if (rc != 0) return yvx_backend_device_fail(backend, rc, where, err);
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvx_backend_scratch(yvex_backend *backend, unsigned long long bytes, void **out,
                        const char *where, yvex_error *err)
{
    int rc;
    *out = NULL;
    if (!bytes) return YVEX_OK;
    if (bytes > backend->scratch_bytes) {
        unsigned long long grown = bytes + bytes / 4ull;
        /* The old arena may still be read by work enqueued on this stream or on one bound
         * earlier (bind_stream): wait for the whole device before releasing it. */
        rc = yvx_cuda_device_synchronize();
        if (rc == 0) rc = yvx_cuda_free(backend->scratch);
        backend->scratch = NULL;
        backend->scratch_bytes = 0ull;
        if (rc == 0) rc = yvx_cuda_malloc(&backend->scratch, grown);
        if (rc != 0) return yvx_backend_device_fail(backend, rc, where, err);
        backend->scratch_bytes = grown;
    }
    *out = backend->scratch;
    return YVEX_OK;
}

/* Host-side fault injection for tests, in the style of the reference's
 * YVEX_TEST_CUDA_LAUNCH_FAILURE / YVEX_TEST_CUDA_SYNC_FAILURE hooks
 * (src/backend/cuda/capability.c:763,806): when the variable names the operator (its `where`
 * string, e.g. "b200.attention.reduce") or "*", the call that would have launched or
 * synchronised reports a backend failure instead and nothing is enqueued. The GPU is never
 * made to fail; what is exercised is the host's handling: typed error, sticky refusal. */
static int injected_failure(const char *variable, const char *where)
{
    const char *value = getenv(variable);
    return value && value[0] && (!strcmp(value, "*") || !strcmp(value, where));
}

static int inject(yvex_backend *backend, const char *what, const char *where, yvex_error *err)
{
    backend->failed = 1;
    backend->failure_reason = strstr(what, "launch") ? 8 : 9;
    yvex_error_set(err, YVEX_ERR_BACKEND, where, what);
    return YVEX_ERR_BACKEND;
}

int yvx_backend_status_arm(yvex_backend *backend, const char *where, yvex_error *err)
{
    int rc;
    if (injected_failure("YVEX_B200_TEST_LAUNCH_FAILURE", where))
        return inject(backend, "injected launch failure (test hook)", where, err);
    if (backend->status_pending) {
        rc = yvx_backend_status_collect(backend, NULL, where, err);
        if (rc != YVEX_OK) return rc;
    }
    rc = yvx_cuda_memset_async(backend->status_device, 0, sizeof(int), backend->stream);
    if (rc != 0) return yvx_backend_device_fail(backend, rc, where, err);
    return YVEX_OK;
}

int yvx_backend_status_collect(yvex_backend *backend, yvex_backend_operation_facts *facts,
                               const char *where, yvex_error *err)
{
    int rc;
    if (injected_failure("YVEX_B200_TEST_SYNC_FAILURE", where)) {
        /* the real work was enqueued: drain it so that nothing is in flight behind the refusal */
        (void)yvx_cuda_stream_synchronize(backend->stream);
        backend->status_pending = 0;
        return inject(backend, "injected synchronisation failure (test hook)", where, err);
    }
    rc = yvx_cuda_download_async(backend->status_host, backend->status_device, sizeof(int),
                                 backend->stream);
    if (rc == 0) rc = yvx_cuda_stream_synchronize(backend->stream);
    backend->status_pending = 0;
    if (rc != 0) {
        if (rc == YVEX_ERR_BACKEND) backend->failure_reason = 9; /* synchronisation failed */
        return yvx_backend_device_fail(backend, rc, where, err);
    }
    if (facts) {
        facts->d2h_bytes += sizeof(int);
        facts->download_count += 1ull;
        facts->device_synchronizations += 1ull;
    }
    if (*backend->status_host == 1)
        return yvx_fail(err, YVEX_ERR_FORMAT, where, "attention produced a non-finite value");
    if (*backend->status_host == 3) {
        /* A bounded device-side wait gave up: a copy that never landed, or a peer that never
         * wrote its rows. Unlike a bad block table this is the device (or a peer) not answering,
         * so it is a backend failure and sticky, as the reference treats a failed synchronisation
         * (src/backend/cuda/capability.c:757-817). After an exchange timeout the arrival counters
         * are out of step with the epoch: the exchange area must be zeroed before it is reused. */
        backend->failed = 1;
        backend->failure_reason = 9; /* synchronisation failed */
        return yvx_fail(err, YVEX_ERR_BACKEND, where,
                        "a bounded device-side wait timed out (a copy or a peer never arrived)");
    }
    if (*backend->status_host != 0)
        return yvx_fail(err, YVEX_ERR_FORMAT, where, "attention kernel reported a contract failure");
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvx_tensor_owned(const yvex_backend *backend, const yvex_device_tensor *tensor)
{
    return backend && tensor && tensor->owner == backend && tensor->data;
}

static int tensor_create(yvex_backend *backend, const yvex_backend_tensor_desc *desc,
                         void *borrowed, yvex_device_tensor **out, const char *where,
                         yvex_error *err)
{
    yvex_device_tensor *tensor;
    unsigned int i;
    int rc;
    if (out) *out = NULL;
    rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (!desc || !out || !desc->bytes || desc->rank > YVEX_TENSOR_MAX_DIMS)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "a complete tensor description is required");
    if (!borrowed && backend->memory_limit_bytes &&
        backend->allocated_bytes + desc->bytes > backend->memory_limit_bytes)
        return yvx_fail(err, YVEX_ERR_NOMEM, where, "backend memory limit exceeded");
    tensor = calloc(1, sizeof(*tensor));
    if (!tensor) return yvx_fail(err, YVEX_ERR_NOMEM, where, "tensor allocation failed");
    if (desc->name) {
        tensor->name = malloc(strlen(desc->name) + 1u);
        if (tensor->name) strcpy(tensor->name, desc->name);
    }
    tensor->owner = backend;
    tensor->owner_id = backend->tensor_id_next++;
    tensor->dtype = desc->dtype;
    tensor->rank = desc->rank;
    for (i = 0; i < desc->rank; ++i) tensor->dims[i] = desc->dims[i];
    tensor->bytes = desc->bytes;
    if (borrowed) {
        tensor->data = borrowed;
        tensor->is_written = 1;
    } else {
        void *device = NULL;
        rc = yvx_cuda_malloc(&device, desc->bytes);
        if (rc != 0) {
            free(tensor->name);
            free(tensor);
            return yvx_backend_device_fail(backend, rc, where, err);
        }
        tensor->data = device;
        tensor->backend_allocation = device;
        tensor->resident_bytes = desc->bytes;
        backend->allocated_bytes += desc->bytes;
    }
    backend->live_tensors += 1ull;
    *out = tensor;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_tensor_alloc(yvex_backend *backend, const yvex_backend_tensor_desc *desc,
                              yvex_device_tensor **out, yvex_error *err)
{
    return tensor_create(backend, desc, NULL, out, "yvex_backend_tensor_alloc", err);
}

int yvex_b200_tensor_wrap(yvex_backend *backend, const yvex_backend_tensor_desc *desc,
                          void *device_pointer, yvex_device_tensor **out, yvex_error *err)
{
    if (!device_pointer)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, "yvex_b200_tensor_wrap", "device pointer is required");
    return tensor_create(backend, desc, device_pointer, out, "yvex_b200_tensor_wrap", err);
}

int yvex_backend_tensor_release(yvex_backend *backend, yvex_device_tensor **handle,
                                yvex_error *err)
{
    const char *where = "yvex_backend_tensor_release";
    yvex_device_tensor *tensor;
    int rc = YVEX_OK;
    if (!handle || !*handle) return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "tensor is required");
    tensor = *handle;
    if (!backend || tensor->owner != backend)
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "tensor must belong to this backend");
    if (tensor->backend_allocation) {
        yvx_cuda_device_select(backend->device);
        rc = yvx_cuda_stream_synchronize(backend->stream);
        if (rc == 0) rc = yvx_cuda_free(tensor->backend_allocation);
        if (rc != 0) return yvx_backend_device_fail(backend, rc, where, err);
        backend->allocated_bytes -= tensor->resident_bytes;
    }
    backend->live_tensors -= 1ull;
    free(tensor->name);
    free(tensor);
    *handle = NULL;
    yvex_error_clear(err);
    return YVEX_OK;
}

void yvex_backend_tensor_free(yvex_backend *backend, yvex_device_tensor *tensor)
{
    yvex_error err;
    if (tensor) (void)yvex_backend_tensor_release(backend, &tensor, &err);
}

static int tensor_rw_admit(yvex_backend *backend, const yvex_device_tensor *tensor,
                           const void *host, unsigned long long len, const char *where,
                           yvex_error *err)
{
    int rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (!tensor || !host) return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "tensor and host buffer are required");
    if (!yvx_tensor_owned(backend, tensor))
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "tensor must belong to this backend");
    if (len > tensor->bytes) return yvx_fail(err, YVEX_ERR_BOUNDS, where, "length exceeds tensor bytes");
    return YVEX_OK;
}

int yvex_backend_tensor_write(yvex_backend *backend, yvex_device_tensor *tensor, const void *src,
                              unsigned long long len, yvex_error *err)
{
    const char *where = "yvex_backend_tensor_write";
    int rc = tensor_rw_admit(backend, tensor, src, len, where, err);
    if (rc != YVEX_OK) return rc;
    rc = yvx_cuda_upload_async(tensor->data, src, len, backend->stream);
    if (rc == 0) rc = yvx_cuda_stream_synchronize(backend->stream);
    if (rc != 0) return yvx_backend_device_fail(backend, rc, where, err);
    tensor->is_written = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_tensor_read(yvex_backend *backend, const yvex_device_tensor *tensor, void *dst,
                             unsigned long long len, yvex_error *err)
{
    const char *where = "yvex_backend_tensor_read";
    int rc = tensor_rw_admit(backend, tensor, dst, len, where, err);
    if (rc != YVEX_OK) return rc;
    if (!tensor->is_written) return yvx_fail(err, YVEX_ERR_STATE, where, "tensor has not been written");
    rc = yvx_cuda_download_async(dst, tensor->data, len, backend->stream);
    if (rc == 0) rc = yvx_cuda_stream_synchronize(backend->stream);
    if (rc != 0) return yvx_backend_device_fail(backend, rc, where, err);
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_tensor_zero(yvex_backend *backend, yvex_device_tensor *tensor, yvex_error *err)
{
    const char *where = "yvex_backend_tensor_zero";
    int rc = yvx_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (!yvx_tensor_owned(backend, tensor))
        return yvx_fail(err, YVEX_ERR_INVALID_ARG, where, "tensor must belong to this backend");
    rc = yvx_cuda_memset_async(tensor->data, 0, tensor->bytes, backend->stream);
    if (rc == 0) rc = yvx_cuda_stream_synchronize(backend->stream);
    if (rc != 0) return yvx_backend_device_fail(backend, rc, where, err);
    tensor->is_written = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}

/* include/yvex/internal/backend.h:258-260, src/backend/core.c:1763-1778. */
int yvex_backend_tensor_f32_subview(const yvex_device_tensor *source, unsigned long long offset,
                                    unsigned long long count, yvex_device_tensor *view)
{
    unsigned long long end;
    if (!source || !view || source->dtype != YVEX_DTYPE_F32 || !yvx_u64_add(offset, count, &end) ||
        end > source->bytes / sizeof(float))
        return 0;
    *view = *source;
    view->rank = 1u;
    view->dims[0] = count;
    view->bytes = count * sizeof(float);
    view->data = source->data + offset * sizeof(float);
    view->backend_allocation = NULL;
    return 1;
}
