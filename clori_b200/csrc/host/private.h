/* Host-side state shared by the C11 operator files. Host code never includes
 * a CUDA header: everything device-side goes through yvex_b200/cuda_shim.h. */
#ifndef YVEX_B200_HOST_PRIVATE_H
#define YVEX_B200_HOST_PRIVATE_H

#include <limits.h>
#include <stddef.h>

#include "yvex_b200/attention.h"
#include "yvex_b200/cuda_shim.h"

enum { YVX_BACKEND_TICKETS = 4096 };

struct yvex_backend {
    int device, sm_count, cc_major, cc_minor;
    char device_name[128];
    void *own_stream, *stream;
    int synchronous;
    /* A failed launch or synchronisation is sticky, as in the reference
     * (src/backend/cuda/capability.c:757-817): later operators are refused. */
    int failed;
    unsigned long long tensor_id_next, allocated_bytes, memory_limit_bytes, live_tensors;
    /* Grow-only device scratch for split-KV partials; backend-owned, like the
     * reference's transient work allocations. */
    void *scratch;
    unsigned long long scratch_bytes;
    int *status_device; /* device status word the kernels publish into */
    int *tickets;       /* YVX_BACKEND_TICKETS zeroed device counters (arrival tickets) */
    int *status_host;   /* pinned mirror */
    int status_pending; /* an asynchronous operator has not been checked yet */
    /* why `failed` was set, in the capability vocabulary (yvex_backend_capability_reason):
     * 8 a launch failed, 9 a synchronisation failed or a bounded device wait ran out */
    int failure_reason;
    /* Encoded weights of the attention job, uploaded on first use and kept until close:
     * the reference resolves weights to resident device memory by their host address
     * (src/backend/cuda/attention.c:560-580); the artifact bytes behind it are immutable. */
    struct yvx_resident_weight {
        const void *host;
        unsigned long long bytes, fingerprint;
        void *device;
    } *weights;
    unsigned int weight_count, weight_capacity;
    /* The runtime's resident weight arena (yvex_backend_resident_attach) and its resolver for
     * mutable state (yvex_backend_state_residency_attach): borrowed mappings from host ranges
     * to device memory the runtime owns (src/backend/residency.c:24-207). */
    const unsigned char *resident_host_base;
    unsigned long long resident_host_bytes, resident_device_address, resident_generation;
    const void *state_residency_context;
    int (*state_residency_resolve)(const void *context, const void *host, unsigned long long bytes,
                                   unsigned long long *device_address);
    unsigned long long state_residency_generation;
    /* Row projections of the attention job go through the tensor-core GEMM from this many
     * tokens on (0: never; yvex_b200_backend_projection_gemm). Its bf16 activation staging
     * is a grow-only buffer of its own. */
    unsigned long long projection_gemm_tokens;
    void *gemm_staging;
    unsigned long long gemm_staging_bytes;
};

static inline int yvx_u64_add(unsigned long long a, unsigned long long b,
                              unsigned long long *out)
{
    if (a > ULLONG_MAX - b) return 0;
    *out = a + b;
    return 1;
}

static inline int yvx_u64_mul(unsigned long long a, unsigned long long b,
                              unsigned long long *out)
{
    if (a && b > ULLONG_MAX / a) return 0;
    *out = a * b;
    return 1;
}

int yvx_fail(yvex_error *err, yvex_status code, const char *where, const char *message);
int yvx_backend_admit(yvex_backend *backend, const char *where, yvex_error *err);
int yvx_backend_scratch(yvex_backend *backend, unsigned long long bytes, void **out,
                        const char *where, yvex_error *err);
int yvx_backend_device_fail(yvex_backend *backend, int rc, const char *where, yvex_error *err);
/* Clears the status word before an operator and reads it back after: returns
 * YVEX_ERR_FORMAT when a kernel published a non-finite or contract failure. */
int yvx_backend_status_arm(yvex_backend *backend, const char *where, yvex_error *err);
int yvx_backend_status_collect(yvex_backend *backend, yvex_backend_operation_facts *facts,
                               const char *where, yvex_error *err);
int yvx_tensor_owned(const yvex_backend *backend, const yvex_device_tensor *tensor);
unsigned long long yvx_dtype_bytes(yvex_dtype dtype);

#endif
