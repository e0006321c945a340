/* TEST INFRASTRUCTURE ONLY.
 *
 * The reference's backend core refers to two functions that live in its CUDA
 * backend. The CPU-only reference build in oracle/_ref does not compile that
 * backend, so these two definitions stand in for it and refuse, which is what
 * the reference itself does when CUDA is unavailable.
 */
#include <yvex/internal/backend.h>

int yvex_backend_open_cuda_impl(yvex_backend **out, const char *device,
                                unsigned long long memory_limit_bytes, yvex_error *err)
{
    (void)device;
    (void)memory_limit_bytes;
    if (out) *out = NULL;
    yvex_error_set(err, YVEX_ERR_UNSUPPORTED, "oracle.ref",
                   "the CPU-only reference build has no CUDA backend");
    return YVEX_ERR_UNSUPPORTED;
}

int yvex_backend_cuda_attention_graph_summary_get(
    const yvex_backend *backend, yvex_backend_cuda_attention_graph_summary *out,
    yvex_error *err)
{
    (void)backend;
    (void)out;
    yvex_error_set(err, YVEX_ERR_UNSUPPORTED, "oracle.ref",
                   "the CPU-only reference build has no CUDA backend");
    return YVEX_ERR_UNSUPPORTED;
}
