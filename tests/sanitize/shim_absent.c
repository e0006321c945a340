/* TEST INFRASTRUCTURE ONLY: a stand-in for the device shim (include/yvex_b200/cuda_shim.h)
 * with no device behind it, so that the C11 host layer can be built with AddressSanitizer
 * and UndefinedBehaviorSanitizer and driven on a machine without a GPU (the reference
 * builds its sanitizer lanes with CUDA disabled as well: Makefile:752-849). Every entry
 * point reports "no device" or refuses; none computes anything. */
#include "yvex_b200/abi.h"
#include "yvex_b200/cuda_shim.h"

#include <stddef.h>
#include <string.h>

#define REFUSE(name, ...) int name(__VA_ARGS__) { return YVEX_ERR_UNSUPPORTED; }

const char *yvx_cuda_last_error_text(void) { return "no device: sanitizer build of the host layer"; }
int yvx_cuda_device_count(int *count) { if (count) *count = 0; return 0; }
int yvx_cuda_device_synchronize(void) { return YVEX_ERR_UNSUPPORTED; }
REFUSE(yvx_cuda_device_select, int device)
REFUSE(yvx_cuda_device_properties, int device, int *sm, int *major, int *minor, unsigned long long *bytes, char *name, size_t cap)
REFUSE(yvx_cuda_malloc, void **out, unsigned long long bytes)
int yvx_cuda_free(void *p) { (void)p; return 0; }
REFUSE(yvx_cuda_host_alloc, void **out, unsigned long long bytes)
int yvx_cuda_host_free(void *p) { (void)p; return 0; }
REFUSE(yvx_cuda_memset_async, void *d, int v, unsigned long long n, void *s)
REFUSE(yvx_cuda_upload_async, void *d, const void *h, unsigned long long n, void *s)
REFUSE(yvx_cuda_download_async, void *h, const void *d, unsigned long long n, void *s)
REFUSE(yvx_cuda_copy_async, void *d, const void *s0, unsigned long long n, void *s)
REFUSE(yvx_cuda_stream_create, void **s)
int yvx_cuda_stream_destroy(void *s) { (void)s; return 0; }
REFUSE(yvx_cuda_stream_synchronize, void *s)
void yvx_cuda_gqa_plan_splits(yvx_gqa_problem *p, int sm) { (void)sm; if (p) { p->chunk_tokens = 64u; p->max_splits = 1u; } }
unsigned long long yvx_cuda_gqa_partials_bytes(const yvx_gqa_problem *p) { (void)p; return 0ull; }
unsigned long long yvx_cuda_gqa_f32_staging_bytes(const yvx_gqa_problem *p) { (void)p; return 0ull; }
REFUSE(yvx_cuda_gqa_attention, const yvx_gqa_problem *p, void *s, unsigned int *n)
REFUSE(yvx_cuda_op_attention_f32, const float *q, const float *k, const float *v, unsigned long long n, unsigned long long p, float sc, int c, unsigned long long hd, float *s0, float *s1, float *o, void *s)
unsigned long long yvx_cuda_latent_reduce_workspace_bytes(const yvx_latent_reduce_args *a) { (void)a; return 0ull; }
REFUSE(yvx_cuda_latent_reduce_launches, const yvx_latent_reduce_args *a, void *s, unsigned int *n)
unsigned long long yvx_cuda_csa_select_workspace_bytes(unsigned long long r, unsigned long long t, unsigned int k) { (void)r; (void)t; (void)k; return 0ull; }
REFUSE(yvx_cuda_csa_select, const yvx_csa_select_args *a, void *s, unsigned int *n)
REFUSE(yvx_cuda_kv_append_rotary, const yvx_kv_append_args *a, void *s)
void yvx_cuda_mla_plan(yvx_mla_problem *p, int sm) { (void)p; (void)sm; }
unsigned long long yvx_cuda_mla_absorbed_bytes(const yvx_mla_problem *p) { (void)p; return 0ull; }
unsigned long long yvx_cuda_mla_partials_bytes(const yvx_mla_problem *p) { (void)p; return 0ull; }
REFUSE(yvx_cuda_mla_decode, const yvx_mla_problem *p, void *s, void *e[4], unsigned int *n)
REFUSE(yvx_cuda_compressor_chunk, const yvx_compressor_args *a, void *s, unsigned long long *e)
REFUSE(yvx_cuda_activation_quant, const yvx_activation_args *a, void *s)
REFUSE(yvx_cuda_rows_publish, const yvx_rows_publish_args *a, void *s)
REFUSE(yvx_cuda_rows_publish_batch, const yvx_rows_publish_args *a, unsigned int n, void *s)
unsigned long long yvx_cuda_qtype_row_bytes(unsigned int q, unsigned long long w)
{
    return q == YVX_QTYPE_F32 ? w * 4ull : (q == YVX_QTYPE_F16 || q == YVX_QTYPE_BF16) ? w * 2ull
           : (q == YVX_QTYPE_Q8_0 && w % 32ull == 0ull) ? w / 32ull * 34ull : 0ull;
}
REFUSE(yvx_cuda_qtype_matvec, const yvx_matvec_args *a, void *s)
REFUSE(yvx_cuda_bf16_gemm, const yvx_gemm_args *a, void *s)
unsigned long long yvx_cuda_bf16_gemm_staging_bytes(unsigned long long t, unsigned long long g, unsigned long long w)
{
    return t * (g ? g : 1ull) * w * 2ull;
}
REFUSE(yvx_cuda_qtype_decode_rows, const void *w, unsigned int q, unsigned long long f, unsigned long long r, unsigned long long wd, float *o, int *st, void *s)
REFUSE(yvx_cuda_round_bf16_rows, float *v, unsigned long long r, unsigned long long w, unsigned long long st, int *status, void *s)
unsigned long long yvx_cuda_q8_record_bytes(void) { return 17408ull; }
