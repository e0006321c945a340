/* TEST INFRASTRUCTURE ONLY: drives the C11 host layer of the library (built with
 * -fsanitize=address,undefined against shim_absent.c) through the paths that need no
 * device: block-pool bookkeeping under a seeded random walk, page and shard geometry, the
 * state-bank layout, rotation frequencies, error helpers, and the refusal ladders of the
 * operators that must stop before any device call. Exits 0 when every check holds; a
 * sanitizer report aborts the process. */
#include "yvex_b200/attention.h"
#include "yvex_b200/attention_job.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define CHECK(cond) do { if (!(cond)) { fprintf(stderr, "check failed: %s (line %d)\n", #cond, __LINE__); return 1; } } while (0)

static unsigned long long state = 0x9E3779B97F4A7C15ull;
static unsigned int draw(unsigned int bound)
{
    state ^= state << 13; state ^= state >> 7; state ^= state << 17;
    return (unsigned int)(state % bound);
}

static int pool_walk(void)
{
    enum { SESSIONS = 6, BLOCKS = 40, BLOCK_TOKENS = 8, PER_SESSION = 12 };
    yvex_b200_kv_pool *pool = yvex_b200_kv_pool_create(BLOCKS, BLOCK_TOKENS, SESSIONS, PER_SESSION);
    unsigned int open[SESSIONS], count = 0, step;
    yvex_b200_kv_copy copy;
    CHECK(pool);
    for (step = 0; step < 20000u; ++step) {
        const unsigned int action = draw(6);
        if ((action == 0 || !count) && count < SESSIONS) {
            unsigned int id;
            if (yvex_b200_kv_pool_session_open(pool, &id) == YVEX_OK) open[count++] = id;
        } else if (action == 1 && count < SESSIONS) {
            unsigned int id;
            if (yvex_b200_kv_pool_session_fork(pool, open[draw(count)], &id) == YVEX_OK) open[count++] = id;
        } else if (action == 2 && count) {
            const unsigned int at = draw(count);
            CHECK(yvex_b200_kv_pool_session_close(pool, open[at]) == YVEX_OK);
            open[at] = open[--count];
        } else if (count) {
            const unsigned int id = open[draw(count)], rows = 1u + draw(20);
            const int rc = yvex_b200_kv_pool_reserve(pool, id, rows, &copy);
            CHECK(rc == YVEX_OK || rc == YVEX_ERR_NOMEM || rc == YVEX_ERR_BOUNDS);
            if (rc == YVEX_OK) {
                const int *row = yvex_b200_kv_pool_table(pool, id);
                const unsigned long long reserved = yvex_b200_kv_pool_reserved(pool, id);
                unsigned long long r;
                for (r = 0; r < reserved; r += BLOCK_TOKENS) CHECK(row[r / BLOCK_TOKENS] >= 0 && row[r / BLOCK_TOKENS] < BLOCKS);
                CHECK(yvex_b200_kv_pool_commit(pool, id, draw(rows + 1u)) == YVEX_OK);
            } else {
                CHECK(yvex_b200_kv_pool_commit(pool, id, 1u) == YVEX_ERR_BOUNDS);
            }
        }
    }
    while (count) CHECK(yvex_b200_kv_pool_session_close(pool, open[--count]) == YVEX_OK);
    CHECK(yvex_b200_kv_pool_free_blocks(pool) == BLOCKS);
    yvex_b200_kv_pool_destroy(pool);
    return 0;
}

static int geometry(void)
{
    yvex_b200_page_request request;
    yvex_b200_kv_bank_component components[3] = {{1, 127, 513, 0, 0}, {1, 10, 512, 0, 0}, {0, 0, 0, 15, 15}};
    yvex_b200_kv_bank_span spans[3];
    yvex_b200_position_policy policy = {10000ull, 16ull, 65536ull, 32ull, 1ull};
    unsigned long long tokens = 0, bytes = 0, first = 0, last = 0, begin = 0, end = 0, total = 0;
    double frequency[32];
    unsigned int i;
    memset(&request, 0, sizeof(request));
    request.logical_block_tokens = 128ull; request.kernel_tile_tokens = 64ull; request.promotion_granularity_tokens = 1ull;
    request.alignment_bytes = 4096ull; request.bytes_per_block = 4096ull; request.page_table_entry_bytes = 8ull;
    request.device_page_bytes = 2ull << 20; request.logical_tokens = 1ull << 20;
    (void)yvex_b200_kv_page_tokens(&request, &tokens, &bytes);
    CHECK(yvex_b200_kv_page_touch(1000ull, 5000ull, 4096ull, &first, &last) && first == 0ull && last == 1ull);
    CHECK(!yvex_b200_kv_page_touch(1ull, 0ull, 4ull, &first, &last));
    for (i = 0; i < 8u; ++i) {
        CHECK(yvex_b200_kv_sequence_shard(131072ull, 8u, i, 64ull, &begin, &end));
        CHECK(end - begin == 16384ull);
    }
    CHECK(!yvex_b200_kv_sequence_shard(100ull, 0u, 0u, 64ull, &begin, &end));
    CHECK(yvex_b200_kv_bank_layout(components, 3u, spans, &total) == 1 && total % 4ull == 0ull);
    CHECK(spans[0].offset[1] % 8ull == 0ull && spans[2].bytes[2] == 60ull);
    CHECK(yvex_b200_rope_frequencies(&policy, 64ull, frequency) == YVEX_OK && frequency[0] == 1.0);
    CHECK(yvex_b200_rope_frequencies(&policy, 1ull, frequency) == YVEX_ERR_INVALID_ARG);
    return 0;
}

static int refusals(void)
{
    yvex_backend *backend = NULL;
    yvex_backend_options options = {YVEX_BACKEND_KIND_CUDA, "0", 0ull};
    yvex_error err;
    yvex_backend_attention_job job;
    yvex_backend_attention_output output;
    yvex_backend_attention_failure failure;
    yvex_backend_capability_result capability;
    yvex_transformer_attention_requirement requirement;
    unsigned long long bytes = 7ull;
    memset(&job, 0, sizeof(job));
    memset(&output, 0, sizeof(output));
    memset(&requirement, 0, sizeof(requirement));
    /* no device behind the stand-in shim: the backend does not open, and says why */
    CHECK(yvex_backend_open(&backend, &options, &err) == YVEX_ERR_UNSUPPORTED && !backend && err.message[0]);
    options.kind = YVEX_BACKEND_KIND_CPU;
    CHECK(yvex_backend_open(&backend, &options, &err) == YVEX_ERR_UNSUPPORTED);
    CHECK(yvex_backend_attention_execute(NULL, &job, &output, &failure, &err) == YVEX_ERR_INVALID_ARG);
    CHECK(failure.code == YVEX_BACKEND_ATTENTION_FAILURE_INVALID_ARGUMENT && failure.stage);
    CHECK(yvex_backend_attention_complete(NULL, NULL, 0, &err) == YVEX_ERR_INVALID_ARG);
    CHECK(yvex_backend_query_capability(NULL, YVEX_BACKEND_VARIANT_ATTENTION_ENCODED, &capability, &err) == YVEX_ERR_INVALID_ARG);
    CHECK(yvex_backend_resident_resolve(NULL, (const unsigned char *)&job, 4ull, &bytes) == YVEX_BACKEND_RESIDENT_MISS && bytes == 0ull);
    CHECK(yvex_backend_state_residency_resolve(NULL, &job, 4ull, &bytes) == YVEX_BACKEND_RESIDENT_MISS);
    CHECK(!strcmp(yvex_backend_operation_variant_name(YVEX_BACKEND_VARIANT_ATTENTION_ENCODED), "encoded-attention"));
    CHECK(!strcmp(yvex_backend_capability_reason_name((yvex_backend_capability_reason)99), "unknown"));
    /* exact-attention admission: geometry first, then the contract */
    CHECK(yvex_b200_transformer_attention_workspace_required(&requirement, &bytes, &err) == YVEX_ERR_INVALID_ARG);
    requirement.query_tokens = 4ull; requirement.key_value_tokens = 4ull; requirement.query_heads = 8ull;
    requirement.key_value_heads = 2ull; requirement.head_dimension = 128ull;
    requirement.query_dtype = requirement.key_dtype = requirement.value_dtype = requirement.output_dtype = YVEX_DTYPE_F32;
    requirement.layout = YVEX_TRANSFORMER_ATTENTION_LAYOUT_TOKEN_HEAD_DIM; requirement.mask = YVEX_TRANSFORMER_ATTENTION_MASK_CAUSAL;
    requirement.numeric_contract = YVEX_TRANSFORMER_ATTENTION_NUMERIC_EXACT_F32; requirement.deterministic = 1;
    CHECK(yvex_b200_transformer_attention_workspace_required(&requirement, &bytes, &err) == YVEX_OK && bytes == 0ull);
    requirement.head_dimension = 257ull;
    CHECK(yvex_b200_transformer_attention_workspace_required(&requirement, &bytes, &err) == YVEX_ERR_UNSUPPORTED);
    requirement.head_dimension = 128ull; requirement.query_start = 1ull;
    CHECK(yvex_b200_transformer_attention_workspace_required(&requirement, &bytes, &err) == YVEX_ERR_INVALID_ARG);
    CHECK(!strcmp(yvex_status_name(YVEX_ERR_BOUNDS), yvex_status_name(YVEX_ERR_BOUNDS)));
    return 0;
}

int main(void)
{
    if (pool_walk() || geometry() || refusals()) return 1;
    puts("host layer clean under the sanitizers");
    return 0;
}
