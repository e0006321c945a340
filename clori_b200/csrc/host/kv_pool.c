/* Block-table bookkeeping for the pooled KV layout: which pool blocks a session
 * owns, shared prefixes, copy-on-write of a shared last block, and the
 * candidate / committed split that speculative decoding needs.
 *
 * The reference keeps two banks per layer (committed and candidate) that are
 * contiguous in virtual address space, copies the committed delta into the
 * candidate bank each transaction and commits pages lazily
 * (src/runtime/state_residency.c:346-483, :678-776); candidate rows become
 * visible only through select_prefix (src/graph/state.c:1329-1413). Here the
 * same contract is kept with one pool: rows [0, committed) of a session are
 * visible, rows [committed, reserved) are candidates that attention may read for
 * the session's own verify step, commit(accepted) moves the boundary and drops
 * the rest, and a forked session shares its parent's blocks until it writes.
 * Everything here is host-side integer bookkeeping; the only device work it
 * asks for is the copy list of a copy-on-write. */
#include "private.h"

#include <stdlib.h>
#include <string.h>

struct yvex_b200_kv_pool {
    unsigned int blocks, block_tokens, max_sessions, max_blocks_per_session;
    unsigned int free_count;
    unsigned int *free_list;     /* stack of free pool blocks */
    unsigned int *refcount;      /* [blocks] */
    int *table;                  /* [max_sessions][max_blocks_per_session], -1 = none */
    unsigned long long *committed, *reserved; /* rows per session */
    unsigned char *open;
};

static unsigned int blocks_for(const yvex_b200_kv_pool *pool, unsigned long long rows)
{
    return (unsigned int)((rows + pool->block_tokens - 1ull) / pool->block_tokens);
}

yvex_b200_kv_pool *yvex_b200_kv_pool_create(unsigned int blocks, unsigned int block_tokens,
                                            unsigned int max_sessions, unsigned int max_blocks_per_session)
{
    yvex_b200_kv_pool *pool;
    unsigned int i;
    size_t cell;
    if (!blocks || !block_tokens || !max_sessions || !max_blocks_per_session || blocks > 0x7fffffffu) return NULL;
    pool = (yvex_b200_kv_pool *)calloc(1, sizeof(*pool));
    if (!pool) return NULL;
    pool->blocks = blocks;
    pool->block_tokens = block_tokens;
    pool->max_sessions = max_sessions;
    pool->max_blocks_per_session = max_blocks_per_session;
    pool->free_list = (unsigned int *)malloc(sizeof(unsigned int) * blocks);
    pool->refcount = (unsigned int *)calloc(blocks, sizeof(unsigned int));
    pool->table = (int *)malloc(sizeof(int) * (size_t)max_sessions * max_blocks_per_session);
    pool->committed = (unsigned long long *)calloc(max_sessions, sizeof(unsigned long long));
    pool->reserved = (unsigned long long *)calloc(max_sessions, sizeof(unsigned long long));
    pool->open = (unsigned char *)calloc(max_sessions, 1);
    if (!pool->free_list || !pool->refcount || !pool->table || !pool->committed || !pool->reserved || !pool->open) {
        yvex_b200_kv_pool_destroy(pool);
        return NULL;
    }
    /* block 0 is handed out first: the stack holds blocks-1 .. 0 */
    for (i = 0; i < blocks; ++i) pool->free_list[i] = blocks - 1u - i;
    pool->free_count = blocks;
    for (cell = 0; cell < (size_t)max_sessions * max_blocks_per_session; ++cell) pool->table[cell] = -1;
    return pool;
}

void yvex_b200_kv_pool_destroy(yvex_b200_kv_pool *pool)
{
    if (!pool) return;
    free(pool->free_list);
    free(pool->refcount);
    free(pool->table);
    free(pool->committed);
    free(pool->reserved);
    free(pool->open);
    free(pool);
}

static int session_ok(const yvex_b200_kv_pool *pool, unsigned int session)
{
    return pool && session < pool->max_sessions && pool->open[session];
}

static void release_block(yvex_b200_kv_pool *pool, int block)
{
    if (block < 0) return;
    if (--pool->refcount[block] == 0u) pool->free_list[pool->free_count++] = (unsigned int)block;
}

int yvex_b200_kv_pool_session_open(yvex_b200_kv_pool *pool, unsigned int *session)
{
    unsigned int s;
    if (!pool || !session) return YVEX_ERR_INVALID_ARG;
    for (s = 0; s < pool->max_sessions; ++s)
        if (!pool->open[s]) {
            pool->open[s] = 1;
            pool->committed[s] = pool->reserved[s] = 0ull;
            *session = s;
            return YVEX_OK;
        }
    return YVEX_ERR_BOUNDS;
}

int yvex_b200_kv_pool_session_close(yvex_b200_kv_pool *pool, unsigned int session)
{
    unsigned int j;
    int *row;
    if (!session_ok(pool, session)) return YVEX_ERR_INVALID_ARG;
    row = pool->table + (size_t)session * pool->max_blocks_per_session;
    for (j = 0; j < pool->max_blocks_per_session; ++j) {
        release_block(pool, row[j]);
        row[j] = -1;
    }
    pool->open[session] = 0;
    pool->committed[session] = pool->reserved[session] = 0ull;
    return YVEX_OK;
}

/* A new session that sees the parent's committed rows without copying them. */
int yvex_b200_kv_pool_session_fork(yvex_b200_kv_pool *pool, unsigned int parent, unsigned int *child)
{
    unsigned int j, used;
    int rc;
    const int *from;
    int *to;
    if (!session_ok(pool, parent) || !child) return YVEX_ERR_INVALID_ARG;
    rc = yvex_b200_kv_pool_session_open(pool, child);
    if (rc != YVEX_OK) return rc;
    from = pool->table + (size_t)parent * pool->max_blocks_per_session;
    to = pool->table + (size_t)*child * pool->max_blocks_per_session;
    used = blocks_for(pool, pool->committed[parent]);
    for (j = 0; j < used; ++j) {
        to[j] = from[j];
        pool->refcount[from[j]]++;
    }
    pool->committed[*child] = pool->reserved[*child] = pool->committed[parent];
    return YVEX_OK;
}

/* Makes rows [committed, committed + new_rows) of the session writable: allocates
 * the blocks they need and, when the block holding row `committed` is shared with
 * another session, replaces it by a private block and reports the copy the caller
 * must make on the device (rows [0, copy_rows) of src block into dst block, for K
 * and for V) before appending. At most one copy per call. Candidate rows of an
 * earlier reserve that were never committed are dropped first. */
int yvex_b200_kv_pool_reserve(yvex_b200_kv_pool *pool, unsigned int session, unsigned int new_rows,
                              yvex_b200_kv_copy *copy)
{
    unsigned long long first, last;
    unsigned int j, first_block, need, have, fresh;
    int *row;
    if (copy) memset(copy, 0, sizeof(*copy));
    if (!session_ok(pool, session) || !new_rows || !copy) return YVEX_ERR_INVALID_ARG;
    row = pool->table + (size_t)session * pool->max_blocks_per_session;
    first = pool->committed[session];
    last = first + new_rows;
    need = blocks_for(pool, last);
    if (need > pool->max_blocks_per_session) return YVEX_ERR_BOUNDS;
    /* drop blocks that only held rejected candidates */
    have = blocks_for(pool, first);
    for (j = have; j < pool->max_blocks_per_session; ++j) {
        release_block(pool, row[j]);
        row[j] = -1;
    }
    /* the candidates are gone whatever follows: a refusal below must not leave a reserved
     * range whose table entries were just released */
    pool->reserved[session] = first;
    first_block = (unsigned int)(first / pool->block_tokens);
    fresh = need - have;
    if (first % pool->block_tokens && pool->refcount[row[first_block]] > 1u) fresh += 1u;
    if (fresh > pool->free_count) return YVEX_ERR_NOMEM;
    if (first % pool->block_tokens && pool->refcount[row[first_block]] > 1u) {
        const unsigned int replacement = pool->free_list[--pool->free_count];
        copy->needed = 1;
        copy->source_block = row[first_block];
        copy->destination_block = (int)replacement;
        copy->rows = (unsigned int)(first % pool->block_tokens);
        pool->refcount[row[first_block]]--;
        pool->refcount[replacement] = 1u;
        row[first_block] = (int)replacement;
    }
    for (j = have; j < need; ++j) {
        const unsigned int block = pool->free_list[--pool->free_count];
        pool->refcount[block] = 1u;
        row[j] = (int)block;
    }
    pool->reserved[session] = last;
    return YVEX_OK;
}

/* Accepts the first `accepted_rows` candidate rows; the others are forgotten. */
int yvex_b200_kv_pool_commit(yvex_b200_kv_pool *pool, unsigned int session, unsigned int accepted_rows)
{
    unsigned int j, keep;
    int *row;
    if (!session_ok(pool, session)) return YVEX_ERR_INVALID_ARG;
    if (pool->committed[session] + accepted_rows > pool->reserved[session]) return YVEX_ERR_BOUNDS;
    pool->committed[session] += accepted_rows;
    pool->reserved[session] = pool->committed[session];
    row = pool->table + (size_t)session * pool->max_blocks_per_session;
    keep = blocks_for(pool, pool->committed[session]);
    for (j = keep; j < pool->max_blocks_per_session; ++j) {
        release_block(pool, row[j]);
        row[j] = -1;
    }
    return YVEX_OK;
}

const int *yvex_b200_kv_pool_table(const yvex_b200_kv_pool *pool, unsigned int session)
{
    return session_ok(pool, session) ? pool->table + (size_t)session * pool->max_blocks_per_session : NULL;
}

unsigned long long yvex_b200_kv_pool_committed(const yvex_b200_kv_pool *pool, unsigned int session)
{
    return session_ok(pool, session) ? pool->committed[session] : 0ull;
}

unsigned long long yvex_b200_kv_pool_reserved(const yvex_b200_kv_pool *pool, unsigned int session)
{
    return session_ok(pool, session) ? pool->reserved[session] : 0ull;
}

unsigned int yvex_b200_kv_pool_free_blocks(const yvex_b200_kv_pool *pool)
{
    return pool ? pool->free_count : 0u;
}

unsigned int yvex_b200_kv_pool_block_refcount(const yvex_b200_kv_pool *pool, unsigned int block)
{
    return pool && block < pool->blocks ? pool->refcount[block] : 0u;
}
