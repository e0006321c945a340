/* KV block and page indexing: integer arithmetic that must agree bit for bit
 * with the reference's capacity plan and page store. */
#include "private.h"

static unsigned long long pages_gcd(unsigned long long a, unsigned long long b)
{
    while (b) {
        unsigned long long r = a % b;
        a = b;
        b = r;
    }
    return a;
}

static int pages_lcm(unsigned long long a, unsigned long long b, unsigned long long *out)
{
    if (!a || !b) return 0;
    return yvx_u64_mul(a / pages_gcd(a, b), b, out);
}

/* src/deployment/plan.c:208-283 (capacity_state_geometry): candidates are the
 * multiples of lcm(logical block, kernel tile, promotion granularity,
 * alignment expressed in tokens) up to what one device page holds; the score
 * of a candidate is page-table bytes + fragmentation bytes + one page when
 * copy-on-write + fragmentation again for a candidate-extent class; candidates
 * whose page bytes miss the alignment are skipped; ties go to fewer tokens. */
int yvex_b200_kv_page_tokens(const yvex_b200_page_request *r, unsigned long long *page_tokens,
                             unsigned long long *page_bytes)
{
    unsigned long long base, align_blocks, align_tokens, limit, candidate;
    unsigned long long best = 0ull, best_score = ULLONG_MAX;
    if (!r || !page_tokens || !page_bytes || !r->logical_block_tokens ||
        !r->kernel_tile_tokens || !r->promotion_granularity_tokens || !r->alignment_bytes ||
        !r->bytes_per_block)
        return 0;
    if (!pages_lcm(r->logical_block_tokens, r->kernel_tile_tokens, &base) ||
        !pages_lcm(base, r->promotion_granularity_tokens, &base))
        return 0;
    align_blocks = r->alignment_bytes / pages_gcd(r->bytes_per_block, r->alignment_bytes);
    if (!yvx_u64_mul(r->logical_block_tokens, align_blocks, &align_tokens) ||
        !pages_lcm(base, align_tokens, &base))
        return 0;
    limit = r->device_page_bytes / r->bytes_per_block;
    if (!yvx_u64_mul(limit, r->logical_block_tokens, &limit)) return 0;
    limit -= limit % base;
    if (limit < base) limit = base;
    for (candidate = base; candidate <= limit;) {
        unsigned long long pages, rounded, blocks, bytes, table, waste, score, spare;
        pages = r->logical_tokens / candidate + (r->logical_tokens % candidate ? 1ull : 0ull);
        if (!yvx_u64_mul(pages, candidate, &rounded)) return 0;
        blocks = candidate / r->logical_block_tokens;
        if (candidate % r->logical_block_tokens || !blocks ||
            !yvx_u64_mul(blocks, r->bytes_per_block, &bytes))
            return 0;
        if (!(bytes % r->alignment_bytes)) {
            if (!yvx_u64_mul(pages, r->page_table_entry_bytes, &table)) return 0;
            spare = rounded - r->logical_tokens;
            blocks = spare / r->logical_block_tokens + (spare % r->logical_block_tokens ? 1ull : 0ull);
            if (!yvx_u64_mul(blocks, r->bytes_per_block, &waste)) return 0;
            score = table;
            if (!yvx_u64_add(score, waste, &score) ||
                !yvx_u64_add(score, r->copy_on_write ? bytes : 0ull, &score) ||
                !yvx_u64_add(score, r->candidate_extent ? waste : 0ull, &score))
                return 0;
            if (score < best_score || (score == best_score && candidate < best)) {
                best_score = score;
                best = candidate;
            }
        }
        if (limit - candidate < base) break;
        candidate += base;
    }
    if (!best) return 0;
    *page_tokens = best;
    return yvx_u64_mul(best / r->logical_block_tokens, r->bytes_per_block, page_bytes);
}

/* src/graph/state_pages.c:660-669: first = start / page, last = (end-1) / page. */
int yvex_b200_kv_page_touch(unsigned long long element_start, unsigned long long element_count,
                            unsigned long long page_elements, unsigned long long *first_page,
                            unsigned long long *last_page)
{
    unsigned long long end;
    if (!element_count || !page_elements || !first_page || !last_page ||
        !yvx_u64_add(element_start, element_count, &end))
        return 0;
    *first_page = element_start / page_elements;
    *last_page = (end - 1ull) / page_elements;
    return 1;
}

/* Logical KV row -> pool row under a block table (extension). */
unsigned long long yvex_b200_kv_block_row(const int *block_table,
                                          unsigned long long block_tokens,
                                          unsigned long long row)
{
    return (unsigned long long)block_table[row / block_tokens] * block_tokens + row % block_tokens;
}

/* Contiguous block-aligned token ranges for KV-sequence sharding: the first
 * (blocks % shards) shards take one block more than the others. */
int yvex_b200_kv_sequence_shard(unsigned long long tokens, unsigned int shards, unsigned int index,
                                unsigned long long block_tokens, unsigned long long *begin,
                                unsigned long long *end)
{
    unsigned long long blocks, base, extra, first;
    if (!shards || index >= shards || !block_tokens || !begin || !end) return 0;
    blocks = tokens / block_tokens + (tokens % block_tokens ? 1ull : 0ull);
    base = blocks / shards;
    extra = blocks % shards;
    first = (unsigned long long)index * base + (index < extra ? index : extra);
    *begin = first * block_tokens;
    *end = (first + base + (index < extra ? 1ull : 0ull)) * block_tokens;
    if (*begin > tokens) *begin = tokens;
    if (*end > tokens) *end = tokens;
    return 1;
}

/* The byte layout of one layer's state bank (src/runtime/state_residency.c:44-54, 346-395):
 * per component three spans, values, positions, auxiliary, each starting at the next 8-byte
 * boundary of a running cursor. A history component holds capacity * value_width floats and
 * capacity u64 positions and no auxiliary bytes; a rolling component holds its kv-state floats
 * as values and its score-state floats as auxiliary. Returns 0 on overflow or bad arguments. */
int yvex_b200_kv_bank_layout(const yvex_b200_kv_bank_component *components, unsigned int count,
                             yvex_b200_kv_bank_span *spans, unsigned long long *bank_bytes)
{
    unsigned long long cursor = 0ull;
    unsigned int i, k;
    if (!components || !spans || !bank_bytes || !count || count > 16u) return 0;
    for (i = 0; i < count; ++i) {
        unsigned long long bytes[3] = {0ull, 0ull, 0ull};
        if (components[i].history) {
            if (!yvx_u64_mul(components[i].capacity, components[i].value_width, &bytes[0]) ||
                !yvx_u64_mul(bytes[0], sizeof(float), &bytes[0]) ||
                !yvx_u64_mul(components[i].capacity, sizeof(unsigned long long), &bytes[1]))
                return 0;
        } else if (!yvx_u64_mul(components[i].kv_state_extent, sizeof(float), &bytes[0]) ||
                   !yvx_u64_mul(components[i].score_state_extent, sizeof(float), &bytes[2])) {
            return 0;
        }
        for (k = 0; k < 3u; ++k) {
            unsigned long long aligned;
            if (cursor > ULLONG_MAX - 7ull) return 0;
            aligned = (cursor + 7ull) & ~7ull;
            if (bytes[k] > ULLONG_MAX - aligned) return 0;
            spans[i].offset[k] = aligned;
            spans[i].bytes[k] = bytes[k];
            cursor = aligned + bytes[k];
        }
    }
    *bank_bytes = cursor;
    return 1;
}
