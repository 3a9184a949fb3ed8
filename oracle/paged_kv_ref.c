/*
 * CPU restatement of the paged KV-cache append and gather in plain C.
 * TEST INFRASTRUCTURE ONLY: the tests, the smoke check and the benchmark's
 * CPU-baseline leg load this; the product never does.
 *
 * Parity status: PINNED through oracle/paged_kv_oracle.py, which is checked
 * against outputs of the unmodified reference (tests/golden); this file is in
 * turn checked against that Python oracle on the same seeded inputs
 * (tests/test_oracle_c.py).
 *
 * The arithmetic follows the reference:
 *   position -> (block, slot) = (pos / page_size, pos % page_size) and one
 *   head_dim row copied per (sequence, head, token) for keys and for values
 *     python/barqtrain/kv_cache.py:84-89   (CPU loop)
 *     csrc/kernels/paged_kv_cache.cu:36-53 (GPU kernel, same index math)
 *   capacity rule "start + new_tokens <= max_cache_len", checked per sequence
 *   in order, earlier sequences stay written
 *     python/barqtrain/kv_cache.py:77-83
 *   flattened read-back of a sequence: blocks back to back, cut at its length
 *     python/barqtrain/kv_cache.py:120-133
 * The block-table forms generalise "block j of sequence b" to
 * "physical page table[b][j]"; with table[b][j] = j they reduce to the above.
 *
 * All sizes are in BYTES so one body serves every element type; the path
 * copies bit patterns and never interprets them.
 */
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int barqkv_ref_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/*
 * Reference layout: cache [max_batch, H, max_blocks, page_size, D], new rows
 * [B, H, T, D], both contiguous.  Returns 0, or 1 + the index of the first
 * sequence that does not fit (sequences before it were appended, as in the
 * reference's CPU loop).
 */
int barqkv_ref_append_legacy(uint8_t* keys, uint8_t* values, int32_t* seq_lens,
                             const uint8_t* k_new, const uint8_t* v_new,
                             int B, int H, int T, int max_blocks, int page_size,
                             int max_cache_len, int64_t row_bytes) {
    const int64_t page_bytes = (int64_t)page_size * row_bytes;
    for (int b = 0; b < B; ++b) {
        const int start = seq_lens[b];
        if (start + T > max_cache_len) return 1 + b;
#pragma omp parallel for collapse(2) schedule(static)
        for (int h = 0; h < H; ++h) {
            for (int t = 0; t < T; ++t) {
                const int pos = start + t;
                const int block = pos / page_size;
                const int slot = pos % page_size;
                const int64_t dst = (((int64_t)b * H + h) * max_blocks + block) * page_bytes + (int64_t)slot * row_bytes;
                const int64_t src = (((int64_t)b * H + h) * T + t) * row_bytes;
                memcpy(keys + dst, k_new + src, (size_t)row_bytes);
                memcpy(values + dst, v_new + src, (size_t)row_bytes);
            }
        }
        seq_lens[b] = start + T;
    }
    return 0;
}

/*
 * Block-table append.  Pool page p of head h starts at
 * h * pool_head_stride + p * pool_page_stride (bytes).  Batch entry i appends
 * tokens cu_new[i] .. cu_new[i+1]-1 of the packed new rows (row of token r,
 * head h at r * new_tok_stride + h * new_head_stride) to sequence slot
 * slots[i] (i when slots is NULL) starting at position start[i].
 * Returns 0, or -1 if a table entry is outside [0, num_pages).
 */
int barqkv_ref_append_paged(uint8_t* k_pool, uint8_t* v_pool,
                            int64_t pool_head_stride, int64_t pool_page_stride, int num_pages,
                            const int32_t* table, int table_stride,
                            const int32_t* slots, const int32_t* start, const int32_t* cu_new, int n,
                            const uint8_t* k_new, const uint8_t* v_new,
                            int64_t new_tok_stride, int64_t new_head_stride,
                            int H, int page_size, int64_t row_bytes) {
    int bad = 0;
    for (int i = 0; i < n; ++i) {
        const int slot_row = slots ? slots[i] : i;
        const int first = cu_new[i];
        const int count = cu_new[i + 1] - first;
#pragma omp parallel for collapse(2) schedule(static) reduction(| : bad)
        for (int h = 0; h < H; ++h) {
            for (int t = 0; t < count; ++t) {
                const int pos = start[i] + t;
                const int page = table[(int64_t)slot_row * table_stride + pos / page_size];
                if (page < 0 || page >= num_pages) { bad |= 1; continue; }
                const int64_t dst = (int64_t)h * pool_head_stride + (int64_t)page * pool_page_stride +
                                    (int64_t)(pos % page_size) * row_bytes;
                const int64_t src = (int64_t)(first + t) * new_tok_stride + (int64_t)h * new_head_stride;
                memcpy(k_pool + dst, k_new + src, (size_t)row_bytes);
                memcpy(v_pool + dst, v_new + src, (size_t)row_bytes);
            }
        }
    }
    return bad ? -1 : 0;
}

/*
 * Block-table gather.  Sequence i (slot slots[i], length lens[i]) is written
 * to out rows cu_out[i] .. cu_out[i]+lens[i]-1; row of token r, head h is at
 * r * out_tok_stride + h * out_head_stride (bytes).
 */
int barqkv_ref_gather_paged(const uint8_t* k_pool, const uint8_t* v_pool,
                            int64_t pool_head_stride, int64_t pool_page_stride, int num_pages,
                            const int32_t* table, int table_stride,
                            const int32_t* slots, const int32_t* lens, const int32_t* cu_out, int n,
                            uint8_t* k_out, uint8_t* v_out,
                            int64_t out_tok_stride, int64_t out_head_stride,
                            int H, int page_size, int64_t row_bytes) {
    int bad = 0;
    for (int i = 0; i < n; ++i) {
        const int slot_row = slots ? slots[i] : i;
        const int len = lens[i];
        const int pages = (len + page_size - 1) / page_size;
#pragma omp parallel for collapse(2) schedule(static) reduction(| : bad)
        for (int h = 0; h < H; ++h) {
            for (int j = 0; j < pages; ++j) {
                const int page = table[(int64_t)slot_row * table_stride + j];
                if (page < 0 || page >= num_pages) { bad |= 1; continue; }
                const int rows = (len - j * page_size) < page_size ? (len - j * page_size) : page_size;
                const int64_t src = (int64_t)h * pool_head_stride + (int64_t)page * pool_page_stride;
                for (int s = 0; s < rows; ++s) {
                    const int64_t dst = (int64_t)(cu_out[i] + j * page_size + s) * out_tok_stride +
                                        (int64_t)h * out_head_stride;
                    memcpy(k_out + dst, k_pool + src + (int64_t)s * row_bytes, (size_t)row_bytes);
                    memcpy(v_out + dst, v_pool + src + (int64_t)s * row_bytes, (size_t)row_bytes);
                }
            }
        }
    }
    return bad ? -1 : 0;
}
