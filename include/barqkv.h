/*
 * barqkv - paged KV-cache append and gather for NVIDIA B200 (sm_100a).
 *
 * C ABI of libbarqkv.so.  Every entry point takes raw device pointers, plain
 * integers and a CUDA stream; nothing here allocates device memory or
 * synchronises with the device (barqkv_max_length, whose job is a blocking read
 * of the lengths, is the one exception), the only lock is the one that guards
 * the second stream of barqkv_update_layers, and the library keeps no mutable
 * process-wide settings.  All functions return 0 on success
 * or a negative BARQKV_E_* code; barqkv_last_error() then holds a message for
 * the calling thread.  Work is enqueued on the given stream and runs
 * asynchronously; device-side guards (bad block-table entry, capacity) never
 * trap: they skip the access and OR a BARQKV_S_* bit into the caller's
 * optional status word.
 *
 * The reference interfaces these replace are cited per function as
 * <file in the BarqTrain tree>:<lines>.
 */
#ifndef BARQKV_H
#define BARQKV_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BARQKV_VERSION 106 /* major*100 + minor */

/* host-side return codes */
#define BARQKV_OK 0
#define BARQKV_E_INVALID (-1) /* bad argument (null pointer, size, alignment) */
#define BARQKV_E_LAUNCH (-2)  /* the CUDA runtime refused the launch */
#define BARQKV_E_LIMIT (-3)   /* a size is beyond a documented maximum, or the page pool is exhausted */
#define BARQKV_E_CAPACITY (-4) /* a sequence would pass max_blocks * page_size tokens (the reference's ValueError, kv_cache.py:80-83) */

/* bits a kernel may OR into *status (device int32, optional) */
#define BARQKV_S_BAD_PAGE 1   /* block-table entry outside [0, num_pages): row skipped */
#define BARQKV_S_CAPACITY 2   /* reference-layout append would pass the cache capacity: nothing written; decode attention: the
                                 lengths add up to more than the total_len the call was given, some pages were not attended */
#define BARQKV_S_TIMEOUT 4    /* a bounded wait on a bulk copy gave up: remaining pages skipped */
#define BARQKV_S_BAD_SLOT 8   /* sequence slot outside the block table: sequence skipped */

/* gather implementations (argument `mode`) */
#define BARQKV_MODE_AUTO 0
#define BARQKV_MODE_VECTOR 1  /* 16-byte ld/st through registers */
#define BARQKV_MODE_BULK 2    /* cp.async.bulk global->shared->global, mbarrier pipelined */

/*
 * BARQKV_FLAG_DESC_STABLE (argument `flags` of the appends; OR-ed into `mode` of barqkv_gather and
 * barqkv_update): the caller vouches that everything the call reads BESIDES the K/V payload - the block
 * table, slots, seq_start / seq_lens, cu_new, cu_out - was completely written before the kernel that
 * precedes this call in `stream` was enqueued, and stays unchanged until this call's kernel has run.
 * True for the second and later layers of a step whose description was uploaded once before the first
 * layer.  The kernel is then launched as a programmatic dependent of its predecessor: its prologue
 * (page counts, first page hand-out, first block-table look-ups) overlaps the predecessor's tail and only
 * its first copy waits for the predecessor to finish.  Consecutive flagged calls that pass `work` must
 * alternate between two work buffers, because the later kernel starts taking pages while the earlier one
 * may still be handing out its last.  Results are the same with and without the flag.
 */
#define BARQKV_FLAG_DESC_STABLE 0x100
/* barqkv_update_layers only: keep every layer on the caller's stream, each launch behind the one before
 * (no second stream).  For callers whose stream has a priority or a capture the second stream should not
 * take part in, and for measuring what the overlap of neighbouring layers is worth. */
#define BARQKV_FLAG_ONE_STREAM 0x200

typedef void* barqkv_stream_t; /* a cudaStream_t */

/*
 * One layer's page pools.  The K pool and the V pool share this geometry.
 * Page p of head h starts at element h*head_stride + p*page_stride and holds
 * page_size rows of head_dim elements, contiguous (row r at +r*head_dim).
 *   [H, P, ps, D] pool:               head_stride = P*ps*D, page_stride = ps*D
 *   reference [B, H, max_blocks, ps, D] (python/barqtrain/kv_cache.py:66-70):
 *     head_stride = max_blocks*ps*D, page_stride = ps*D,
 *     page of (b, j) = b*H*max_blocks + j   (see implicit_pages_per_slot)
 */
typedef struct barqkv_pool_layout {
    int32_t num_heads;   /* KV heads held by this GPU */
    int32_t head_dim;
    int32_t page_size;   /* tokens per page */
    int32_t elem_bytes;  /* 1, 2, 4 or 8; payload is copied bit for bit */
    int32_t num_pages;   /* valid physical page ids are [0, num_pages) */
    int32_t reserved;
    int64_t head_stride; /* elements */
    int64_t page_stride; /* elements */
} barqkv_pool_layout;

/*
 * Which pages a batch entry's sequence owns.  Entry i uses row
 * slots[i] (i when slots is NULL) of the table; logical page j of that row is
 * physical page table[row*table_stride + j].  With table == NULL the page is
 * row*implicit_pages_per_slot + j (the reference's arithmetic paging,
 * python/barqtrain/kv_cache.py:84-87) and table_stride bounds j.
 */
typedef struct barqkv_block_table {
    const int32_t* table; /* device, int32 [table_rows, table_stride] or NULL */
    const int32_t* slots; /* device, int32 [n] or NULL */
    int32_t table_rows;
    int32_t table_stride;
    int32_t implicit_pages_per_slot;
    int32_t reserved;
} barqkv_block_table;

/*
 * Addressing of per-token rows outside the pool (new K/V rows for append,
 * gathered rows for gather).  Row (entry i, token t of that entry, head h)
 * starts at element  i*seq_stride + (base_i + t)*tok_stride + h*head_stride,
 * base_i = cu[i] when `packed` is non-zero, else 0.  head_dim elements
 * contiguous.
 *   packed [N_tok, H, D]:  seq_stride 0,      tok_stride H*D, head_stride D,   packed 1
 *   packed [H, N_tok, D]:  seq_stride 0,      tok_stride D,   head_stride N*D, packed 1
 *   batched [B, H, T, D]:  seq_stride H*T*D,  tok_stride D,   head_stride T*D, packed 0
 *   view of [B, T, H, D]:  seq_stride T*H*D,  tok_stride H*D, head_stride D,   packed 0
 */
typedef struct barqkv_rows_layout {
    int64_t seq_stride;  /* elements */
    int64_t tok_stride;  /* elements */
    int64_t head_stride; /* elements */
    int32_t packed;
    int32_t reserved;
} barqkv_rows_layout;

int barqkv_version(void);
const char* barqkv_last_error(void);

/* Number of SMs of the current device (cached); used by callers that size work. */
int barqkv_sm_count(void);

/* Kernels this library has enqueued so far in this process (every entry point counts its launches). */
int64_t barqkv_launch_count(void);

/*
 * Append new K/V rows through the block table.
 * Replaces: the scatter of paged_kv_append_kernel
 *           (csrc/kernels/paged_kv_cache.cu:15-54) and the CPU loop
 *           _python_append (python/barqtrain/kv_cache.py:75-91), generalised
 *           from "block j of sequence b" to "page table[b][j]" and from one
 *           T for all sequences to a ragged batch.
 * Entry i appends cu_new[i+1]-cu_new[i] tokens (tokens_per_entry each when
 * cu_new is NULL) to its sequence, the first one landing at position
 * seq_start[i].  total_tokens = cu_new[n] (n*tokens_per_entry), known to the
 * host.  Pages must already be in the table; lengths are kept by the caller.
 * work: device int32[2] scratch, zero before its first use, or NULL (same rules
 * as for barqkv_gather: the kernel leaves it zero, launches that may overlap
 * must not share it).  With it, appends that bring at least a page of tokens
 * per entry on average (prefill chunks) move whole pages with the copy engine
 * - one tiled TMA load of a [page_size][1 head][head_dim] box of the new rows
 * (token-major sources) or one bulk copy (head-major sources) and one bulk
 * store per page, head and K/V - when rows and strides are 16-byte aligned and
 * the new rows are packed.  Everything else (decode, unaligned rows, NULL)
 * takes the 16-byte-vector row kernel; results are identical.
 * flags: 0 or BARQKV_FLAG_DESC_STABLE.
 */
int barqkv_append(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                  const barqkv_block_table* table,
                  const int32_t* seq_start, const int32_t* cu_new,
                  int32_t n, int32_t tokens_per_entry, int32_t total_tokens,
                  const void* k_new, const void* v_new, const barqkv_rows_layout* new_rows,
                  int32_t* status, int32_t* work, int32_t flags, barqkv_stream_t stream);

/*
 * barqkv_append for `layers` layers from one call, one launch per layer: layer l uses the pools at
 * k_pool/v_pool + l*pool_layer_stride elements and the new rows at k_new[l] / v_new[l] (host arrays of
 * `layers` device pointers; every layer's rows share `new_rows`); the block table, positions and counts are
 * shared.  Equals `layers` calls of barqkv_append - what the reference does with one paged_kv_append_ per
 * BarqPagedKVCacheLayer (python/barqtrain/kv_cache.py:207-219) - without their host cost between launches: from
 * the second on every launch is a programmatic dependent of the one before, and for page-sized appends the
 * launches alternate between the two counter pairs of `work`, clear each other's, and only the last counts its
 * finished blocks to clear its own.  work: device int32[4], zero before its first use and again when the
 * call's kernels have run, or NULL.  flags: 0 or BARQKV_FLAG_DESC_STABLE for the first layer's launch.  For
 * callers that hold a step's rows of every layer in separate buffers (a chunk of a transferred or restored
 * cache, a prefill whose rows were kept per layer); with one buffer for all layers barqkv_append_layers
 * needs a single launch.
 */
int barqkv_append_each_layer(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                             int32_t layers, int64_t pool_layer_stride,
                             const barqkv_block_table* table,
                             const int32_t* seq_start, const int32_t* cu_new,
                             int32_t n, int32_t tokens_per_entry, int32_t total_tokens,
                             const void* const* k_new, const void* const* v_new, const barqkv_rows_layout* new_rows,
                             int32_t* status, int32_t* work, int32_t flags, barqkv_stream_t stream);

/*
 * barqkv_append for `layers` layers in ONE launch: layer l uses the pools at
 * k_pool/v_pool + l*pool_layer_stride elements and the new rows at k_new/v_new +
 * l*new_layer_stride elements; the block table, positions and counts are shared (every layer
 * of a model appends the same tokens).  Replaces `layers` calls of the reference's
 * paged_kv_append_ (one per BarqPagedKVCacheLayer, python/barqtrain/kv_cache.py:207-219) when a
 * step's rows for all layers are at hand - a decode step is then one launch of 16 MiB instead of
 * 32 launches of 512 KiB.
 */
int barqkv_append_layers(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                         int32_t layers, int64_t pool_layer_stride,
                         const barqkv_block_table* table,
                         const int32_t* seq_start, const int32_t* cu_new,
                         int32_t n, int32_t tokens_per_entry, int32_t total_tokens,
                         const void* k_new, const void* v_new, const barqkv_rows_layout* new_rows,
                         int64_t new_layer_stride, int32_t* status, int32_t* work, int32_t flags,
                         barqkv_stream_t stream);

/*
 * Largest of seq_lens[0..n) (device int32), read back on `stream`: copies the n values to the host,
 * waits for `stream` and returns the maximum in *max_out.  Replaces the launcher's capacity read
 * `seq_lens_int.narrow(0, 0, batch_size).max().item<int32_t>()` (csrc/kernels/paged_kv_cache.cu:93),
 * which costs a slice, a reduction kernel and a blocking read; callers that mirror the lengths on the
 * host do not need it at all.
 */
int barqkv_max_length(const int32_t* seq_lens, int32_t n, int32_t* max_out, barqkv_stream_t stream);

/*
 * Host-side plumbing of the block table (no counterpart in the reference, which has no table):
 * barqkv_upload is cudaMemcpyAsync host->device on `stream` (src should be pinned memory that stays
 * untouched until the copy has run); barqkv_table_scatter writes n changed entries into the device
 * table, pairs[2i] = flat index row*table_stride + column, pairs[2i+1] = page id (device int32[2n]).
 * A step's description and its table changes travel in one upload, however large the table is.
 */
int barqkv_upload(void* dst_device, const void* src_host, int64_t bytes, barqkv_stream_t stream);
int barqkv_table_scatter(int32_t* table, int64_t table_words, const int32_t* pairs, int32_t n, barqkv_stream_t stream);

/*
 * Copy whole pages inside the pools: page src_pages[i] -> dst_pages[i] for every head, K and V, and
 * `layers` layers (pool_layer_stride elements apart).
 * Replaces: the physical row copies of batch_repeat_interleave / batch_select_indices
 *           (python/barqtrain/kv_cache.py:166-186).  With a block table a forked sequence shares its
 *           full pages with its parent and only the partial last page, which both will write, is
 *           duplicated.
 */
int barqkv_copy_pages(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                      int32_t layers, int64_t pool_layer_stride,
                      const int32_t* src_pages, const int32_t* dst_pages, int32_t n,
                      int32_t* status, barqkv_stream_t stream);

/*
 * barqkv_append with rotary position embedding applied to the K rows on the way into the pages:
 *   k_out = k * cos + rotate_half(k) * sin      (halves convention: rotate_half(x) = [-x2, x1])
 * the formula of the reference's helper apply_rope_to_qk (python/barqtrain/ops.py:376-428) and of
 * Hugging Face models, with cos / sin given per new token: [total_tokens, head_dim] in the pool's element
 * type (dtype), rope_tok_stride elements apart, row r for packed new token r.  Products and sum are
 * rounded to the element type one at a time, so the stored rows equal "rotate, then append" bit for bit;
 * V rows are copied unchanged.  Saves the separate read and write of the new K rows.
 * Needs 16-byte aligned rows, strides and pointers and head_dim a multiple of 16 (2-byte) / 8 (4-byte).
 */
#define BARQKV_DTYPE_BF16 0
#define BARQKV_DTYPE_F16 1
#define BARQKV_DTYPE_F32 2
int barqkv_append_rope(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                       const barqkv_block_table* table,
                       const int32_t* seq_start, const int32_t* cu_new,
                       int32_t n, int32_t tokens_per_entry, int32_t total_tokens,
                       const void* k_new, const void* v_new, const barqkv_rows_layout* new_rows,
                       const void* cos, const void* sin, int64_t rope_tok_stride, int32_t dtype,
                       int32_t* status, barqkv_stream_t stream);

/*
 * The reference's native entry point, same semantics:
 *   void paged_kv_append_(key_cache, value_cache, seq_lens, key_states, value_states)
 *   csrc/src/bindings.cpp:43-49,74-75 -> paged_kv_append_cuda
 *   (csrc/kernels/paged_kv_cache.cu:58-128).
 * key_cache/value_cache: [max_batch, heads, max_blocks, page_size, head_dim]
 * contiguous; seq_lens: int32 [>= batch]; new rows [batch, heads, tokens,
 * head_dim] addressed by new_rows (packed must be 0), so a transposed view
 * needs no copy.  Writes rows at positions seq_lens[b] .. +tokens-1 and then
 * adds `tokens` to seq_lens[0..batch) in the same launch.  If any sequence
 * would pass max_blocks*page_size nothing is written, seq_lens stay, and
 * BARQKV_S_CAPACITY is set (the reference checks the same bound on the host
 * after a device sync, paged_kv_cache.cu:92-99).
 * ticket: device int32 scratch word, zero before its first use; the kernel
 * leaves it zero.  Concurrent launches must not share a ticket.
 */
int barqkv_append_legacy(void* key_cache, void* value_cache, int32_t* seq_lens,
                         const void* k_new, const void* v_new, const barqkv_rows_layout* new_rows,
                         int32_t batch, int32_t max_batch, int32_t heads, int32_t tokens,
                         int32_t head_dim, int32_t max_blocks, int32_t page_size, int32_t elem_bytes,
                         int32_t* ticket, int32_t* status, barqkv_stream_t stream);

/*
 * Gather sequences' pages into contiguous rows.
 * Replaces: _flatten_pages + current_tensors (python/barqtrain/kv_cache.py:
 *           120-133), which can be a zero-copy view only because the
 *           reference's pages of one sequence are adjacent; with a block
 *           table the pages are scattered and this copy materialises them.
 * Entry i (length seq_lens[i]) is written to rows addressed by out_rows with
 * base_i = cu_out[i] (packed) - e.g. [sum_len, H, D] or [H, sum_len, D] - or
 * into a padded [n, H, max_len, D] batch (packed 0).  Rows at and beyond a
 * sequence's length are not touched.  total_tokens_hint: an upper bound of
 * sum(seq_lens) used only to size the grid (0 = unknown).
 * work: device int32[2] scratch, zero before its first use, or NULL.  With it
 * the bulk gather hands pages to its persistent CTAs through an atomic counter
 * (SMs differ in how fast they reach memory; equal static shares leave the
 * fast ones idle at the end).  The kernel leaves both words zero.  Launches
 * that may overlap on the device must not share a work buffer.  NULL selects
 * equal static shares.
 */
int barqkv_gather(const barqkv_pool_layout* pool, const void* k_pool, const void* v_pool,
                  const barqkv_block_table* table,
                  const int32_t* seq_lens, const int32_t* cu_out, int32_t n,
                  int64_t total_tokens_hint,
                  void* k_out, void* v_out, const barqkv_rows_layout* out_rows,
                  int32_t mode, int32_t* status, int32_t* work, barqkv_stream_t stream);

/*
 * Append and gather in one call - what the reference's layer does per attention call:
 *   update(key_states, value_states) = append(...) then current_tensors()
 *   (python/barqtrain/kv_cache.py:135-142).
 * Arguments are those of barqkv_append (seq_start = lengths BEFORE the append, cu_new /
 * tokens_per_entry, new rows) followed by those of barqkv_gather, where cu_out and
 * total_tokens_hint refer to the lengths AFTER the append, and seq_lens_after holds those
 * lengths (device int32[n]).  On return (stream order) the pool holds the new rows and the
 * output holds every sequence including them.
 * When the bulk gather applies (16-byte aligned rows and strides, pages <= 16 KiB, mode not
 * VECTOR) and the call brings at most page_size new tokens per entry on average (decode,
 * short chunks), ONE kernel does both: the new rows are read once, joined with the page's
 * old rows in shared memory, and stored to the output and to their page slots.  Otherwise
 * the append kernel and the gather kernel run back to back; results are identical.
 */
int barqkv_update(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                  const barqkv_block_table* table,
                  const int32_t* seq_start, const int32_t* cu_new,
                  int32_t n, int32_t tokens_per_entry, int32_t total_new_tokens,
                  const void* k_new, const void* v_new, const barqkv_rows_layout* new_rows,
                  const int32_t* cu_out, int64_t total_tokens_hint,
                  void* k_out, void* v_out, const barqkv_rows_layout* out_rows,
                  int32_t mode, int32_t* status, int32_t* work, const int32_t* seq_lens_after,
                  barqkv_stream_t stream);

/*
 * barqkv_update for `layers` layers, one launch per layer, issued by one call: layer l uses the pools
 * at k_pool / v_pool + l * pool_layer_stride, the new rows at k_new / v_new + l * new_layer_stride
 * (strides in elements) and writes its gathered rows to k_out[l % num_out] / v_out[l % num_out] (host
 * arrays of device pointers: two pairs let consecutive layers alternate buffers).  The batch
 * description (seq_start, cu_new, cu_out, seq_lens_after) and the block table are shared by all
 * layers and must not change while the launches run.
 * Replaces `layers` calls of the reference layer's update() (python/barqtrain/kv_cache.py:135-142), each
 * of which costs two kernel launches and two device synchronisations there
 * (csrc/kernels/paged_kv_cache.cu:93,104-127, kv_cache.py:150-153).  Here the host pays one call, and
 * the launches are chained as programmatic dependents: because a layer reads the same, unchanged
 * description as the one before, its prologue (page counts, first hand-out, first block-table look-ups)
 * runs while the earlier layer's last copies drain, and only its first copy waits for that layer to finish.
 * Layers next to one another are independent when they write to different outputs (each touches its own
 * layer's pools only).  With an even num_out (or num_out >= layers) and pairwise distinct, non-overlapping
 * outputs, even layers are therefore issued on `stream` and odd layers on a second, library-owned stream
 * that is forked from `stream` at the start of the call and joined back to it before the call returns
 * (events only; also inside a stream capture): layer l is ordered behind layer l - 2, the layer whose
 * output it overwrites, and runs beside layer l - 1.  Work issued to `stream` after the call is ordered
 * behind every layer.  Other calls, and calls whose `mode` carries BARQKV_FLAG_ONE_STREAM, keep all layers on
 * `stream`, each behind the one before.
 * With total_new_tokens == 0 (k_new, v_new and new_rows may then be NULL; seq_start holds the lengths) the call
 * is barqkv_gather for every layer, chained the same way.
 * work: device int32[8] scratch, zero before its first use (four counter pairs, so that launches that can be
 * on the device together never share one); zero again when the call's last kernels have run (inside the call
 * a launch clears the pair of its neighbours in its stream's chain, only the last launch of a chain its own).  For callers that have every layer's
 * new rows at hand (a recorded decode step, cache import); results equal `layers` calls of barqkv_update.
 */
int barqkv_update_layers(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                         int32_t layers, int64_t pool_layer_stride,
                         const barqkv_block_table* table,
                         const int32_t* seq_start, const int32_t* cu_new,
                         int32_t n, int32_t tokens_per_entry, int32_t total_new_tokens,
                         const void* k_new, const void* v_new, const barqkv_rows_layout* new_rows,
                         int64_t new_layer_stride,
                         const int32_t* cu_out, int64_t total_tokens_hint,
                         void* const* k_out, void* const* v_out, int32_t num_out,
                         const barqkv_rows_layout* out_rows,
                         int32_t mode, int32_t* status, int32_t* work, const int32_t* seq_lens_after,
                         barqkv_stream_t stream);

/*
 * Self-test of the bounded waits (no counterpart in the reference, which has no device-side waits).
 * Runs the bulk gather on the given small batch with ONE CTA whose ring stages each expect 16 bytes
 * more than their copies bring, so the first wait can never be satisfied, and with every wait bounded
 * by wait_cycles clock cycles (1 .. 2e9) instead of the default ~1 s.  The kernel must give up, let the
 * copies it had already issued land, OR BARQKV_S_TIMEOUT into *status (required) and return; the
 * context stays usable and nothing spins beyond the bound.  The output is left partly written.
 */
int barqkv_gather_wait_selftest(const barqkv_pool_layout* pool, const void* k_pool, const void* v_pool,
                                const barqkv_block_table* table,
                                const int32_t* seq_lens, const int32_t* cu_out, int32_t n,
                                void* k_out, void* v_out, const barqkv_rows_layout* out_rows,
                                int64_t wait_cycles, int32_t* status, barqkv_stream_t stream);

/*
 * barqkv_gather for several layers in one launch: layer l reads the pools at k_pool / v_pool +
 * l * pool_layer_stride and writes its outputs at k_out / v_out + l * out_layer_stride (strides in
 * elements); everything else as in barqkv_gather, bulk path only (16-byte aligned rows and strides),
 * `work` and total_tokens (the sum of the lengths, or an upper bound) required.  The fixed cost of a launch
 * is paid once instead of once per layer, which matters when a GPU holds one KV head.
 * No counterpart in the reference (its gather is a view per layer, kv_cache.py:129-133).
 */
int barqkv_gather_layers(const barqkv_pool_layout* pool, const void* k_pool, const void* v_pool,
                         int32_t layers, int64_t pool_layer_stride, const barqkv_block_table* table,
                         const int32_t* seq_lens, const int32_t* cu_out, int32_t n, int64_t total_tokens,
                         void* k_out, void* v_out, const barqkv_rows_layout* out_rows, int64_t out_layer_stride,
                         int32_t* status, int32_t* work, barqkv_stream_t stream);

/*
 * Decode attention straight from the pages: one query token per sequence attends over the sequence's
 * K/V through the block table, so the gather's copy is not needed for decode.
 * No counterpart in the reference (its attention kernel, csrc/kernels/flash_attention.cu, reads
 * contiguous K/V; the reference roadmap lists "attention over pages" as future work).  The numerical
 * reference is softmax(q k^T * scale) v in fp32 over the gathered sequence.
 * q / out: [n, num_q_heads, 128] in the pool's 2-byte type (is_bf16 selects bf16 or fp16), strides in
 * elements; query head j uses KV head j / (num_q_heads / kv_heads).  seq_lens: lengths including the
 * current token (append first).  max_len: an upper bound of the lengths known to the host; total_len:
 * the host's sum of the lengths or an upper bound of it, or 0 when it is not known (a sum smaller than the real
 * one sets BARQKV_S_CAPACITY for batches of up to 256 sequences, whose launch is sized from it).  The two fix how many splits a sequence's
 * pages are cut into (with the sum the splits are sized to fill the GPU's resident CTAs once or twice
 * when the batch is small); pass the same values to both functions.  workspace: 16-byte aligned device
 * scratch of barqkv_paged_decode_workspace_bytes(...) bytes (0 when one split suffices); its contents on
 * entry do not matter.  With more than one split the call enqueues two kernels: the attention kernel, whose
 * splits leave their partial results in the workspace, and a small one behind it (a programmatic dependent)
 * that combines them into `out`.  Calls that may overlap on the device need separate workspaces.
 * Limits: head_dim 128, page_size 16, 32 or 64, 2-byte elements, at most 8 query heads per KV head.
 */
int64_t barqkv_paged_decode_workspace_bytes(int32_t n, int32_t kv_heads, int64_t max_len, int64_t total_len,
                                            int32_t page_size);
int barqkv_paged_decode_attention(const barqkv_pool_layout* pool, const void* k_pool, const void* v_pool,
                                  const barqkv_block_table* table, const int32_t* seq_lens, int32_t n,
                                  const void* q, int64_t q_seq_stride, int64_t q_head_stride,
                                  void* out, int64_t out_seq_stride, int64_t out_head_stride,
                                  int32_t num_q_heads, float softmax_scale, int32_t is_bf16, int64_t max_len,
                                  int64_t total_len,
                                  void* workspace, int64_t workspace_bytes, int32_t* status, barqkv_stream_t stream);

/*
 * A decode layer in one call: barqkv_append of the step's token (one new K/V row per sequence and KV
 * head) fused into barqkv_paged_decode_attention (the same kernels, the same count).  What the reference does per layer and step - append
 * (csrc/kernels/paged_kv_cache.cu:58-128), current_tensors (python/barqtrain/kv_cache.py:129-133), then an
 * attention call over the returned views - with neither a separate append launch nor any gathered copy.
 * seq_lens_after: lengths INCLUDING the new token (its position is length - 1; its page must already be
 * in the table).  k_new / v_new: [n, kv_heads, 128] rows addressed by new_seq_stride / new_head_stride
 * (elements), 16-byte aligned.  The CTA that owns a sequence's last page attends the new row from the
 * caller's buffer and stores it into its page slot; on return (stream order) the pool holds the row, bit
 * for bit what barqkv_append would have stored, and `out` equals append-then-attend.  Other arguments
 * as for barqkv_paged_decode_attention.  flags: 0 or BARQKV_FLAG_DESC_STABLE (lengths, slots and table
 * older than the preceding kernel; q, the new rows and the workspace are never read early).
 */
int barqkv_paged_decode_update(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                               const barqkv_block_table* table, const int32_t* seq_lens_after, int32_t n,
                               const void* k_new, const void* v_new, int64_t new_seq_stride, int64_t new_head_stride,
                               const void* q, int64_t q_seq_stride, int64_t q_head_stride,
                               void* out, int64_t out_seq_stride, int64_t out_head_stride,
                               int32_t num_q_heads, float softmax_scale, int32_t is_bf16, int64_t max_len,
                               int64_t total_len, void* workspace, int64_t workspace_bytes, int32_t flags,
                               int32_t* status, barqkv_stream_t stream);

/*
 * barqkv_gather for callers that cannot allocate device memory.
 * No counterpart in the reference (it never needs scratch memory).
 *
 * Same arguments and results as barqkv_gather, except that the two hand-out
 * counters come from a 4 KiB array built into the library instead of a
 * caller-owned `work` buffer.  Meant for callers such as a server that has
 * already given all free device memory to its own arena, or a plugin host that
 * forbids allocation inside an operator call.  This function and everything it
 * calls make no allocation call of their own, on the host or on the device.
 * One caveat: the array is part of the library's device code, so the CUDA
 * runtime reserves its 4 KiB (with the rest of the code image) when it loads
 * the library's module on a device - at the first call of ANY function of this
 * library on that device, this one included, under CUDA's lazy loading.  A
 * caller whose arena takes all remaining memory should make one call of this
 * library before the arena is created.
 *
 * work_slot selects one of BARQKV_STATIC_WORK_SLOTS counter pairs; a value
 * outside [0, BARQKV_STATIC_WORK_SLOTS) is refused with BARQKV_E_LIMIT.  All
 * calls on a device share the array, and a slot still holds what its last
 * user left: each call first checks its arguments and then clears its slot on
 * `stream` (a refused call enqueues nothing).  Two calls that can
 * be in flight on the GPU at the same time (different streams) must use
 * different slots, or they corrupt each other's page hand-out.
 *
 * The first call on each device looks up the array's device address (with
 * that device current).  Make that first call outside any stream capture.
 */
#define BARQKV_STATIC_WORK_SLOTS 32
int barqkv_gather_noalloc(const barqkv_pool_layout* pool, const void* k_pool, const void* v_pool,
                          const barqkv_block_table* table,
                          const int32_t* seq_lens, const int32_t* cu_out, int32_t n,
                          int64_t total_tokens_hint,
                          void* k_out, void* v_out, const barqkv_rows_layout* out_rows,
                          int32_t mode, int32_t* status, int32_t work_slot, barqkv_stream_t stream);

/*
 * ---------------------------------------------------------------------------------------------
 * Host-side bookkeeping of the block-table cache: the page free list, the block table's host copy
 * and the per-step description.  Host code only; the library owns no device memory here - every
 * buffer is the caller's.
 * The reference needs none of this: it allocates every sequence's pages up front
 * (lazy_initialization, python/barqtrain/kv_cache.py:53-73), addresses them arithmetically (:84-89)
 * and can only release a whole layer (reset, :188-194).  These calls are what "allocation" and
 * "sequence release" become with a shared page pool, kept native because at 256 live sequences the
 * interpreted version of barqkv_host_begin costs more than the step's kernels.
 * Not thread-safe: one thread drives one table.
 * ---------------------------------------------------------------------------------------------
 */
typedef struct barqkv_host_table barqkv_host_table;

/*
 * free_order: the initial free list (a permutation of 0..num_pages-1; NULL = ascending); pages are
 * handed out from its front, released pages queue at its back.  table_host: pinned int32
 * [max_seqs, max_blocks], the authoritative block table, filled with -1 by the caller; lengths /
 * page_count: int64 [max_seqs] each, zero-filled by the caller, tokens held and pages owned per
 * slot.  The caller keeps all three alive, may read them at any time, and writes `lengths` itself
 * when an append has been issued (the library only reads it, except that release zeroes a slot).
 * Returns NULL on bad arguments (barqkv_last_error() says why).
 */
barqkv_host_table* barqkv_host_create(int32_t num_pages, const int32_t* free_order, int32_t max_seqs,
                                      int32_t max_blocks, int32_t page_size, int32_t* table_host,
                                      int64_t* lengths, int64_t* page_count);
void barqkv_host_destroy(barqkv_host_table* table);

/*
 * The free list.  take: `count` pages from the front (BARQKV_E_LIMIT when fewer are free; nothing
 * changes then).  share: one more holder for pages already held (a forked sequence shares its parent's
 * full pages).  give_back: one holder fewer per listed page; pages nobody holds any more join the back
 * of the list in the order first listed; the whole list is checked before anything changes
 * (BARQKV_E_INVALID: a page released that is not held, or more often than it is held).
 * stats: out = {free, resident, peak resident, take calls, give_back calls, num_pages}.
 * free_list: copies up to `capacity` ids, front first; returns the number of free pages.
 */
int barqkv_host_take(barqkv_host_table* table, int32_t count, int32_t* out_pages);
int barqkv_host_share(barqkv_host_table* table, const int32_t* pages, int32_t n);
int barqkv_host_give_back(barqkv_host_table* table, const int32_t* pages, int32_t n);
int32_t barqkv_host_holders(const barqkv_host_table* table, int32_t page);
int barqkv_host_stats(const barqkv_host_table* table, int64_t out[6]);
int32_t barqkv_host_free_list(const barqkv_host_table* table, int32_t* out, int32_t capacity);

/*
 * Table rows.  reserve: make the slot own pages for new_length tokens (BARQKV_E_CAPACITY beyond
 * max_blocks * page_size, BARQKV_E_LIMIT when the pool cannot serve it).  set_pages: replace the
 * slot's page list (fork, crop, beam reordering; holder counts are the caller's business through
 * share / give_back).  release: give the slot's pages back, clear its row in the host table and zero
 * its length.  Entries changed by any of these are remembered and sent to the device copy by the next
 * barqkv_host_begin.
 */
int barqkv_host_reserve(barqkv_host_table* table, int32_t slot, int64_t new_length);
int barqkv_host_set_pages(barqkv_host_table* table, int32_t slot, const int32_t* pages, int32_t n);
int barqkv_host_release(barqkv_host_table* table, int32_t slot);
int64_t barqkv_host_pending_changes(const barqkv_host_table* table);

/*
 * Device side of the table, all caller-owned: table_dev (int32 [max_seqs, max_blocks], the copy the
 * kernels read), two step buffers of step_words int32 each (one for append descriptions, one for
 * gather descriptions) and pinned staging memory of staging_words int32, used as a ring of
 * staging_words / step_words slots (at least 2, at most 64) whose reuse is guarded by CUDA events: that
 * is how many steps the host may run ahead of the device.  May be called again with larger buffers.
 */
int barqkv_host_attach(barqkv_host_table* table, int32_t* table_dev, int32_t* step_dev_append, int32_t* step_dev_gather,
                       int64_t step_words, int32_t* staging_host, int64_t staging_words);

/*
 * One step's host work in one call.  kind 0 (append): entry i will append counts[i] tokens to
 * slots[i]; pages for them are reserved (all or nothing: BARQKV_E_CAPACITY / BARQKV_E_LIMIT leave
 * everything as it was).  kind 1 (gather): the entries' current lengths.  Then every block-table
 * entry changed since the last call and the description are written into a staging slot, sent with
 * ONE cudaMemcpyAsync on `stream`, and the changed entries are applied to table_dev by a small
 * kernel.  The description sits at the start of the kind's step buffer - an address that never
 * changes, so a recorded CUDA graph can keep reading it - and the changed entries follow it.
 * layout 0: the description is [slots n | first n | cu n+1] (first = start position for an append,
 * length for a gather; cu = packed row offsets).  layout 1 (a decode step, one token per entry, kind
 * 0): [slots n | start n | cu_new n+1 | lengths_after n | cu_out n+1], everything a fused append +
 * gather of the step needs.  More changed entries than a staging slot holds (after bulk edits) go in
 * several uploads.
 * info: {total tokens, largest first, device address of the description, changed entries sent, host
 * address of the description (readable until the staging ring comes round), pages taken, copies +
 * kernels enqueued, words sent}.  When not even the description fits the attached buffers the call
 * fails with BARQKV_E_LIMIT and info[7] holds the words needed.
 */
int barqkv_host_begin(barqkv_host_table* table, int32_t kind, const int32_t* slots, const int32_t* counts, int32_t n,
                      int32_t layout, barqkv_stream_t stream, int64_t info[8]);

#ifdef __cplusplus
}
#endif
#endif /* BARQKV_H */
