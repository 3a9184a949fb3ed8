// Host-side bookkeeping of the block-table cache (included at the end of barqkv.cu; same translation unit).
//
// The reference sizes every sequence's pages up front (one torch.zeros of the whole capacity,
// python/barqtrain/kv_cache.py:53-73) and never recycles them (reset() zeroes everything, :188-194), so
// its per-step host work is a length read.  With a shared page pool every step has host work: pages
// for the tokens about to be appended, block-table entries for them, and the step's description
// (slots, start positions / lengths, packed offsets) on its way to the device.  Done in an interpreted
// language that work (about 0.2 ms for 256 sequences) is longer than the step's kernels, so it lives here:
// plain C++, no device memory of its own.  The caller owns every buffer - the pinned host copy of the block
// table, the length and page-count arrays, the pinned staging memory and the device buffers the uploads
// land in.
//
//   barqkv_host_*          free list (a ring of page ids) with a holder count per page, table rows,
//                          sequence release
//   barqkv_host_begin      one step: reserve pages for the new tokens, collect the table entries that
//                          changed since the last step, write the description and those entries into
//                          a pinned staging slot, ONE cudaMemcpyAsync for both, then the scatter kernel
//                          that applies the changed entries to the device table

namespace {

constexpr int kHostRing = 64;          // most staging slots in flight (the caller's staging memory decides how many)

struct HostTable {
    int num_pages = 0, max_seqs = 0, max_blocks = 0, page_size = 0;
    // free list: a page is either free or held, so a ring of num_pages entries holds every possible list
    std::vector<int32_t> ring;
    int head = 0;
    int pages_free = 0;
    std::vector<int32_t> refs;         // sequences holding each page (forks share full pages)
    std::vector<int32_t> mark;         // scratch: times a page is listed in the call being checked
    long long resident = 0, peak = 0, alloc_calls = 0, release_calls = 0;
    // caller-owned host arrays
    int32_t* table = nullptr;          // [max_seqs][max_blocks], pinned; authoritative copy of the block table
    int64_t* lengths = nullptr;        // [max_seqs] tokens held
    int64_t* page_count = nullptr;     // [max_seqs] pages owned
    // entries of `table` the device copy does not have yet: (flat index, page id), oldest first
    std::vector<std::pair<int32_t, int32_t>> changes;
    // device side, registered by barqkv_host_attach
    int32_t* table_dev = nullptr;
    int32_t* step_dev[2] = {nullptr, nullptr};     // per kind (0 append, 1 gather): [pairs | slots | first | cu]
    long long step_words = 0;
    int32_t* staging = nullptr;        // pinned, ring_slots slots of slot_words int32 each
    long long slot_words = 0;
    int ring_slots = 0;
    int pos = 0;
    cudaEvent_t done[kHostRing] = {};
    bool pending[kHostRing] = {};
    bool attached = false;
};

int host_take(HostTable* h, int count, int32_t* out) {
    if (count < 0) return fail(BARQKV_E_INVALID, "take: negative page count");
    if (count > h->pages_free) {
        snprintf(g_err, sizeof(g_err), "need %d pages, %d free of %d", count, h->pages_free, h->num_pages);
        return BARQKV_E_LIMIT;
    }
    int at = h->head;
    for (int i = 0; i < count; ++i) {
        const int32_t p = h->ring[at];
        if (h->refs[p] != 0) {
            snprintf(g_err, sizeof(g_err), "page %d handed out twice", p);
            return BARQKV_E_INVALID;
        }
        if (++at == h->num_pages) at = 0;
    }
    at = h->head;
    for (int i = 0; i < count; ++i) {
        const int32_t p = h->ring[at];
        h->refs[p] = 1;
        out[i] = p;
        if (++at == h->num_pages) at = 0;
    }
    if (count) h->head = at;
    h->pages_free -= count;
    h->resident += count;
    if (h->resident > h->peak) h->peak = h->resident;
    ++h->alloc_calls;
    return 0;
}

// Drop one holder per listed page; pages nobody holds any more join the back of the free list in the
// order they were first listed.  Checked in full before anything changes.
int host_give_back(HostTable* h, const int32_t* pages, int n) {
    ++h->release_calls;
    int bad = -1;
    bool range_error = false;
    for (int i = 0; i < n; ++i) {
        const int32_t p = pages[i];
        if (p < 0 || p >= h->num_pages) { bad = p; range_error = true; break; }
        if (++h->mark[p] > h->refs[p] && bad < 0) bad = p;
    }
    if (bad >= 0 || range_error) {
        for (int i = 0; i < n; ++i)
            if (pages[i] >= 0 && pages[i] < h->num_pages) h->mark[pages[i]] = 0;
        if (range_error) snprintf(g_err, sizeof(g_err), "page %d is outside the pool", bad);
        else snprintf(g_err, sizeof(g_err), h->refs[bad] == 0 ? "page %d released but not owned" : "page %d released twice", bad);
        return BARQKV_E_INVALID;
    }
    for (int i = 0; i < n; ++i) --h->refs[pages[i]];
    int tail = h->head + h->pages_free;
    if (tail >= h->num_pages) tail -= h->num_pages;
    for (int i = 0; i < n; ++i) {
        const int32_t p = pages[i];
        if (h->mark[p] == 0) continue;           // already queued by an earlier mention
        h->mark[p] = 0;
        if (h->refs[p] == 0) {
            h->ring[tail] = p;
            if (++tail == h->num_pages) tail = 0;
            ++h->pages_free;
            --h->resident;
        }
    }
    return 0;
}

inline void host_note(HostTable* h, int slot, int col, int32_t page) {
    h->table[(long long)slot * h->max_blocks + col] = page;
    h->changes.emplace_back((int32_t)((long long)slot * h->max_blocks + col), page);
}

bool host_slot_ok(const HostTable* h, int slot) { return slot >= 0 && slot < h->max_seqs; }

}  // namespace

extern "C" {

barqkv_host_table* barqkv_host_create(int32_t num_pages, const int32_t* free_order, int32_t max_seqs,
                                      int32_t max_blocks, int32_t page_size, int32_t* table_host,
                                      int64_t* lengths, int64_t* page_count) {
    if (num_pages <= 0 || max_seqs < 0 || max_blocks < 0 || page_size <= 0) {
        fail(BARQKV_E_INVALID, "host_create: sizes must be positive");
        return nullptr;
    }
    if ((long long)max_seqs * max_blocks > 0x7fffffffLL) {
        fail(BARQKV_E_LIMIT, "host_create: block table has more than 2^31 entries");
        return nullptr;
    }
    if (max_seqs > 0 && (!table_host || !lengths || !page_count)) {
        fail(BARQKV_E_INVALID, "host_create: a table with rows needs table_host, lengths and page_count");
        return nullptr;
    }
    HostTable* h = new (std::nothrow) HostTable();
    if (!h) {
        fail(BARQKV_E_LIMIT, "host_create: out of host memory");
        return nullptr;
    }
    h->num_pages = num_pages;
    h->max_seqs = max_seqs;
    h->max_blocks = max_blocks;
    h->page_size = page_size;
    h->ring.resize(num_pages);
    h->refs.assign(num_pages, 0);
    h->mark.assign(num_pages, 0);
    for (int i = 0; i < num_pages; ++i) {
        const int32_t p = free_order ? free_order[i] : i;
        if (p < 0 || p >= num_pages || h->mark[p]) {
            delete h;
            fail(BARQKV_E_INVALID, "free-list order must be a permutation of range(num_pages)");
            return nullptr;
        }
        h->mark[p] = 1;
        h->ring[i] = p;
    }
    std::fill(h->mark.begin(), h->mark.end(), 0);
    h->pages_free = num_pages;
    h->table = table_host;
    h->lengths = lengths;
    h->page_count = page_count;
    return reinterpret_cast<barqkv_host_table*>(h);
}

void barqkv_host_destroy(barqkv_host_table* handle) {
    HostTable* h = reinterpret_cast<HostTable*>(handle);
    if (!h) return;
    for (int i = 0; i < kHostRing; ++i)
        if (h->done[i]) cudaEventDestroy(h->done[i]);
    delete h;
}

int barqkv_host_take(barqkv_host_table* handle, int32_t count, int32_t* out_pages) {
    HostTable* h = reinterpret_cast<HostTable*>(handle);
    if (!h || (count > 0 && !out_pages)) return fail(BARQKV_E_INVALID, "host_take: null argument");
    return host_take(h, count, out_pages);
}

int barqkv_host_share(barqkv_host_table* handle, const int32_t* pages, int32_t n) {
    HostTable* h = reinterpret_cast<HostTable*>(handle);
    if (!h || n < 0 || (n && !pages)) return fail(BARQKV_E_INVALID, "host_share: bad arguments");
    for (int i = 0; i < n; ++i) {
        if (pages[i] < 0 || pages[i] >= h->num_pages || h->refs[pages[i]] == 0) {
            snprintf(g_err, sizeof(g_err), "page %d shared but not owned", pages[i]);
            return BARQKV_E_INVALID;
        }
    }
    for (int i = 0; i < n; ++i) ++h->refs[pages[i]];
    return 0;
}

int barqkv_host_give_back(barqkv_host_table* handle, const int32_t* pages, int32_t n) {
    HostTable* h = reinterpret_cast<HostTable*>(handle);
    if (!h || n < 0 || (n && !pages)) return fail(BARQKV_E_INVALID, "host_give_back: bad arguments");
    return host_give_back(h, pages, n);
}

int32_t barqkv_host_holders(const barqkv_host_table* handle, int32_t page) {
    const HostTable* h = reinterpret_cast<const HostTable*>(handle);
    if (!h || page < 0 || page >= h->num_pages) return -1;
    return h->refs[page];
}

int barqkv_host_stats(const barqkv_host_table* handle, int64_t out[6]) {
    const HostTable* h = reinterpret_cast<const HostTable*>(handle);
    if (!h || !out) return fail(BARQKV_E_INVALID, "host_stats: null argument");
    out[0] = h->pages_free;
    out[1] = h->resident;
    out[2] = h->peak;
    out[3] = h->alloc_calls;
    out[4] = h->release_calls;
    out[5] = h->num_pages;
    return 0;
}

int32_t barqkv_host_free_list(const barqkv_host_table* handle, int32_t* out, int32_t capacity) {
    const HostTable* h = reinterpret_cast<const HostTable*>(handle);
    if (!h || capacity < 0 || (capacity && !out)) return fail(BARQKV_E_INVALID, "host_free_list: bad arguments");
    int at = h->head;
    const int count = h->pages_free < capacity ? h->pages_free : capacity;
    for (int i = 0; i < count; ++i) {
        out[i] = h->ring[at];
        if (++at == h->num_pages) at = 0;
    }
    return h->pages_free;
}

int barqkv_host_release(barqkv_host_table* handle, int32_t slot) {
    HostTable* h = reinterpret_cast<HostTable*>(handle);
    if (!h || !host_slot_ok(h, slot)) return fail(BARQKV_E_INVALID, "host_release: slot outside the block table");
    int32_t* row = h->table + (long long)slot * h->max_blocks;
    const int used = (int)h->page_count[slot];
    if (int rc = host_give_back(h, row, used)) return rc;
    // Host copy only: kernels never read entries beyond a sequence's length, so the device copy may keep
    // the stale ids until a new owner of the row overwrites them.
    for (int j = 0; j < used; ++j) row[j] = -1;
    h->page_count[slot] = 0;
    h->lengths[slot] = 0;
    return 0;
}

int barqkv_host_set_pages(barqkv_host_table* handle, int32_t slot, const int32_t* pages, int32_t n) {
    HostTable* h = reinterpret_cast<HostTable*>(handle);
    if (!h || !host_slot_ok(h, slot) || n < 0 || n > h->max_blocks || (n && !pages))
        return fail(BARQKV_E_INVALID, "host_set_pages: bad arguments");
    const int old = (int)h->page_count[slot];
    for (int j = 0; j < n; ++j) host_note(h, slot, j, pages[j]);
    for (int j = n; j < old; ++j) host_note(h, slot, j, -1);
    h->page_count[slot] = n;
    return 0;
}

int barqkv_host_reserve(barqkv_host_table* handle, int32_t slot, int64_t new_length) {
    HostTable* h = reinterpret_cast<HostTable*>(handle);
    if (!h || !host_slot_ok(h, slot)) return fail(BARQKV_E_INVALID, "host_reserve: slot outside the block table");
    const long long need = (new_length + h->page_size - 1) / h->page_size;
    const int have = (int)h->page_count[slot];
    if (need <= have) return 0;
    if (need > h->max_blocks) {
        snprintf(g_err, sizeof(g_err), "paged KV cache capacity exceeded: requested %lld, max_cache_len=%lld",
                 (long long)new_length, (long long)h->max_blocks * h->page_size);
        return BARQKV_E_CAPACITY;
    }
    std::vector<int32_t> got(need - have);
    if (int rc = host_take(h, (int)(need - have), got.data())) return rc;
    for (int j = have; j < need; ++j) host_note(h, slot, j, got[j - have]);
    h->page_count[slot] = need;
    return 0;
}

int barqkv_host_attach(barqkv_host_table* handle, int32_t* table_dev, int32_t* step_dev_append, int32_t* step_dev_gather,
                       int64_t step_words, int32_t* staging_host, int64_t staging_words) {
    HostTable* h = reinterpret_cast<HostTable*>(handle);
    if (!h || !table_dev || !step_dev_append || !step_dev_gather || !staging_host || step_words <= 0 ||
        staging_words < 2 * step_words)
        return fail(BARQKV_E_INVALID, "host_attach: bad arguments (the staging memory must hold at least two steps)");
    // copies out of the old staging memory must have run before it is replaced
    for (int i = 0; i < kHostRing; ++i) {
        if (h->pending[i]) {
            const cudaError_t e = cudaEventSynchronize(h->done[i]);
            if (e != cudaSuccess) return fail_cuda("host_attach: cudaEventSynchronize", e);
            h->pending[i] = false;
        }
        if (!h->done[i]) {
            const cudaError_t e = cudaEventCreateWithFlags(&h->done[i], cudaEventDisableTiming);
            if (e != cudaSuccess) return fail_cuda("host_attach: cudaEventCreate", e);
        }
    }
    h->table_dev = table_dev;
    h->step_dev[0] = step_dev_append;
    h->step_dev[1] = step_dev_gather;
    h->step_words = step_words;
    h->staging = staging_host;
    // as many whole steps as the staging memory holds, at most kHostRing: the host may run that many steps
    // ahead of the device before a slot's earlier upload has to be waited for
    h->ring_slots = (int)(staging_words / step_words < kHostRing ? staging_words / step_words : kHostRing);
    h->slot_words = step_words;
    h->pos = 0;
    h->attached = true;
    return 0;
}

int64_t barqkv_host_pending_changes(const barqkv_host_table* handle) {
    const HostTable* h = reinterpret_cast<const HostTable*>(handle);
    return h ? (int64_t)h->changes.size() : 0;
}

int barqkv_host_begin(barqkv_host_table* handle, int32_t kind, const int32_t* slots, const int32_t* counts, int32_t n,
                      int32_t layout, barqkv_stream_t stream, int64_t info[8]) {
    HostTable* h = reinterpret_cast<HostTable*>(handle);
    if (!h || !info || n < 0 || (n && !slots) || (kind != 0 && kind != 1) || (layout != 0 && layout != 1))
        return fail(BARQKV_E_INVALID, "host_begin: bad arguments");
    if (!h->attached) return fail(BARQKV_E_INVALID, "host_begin: barqkv_host_attach has not been called");
    if (kind == 0 && n && !counts) return fail(BARQKV_E_INVALID, "host_begin: an append needs counts");
    const int ps = h->page_size;

    // 1. check everything before anything changes: slots, capacity, pool
    long long extra = 0;
    for (int i = 0; i < n; ++i) {
        if (!host_slot_ok(h, slots[i])) return fail(BARQKV_E_INVALID, "host_begin: slot outside the block table");
        if (kind == 0) {
            if (counts[i] < 0) return fail(BARQKV_E_INVALID, "host_begin: negative token count");
            const long long after = h->lengths[slots[i]] + counts[i];
            const long long need = (after + ps - 1) / ps;
            if (need > h->page_count[slots[i]]) {
                if (need > h->max_blocks) {
                    snprintf(g_err, sizeof(g_err), "paged KV cache capacity exceeded: requested %lld, max_cache_len=%lld",
                             after, (long long)h->max_blocks * ps);
                    return BARQKV_E_CAPACITY;
                }
                extra += need - h->page_count[slots[i]];
            }
        }
    }
    if (extra > h->pages_free) {
        snprintf(g_err, sizeof(g_err), "need %lld pages, %d free of %d", extra, h->pages_free, h->num_pages);
        return BARQKV_E_LIMIT;
    }
    // The description comes first, at an address that depends on nothing but the kind (a recorded CUDA graph
    // keeps reading it there step after step); the changed table entries follow it.
    // layout 0: [slots n | first n | cu n+1 | pairs 2m]
    // layout 1 (decode step, one token per entry): [slots n | start n | cu_new n+1 | after n | cu_out n+1 | pairs 2m]
    const long long desc_words = layout == 0 ? 3LL * n + 1 : 5LL * n + 2;
    const long long room = (h->slot_words < h->step_words ? h->slot_words : h->step_words) - desc_words;
    if (room < 2) {
        info[7] = desc_words + 2;
        return fail(BARQKV_E_LIMIT, "host_begin: the step does not fit the staging or device buffers; attach larger ones");
    }

    // 2. pages for the entries that cross into new ones, in entry order (a same slot listed twice
    //    sees the pages its first mention took)
    if (extra) {
        for (int i = 0; i < n; ++i) {
            const int slot = slots[i];
            const long long need = (h->lengths[slot] + counts[i] + ps - 1) / ps;
            int have = (int)h->page_count[slot];
            while (have < need) {
                int32_t page;
                if (int rc = host_take(h, 1, &page)) return rc;     // cannot happen: checked above
                --h->alloc_calls;
                host_note(h, slot, have++, page);
            }
            h->page_count[slot] = have;
        }
        ++h->alloc_calls;
    }

    // 3. changed table entries, one pair per entry: an entry written twice keeps its last value (the
    //    scatter kernel applies pairs in no particular order)
    auto& c = h->changes;
    long long m = 0;
    if (c.size() > 1) {
        std::stable_sort(c.begin(), c.end(), [](const std::pair<int32_t, int32_t>& x, const std::pair<int32_t, int32_t>& y) {
            return x.first < y.first;
        });
        for (size_t i = 0; i < c.size(); ++i) {
            if (i + 1 < c.size() && c[i + 1].first == c[i].first) continue;
            c[m++] = c[i];
        }
    } else {
        m = (long long)c.size();
    }

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t* dev = h->step_dev[kind];
    const long long table_words = (long long)h->max_seqs * h->max_blocks;
    long long total = 0, max_first = 0, uploads = 0, kernels = 0, sent_words = 0;
    int32_t* d = nullptr;
    // 4. staging slots nobody reads any more; all but the last carry table entries only (a step changes
    //    more entries than one slot holds only after bulk edits, e.g. many forks)
    for (long long at = 0;;) {
        const long long here = (m - at) * 2 <= room ? m - at : room / 2;
        const bool last = at + here == m;
        const int s_ = h->pos;
        if (h->pending[s_]) {
            const cudaError_t e = cudaEventSynchronize(h->done[s_]);
            if (e != cudaSuccess) return fail_cuda("host_begin: cudaEventSynchronize", e);
            h->pending[s_] = false;
        }
        int32_t* w = h->staging + (long long)s_ * h->slot_words;
        int32_t* pairs = w + desc_words;
        for (long long i = 0; i < here; ++i) {
            pairs[2 * i] = c[at + i].first;
            pairs[2 * i + 1] = c[at + i].second;
        }
        if (last) {
            // 5. the description
            d = w;
            if (layout == 0) {
                int32_t* d_slots = d;
                int32_t* d_first = d + n;
                int32_t* d_cu = d + 2LL * n;
                for (int i = 0; i < n; ++i) {
                    const long long len = h->lengths[slots[i]];
                    const long long cnt = kind == 0 ? counts[i] : len;
                    d_slots[i] = slots[i];
                    d_first[i] = (int32_t)len;
                    d_cu[i] = (int32_t)total;
                    total += cnt;
                    if (len > max_first) max_first = len;
                }
                d_cu[n] = (int32_t)total;
            } else {
                int32_t* d_slots = d;
                int32_t* d_start = d + n;
                int32_t* d_cu_new = d + 2LL * n;
                int32_t* d_after = d + 3LL * n + 1;
                int32_t* d_cu_out = d + 4LL * n + 1;
                d_cu_out[0] = 0;
                for (int i = 0; i < n; ++i) {
                    const long long len = h->lengths[slots[i]];
                    d_slots[i] = slots[i];
                    d_start[i] = (int32_t)len;
                    d_cu_new[i] = i;
                    d_after[i] = (int32_t)(len + 1);
                    total += len + 1;
                    d_cu_out[i + 1] = (int32_t)total;
                    if (len > max_first) max_first = len;
                }
                d_cu_new[n] = n;
            }
            if (total > 0x7fffffffLL) return fail(BARQKV_E_LIMIT, "host_begin: more than 2^31 tokens in one step");
        }
        // 6. one upload per slot, then the scatter of its entries
        const long long from = last ? 0 : desc_words;
        const long long words = desc_words + 2 * here - from;
        cudaError_t e = cudaMemcpyAsync(dev + from, w + from, (size_t)words * 4, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return fail_cuda("host_begin: upload", e);
        e = cudaEventRecord(h->done[s_], st);
        if (e != cudaSuccess) return fail_cuda("host_begin: cudaEventRecord", e);
        h->pending[s_] = true;
        h->pos = (s_ + 1) % h->ring_slots;
        ++uploads;
        sent_words += words;
        if (here) {
            table_scatter_kernel<<<(unsigned)((here + 127) / 128), 128, 0, st>>>(h->table_dev, dev + desc_words, (int)here,
                                                                              table_words);
            e = cudaGetLastError();
            if (e != cudaSuccess) return fail_cuda("host_begin: table scatter launch", e);
            g_launches.fetch_add(1, std::memory_order_relaxed);
            ++kernels;
        }
        at += here;
        if (last) break;
    }
    c.clear();
    info[0] = total;
    info[1] = max_first;
    info[2] = (int64_t)reinterpret_cast<uintptr_t>(dev);             // device address of the description
    info[3] = m;
    info[4] = (int64_t)reinterpret_cast<uintptr_t>(d);               // host address of the description (valid until the
                                                                     // staging slot comes round again)
    info[5] = extra;
    info[6] = uploads + kernels;                                     // copies + kernels enqueued
    info[7] = sent_words;
    return 0;
}

}  // extern "C"
