// barqkv: paged KV-cache append and gather kernels for NVIDIA B200 (sm_100a)
// and the C ABI declared in include/barqkv.h.
//
// The path is integer-indexed byte movement, so there is no arithmetic on the
// payload and no tensor-core use: the roofline is HBM bandwidth.  Kernels:
//
//   append_rows_kernel   new K/V rows -> page slots through the block table.
//                        A CTA takes a tile of consecutive new tokens, resolves
//                        each token's (entry, position, page) once into shared
//                        memory, then all threads stream (token, head, K|V)
//                        rows with the widest vector the alignment allows
//                        (16 B for every real configuration: a head_dim row is
//                        256 B, i.e. 16 lanes, so one warp moves the K row and
//                        the V row of a (token, head) pair per instruction).
//                        gridDim.y carries layers when several are appended at
//                        once; the LEGACY variant adds the reference layout's
//                        semantics (capacity guard, seq_lens bump by ticket).
//   gather_bulk_kernel   pages -> contiguous rows with the copy engine:
//                        cp.async.bulk global -> shared (mbarrier complete_tx)
//                        -> global (bulk_group), a ring of stages per one-warp
//                        persistent CTA, the K page and V page of one head per
//                        stage.  Token-major outputs take one tiled TMA store
//                        per full page.  Optionally the step's new rows join
//                        the stage and are also written to their page slots
//                        (append fused into the gather: barqkv_update).  No
//                        multicast, no peer memory.
//   gather_vector_kernel pages -> contiguous rows with 16-byte ld/st through
//                        registers; serves every alignment and layout.
//   copy_pages_kernel    whole-page duplicates for forked sequences.
//
// Both gathers share one work decomposition: every CTA scans the batch's page
// counts into shared memory (the batch is small: <= kMaxEntries sequences) and
// resolves block-table entries a group at a time into shared memory before the
// copies that use them are issued.  The bulk gather hands (sequence, page) tiles
// to its CTAs through an atomic counter; the vector gather splits them evenly.
//
// Device-side guards never trap and never spin without a bound.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <algorithm>
#include <atomic>
#include <mutex>
#include <initializer_list>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <new>
#include <utility>
#include <vector>

#include "barqkv.h"
#ifdef BARQKV_TUNING
#include "barqkv_experimental.h"
#endif

namespace {

constexpr int kMaxEntries = 8192;      // sequences per launch (shared-memory scan)
constexpr int kAppendThreads = 256;
constexpr int kAppendMaxTile = 64;     // new tokens resolved per CTA
constexpr int kGatherThreads = 256;
constexpr int kGroup = 32;             // (sequence, page) tiles resolved at a time
constexpr int kUnroll = 4;
constexpr int kBulkMaxStage = 32 * 1024;   // K page + V page of one head
constexpr long long kWaitCycles = 2000000000LL;  // ~1 s: bound of any mbarrier wait
constexpr long long kDrainCycles = 2000000LL;    // ~1 ms: after a give-up, per copy still on its way

thread_local char g_err[256] = "";
std::atomic<long long> g_launches{0};   // kernels enqueued by this library, process-wide

int fail(int code, const char* msg) {
    snprintf(g_err, sizeof(g_err), "%s", msg);
    return code;
}

int fail_cuda(const char* what, cudaError_t e) {
    snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
    return BARQKV_E_LAUNCH;
}

// --------------------------------------------------------------------------
// kernel arguments (byte units everywhere)
// --------------------------------------------------------------------------
struct Table {
    const int32_t* table;
    const int32_t* slots;
    int rows;
    int stride;
    int implicit;
    int num_pages;
};

struct RowsB {            // barqkv_rows_layout in bytes
    long long seq, tok, head;
    int packed;
};

struct AppendArgs {
    unsigned char* k_pool;
    unsigned char* v_pool;
    const unsigned char* k_new;
    const unsigned char* v_new;
    Table tb;
    const int32_t* seq_start;
    const int32_t* cu_new;
    int n, tokens_per_entry, total_tokens, tile;
    int heads, page_size, row_bytes;
    long long pool_head, pool_page;   // bytes
    RowsB nr;
    // several layers in one launch (gridDim.y = layers): byte strides between consecutive layers
    long long pool_layer, new_layer;
    // reference-layout extras
    int32_t* seq_lens_rw;
    int32_t* ticket;
    int capacity;
    int early;              // the batch description and the block table are older than the kernel before this one in
                            // the stream: they may be read while that kernel is still running
    int32_t* status;
};

struct GatherArgs {
    const unsigned char* k_pool;
    const unsigned char* v_pool;
    unsigned char* k_out;
    unsigned char* v_out;
    Table tb;
    const int32_t* seq_lens;
    const int32_t* cu_out;
    int n;
    int heads, page_size, row_bytes;
    long long pool_head, pool_page;
    RowsB orow;
    int stages;            // bulk kernel only
    int interleave;        // 1: CTAs take every gridDim-th group of tiles instead of one contiguous share
    int32_t* work;         // bulk kernel: [0] next group to hand out, [1] CTAs finished; null = static shares
    int32_t* zero_ahead;   // bulk kernel: another counter pair, cleared once the kernel before this one has finished
    int rearm;             // bulk kernel: the last CTA to finish clears `work` (else a later launch's zero_ahead does)
    int group_tiles;       // bulk kernel, dynamic hand-out: (sequence, page) tiles per group
    int static_permille;   // bulk kernel, dynamic hand-out: thousandths of the tiles split evenly up front
    int first_group;       // bulk kernel, dynamic hand-out: tiles of every CTA's first group (fetched before the scan)
    int layers;            // bulk kernel: the batch is gathered from this many pools, one launch (1 = the usual case)
    long long pool_layer, out_layer;   // byte strides between layers' pools and outputs
    int tensor_store;      // bulk kernel: full pages go to a row-strided output with one tiled TMA store per K/V
    int early;             // bulk kernel: the batch description and the block table are older than the kernel before
                           // this one in the stream, so they may be read before that kernel has finished
    long long wait_cycles; // bulk kernel: bound of every mbarrier wait, in clock cycles
    int extra_tx;          // bulk kernel, self-test only: bytes every stage expects beyond those its copies bring
    int32_t* status;
    // Fused append ("update", bulk kernel only; k_new == null means plain gather): seq_lens then holds
    // the lengths BEFORE the append, entry i brings cu_new[i+1]-cu_new[i] (or tokens_per_entry) new rows,
    // which are written to the output AND into their page slots of the pool.
    const unsigned char* k_new;
    const unsigned char* v_new;
    unsigned char* k_pool_w;
    unsigned char* v_pool_w;
    const int32_t* cu_new;
    int tokens_per_entry;
    RowsB nr;
};

// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may become
// resident while the kernel before it in the stream is still running.  pdl_wait_for_predecessor() blocks
// until that kernel has completed and its writes are visible; pdl_let_successor_in() allows the kernel
// after this one to become resident.  Every kernel here calls them in that order, so at most two kernels
// of a stream overlap.  Without the launch attribute both instructions do nothing.
__device__ __forceinline__ void pdl_let_successor_in() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_for_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void raise(int32_t* status, int bit) {
    if (status) atomicOr(status, bit);
}

// Physical page of logical page j of batch entry i; -1 (and a status bit) if out of range.
__device__ __forceinline__ long long resolve_page(const Table& tb, int i, int j, int32_t* status) {
    const int row = tb.slots ? tb.slots[i] : i;
    if (row < 0 || row >= tb.rows || j < 0 || j >= tb.stride) {
        raise(status, BARQKV_S_BAD_SLOT);
        return -1;
    }
    long long page;
    if (tb.table) {
        page = tb.table[(long long)row * tb.stride + j];
    } else {
        page = (long long)row * tb.implicit + j;
    }
    if (page < 0 || page >= tb.num_pages) {
        raise(status, BARQKV_S_BAD_PAGE);
        return -1;
    }
    return page;
}

// Where new token r of the call (flat index over the batch) goes and where its rows come from:
// *dst = byte offset of its slot in head 0's pool (-1 = skip), *src = byte offset of its head-0 row.
__device__ __forceinline__ void resolve_new_token(const AppendArgs& a, int r, long long* dst, long long* src) {
    int i, t;
    if (a.cu_new) {
        int lo = 0, hi = a.n - 1;             // largest i with cu_new[i] <= r
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (a.cu_new[mid] <= r) lo = mid; else hi = mid - 1;
        }
        i = lo;
        t = r - a.cu_new[i];
    } else {
        i = r / a.tokens_per_entry;
        t = r - i * a.tokens_per_entry;
    }
    const int pos = a.seq_start[i] + t;
    const int j = pos / a.page_size;
    const int slot = pos - j * a.page_size;
    const long long page = pos < 0 ? -1 : resolve_page(a.tb, i, j, a.status);
    *dst = page < 0 ? -1 : page * a.pool_page + (long long)slot * a.row_bytes;
    *src = (long long)i * a.nr.seq + (long long)(a.nr.packed ? r : t) * a.nr.tok;
}

// --------------------------------------------------------------------------
// append
// --------------------------------------------------------------------------
template <typename V, bool LEGACY>
__global__ void __launch_bounds__(kAppendThreads)
append_rows_kernel(const AppendArgs a) {
    __shared__ long long s_dst[kAppendMaxTile];   // byte offset of the token's slot in head 0's pool, -1 = skip
    __shared__ long long s_src[kAppendMaxTile];   // byte offset of the token's head-0 row in the new rows
    __shared__ int s_flag;

    const int tid = threadIdx.x;
    const int first_tok = blockIdx.x * a.tile;
    const int ntok = min(a.tile, a.total_tokens - first_tok);
    const long long layer_pool = (long long)blockIdx.y * a.pool_layer;
    const long long layer_new = (long long)blockIdx.y * a.new_layer;
    if (LEGACY || !a.early) {
        pdl_wait_for_predecessor();
        pdl_let_successor_in();
    }

    bool refuse = false;
    if (LEGACY) {
        // All-or-nothing capacity rule of the reference launcher: the longest
        // sequence plus the new tokens must fit.
        if (tid == 0) s_flag = 0;
        __syncthreads();
        int longest = 0;
        for (int i = tid; i < a.n; i += blockDim.x) longest = max(longest, a.seq_start[i]);
        if (longest + a.tokens_per_entry > a.capacity) s_flag = 1;
        __syncthreads();
        refuse = s_flag != 0;
    }

    if (tid < ntok && !refuse) resolve_new_token(a, first_tok + tid, &s_dst[tid], &s_src[tid]);
    __syncthreads();
    if (!LEGACY && a.early) {
        pdl_wait_for_predecessor();     // the look-ups above ran beside the previous kernel's tail; the rows wait for it
        pdl_let_successor_in();
    }

    if (!refuse) {
        const int vpr = a.row_bytes / (int)sizeof(V);      // vectors per row
        const int per_tok = a.heads * 2 * vpr;             // order inside a token: head, K|V, vector
        const int items = ntok * per_tok;
        for (int base = tid; base < items; base += blockDim.x * kUnroll) {
            V val[kUnroll];
            V* out[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int idx = base + u * blockDim.x;
                out[u] = nullptr;
                if (idx < items) {
                    const int t = idx / per_tok;
                    const int rem = idx - t * per_tok;
                    const int hk = rem / vpr;
                    const int vec = rem - hk * vpr;
                    const int h = hk >> 1;
                    const bool is_v = hk & 1;
                    const long long d = s_dst[t];
                    if (d >= 0) {
                        const unsigned char* src = (is_v ? a.v_new : a.k_new) + layer_new + s_src[t] + h * a.nr.head;
                        unsigned char* dst = (is_v ? a.v_pool : a.k_pool) + layer_pool + d + h * a.pool_head;
                        val[u] = __ldcs(reinterpret_cast<const V*>(src) + vec);
                        out[u] = reinterpret_cast<V*>(dst) + vec;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                if (out[u]) *out[u] = val[u];
            }
        }
    }

    if (LEGACY) {
        // The launch also advances seq_lens (the reference does it with a
        // second kernel).  Every CTA has read the lengths it needs above; the
        // last one to take a ticket performs the update and re-arms the ticket.
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            const int t = atomicAdd(a.ticket, 1);
            s_flag = (t == (int)gridDim.x - 1) ? (refuse ? 2 : 1) : 0;
        }
        __syncthreads();
        if (s_flag) {
            if (s_flag == 1) {
                for (int i = tid; i < a.n; i += blockDim.x) a.seq_lens_rw[i] += a.tokens_per_entry;
            } else if (tid == 0) {
                raise(a.status, BARQKV_S_CAPACITY);
            }
            if (tid == 0) *a.ticket = 0;
        }
    }
}

// --------------------------------------------------------------------------
// append with rotary position embedding applied to the K rows on the way in
// --------------------------------------------------------------------------
// k_out[d]        = k[d]        * cos[d]        - k[d + D/2] * sin[d]
// k_out[d + D/2]  = k[d + D/2]  * cos[d + D/2]  + k[d]       * sin[d + D/2]      (d < D/2)
// i.e. k * cos + rotate_half(k) * sin with the halves convention of the reference's helper
// (python/barqtrain/ops.py:376-428) and of Hugging Face models.  Each product and the sum are rounded
// to the element type one by one, exactly as the unfused tensor expression rounds them, so the stored
// rows are bit-identical to "rotate first, append after".  V rows are copied unchanged.
template <typename T> struct RopeMath;
template <> struct RopeMath<float> {
    static __device__ __forceinline__ float rot(float a, float ca, float b, float sb, bool minus) {
        const float p = __fmul_rn(a, ca), q = __fmul_rn(b, sb);
        return minus ? __fsub_rn(p, q) : __fadd_rn(p, q);
    }
};
template <> struct RopeMath<__nv_bfloat16> {
    static __device__ __forceinline__ __nv_bfloat16 rot(__nv_bfloat16 a, __nv_bfloat16 ca, __nv_bfloat16 b,
                                                       __nv_bfloat16 sb, bool minus) {
        const float p = __bfloat162float(__float2bfloat16_rn(__fmul_rn(__bfloat162float(a), __bfloat162float(ca))));
        const float q = __bfloat162float(__float2bfloat16_rn(__fmul_rn(__bfloat162float(b), __bfloat162float(sb))));
        return __float2bfloat16_rn(minus ? __fsub_rn(p, q) : __fadd_rn(p, q));
    }
};
template <> struct RopeMath<__half> {
    static __device__ __forceinline__ __half rot(__half a, __half ca, __half b, __half sb, bool minus) {
        const float p = __half2float(__float2half_rn(__fmul_rn(__half2float(a), __half2float(ca))));
        const float q = __half2float(__float2half_rn(__fmul_rn(__half2float(b), __half2float(sb))));
        return __float2half_rn(minus ? __fsub_rn(p, q) : __fadd_rn(p, q));
    }
};

struct RopeArgs {
    const unsigned char* cos;    // [total_tokens][head_dim] in the element type, row r for new token r
    const unsigned char* sin;
    long long tok;               // byte stride between token rows of cos / sin
};

template <typename T>
__global__ void __launch_bounds__(kAppendThreads)
append_rope_kernel(const AppendArgs a, const RopeArgs rp) {
    constexpr int E = 16 / (int)sizeof(T);            // elements per 16-byte vector
    __shared__ long long s_dst[kAppendMaxTile];
    __shared__ long long s_src[kAppendMaxTile];
    const int tid = threadIdx.x;
    const int first_tok = blockIdx.x * a.tile;
    const int ntok = min(a.tile, a.total_tokens - first_tok);
    pdl_wait_for_predecessor();
    pdl_let_successor_in();
    if (tid < ntok) resolve_new_token(a, first_tok + tid, &s_dst[tid], &s_src[tid]);
    __syncthreads();

    const int vpr = a.row_bytes / 16;                 // vectors per row
    const int half = vpr / 2;                         // vectors per half row
    // per token and head: `half` K items (two vectors each) and `vpr` V items (one vector each)
    const int per_head = half + vpr;
    const int per_tok = a.heads * per_head;
    const int items = ntok * per_tok;
    for (int idx = tid; idx < items; idx += blockDim.x) {
        const int t = idx / per_tok;
        const int rem = idx - t * per_tok;
        const int h = rem / per_head;
        const int w = rem - h * per_head;
        const long long d = s_dst[t];
        if (d < 0) continue;
        if (w >= half) {                               // V: plain copy of vector w - half
            const int vec = w - half;
            const uint4 x = __ldcs(reinterpret_cast<const uint4*>(a.v_new + s_src[t] + h * a.nr.head) + vec);
            reinterpret_cast<uint4*>(a.v_pool + d + h * a.pool_head)[vec] = x;
            continue;
        }
        const uint4* krow = reinterpret_cast<const uint4*>(a.k_new + s_src[t] + h * a.nr.head);
        const uint4* crow = reinterpret_cast<const uint4*>(rp.cos + (long long)(first_tok + t) * rp.tok);
        const uint4* srow = reinterpret_cast<const uint4*>(rp.sin + (long long)(first_tok + t) * rp.tok);
        union Pack { uint4 v; T e[E]; };
        Pack lo, hi, clo, chi, slo, shi, olo, ohi;
        lo.v = __ldcs(krow + w);
        hi.v = __ldcs(krow + w + half);
        clo.v = __ldg(crow + w);
        chi.v = __ldg(crow + w + half);
        slo.v = __ldg(srow + w);
        shi.v = __ldg(srow + w + half);
#pragma unroll
        for (int e = 0; e < E; ++e) {
            olo.e[e] = RopeMath<T>::rot(lo.e[e], clo.e[e], hi.e[e], slo.e[e], true);
            ohi.e[e] = RopeMath<T>::rot(hi.e[e], chi.e[e], lo.e[e], shi.e[e], false);
        }
        uint4* out = reinterpret_cast<uint4*>(a.k_pool + d + h * a.pool_head);
        out[w] = olo.v;
        out[w + half] = ohi.v;
    }
}

// --------------------------------------------------------------------------
// page copies (fork / beam search: a sequence's partial last page is duplicated)
// --------------------------------------------------------------------------
struct CopyArgs {
    unsigned char* k_pool;
    unsigned char* v_pool;
    const int32_t* src;
    const int32_t* dst;
    int n, heads, num_pages, page_bytes;
    long long pool_head, pool_page, pool_layer;
    int32_t* status;
};

// gridDim = (pairs * heads, layers, 2 [K, V]); a CTA copies one page of one head.
template <typename V>
__global__ void __launch_bounds__(128)
copy_pages_kernel(const CopyArgs a) {
    pdl_wait_for_predecessor();
    pdl_let_successor_in();
    const int pair = blockIdx.x / a.heads;
    const int head = blockIdx.x - pair * a.heads;
    const int from = a.src[pair], to = a.dst[pair];
    if (from < 0 || from >= a.num_pages || to < 0 || to >= a.num_pages) {
        if (threadIdx.x == 0) raise(a.status, BARQKV_S_BAD_PAGE);
        return;
    }
    unsigned char* base = (blockIdx.z ? a.v_pool : a.k_pool) + (long long)blockIdx.y * a.pool_layer + head * a.pool_head;
    const V* in = reinterpret_cast<const V*>(base + (long long)from * a.pool_page);
    V* out = reinterpret_cast<V*>(base + (long long)to * a.pool_page);
    const int count = a.page_bytes / (int)sizeof(V);
    for (int i = threadIdx.x; i < count; i += blockDim.x) out[i] = in[i];
}

// --------------------------------------------------------------------------
// block-table maintenance: the host sends only the entries that changed
// --------------------------------------------------------------------------
// pairs[2*i] = flat index into the table, pairs[2*i+1] = new page id (or -1)
__global__ void __launch_bounds__(128)
table_scatter_kernel(int32_t* __restrict__ table, const int32_t* __restrict__ pairs, int n, long long table_words) {
    pdl_wait_for_predecessor();
    pdl_let_successor_in();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const long long at = pairs[2 * i];
        if (at >= 0 && at < table_words) table[at] = pairs[2 * i + 1];
    }
}

// --------------------------------------------------------------------------
// gather: shared work decomposition
// --------------------------------------------------------------------------
// Exclusive prefix sum of per-entry page counts into s_cu[0..n]; returns nothing,
// callers read s_cu[n] for the total after the trailing barrier.
// Tokens entry i holds once the call is done (old length plus, when an append is fused in, its new rows).
__device__ __forceinline__ int entry_new_rows(const GatherArgs& a, int i) {
    if (!a.k_new) return 0;
    return a.cu_new ? a.cu_new[i + 1] - a.cu_new[i] : a.tokens_per_entry;
}
__device__ __forceinline__ int entry_len(const GatherArgs& a, int i) {
    return max(a.seq_lens[i], 0) + entry_new_rows(a, i);
}

__device__ void scan_pages(const GatherArgs& a, int* s_cu, int* s_part) {
    const int n = a.n, page_size = a.page_size;
    const int tid = threadIdx.x;
    const int nthr = blockDim.x;
    const int chunk = (n + nthr - 1) / nthr;
    const int lo = min(n, tid * chunk);
    const int hi = min(n, lo + chunk);
    int sum = 0;
    for (int i = lo; i < hi; ++i) sum += (entry_len(a, i) + page_size - 1) / page_size;
    // inclusive scan inside the warp
    const int lane = tid & 31;
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
    }
    if (lane == 31) s_part[tid >> 5] = incl;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < (tid >> 5); ++w) before += s_part[w];
    int run = before + incl - sum;
    for (int i = lo; i < hi; ++i) {
        s_cu[i] = run;
        run += (entry_len(a, i) + page_size - 1) / page_size;
    }
    if (lo < hi && hi == n) s_cu[n] = run;      // the thread that owns the last entry
    if (n == 0 && tid == 0) s_cu[0] = 0;
    __syncthreads();
}

struct TileInfo {
    long long src;   // byte offset of the physical page within head 0's pool
    long long dst;   // byte offset of the page's first row (head 0) in the output
    int rows;        // valid rows in this page, 0 = skip
    int rows_old;    // of those, rows already in the pool; the rest come from the new rows (fused append)
    long long new_src;  // byte offset of the page's first new row (head 0) in the new rows
};

// Resolve flat tile q (a (sequence, page) pair) using the scanned page counts.
__device__ __forceinline__ TileInfo resolve_tile(const GatherArgs& a, const int* s_cu, int q) {
    int lo = 0, hi = a.n - 1;                 // largest i with s_cu[i] <= q
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_cu[mid] <= q) lo = mid; else hi = mid - 1;
    }
    const int i = lo;
    const int j = q - s_cu[i];
    const int len_old = max(a.seq_lens[i], 0);
    const int len = len_old + entry_new_rows(a, i);
    TileInfo t;
    t.rows = min(a.page_size, len - j * a.page_size);
    t.rows_old = min(t.rows, max(len_old - j * a.page_size, 0));
    t.new_src = 0;
    if (t.rows_old < t.rows) {
        const long long tok = (long long)j * a.page_size + t.rows_old - len_old;      // index among the entry's new rows
        const long long base = a.nr.packed ? (a.cu_new ? (long long)a.cu_new[i] : (long long)i * a.tokens_per_entry) : 0;
        t.new_src = (long long)i * a.nr.seq + (base + tok) * a.nr.tok;
    }
    const long long page = resolve_page(a.tb, i, j, a.status);
    if (page < 0) t.rows = t.rows_old = 0;
    t.src = page * a.pool_page;
    const long long base_tok = (a.orow.packed ? (long long)a.cu_out[i] : 0) + (long long)j * a.page_size;
    t.dst = (long long)i * a.orow.seq + base_tok * a.orow.tok;
    return t;
}

template <typename V>
__global__ void __launch_bounds__(kGatherThreads)
gather_vector_kernel(const GatherArgs a) {
    extern __shared__ int s_dyn[];            // s_cu[n + 1]
    __shared__ int s_part[kGatherThreads / 32];
    __shared__ long long s_src[kGroup];
    __shared__ long long s_dst[kGroup];
    __shared__ int s_rows[kGroup];

    int* s_cu = s_dyn;
    pdl_wait_for_predecessor();
    pdl_let_successor_in();
    scan_pages(a, s_cu, s_part);
    const int total = s_cu[a.n];
    int lo, hi, group_step;
    if (a.interleave) {
        lo = (int)blockIdx.x * kGroup;
        hi = total;
        group_step = (int)gridDim.x * kGroup;
    } else {
        const int per = (total + (int)gridDim.x - 1) / (int)gridDim.x;
        lo = min(total, (int)blockIdx.x * per);
        hi = min(total, lo + per);
        group_step = kGroup;
    }

    const int tid = threadIdx.x;
    const int vpr = a.row_bytes / (int)sizeof(V);
    const int page_vecs = a.page_size * vpr;
    const int per_tile = a.heads * 2 * page_vecs;          // order inside a tile: head, K|V, row, vector

    for (int g0 = lo; g0 < hi; g0 += group_step) {
        const int nt = min(kGroup, hi - g0);
        __syncthreads();
        if (tid < nt) {
            const TileInfo t = resolve_tile(a, s_cu, g0 + tid);
            s_src[tid] = t.src;
            s_dst[tid] = t.dst;
            s_rows[tid] = t.rows;
        }
        __syncthreads();
        const int items = nt * per_tile;
        for (int base = tid; base < items; base += blockDim.x * kUnroll) {
            V val[kUnroll];
            V* out[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int idx = base + u * blockDim.x;
                out[u] = nullptr;
                if (idx < items) {
                    const int t = idx / per_tile;
                    const int rem = idx - t * per_tile;
                    const int hk = rem / page_vecs;
                    const int pv = rem - hk * page_vecs;
                    const int row = pv / vpr;
                    const int vec = pv - row * vpr;
                    if (row < s_rows[t]) {
                        const int h = hk >> 1;
                        const bool is_v = hk & 1;
                        const unsigned char* src = (is_v ? a.v_pool : a.k_pool) + s_src[t] + h * a.pool_head;
                        unsigned char* dst = (is_v ? a.v_out : a.k_out) + s_dst[t] + h * a.orow.head +
                                             (long long)row * a.orow.tok;
                        val[u] = __ldcs(reinterpret_cast<const V*>(src) + pv);
                        out[u] = reinterpret_cast<V*>(dst) + vec;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                if (out[u]) __stcs(out[u], val[u]);
            }
        }
    }
}

// --------------------------------------------------------------------------
// gather with bulk asynchronous copies
// --------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src_gmem, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
        "l"(__cvta_generic_to_global(src_gmem)), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst_gmem, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(__cvta_generic_to_global(dst_gmem)),
                 "r"(src_smem), "r"(bytes)
                 : "memory");
}
// Tiled TMA store of a [page_size][1 head][head_dim] box from dense shared memory into an output whose
// rows are strided (token-major [tokens, heads, head_dim]); coordinates are (element 0, head, token).
// The innermost coordinate is always 0, so the 16-byte rule on it holds by construction.
__device__ __forceinline__ void tensor_store_3d(const CUtensorMap* map, uint32_t src_smem, int head, int token) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(0), "r"(head), "r"(token), "r"(src_smem)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// One warp per CTA.  A "unit" is one (page, head): the K page and the V page of
// that head travel together through one ring stage.  The store of unit g is
// issued once unit g + lag has been loaded (lag = stages - 2), so `lag` loads
// are in flight while at most two stores are still reading shared memory.
__global__ void __launch_bounds__(32)
gather_bulk_kernel(const GatherArgs a, const __grid_constant__ CUtensorMap out_map_k,
                   const __grid_constant__ CUtensorMap out_map_v) {
    extern __shared__ __align__(128) unsigned char s_raw[];
    const int lane = threadIdx.x;
    const int S = a.stages;
    const int lag = S - 2;
    const int page_bytes = a.page_size * a.row_bytes;

    unsigned char* s_data = s_raw;                                          // [S][2][page_bytes]
    unsigned long long* s_bar = reinterpret_cast<unsigned long long*>(s_data + (size_t)S * 2 * page_bytes);
    long long* s_slot_dst = reinterpret_cast<long long*>(s_bar + S);        // [S] output offset incl. head
    long long* s_slot_pool = s_slot_dst + S;                                // [S] pool offset incl. head
    long long* s_src = s_slot_pool + S;                                     // [kGroup]
    long long* s_dst = s_src + kGroup;                                      // [kGroup]
    long long* s_new = s_dst + kGroup;                                      // [kGroup] first new row (fused append)
    int* s_rows = reinterpret_cast<int*>(s_new + kGroup);                   // [kGroup]
    int* s_rows_old = s_rows + kGroup;                                      // [kGroup]
    int* s_slot_rows = s_rows_old + kGroup;                                 // [S]
    int* s_slot_rows_old = s_slot_rows + S;                                 // [S]
    int* s_slot_tok = s_slot_rows_old + S;                                  // [S] output token index of the page's first row
    int* s_slot_head = s_slot_tok + S;                                      // [S]
    int* s_part = s_slot_head + S;                                          // [1]
    int* s_cu = s_part + 1;                                                 // [n + 1]

    if (lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(smem_addr(&s_bar[s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Everything up to the first copy reads only the batch description and the block table.  When the
    // caller vouches that those are older than the kernel before this one (a.early), that part runs
    // while that kernel is still draining; otherwise it starts after it.
    // In a chain of launches that alternate between two counter pairs nobody counts finished CTAs: the launch that
    // uses one pair clears the other - last used by the launch before it, which has finished when the wait below
    // returns, and next used by the launch after it, which cannot start its prologue before every CTA of this
    // launch, the clearing one included, has let it in.
    auto clear_other_pair = [&]() {
        if (a.zero_ahead && blockIdx.x == 0 && lane == 0) {
            a.zero_ahead[0] = 0;
            a.zero_ahead[1] = 0;
            __threadfence();
        }
    };
    if (!a.early) {
        pdl_wait_for_predecessor();
        clear_other_pair();
        pdl_let_successor_in();
    }
    // The first group's size comes from the host's bound of the tile count, so its fetch can travel
    // to L2 and back while the lengths are being scanned.
    const bool early = a.work != nullptr && a.static_permille == 0;
    int early_first = 0;
    if (early && lane == 0) early_first = atomicAdd(a.work, a.first_group);
    scan_pages(a, s_cu, s_part);   // ends with a CTA barrier

    // This CTA's tiles come in groups of consecutive tiles of the flat list:
    //  - dynamic (a.work != null): groups of a.group_tiles handed out by an atomic
    //    counter, so SMs that reach memory faster simply take more groups;
    //  - static: one contiguous share (interleave == 0) or every gridDim-th group.
    const int tiles = s_cu[a.n];               // (sequence, page) tiles of one layer
    const int total = tiles * a.layers;        // the flat list repeats them layer after layer
    const bool dynamic = a.work != nullptr;
    const int gt_max = dynamic ? a.group_tiles : kGroup;
    int gt = gt_max;                       // tiles in the current group
    int group_base, group_step = 0, end = total;
    int pending = 0, pending_n = 0;        // lane 0: the group fetched ahead of need (first tile, tile count)
    // Dynamic hand-out: every CTA first works through a fixed share of the front part of the list
    // (a.static_permille of the tiles, no atomics, no fetch latency at the start), then takes groups
    // of the rest from an atomic tile counter.  Those groups shrink as the work runs out
    // (remaining / 2*CTAs, at most group_tiles, at least 1) so that all CTAs finish together.
    const int share = dynamic ? (int)((long long)total * a.static_permille / 1000 / (int)gridDim.x) : 0;
    const int dyn_first = share * (int)gridDim.x;           // first tile that is handed out dynamically
    bool fixed_share = false;                               // still inside the fixed share
    auto fetch_ahead = [&](int seen) {
        int k = (total - seen) / (2 * (int)gridDim.x);
        k = max(1, min(k, gt_max));
        pending_n = k;
        pending = dyn_first + atomicAdd(a.work, k);
    };
    if (dynamic) {
        if (lane == 0) {
            if (early) { pending = early_first; pending_n = a.first_group; }
            else fetch_ahead(dyn_first);
        }
        if (share > 0) {
            fixed_share = true;
            group_base = (int)blockIdx.x * share;
            end = group_base + share;
            gt = kGroup;
        } else {
            group_base = min(end, __shfl_sync(0xffffffffu, pending, 0));
            gt = __shfl_sync(0xffffffffu, pending_n, 0);
            if (lane == 0 && group_base < end) fetch_ahead(group_base);
        }
    } else if (a.interleave) {
        group_base = (int)blockIdx.x * kGroup;
        group_step = (int)gridDim.x * kGroup;
    } else {
        const int per = (total + (int)gridDim.x - 1) / (int)gridDim.x;
        group_base = min(total, (int)blockIdx.x * per);
        group_step = kGroup;
        end = min(total, group_base + per);
    }
    const bool contiguous_rows = a.orow.tok == a.row_bytes;   // a page's rows are adjacent in the output

    bool more = group_base < end;          // issue side still has units
    bool staged = false;                   // current group resolved into shared memory
    int ti = 0, head = 0;                  // issue cursor inside the group
    int islot = 0, cslot = 0;              // ring positions
    uint32_t cphase = 0;
    long long issued = 0, consumed = 0;
    bool dead = false;

    // Resolve the current group's tiles (block-table look-ups included) into shared memory.
    auto stage_group = [&]() {
        __syncwarp();
        if (lane < gt && group_base + lane < end) {
            const int flat = group_base + lane;
            const int layer = a.layers > 1 ? flat / tiles : 0;
            const TileInfo t = resolve_tile(a, s_cu, flat - layer * tiles);
            s_src[lane] = t.src + layer * a.pool_layer;
            s_dst[lane] = t.dst + layer * a.out_layer;
            s_new[lane] = t.new_src;
            s_rows[lane] = t.rows;
            s_rows_old[lane] = t.rows_old;
        }
        __syncwarp();
        staged = true;
    };
    if (a.early) {
        if (more) stage_group();
        pdl_wait_for_predecessor();     // from here on the pools, the new rows and the outputs are touched
        clear_other_pair();
        pdl_let_successor_in();
    }

    while ((more || consumed < issued) && !dead) {
        if (more) {
            if (!staged) stage_group();
            if (issued >= S) {
                bulk_wait_read<1>();       // the stores that read this stage one ring round ago are done with it
                __syncwarp();
            }
            const int rows = s_rows[ti];
            const int rows_old = s_rows_old[ti];
            const uint32_t bytes = (uint32_t)(rows * a.row_bytes);
            const uint32_t bar = smem_addr(&s_bar[islot]);
            const long long pool_off = s_src[ti] + head * a.pool_head;
            if (lane == 0) {
                s_slot_rows[islot] = rows;
                s_slot_rows_old[islot] = rows_old;
                s_slot_dst[islot] = s_dst[ti] + head * a.orow.head;
                s_slot_pool[islot] = pool_off;
                if (a.tensor_store) {
                    s_slot_tok[islot] = (int)(s_dst[ti] / a.orow.tok);
                    s_slot_head[islot] = head;
                }
                if (bytes) mbar_arrive_expect(bar, 2 * bytes + (uint32_t)a.extra_tx); else mbar_arrive(bar);
            }
            __syncwarp();
            unsigned char* stage = s_data + (size_t)islot * 2 * page_bytes;
            if (lane < 2 && rows_old) {
                bulk_load(smem_addr(stage + lane * page_bytes), (lane ? a.v_pool : a.k_pool) + pool_off,
                          (uint32_t)(rows_old * a.row_bytes), bar);
            }
            if (rows_old < rows) {
                // rows this call appends: one small copy each, straight from the new rows into the stage
                const long long src0 = s_new[ti] + head * a.nr.head;
                for (int op = lane; op < 2 * (rows - rows_old); op += 32) {
                    const int r = op >> 1, kv = op & 1;
                    bulk_load(smem_addr(stage + kv * page_bytes + (rows_old + r) * a.row_bytes),
                              (kv ? a.v_new : a.k_new) + src0 + (long long)r * a.nr.tok, (uint32_t)a.row_bytes, bar);
                }
            }
            ++issued;
            if (++islot == S) islot = 0;
            if (++head == a.heads) {
                head = 0;
                if (++ti == gt || group_base + ti >= end) {
                    ti = 0;
                    staged = false;
                    if (fixed_share && group_base + gt < end) {
                        group_base += gt;                   // next group of the fixed share
                    } else if (dynamic) {
                        fixed_share = false;
                        end = total;
                        group_base = min(end, __shfl_sync(0xffffffffu, pending, 0));
                        gt = __shfl_sync(0xffffffffu, pending_n, 0);
                        if (lane == 0 && group_base < end) fetch_ahead(group_base);
                    } else {
                        group_base += group_step;
                    }
                    more = group_base < end;
                }
            }
        }
        if (issued - consumed > lag || (!more && consumed < issued)) {
            const uint32_t bar = smem_addr(&s_bar[cslot]);
            const long long t0 = clock64();
            while (!mbar_try_wait(bar, cphase)) {
                if (clock64() - t0 > a.wait_cycles) { dead = true; break; }
            }
            dead = __any_sync(0xffffffffu, dead);
            if (!dead) {
                const int rows = s_slot_rows[cslot];
                const int rows_old = s_slot_rows_old[cslot];
                const long long dst = s_slot_dst[cslot];
                if (rows) {
                    fence_async_smem();
                    const uint32_t sk = smem_addr(s_data + (size_t)cslot * 2 * page_bytes);
                    if (rows_old < rows && lane < 2) {
                        // fused append: the new rows also go to their slots of the page
                        bulk_store((lane ? a.v_pool_w : a.k_pool_w) + s_slot_pool[cslot] + (long long)rows_old * a.row_bytes,
                                   sk + lane * page_bytes + rows_old * a.row_bytes,
                                   (uint32_t)((rows - rows_old) * a.row_bytes));
                    }
                    if (contiguous_rows) {
                        if (lane < 2) {
                            bulk_store((lane ? a.v_out : a.k_out) + dst, sk + lane * page_bytes,
                                       (uint32_t)(rows * a.row_bytes));
                        }
                    } else if (a.tensor_store && rows == a.page_size) {
                        if (lane < 2) {
                            tensor_store_3d(lane ? &out_map_v : &out_map_k, sk + lane * page_bytes, s_slot_head[cslot],
                                            s_slot_tok[cslot]);
                        }
                    } else {
                        for (int op = lane; op < 2 * rows; op += 32) {
                            const int r = op >> 1, kv = op & 1;
                            bulk_store((kv ? a.v_out : a.k_out) + dst + (long long)r * a.orow.tok,
                                       sk + kv * page_bytes + r * a.row_bytes, (uint32_t)a.row_bytes);
                        }
                    }
                }
                bulk_commit();
                ++consumed;
                if (++cslot == S) { cslot = 0; cphase ^= 1; }
            }
        }
    }
    bulk_wait_read<0>();
    if (dead) {
        // Gave up on a wait: nothing more is issued.  Copies already on their way into this CTA's shared
        // memory get a last, short chance to land before the CTA leaves (a landed copy flips its barrier;
        // one that never will is not waited for twice).
        const long long grace = a.wait_cycles < kDrainCycles ? a.wait_cycles : kDrainCycles;
        while (consumed < issued) {
            const uint32_t bar = smem_addr(&s_bar[cslot]);
            const long long t0 = clock64();
            while (!mbar_try_wait(bar, cphase) && clock64() - t0 <= grace) {}
            ++consumed;
            if (++cslot == S) { cslot = 0; cphase ^= 1; }
        }
        if (lane == 0) raise(a.status, BARQKV_S_TIMEOUT);
    }
    if (dynamic && a.rearm && lane == 0) {
        // The last CTA to finish re-arms the counters for the next launch.
        __threadfence();
        const int finished = atomicAdd(a.work + 1, 1);
        if (finished == (int)gridDim.x - 1) {
            __threadfence();
            a.work[0] = 0;
            a.work[1] = 0;
        }
    }
}

// --------------------------------------------------------------------------
// append with bulk asynchronous copies (page-sized appends: prefill chunks)
// --------------------------------------------------------------------------
// The mirror image of the bulk gather.  A "tile" is the part of one page that one batch entry's new
// tokens fill (a whole page except at the ends of the entry's token range); a "unit" is a tile of one
// head, K and V together in one ring stage.  The new rows of a unit come in with ONE copy per K / V:
//   - rows of a head adjacent in memory ([heads, tokens, head_dim] sources): a plain bulk copy;
//   - token-major sources ([tokens, heads, head_dim], rows of a head one token-stride apart): a tiled
//     TMA load of a [page_size][1 head][head_dim] box starting at the tile's first token.  The box is
//     always page_size rows; rows past the tile (the next tokens, or zero fill past the last token)
//     land in the stage and are simply not stored.  The innermost coordinate is always 0.
// and leave with one bulk store into the page's slots.  Units are handed to the persistent one-warp
// CTAs through the same atomic counter scheme as in the gather.  No multicast, no peer memory.
struct AppendBulkArgs {
    int stages;
    int32_t* work;          // [0] next tile to hand out, [1] CTAs finished
    int32_t* zero_ahead;    // another counter pair, cleared once the kernel before this one has finished (chained launches)
    int rearm;              // the last CTA to finish clears `work` (else a later launch's zero_ahead does)
    int group_tiles, first_group;
    int tensor_load;        // 1: tiled TMA loads (token-major source); 0: plain bulk copies (rows adjacent)
    int layers;
    long long wait_cycles;
};

// Tiles entry i contributes: pages its new tokens touch.
__device__ __forceinline__ int entry_new_tiles(const AppendArgs& a, int i) {
    const int cnt = a.cu_new ? a.cu_new[i + 1] - a.cu_new[i] : a.tokens_per_entry;
    const int start = a.seq_start[i];
    if (cnt <= 0 || start < 0) return 0;
    return (start + cnt - 1) / a.page_size - start / a.page_size + 1;
}

__global__ void __launch_bounds__(32)
append_bulk_kernel(const AppendArgs a, const AppendBulkArgs x, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v) {
    extern __shared__ __align__(128) unsigned char s_raw[];
    const int lane = threadIdx.x;
    const int S = x.stages;
    const int lag = S - 2;
    const int page_bytes = a.page_size * a.row_bytes;

    unsigned char* s_data = s_raw;                                          // [S][2][page_bytes]
    unsigned long long* s_bar = reinterpret_cast<unsigned long long*>(s_data + (size_t)S * 2 * page_bytes);
    long long* s_slot_dst = reinterpret_cast<long long*>(s_bar + S);        // [S] pool offset incl. head and first row
    long long* s_dst = s_slot_dst + S;                                      // [kGroup] pool offset of the tile's first row, head 0
    long long* s_src = s_dst + kGroup;                                      // [kGroup] byte offset of the tile's first new row, head 0
    int* s_tok = reinterpret_cast<int*>(s_src + kGroup);                    // [kGroup] flat index of the tile's first new token
    int* s_rows = s_tok + kGroup;                                           // [kGroup]
    int* s_lay = s_rows + kGroup;                                           // [kGroup]
    int* s_slot_rows = s_lay + kGroup;                                      // [S]
    int* s_cu = s_slot_rows + S;                                            // [n + 1]

    if (lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(smem_addr(&s_bar[s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // chained launches alternate between two counter pairs and clear each other's (see gather_bulk_kernel)
    auto clear_other_pair = [&]() {
        if (x.zero_ahead && blockIdx.x == 0 && lane == 0) {
            x.zero_ahead[0] = 0;
            x.zero_ahead[1] = 0;
            __threadfence();
        }
    };
    if (!a.early) {
        pdl_wait_for_predecessor();
        clear_other_pair();
        pdl_let_successor_in();
    }
    int early_first = 0;
    if (lane == 0) early_first = atomicAdd(x.work, x.first_group);

    // exclusive prefix sum of the entries' tile counts (one warp; the batch is small)
    {
        const int n = a.n;
        const int chunk = (n + 31) / 32;
        const int lo = min(n, lane * chunk), hi = min(n, lo + chunk);
        int sum = 0;
        for (int i = lo; i < hi; ++i) sum += entry_new_tiles(a, i);
        int incl = sum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += up;
        }
        int run = incl - sum;
        for (int i = lo; i < hi; ++i) {
            s_cu[i] = run;
            run += entry_new_tiles(a, i);
        }
        const int all = __shfl_sync(0xffffffffu, incl, 31);
        if (lane == 0) s_cu[n] = all;
        __syncwarp();
    }
    const int tiles = s_cu[a.n];
    const int total = tiles * x.layers;
    const int gt_max = x.group_tiles;
    int gt, group_base;
    int pending = 0, pending_n = 0;
    auto fetch_ahead = [&](int seen) {
        int k = (total - seen) / (2 * (int)gridDim.x);
        k = max(1, min(k, gt_max));
        pending_n = k;
        pending = atomicAdd(x.work, k);
    };
    group_base = min(total, __shfl_sync(0xffffffffu, early_first, 0));
    gt = x.first_group;
    if (lane == 0 && group_base < total) fetch_ahead(group_base);

    bool more = group_base < total;
    bool staged = false;
    int ti = 0, head = 0;
    int islot = 0, cslot = 0;
    uint32_t cphase = 0;
    long long issued = 0, consumed = 0;
    bool dead = false;

    auto stage_group = [&]() {
                __syncwarp();
                if (lane < gt && group_base + lane < total) {
                    const int flat = group_base + lane;
                    const int layer = x.layers > 1 ? flat / tiles : 0;
                    const int q = flat - layer * tiles;
                    int lo = 0, hi = a.n - 1;             // largest i with s_cu[i] <= q
                    while (lo < hi) {
                        const int mid = (lo + hi + 1) >> 1;
                        if (s_cu[mid] <= q) lo = mid; else hi = mid - 1;
                    }
                    const int i = lo;
                    const int start = a.seq_start[i];
                    const int cnt = a.cu_new ? a.cu_new[i + 1] - a.cu_new[i] : a.tokens_per_entry;
                    const int j = start / a.page_size + (q - s_cu[i]);
                    const int first = max(start, j * a.page_size);                 // first position this tile fills
                    const int last = min(start + cnt, (j + 1) * a.page_size);      // one past the last
                    const int t = first - start;                                   // index among the entry's new tokens
                    const long long base = a.cu_new ? (long long)a.cu_new[i] : (long long)i * a.tokens_per_entry;
                    const long long page = resolve_page(a.tb, i, j, a.status);
                    s_rows[lane] = page < 0 ? 0 : last - first;
                    s_dst[lane] = page * a.pool_page + (long long)(first - j * a.page_size) * a.row_bytes +
                                  layer * a.pool_layer;
                    s_src[lane] = (long long)i * a.nr.seq + (a.nr.packed ? base + t : (long long)t) * a.nr.tok +
                                  layer * a.new_layer;
                    s_tok[lane] = (int)(base + t);
                    s_lay[lane] = layer;
                }
                __syncwarp();
                staged = true;
    };
    if (a.early) {
        if (more) stage_group();
        pdl_wait_for_predecessor();     // from here on the new rows are read and the pools written
        clear_other_pair();
        pdl_let_successor_in();
    }

    while ((more || consumed < issued) && !dead) {
        if (more) {
            if (!staged) stage_group();
            if (issued >= S) {
                bulk_wait_read<1>();       // the store that read this stage one ring round ago is done with it
                __syncwarp();
            }
            const int rows = s_rows[ti];
            const uint32_t bar = smem_addr(&s_bar[islot]);
            const uint32_t tx = x.tensor_load ? (uint32_t)page_bytes : (uint32_t)(rows * a.row_bytes);
            if (lane == 0) {
                s_slot_rows[islot] = rows;
                s_slot_dst[islot] = s_dst[ti] + head * a.pool_head;
                if (rows) mbar_arrive_expect(bar, 2 * tx); else mbar_arrive(bar);
            }
            __syncwarp();
            if (lane < 2 && rows) {
                const uint32_t dst = smem_addr(s_data + (size_t)islot * 2 * page_bytes + lane * page_bytes);
                if (x.tensor_load) {
                    asm volatile(
                        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(lane ? &map_v : &map_k)), "r"(0), "r"(head), "r"(s_tok[ti]),
                        "r"(s_lay[ti]), "r"(bar)
                        : "memory");
                } else {
                    bulk_load(dst, (lane ? a.v_new : a.k_new) + s_src[ti] + head * a.nr.head, tx, bar);
                }
            }
            ++issued;
            if (++islot == S) islot = 0;
            if (++head == a.heads) {
                head = 0;
                if (++ti == gt || group_base + ti >= total) {
                    ti = 0;
                    staged = false;
                    group_base = min(total, __shfl_sync(0xffffffffu, pending, 0));
                    gt = __shfl_sync(0xffffffffu, pending_n, 0);
                    if (lane == 0 && group_base < total) fetch_ahead(group_base);
                    more = group_base < total;
                }
            }
        }
        if (issued - consumed > lag || (!more && consumed < issued)) {
            const uint32_t bar = smem_addr(&s_bar[cslot]);
            const long long t0 = clock64();
            while (!mbar_try_wait(bar, cphase)) {
                if (clock64() - t0 > x.wait_cycles) { dead = true; break; }
            }
            dead = __any_sync(0xffffffffu, dead);
            if (!dead) {
                const int rows = s_slot_rows[cslot];
                if (rows) {
                    fence_async_smem();
                    if (lane < 2) {
                        bulk_store((lane ? a.v_pool : a.k_pool) + s_slot_dst[cslot],
                                   smem_addr(s_data + (size_t)cslot * 2 * page_bytes + lane * page_bytes),
                                   (uint32_t)(rows * a.row_bytes));
                    }
                }
                bulk_commit();
                ++consumed;
                if (++cslot == S) { cslot = 0; cphase ^= 1; }
            }
        }
    }
    bulk_wait_read<0>();
    if (dead) {
        const long long grace = x.wait_cycles < kDrainCycles ? x.wait_cycles : kDrainCycles;
        while (consumed < issued) {
            const uint32_t bar = smem_addr(&s_bar[cslot]);
            const long long t0 = clock64();
            while (!mbar_try_wait(bar, cphase) && clock64() - t0 <= grace) {}
            ++consumed;
            if (++cslot == S) { cslot = 0; cphase ^= 1; }
        }
        if (lane == 0) raise(a.status, BARQKV_S_TIMEOUT);
    }
    if (x.rearm && lane == 0) {
        __threadfence();
        const int finished = atomicAdd(x.work + 1, 1);
        if (finished == (int)gridDim.x - 1) {
            __threadfence();
            x.work[0] = 0;
            x.work[1] = 0;
        }
    }
}

// --------------------------------------------------------------------------
// host side
// --------------------------------------------------------------------------
// Experiment knobs.  A normal build has none: the values below are compile-time defaults and the library
// keeps no mutable process-wide settings.  A build with -DBARQKV_TUNING turns them into variables that
// barqkv_set_tuning (include/barqkv_experimental.h) changes; that build is for sweeps, not for serving.
struct Knobs {
    int stages = 0;              // ring stages of the bulk gather; 0 = automatic
    int bulk_ctas_per_sm = 0;    // 0 = as many as shared memory holds
    int vector_ctas_per_sm = 0;
    int interleave = -1;
    int group_tiles = 0;
    int static_shares = 0;
    int pdl = -1;                // -1: programmatic dependent launch where the entry point allows it; 0: never
    int static_permille = -1;
    int tensor_store = -1;
    int attn_promotion = -1;
    int attn_split_tokens = 0;
    int append_bulk = -1;        // -1: page-sized appends go through the copy engine; 0: always the row kernel
    int layer_overlap = 1;       // update_layers issues odd layers on a second stream (0: one stream, one chain)
    int attn_page_box = 2;       // decode attention loads a head's page of K and of V with one copy instruction where the pools allow it
                                 // (1: one instruction for K, one for V; 0: two half-page boxes each)
    int zero_ahead = 1;          // update_layers: a launch clears the counter pair of its neighbours in the chain instead of
                                 // every launch counting its finished CTAs to clear its own (0: every launch re-arms itself)
    int attn_probe = 0;          // timing probes (results are wrong): 1 = decode attention loads pages without attending them, 2 = writes no result
    int attn_compact = 1;        // decode attention: the grid lists only splits that have pages (0: one CTA per possible split)
    int attn_wide = -1;          // decode attention updates its softmax state every 32 tokens (1) or 16 (0);
                                 // -1: 32 for pages of 32 and 64, 16 for pages of 16
};
#ifdef BARQKV_TUNING
Knobs g_knobs;
#else
constexpr Knobs g_knobs{};
#endif

struct DeviceInfo {
    int sms = 0;
    int smem_optin = 0;
    std::atomic<bool> bulk_attr_set{false};     // cudaFuncSetAttribute done for the bulk gather / bulk append
    std::atomic<bool> append_attr_set{false};
    // Second stream of barqkv_update_layers (odd layers), with the events that fork it from and join it to the
    // caller's stream.  Made by the first call that is not being captured into a graph; `lane_mu` serialises
    // the callers that issue through it.
    std::mutex lane_mu;
    cudaStream_t lane = nullptr;
    cudaEvent_t lane_fork = nullptr, lane_join = nullptr;
};
DeviceInfo g_dev[64];
std::once_flag g_dev_once[64];

// Properties of the current device, queried once per device however many threads ask first.
DeviceInfo* device_info() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    DeviceInfo* d = &g_dev[dev];
    std::call_once(g_dev_once[dev], [d, dev]() {
        int sms = 0, optin = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return;
        if (cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return;
        d->smem_optin = optin;
        d->sms = sms;
    });
    return d->sms > 0 ? d : nullptr;
}

// The device's second stream for barqkv_update_layers, or null when it does not exist yet and `caller` is
// being captured (streams and events are not created in the middle of a capture).  Call with lane_mu held.
bool second_stream(DeviceInfo* d, cudaStream_t caller) {
    if (d->lane) return true;
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(caller, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return false;
    }
    cudaStream_t st = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&join, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        if (join) cudaEventDestroy(join);
        if (fork) cudaEventDestroy(fork);
        if (st) cudaStreamDestroy(st);
        return false;
    }
    d->lane_fork = fork;
    d->lane_join = join;
    d->lane = st;
    return true;
}

inline bool aligned(const void* p, int a) { return (reinterpret_cast<uintptr_t>(p) % (uintptr_t)a) == 0; }
inline bool multiple(long long v, int a) { return (v % a) == 0; }

int check_pool(const barqkv_pool_layout* p) {
    if (!p) return fail(BARQKV_E_INVALID, "pool layout is null");
    if (p->num_heads <= 0 || p->head_dim <= 0 || p->page_size <= 0 || p->num_pages <= 0)
        return fail(BARQKV_E_INVALID, "pool layout: num_heads, head_dim, page_size, num_pages must be positive");
    if (p->elem_bytes != 1 && p->elem_bytes != 2 && p->elem_bytes != 4 && p->elem_bytes != 8)
        return fail(BARQKV_E_INVALID, "pool layout: elem_bytes must be 1, 2, 4 or 8");
    if (p->page_stride < (int64_t)p->page_size * p->head_dim)
        return fail(BARQKV_E_INVALID, "pool layout: page_stride is smaller than one page");
    if (p->head_stride < 0) return fail(BARQKV_E_INVALID, "pool layout: negative head_stride");
    return 0;
}

int check_table(const barqkv_block_table* t, int n) {
    if (!t) return fail(BARQKV_E_INVALID, "block table descriptor is null");
    if (t->table_rows <= 0 || t->table_stride <= 0)
        return fail(BARQKV_E_INVALID, "block table: table_rows and table_stride must be positive");
    if (!t->table && t->implicit_pages_per_slot <= 0)
        return fail(BARQKV_E_INVALID, "block table: implicit paging needs implicit_pages_per_slot > 0");
    if (!t->slots && n > t->table_rows)
        return fail(BARQKV_E_INVALID, "block table: more batch entries than table rows");
    return 0;
}

Table make_table(const barqkv_block_table* t, int num_pages) {
    Table tb;
    tb.table = t->table;
    tb.slots = t->slots;
    tb.rows = t->table_rows;
    tb.stride = t->table_stride;
    tb.implicit = t->implicit_pages_per_slot;
    tb.num_pages = num_pages;
    return tb;
}

// Widest power-of-two vector (bytes) that divides every offset the kernels form.
int vector_bytes(int row_bytes, std::initializer_list<long long> strides, std::initializer_list<const void*> ptrs) {
    for (int v = 16; v >= 2; v >>= 1) {
        bool ok = multiple(row_bytes, v);
        for (long long s : strides) ok = ok && multiple(s, v);
        for (const void* p : ptrs) ok = ok && aligned(p, v);
        if (ok) return v;
    }
    return 1;
}

// Launch `kernel`; with `dependent` as a programmatic dependent of the kernel before it in the stream, so that
// the part of it that precedes its griddepcontrol.wait may run while that kernel is still finishing.
template <typename... KernelArgs, typename... Args>
cudaError_t launch(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool dependent,
                   Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <bool LEGACY>
int launch_append(const AppendArgs& a, int vec, dim3 grid, int threads, cudaStream_t st) {
    const bool dep = !LEGACY && a.early != 0;
    cudaError_t e;
    switch (vec) {
        case 16: e = launch(append_rows_kernel<uint4, LEGACY>, grid, dim3(threads), 0, st, dep, a); break;
        case 8: e = launch(append_rows_kernel<uint2, LEGACY>, grid, dim3(threads), 0, st, dep, a); break;
        case 4: e = launch(append_rows_kernel<uint32_t, LEGACY>, grid, dim3(threads), 0, st, dep, a); break;
        case 2: e = launch(append_rows_kernel<uint16_t, LEGACY>, grid, dim3(threads), 0, st, dep, a); break;
        default: e = launch(append_rows_kernel<uint8_t, LEGACY>, grid, dim3(threads), 0, st, dep, a); break;
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    return e == cudaSuccess ? 0 : fail_cuda("append launch", e);
}

// Tokens per CTA and threads per CTA: enough CTAs to cover the machine for small
// (decode) batches, ~32 KiB of payload per CTA for bulk (prefill) batches.
void append_shape(const DeviceInfo* d, int total_tokens, int heads, int row_bytes, int vec, int* tile, int* threads) {
    const long long tok_bytes = 2LL * heads * row_bytes;
    int t = (int)((32 * 1024 + tok_bytes - 1) / tok_bytes);
    if (t > kAppendMaxTile) t = kAppendMaxTile;
    const int want_ctas = 4 * d->sms;
    while (t > 1 && (total_tokens + t - 1) / t < want_ctas) t >>= 1;
    if (t < 1) t = 1;
    const long long items = (long long)t * heads * 2 * (row_bytes / vec);
    int th = kAppendThreads;
    while (th > 32 && th / 2 >= items && th / 2 >= t) th >>= 1;
    if (th < t) th = kAppendThreads;
    *tile = t;
    *threads = th;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point query (no link against libcuda).
PFN_cuTensorMapEncodeTiled tensor_map_encoder() {
    static PFN_cuTensorMapEncodeTiled fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
    }
    return fn;
}

// Describes a packed token-major output [tokens][heads][head_dim] (strides in bytes) for page-sized stores.
bool make_out_map(CUtensorMap* map, void* base, int elem_bytes, int head_dim, int heads, long long head_stride,
                  long long tok_stride, long long tokens, int page_size) {
    PFN_cuTensorMapEncodeTiled enc = tensor_map_encoder();
    if (!enc) return false;
    CUtensorMapDataType dt;
    switch (elem_bytes) {
        case 1: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
        case 2: dt = CU_TENSOR_MAP_DATA_TYPE_UINT16; break;
        case 4: dt = CU_TENSOR_MAP_DATA_TYPE_UINT32; break;
        default: dt = CU_TENSOR_MAP_DATA_TYPE_UINT64; break;
    }
    const cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)heads, (cuuint64_t)tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)head_stride, (cuuint64_t)tok_stride};
    const cuuint32_t box[3] = {(cuuint32_t)head_dim, 1u, (cuuint32_t)page_size};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    return enc(map, dt, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Describes token-major new rows [layers][tokens][heads][head_dim] (strides in bytes) for page-sized loads.
bool make_rows_map(CUtensorMap* map, const void* base, int elem_bytes, int head_dim, int heads, long long head_stride,
                   long long tok_stride, long long tokens, int layers, long long layer_stride, int page_size) {
    PFN_cuTensorMapEncodeTiled enc = tensor_map_encoder();
    if (!enc) return false;
    CUtensorMapDataType dt;
    switch (elem_bytes) {
        case 1: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
        case 2: dt = CU_TENSOR_MAP_DATA_TYPE_UINT16; break;
        case 4: dt = CU_TENSOR_MAP_DATA_TYPE_UINT32; break;
        default: dt = CU_TENSOR_MAP_DATA_TYPE_UINT64; break;
    }
    const cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)heads, (cuuint64_t)tokens, (cuuint64_t)layers};
    const cuuint64_t strides[3] = {(cuuint64_t)head_stride, (cuuint64_t)tok_stride, (cuuint64_t)layer_stride};
    const cuuint32_t box[4] = {(cuuint32_t)head_dim, 1u, (cuuint32_t)page_size, 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    return enc(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" {

int barqkv_version(void) { return BARQKV_VERSION; }

const char* barqkv_last_error(void) { return g_err; }

int64_t barqkv_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int barqkv_sm_count(void) {
    DeviceInfo* d = device_info();
    if (!d) return fail(BARQKV_E_LAUNCH, "no CUDA device is current");
    return d->sms;
}

#ifdef BARQKV_TUNING
int barqkv_set_tuning(int32_t knob, int32_t value) {
    switch (knob) {
        case BARQKV_KNOB_BULK_STAGES: g_knobs.stages = value; return 0;
        case BARQKV_KNOB_BULK_CTAS_PER_SM: g_knobs.bulk_ctas_per_sm = value; return 0;
        case BARQKV_KNOB_VECTOR_CTAS_PER_SM: g_knobs.vector_ctas_per_sm = value; return 0;
        case BARQKV_KNOB_INTERLEAVE: g_knobs.interleave = value; return 0;
        case BARQKV_KNOB_GROUP_TILES: g_knobs.group_tiles = value; return 0;
        case BARQKV_KNOB_STATIC_SHARES: g_knobs.static_shares = value; return 0;
        case BARQKV_KNOB_PDL: g_knobs.pdl = value; return 0;
        case BARQKV_KNOB_STATIC_PERMILLE: g_knobs.static_permille = value > 1000 ? 1000 : value; return 0;
        case BARQKV_KNOB_TENSOR_STORE: g_knobs.tensor_store = value; return 0;
        case BARQKV_KNOB_ATTN_L2_PROMOTION: g_knobs.attn_promotion = value; return 0;
        case BARQKV_KNOB_ATTN_SPLIT_TOKENS: g_knobs.attn_split_tokens = value; return 0;
        case BARQKV_KNOB_APPEND_BULK: g_knobs.append_bulk = value; return 0;
        case BARQKV_KNOB_ATTN_WIDE: g_knobs.attn_wide = value; return 0;
        case BARQKV_KNOB_LAYER_OVERLAP: g_knobs.layer_overlap = value; return 0;
        case BARQKV_KNOB_ATTN_PAGE_BOX: g_knobs.attn_page_box = value; return 0;
        case BARQKV_KNOB_ATTN_COMPACT: g_knobs.attn_compact = value; return 0;
        case BARQKV_KNOB_ATTN_PROBE: g_knobs.attn_probe = value; return 0;
        case BARQKV_KNOB_ZERO_AHEAD: g_knobs.zero_ahead = value; return 0;
        default: return fail(BARQKV_E_INVALID, "set_tuning: unknown knob");
    }
}
#endif

static int append_common(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                         const barqkv_block_table* table,
                         const int32_t* seq_start, const int32_t* cu_new,
                         int32_t n, int32_t tokens_per_entry, int32_t total_tokens,
                         const void* k_new, const void* v_new, const barqkv_rows_layout* new_rows,
                         int32_t* status, int32_t* work, int32_t flags, barqkv_stream_t stream,
                         int32_t layers, int64_t pool_layer_stride, int64_t new_layer_stride,
                         int32_t* zero_ahead = nullptr, bool rearm = true, bool* used_counters = nullptr) {
    if (used_counters) *used_counters = false;
    if (int rc = check_pool(pool)) return rc;
    if (flags & ~BARQKV_FLAG_DESC_STABLE) return fail(BARQKV_E_INVALID, "append: unknown flag");
    if (layers <= 0 || layers > 65535) return fail(BARQKV_E_INVALID, "append: layers must be in 1..65535");
    if (n < 0 || total_tokens < 0) return fail(BARQKV_E_INVALID, "append: negative batch size or token count");
    if (n == 0 || total_tokens == 0) return 0;
    if (int rc = check_table(table, n)) return rc;
    if (!k_pool || !v_pool || !k_new || !v_new || !seq_start || !new_rows)
        return fail(BARQKV_E_INVALID, "append: null pointer argument");
    if (!cu_new && (tokens_per_entry <= 0 || (long long)tokens_per_entry * n != total_tokens))
        return fail(BARQKV_E_INVALID, "append: without cu_new, total_tokens must equal n * tokens_per_entry");
    if (new_rows->packed && !cu_new && tokens_per_entry != 1)
        return fail(BARQKV_E_INVALID, "append: packed rows with more than one token per entry need cu_new");
    DeviceInfo* d = device_info();
    if (!d) return fail(BARQKV_E_LAUNCH, "no CUDA device is current");

    const long long e = pool->elem_bytes;
    AppendArgs a;
    memset(&a, 0, sizeof(a));
    a.k_pool = static_cast<unsigned char*>(k_pool);
    a.v_pool = static_cast<unsigned char*>(v_pool);
    a.k_new = static_cast<const unsigned char*>(k_new);
    a.v_new = static_cast<const unsigned char*>(v_new);
    a.tb = make_table(table, pool->num_pages);
    a.seq_start = seq_start;
    a.cu_new = cu_new;
    a.n = n;
    a.tokens_per_entry = tokens_per_entry;
    a.total_tokens = total_tokens;
    a.heads = pool->num_heads;
    a.page_size = pool->page_size;
    a.row_bytes = (int)(pool->head_dim * e);
    a.pool_head = pool->head_stride * e;
    a.pool_page = pool->page_stride * e;
    a.nr.seq = new_rows->seq_stride * e;
    a.nr.tok = new_rows->tok_stride * e;
    a.nr.head = new_rows->head_stride * e;
    a.nr.packed = new_rows->packed;
    a.status = status;

    a.pool_layer = pool_layer_stride * e;
    a.new_layer = new_layer_stride * e;
    a.early = (flags & BARQKV_FLAG_DESC_STABLE) && g_knobs.pdl != 0 ? 1 : 0;

    const int vec = vector_bytes(a.row_bytes, {a.pool_head, a.pool_page, a.nr.seq, a.nr.tok, a.nr.head,
                                               layers > 1 ? a.pool_layer : 0, layers > 1 ? a.new_layer : 0},
                                 {k_pool, v_pool, k_new, v_new});
    // Page-sized appends (on average at least a page per entry: prefill chunks) move whole pages with the
    // copy engine when the caller lends the two hand-out counters and the rows' layout allows one copy per
    // page: rows of a head adjacent in memory, or a packed token-major source a tensor map can describe.
    const long long page_bytes = (long long)a.page_size * a.row_bytes;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (work && g_knobs.append_bulk != 0 && vec == 16 && n <= kMaxEntries && 2 * page_bytes <= kBulkMaxStage &&
        total_tokens >= (long long)n * a.page_size) {
        const bool adjacent = a.nr.tok == a.row_bytes;
        const bool mappable = a.nr.packed && a.nr.seq == 0 && a.nr.tok > 0 && a.nr.head > 0 && a.nr.tok < (1LL << 40) &&
                              a.nr.head < (1LL << 40) && pool->head_dim <= 256 && a.page_size <= 256 &&
                              page_bytes % 128 == 0 && (layers == 1 || (a.new_layer > 0 && a.new_layer < (1LL << 40)));
        CUtensorMap map_k, map_v;
        memset(&map_k, 0, sizeof(map_k));
        memset(&map_v, 0, sizeof(map_v));
        bool tensor_load = false;
        if (!adjacent && mappable) {
            const long long lstride = layers > 1 ? a.new_layer : a.nr.tok;
            tensor_load = make_rows_map(&map_k, k_new, pool->elem_bytes, pool->head_dim, a.heads, a.nr.head, a.nr.tok,
                                        total_tokens, layers, lstride, a.page_size) &&
                          make_rows_map(&map_v, v_new, pool->elem_bytes, pool->head_dim, a.heads, a.nr.head, a.nr.tok,
                                        total_tokens, layers, lstride, a.page_size);
        }
        if (adjacent || tensor_load) {
            AppendBulkArgs x;
            memset(&x, 0, sizeof(x));
            x.work = work;
            x.zero_ahead = zero_ahead;
            x.rearm = rearm || !zero_ahead ? 1 : 0;
            x.tensor_load = tensor_load ? 1 : 0;
            x.layers = layers;
            x.wait_cycles = kWaitCycles;
            long long tiles_bound = ((long long)total_tokens + a.page_size - 1) / a.page_size + n;
            tiles_bound *= layers;
            if (tiles_bound <= 0x7fffffffLL) {
                int S = (int)(64 * 1024 / (2 * page_bytes));
                if (S > 8) S = 8;
                if (tiles_bound * a.heads < 96LL * d->sms && S > 4) S = 4;
                if (g_knobs.stages) S = g_knobs.stages;
                if (S < 3) S = 3;
                if (S > 32) S = 32;
                x.stages = S;
                const size_t smem = (size_t)S * 2 * page_bytes + (size_t)S * 8 /*bar*/ + (size_t)S * 8 /*slot dst*/ +
                                    2 * kGroup * 8 + 3 * kGroup * 4 + (size_t)S * 4 + (size_t)(n + 1) * 4 + 16;
                if ((long long)smem <= d->smem_optin) {
                    if (!d->append_attr_set.load(std::memory_order_acquire)) {
                        const cudaError_t ce = cudaFuncSetAttribute(append_bulk_kernel,
                                                                    cudaFuncAttributeMaxDynamicSharedMemorySize, d->smem_optin);
                        if (ce != cudaSuccess) return fail_cuda("append: cudaFuncSetAttribute", ce);
                        d->append_attr_set.store(true, std::memory_order_release);
                    }
                    int per_sm = (int)((220 * 1024) / (smem + 1024));
                    if (per_sm < 1) per_sm = 1;
                    if (per_sm > 8) per_sm = 8;
                    if (g_knobs.bulk_ctas_per_sm) per_sm = g_knobs.bulk_ctas_per_sm;
                    long long grid = (long long)d->sms * per_sm;
                    const long long want = (tiles_bound * a.heads + 1) / 2;      // at least two units per CTA
                    if (want < grid) grid = want < 1 ? 1 : want;
                    x.group_tiles = g_knobs.group_tiles ? g_knobs.group_tiles : (a.heads >= 8 ? 1 : 8 / a.heads);
                    if (x.group_tiles > kGroup) x.group_tiles = kGroup;
                    if (x.group_tiles < 1) x.group_tiles = 1;
                    const long long k = tiles_bound / (4 * grid);
                    x.first_group = (int)(k < 1 ? 1 : (k > x.group_tiles ? x.group_tiles : k));
                    cudaError_t ce = launch(append_bulk_kernel, dim3((unsigned)grid), dim3(32), smem, st, a.early != 0, a, x,
                                            map_k, map_v);
                    if (ce == cudaSuccess) ce = cudaGetLastError();
                    if (ce == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
                    if (ce == cudaSuccess && used_counters) *used_counters = true;
                    return ce == cudaSuccess ? 0 : fail_cuda("append launch", ce);
                }
            }
        }
    }

    int threads;
    // tile chosen as if the layers' tokens were one batch, so that the whole grid covers the machine
    long long work_tokens = (long long)total_tokens * layers;
    if (work_tokens > 0x7fffffffLL) work_tokens = 0x7fffffffLL;
    append_shape(d, (int)work_tokens, a.heads, a.row_bytes, vec, &a.tile, &threads);
    const dim3 grid((unsigned)((total_tokens + a.tile - 1) / a.tile), (unsigned)layers);
    return launch_append<false>(a, vec, grid, threads, static_cast<cudaStream_t>(stream));
}

int barqkv_append(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                  const barqkv_block_table* table,
                  const int32_t* seq_start, const int32_t* cu_new,
                  int32_t n, int32_t tokens_per_entry, int32_t total_tokens,
                  const void* k_new, const void* v_new, const barqkv_rows_layout* new_rows,
                  int32_t* status, int32_t* work, int32_t flags, barqkv_stream_t stream) {
    return append_common(pool, k_pool, v_pool, table, seq_start, cu_new, n, tokens_per_entry, total_tokens, k_new, v_new,
                         new_rows, status, work, flags, stream, 1, 0, 0);
}

int barqkv_append_layers(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                         int32_t layers, int64_t pool_layer_stride,
                         const barqkv_block_table* table,
                         const int32_t* seq_start, const int32_t* cu_new,
                         int32_t n, int32_t tokens_per_entry, int32_t total_tokens,
                         const void* k_new, const void* v_new, const barqkv_rows_layout* new_rows,
                         int64_t new_layer_stride, int32_t* status, int32_t* work, int32_t flags, barqkv_stream_t stream) {
    return append_common(pool, k_pool, v_pool, table, seq_start, cu_new, n, tokens_per_entry, total_tokens, k_new, v_new,
                         new_rows, status, work, flags, stream, layers, pool_layer_stride, new_layer_stride);
}

int barqkv_append_each_layer(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                             int32_t layers, int64_t pool_layer_stride,
                             const barqkv_block_table* table,
                             const int32_t* seq_start, const int32_t* cu_new,
                             int32_t n, int32_t tokens_per_entry, int32_t total_tokens,
                             const void* const* k_new, const void* const* v_new, const barqkv_rows_layout* new_rows,
                             int32_t* status, int32_t* work, int32_t flags, barqkv_stream_t stream) {
    if (layers <= 0 || layers > 65535) return fail(BARQKV_E_INVALID, "append_each_layer: bad layer count");
    if (pool_layer_stride < 0) return fail(BARQKV_E_INVALID, "append_each_layer: negative layer stride");
    if (!k_new || !v_new || !pool || !k_pool || !v_pool) return fail(BARQKV_E_INVALID, "append_each_layer: null pointer argument");
    if (flags & ~BARQKV_FLAG_DESC_STABLE) return fail(BARQKV_E_INVALID, "append_each_layer: unknown flag");
    const long long e = pool->elem_bytes;
    const bool chained = work && g_knobs.zero_ahead != 0;
    bool pending = false;       // the launch before left its counters for its successor to clear
    int rc = 0;
    for (int l = 0; l < layers; ++l) {
        // One launch per layer.  From the second on each is a programmatic dependent of the one before, whose
        // batch description it shares; the launches alternate between the two counter pairs of `work`, clear
        // each other's, and only the last one counts its finished CTAs to clear its own.
        unsigned char* kp = static_cast<unsigned char*>(k_pool) + (long long)l * pool_layer_stride * e;
        unsigned char* vp = static_cast<unsigned char*>(v_pool) + (long long)l * pool_layer_stride * e;
        const bool last = l == layers - 1;
        bool counters = false;
        rc = append_common(pool, kp, vp, table, seq_start, cu_new, n, tokens_per_entry, total_tokens, k_new[l], v_new[l],
                           new_rows, status, work ? work + 2 * (l & 1) : nullptr, l > 0 ? BARQKV_FLAG_DESC_STABLE : flags,
                           stream, 1, 0, 0, chained ? work + 2 * ((l + 1) & 1) : nullptr, last, &counters);
        if (rc) break;
        if (counters) {
            pending = chained && !last;                            // and it cleared its predecessor's pair
        } else if (pending) {
            // this layer's rows took the kernel without counters (another alignment): nobody cleared for the one before
            cudaMemsetAsync(work, 0, 4 * sizeof(int32_t), static_cast<cudaStream_t>(stream));
            pending = false;
        }
    }
    // an error broke the chain off: the launch that left its counters to a successor has none
    if (pending) cudaMemsetAsync(work, 0, 4 * sizeof(int32_t), static_cast<cudaStream_t>(stream));
    return rc;
}

int barqkv_append_rope(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                       const barqkv_block_table* table,
                       const int32_t* seq_start, const int32_t* cu_new,
                       int32_t n, int32_t tokens_per_entry, int32_t total_tokens,
                       const void* k_new, const void* v_new, const barqkv_rows_layout* new_rows,
                       const void* cos, const void* sin, int64_t rope_tok_stride, int32_t dtype,
                       int32_t* status, barqkv_stream_t stream) {
    if (int rc = check_pool(pool)) return rc;
    if (n < 0 || total_tokens < 0) return fail(BARQKV_E_INVALID, "append_rope: negative batch size or token count");
    if (n == 0 || total_tokens == 0) return 0;
    if (int rc = check_table(table, n)) return rc;
    if (!k_pool || !v_pool || !k_new || !v_new || !seq_start || !new_rows || !cos || !sin)
        return fail(BARQKV_E_INVALID, "append_rope: null pointer argument");
    if (!cu_new && (tokens_per_entry <= 0 || (long long)tokens_per_entry * n != total_tokens))
        return fail(BARQKV_E_INVALID, "append_rope: without cu_new, total_tokens must equal n * tokens_per_entry");
    if (new_rows->packed && !cu_new && tokens_per_entry != 1)
        return fail(BARQKV_E_INVALID, "append_rope: packed rows with more than one token per entry need cu_new");
    const int want_bytes = dtype == BARQKV_DTYPE_F32 ? 4 : 2;
    if (dtype < BARQKV_DTYPE_BF16 || dtype > BARQKV_DTYPE_F32 || pool->elem_bytes != want_bytes)
        return fail(BARQKV_E_INVALID, "append_rope: dtype must be bf16, fp16 or fp32 and match elem_bytes");
    DeviceInfo* d = device_info();
    if (!d) return fail(BARQKV_E_LAUNCH, "no CUDA device is current");

    const long long e = pool->elem_bytes;
    AppendArgs a;
    memset(&a, 0, sizeof(a));
    a.k_pool = static_cast<unsigned char*>(k_pool);
    a.v_pool = static_cast<unsigned char*>(v_pool);
    a.k_new = static_cast<const unsigned char*>(k_new);
    a.v_new = static_cast<const unsigned char*>(v_new);
    a.tb = make_table(table, pool->num_pages);
    a.seq_start = seq_start;
    a.cu_new = cu_new;
    a.n = n;
    a.tokens_per_entry = tokens_per_entry;
    a.total_tokens = total_tokens;
    a.heads = pool->num_heads;
    a.page_size = pool->page_size;
    a.row_bytes = (int)(pool->head_dim * e);
    a.pool_head = pool->head_stride * e;
    a.pool_page = pool->page_stride * e;
    a.nr.seq = new_rows->seq_stride * e;
    a.nr.tok = new_rows->tok_stride * e;
    a.nr.head = new_rows->head_stride * e;
    a.nr.packed = new_rows->packed;
    a.status = status;
    RopeArgs rp;
    rp.cos = static_cast<const unsigned char*>(cos);
    rp.sin = static_cast<const unsigned char*>(sin);
    rp.tok = rope_tok_stride * e;
    const int vec = vector_bytes(a.row_bytes, {a.pool_head, a.pool_page, a.nr.seq, a.nr.tok, a.nr.head, rp.tok},
                                 {k_pool, v_pool, k_new, v_new, cos, sin});
    if (vec != 16 || (a.row_bytes / 16) % 2)
        return fail(BARQKV_E_INVALID, "append_rope: rows, strides and pointers must be 16-byte aligned and a half row "
                                      "a whole number of 16-byte vectors");
    int threads;
    append_shape(d, total_tokens, a.heads, a.row_bytes, 16, &a.tile, &threads);
    const int grid = (total_tokens + a.tile - 1) / a.tile;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case BARQKV_DTYPE_BF16: append_rope_kernel<__nv_bfloat16><<<grid, kAppendThreads, 0, st>>>(a, rp); break;
        case BARQKV_DTYPE_F16: append_rope_kernel<__half><<<grid, kAppendThreads, 0, st>>>(a, rp); break;
        default: append_rope_kernel<float><<<grid, kAppendThreads, 0, st>>>(a, rp); break;
    }
    const cudaError_t ce = cudaGetLastError();
    if (ce == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    return ce == cudaSuccess ? 0 : fail_cuda("append_rope launch", ce);
}

int barqkv_upload(void* dst_device, const void* src_host, int64_t bytes, barqkv_stream_t stream) {
    if (bytes < 0 || (bytes && (!dst_device || !src_host))) return fail(BARQKV_E_INVALID, "upload: bad arguments");
    if (bytes == 0) return 0;
    const cudaError_t e = cudaMemcpyAsync(dst_device, src_host, (size_t)bytes, cudaMemcpyHostToDevice,
                                          static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : fail_cuda("upload", e);
}

int barqkv_max_length(const int32_t* seq_lens, int32_t n, int32_t* max_out, barqkv_stream_t stream) {
    if (n < 0 || !max_out || (n && !seq_lens)) return fail(BARQKV_E_INVALID, "max_length: bad arguments");
    *max_out = 0;
    if (n == 0) return 0;
    constexpr int kChunk = 8192;
    static thread_local int32_t host[kChunk];
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t m = INT32_MIN;
    for (int at = 0; at < n; at += kChunk) {
        const int count = n - at < kChunk ? n - at : kChunk;
        cudaError_t e = cudaMemcpyAsync(host, seq_lens + at, (size_t)count * 4, cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) return fail_cuda("max_length", e);
        for (int i = 0; i < count; ++i) m = host[i] > m ? host[i] : m;
    }
    *max_out = m;
    return 0;
}

int barqkv_table_scatter(int32_t* table, int64_t table_words, const int32_t* pairs, int32_t n, barqkv_stream_t stream) {
    if (n < 0 || (n && (!table || !pairs))) return fail(BARQKV_E_INVALID, "table_scatter: bad arguments");
    if (n == 0) return 0;
    table_scatter_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(table, pairs, n, table_words);
    const cudaError_t ce = cudaGetLastError();
    if (ce == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    return ce == cudaSuccess ? 0 : fail_cuda("table_scatter launch", ce);
}

int barqkv_copy_pages(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                      int32_t layers, int64_t pool_layer_stride,
                      const int32_t* src_pages, const int32_t* dst_pages, int32_t n,
                      int32_t* status, barqkv_stream_t stream) {
    if (int rc = check_pool(pool)) return rc;
    if (n < 0 || layers <= 0 || layers > 65535) return fail(BARQKV_E_INVALID, "copy_pages: bad page or layer count");
    if (n == 0) return 0;
    if (!k_pool || !v_pool || !src_pages || !dst_pages) return fail(BARQKV_E_INVALID, "copy_pages: null pointer argument");
    if ((long long)n * pool->num_heads > 0x7fffffffLL) return fail(BARQKV_E_LIMIT, "copy_pages: too many pages in one call");
    const long long e = pool->elem_bytes;
    CopyArgs a;
    memset(&a, 0, sizeof(a));
    a.k_pool = static_cast<unsigned char*>(k_pool);
    a.v_pool = static_cast<unsigned char*>(v_pool);
    a.src = src_pages;
    a.dst = dst_pages;
    a.n = n;
    a.heads = pool->num_heads;
    a.num_pages = pool->num_pages;
    a.page_bytes = (int)(pool->page_size * pool->head_dim * e);
    a.pool_head = pool->head_stride * e;
    a.pool_page = pool->page_stride * e;
    a.pool_layer = pool_layer_stride * e;
    a.status = status;
    const int vec = vector_bytes(a.page_bytes, {a.pool_head, a.pool_page, layers > 1 ? a.pool_layer : 0}, {k_pool, v_pool});
    const dim3 grid((unsigned)(n * a.heads), (unsigned)layers, 2);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (vec) {
        case 16: copy_pages_kernel<uint4><<<grid, 128, 0, st>>>(a); break;
        case 8: copy_pages_kernel<uint2><<<grid, 128, 0, st>>>(a); break;
        case 4: copy_pages_kernel<uint32_t><<<grid, 128, 0, st>>>(a); break;
        case 2: copy_pages_kernel<uint16_t><<<grid, 128, 0, st>>>(a); break;
        default: copy_pages_kernel<uint8_t><<<grid, 128, 0, st>>>(a); break;
    }
    const cudaError_t ce = cudaGetLastError();
    if (ce == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    return ce == cudaSuccess ? 0 : fail_cuda("copy_pages launch", ce);
}

int barqkv_append_legacy(void* key_cache, void* value_cache, int32_t* seq_lens,
                         const void* k_new, const void* v_new, const barqkv_rows_layout* new_rows,
                         int32_t batch, int32_t max_batch, int32_t heads, int32_t tokens,
                         int32_t head_dim, int32_t max_blocks, int32_t page_size, int32_t elem_bytes,
                         int32_t* ticket, int32_t* status, barqkv_stream_t stream) {
    if (!key_cache || !value_cache || !seq_lens || !k_new || !v_new || !new_rows || !ticket)
        return fail(BARQKV_E_INVALID, "append_legacy: null pointer argument");
    if (batch < 0 || tokens < 0 || max_batch <= 0 || heads <= 0 || head_dim <= 0 || max_blocks <= 0 || page_size <= 0)
        return fail(BARQKV_E_INVALID, "append_legacy: sizes must be positive");
    if (batch > max_batch) return fail(BARQKV_E_INVALID, "key_cache batch dimension is too small");
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8)
        return fail(BARQKV_E_INVALID, "append_legacy: elem_bytes must be 1, 2, 4 or 8");
    if (new_rows->packed) return fail(BARQKV_E_INVALID, "append_legacy: new rows must be batched, not packed");
    if ((long long)max_batch * heads * max_blocks > 0x7fffffffLL || (long long)batch * tokens > 0x7fffffffLL)
        return fail(BARQKV_E_LIMIT, "append_legacy: cache has more than 2^31 pages or the call more than 2^31 tokens");
    if (batch == 0 || tokens == 0) return 0;
    DeviceInfo* d = device_info();
    if (!d) return fail(BARQKV_E_LAUNCH, "no CUDA device is current");

    const long long e = elem_bytes;
    AppendArgs a;
    memset(&a, 0, sizeof(a));
    a.k_pool = static_cast<unsigned char*>(key_cache);
    a.v_pool = static_cast<unsigned char*>(value_cache);
    a.k_new = static_cast<const unsigned char*>(k_new);
    a.v_new = static_cast<const unsigned char*>(v_new);
    a.tb.table = nullptr;
    a.tb.slots = nullptr;
    a.tb.rows = max_batch;
    a.tb.stride = max_blocks;
    a.tb.implicit = heads * max_blocks;
    a.tb.num_pages = max_batch * heads * max_blocks;
    a.seq_start = seq_lens;
    a.cu_new = nullptr;
    a.n = batch;
    a.tokens_per_entry = tokens;
    a.total_tokens = batch * tokens;
    a.heads = heads;
    a.page_size = page_size;
    a.row_bytes = (int)(head_dim * e);
    a.pool_page = (long long)page_size * head_dim * e;
    a.pool_head = (long long)max_blocks * a.pool_page;
    a.nr.seq = new_rows->seq_stride * e;
    a.nr.tok = new_rows->tok_stride * e;
    a.nr.head = new_rows->head_stride * e;
    a.nr.packed = 0;
    a.seq_lens_rw = seq_lens;
    a.ticket = ticket;
    a.capacity = max_blocks * page_size;
    a.status = status;

    const int vec = vector_bytes(a.row_bytes, {a.pool_head, a.pool_page, a.nr.seq, a.nr.tok, a.nr.head},
                                 {key_cache, value_cache, k_new, v_new});
    int threads;
    append_shape(d, a.total_tokens, heads, a.row_bytes, vec, &a.tile, &threads);
    const dim3 grid((unsigned)((a.total_tokens + a.tile - 1) / a.tile));
    return launch_append<true>(a, vec, grid, threads, static_cast<cudaStream_t>(stream));
}

// New rows joining a gather (barqkv_update); null k_new = plain gather.
struct FusedRows {
    const void* k_new;
    const void* v_new;
    const barqkv_rows_layout* rows;
    const int32_t* cu_new;
    int tokens_per_entry;
};
constexpr int kNotFusable = 1;   // gather_common: the fused form cannot run on these arguments
// Several layers' pools gathered by one launch (barqkv_gather_layers); null = one layer.
struct LayerSpan {
    int layers;
    long long pool_stride, out_stride;   // elements
};

// How a gather is launched, beyond what its arguments describe.
struct LaunchOpts {
    bool after_own_kernel = false;   // the kernel before this one in the stream is this library's gather over the
                                     // same, unchanged batch description and block table: launch as its programmatic
                                     // dependent and let the prologue overlap its tail
    long long wait_cycles = kWaitCycles;
    int extra_tx = 0;                // self-test: make every stage wait for bytes that never come
    int max_ctas = 0;                // self-test: cap of the grid (0 = none)
    bool validate_only = false;      // check the arguments, enqueue nothing
    int32_t* zero_ahead = nullptr;   // chained launches: the counter pair of the launch before and after this one, which
                                     // this launch clears; with it and rearm = false nobody counts finished CTAs
    bool rearm = true;               // the launch leaves its own counter pair zero
};

static int gather_common(const barqkv_pool_layout* pool, const void* k_pool, const void* v_pool,
                         const barqkv_block_table* table,
                         const int32_t* seq_lens, const int32_t* cu_out, int32_t n,
                         int64_t total_tokens_hint,
                         void* k_out, void* v_out, const barqkv_rows_layout* out_rows,
                         int32_t mode, int32_t* status, int32_t* work, barqkv_stream_t stream,
                         const FusedRows* fused, const LayerSpan* span = nullptr, const LaunchOpts& opts = LaunchOpts()) {
    if (int rc = check_pool(pool)) return rc;
    if (n < 0) return fail(BARQKV_E_INVALID, "gather: negative batch size");
    if (n == 0) return 0;
    if (n > kMaxEntries) return fail(BARQKV_E_LIMIT, "gather: more than 8192 sequences in one call; split the batch");
    if (int rc = check_table(table, n)) return rc;
    if (!k_pool || !v_pool || !k_out || !v_out || !seq_lens || !out_rows)
        return fail(BARQKV_E_INVALID, "gather: null pointer argument");
    if (out_rows->packed && !cu_out) return fail(BARQKV_E_INVALID, "gather: packed output needs cu_out");
    const bool stable = (mode & BARQKV_FLAG_DESC_STABLE) != 0;
    mode &= ~BARQKV_FLAG_DESC_STABLE;
    if (mode < BARQKV_MODE_AUTO || mode > BARQKV_MODE_BULK) return fail(BARQKV_E_INVALID, "gather: unknown mode");
    DeviceInfo* d = device_info();
    if (!d) return fail(BARQKV_E_LAUNCH, "no CUDA device is current");
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    const long long e = pool->elem_bytes;
    GatherArgs a;
    memset(&a, 0, sizeof(a));
    a.k_pool = static_cast<const unsigned char*>(k_pool);
    a.v_pool = static_cast<const unsigned char*>(v_pool);
    a.k_out = static_cast<unsigned char*>(k_out);
    a.v_out = static_cast<unsigned char*>(v_out);
    a.tb = make_table(table, pool->num_pages);
    a.seq_lens = seq_lens;
    a.cu_out = cu_out;
    a.n = n;
    a.heads = pool->num_heads;
    a.page_size = pool->page_size;
    a.row_bytes = (int)(pool->head_dim * e);
    a.pool_head = pool->head_stride * e;
    a.pool_page = pool->page_stride * e;
    a.orow.seq = out_rows->seq_stride * e;
    a.orow.tok = out_rows->tok_stride * e;
    a.orow.head = out_rows->head_stride * e;
    a.orow.packed = out_rows->packed;
    a.status = status;
    a.interleave = g_knobs.interleave < 0 ? 0 : g_knobs.interleave;
    a.work = g_knobs.static_shares ? nullptr : work;
    a.zero_ahead = a.work ? opts.zero_ahead : nullptr;
    a.rearm = opts.rearm || !a.zero_ahead ? 1 : 0;
    // tiles per hand-out: about 4 (page, head) units, i.e. 32 KiB of K and V, per atomic fetch
    a.group_tiles = g_knobs.group_tiles ? g_knobs.group_tiles : (a.heads >= 4 ? (a.heads >= 8 ? 1 : 2) : 4);
    if (a.group_tiles > kGroup) a.group_tiles = kGroup;
    if (a.group_tiles < 1) a.group_tiles = 1;
    a.static_permille = g_knobs.static_permille >= 0 ? g_knobs.static_permille : 0;
    a.wait_cycles = opts.wait_cycles;
    a.extra_tx = opts.extra_tx;
    a.layers = 1;
    if (span) {
        a.layers = span->layers;
        a.pool_layer = span->pool_stride * e;
        a.out_layer = span->out_stride * e;
    }

    int vec = vector_bytes(a.row_bytes, {a.pool_head, a.pool_page, a.orow.seq, a.orow.tok, a.orow.head,
                                         a.pool_layer, a.out_layer},
                           {k_pool, v_pool, k_out, v_out});
    if (fused) {
        a.k_new = static_cast<const unsigned char*>(fused->k_new);
        a.v_new = static_cast<const unsigned char*>(fused->v_new);
        a.k_pool_w = const_cast<unsigned char*>(a.k_pool);
        a.v_pool_w = const_cast<unsigned char*>(a.v_pool);
        a.cu_new = fused->cu_new;
        a.tokens_per_entry = fused->tokens_per_entry;
        a.nr.seq = fused->rows->seq_stride * e;
        a.nr.tok = fused->rows->tok_stride * e;
        a.nr.head = fused->rows->head_stride * e;
        a.nr.packed = fused->rows->packed;
        const int vec_new = vector_bytes(a.row_bytes, {a.nr.seq, a.nr.tok, a.nr.head}, {fused->k_new, fused->v_new});
        if (vec_new < vec) vec = vec_new;
    }
    const long long page_bytes = (long long)a.page_size * a.row_bytes;
    const bool bulk_ok = vec == 16 && 2 * page_bytes <= kBulkMaxStage;
    if (fused && (!bulk_ok || mode == BARQKV_MODE_VECTOR)) return kNotFusable;
    if (mode == BARQKV_MODE_BULK && !bulk_ok)
        return fail(BARQKV_E_INVALID, "gather: bulk mode needs 16-byte aligned rows and strides and pages of at most 16 KiB");
    const bool use_bulk = mode == BARQKV_MODE_BULK || (mode == BARQKV_MODE_AUTO && bulk_ok);

    // Upper bound of (sequence, page) tiles, to keep tiny gathers from launching a full machine.
    long long tiles_bound = 0x7fffffffLL;
    if (total_tokens_hint > 0) tiles_bound = (total_tokens_hint + a.page_size - 1) / a.page_size + n;
    if (a.layers > 1) {
        if (!use_bulk) return fail(BARQKV_E_INVALID, "gather_layers: needs the bulk path (16-byte aligned rows and strides)");
        if (total_tokens_hint <= 0) return fail(BARQKV_E_INVALID, "gather_layers: needs the total number of tokens");
        tiles_bound *= a.layers;
        if (tiles_bound > 0x7fffffffLL) return fail(BARQKV_E_LIMIT, "gather_layers: too many (layer, sequence, page) tiles");
    }

    if (use_bulk) {
        int S = (int)(64 * 1024 / (2 * page_bytes));
        if (S > 8) S = 8;
        // A launch with few units (a single KV head per GPU) is dominated by filling and draining the
        // rings: half the depth, twice the CTAs.
        if (tiles_bound * a.heads < 96LL * d->sms && S > 4) S = 4;
        if (g_knobs.stages) S = g_knobs.stages;
        if (S < 3) S = 3;
        if (S > 32) S = 32;
        a.stages = S;
        const size_t smem = (size_t)S * 2 * page_bytes + (size_t)S * 8 /*bar*/ + (size_t)S * 16 /*slot dst, pool*/ +
                            3 * kGroup * 8 + 2 * kGroup * 4 + (size_t)S * 16 + 4 + (size_t)(n + 1) * 4;
        if ((long long)smem > d->smem_optin)
            return fail(BARQKV_E_LIMIT, "gather: bulk pipeline does not fit in shared memory");
        if (!d->bulk_attr_set.load(std::memory_order_acquire)) {
            const cudaError_t ce = cudaFuncSetAttribute(gather_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                        d->smem_optin);
            if (ce != cudaSuccess) return fail_cuda("gather: cudaFuncSetAttribute", ce);
            d->bulk_attr_set.store(true, std::memory_order_release);
        }
        int per_sm = (int)((220 * 1024) / (smem + 1024));
        if (per_sm < 1) per_sm = 1;
        if (per_sm > 8) per_sm = 8;
        if (g_knobs.bulk_ctas_per_sm) per_sm = g_knobs.bulk_ctas_per_sm;
        long long grid = (long long)d->sms * per_sm;
        const long long units_bound = tiles_bound * a.heads;
        const long long want = (units_bound + 2 * S - 1) / (2 * S);   // at least two ring rounds per CTA
        if (want < grid) grid = want < 1 ? 1 : want;
        {
            // half the size the guided hand-out would start with: tiles_bound is an upper bound, and a
            // first group sized from a loose one must not starve the other CTAs
            long long k = tiles_bound / (4 * grid);
            a.first_group = (int)(k < 1 ? 1 : (k > a.group_tiles ? a.group_tiles : k));
        }
        // A token-major output (rows of a page are head-stride apart) takes one tiled TMA store per full
        // page instead of page_size row copies, when the output is packed and its shape fits a tensor map.
        CUtensorMap map_k, map_v;
        memset(&map_k, 0, sizeof(map_k));
        memset(&map_v, 0, sizeof(map_v));
        if (a.layers == 1 && a.orow.tok != a.row_bytes && a.orow.seq == 0 && a.orow.packed && g_knobs.tensor_store != 0 &&
            pool->head_dim <= 256 && a.page_size <= 256 && page_bytes % 128 == 0 && a.orow.tok > 0 && a.orow.head > 0 &&
            a.orow.tok < (1LL << 40) && a.orow.head < (1LL << 40)) {
            const long long tokens = 0x7fffffffLL;      // full pages never reach past their sequence; no clipping needed
            a.tensor_store = make_out_map(&map_k, k_out, pool->elem_bytes, pool->head_dim, a.heads, a.orow.head,
                                          a.orow.tok, tokens, a.page_size) &&
                             make_out_map(&map_v, v_out, pool->elem_bytes, pool->head_dim, a.heads, a.orow.head,
                                          a.orow.tok, tokens, a.page_size);
        }
        if (opts.max_ctas > 0 && grid > opts.max_ctas) grid = opts.max_ctas;
        if (opts.validate_only) return 0;
        const bool dependent = (opts.after_own_kernel || stable) && g_knobs.pdl != 0 && a.work;
        a.early = dependent ? 1 : 0;
        const cudaError_t le = launch(gather_bulk_kernel, dim3((unsigned)grid), dim3(32), smem, st, dependent, a, map_k, map_v);
        if (le != cudaSuccess) return fail_cuda("gather launch", le);
    } else {
        const size_t smem = (size_t)(n + 1) * 4;
        long long grid = (long long)d->sms * (g_knobs.vector_ctas_per_sm ? g_knobs.vector_ctas_per_sm : 8);
        const long long want = (tiles_bound + 3) / 4;
        if (want < grid) grid = want < 1 ? 1 : want;
        if (opts.validate_only) return 0;
        switch (vec) {
            case 16: gather_vector_kernel<uint4><<<(int)grid, kGatherThreads, smem, st>>>(a); break;
            case 8: gather_vector_kernel<uint2><<<(int)grid, kGatherThreads, smem, st>>>(a); break;
            case 4: gather_vector_kernel<uint32_t><<<(int)grid, kGatherThreads, smem, st>>>(a); break;
            case 2: gather_vector_kernel<uint16_t><<<(int)grid, kGatherThreads, smem, st>>>(a); break;
            default: gather_vector_kernel<uint8_t><<<(int)grid, kGatherThreads, smem, st>>>(a); break;
        }
    }
    const cudaError_t ce = cudaGetLastError();
    if (ce == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    return ce == cudaSuccess ? 0 : fail_cuda("gather launch", ce);
}

int barqkv_gather(const barqkv_pool_layout* pool, const void* k_pool, const void* v_pool,
                  const barqkv_block_table* table,
                  const int32_t* seq_lens, const int32_t* cu_out, int32_t n,
                  int64_t total_tokens_hint,
                  void* k_out, void* v_out, const barqkv_rows_layout* out_rows,
                  int32_t mode, int32_t* status, int32_t* work, barqkv_stream_t stream) {
    return gather_common(pool, k_pool, v_pool, table, seq_lens, cu_out, n, total_tokens_hint, k_out, v_out, out_rows,
                         mode, status, work, stream, nullptr);
}

int barqkv_gather_layers(const barqkv_pool_layout* pool, const void* k_pool, const void* v_pool,
                         int32_t layers, int64_t pool_layer_stride, const barqkv_block_table* table,
                         const int32_t* seq_lens, const int32_t* cu_out, int32_t n, int64_t total_tokens,
                         void* k_out, void* v_out, const barqkv_rows_layout* out_rows, int64_t out_layer_stride,
                         int32_t* status, int32_t* work, barqkv_stream_t stream) {
    if (layers <= 0 || layers > 65535) return fail(BARQKV_E_INVALID, "gather_layers: bad layer count");
    if (pool_layer_stride < 0 || out_layer_stride < 0) return fail(BARQKV_E_INVALID, "gather_layers: negative layer stride");
    if (!work) return fail(BARQKV_E_INVALID, "gather_layers: needs the two-word work buffer");
    const LayerSpan span{layers, pool_layer_stride, out_layer_stride};
    return gather_common(pool, k_pool, v_pool, table, seq_lens, cu_out, n, total_tokens, k_out, v_out, out_rows,
                         BARQKV_MODE_BULK, status, work, stream, nullptr, layers > 1 ? &span : nullptr);
}

int barqkv_update(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                  const barqkv_block_table* table,
                  const int32_t* seq_start, const int32_t* cu_new,
                  int32_t n, int32_t tokens_per_entry, int32_t total_new_tokens,
                  const void* k_new, const void* v_new, const barqkv_rows_layout* new_rows,
                  const int32_t* cu_out, int64_t total_tokens_hint,
                  void* k_out, void* v_out, const barqkv_rows_layout* out_rows,
                  int32_t mode, int32_t* status, int32_t* work, const int32_t* seq_lens_after,
                  barqkv_stream_t stream) {
    if (n < 0 || total_new_tokens < 0) return fail(BARQKV_E_INVALID, "update: negative batch size or token count");
    if (n == 0) return 0;
    if (int rc = check_pool(pool)) return rc;
    if (!seq_start || !new_rows || (total_new_tokens && (!k_new || !v_new)))
        return fail(BARQKV_E_INVALID, "update: null pointer argument");
    if (!cu_new && (tokens_per_entry < 0 || (long long)tokens_per_entry * n != total_new_tokens))
        return fail(BARQKV_E_INVALID, "update: without cu_new, total_new_tokens must equal n * tokens_per_entry");
    if (new_rows->packed && !cu_new && tokens_per_entry > 1)
        return fail(BARQKV_E_INVALID, "update: packed rows with more than one token per entry need cu_new");
    // One launch when the copy engine path applies and the append is small next to the gather
    // (decode, short chunks); otherwise the two kernels run back to back with the same result.
    if (pool && total_new_tokens > 0 && total_new_tokens <= (long long)n * pool->page_size) {
        const FusedRows fused = {k_new, v_new, new_rows, cu_new, tokens_per_entry};
        const int rc = gather_common(pool, k_pool, v_pool, table, seq_start, cu_out, n, total_tokens_hint, k_out, v_out,
                                     out_rows, mode, status, work, stream, &fused);
        if (rc != kNotFusable) return rc;
    }
    if (!seq_lens_after)
        return fail(BARQKV_E_INVALID, "update: this call cannot run as one launch; pass seq_lens_after (lengths after "
                                      "the append, device int32[n]) so that it can run as append + gather");
    if (total_new_tokens) {
        if (int rc = barqkv_append(pool, k_pool, v_pool, table, seq_start, cu_new, n, tokens_per_entry, total_new_tokens,
                                   k_new, v_new, new_rows, status, work, 0, stream))
            return rc;
    }
    // two kernels that share `work`: the gather must not start taking pages while the append still does
    return barqkv_gather(pool, k_pool, v_pool, table, seq_lens_after, cu_out, n, total_tokens_hint, k_out, v_out,
                         out_rows, mode & ~BARQKV_FLAG_DESC_STABLE, status, work, stream);
}

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
                         barqkv_stream_t stream) {
    if (layers <= 0 || layers > 65535) return fail(BARQKV_E_INVALID, "update_layers: bad layer count");
    if (num_out <= 0 || !k_out || !v_out) return fail(BARQKV_E_INVALID, "update_layers: needs at least one output pair");
    if (pool_layer_stride < 0 || new_layer_stride < 0) return fail(BARQKV_E_INVALID, "update_layers: negative layer stride");
    if (n < 0 || total_new_tokens < 0) return fail(BARQKV_E_INVALID, "update_layers: negative batch size or token count");
    if (n == 0) return 0;
    if (int rc = check_pool(pool)) return rc;
    if (!k_pool || !v_pool || !seq_start || (total_new_tokens && (!k_new || !v_new || !new_rows)))
        return fail(BARQKV_E_INVALID, "update_layers: null pointer argument");
    if (!cu_new && (tokens_per_entry < 0 || (long long)tokens_per_entry * n != total_new_tokens))
        return fail(BARQKV_E_INVALID, "update_layers: without cu_new, total_new_tokens must equal n * tokens_per_entry");
    if (total_new_tokens && new_rows->packed && !cu_new && tokens_per_entry > 1)
        return fail(BARQKV_E_INVALID, "update_layers: packed rows with more than one token per entry need cu_new");
    const long long e = pool->elem_bytes;
    const bool one_stream = (mode & BARQKV_FLAG_ONE_STREAM) != 0;
    mode &= ~(BARQKV_FLAG_DESC_STABLE | BARQKV_FLAG_ONE_STREAM);   // the first layer waits for whatever precedes it; the rest are chained here
    // nothing to append: the same chain of launches, each a plain gather (seq_start then holds the lengths)
    const bool only_gather = total_new_tokens == 0;
    const bool try_fused = only_gather || total_new_tokens <= (long long)n * pool->page_size;
    bool fused_ok = try_fused;

    // Two layers next to one another touch nothing in common when they write to different outputs: each reads
    // and writes its own layer's pools.  Even layers are then issued on the caller's stream and odd layers on a
    // second stream forked from it, each stream a chain of programmatic dependents (layer l behind layer l - 2,
    // the layer whose output buffer it may reuse), and the two chains run side by side: the first blocks of one
    // layer take the SMs that the last blocks of the layer before leave, so no layer pays for an empty machine
    // at its start or its end.  An even and an odd layer share an output only if num_out is odd and smaller than
    // `layers`; such calls, and calls whose outputs are not all distinct, keep to one stream.
    cudaStream_t main_stream = static_cast<cudaStream_t>(stream);
    DeviceInfo* dev = device_info();
    bool overlap = !one_stream && try_fused && layers >= 2 && work && dev && g_knobs.layer_overlap != 0 && g_knobs.pdl != 0 &&
                   (num_out % 2 == 0 || num_out >= layers) && num_out <= 128;
    for (int i = 0; overlap && i < num_out; ++i)
        for (int j = 0; j < i; ++j)
            if (k_out[i] == k_out[j] || v_out[i] == v_out[j] || k_out[i] == v_out[j] || v_out[i] == k_out[j]) overlap = false;
    // Launches may leave their counters to their successor only if every layer takes the same kernel: the one
    // with counters needs 16-byte aligned rows, so the layers' pools and outputs must agree in that.
    bool same_kernel = layers == 1 || multiple(pool_layer_stride * e, 16);
    for (int i = 1; same_kernel && i < num_out; ++i)
        same_kernel = aligned(k_out[i], 16) == aligned(k_out[0], 16) && aligned(v_out[i], 16) == aligned(v_out[0], 16);
    if (total_new_tokens) same_kernel = same_kernel && multiple(new_layer_stride * e, 16);
    std::unique_lock<std::mutex> lane_lock;
    if (overlap) {
        lane_lock = std::unique_lock<std::mutex>(dev->lane_mu);
        overlap = second_stream(dev, main_stream) &&
                  cudaEventRecord(dev->lane_fork, main_stream) == cudaSuccess &&
                  cudaStreamWaitEvent(dev->lane, dev->lane_fork, 0) == cudaSuccess;
        if (!overlap) {
            cudaGetLastError();
            lane_lock.unlock();
        }
    }
    // whatever happens below, the second stream is joined back before the call returns
    bool chained_pairs = false;      // some launch left clearing its counter pair to its successor
    auto done = [&](int rc) {
        if (rc != 0 && chained_pairs) {
            // the chain broke off: the successor that would have cleared the last launch's pair never came
            if (overlap) cudaMemsetAsync(work, 0, 8 * sizeof(int32_t), dev->lane);
            cudaMemsetAsync(work, 0, 8 * sizeof(int32_t), main_stream);
        }
        if (overlap && (cudaEventRecord(dev->lane_join, dev->lane) != cudaSuccess ||
                        cudaStreamWaitEvent(main_stream, dev->lane_join, 0) != cudaSuccess) && rc == 0)
            rc = fail(BARQKV_E_LAUNCH, "update_layers: could not join the second stream");
        return rc;
    };
    for (int l = 0; l < layers; ++l) {
        unsigned char* kp = static_cast<unsigned char*>(k_pool) + (long long)l * pool_layer_stride * e;
        unsigned char* vp = static_cast<unsigned char*>(v_pool) + (long long)l * pool_layer_stride * e;
        const unsigned char* kn = k_new ? static_cast<const unsigned char*>(k_new) + (long long)l * new_layer_stride * e : nullptr;
        const unsigned char* vn = v_new ? static_cast<const unsigned char*>(v_new) + (long long)l * new_layer_stride * e : nullptr;
        void* ko = k_out[l % num_out];
        void* vo = v_out[l % num_out];
        if (fused_ok) {
            // Launches that may be on the device together never share a counter pair of `work`: a layer takes its
            // first pages while the layer before it in its stream is still handing out its last ones, and the two
            // streams use different pairs.  Within a stream each launch is a programmatic dependent of the one
            // before, whose batch description it shares.
            const FusedRows fused = {kn, vn, new_rows, cu_new, tokens_per_entry};
            LaunchOpts opts;
            opts.after_own_kernel = overlap ? l >= 2 : l > 0;
            int32_t* pair = !work ? nullptr : work + 2 * (overlap ? (l & 3) : (l & 1));
            if (work && g_knobs.zero_ahead != 0 && same_kernel) {
                // a chain alternates between two pairs; each launch clears the one it does not use, and only the
                // chain's last launch counts its finished CTAs to clear its own
                opts.zero_ahead = work + 2 * (overlap ? ((l + 2) & 3) : ((l + 1) & 1));
                opts.rearm = l + (overlap ? 2 : 1) >= layers;
                chained_pairs = true;
            }
            const int rc = gather_common(pool, kp, vp, table, only_gather && seq_lens_after ? seq_lens_after : seq_start, cu_out, n,
                                         total_tokens_hint, ko, vo, out_rows, mode, status, pair,
                                         overlap && (l & 1) ? static_cast<barqkv_stream_t>(dev->lane) : stream,
                                         only_gather ? nullptr : &fused, nullptr, opts);
            if (rc == 0) continue;
            if (rc != kNotFusable || l > 0) return done(rc);
            fused_ok = false;
        }
        if (!seq_lens_after)
            return done(fail(BARQKV_E_INVALID, "update_layers: this call cannot run as one launch per layer; pass seq_lens_after "
                                               "(lengths after the append, device int32[n]) so that it can run as append + gather"));
        if (total_new_tokens) {
            if (int rc = barqkv_append(pool, kp, vp, table, seq_start, cu_new, n, tokens_per_entry, total_new_tokens, kn, vn,
                                       new_rows, status, work, 0, stream))
                return done(rc);
        }
        if (int rc = barqkv_gather(pool, kp, vp, table, seq_lens_after, cu_out, n, total_tokens_hint, ko, vo, out_rows,
                                   mode & ~BARQKV_FLAG_DESC_STABLE, status, work, stream))
            return done(rc);
    }
    return done(0);
}

int barqkv_gather_wait_selftest(const barqkv_pool_layout* pool, const void* k_pool, const void* v_pool,
                                const barqkv_block_table* table,
                                const int32_t* seq_lens, const int32_t* cu_out, int32_t n,
                                void* k_out, void* v_out, const barqkv_rows_layout* out_rows,
                                int64_t wait_cycles, int32_t* status, barqkv_stream_t stream) {
    if (wait_cycles <= 0 || wait_cycles > kWaitCycles)
        return fail(BARQKV_E_INVALID, "gather_wait_selftest: wait_cycles must be in 1..2e9");
    if (!status) return fail(BARQKV_E_INVALID, "gather_wait_selftest: needs the status word");
    LaunchOpts opts;
    opts.wait_cycles = wait_cycles;
    opts.extra_tx = 16;       // every stage waits for 16 bytes that no copy brings
    opts.max_ctas = 1;
    return gather_common(pool, k_pool, v_pool, table, seq_lens, cu_out, n, 0, k_out, v_out, out_rows, BARQKV_MODE_BULK,
                         status, nullptr, stream, nullptr, nullptr, opts);
}

// --------------------------------------------------------------------------
// gather for callers that cannot allocate device memory
// --------------------------------------------------------------------------
// The hand-out counters of the bulk gather normally live in a caller-owned
// device buffer (`work`).  Some callers have no way to own one: an inference
// server that gave every free byte of HBM to its own arena at start-up (a later
// cudaMalloc fails, or stalls the device while the driver makes room), or an
// operator plugin whose host forbids allocation inside a call.  For them the
// counters live in this array, which is part of the library image: every GPU
// that loads the library holds these 4 KiB until the process exits.
//
// BARQKV_STATIC_WORK_SLOTS pairs of counters, one 128-byte line apart so that
// launches using different slots do not contend on a line.
constexpr int kStaticWorkStride = 32;   // int32 words between slots
static __device__ __align__(256) int32_t g_static_work[BARQKV_STATIC_WORK_SLOTS * kStaticWorkStride];

// Device address of g_static_work per device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel can use, so it is
// translated once per device with that device current.  Published with
// release/acquire: two threads that make the first call together both look the
// address up and store the same value.
static std::atomic<int32_t*> g_static_work_addr[64];

int barqkv_gather_noalloc(const barqkv_pool_layout* pool, const void* k_pool, const void* v_pool,
                          const barqkv_block_table* table,
                          const int32_t* seq_lens, const int32_t* cu_out, int32_t n,
                          int64_t total_tokens_hint,
                          void* k_out, void* v_out, const barqkv_rows_layout* out_rows,
                          int32_t mode, int32_t* status, int32_t work_slot, barqkv_stream_t stream) {
    if (work_slot < 0 || work_slot >= BARQKV_STATIC_WORK_SLOTS)
        return fail(BARQKV_E_LIMIT, "gather_noalloc: work_slot is outside the built-in scratch (32 slots: 0..31)");
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail_cuda("gather_noalloc: cudaGetDevice", e);
    if (dev < 0 || dev >= 64) return fail(BARQKV_E_LIMIT, "gather_noalloc: device ordinal above 63");
    int32_t* base = g_static_work_addr[dev].load(std::memory_order_acquire);
    if (!base) {
        void* addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_static_work);
        if (e != cudaSuccess || !addr) return fail_cuda("gather_noalloc: cudaGetSymbolAddress", e);
        base = static_cast<int32_t*>(addr);
        g_static_work_addr[dev].store(base, std::memory_order_release);
    }
    int32_t* work = base + (size_t)work_slot * kStaticWorkStride;
    // Arguments are checked before anything is enqueued: a refused call leaves the slot as it was.
    LaunchOpts check;
    check.validate_only = true;
    if (int rc = gather_common(pool, k_pool, v_pool, table, seq_lens, cu_out, n, total_tokens_hint, k_out, v_out, out_rows,
                               mode, status, work, stream, nullptr, nullptr, check))
        return rc;
    if (n == 0) return 0;
    // The slot keeps whatever its previous user left; the counters must start at zero.
    e = cudaMemsetAsync(work, 0, 2 * sizeof(int32_t), static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail_cuda("gather_noalloc: cudaMemsetAsync", e);
    return barqkv_gather(pool, k_pool, v_pool, table, seq_lens, cu_out, n, total_tokens_hint, k_out, v_out, out_rows,
                         mode, status, work, stream);
}

}  // extern "C"

#include "paged_attention.cuh"
#include "host_table.cuh"
