// Decode attention straight from the pages (included at the end of barqkv.cu; same translation unit).
//
// One query token per sequence attends over that sequence's K/V pages through the block table, so the
// gather's copy is not needed for decode: K and V are read once, where gather + attention read them
// twice and write them once.  Grouped-query attention: the `group` query heads that share a KV head
// form the rows of one 16-row MMA tile.
//
//   paged_decode_kernel   one warp per (sequence, KV head, split of the sequence's pages).  Pages travel
//                         through a ring of stages with tiled TMA loads (one box per page of K and of V
//                         from a 5-D tensor map over the pool, 128-byte swizzle, mbarrier completion; no
//                         multicast); Q.K^T and P.V run on
//                         mma.sync m16n8k16 with ldmatrix from the swizzled tiles; softmax is kept
//                         online in fp32 (base-2 exponent).  Memory-bound: the tensor-core work is
//                         ~6 warp instructions per token, the limit is reading 512 B per token and head.
//                         With several splits per sequence each warp leaves a partial (max, sum, output)
//                         triple in the workspace and is gone; paged_decode_merge_kernel, a small kernel
//                         launched behind it as a programmatic dependent, combines the triples (they are
//                         still in L2) and writes the output.  (Combining inside the launch - a fence, a
//                         counter per sequence, the last split to arrive does it - kept every split's
//                         place on the SM for microseconds with no page in flight and cost a tenth of the
//                         bandwidth.)  Optionally the step's append is fused in: the
//                         CTA that owns a sequence's last page takes the new K/V row from the caller's
//                         buffers, patches it into the page's tile in shared memory (the pool still holds
//                         whatever was in that slot) and writes it to the pool: no separate append, no gather.
//
// Restrictions (checked on the host): 2-byte elements (bf16 / fp16), head_dim 128, page_size 16, 32 or 64,
// group <= 8.  Every wait is bounded; a guard failure skips the sequence and sets a status bit.

namespace {

constexpr int kAttnSplitTokens = 512;                 // tokens per split by default
constexpr int kAttnMaxSplits = 64;                    // most splits of one sequence (bounds the workspace)
constexpr int kAttnCompactSeqs = 256;                 // largest batch whose splits are listed without gaps (8 sequences per lane)
// Per page size: bytes of one head's page of K (or V), of a stage (K + V), and ring depth.
template <int PS, bool WIDE> struct AttnTile {
    static constexpr int kHalf = PS * 128;            // one half tile: PS rows x 64 dims x 2 bytes
    static constexpr int kPage = 2 * kHalf;
    static constexpr int kStage = 2 * kPage;
    // 16-token pages attended two at a time keep three pages in flight beside the two in use
    static constexpr int kStages = PS <= 16 ? (WIDE ? 5 : 4) : 3;
};

struct AttnArgs {
    Table tb;
    const int32_t* seq_lens;
    const unsigned char* q;
    unsigned char* out;
    long long q_seq, q_head, o_seq, o_head;   // byte strides
    float* ws_o;                              // [n][kv_heads][splits][8][128] partial outputs
    float* ws_ml;                             // [n][kv_heads][splits][8][2]   (running max, running sum)
    int n, kv_heads, group, split_pages, splits, page_size;
    int probe;                                // timing probes of the tuning build: 1 = pages are loaded but not attended, 2 = no result is written
    int compact;                              // grid x counts the splits that have pages, one sequence after another (n <= kAttnCompactSeqs)
    float scale_log2;                         // softmax scale * log2(e)
    int32_t* status;
    // Fused append (null k_new = plain attention): the step's new K/V row of every (sequence, KV head) - the
    // token at position len - 1 - comes from k_new / v_new instead of the pool; the CTA that owns the
    // sequence's last page attends it and stores it into its page slot.
    const unsigned char* k_new;
    const unsigned char* v_new;
    unsigned char* k_pool_w;
    unsigned char* v_pool_w;
    long long new_seq, new_head;              // byte strides of the new rows
    long long pool_head, pool_page;           // byte strides of the pools
    int early;                                // lengths, slots and table are older than the kernel before this one
    int page_box;                             // 2: one 5-d box is a head's page of K and of V; 1: of K or of V; 0: 4-d maps, half a page per box
};

__device__ __forceinline__ void tensor_load_4d(uint32_t dst_smem, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                               uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tensor_load_5d(uint32_t dst_smem, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4,
                                               uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

template <bool BF16>
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    if (BF16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if (BF16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `chunk` (0..7) of row `r` inside one half tile ([page_size rows][128 B])
// written by TMA with the 128-byte swizzle (the pattern repeats every 8 rows = 1024 bytes).
__device__ __forceinline__ uint32_t swz(int r, int chunk) {
    return (uint32_t)(((r >> 3) << 10) + ((r & 7) << 7) + (((chunk ^ (r & 7)) & 7) << 4));
}

template <bool BF16, int PS, bool WIDE>
__global__ void __launch_bounds__(32)
paged_decode_kernel(const AttnArgs a, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
    extern __shared__ unsigned char s_attn_raw[];
    using Tile = AttnTile<PS, WIDE>;
    constexpr int kAttnStages = Tile::kStages;
    constexpr int kAttnStageBytes = Tile::kStage;
    constexpr int kAttnPageBytes = Tile::kPage;
    constexpr int kHalf = Tile::kHalf;
    __shared__ unsigned long long s_bar[kAttnStages];
    // the 128-byte swizzle pattern repeats every 1024 bytes of shared-memory address: align the tiles to it
    unsigned char* s_attn = s_attn_raw + ((1024u - (smem_addr(s_attn_raw) & 1023u)) & 1023u);
    const int lane = threadIdx.x;
    const int kvh = blockIdx.y;
    int split = blockIdx.x, seq = blockIdx.z;

    // Lengths, slots and block-table entries may be read before the kernel ahead of this one has finished
    // when the caller vouches that they are older than it; the query, the new rows and the pools may not.
    if (!a.early) {
        pdl_wait_for_predecessor();
        pdl_let_successor_in();
    }
    int len, row;
    if (a.compact) {
        // blockIdx.x counts splits that have pages, sequence after sequence, so that only the few CTAs beyond
        // the batch's real count (the grid is sized from the caller's bounds) find nothing to do - a CTA that
        // starts only to leave again holds up the one behind it.  Every lane reads the lengths and slots of up
        // to kAttnCompactSeqs / 32 sequences (all loads in flight together); a running sum of the sequences'
        // split counts finds the one this CTA's split belongs to.
        int my_len[kAttnCompactSeqs / 32], my_row[kAttnCompactSeqs / 32];
#pragma unroll
        for (int c = 0; c < kAttnCompactSeqs / 32; ++c) {
            const int i = c * 32 + lane;
            my_len[c] = i < a.n ? a.seq_lens[i] : 0;
            my_row[c] = i < a.n ? (a.tb.slots ? a.tb.slots[i] : i) : 0;
        }
        const int item = blockIdx.x;
        // the first CTA adds the counts up to the end: the grid was sized from the caller's sum of the lengths,
        // and a batch with more splits than that would lose some without a trace
        const bool count_all = blockIdx.x == 0 && blockIdx.y == 0;
        int before = 0;
        seq = -1;
        len = row = 0;
#pragma unroll
        for (int c = 0; c < kAttnCompactSeqs / 32; ++c) {
            if ((seq < 0 || count_all) && c * 32 < a.n) {
                const int pg = (max(my_len[c], 0) + PS - 1) / PS;
                const int count = min(a.splits, (pg + a.split_pages - 1) / a.split_pages);
                int upto = count;                                   // inclusive running sum over the lanes
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, upto, d);
                    if (lane >= d) upto += t;
                }
                const unsigned holds = seq < 0 ? __ballot_sync(0xffffffffu, before + upto > item) : 0u;
                if (holds) {
                    const int src = __ffs(holds) - 1;
                    seq = c * 32 + src;
                    len = __shfl_sync(0xffffffffu, my_len[c], src);
                    row = __shfl_sync(0xffffffffu, my_row[c], src);
                    split = item - before - __shfl_sync(0xffffffffu, upto - count, src);
                }
                before += __shfl_sync(0xffffffffu, upto, 31);
            }
        }
        if (count_all && lane == 0 && before > (int)gridDim.x) raise(a.status, BARQKV_S_CAPACITY);
        if (seq < 0) {
            if (a.early) { pdl_wait_for_predecessor(); pdl_let_successor_in(); }
            return;
        }
    } else {
        // the length and the table row are independent loads: both are in flight before either is used
        len = a.seq_lens[seq];
        row = a.tb.slots ? a.tb.slots[seq] : seq;
    }
    const int pages = (len + PS - 1) / PS;
    const int sp = a.split_pages;
    const int p0 = split * sp;
    if (len <= 0 || p0 >= pages) {
        if (a.early) { pdl_wait_for_predecessor(); pdl_let_successor_in(); }
        return;
    }
    const int p1 = min(pages, p0 + sp);
    if (row < 0 || row >= a.tb.rows || pages > a.tb.stride) {
        if (a.early) { pdl_wait_for_predecessor(); pdl_let_successor_in(); }
        if (lane == 0) raise(a.status, BARQKV_S_BAD_SLOT);
        return;
    }
    if (lane == 0) {
        for (int s = 0; s < kAttnStages; ++s) mbar_init(smem_addr(&s_bar[s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    float acc[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;      // for row g (the c0/c1 half of the fragments)

    // block-table entries of this split, 32 at a time, one per lane
    int table_base = p0;
    int my_page = (p0 + lane < p1) ? a.tb.table[(long long)row * a.tb.stride + p0 + lane] : -1;
    bool bad = false, dead = false;
    if (a.early) {
        pdl_wait_for_predecessor();
        pdl_let_successor_in();
    }

    // Q as the A operand: rows = query heads of this KV head (lane/4), zero rows beyond the group.
    const int g = lane >> 2, tq = lane & 3;
    uint32_t qa[8][2];
    {
        const unsigned char* qrow = a.q + (long long)seq * a.q_seq + (long long)(kvh * a.group + g) * a.q_head;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            qa[ks][0] = g < a.group ? *reinterpret_cast<const uint32_t*>(qrow + (ks * 16 + tq * 2) * 2) : 0u;
            qa[ks][1] = g < a.group ? *reinterpret_cast<const uint32_t*>(qrow + (ks * 16 + 8 + tq * 2) * 2) : 0u;
        }
    }

    // Fused append: this CTA owns the sequence's last page; lanes 0-15 carry the 16-byte chunks of the new K
    // row, lanes 16-31 those of the new V row (loaded now, used when the page arrives).
    const bool owns_new = a.k_new != nullptr && p1 == pages;
    uint4 new_chunk = make_uint4(0u, 0u, 0u, 0u);
    if (owns_new) {
        const unsigned char* src = (lane < 16 ? a.k_new : a.v_new) + (long long)seq * a.new_seq + (long long)kvh * a.new_head;
        new_chunk = *reinterpret_cast<const uint4*>(src + (lane & 15) * 16);
    }

    auto issue = [&](int p) {                  // load page p of this split into stage (p - p0) % stages
        if (p - table_base >= 32) {
            table_base += 32;
            my_page = (table_base + lane < p1) ? a.tb.table[(long long)row * a.tb.stride + table_base + lane] : -1;
        }
        const int phys = __shfl_sync(0xffffffffu, my_page, p - table_base);
        const int st = (p - p0) % kAttnStages;
        const uint32_t bar = smem_addr(&s_bar[st]);
        const bool ok = phys >= 0 && phys < a.tb.num_pages;
        if (!ok) bad = true;
        if (lane == 0) {
            if (ok) mbar_arrive_expect(bar, kAttnStageBytes); else mbar_arrive(bar);
        }
        __syncwarp();
        if (ok && a.page_box == 2) {
            // lane 0: the head's page of K and, one pool further on, of V, in one box
            if (lane == 0)
                tensor_load_5d(smem_addr(s_attn + (size_t)st * kAttnStageBytes), &map_k, 0, 0, 0, kvh * a.tb.num_pages + phys, 0, bar);
        } else if (ok && a.page_box) {
            // lanes 0 and 1: the head's page of K, of V (both halves of every row in one box)
            if (lane < 2)
                tensor_load_5d(smem_addr(s_attn + (size_t)st * kAttnStageBytes + lane * kAttnPageBytes), lane ? &map_v : &map_k,
                               0, 0, 0, phys, kvh, bar);
        } else if (ok && lane < 4) {
            // lanes 0..3: K dims 0-63, K dims 64-127, V dims 0-63, V dims 64-127 (one half tile each)
            const uint32_t dst = smem_addr(s_attn + (size_t)st * kAttnStageBytes + lane * kHalf);
            tensor_load_4d(dst, lane < 2 ? &map_k : &map_v, (lane & 1) * 64, 0, phys, kvh, bar);
        }
    };

    // One 16-token block of a tile: scores (two n-tiles of 8 tokens) and, later, its share of P.V.
    auto block_qk = [&](const unsigned char* kt, int r0, float (&s0)[4], float (&s1)[4]) {
        const int tile = lane >> 3, r8 = lane & 7;
        const int trow = r0 + (tile >> 1) * 8 + r8;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const uint32_t addr = smem_addr(kt + (ks >> 2) * kHalf) + swz(trow, (ks & 3) * 2 + (tile & 1));
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(addr, b0, b1, b2, b3);
            mma_16816<BF16>(s0, qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
            mma_16816<BF16>(s1, qa[ks][0], 0u, qa[ks][1], 0u, b2, b3);
        }
    };
    auto block_pv = [&](const unsigned char* vt, int r0, uint32_t pa0, uint32_t pa2) {
        const int tile = lane >> 3, r8 = lane & 7;
        const int trow = r0 + (tile & 1) * 8 + r8;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
            const uint32_t addr = smem_addr(vt + (nb >> 2) * kHalf) + swz(trow, (nb & 3) * 2 + (tile >> 1));
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(addr, b0, b1, b2, b3);
            mma_16816<BF16>(acc[2 * nb], pa0, 0u, pa2, 0u, b0, b1);
            mma_16816<BF16>(acc[2 * nb + 1], pa0, 0u, pa2, 0u, b2, b3);
        }
    };
    // rows past the sequence's end hold whatever the page held before: keep them out of P.V
    auto clear_v_tail = [&](unsigned char* vt, int r0, int valid) {
        for (int idx = lane; idx < (16 - valid) * 16; idx += 32) {
            const int r = r0 + valid + (idx >> 4), c = idx & 15;
            *reinterpret_cast<uint4*>(vt + (c >> 3) * kHalf + ((r >> 3) << 10) + ((r & 7) << 7) + ((c & 7) << 4)) =
                make_uint4(0u, 0u, 0u, 0u);
        }
        __syncwarp();
    };
    // Up to 32 tokens at a time: block A (16 rows from r0a of tile A, valid_a of them hold tokens) and, when
    // valid_b > 0, block B.  One running-maximum update, one rescale of the accumulators and one pass of
    // exponentials serve both blocks, and their score products are independent instruction streams.
    auto attend = [&](unsigned char* kta, unsigned char* vta, int r0a, int valid_a, unsigned char* ktb, unsigned char* vtb,
                      int r0b, int valid_b) {
        if (valid_a < 16) clear_v_tail(vta, r0a, valid_a);
        if (valid_b > 0 && valid_b < 16) clear_v_tail(vtb, r0b, valid_b);
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        float s2[4] = {0.f, 0.f, 0.f, 0.f}, s3[4] = {0.f, 0.f, 0.f, 0.f};
        block_qk(kta, r0a, s0, s1);
        if (valid_b > 0) block_qk(ktb, r0b, s2, s3);
        // online softmax for row g: this lane holds tokens tq*2, tq*2+1 (n-tile 0) and +8 (n-tile 1) of each block
        const int t_first = tq * 2;
        float x[8] = {s0[0] * a.scale_log2, s0[1] * a.scale_log2, s1[0] * a.scale_log2, s1[1] * a.scale_log2,
                      s2[0] * a.scale_log2, s2[1] * a.scale_log2, s3[0] * a.scale_log2, s3[1] * a.scale_log2};
        if (t_first >= valid_a) x[0] = -INFINITY;
        if (t_first + 1 >= valid_a) x[1] = -INFINITY;
        if (t_first + 8 >= valid_a) x[2] = -INFINITY;
        if (t_first + 9 >= valid_a) x[3] = -INFINITY;
        if (t_first >= valid_b) x[4] = -INFINITY;
        if (t_first + 1 >= valid_b) x[5] = -INFINITY;
        if (t_first + 8 >= valid_b) x[6] = -INFINITY;
        if (t_first + 9 >= valid_b) x[7] = -INFINITY;
        float mx = fmaxf(fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3])), fmaxf(fmaxf(x[4], x[5]), fmaxf(x[6], x[7])));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);              // finite: the first token of every block A reached is valid
        const float alpha = exp2f(m_run - m_new);
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = exp2f(x[i] - m_new);
        l_run = l_run * alpha + ((e[0] + e[1]) + (e[2] + e[3])) + ((e[4] + e[5]) + (e[6] + e[7]));
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < 16; ++i) { acc[i][0] *= alpha; acc[i][1] *= alpha; }
        block_pv(vta, r0a, pack2<BF16>(e[0], e[1]), pack2<BF16>(e[2], e[3]));
        if (valid_b > 0) block_pv(vtb, r0b, pack2<BF16>(e[4], e[5]), pack2<BF16>(e[6], e[7]));
    };
    auto wait_page = [&](int p) {              // false (and `dead`) when the bounded wait ran out
        const int st = (p - p0) % kAttnStages;
        const uint32_t phase = (uint32_t)(((p - p0) / kAttnStages) & 1);
        const uint32_t bar = smem_addr(&s_bar[st]);
        const long long t0 = clock64();
        while (!mbar_try_wait(bar, phase)) {
            if (clock64() - t0 > kWaitCycles) { dead = true; break; }
        }
        dead = __any_sync(0xffffffffu, dead);
        return !dead;
    };
    // The step's own token (fused append): into the tile - the pool's slot still holds stale bytes - and into the pool.
    auto place_new_row = [&](int p, unsigned char* kt, unsigned char* vt) {
        const int r = (len - 1) - p * PS;
        const int j = lane & 15;
        unsigned char* tile = lane < 16 ? kt : vt;
        *reinterpret_cast<uint4*>(tile + (j >> 3) * kHalf + swz(r, j & 7)) = new_chunk;
        const int phys = __shfl_sync(0xffffffffu, my_page, p - table_base);
        unsigned char* dst = (lane < 16 ? a.k_pool_w : a.v_pool_w) + (long long)phys * a.pool_page +
                             (long long)kvh * a.pool_head + (long long)r * 256 + j * 16;
        *reinterpret_cast<uint4*>(dst) = new_chunk;
        __syncwarp();
    };

    if (PS == 16 && WIDE) {
        // Two pages per iteration.  While pages p and p + 1 are attended, p + 2 .. p + kStages - 1 are on their way;
        // the two stages freed by the previous iteration are re-armed first.
        constexpr int ahead = kAttnStages - 2;
        for (int p = p0; p < min(p1, p0 + ahead); ++p) issue(p);
        for (int p = p0; p < p1; p += 2) {
            if (p + ahead < p1) issue(p + ahead);
            if (p + ahead + 1 < p1) issue(p + ahead + 1);
            const bool two = p + 1 < p1;
            if (!wait_page(p)) break;
            if (two && !wait_page(p + 1)) break;
            if (bad) continue;                     // keep draining the loads already issued, compute nothing
            unsigned char* kta = s_attn + (size_t)((p - p0) % kAttnStages) * kAttnStageBytes;
            unsigned char* ktb = s_attn + (size_t)((p + 1 - p0) % kAttnStages) * kAttnStageBytes;
            const int last = two ? p + 1 : p;
            if (owns_new && last == pages - 1) place_new_row(last, two ? ktb : kta, (two ? ktb : kta) + kAttnPageBytes);
            attend(kta, kta + kAttnPageBytes, 0, min(16, len - p * PS), ktb, ktb + kAttnPageBytes, 0,
                   two ? min(16, len - (p + 1) * PS) : 0);
            __syncwarp();      // every lane is done with both stages before lane 0 re-arms them
        }
    } else {
        constexpr int ahead = kAttnStages - 1;
        for (int p = p0; p < min(p1, p0 + ahead); ++p) issue(p);
        for (int p = p0; p < p1; ++p) {
            if (p + ahead < p1) issue(p + ahead);
            if (!wait_page(p)) break;
            if (bad) continue;                     // keep draining the loads already issued, compute nothing
            unsigned char* kt = s_attn + (size_t)((p - p0) % kAttnStages) * kAttnStageBytes;
            unsigned char* vt = kt + kAttnPageBytes;
            if (owns_new && p == pages - 1) place_new_row(p, kt, vt);
            constexpr int kStep = WIDE ? 32 : 16;              // tokens per softmax update
#pragma unroll 1
            for (int r0 = 0; r0 < PS; r0 += kStep) {
                const int valid_a = min(16, len - p * PS - r0);
                if (valid_a <= 0) break;
                const int valid_b = WIDE ? min(16, len - p * PS - r0 - 16) : 0;
    #ifdef BARQKV_TUNING
                if (a.probe & 1) continue;
#endif
                attend(kt, vt, r0, valid_a, kt, vt, r0 + 16, valid_b);
            }
            __syncwarp();      // every lane is done with this stage before lane 0 re-arms it
        }
    }

#ifdef BARQKV_TUNING
    if (a.probe & 2) return;
#endif
    const bool failed = dead || bad;
    if (failed && lane == 0) raise(a.status, dead ? BARQKV_S_TIMEOUT : BARQKV_S_BAD_PAGE);

    float l_tot = l_run + __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_tot += __shfl_xor_sync(0xffffffffu, l_tot, 2);
    if (a.splits == 1) {
        if (!failed && g < a.group) {
            unsigned char* orow = a.out + (long long)seq * a.o_seq + (long long)(kvh * a.group + g) * a.o_head;
            const float inv = 1.f / l_tot;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                *reinterpret_cast<uint32_t*>(orow + (i * 8 + tq * 2) * 2) = pack2<BF16>(acc[i][0] * inv, acc[i][1] * inv);
        }
        return;
    }

    // Several splits per sequence: this one leaves its (maximum, sum, output) in the workspace and goes away -
    // no fence, no counter, nothing that would keep its place on the SM busy with no page in flight.
    // paged_decode_merge_kernel, launched behind this kernel, combines them.
    if (!failed && g < a.group) {
        const long long item = ((((long long)seq * a.kv_heads + kvh) * a.splits) + split) * 8 + g;
        float* wo = a.ws_o + item * 128;
#pragma unroll
        for (int i = 0; i < 16; ++i) __stcg(reinterpret_cast<float2*>(wo + i * 8 + tq * 2), make_float2(acc[i][0], acc[i][1]));
        if (tq == 0) __stcg(reinterpret_cast<float2*>(a.ws_ml + item * 2), make_float2(m_run, l_tot));
    }
}

// Combines the partial results of a launch of paged_decode_kernel whose splits left them in the workspace and
// went away without waiting for one another.  One CTA per (sequence, KV head), 128 threads per part: a warp per
// query head (two rounds for more than four), four output dims per thread, one pass over the splits with a
// running maximum.  For up to eight splits that is all (no shared memory, every CTA of the grid resident at
// once); for more, PARTS parts take every PARTS-th split each and part 0 folds their results, which meet in
// shared memory.  Launched as a programmatic dependent of the attention kernel, and lets its own successor in
// at once: both are in place, their prologues done, when the last split finishes.
template <bool BF16, int PARTS>
__global__ void __launch_bounds__(128 * PARTS)
paged_decode_merge_kernel(const AttnArgs a) {
    __shared__ float4 s_num[PARTS > 1 ? PARTS - 1 : 1][128];
    __shared__ float2 s_ml[PARTS > 1 ? PARTS - 1 : 1][128];
    pdl_let_successor_in();
    const int seq = blockIdx.x / a.kv_heads, kvh = blockIdx.x % a.kv_heads;
    // the lengths are older than the kernel before this one: it read them itself before it let this one in
    const int len = a.seq_lens[seq];
    const int row = a.tb.slots ? a.tb.slots[seq] : seq;
    const int pages = (len + a.page_size - 1) / a.page_size;
    const int used = min(a.splits, (pages + a.split_pages - 1) / a.split_pages);
    pdl_wait_for_predecessor();
    if (row < 0 || row >= a.tb.rows || pages > a.tb.stride) return;      // the attention kernel skipped this sequence
    const long long item0 = (((long long)seq * a.kv_heads + kvh) * a.splits) * 8;
    const int t = threadIdx.x & 127, part = threadIdx.x >> 7;
    const int d0 = (t & 31) * 4;
    if (used <= 0) return;
    for (int r0 = 0; r0 < a.group; r0 += 4) {                    // the same trip count for every thread of the CTA
        const int r = r0 + (t >> 5);
        const bool row = r < a.group;
        const float* ml = a.ws_ml + (item0 + r) * 2;
        const float* po = a.ws_o + (item0 + r) * 128 + d0;
        float m = -INFINITY, den = 0.f;
        float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
        auto fold = [&](float m_in, float den_in, const float4& o) {
            const float m_new = fmaxf(m, m_in);
            const float keep = m == -INFINITY ? 0.f : exp2f(m - m_new), wgt = m_in == -INFINITY ? 0.f : exp2f(m_in - m_new);
            m = m_new;
            den = den * keep + wgt * den_in;
            num.x = num.x * keep + wgt * o.x;
            num.y = num.y * keep + wgt * o.y;
            num.z = num.z * keep + wgt * o.z;
            num.w = num.w * keep + wgt * o.w;
        };
#pragma unroll 8
        for (int s = part; s < used && row; s += PARTS) {
            const float2 x = __ldcg(reinterpret_cast<const float2*>(ml + (long long)s * 16));
            const float4 o = __ldcg(reinterpret_cast<const float4*>(po + (long long)s * 1024));
            fold(x.x, x.y, o);
        }
        if (PARTS > 1) {
            if (part > 0) { s_num[part - 1][t] = num; s_ml[part - 1][t] = make_float2(m, den); }
            __syncthreads();
            if (part == 0) {
#pragma unroll
                for (int k = 0; k < PARTS - 1; ++k) fold(s_ml[k][t].x, s_ml[k][t].y, s_num[k][t]);
            }
            __syncthreads();                                      // read before the next round overwrites
        }
        if (part > 0 || !row) continue;
        const float inv = 1.f / den;
        unsigned char* orow = a.out + (long long)seq * a.o_seq + (long long)(kvh * a.group + r) * a.o_head + d0 * 2;
        *reinterpret_cast<uint32_t*>(orow) = pack2<BF16>(num.x * inv, num.y * inv);
        *reinterpret_cast<uint32_t*>(orow + 4) = pack2<BF16>(num.z * inv, num.w * inv);
    }
}

// 5-D map over one layer's K (or V) pool: (64 dims, row in page, half of the row, page, head); box = one
// head's page, which lands in shared memory as [half][row][64 dims] - what two boxes of the 4-D map below
// leave there - from ONE copy instruction.  An instruction costs the issuing warp, and the copy engine, about
// 100 cycles for a 2 KiB box and 140 for a 4 KiB one (measured with a warp that does nothing but issue them),
// so four boxes per 16-token page cap an SM near 39 KB/us - below its share of the memory bandwidth - and two
// boxes do not.  (The half's stride, 128 bytes, is smaller than the row's, 256: the dimensions are listed in
// the order shared memory wants, not by stride.  If the driver refuses the map the 4-D one is used.)
bool make_page_map(CUtensorMap* map, const void* base, const barqkv_pool_layout* pool) {
    PFN_cuTensorMapEncodeTiled enc = tensor_map_encoder();
    if (!enc) return false;
    const long long e = pool->elem_bytes;
    const cuuint64_t dims[5] = {64u, (cuuint64_t)pool->page_size, 2u, (cuuint64_t)pool->num_pages, (cuuint64_t)pool->num_heads};
    const cuuint64_t strides[4] = {(cuuint64_t)(pool->head_dim * e), 128u, (cuuint64_t)(pool->page_stride * e),
                                   (cuuint64_t)(pool->head_stride * e)};
    const cuuint32_t box[5] = {64u, (cuuint32_t)pool->page_size, 2u, 1u, 1u};
    const cuuint32_t estr[5] = {1u, 1u, 1u, 1u, 1u};
    const CUtensorMapL2promotion promo = g_knobs.attn_promotion == 1   ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                         : g_knobs.attn_promotion == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B
                                                                      : CU_TENSOR_MAP_L2_PROMOTION_NONE;
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 5, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same when the V pool lies a fixed distance behind the K pool (one allocation holds both) and a pool's heads
// are adjacent: (64 dims, row in page, half of the row, head * pages + page, K or V); the box is a head's page
// of K AND of V, so a ring stage is filled by one copy instruction instead of two.
bool make_kv_page_map(CUtensorMap* map, const void* k_base, const void* v_base, const barqkv_pool_layout* pool) {
    PFN_cuTensorMapEncodeTiled enc = tensor_map_encoder();
    if (!enc) return false;
    const long long e = pool->elem_bytes;
    const long long apart = static_cast<const unsigned char*>(v_base) - static_cast<const unsigned char*>(k_base);
    if (apart <= 0 || apart % 16 || apart >= (1LL << 40)) return false;
    if (pool->head_stride != (long long)pool->num_pages * pool->page_stride) return false;
    if ((long long)pool->num_pages * pool->num_heads * pool->page_stride * e > apart) return false;     // the pools overlap
    const cuuint64_t dims[5] = {64u, (cuuint64_t)pool->page_size, 2u, (cuuint64_t)pool->num_pages * (cuuint64_t)pool->num_heads, 2u};
    const cuuint64_t strides[4] = {(cuuint64_t)(pool->head_dim * e), 128u, (cuuint64_t)(pool->page_stride * e), (cuuint64_t)apart};
    const cuuint32_t box[5] = {64u, (cuuint32_t)pool->page_size, 2u, 1u, 2u};
    const cuuint32_t estr[5] = {1u, 1u, 1u, 1u, 1u};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 5, const_cast<void*>(k_base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 4-D map over one layer's K (or V) pool: (dim, row in page, page, head); box = 64 dims x 16 rows.
bool make_pool_map(CUtensorMap* map, const void* base, const barqkv_pool_layout* pool) {
    PFN_cuTensorMapEncodeTiled enc = tensor_map_encoder();
    if (!enc) return false;
    const long long e = pool->elem_bytes;
    const cuuint64_t dims[4] = {(cuuint64_t)pool->head_dim, (cuuint64_t)pool->page_size, (cuuint64_t)pool->num_pages,
                                (cuuint64_t)pool->num_heads};
    const cuuint64_t strides[3] = {(cuuint64_t)(pool->head_dim * e), (cuuint64_t)(pool->page_stride * e),
                                   (cuuint64_t)(pool->head_stride * e)};
    const cuuint32_t box[4] = {64u, (cuuint32_t)pool->page_size, 1u, 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    const CUtensorMapL2promotion promo = g_knobs.attn_promotion == 1   ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                         : g_knobs.attn_promotion == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B
                                                                      : CU_TENSOR_MAP_L2_PROMOTION_NONE;
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Pages per split.  Default 32 (512 tokens): enough CTAs for the tail when the batch fills the machine
// several times over.  When it does not (few sequences, a single KV head per GPU) the split is sized so
// that the CTAs with work fill the resident slots once or twice: from the caller's total of the lengths
// when it is given, else from the longest length alone by halving.  Never more than 64 splits per sequence.
int attn_splits(int n, int kv_heads, long long max_len, long long total_len, int page_size, int* split_pages,
                long long* live_bound = nullptr) {
    const long long pages = (max_len + page_size - 1) / page_size;
    int sms = 148;
    if (DeviceInfo* d = device_info()) sms = d->sms;
    const int cap = (g_knobs.attn_split_tokens > 0 ? g_knobs.attn_split_tokens : kAttnSplitTokens) / page_size;
    int sp = cap < 1 ? 1 : cap;
    if (total_len > 0 && g_knobs.attn_split_tokens <= 0) {
        const int floor_pages = 64 / page_size > 1 ? 64 / page_size : 1;
        const long long slots = (long long)sms * (page_size <= 16 ? (g_knobs.attn_wide > 0 ? 5 : 6)
                                                                   : page_size <= 32 ? 4 : 2);       // resident one-warp CTAs
        const long long units = ((total_len + page_size - 1) / page_size + n) * kv_heads;           // (page, head) units, rounded up
        const long long partial = (long long)n * kv_heads / 2;                                      // last splits are half full on average
        for (int waves = 1; waves <= 2; ++waves) {
            const long long room = waves * slots - partial;
            if (room <= 0) continue;
            const long long fit = (units + room - 1) / room;
            if (fit <= sp) {
                sp = (int)(fit < floor_pages ? floor_pages : fit);
                break;
            }
        }
    } else {
        const long long per_cta = (long long)n * kv_heads * pages / (8LL * sms);
        while (sp * page_size > 64 && sp > per_cta) sp >>= 1;
    }
    while ((pages + sp - 1) / sp > kAttnMaxSplits) sp *= 2;
    *split_pages = sp;
    long long splits = (pages + sp - 1) / sp;
    if (splits < 1) splits = 1;
    if (live_bound) {
        // splits with pages: every sequence at most `splits`; all together at most (pages of the batch) / sp + n
        long long bound = (long long)n * splits;
        if (total_len > 0) {
            const long long batch_pages = (total_len + page_size - 1) / page_size + n;
            const long long by_total = batch_pages / sp + n;
            if (by_total < bound) bound = by_total;
        }
        *live_bound = bound;
    }
    return (int)splits;
}


}  // namespace

extern "C" {

int64_t barqkv_paged_decode_workspace_bytes(int32_t n, int32_t kv_heads, int64_t max_len, int64_t total_len,
                                            int32_t page_size) {
    if (n <= 0 || kv_heads <= 0 || max_len <= 0 || page_size <= 0) return 0;
    int sp;
    const int splits = attn_splits(n, kv_heads, max_len, total_len, page_size, &sp);
    if (splits == 1) return 0;
    return (int64_t)n * kv_heads * splits * 8 * (128 + 2) * (int64_t)sizeof(float);
}

}  // extern "C"

namespace {

int attention_common(const barqkv_pool_layout* pool, const void* k_pool, const void* v_pool,
                     const barqkv_block_table* table, const int32_t* seq_lens, int32_t n,
                     const void* k_new, const void* v_new, int64_t new_seq_stride, int64_t new_head_stride,
                     const void* q, int64_t q_seq_stride, int64_t q_head_stride,
                     void* out, int64_t out_seq_stride, int64_t out_head_stride,
                     int32_t num_q_heads, float softmax_scale, int32_t is_bf16, int64_t max_len,
                     int64_t total_len,
                     void* workspace, int64_t workspace_bytes, int32_t flags, int32_t* status, barqkv_stream_t stream_) {
    if (int rc = check_pool(pool)) return rc;
    if (flags & ~BARQKV_FLAG_DESC_STABLE) return fail(BARQKV_E_INVALID, "decode_attention: unknown flag");
    if (n < 0) return fail(BARQKV_E_INVALID, "decode_attention: negative batch size");
    if (n == 0) return 0;
    if (int rc = check_table(table, n)) return rc;
    if (!table->table) return fail(BARQKV_E_INVALID, "decode_attention: needs an explicit block table");
    if (!k_pool || !v_pool || !seq_lens || !q || !out) return fail(BARQKV_E_INVALID, "decode_attention: null pointer argument");
    if (pool->elem_bytes != 2 || pool->head_dim != 128 ||
        (pool->page_size != 16 && pool->page_size != 32 && pool->page_size != 64))
        return fail(BARQKV_E_LIMIT, "decode_attention: supports 2-byte elements, head_dim 128, page_size 16, 32 or 64");
    if (num_q_heads <= 0 || num_q_heads % pool->num_heads || num_q_heads / pool->num_heads > 8)
        return fail(BARQKV_E_LIMIT, "decode_attention: query heads must be 1..8 times the KV heads");
    if (n > 65535 || pool->num_heads > 65535 || (long long)n * pool->num_heads > 0x7fffffffLL)
        return fail(BARQKV_E_LIMIT, "decode_attention: more than 65535 sequences or heads");
    if (max_len <= 0) return fail(BARQKV_E_INVALID, "decode_attention: max_len (upper bound of the lengths) must be positive");
    const long long e = 2;
    if (!aligned(q, 4) || !aligned(out, 4) || !multiple(q_seq_stride * e, 4) || !multiple(q_head_stride * e, 4) ||
        !multiple(out_seq_stride * e, 4) || !multiple(out_head_stride * e, 4))
        return fail(BARQKV_E_INVALID, "decode_attention: q and out rows must be 4-byte aligned");
    if (!aligned(k_pool, 16) || !aligned(v_pool, 16) || !multiple(pool->page_stride * e, 16) || !multiple(pool->head_stride * e, 16))
        return fail(BARQKV_E_INVALID, "decode_attention: pools must be 16-byte aligned");
    DeviceInfo* d = device_info();
    if (!d) return fail(BARQKV_E_LAUNCH, "no CUDA device is current");

    AttnArgs a;
    memset(&a, 0, sizeof(a));
    a.tb = make_table(table, pool->num_pages);
    a.seq_lens = seq_lens;
    a.q = static_cast<const unsigned char*>(q);
    a.out = static_cast<unsigned char*>(out);
    a.q_seq = q_seq_stride * e;
    a.q_head = q_head_stride * e;
    a.o_seq = out_seq_stride * e;
    a.o_head = out_head_stride * e;
    a.n = n;
    a.kv_heads = pool->num_heads;
    a.group = num_q_heads / pool->num_heads;
    a.page_size = pool->page_size;
    long long live_bound = 0;
    a.splits = attn_splits(n, a.kv_heads, max_len, total_len, a.page_size, &a.split_pages, &live_bound);
    a.probe = g_knobs.attn_probe;
    a.compact = n <= kAttnCompactSeqs && a.splits > 1 && g_knobs.attn_compact != 0 ? 1 : 0;
    a.scale_log2 = softmax_scale * 1.4426950408889634f;
    a.status = status;
    a.early = (flags & BARQKV_FLAG_DESC_STABLE) && g_knobs.pdl != 0 ? 1 : 0;
    if (k_new || v_new) {
        if (!k_new || !v_new) return fail(BARQKV_E_INVALID, "decode_update: needs both the new K rows and the new V rows");
        if (!aligned(k_new, 16) || !aligned(v_new, 16) || !multiple(new_seq_stride * e, 16) || !multiple(new_head_stride * e, 16))
            return fail(BARQKV_E_INVALID, "decode_update: new rows must be 16-byte aligned");
        a.k_new = static_cast<const unsigned char*>(k_new);
        a.v_new = static_cast<const unsigned char*>(v_new);
        a.k_pool_w = static_cast<unsigned char*>(const_cast<void*>(k_pool));
        a.v_pool_w = static_cast<unsigned char*>(const_cast<void*>(v_pool));
        a.new_seq = new_seq_stride * e;
        a.new_head = new_head_stride * e;
        a.pool_head = pool->head_stride * e;
        a.pool_page = pool->page_stride * e;
    }
    if (a.splits > 1) {
        const int64_t need = barqkv_paged_decode_workspace_bytes(n, a.kv_heads, max_len, total_len, a.page_size);
        if (!workspace || workspace_bytes < need || !aligned(workspace, 16))
            return fail(BARQKV_E_INVALID, "decode_attention: workspace missing or smaller than "
                                          "barqkv_paged_decode_workspace_bytes(n, kv_heads, max_len, total_len, page_size)");
        a.ws_o = static_cast<float*>(workspace);
        a.ws_ml = a.ws_o + (size_t)n * a.kv_heads * a.splits * 8 * 128;
    }
    CUtensorMap map_k, map_v;
    if (g_knobs.attn_page_box == 2 && make_kv_page_map(&map_k, k_pool, v_pool, pool)) {
        a.page_box = 2;
        map_v = map_k;
    } else {
        a.page_box = g_knobs.attn_page_box != 0 && make_page_map(&map_k, k_pool, pool) && make_page_map(&map_v, v_pool, pool);
    }
    if (!a.page_box && (!make_pool_map(&map_k, k_pool, pool) || !make_pool_map(&map_v, v_pool, pool)))
        return fail(BARQKV_E_LAUNCH, "decode_attention: could not describe the pools to the copy engine");

    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    const dim3 grid = a.compact ? dim3((unsigned)live_bound, (unsigned)a.kv_heads, 1u)
                                : dim3((unsigned)a.splits, (unsigned)a.kv_heads, (unsigned)n);
    auto launch = [&](auto kernel, size_t smem) -> cudaError_t {
        if (smem > 48 * 1024) {
            const cudaError_t se = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (se != cudaSuccess) return se;
        }
        return ::launch(kernel, grid, dim3(32), smem, st, a.early != 0, a, map_k, map_v);
    };
    cudaError_t le;
    // + 1024 bytes of slack to align the tiles to the swizzle period
#define BARQKV_ATTN_LAUNCH(PS, W)                                                                                      \
    le = is_bf16 ? launch(paged_decode_kernel<true, PS, W>, (size_t)AttnTile<PS, W>::kStages * AttnTile<PS, W>::kStage + 1024) \
                 : launch(paged_decode_kernel<false, PS, W>, (size_t)AttnTile<PS, W>::kStages * AttnTile<PS, W>::kStage + 1024)
    // 32-token softmax blocks pay for pages of 32 and 64; pages of 16 would need a fifth ring stage for them
    const bool wide = g_knobs.attn_wide >= 0 ? g_knobs.attn_wide != 0 : a.page_size >= 32;
    if (a.page_size == 16) { if (wide) { BARQKV_ATTN_LAUNCH(16, true); } else { BARQKV_ATTN_LAUNCH(16, false); } }
    else if (a.page_size == 32) { if (wide) { BARQKV_ATTN_LAUNCH(32, true); } else { BARQKV_ATTN_LAUNCH(32, false); } }
    else { if (wide) { BARQKV_ATTN_LAUNCH(64, true); } else { BARQKV_ATTN_LAUNCH(64, false); } }
#undef BARQKV_ATTN_LAUNCH
    if (le != cudaSuccess) return fail_cuda("decode_attention: cudaFuncSetAttribute", le);
    cudaError_t ce = cudaGetLastError();
    if (ce != cudaSuccess) return fail_cuda("decode_attention launch", ce);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (a.splits > 1) {
        const dim3 mgrid((unsigned)((long long)n * a.kv_heads));
        if (a.splits > 8)
            le = is_bf16 ? ::launch(paged_decode_merge_kernel<true, 4>, mgrid, dim3(512), 0, st, g_knobs.pdl != 0, a)
                         : ::launch(paged_decode_merge_kernel<false, 4>, mgrid, dim3(512), 0, st, g_knobs.pdl != 0, a);
        else
            le = is_bf16 ? ::launch(paged_decode_merge_kernel<true, 1>, mgrid, dim3(128), 0, st, g_knobs.pdl != 0, a)
                         : ::launch(paged_decode_merge_kernel<false, 1>, mgrid, dim3(128), 0, st, g_knobs.pdl != 0, a);
        if (le != cudaSuccess) return fail_cuda("decode_attention merge launch", le);
        g_launches.fetch_add(1, std::memory_order_relaxed);
    }
    return 0;
}

}  // namespace

extern "C" {

int barqkv_paged_decode_attention(const barqkv_pool_layout* pool, const void* k_pool, const void* v_pool,
                                  const barqkv_block_table* table, const int32_t* seq_lens, int32_t n,
                                  const void* q, int64_t q_seq_stride, int64_t q_head_stride,
                                  void* out, int64_t out_seq_stride, int64_t out_head_stride,
                                  int32_t num_q_heads, float softmax_scale, int32_t is_bf16, int64_t max_len,
                                  int64_t total_len,
                                  void* workspace, int64_t workspace_bytes, int32_t* status, barqkv_stream_t stream) {
    return attention_common(pool, k_pool, v_pool, table, seq_lens, n, nullptr, nullptr, 0, 0, q, q_seq_stride, q_head_stride,
                            out, out_seq_stride, out_head_stride, num_q_heads, softmax_scale, is_bf16, max_len, total_len,
                            workspace, workspace_bytes, 0, status, stream);
}

int barqkv_paged_decode_update(const barqkv_pool_layout* pool, void* k_pool, void* v_pool,
                               const barqkv_block_table* table, const int32_t* seq_lens_after, int32_t n,
                               const void* k_new, const void* v_new, int64_t new_seq_stride, int64_t new_head_stride,
                               const void* q, int64_t q_seq_stride, int64_t q_head_stride,
                               void* out, int64_t out_seq_stride, int64_t out_head_stride,
                               int32_t num_q_heads, float softmax_scale, int32_t is_bf16, int64_t max_len,
                               int64_t total_len, void* workspace, int64_t workspace_bytes, int32_t flags,
                               int32_t* status, barqkv_stream_t stream) {
    if (!k_new || !v_new) return fail(BARQKV_E_INVALID, "decode_update: null new rows");
    return attention_common(pool, k_pool, v_pool, table, seq_lens_after, n, k_new, v_new, new_seq_stride, new_head_stride, q,
                            q_seq_stride, q_head_stride, out, out_seq_stride, out_head_stride, num_q_heads, softmax_scale,
                            is_bf16, max_len, total_len, workspace, workspace_bytes, flags, status, stream);
}

}  // extern "C"
