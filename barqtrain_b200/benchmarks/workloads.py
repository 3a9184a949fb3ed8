"""Timed loops for the chunked-prefill, 70B-shaped gather and continuous-batching configurations.

Each function builds the configuration's cache on ``device`` for this rank's KV-head shard, runs
``warmup`` untimed and ``steps`` timed steps bracketed by CUDA events, and returns a dict with the
algorithmic bytes moved on this rank, the elapsed milliseconds and a description.  Algorithmic bytes
are 4*tokens*H*D*e per layer for both append and gather (K and V, read + write).  ``heads`` overrides
the rank's share of the 8 KV heads (e.g. 1 to run an 8-GPU shard's work on a single GPU).
"""

from __future__ import annotations

import math
import time
from typing import Dict

import numpy as np
import torch

from ..block_table import BlockTableKVCache
from ..sharding import kv_head_shard

D = 128


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def chunked_prefill(world: int, rank: int, device, steps: int, warmup: int, page_size: int = 16,
                    layers: int = 32, all_layers: bool = False, heads: int = 0, calls_per_layer: bool = False,
                    sync=lambda: None) -> Dict:
    """32 layers, 8 KV heads, head_dim 128, fp16; 16 sequences of 8192 tokens appended in 2048-token
    chunks into a pool shuffled by a seeded permutation.  A step appends one chunk of every sequence
    in every layer; after four chunks the sequences are released and re-opened.  One launch per layer, issued
    by one native call for the step (``calls_per_layer``: by one call from Python per layer, as a model's forward
    pass would; ``all_layers``: one launch for all layers)."""
    H = heads or kv_head_shard(8, world, rank)[1]
    B, chunk, chunks = 16, 2048, 4
    dtype = torch.float16
    pages = B * chunk * chunks // page_size
    cache = BlockTableKVCache(layers, H, D, page_size=page_size, num_pages=pages, max_seqs=B,
                              max_blocks_per_seq=chunk * chunks // page_size, dtype=dtype, device=device,
                              seed=1237, zero_pages=False)
    gen = torch.Generator(device=device).manual_seed(1237 + rank)
    # every layer appends rows of its own ([layers, tokens, H, D] for K and for V), so no layer's reads can be
    # served by what another layer left in L2
    k_all = torch.empty(layers, B * chunk, H, D, dtype=dtype, device=device)
    v_all = torch.empty_like(k_all)
    for layer in range(layers):
        k_all[layer] = torch.randn(B * chunk, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
        v_all[layer] = torch.randn(B * chunk, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
    k_rows, v_rows = list(k_all.unbind(0)), list(v_all.unbind(0))
    state = {"ids": list(range(B)), "slots": [cache.open(i) for i in range(B)], "done": 0, "next": B}

    def step():
        if state["done"] == chunks:
            for sid in state["ids"]:
                cache.release(sid)
            state["ids"] = list(range(state["next"], state["next"] + B))
            state["next"] += B
            state["slots"] = [cache.open(i) for i in state["ids"]]
            state["done"] = 0
        batch = cache.begin_append(state["slots"], [chunk] * B)
        if all_layers:
            cache.append_layers(batch, k_all, v_all)
        elif calls_per_layer:
            for layer in range(layers):
                cache.append(layer, batch, k_all[layer], v_all[layer])
        else:
            cache.append_each_layer(batch, k_rows, v_rows)
        cache.end_append(batch)
        state["done"] += 1

    for _ in range(max(warmup, 1)):
        step()
    sync()
    e0, e1 = _events()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    cache.check_device_status()
    per_step = 4 * B * chunk * H * D * 2 * layers
    return {"bytes": per_step * steps, "ms": ms, "tokens": B * chunk * steps,
            "launches": (1 if all_layers else layers) * steps,
            "config": {"workload": "chunked-prefill",
                       "launch": "all layers per launch" if all_layers else
                                 "one per layer, one call from Python each" if calls_per_layer else
                                 "one per layer, all issued by one native call",
                       "layers": layers, "kv_heads_per_gpu": H, "dtype": "fp16",
                       "page_size": page_size, "sequences": B, "chunk_tokens": chunk,
                       "step": "append one 2048-token chunk of 16 sequences in every layer",
                       "l2": "inputs larger than L2: every layer reads its own 134 MB of K and of V rows at 8 heads "
                             "(%.1f GB of sources), pool %.0f GB" % (2 * k_all.numel() * 2 / 1e9, cache.pools.numel() * 2 / 1e9)}}


def gather_70b(world: int, rank: int, device, steps: int, warmup: int, layers: int = 80, heads: int = 0,
               all_layers: bool = False, calls_per_layer: bool = False, sync=lambda: None) -> Dict:
    """80 layers, 8 KV heads sharded by head, head_dim 128, bf16, page 16; 32 sequences with seeded
    lengths log-uniform in [1k, 32k]; fragmented block tables.  A step gathers every sequence to
    contiguous ``[H, sum_len, D]`` K and V in every layer: one launch per layer into two alternating
    outputs, the step's launches issued by one native call (``calls_per_layer``: by one call from Python per
    layer), or (``all_layers``) one launch for all layers into ``[layers, H, sum_len, D]``."""
    H = heads or kv_head_shard(8, world, rank)[1]
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(1238)
    u = torch.rand(32, generator=g, dtype=torch.float64)
    lens = [int(round(math.exp(math.log(1024) + float(x) * (math.log(32768) - math.log(1024))))) for x in u]
    pages = sum(-(-n // 16) for n in lens)
    cache = BlockTableKVCache(layers, H, D, page_size=16, num_pages=pages, max_seqs=32,
                              max_blocks_per_seq=-(-max(lens) // 16), dtype=dtype, device=device,
                              free_order=torch.randperm(pages, generator=g).tolist(), zero_pages=False)
    slots = [cache.open(i) for i in range(32)]
    gen = torch.Generator(device=device).manual_seed(1238 + rank)
    total = sum(lens)
    k = torch.randn(total, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
    batch = cache.begin_append(slots, lens)
    for layer in range(layers):                         # set-up: fill the pools through the append kernel
        cache.append(layer, batch, k, k)
    cache.end_append(batch)
    del k
    gb = cache.begin_gather(slots)
    if all_layers:
        out_all = (torch.empty(layers, H, total, D, dtype=dtype, device=device),
                   torch.empty(layers, H, total, D, dtype=dtype, device=device))

        def step():
            cache.gather_layers(gb, "HND", out=out_all)
    else:
        outs = [(torch.empty(H, total, D, dtype=dtype, device=device), torch.empty(H, total, D, dtype=dtype, device=device))
                for _ in range(2)]

        def step():
            if calls_per_layer:
                for layer in range(layers):
                    cache.gather(layer, gb, "HND", out=outs[layer & 1])
            else:
                cache.gather_each_layer(gb, outs, "HND")

    for _ in range(max(warmup, 1)):
        step()
    sync()
    e0, e1 = _events()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    cache.check_device_status()
    per_step = 4 * total * H * D * 2 * layers
    return {"bytes": per_step * steps, "ms": ms, "tokens": total * steps, "launches": (1 if all_layers else layers) * steps,
            "config": {"workload": "llama3-70b-gather", "launch": "all layers per launch" if all_layers else
                       "one per layer, one call from Python each" if calls_per_layer else
                       "one per layer, all issued by one native call (neighbouring layers overlap at their ends)",
                       "layers": layers, "kv_heads_per_gpu": H, "dtype": "bf16",
                       "page_size": 16, "sequences": 32, "sum_len_tokens": total,
                       "lengths": "log-uniform [1024, 32768] seeded",
                       "step": "gather all sequences to [H,sum_len,D] in every layer",
                       "l2": "inputs larger than L2: %.2f GB per launch" % (4 * total * H * D * 2 / 1e9)}}


def churn(world: int, rank: int, device, steps: int, warmup: int, layers: int = 32, verify: bool = False,
          heads: int = 0, attend: bool = False, sync=lambda: None) -> Dict:
    """Continuous batching: 32 layers, 8 KV heads, head_dim 128, fp16, page 16; 256 live sequences with
    initial lengths uniform in [128, 2048]; every step appends one token to every live sequence in every
    layer, then each sequence finishes with seeded probability 0.01, returns its pages to the free list
    and is replaced by a new sequence with a 512-token prefill.  The replacements' prompts travel in the next
    step's launch, beside the other sequences' decode tokens - one ragged batch per step, as a server that
    mixes prefill chunks and decode tokens forms it.  ``attend``: the decode step also attends
    over the pages (4 query heads per KV head) - per layer one call that stores the token and attends,
    replayed from a CUDA graph whose batch rows are re-pointed at the replacements (``DecodeGraphs``)."""
    H = heads or kv_head_shard(8, world, rank)[1]
    dtype = torch.float16
    g = torch.Generator().manual_seed(1239)
    live = 256
    lens0 = torch.randint(128, 2049, (live,), generator=g).tolist()
    total_steps = steps + max(warmup, 1)
    cap = 2048 + total_steps + 512
    pages = sum(-(-(n + total_steps) // 16) for n in lens0) + live * 8 + 4096
    cache = BlockTableKVCache(layers, H, D, page_size=16, num_pages=pages, max_seqs=live,
                              max_blocks_per_seq=-(-cap // 16), dtype=dtype, device=device,
                              free_order=torch.randperm(pages, generator=g).tolist(), zero_pages=False)
    gen = torch.Generator(device=device).manual_seed(1239 + rank)
    rows = torch.randn(max(max(lens0), 512 * 4) * 8 + live, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
    ids = list(range(live))
    slots = np.array([cache.open(i) for i in ids], dtype=np.int32)
    next_id = live
    # set-up: initial contents, in slices so that the packed source stays small
    origin = [None] * live            # per live sequence: (first row, count) of its prefill in `rows`
    decoded = np.zeros(live, dtype=np.int64)   # decode tokens appended since (each is rows[j]; `attend` only)
    history = [[] for _ in range(live)]        # per live sequence: (first row, count) of every append (``verify``)
    for lo in range(0, live, 8):
        part, counts = slots[lo:lo + 8].tolist(), lens0[lo:lo + 8]
        at = 0
        for j, c in zip(range(lo, lo + 8), counts):
            origin[j] = (at, c)
            history[j].append((at, c))
            at += c
        batch = cache.begin_append(part, counts)
        for layer in range(layers):
            cache.append(layer, batch, rows[: sum(counts)], rows[: sum(counts)])
        cache.end_append(batch)
    # the step's new rows, [layers, live, H, D], and the replacement prompts' rows, [layers, 32 * 512, H, D]: every
    # layer has rows of its own (layer l holds the shared rows, so that the read-back check stays simple)
    one_all = rows[:live].unsqueeze(0).repeat(layers, 1, 1, 1) if attend else None
    prompt_all = rows[: 512 * 32].unsqueeze(0).repeat(layers, 1, 1, 1) if attend else None
    # a mixed step's packed rows, [layers, up to 32 prompts + live tokens, H, D]: entry j of the batch takes the
    # rows from its offset in the step's running count
    mixed_all = None if attend else rows[: 512 * 32 + live].unsqueeze(0).repeat(layers, 1, 1, 1)
    fresh_at: list = []               # batch positions whose sequence was opened after the last launch
    finished = (torch.rand(total_steps, live, generator=g) < 0.01).numpy()
    ones = np.ones(live, dtype=np.int32)
    counters = {"tokens": 0, "host_s": 0.0, "released": 0, "launches": 0, "attended": 0}
    graphs = None
    if attend:
        from ..block_table import DecodeGraphs

        graphs = DecodeGraphs(cache, capacity_tokens=live * cap, what="attention", q_heads=4 * H, max_len=cap)
        g0 = graphs.graph_for(slots.tolist())
        g0.k_in.copy_(one_all)
        g0.v_in.copy_(one_all)
        g0.q_in.normal_(generator=gen)

    def step(i):
        nonlocal next_id, fresh_at
        if attend:
            t0 = time.perf_counter()
            graph = graphs.step(slots.tolist())                # host work of the step is inside (native description)
            counters["host_s"] += time.perf_counter() - t0
            counters["attended"] += graph.total
            counters["launches"] += layers
        else:
            t0 = time.perf_counter()
            counts = ones
            if fresh_at:
                counts = ones.copy()
                counts[fresh_at] = 512
            batch = cache.begin_append(slots, counts)
            counters["host_s"] += time.perf_counter() - t0
            total = live + 511 * len(fresh_at)
            mixed = mixed_all[:, :total]
            cache.append_layers(batch, mixed, mixed)           # all layers' rows of the step in one launch
            cache.end_append(batch)
            counters["launches"] += 1
            counters["tokens"] += total - live                 # the prompts; the decode tokens are counted below
            if verify:
                at = 0
                for j in range(live):
                    history[j].append((at, int(counts[j])))
                    at += int(counts[j])
            fresh_at = []
        counters["tokens"] += live
        decoded[:] += 1
        gone = np.nonzero(finished[i])[0].tolist()
        if gone and not attend:
            t0 = time.perf_counter()
            for j in gone[:32]:        # a step's packed rows hold 32 prompts; more than 32 of 256 finishing in one
                #                        step at p = 0.01 has probability < 1e-30, the rest would wait a step
                cache.release(ids[j])
                ids[j] = next_id
                next_id += 1
                slots[j] = cache.open(ids[j])
                history[j] = []
                fresh_at.append(j)
            counters["host_s"] += time.perf_counter() - t0
            counters["released"] += len(fresh_at)
        elif gone:
            t0 = time.perf_counter()
            fresh = []
            for j in gone[:32]:        # the packed prefill source holds 32 prompts; more than 32 of 256 finishing in
                #                        one step at p = 0.01 has probability < 1e-30, the rest would wait a step
                cache.release(ids[j])
                ids[j] = next_id
                next_id += 1
                slots[j] = cache.open(ids[j])
                origin[j], decoded[j] = (512 * len(fresh), 512), 0
                fresh.append(slots[j])
            batch = cache.begin_append(fresh, [512] * len(fresh))
            counters["host_s"] += time.perf_counter() - t0
            prompt = prompt_all[:, : 512 * len(fresh)]
            cache.append_layers(batch, prompt, prompt)
            cache.end_append(batch)
            counters["tokens"] += 512 * len(fresh)
            counters["released"] += len(fresh)
            counters["launches"] += 1

    for i in range(max(warmup, 1)):
        step(i)
    sync()
    for key in counters:
        counters[key] = 0 if key != "host_s" else 0.0
    e0, e1 = _events()
    e0.record()
    for i in range(steps):
        step(max(warmup, 1) + i)
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    cache.check_device_status()
    verified = None
    if verify:
        # every live sequence must read back as its prefill rows followed by its decode rows, in both K and V
        verified = True
        gb = cache.begin_gather(slots)
        for layer in sorted({0, layers - 1}):
            kn, vn = cache.gather(layer, gb, "NHD")
            for j in range(live):
                if attend:
                    first, count = origin[j]
                    want = torch.cat([rows[first:first + count], rows[j:j + 1].expand(int(decoded[j]), -1, -1)])
                else:
                    index = np.concatenate([np.arange(first, first + count) for first, count in history[j]] or
                                           [np.zeros(0, dtype=np.int64)])
                    want = rows[torch.from_numpy(index).to(device)]
                a, b = gb.cu[j], gb.cu[j + 1]
                if b - a != want.shape[0] or not torch.equal(kn[a:b], want) or not torch.equal(vn[a:b], want):
                    verified = False
    st = cache.stats()
    return {"bytes": (4 * counters["tokens"] + 2 * counters["attended"]) * H * D * 2 * layers, "ms": ms,
            "tokens": counters["tokens"], "verified": verified,
            "launches": counters["launches"],
            "config": {"workload": "continuous-batching-churn", "layers": layers, "kv_heads_per_gpu": H,
                       "dtype": "fp16", "page_size": 16, "live_sequences": live,
                       "step": ("per layer, store 1 token of 256 sequences and attend over their pages (one call per "
                                "layer, CUDA graph); finished sequences (p=0.01) release their pages and are replaced "
                                "by a 512-token prefill" if attend else
                                "one ragged launch for all layers: 1 token for each of 256 sequences, and the 512-token "
                                "prompt of every sequence that replaced one that finished (p=0.01) and released its "
                                "pages the step before"),
                       "l2": "a step's decode rows are 2 MB per layer (L2-resident); the prompts stream"},
            "extra": {"sequences_released": counters["released"], "pages_total": st.pages_total,
                      "pages_resident": st.pages_resident, "pages_peak": st.pages_peak,
                      "bytes_peak": st.bytes_peak,
                      "host_allocator_us_per_step": round(counters["host_s"] * 1e6 / max(steps, 1), 1)}}


def decode_attention(world: int, rank: int, device, steps: int, warmup: int, layers: int = 32, heads: int = 0,
                     eager: bool = False, sync=lambda: None) -> Dict:
    """The decode configuration (32 layers, 8 KV heads x 4 query heads, head_dim 128, bf16, page 16, 64
    sequences uniform [512, 4096]) with attention reading the pages directly: a step is, per layer, ONE
    call that stores the step's token and attends over the pages - no separate append, no gather; the
    attention kernel and the small kernel that combines its splits' partial results - replayed from a CUDA
    graph (``eager``: append + attention called per layer from Python).
    Bytes counted: K and V read once (2*sum_len*H*D*e per layer) plus the append's 4*B*H*D*e."""
    from ..block_table import DecodeStepGraph

    H = heads or kv_head_shard(8, world, rank)[1]
    group, B, dtype = 4, 64, torch.bfloat16
    g = torch.Generator().manual_seed(1236)
    lens = torch.randint(512, 4097, (B,), generator=g).tolist()
    total_steps = steps + max(warmup, 1) + 4
    pages = sum(-(-(n + total_steps) // 16) for n in lens)
    cache = BlockTableKVCache(layers, H, D, page_size=16, num_pages=pages, max_seqs=B,
                              max_blocks_per_seq=-(-(max(lens) + total_steps) // 16), dtype=dtype, device=device,
                              free_order=torch.randperm(pages, generator=g).tolist(), zero_pages=False)
    slots = [cache.open(i) for i in range(B)]
    gen = torch.Generator(device=device).manual_seed(1236 + rank)
    k = torch.randn(sum(lens), H, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
    batch = cache.begin_append(slots, lens)
    for layer in range(layers):
        cache.append(layer, batch, k, k)
    cache.end_append(batch)
    del k
    new_rows = torch.randn(layers, B, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
    q = torch.randn(B, H * group, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
    moved = {"bytes": 0}
    if eager:
        out = torch.empty_like(q)

        def step():
            new = cache.begin_append(slots, [1] * B)
            cache.end_append(new)
            full = cache.begin_gather(slots)
            for layer in range(layers):
                cache.append(layer, new, new_rows[layer], new_rows[layer])
                cache.decode_attention(layer, full, q, out=out)
            moved["bytes"] += (2 * full.total + 4 * B) * H * D * 2 * layers
    else:
        graph = DecodeStepGraph(cache, slots, capacity_tokens=sum(lens) + B * total_steps, what="attention",
                                q_heads=H * group, max_len=max(lens) + total_steps)
        graph.k_in.copy_(new_rows)
        graph.v_in.copy_(new_rows)
        graph.q_in.copy_(q)
        graph.step()
        graph.record()

        def step():
            total = graph.step()
            moved["bytes"] += (2 * total + 4 * B) * H * D * 2 * layers

    for _ in range(max(warmup, 1)):
        step()
    sync()
    moved["bytes"] = 0
    # kernels per step, by the library's own count: eager steps count as they go, a replay runs what was recorded
    before = cache.backend.launches
    if eager:
        step()
        sync()
        moved["bytes"] = 0
    per_step = cache.backend.launches - before if eager else graph.launches_per_replay
    e0, e1 = _events()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    cache.check_device_status()
    return {"bytes": moved["bytes"], "ms": ms, "tokens": B * steps, "launches": per_step * steps,
            "config": {"workload": "llama3-8b-decode-attention-from-pages", "layers": layers, "kv_heads_per_gpu": H,
                       "query_heads_per_kv_head": group, "dtype": "bf16", "page_size": 16, "sequences": B,
                       "launch": "append + attention per layer, called from Python" if eager
                       else "one call per layer (append fused into attention; the attention kernel and the kernel that "
                            "combines its splits), replayed from a CUDA graph",
                       "step": "per layer: store 1 token/seq and attend over the pages (no gather); bytes = K and V "
                               "read once + appended rows",
                       "l2": "inputs larger than L2: each step reads ~%.1f GB of pool per GPU"
                             % (2 * sum(lens) * H * D * 2 * layers / 1e9)}}


WORKLOADS = {"prefill": chunked_prefill, "gather70b": gather_70b, "churn": churn, "decode-attn": decode_attention}
