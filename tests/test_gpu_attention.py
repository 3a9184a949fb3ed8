"""Decode attention over the pages against an fp32 reference over the gathered sequences.

This is a floating-point kernel (bf16/fp16 inputs, fp32 accumulation, probabilities rounded to the input
type before the P.V product), so the comparison has a tolerance: |got - want| <= 8e-3 + 2e-2 * |want|
against softmax(q k^T / sqrt(d)) v computed by torch in fp32 on the same values.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
ATOL, RTOL = 8e-3, 2e-2

# A launch that fills the GPU's resident warps several times over (44 sequences, 103k tokens, 8 KV heads):
# lengths on both sides of every page and split boundary (16 and 512 tokens) and a bulk of long sequences.
LARGE_LENS = (1, 15, 16, 17, 127, 128, 129, 511, 512, 513, 639, 640, 641, 1023, 1024, 1025, 2047, 2048, 2049, 4095,
              4096, 4097) + tuple(2500 + 97 * i for i in range(22))


def _reference(cache, layer, slots, q, scale):
    gb = cache.begin_gather(slots)
    kh, vh = cache.gather(layer, gb, "HND")                       # [Hkv, total, D]
    n, hq, d = q.shape
    group = hq // cache.num_kv_heads
    want = torch.empty(n, hq, d, dtype=torch.float32, device=q.device)
    for i in range(n):
        a, b = gb.cu[i], gb.cu[i + 1]
        k = kh[:, a:b].float().repeat_interleave(group, dim=0)     # [Hq, len, D]
        v = vh[:, a:b].float().repeat_interleave(group, dim=0)
        s = torch.einsum("hd,hld->hl", q[i].float(), k) * scale
        want[i] = torch.einsum("hl,hld->hd", torch.softmax(s, dim=-1), v)
    return gb, want


@pytest.mark.parametrize("case", [
    dict(dtype=torch.bfloat16, hkv=8, group=4, lens=(1, 15, 16, 17, 37, 500, 512, 513, 1500), seed=1),
    dict(dtype=torch.float16, hkv=2, group=8, lens=(700, 33, 4096 + 5), seed=2),
    dict(dtype=torch.bfloat16, hkv=4, group=1, lens=(64, 129, 2), seed=3),
    dict(dtype=torch.float16, hkv=1, group=4, lens=(3000, 16, 1024), seed=4),
    dict(dtype=torch.bfloat16, hkv=2, group=4, lens=(1, 31, 32, 33, 47, 48, 49, 1000, 2100), seed=5, ps=32),
    dict(dtype=torch.float16, hkv=2, group=2, lens=(63, 64, 65, 17, 700), seed=6, ps=64),
    dict(dtype=torch.bfloat16, hkv=8, group=4, lens=LARGE_LENS, seed=7),
    dict(dtype=torch.float16, hkv=8, group=2, lens=LARGE_LENS, seed=8),
    # one long sequence in a small batch: 40 splits, combined by the four-part form of the combining kernel,
    # eight query heads per KV head (two rounds of four warps)
    dict(dtype=torch.bfloat16, hkv=1, group=8, lens=(20000, 700, 5), seed=9),
    # more than 256 sequences: the grid has one CTA per possible split instead of the gap-free list
    dict(dtype=torch.float16, hkv=2, group=4, lens=tuple(300 + 3 * i for i in range(300)), seed=10),
])
def test_decode_attention_matches_fp32_reference(case):
    from barqtrain_b200 import BlockTableKVCache, _ffi

    backend = _ffi.require_cuda_backend()
    dtype, hkv, group, lens = case["dtype"], case["hkv"], case["group"], case["lens"]
    D, ps, n = 128, case.get("ps", 16), len(case["lens"])
    g = torch.Generator(device=DEV).manual_seed(case["seed"])
    pages = sum(-(-x // ps) for x in lens) + 3
    cache = BlockTableKVCache(2, hkv, D, page_size=ps, num_pages=pages, max_seqs=n,
                              max_blocks_per_seq=-(-max(lens) // ps), dtype=dtype, device=DEV, seed=case["seed"],
                              zero_pages=False)
    cache.pools.fill_(float("nan"))              # unused rows of partial pages must never leak into the result
    slots = [cache.open(i) for i in range(n)]
    total = sum(lens)
    for layer in range(2):
        k = torch.randn(total, hkv, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
        v = torch.randn(total, hkv, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
        batch = cache.begin_append(slots, lens) if layer == 0 else batch
        cache.append(layer, batch, k, v)
    cache.end_append(batch)
    q = torch.randn(n, hkv * group, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
    scale = D ** -0.5
    for layer in range(2):
        gb, want = _reference(cache, layer, slots, q, scale)
        got = cache.decode_attention(layer, gb, q)
        assert got.shape == q.shape and got.dtype == dtype
        err = (got.float() - want).abs()
        bound = ATOL + RTOL * want.abs()
        assert bool((err <= bound).all()), f"max err {err.max().item():.4g}, worst excess {(err - bound).max().item():.4g}"
        assert torch.isfinite(got.float()).all()
    # a subset of the batch in another order, through a strided q view
    order = list(range(n - 1, -1, -2))
    wide = torch.randn(len(order), hkv * group + 1, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
    q2 = wide[:, 1:]
    gb, want = _reference(cache, 1, [slots[i] for i in order], q2, scale)
    got = cache.decode_attention(1, gb, q2)
    assert bool(((got.float() - want).abs() <= ATOL + RTOL * want.abs()).all())
    assert backend.read_status(DEV) == 0


def test_decode_attention_with_pools_in_separate_allocations():
    """The C entry point with a V pool that does not lie behind the K pool in one allocation (here: before it),
    so a ring stage is filled by one copy per pool instead of one for both: same result as the cache's own call."""
    from barqtrain_b200 import BlockTableKVCache, _ffi

    backend = _ffi.require_cuda_backend()
    dtype, hkv, group, D, ps = torch.bfloat16, 2, 4, 128, 16
    lens = [1500, 40, 700, 2049]
    n = len(lens)
    g = torch.Generator(device=DEV).manual_seed(31)
    cache = BlockTableKVCache(1, hkv, D, page_size=ps, num_pages=sum(-(-x // ps) for x in lens) + 2, max_seqs=n,
                              max_blocks_per_seq=-(-max(lens) // ps), dtype=dtype, device=DEV, seed=31)
    slots = [cache.open(i) for i in range(n)]
    k = torch.randn(sum(lens), hkv, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
    v = torch.randn(sum(lens), hkv, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
    cache.append_step(slots, lens, [k], [v])
    q = torch.randn(n, hkv * group, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
    full = cache.begin_gather(slots)
    want = cache.decode_attention(0, full, q).clone()
    both = torch.empty(2, *cache.pools[0, 0].shape, dtype=dtype, device=DEV)      # V first, K behind it
    both[0].copy_(cache.pools[0, 1])
    both[1].copy_(cache.pools[0, 0])
    got = torch.empty_like(q)
    lib = backend.lib
    need = int(lib.barqkv_paged_decode_workspace_bytes(n, hkv, full.max_first, full.total, ps))
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    stream = full.stream
    rc = lib.barqkv_paged_decode_attention(
        cache._pool_ref, both[1].data_ptr(), both[0].data_ptr(), full.table_ref, full.p_first, n,
        q.data_ptr(), q.stride(0), q.stride(1), got.data_ptr(), got.stride(0), got.stride(1), hkv * group,
        float(D ** -0.5), 1, full.max_first, full.total, ws.data_ptr() if need else None, need, None, stream)
    assert rc == 0, backend.last_error()
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert backend.read_status(DEV) == 0


def test_decode_attention_flags_an_understated_sum_of_lengths():
    """The launch of a small batch is sized from the caller's sum of the lengths; a sum smaller than the real one
    must not lose pages silently: the status word says so (and a correct sum clears the matter)."""
    from barqtrain_b200 import BlockTableKVCache, _ffi

    backend = _ffi.require_cuda_backend()
    dtype, hkv, group, D, ps = torch.bfloat16, 2, 4, 128, 16
    lens = [1500, 2100, 900]
    n = len(lens)
    g = torch.Generator(device=DEV).manual_seed(41)
    cache = BlockTableKVCache(1, hkv, D, page_size=ps, num_pages=sum(-(-x // ps) for x in lens) + 2, max_seqs=n,
                              max_blocks_per_seq=-(-max(lens) // ps), dtype=dtype, device=DEV, seed=41)
    slots = [cache.open(i) for i in range(n)]
    k = torch.randn(sum(lens), hkv, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
    cache.append_step(slots, lens, [k], [k])
    q = torch.randn(n, hkv * group, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
    gb, want = _reference(cache, 0, slots, q, D ** -0.5)
    assert backend.read_status(DEV) == 0
    cache.decode_attention(0, gb, q, total_len=600)
    assert backend.read_status(DEV) == _ffi.S_CAPACITY
    got = cache.decode_attention(0, gb, q, total_len=sum(lens) + 100)        # an upper bound is fine
    assert bool(((got.float() - want).abs() <= ATOL + RTOL * want.abs()).all())
    assert backend.read_status(DEV) == 0


def test_decode_attention_argument_limits():
    from barqtrain_b200 import BlockTableKVCache, _ffi

    cache = BlockTableKVCache(1, 2, 64, page_size=16, num_pages=4, max_seqs=1, max_blocks_per_seq=2,
                              dtype=torch.bfloat16, device=DEV)
    s = cache.open(0)
    k = torch.zeros(3, 2, 64, dtype=torch.bfloat16, device=DEV)
    cache.append_step([s], [3], [k], [k])
    gb = cache.begin_gather([s])
    with pytest.raises(_ffi.BarqKVError, match="head_dim 128"):
        cache.decode_attention(0, gb, torch.zeros(1, 2, 64, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(ValueError):
        cache.decode_attention(0, gb, torch.zeros(2, 2, 64, dtype=torch.bfloat16, device=DEV))


def test_decode_attention_workspace_survives_changing_batches():
    """Sequences long enough for several splits, attended in batches of changing size through the one
    workspace the cache keeps: its contents on entry must not matter, so a larger batch after a smaller one
    must not trip over the smaller one's partial results (the workspace is filled with NaNs to start with)."""
    from barqtrain_b200 import BlockTableKVCache, _ffi

    backend = _ffi.require_cuda_backend()
    dtype, hkv, group, D, ps = torch.bfloat16, 2, 4, 128, 16
    lens = [1500, 2100, 700, 1024, 3000, 513, 40, 1800, 2500, 900, 1300, 2047]
    n = len(lens)
    g = torch.Generator(device=DEV).manual_seed(11)
    cache = BlockTableKVCache(1, hkv, D, page_size=ps, num_pages=sum(-(-x // ps) for x in lens), max_seqs=n,
                              max_blocks_per_seq=-(-max(lens) // ps), dtype=dtype, device=DEV, seed=11)
    slots = [cache.open(i) for i in range(n)]
    total = sum(lens)
    k = torch.randn(total, hkv, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
    v = torch.randn(total, hkv, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
    batch = cache.begin_append(slots, lens)
    cache.append(0, batch, k, v)
    cache.end_append(batch)
    scale = D ** -0.5
    for i, take in enumerate((n, 2, n, n, 5, 1, 9, n)):
        part = slots[:take]
        q = torch.randn(take, hkv * group, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
        gb, want = _reference(cache, 0, part, q, scale)
        got = cache.decode_attention(0, gb, q)
        assert bool(((got.float() - want).abs() <= ATOL + RTOL * want.abs()).all()), f"batch of {take}"
        if i == 0:
            assert cache._attn_ws is not None
            cache._attn_ws.view(torch.float32).fill_(float("nan"))
    assert backend.read_status(DEV) == 0


@pytest.mark.parametrize("case", [
    dict(dtype=torch.bfloat16, hkv=8, group=4, lens=(1, 15, 16, 17, 37, 500, 512, 513, 1500), ps=16),
    dict(dtype=torch.float16, hkv=2, group=8, lens=(700, 33, 2100), ps=32),
    dict(dtype=torch.bfloat16, hkv=1, group=4, lens=(64, 65, 1, 3000), ps=64),
    dict(dtype=torch.bfloat16, hkv=8, group=4, lens=LARGE_LENS, ps=16),
])
def test_append_fused_into_decode_attention(case):
    """``decode_update`` (one call: store the step's rows and attend) against append-then-attend on a twin
    cache: the pools end up bit-identical, the attention outputs are identical too (the same arithmetic on the
    same values), and both stay within the fp32 reference's tolerance.  Two steps in a row, so the second
    attends a token the first one stored."""
    from barqtrain_b200 import BlockTableKVCache, _ffi

    backend = _ffi.require_cuda_backend()
    dtype, hkv, group, lens, ps = case["dtype"], case["hkv"], case["group"], list(case["lens"]), case["ps"]
    D, n = 128, len(lens)
    g = torch.Generator(device=DEV).manual_seed(12)
    pages = sum(-(-(x + 2) // ps) for x in lens) + 2
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(3)).tolist()

    def make():
        c = BlockTableKVCache(1, hkv, D, page_size=ps, num_pages=pages, max_seqs=n, max_blocks_per_seq=-(-(max(lens) + 2) // ps),
                              dtype=dtype, device=DEV, free_order=order, zero_pages=False)
        c.pools.fill_(float("nan"))
        return c, [c.open(i) for i in range(n)]

    fused, fs = make()
    plain, pl = make()
    k = torch.randn(sum(lens), hkv, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
    v = torch.randn(sum(lens), hkv, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
    fused.append_step(fs, lens, [k], [v])
    plain.append_step(pl, lens, [k], [v])
    scale = D ** -0.5
    for _ in range(2):
        k1 = torch.randn(n, hkv, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
        v1 = torch.randn(n, hkv, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
        q = torch.randn(n, hkv * group, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
        launches = backend.launches
        new = fused.begin_append(fs, [1] * n)
        fused.end_append(new)
        full = fused.begin_gather(fs)
        mid = backend.launches
        got = fused.decode_update(0, full, k1, v1, q)
        # the attention kernel, plus the small kernel that combines the splits' partial results when sequences
        # are long enough to be split; the rest is table upkeep
        assert backend.launches - mid in (1, 2) and mid - launches <= 2
        new = plain.begin_append(pl, [1] * n)
        plain.append(0, new, k1, v1)
        plain.end_append(new)
        full_p = plain.begin_gather(pl)
        want = plain.decode_attention(0, full_p, q)
        torch.cuda.synchronize()
        used = torch.tensor(sorted(p for s_ in fs for p in fused.pages_of[s_]), device=DEV)
        assert torch.equal(fused.pools[:, :, :, used].view(torch.int16), plain.pools[:, :, :, used].view(torch.int16))
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        _, ref = _reference(plain, 0, pl, q, scale)
        assert torch.allclose(got.float(), ref, atol=ATOL, rtol=RTOL)
    fused.check_device_status()
    plain.check_device_status()


def test_decode_graph_with_attention_replays_what_eager_steps_compute():
    """``DecodeStepGraph(what="attention")``: one fused launch per layer recorded once and replayed; the pools and
    the last layer's attention output must equal a twin cache stepped eagerly (append + attention per layer)."""
    from barqtrain_b200 import BlockTableKVCache, DecodeStepGraph, _ffi

    backend = _ffi.require_cuda_backend()
    L, hkv, group, D, ps, dtype = 3, 2, 4, 128, 16, torch.bfloat16
    lens = [30, 700, 15, 129]
    n, steps = len(lens), 6
    g = torch.Generator(device=DEV).manual_seed(21)
    pages = sum(-(-(x + steps + 1) // ps) for x in lens)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(4)).tolist()

    def make():
        c = BlockTableKVCache(L, hkv, D, page_size=ps, num_pages=pages, max_seqs=n,
                              max_blocks_per_seq=-(-(max(lens) + steps + 1) // ps), dtype=dtype, device=DEV, free_order=order)
        return c, [c.open(i) for i in range(n)]

    a, sa = make()
    b, sb = make()
    for layer_rows in [[torch.randn(sum(lens), hkv, D, generator=g, device=DEV, dtype=torch.float32).to(dtype) for _ in range(L)]]:
        a.append_step(sa, lens, layer_rows, layer_rows)
        b.append_step(sb, lens, layer_rows, layer_rows)
    graph = DecodeStepGraph(a, sa, capacity_tokens=sum(lens) + n * (steps + 1), what="attention", q_heads=hkv * group,
                            max_len=max(lens) + steps + 1)
    out_b = torch.empty(n, hkv * group, D, dtype=dtype, device=DEV)
    for step in range(steps):
        rows = torch.randn(L, n, hkv, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
        q = torch.randn(n, hkv * group, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
        graph.k_in.copy_(rows)
        graph.v_in.copy_(rows.flip(0))
        graph.q_in.copy_(q)
        graph.step()
        if step == 1:
            graph.record()
            assert graph.launches_per_replay in (L, 2 * L)       # per layer: attention (+ the combining kernel)
        new = b.begin_append(sb, [1] * n)
        b.end_append(new)
        full = b.begin_gather(sb)
        for layer in range(L):
            b.append(layer, new, rows[layer], rows.flip(0)[layer])
            b.decode_attention(layer, full, q, out=out_b, max_len=max(lens) + steps + 1, total_len=graph.capacity)
        torch.cuda.synchronize()
        assert torch.equal(a.pools.view(torch.int16), b.pools.view(torch.int16)), step
        assert torch.equal(graph.attn_out.view(torch.int16), out_b.view(torch.int16)), step
    assert graph.graph is not None
    a.check_device_status()
    assert backend.read_status(DEV) == 0
