"""Parity of the CUDA path (through the C ABI) with the oracle and the reference's golden vectors.

Everything here is bit-exact: the path copies bit patterns, so there is no tolerance.
"""

import numpy as np
import pytest
import torch

from tests import scenarios as S

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _np(t):
    return S.bits(t).numpy()


@pytest.fixture(scope="module")
def backend():
    from barqtrain_b200 import _ffi

    be = _ffi.require_cuda_backend()
    assert be.read_status(DEV) == 0
    yield be
    assert be.read_status(DEV) == 0, "a kernel guard fired during the module"


# ---------------------------------------------------------------------------
# reference layout (identity block table)
# ---------------------------------------------------------------------------
def test_reference_known_answer_on_gpu(backend, golden_dir):
    """The reference's own test (tests/test_kv_cache.py:24-47) with the append on the GPU."""
    from barqtrain_b200 import BarqPagedKVCacheLayer

    gold = np.load(golden_dir / "ref_known_answer.npz")
    ctor, steps = S.ref_known_answer()
    layer = BarqPagedKVCacheLayer(**ctor)
    launches = backend.launches
    for i, (k, v) in enumerate(steps):
        ks, vs = layer.update(k.to(DEV), v.to(DEV))
        assert np.array_equal(_np(ks), gold[f"ret_k_{i}"])
        assert np.array_equal(_np(vs), gold[f"ret_v_{i}"])
        assert np.array_equal(_np(layer.keys), gold[f"keys_{i}"])
        assert np.array_equal(_np(layer.values), gold[f"values_{i}"])
        assert np.array_equal(layer.seq_lens.cpu().numpy(), gold[f"lens_{i}"])
        assert layer.get_seq_length() == int(gold[f"seq_length_{i}"])
    assert ks.shape == (1, 2, 5, 4) and vs.shape == (1, 2, 5, 4)
    assert torch.equal(ks[:, :, :3].cpu(), steps[0][0]) and torch.equal(ks[:, :, 3:].cpu(), steps[1][0])
    assert torch.equal(vs[:, :, :3].cpu(), steps[0][1]) and torch.equal(vs[:, :, 3:].cpu(), steps[1][1])
    assert backend.launches == launches + 2, "the native kernel must have been launched once per append"
    gk, gv = layer.gather_contiguous()
    assert gk.is_contiguous() and torch.equal(gk, ks) and torch.equal(gv, vs)


@pytest.mark.parametrize("dtype_name", ["fp32", "fp64", "fp16", "bf16"])
def test_legacy_script_against_reference(backend, golden_dir, dtype_name):
    from barqtrain_b200 import BarqPagedKVCacheLayer

    gold = np.load(golden_dir / f"legacy_{dtype_name}.npz")
    ctor, ops = S.legacy_script(dtype_name)
    ops = [tuple(x.to(DEV) if isinstance(x, torch.Tensor) and x.is_floating_point() else x for x in op) for op in ops]
    layer = BarqPagedKVCacheLayer(**ctor)

    def check(lay, i, op):
        assert np.array_equal(_np(lay.keys), gold[f"keys_{i}"]), (i, op[0])
        assert np.array_equal(_np(lay.values), gold[f"values_{i}"]), (i, op[0])
        assert np.array_equal(lay.seq_lens.cpu().numpy(), gold[f"lens_{i}"]), (i, op[0])
        assert lay.current_batch_size == int(gold[f"batch_{i}"])
        assert lay.get_seq_length() == int(gold[f"seq_length_{i}"])
        if lay.current_batch_size:
            ks, vs = lay.current_tensors()
            assert np.array_equal(_np(ks), gold[f"cur_k_{i}"])
            assert np.array_equal(_np(vs), gold[f"cur_v_{i}"])
            for mode in ("vector", "bulk"):
                gk, gv = lay.gather_contiguous(mode=mode)
                lens = lay.seq_lens.cpu().tolist()
                for b in range(lay.current_batch_size):
                    assert torch.equal(S.bits(gk[b, :, :lens[b]]), S.bits(ks[b, :, :lens[b]])), (i, mode, b)
                    assert torch.equal(S.bits(gv[b, :, :lens[b]]), S.bits(vs[b, :, :lens[b]])), (i, mode, b)
                    assert not gk[b, :, lens[b]:].any() and not gv[b, :, lens[b]:].any()

    S.run_legacy_script(layer, ops, check)


def test_legacy_capacity_is_all_or_nothing(backend, golden_dir):
    """The reference's CUDA launcher refuses the whole call (paged_kv_cache.cu:92-99);
    so does this path, on the host and - when the host check is bypassed - on the device."""
    from barqtrain_b200 import BarqPagedKVCacheLayer

    ctor, ops = S.legacy_overflow_script()
    ops = [tuple(x.to(DEV) if isinstance(x, torch.Tensor) and x.is_floating_point() else x for x in op) for op in ops]
    layer = BarqPagedKVCacheLayer(**ctor)
    S.run_legacy_script(layer, ops[:3], lambda *a: None)
    before = (layer.keys.clone(), layer.values.clone(), layer.seq_lens.clone())
    with pytest.raises(RuntimeError, match="paged KV cache capacity exceeded: requested 9 tokens, max_cache_len=8"):
        layer.append(ops[3][1], ops[3][2])
    assert torch.equal(layer.keys, before[0]) and torch.equal(layer.seq_lens, before[2])
    # without the host-side hint the call reads the lengths back, as the reference does
    with pytest.raises(RuntimeError, match="capacity exceeded"):
        backend.paged_kv_append_(layer.keys, layer.values, layer.seq_lens, ops[3][1], ops[3][2])
    # a wrong hint reaches the kernel: it must write nothing, keep seq_lens and flag the call
    backend.paged_kv_append_(layer.keys, layer.values, layer.seq_lens, ops[3][1], ops[3][2], max_start=0)
    assert backend.read_status(DEV) == 2
    assert torch.equal(layer.keys, before[0]) and torch.equal(layer.values, before[1])
    assert torch.equal(layer.seq_lens, before[2])
    # and the ticket was re-armed: the next valid call works
    ok_k, ok_v = ops[3][1][:, :, :3], ops[3][2][:, :, :3]
    backend.paged_kv_append_(layer.keys, layer.values, layer.seq_lens, ok_k, ok_v)
    assert layer.seq_lens.cpu().tolist() == [5, 8, 8]
    assert backend.read_status(DEV) == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_legacy_append_reads_transposed_views_without_copy(backend, dtype):
    """[B, T, H, D].transpose(1, 2) - what HF attention passes - gives the same cache as a contiguous copy."""
    from barqtrain_b200 import BarqPagedKVCacheLayer
    from oracle.paged_kv_oracle import OracleLayer

    g = torch.Generator().manual_seed(5)
    B, T, H, D = 3, 37, 4, 64
    a, b = BarqPagedKVCacheLayer(B, 64, 16), OracleLayer(B, 64, 16)
    for T_i in (T, 1, 1, 20):
        k = S.randn(g, (B, T_i, H, D), dtype)
        v = S.randn(g, (B, T_i, H, D), dtype)
        a.append(k.to(DEV).transpose(1, 2), v.to(DEV).transpose(1, 2))
        b.append(k.transpose(1, 2), v.transpose(1, 2))
        assert torch.equal(S.bits(a.keys), S.bits(b.keys)) and torch.equal(S.bits(a.values), S.bits(b.values))
        assert a.seq_lens.cpu().tolist() == b.seq_lens.tolist()


@pytest.mark.parametrize("shape", [(2, 3, 5, 3, torch.float32), (1, 2, 9, 5, torch.float16), (2, 1, 4, 4, torch.float64),
                                   (2, 2, 7, 1, torch.float32)])
def test_legacy_odd_row_sizes_take_narrow_vectors(backend, shape):
    """Rows of 12, 10, 32 and 4 bytes: the kernel drops to 4-, 2-, 16- and 4-byte accesses."""
    from barqtrain_b200 import BarqPagedKVCacheLayer
    from oracle.paged_kv_oracle import OracleLayer

    B, H, T, D, dtype = shape
    g = torch.Generator().manual_seed(11)
    a, b = BarqPagedKVCacheLayer(B, 24, 4), OracleLayer(B, 24, 4)
    for T_i in (T, 1, T):
        k, v = S.randn(g, (B, H, T_i, D), dtype), S.randn(g, (B, H, T_i, D), dtype)
        a.append(k.to(DEV), v.to(DEV))
        b.append(k, v)
    assert torch.equal(S.bits(a.keys), S.bits(b.keys)) and torch.equal(S.bits(a.values), S.bits(b.values))
    for mode in ("vector", "auto"):
        gk, gv = a.gather_contiguous(mode=mode)
        rk, rv = b.current_tensors()
        assert torch.equal(S.bits(gk), S.bits(rk)) and torch.equal(S.bits(gv), S.bits(rv))


# ---------------------------------------------------------------------------
# block table
# ---------------------------------------------------------------------------
SMALL = {
    "small_paged_fp32": {},
    "small_paged_bf16": dict(dtype=torch.bfloat16, kv_heads=2, head_dim=128, prefill=(21, 64, 90),
                             decode_steps=5, num_pages=40, seed=2001),
    "small_paged_fp16_ps32": dict(dtype=torch.float16, kv_heads=8, head_dim=128, page_size=32,
                                  prefill=(100, 33), decode_steps=3, num_pages=16, seed=2002, num_layers=1),
}


@pytest.mark.parametrize("mode", ["vector", "bulk"])
@pytest.mark.parametrize("name", sorted(SMALL))
def test_small_paged_against_reference(backend, golden_dir, name, mode):
    """Prefill + decode through a shuffled free list; every step's gather and the final pages
    must equal what the unmodified reference produced (tests/golden)."""
    from barqtrain_b200 import BlockTableKVCache

    gold = np.load(golden_dir / f"{name}.npz")
    sc = S.small_paged(**SMALL[name])
    finals = sc.final_lengths()
    nseq = len(finals)
    cache = BlockTableKVCache(sc.num_layers, sc.kv_heads, sc.head_dim, page_size=sc.page_size,
                              num_pages=sc.num_pages, max_seqs=nseq + 1, max_blocks_per_seq=8, dtype=sc.dtype,
                              device=DEV, free_order=gold["free_list"].tolist(), gather_mode=mode)
    slots = [cache.open(s) for s in range(nseq)]
    for i, step in enumerate(sc.steps):
        counts = [step[0][s][0].shape[1] for s in range(nseq)]
        # packed [total, H, D] rows per layer: sequences back to back
        k_layers = [torch.cat([kv[0].transpose(0, 1) for kv in step[l]], 0).to(DEV) for l in range(sc.num_layers)]
        v_layers = [torch.cat([kv[1].transpose(0, 1) for kv in step[l]], 0).to(DEV) for l in range(sc.num_layers)]
        cache.append_step(slots, counts, k_layers, v_layers)
        gb = cache.begin_gather(slots)
        col = 0
        for l in range(sc.num_layers):
            kh, vh = cache.gather(l, gb, "HND")
            kn, vn = cache.gather(l, gb, "NHD")
            assert torch.equal(kh, kn.transpose(0, 1)) and torch.equal(vh, vn.transpose(0, 1))
            for s in range(nseq):
                a, b = gb.cu[s], gb.cu[s + 1]
                assert S.digest(kh[:, a:b], vh[:, a:b]) == str(gold["gather_digests"][i][col]), (i, l, s)
                col += 1
    for l in range(sc.num_layers):
        for s, n in enumerate(finals):
            pages = -(-n // sc.page_size)
            k_all = torch.stack([cache.logical_page(l, s, j)[0] for j in range(pages)], dim=1)
            v_all = torch.stack([cache.logical_page(l, s, j)[1] for j in range(pages)], dim=1)
            assert np.array_equal(_np(k_all), gold[f"keys_l{l}_s{s}"])     # zero tails included
            assert np.array_equal(_np(v_all), gold[f"values_l{l}_s{s}"])
            gk, gv = cache.gather_sequence(l, s, "NHD")
            assert gk.shape == (n, sc.kv_heads, sc.head_dim)
    # pages nobody owns were never written
    owned = sorted(p for s in slots for p in cache.pages_of[s])
    free = [p for p in range(sc.num_pages) if p not in owned]
    assert not cache.pools[:, :, :, free].any()
    cache.check_device_status()
    st = cache.stats()
    assert st.pages_resident == len(owned) == sum(-(-n // sc.page_size) for n in finals) == st.pages_peak


def _ragged_case(seed, nseq, lo, hi, H, D, ps, dtype, layers, chunk, decode):
    g = torch.Generator().manual_seed(seed)
    lens = S.ragged_lengths(g, nseq, lo, hi)
    max_len = max(lens) + decode
    pages = sum(-(-(n + decode) // ps) for n in lens) + 7
    order = torch.randperm(pages, generator=g).tolist()
    return g, lens, max_len, pages, order


@pytest.mark.parametrize("mode", ["vector", "bulk"])
@pytest.mark.parametrize("cfg", [
    dict(seed=31, nseq=24, lo=1, hi=700, H=8, D=128, ps=16, dtype=torch.bfloat16, layers=2, chunk=256, decode=3),
    dict(seed=32, nseq=5, lo=300, hi=2100, H=8, D=128, ps=32, dtype=torch.float16, layers=1, chunk=512, decode=2),
    dict(seed=33, nseq=40, lo=0, hi=90, H=1, D=128, ps=16, dtype=torch.bfloat16, layers=1, chunk=64, decode=4),
    dict(seed=34, nseq=7, lo=1, hi=150, H=3, D=80, ps=8, dtype=torch.float32, layers=1, chunk=50, decode=2),
])
def test_ragged_chunked_prefill_and_decode_against_c_oracle(backend, cfg, mode):
    """Scaled-down shapes of the large configurations: chunked prefill of a ragged batch into a
    shuffled pool, then decode steps; whole pools and all gathers equal the C oracle's."""
    from barqtrain_b200 import BlockTableKVCache
    from oracle import c_oracle

    g, lens, max_len, pages, order = _ragged_case(**cfg)
    H, D, ps, dtype, L = cfg["H"], cfg["D"], cfg["ps"], cfg["dtype"], cfg["layers"]
    nseq = len(lens)
    cache = BlockTableKVCache(L, H, D, page_size=ps, num_pages=pages, max_seqs=nseq,
                              max_blocks_per_seq=-(-max_len // ps), dtype=dtype, device=DEV, free_order=order,
                              gather_mode=mode)
    slots = [cache.open(s) for s in range(nseq)]
    ref_k = [torch.zeros(H, pages, ps, D, dtype=dtype) for _ in range(L)]
    ref_v = [torch.zeros(H, pages, ps, D, dtype=dtype) for _ in range(L)]
    done = [0] * nseq

    def step(counts):
        total = sum(counts)
        batch = cache.begin_append(slots, counts)
        table = cache.table_host.clone()
        start = torch.tensor(done, dtype=torch.int32)
        cu = torch.tensor(batch.cu, dtype=torch.int32)
        for l in range(L):
            k = S.randn(g, (total, H, D), dtype)
            v = S.randn(g, (total, H, D), dtype)
            cache.append(l, batch, k.to(DEV), v.to(DEV))
            assert c_oracle.append_paged(ref_k[l], ref_v[l], table, None, start, cu, k, v) == 0
        cache.end_append(batch)
        for s, c in enumerate(counts):
            done[s] += c

    while any(d < n for d, n in zip(done, lens)):
        step([min(cfg["chunk"], n - d) for d, n in zip(done, lens)])
    for _ in range(cfg["decode"]):
        step([1] * nseq)

    for l in range(L):
        assert torch.equal(S.bits(cache.pools[l, 0]), S.bits(ref_k[l])), "K pool differs"
        assert torch.equal(S.bits(cache.pools[l, 1]), S.bits(ref_v[l])), "V pool differs"
    gb = cache.begin_gather(slots)
    total = gb.total
    lens_t = torch.tensor(done, dtype=torch.int32)
    cu_t = torch.tensor(gb.cu[:-1], dtype=torch.int32)
    table = cache.table_host.clone()
    for l in range(L):
        want_k = torch.zeros(total, H, D, dtype=dtype)
        want_v = torch.zeros(total, H, D, dtype=dtype)
        assert c_oracle.gather_paged(ref_k[l], ref_v[l], table, None, lens_t, cu_t, want_k, want_v) == 0
        kn, vn = cache.gather(l, gb, "NHD")
        kh, vh = cache.gather(l, gb, "HND")
        assert torch.equal(S.bits(kn), S.bits(want_k)) and torch.equal(S.bits(vn), S.bits(want_v))
        assert torch.equal(S.bits(kh.transpose(0, 1)), S.bits(want_k))
        assert torch.equal(S.bits(vh.transpose(0, 1)), S.bits(want_v))
    cache.check_device_status()


@pytest.mark.parametrize("layout", ["HND", "NHD"])
@pytest.mark.parametrize("cfg", [
    dict(H=8, D=128, ps=16, dtype=torch.bfloat16, lens=(37, 50, 16, 0, 1, 255), news=((1,) * 6, (3, 0, 16, 5, 1, 2))),
    dict(H=1, D=128, ps=16, dtype=torch.float16, lens=(15, 16, 17, 700), news=((1, 1, 1, 1), (16, 1, 15, 0))),
    dict(H=2, D=64, ps=32, dtype=torch.float32, lens=(31, 64, 5), news=((1, 1, 1), (2, 32, 27))),
    dict(H=3, D=5, ps=4, dtype=torch.float32, lens=(3, 9), news=((1, 1), (2, 4))),     # 20-byte rows: two launches
])
def test_update_in_one_launch_equals_append_then_gather(backend, cfg, layout):
    """``update`` (append + gather, one kernel for decode-sized appends) against the two separate
    calls on a twin cache: same pools, same gathered tensors, and the expected launch count."""
    from barqtrain_b200 import BlockTableKVCache

    H, D, ps, dtype = cfg["H"], cfg["D"], cfg["ps"], cfg["dtype"]
    g = torch.Generator().manual_seed(61)
    n = len(cfg["lens"])
    order = torch.randperm(64, generator=g).tolist()

    def make():
        c = BlockTableKVCache(1, H, D, page_size=ps, num_pages=64, max_seqs=n, max_blocks_per_seq=48,
                              dtype=dtype, device=DEV, free_order=order)
        return c, [c.open(i) for i in range(n)]

    fused, fs = make()
    plain, pl = make()
    k0 = S.randn(g, (sum(cfg["lens"]), H, D), dtype).to(DEV)
    v0 = S.randn(g, (sum(cfg["lens"]), H, D), dtype).to(DEV)
    fused.append_step(fs, cfg["lens"], [k0], [v0])
    plain.append_step(pl, cfg["lens"], [k0], [v0])
    one_launch = (D * k0.element_size()) % 16 == 0
    for counts in cfg["news"]:
        k = S.randn(g, (sum(counts), H, D), dtype).to(DEV)
        v = S.randn(g, (sum(counts), H, D), dtype).to(DEV)
        plain.append_step(pl, counts, [k], [v])
        want_k, want_v = plain.gather(0, plain.begin_gather(pl), layout)
        new = fused.begin_append(fs, counts)
        fused.end_append(new)
        full = fused.begin_gather(fs)
        before = backend.launches
        got_k, got_v = fused.update(0, new, full, k, v, layout)
        assert backend.launches - before == (1 if one_launch else 2)
        assert torch.equal(S.bits_dev(got_k), S.bits_dev(want_k)) and torch.equal(S.bits_dev(got_v), S.bits_dev(want_v))
        assert torch.equal(S.bits_dev(fused.pools), S.bits_dev(plain.pools))
    fused.check_device_status()


def test_all_layers_in_one_launch_equals_per_layer_appends(backend):
    """``append_layers`` (gridDim.y = layers) against one ``append`` per layer on a twin cache."""
    from barqtrain_b200 import BlockTableKVCache

    L, H, D, ps, dtype = 5, 2, 128, 16, torch.float16
    g = torch.Generator().manual_seed(23)
    order = torch.randperm(80, generator=g).tolist()

    def make():
        c = BlockTableKVCache(L, H, D, page_size=ps, num_pages=80, max_seqs=4, max_blocks_per_seq=20, dtype=dtype,
                              device=DEV, free_order=order)
        return c, [c.open(i) for i in range(4)]

    one, s1 = make()
    many, s2 = make()
    for counts in ((70, 3, 0, 129), (1, 1, 1, 1), (15, 0, 16, 2), (1, 1, 1, 1)):
        total = sum(counts)
        wide_k = S.randn(g, (L, total, H + 1, D), dtype).to(DEV)      # rows are a strided slice of a wider tensor
        wide_v = S.randn(g, (L, total, H + 1, D), dtype).to(DEV)
        k_all, v_all = wide_k[:, :, :H], wide_v[:, :, :H]
        b1 = one.begin_append(s1, counts)
        before = backend.launches
        one.append_layers(b1, k_all, v_all)
        assert backend.launches - before == 1
        one.end_append(b1)
        many.append_step(s2, counts, list(k_all.unbind(0)), list(v_all.unbind(0)))
        assert torch.equal(S.bits_dev(one.pools), S.bits_dev(many.pools))
    # the same rows for every layer (layer stride 0)
    k1 = S.randn(g, (4, H, D), dtype).to(DEV)
    b1 = one.begin_append(s1, [1] * 4)
    one.append_layers(b1, k1.expand(L, 4, H, D), k1.expand(L, 4, H, D))
    one.end_append(b1)
    many.append_step(s2, [1] * 4, [k1] * L, [k1] * L)
    assert torch.equal(S.bits_dev(one.pools), S.bits_dev(many.pools))
    one.check_device_status()


@pytest.mark.parametrize("num_out", [1, 2, 3, 4, 6])
def test_update_of_all_layers_in_one_call_for_any_number_of_outputs(backend, num_out):
    """``update_layers``: with an even number of outputs (or one per layer) odd layers run on the library's
    second stream beside the even ones; with an odd number, or a single pair, all stay on one stream.  Whatever
    the schedule, the pools and the outputs of the last ``num_out`` layers must equal per-layer ``update``
    calls on a twin cache, and work queued on the caller's stream afterwards must see every layer done."""
    from barqtrain_b200 import BlockTableKVCache

    L, H, D, ps, dtype = 6, 2, 128, 16, torch.float16
    lens = [500, 31, 16, 1200, 257, 64, 900]
    n = len(lens)
    g = torch.Generator().manual_seed(num_out)
    pages = sum(-(-(x + 8) // ps) for x in lens)
    order = torch.randperm(pages, generator=g).tolist()

    def make():
        c = BlockTableKVCache(L, H, D, page_size=ps, num_pages=pages, max_seqs=n, max_blocks_per_seq=-(-(max(lens) + 8) // ps),
                              dtype=dtype, device=DEV, free_order=order)
        return c, [c.open(i) for i in range(n)]

    fast, fs = make()
    slow, ss = make()
    k0 = [S.randn(g, (sum(lens), H, D), dtype).to(DEV) for _ in range(L)]
    fast.append_step(fs, lens, k0, k0[::-1])
    slow.append_step(ss, lens, k0, k0[::-1])
    cap = sum(lens) + 8 * n
    outs = [(torch.zeros(H, cap, D, dtype=dtype, device=DEV), torch.zeros(H, cap, D, dtype=dtype, device=DEV))
            for _ in range(num_out)]
    for step in range(5):
        k = S.randn(g, (L, n, H, D), dtype).to(DEV)
        v = S.randn(g, (L, n, H, D), dtype).to(DEV)
        new = fast.begin_append(fs, [1] * n)
        fast.end_append(new)
        full = fast.begin_gather(fs)
        before = backend.launches
        fast.update_layers(new, full, k, v, outs, "HND", tokens_hint=cap, one_stream=step % 2 == 1)
        assert backend.launches - before == L
        # copies queued behind the call on the same stream: they must read finished outputs
        snap = [(ko.clone(), vo.clone()) for ko, vo in outs]
        slow.append_step(ss, [1] * n, list(k.unbind(0)), list(v.unbind(0)))
        gb = slow.begin_gather(ss)
        for layer in range(L - min(num_out, L), L):
            want_k, want_v = slow.gather(layer, gb, "HND")
            got_k, got_v = snap[layer % num_out]
            assert torch.equal(S.bits_dev(got_k[:, :gb.total]), S.bits_dev(want_k)), (step, layer)
            assert torch.equal(S.bits_dev(got_v[:, :gb.total]), S.bits_dev(want_v)), (step, layer)
        assert torch.equal(S.bits_dev(fast.pools), S.bits_dev(slow.pools)), step
        # inside the call a launch leaves its hand-out counters to its neighbour to clear; after it all are zero
        assert int(backend.work_words(DEV).abs().sum()) == 0, step
    fast.check_device_status()
    assert backend.read_status(DEV) == 0


@pytest.mark.parametrize("L,num_out", [(1, 1), (2, 2), (3, 2), (5, 2), (4, 4), (5, 3)])
def test_gather_of_every_layer_from_one_call(backend, L, num_out):
    """``gather_each_layer`` (one native call, one chained launch per layer, neighbouring layers on two streams
    when the outputs allow it) against ``gather`` layer by layer: the last ``num_out`` layers' outputs, read by
    work queued behind the call, and counters that are zero again after it."""
    from barqtrain_b200 import BlockTableKVCache

    H, D, ps, dtype = 2, 128, 16, torch.bfloat16
    lens = [700, 31, 1200, 64, 16]
    n = len(lens)
    g = torch.Generator().manual_seed(90 + L)
    pages = sum(-(-x // ps) for x in lens) + 1
    cache = BlockTableKVCache(L, H, D, page_size=ps, num_pages=pages, max_seqs=n, max_blocks_per_seq=-(-max(lens) // ps),
                              dtype=dtype, device=DEV, free_order=torch.randperm(pages, generator=g).tolist())
    slots = [cache.open(i) for i in range(n)]
    rows = [S.randn(g, (sum(lens), H, D), dtype).to(DEV) for _ in range(L)]
    cache.append_step(slots, lens, rows, rows[::-1])
    gb = cache.begin_gather(slots)
    outs = [(torch.zeros(H, gb.total, D, dtype=dtype, device=DEV), torch.zeros(H, gb.total, D, dtype=dtype, device=DEV))
            for _ in range(num_out)]
    for turn in range(4):
        before = backend.launches
        cache.gather_each_layer(gb, outs, "HND", one_stream=turn == 3)
        assert backend.launches - before == L
        snap = [(ko.clone(), vo.clone()) for ko, vo in outs]
        torch.cuda.synchronize()
        assert int(backend.work_words(DEV).abs().sum()) == 0, turn
        for layer in range(L - min(num_out, L), L):
            want_k, want_v = cache.gather(layer, gb, "HND")
            assert torch.equal(S.bits_dev(snap[layer % num_out][0]), S.bits_dev(want_k)), (turn, layer)
            assert torch.equal(S.bits_dev(snap[layer % num_out][1]), S.bits_dev(want_v)), (turn, layer)
        for ko, vo in outs:
            ko.zero_()
            vo.zero_()
    cache.check_device_status()
    assert backend.read_status(DEV) == 0


@pytest.mark.parametrize("L,odd_one", [(1, None), (2, None), (4, 2), (5, 0), (5, 4), (3, 1)])
def test_append_of_every_layer_from_one_call(backend, L, odd_one):
    """``append_each_layer`` (one native call, one chained launch per layer) against ``append`` layer by layer on a
    twin cache: page-sized chunks (the launches hand pages out through counters that they clear for one another)
    and single tokens, with one layer's rows at an address that is not 16-byte aligned (that layer takes the
    kernel without counters in the middle of the chain).  Same pools, counters zero after every call."""
    from barqtrain_b200 import BlockTableKVCache

    H, D, ps, dtype = 2, 128, 16, torch.float16
    counts_per_step = ([700, 48, 1200, 16], [64, 17, 33, 512], [1, 1, 1, 1])
    n = 4
    g = torch.Generator().manual_seed(70 + L)
    pages = sum(-(-sum(c[i] for c in counts_per_step) // ps) + 1 for i in range(n))
    order = torch.randperm(pages, generator=g).tolist()

    def make():
        c = BlockTableKVCache(L, H, D, page_size=ps, num_pages=pages, max_seqs=n, max_blocks_per_seq=pages, dtype=dtype,
                              device=DEV, free_order=order)
        return c, [c.open(i) for i in range(n)]

    fast, fs = make()
    slow, ss = make()
    for counts in counts_per_step:
        total = sum(counts)
        rows_k, rows_v = [], []
        for layer in range(L):
            if layer == odd_one:      # same shape and strides, but the rows start 6 bytes into a 16-byte line
                flat = S.randn(g, (2 * total * H * D + 3,), dtype).to(DEV)
                rows_k.append(flat[3:3 + total * H * D].view(total, H, D))
                rows_v.append(flat[3 + total * H * D:].view(total, H, D))
            else:
                rows_k.append(S.randn(g, (total, H, D), dtype).to(DEV))
                rows_v.append(S.randn(g, (total, H, D), dtype).to(DEV))
        batch = fast.begin_append(fs, counts)
        before = backend.launches
        fast.append_each_layer(batch, rows_k, rows_v)
        assert backend.launches - before == L
        fast.end_append(batch)
        torch.cuda.synchronize()
        assert int(backend.work_words(DEV).abs().sum()) == 0, counts
        batch = slow.begin_append(ss, counts)
        for layer in range(L):
            slow.append(layer, batch, rows_k[layer], rows_v[layer])
        slow.end_append(batch)
        assert torch.equal(S.bits_dev(fast.pools), S.bits_dev(slow.pools)), counts
    fast.check_device_status()
    assert backend.read_status(DEV) == 0


@pytest.mark.parametrize("L", [1, 2, 3, 5])
def test_update_of_all_layers_leaves_the_counters_zero_for_any_number_of_layers(backend, L):
    """``update_layers`` chains its launches: each clears the hand-out counters of its neighbours and only the
    last launch of a chain its own.  For chains of every length, on one stream and on two, the counters must be
    zero after the call and the next call (same buffer) must gather the right rows."""
    from barqtrain_b200 import BlockTableKVCache

    H, D, ps, dtype = 2, 128, 16, torch.bfloat16
    lens = [700, 31, 1200, 64]
    n = len(lens)
    g = torch.Generator().manual_seed(50 + L)
    pages = sum(-(-(x + 8) // ps) for x in lens)
    order = torch.randperm(pages, generator=g).tolist()

    def make():
        c = BlockTableKVCache(L, H, D, page_size=ps, num_pages=pages, max_seqs=n, max_blocks_per_seq=-(-(max(lens) + 8) // ps),
                              dtype=dtype, device=DEV, free_order=order)
        return c, [c.open(i) for i in range(n)]

    fast, fs = make()
    slow, ss = make()
    k0 = [S.randn(g, (sum(lens), H, D), dtype).to(DEV) for _ in range(L)]
    fast.append_step(fs, lens, k0, k0)
    slow.append_step(ss, lens, k0, k0)
    cap = sum(lens) + 8 * n
    outs = [(torch.zeros(H, cap, D, dtype=dtype, device=DEV), torch.zeros(H, cap, D, dtype=dtype, device=DEV))
            for _ in range(L)]
    for step in range(6):
        k = S.randn(g, (L, n, H, D), dtype).to(DEV)
        new = fast.begin_append(fs, [1] * n)
        fast.end_append(new)
        full = fast.begin_gather(fs)
        fast.update_layers(new, full, k, k, outs, "HND", tokens_hint=cap, one_stream=step % 3 == 2)
        torch.cuda.synchronize()
        assert int(backend.work_words(DEV).abs().sum()) == 0, step
        slow.append_step(ss, [1] * n, list(k.unbind(0)), list(k.unbind(0)))
        gb = slow.begin_gather(ss)
        for layer in range(L):
            want_k, want_v = slow.gather(layer, gb, "HND")
            assert torch.equal(S.bits_dev(outs[layer][0][:, :gb.total]), S.bits_dev(want_k)), (step, layer)
            assert torch.equal(S.bits_dev(outs[layer][1][:, :gb.total]), S.bits_dev(want_v)), (step, layer)
    fast.check_device_status()
    assert backend.read_status(DEV) == 0


@pytest.mark.parametrize("H", [8, 1])
def test_decode_step_graph_replays_what_eager_steps_compute(backend, H):
    """A decode step recorded into a CUDA graph: every replay must leave the same pools and gathered
    tensors as eager append + gather on a twin cache, across page boundaries and growing lengths."""
    from barqtrain_b200 import BlockTableKVCache, DecodeStepGraph

    L, D, ps, dtype, B = 3, 128, 16, torch.bfloat16, 5
    g = torch.Generator().manual_seed(17)
    lens = [14, 15, 16, 33, 100]
    order = torch.randperm(96, generator=g).tolist()

    def make():
        c = BlockTableKVCache(L, H, D, page_size=ps, num_pages=96, max_seqs=B, max_blocks_per_seq=16, dtype=dtype,
                              device=DEV, free_order=order)
        return c, [c.open(i) for i in range(B)]

    fast, fs = make()
    slow, ss = make()
    k0 = [S.randn(g, (sum(lens), H, D), dtype).to(DEV) for _ in range(L)]
    v0 = [S.randn(g, (sum(lens), H, D), dtype).to(DEV) for _ in range(L)]
    fast.append_step(fs, lens, k0, v0)
    slow.append_step(ss, lens, k0, v0)
    steps = DecodeStepGraph(fast, fs, capacity_tokens=sum(lens) + B * 24)
    for i in range(20):
        if i == 2:
            steps.record()
        k = S.randn(g, (L, B, H, D), dtype).to(DEV)
        v = S.randn(g, (L, B, H, D), dtype).to(DEV)
        steps.k_in.copy_(k)
        steps.v_in.copy_(v)
        before = backend.launches
        total = steps.step()
        # eager steps launch one kernel per layer, a replay makes no launch through the library; either may
        # be preceded by the small kernel that patches changed block-table entries
        assert backend.launches - before in ((L, L + 1) if i < 2 else (0, 1))
        assert i < 2 or steps.launches_per_replay == L
        slow.append_step(ss, [1] * B, list(k.unbind(0)), list(v.unbind(0)))
        gb = slow.begin_gather(ss)
        assert total == gb.total == sum(lens) + B * (i + 1)
        for layer in (L - 2, L - 1):                      # the two buffer pairs still hold the last two layers
            want_k, want_v = slow.gather(layer, gb, "HND")
            got_k, got_v = steps.outputs(layer)
            assert torch.equal(S.bits_dev(got_k), S.bits_dev(want_k)), (i, layer)
            assert torch.equal(S.bits_dev(got_v), S.bits_dev(want_v)), (i, layer)
        assert torch.equal(S.bits_dev(fast.pools), S.bits_dev(slow.pools)), i
    assert steps.graph is not None
    with pytest.raises(ValueError, match="capacity"):
        for _ in range(10):
            steps.step()
    backend.read_status(DEV)


def test_release_recycles_pages_and_keeps_live_sequences_intact(backend):
    """Continuous-batching churn in small: sequences finish, their pages go back to the free
    list and are handed to new sequences; live sequences always gather to what was appended."""
    from barqtrain_b200 import BlockTableKVCache

    g = torch.Generator().manual_seed(77)
    H, D, ps, dtype, L = 2, 64, 16, torch.float16, 2
    live_max, pages = 6, 40
    cache = BlockTableKVCache(L, H, D, page_size=ps, num_pages=pages, max_seqs=live_max, max_blocks_per_seq=8,
                              dtype=dtype, device=DEV, seed=3)
    truth = {}          # seq_id -> per-layer (k [len, H, D], v)
    next_id = 0

    def admit(n_tokens):
        nonlocal next_id
        sid = next_id
        next_id += 1
        slot = cache.open(sid)
        batch = cache.begin_append([slot], [n_tokens])
        per_layer = []
        for l in range(L):
            k, v = S.randn(g, (n_tokens, H, D), dtype), S.randn(g, (n_tokens, H, D), dtype)
            cache.append(l, batch, k.to(DEV), v.to(DEV))
            per_layer.append((k, v))
        cache.end_append(batch)
        truth[sid] = per_layer

    for n in (30, 17, 64, 5):
        admit(n)
    for step in range(40):
        ids = sorted(truth)
        slots = [cache.slot(i) for i in ids]
        batch = cache.begin_append(slots, [1] * len(ids))
        for l in range(L):
            k, v = S.randn(g, (len(ids), H, D), dtype), S.randn(g, (len(ids), H, D), dtype)
            cache.append(l, batch, k.to(DEV), v.to(DEV))
            for row, i in enumerate(ids):
                tk, tv = truth[i][l]
                truth[i][l] = (torch.cat([tk, k[row:row + 1]]), torch.cat([tv, v[row:row + 1]]))
        cache.end_append(batch)
        if step % 5 == 4:                       # one sequence finishes, a new one is admitted
            victim = ids[(step // 5) % len(ids)]
            cache.release(victim)
            del truth[victim]
            admit(20 + step)
        ids = sorted(truth)
        gb = cache.begin_gather([cache.slot(i) for i in ids])
        for l in range(L):
            kn, vn = cache.gather(l, gb, "NHD")
            for row, i in enumerate(ids):
                a, b = gb.cu[row], gb.cu[row + 1]
                assert torch.equal(S.bits(kn[a:b]), S.bits(truth[i][l][0])), (step, l, i)
                assert torch.equal(S.bits(vn[a:b]), S.bits(truth[i][l][1])), (step, l, i)
    st = cache.stats()
    assert st.pages_resident == sum(len(cache.pages_of[cache.slot(i)]) for i in truth)
    assert st.pages_peak >= st.pages_resident and st.sequences_live == len(truth)
    assert cache.allocator.release_calls == 8
    cache.check_device_status()


def test_fork_crop_and_beam_reorder_against_copied_reference_layers(backend):
    """The reference copies whole cache rows for beam search (``batch_repeat_interleave``,
    ``batch_select_indices``, kv_cache.py:166-186); here forks share full pages and copy one.  Contents
    must equal deep copies of the reference layers after every operation and every later append."""
    import copy

    from barqtrain_b200 import BlockTableKVCache
    from oracle.paged_kv_oracle import OracleLayer

    L, H, D, ps, dtype = 2, 2, 64, 16, torch.float16
    g = torch.Generator().manual_seed(88)
    cache = BlockTableKVCache(L, H, D, page_size=ps, num_pages=40, max_seqs=8, max_blocks_per_seq=8, dtype=dtype,
                              device=DEV, seed=4)
    truth = {}                                   # seq id -> [OracleLayer per layer], reference contents

    def append(ids, counts):
        slots = [cache.slot(i) for i in ids]
        batch = cache.begin_append(slots, counts)
        for l in range(L):
            k, v = S.randn(g, (sum(counts), H, D), dtype), S.randn(g, (sum(counts), H, D), dtype)
            cache.append(l, batch, k.to(DEV), v.to(DEV))
            at = 0
            for i, c in zip(ids, counts):
                if c:
                    truth[i][l].append(k[at:at + c].transpose(0, 1).unsqueeze(0), v[at:at + c].transpose(0, 1).unsqueeze(0))
                at += c
        cache.end_append(batch)

    def check(ids):
        gb = cache.begin_gather([cache.slot(i) for i in ids])
        for l in range(L):
            kh, vh = cache.gather(l, gb, "HND")
            for row, i in enumerate(ids):
                wk, wv = truth[i][l].current_tensors()
                a, b = gb.cu[row], gb.cu[row + 1]
                assert b - a == truth[i][l].get_seq_length()
                assert torch.equal(S.bits(kh[:, a:b]), S.bits(wk[0])), (l, i)
                assert torch.equal(S.bits(vh[:, a:b]), S.bits(wv[0])), (l, i)
        owned = {}
        for i in ids:
            for p in cache.pages_of[cache.slot(i)]:
                owned[p] = owned.get(p, 0) + 1
        assert all(cache.allocator.holders(p) == c for p, c in owned.items())
        assert cache.stats().pages_resident == len(owned)

    for i in "abc":
        cache.open(i)
        truth[i] = [OracleLayer(1, 128, ps) for _ in range(L)]
    append(list("abc"), [21, 16, 40])
    append(list("abc"), [1, 1, 1])
    check(list("abc"))

    def fork(src, dst):
        cache.fork(src, dst)
        truth[dst] = copy.deepcopy(truth[src])

    fork("a", "a2")                              # 22 tokens: one full page shared, 6 rows copied
    fork("b", "b2")                              # 17 tokens
    cache.crop("c", 32)                          # exactly two pages: the fork copies nothing
    for lay in truth["c"]:
        lay.crop(32)
    fork("c", "c2")
    assert cache.pages_of[cache.slot("c")] == cache.pages_of[cache.slot("c2")]
    ids = ["a", "a2", "b", "b2", "c", "c2"]
    check(ids)
    for _ in range(18):                          # diverge, crossing page boundaries
        append(ids, [1] * len(ids))
    check(ids)
    cache.crop("a2", 10)                         # back into the page shared with "a": copy before writing
    for lay in truth["a2"]:
        lay.crop(10)
    cache.crop("b2", -3)
    for lay in truth["b2"]:
        lay.crop(-3)
    append(ids, [3, 9, 0, 2, 1, 1])
    check(ids)
    new_ids = cache.reorder(ids, [1, 1, 4, 1, 2, 2])     # beams continue a2 (three times), c, b (twice)
    src = ["a2", "a2", "c", "a2", "b", "b"]
    fresh = {}
    for nid, sid in zip(new_ids, src):
        fresh[nid] = truth[sid] if nid == sid else copy.deepcopy(truth[sid])
    truth.clear()
    truth.update(fresh)
    assert sorted(map(str, new_ids)) == sorted(map(str, truth)) and cache.stats().sequences_live == 6
    check(new_ids)
    append(new_ids, [2] * 6)
    check(new_ids)
    for sid in new_ids:
        cache.release(sid)
    assert cache.stats().pages_resident == 0 and cache.allocator.pages_free == 40
    cache.check_device_status()


def test_corrupt_table_entry_is_skipped_and_flagged(backend):
    """A page id outside the pool never reaches memory: the rows are skipped, a status bit is set,
    the other sequences are unaffected and the context stays usable."""
    from barqtrain_b200 import BlockTableKVCache

    H, D, ps = 2, 64, 16
    cache = BlockTableKVCache(1, H, D, page_size=ps, num_pages=8, max_seqs=2, max_blocks_per_seq=2,
                              dtype=torch.float16, device=DEV)
    s0, s1 = cache.open("a"), cache.open("b")
    batch = cache.begin_append([s0, s1], [20, 20])
    cache.table_dev[s1, 1] = 1000                       # corrupt the device copy only
    k = torch.ones(40, H, D, dtype=torch.float16, device=DEV)
    cache.append(0, batch, k, k * 2)
    cache.end_append(batch)
    assert backend.read_status(DEV) == 1
    for mode in ("vector", "bulk"):
        gb = cache.begin_gather([s0, s1])
        kn, vn = cache.gather(0, gb, "NHD", out=(torch.zeros(40, H, D, dtype=torch.float16, device=DEV),
                                                  torch.zeros(40, H, D, dtype=torch.float16, device=DEV)), mode=mode)
        assert backend.read_status(DEV) == 1
        assert bool((kn[:36] == 1).all()) and bool((vn[:36] == 2).all())
        assert not kn[36:].any()                         # the skipped page's rows were left alone
    torch.cuda.synchronize()


def test_empty_and_degenerate_batches(backend):
    from barqtrain_b200 import BlockTableKVCache

    H, D = 2, 32
    cache = BlockTableKVCache(1, H, D, page_size=4, num_pages=8, max_seqs=3, max_blocks_per_seq=4,
                              dtype=torch.float32, device=DEV)
    slots = [cache.open(i) for i in range(3)]
    launches = backend.launches
    cache.append_step([], [], [torch.zeros(0, H, D, device=DEV)], [torch.zeros(0, H, D, device=DEV)])
    cache.append_step(slots, [0, 0, 0], [torch.zeros(0, H, D, device=DEV)], [torch.zeros(0, H, D, device=DEV)])
    assert backend.launches == launches
    k = torch.arange(5 * H * D, dtype=torch.float32, device=DEV).view(5, H, D)
    cache.append_step(slots, [0, 5, 0], [k], [k + 0.5])            # empty neighbours on both sides
    gb = cache.begin_gather(slots)
    assert gb.cu == [0, 0, 5, 5]
    kn, vn = cache.gather(0, gb, "NHD")
    assert torch.equal(kn, k) and torch.equal(vn, k + 0.5)
    gb = cache.begin_gather([slots[0], slots[2]])
    kn, vn = cache.gather(0, gb, "HND")
    assert kn.shape == (H, 0, D)
    with pytest.raises(ValueError, match="capacity exceeded"):
        cache.begin_append([slots[1]], [12])
    cache.check_device_status()


# ---------------------------------------------------------------------------
# full-size shapes: size-independent properties
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("ps,dtype", [(16, torch.float16), (32, torch.float16), (16, torch.bfloat16)])
def test_full_size_chunk_round_trip(backend, ps, dtype):
    """One layer of the chunked-prefill configuration at full width (16 sequences x 2048-token
    chunks, 8 heads, head_dim 128): append -> gather returns the appended rows, pages outside the
    table stay zero, and the vector and bulk gathers agree bit for bit."""
    from barqtrain_b200 import BlockTableKVCache

    nseq, chunk, chunks, H, D = 16, 2048, 2, 8, 128
    g = torch.Generator(device=DEV).manual_seed(9)
    pages = nseq * chunk * chunks // ps + 64
    cache = BlockTableKVCache(1, H, D, page_size=ps, num_pages=pages, max_seqs=nseq,
                              max_blocks_per_seq=chunk * chunks // ps, dtype=dtype, device=DEV, seed=12)
    slots = [cache.open(i) for i in range(nseq)]
    sent_k, sent_v = [], []
    for _ in range(chunks):
        k = torch.randn(nseq * chunk, H, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
        v = torch.randn(nseq * chunk, H, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
        cache.append_step(slots, [chunk] * nseq, [k], [v])
        sent_k.append(k.view(nseq, chunk, H, D))
        sent_v.append(v.view(nseq, chunk, H, D))
    want_k = torch.cat(sent_k, 1).reshape(nseq * chunk * chunks, H, D)
    want_v = torch.cat(sent_v, 1).reshape(nseq * chunk * chunks, H, D)
    gb = cache.begin_gather(slots)
    kv, vv = cache.gather(0, gb, "NHD", mode="vector")
    kb, vb = cache.gather(0, gb, "NHD", mode="bulk")
    assert torch.equal(S.bits_dev(kv), S.bits_dev(want_k)) and torch.equal(S.bits_dev(vv), S.bits_dev(want_v))
    assert torch.equal(S.bits_dev(kb), S.bits_dev(want_k)) and torch.equal(S.bits_dev(vb), S.bits_dev(want_v))
    kh, vh = cache.gather(0, gb, "HND", mode="bulk")
    assert torch.equal(S.bits_dev(kh.transpose(0, 1)), S.bits_dev(want_k))
    assert torch.equal(S.bits_dev(vh.transpose(0, 1)), S.bits_dev(want_v))
    owned = torch.zeros(pages, dtype=torch.bool, device=DEV)
    owned[torch.tensor([p for s in slots for p in cache.pages_of[s]], device=DEV)] = True
    assert not cache.pools[0][:, :, ~owned].any()
    cache.check_device_status()


@pytest.mark.parametrize("shape", ["decode-8b", "gather-70b"])
def test_full_size_layer_against_c_oracle(backend, shape):
    """One layer at the full width of the decode and the 70B-gather configurations (64 sequences
    uniform [512, 4096] / 32 sequences log-uniform [1k, 32k]; 8 heads, head_dim 128, bf16, page 16,
    shuffled pool): prefill, three fused decode updates, then every gathered byte and the whole pool
    compared with the C oracle."""
    from barqtrain_b200 import BlockTableKVCache
    from oracle import c_oracle

    H, D, ps, dtype = 8, 128, 16, torch.bfloat16
    g = torch.Generator().manual_seed(1236 if shape == "decode-8b" else 1238)
    lens = (S.ragged_lengths(g, 64, 512, 4096) if shape == "decode-8b"
            else S.ragged_lengths(g, 32, 1024, 32768, log_uniform=True))
    n, steps = len(lens), 3
    pages = sum(-(-(x + steps) // ps) for x in lens)
    order = torch.randperm(pages, generator=g).tolist()
    cache = BlockTableKVCache(1, H, D, page_size=ps, num_pages=pages, max_seqs=n,
                              max_blocks_per_seq=-(-(max(lens) + steps) // ps), dtype=dtype, device=DEV,
                              free_order=order)
    slots = [cache.open(i) for i in range(n)]
    ref_k = torch.zeros(H, pages, ps, D, dtype=dtype)
    ref_v = torch.zeros_like(ref_k)
    gen = torch.Generator(device=DEV).manual_seed(5)
    have = [0] * n

    def rows(count):
        k = torch.randn(count, H, D, generator=gen, device=DEV, dtype=torch.float32).to(dtype)
        v = torch.randn(count, H, D, generator=gen, device=DEV, dtype=torch.float32).to(dtype)
        return k, v

    def mirror(batch, k, v):
        start = torch.tensor(have, dtype=torch.int32)
        cu = torch.tensor(batch.cu, dtype=torch.int32)
        assert c_oracle.append_paged(ref_k, ref_v, cache.table_host.clone(), None, start, cu, k.cpu(), v.cpu()) == 0
        for i in range(n):
            have[i] += batch.cu[i + 1] - batch.cu[i]

    k, v = rows(sum(lens))
    batch = cache.begin_append(slots, lens)
    cache.append(0, batch, k, v)
    cache.end_append(batch)
    mirror(batch, k, v)
    for _ in range(steps):
        k, v = rows(n)
        new = cache.begin_append(slots, [1] * n)
        cache.end_append(new)
        full = cache.begin_gather(slots)
        got_k, got_v = cache.update(0, new, full, k, v, "NHD")
        mirror(new, k, v)
    total = sum(have)
    want_k = torch.zeros(total, H, D, dtype=dtype)
    want_v = torch.zeros_like(want_k)
    cu_out = torch.tensor(full.cu[:-1], dtype=torch.int32)
    assert c_oracle.gather_paged(ref_k, ref_v, cache.table_host.clone(), None, torch.tensor(have, dtype=torch.int32),
                                 cu_out, want_k, want_v) == 0
    assert torch.equal(S.bits(got_k), S.bits(want_k)) and torch.equal(S.bits(got_v), S.bits(want_v))
    kh, vh = cache.gather(0, full, "HND")
    assert torch.equal(S.bits(kh.transpose(0, 1)), S.bits(want_k))
    assert torch.equal(S.bits(vh.transpose(0, 1)), S.bits(want_v))
    assert torch.equal(S.bits(cache.pools[0, 0]), S.bits(ref_k)) and torch.equal(S.bits(cache.pools[0, 1]), S.bits(ref_v))
    cache.check_device_status()


@pytest.mark.parametrize("ps", [16, 32])
def test_full_size_chunked_prefill_against_c_oracle(backend, ps):
    """One layer of the chunked-prefill configuration at full size (16 sequences of 8192 tokens in four
    2048-token chunks, 8 heads, head_dim 128, fp16, pool shuffled by a seeded permutation; page 16 and
    32): every chunk goes through ``append`` - token-major rows for three chunks, a head-major source for
    the last, so both page-sized copy paths run - and the whole pool and every gathered row equal the C
    oracle's."""
    from barqtrain_b200 import BlockTableKVCache
    from oracle import c_oracle

    B, chunk, chunks, H, D, dtype = 16, 2048, 4, 8, 128, torch.float16
    pages = B * chunk * chunks // ps
    cache = BlockTableKVCache(1, H, D, page_size=ps, num_pages=pages, max_seqs=B, max_blocks_per_seq=chunk * chunks // ps,
                              dtype=dtype, device=DEV, seed=1237)
    slots = [cache.open(i) for i in range(B)]
    ref_k = torch.zeros(H, pages, ps, D, dtype=dtype)
    ref_v = torch.zeros_like(ref_k)
    gen = torch.Generator(device=DEV).manual_seed(9)
    launches = backend.launches
    for c in range(chunks):
        total = B * chunk
        if c < chunks - 1:
            k = torch.randn(total, H, D, generator=gen, device=DEV, dtype=torch.float32).to(dtype)
            v = torch.randn(total, H, D, generator=gen, device=DEV, dtype=torch.float32).to(dtype)
        else:                                    # [H, total, D] in memory, handed over as [total, H, D]
            k = torch.randn(H, total, D, generator=gen, device=DEV, dtype=torch.float32).to(dtype).transpose(0, 1)
            v = torch.randn(H, total, D, generator=gen, device=DEV, dtype=torch.float32).to(dtype).transpose(0, 1)
        batch = cache.begin_append(slots, [chunk] * B)
        cache.append(0, batch, k, v)
        start = torch.full((B,), c * chunk, dtype=torch.int32)
        cu = torch.tensor(batch.cu, dtype=torch.int32)
        assert c_oracle.append_paged(ref_k, ref_v, cache.table_host.clone(), None, start, cu, k.cpu().contiguous(),
                                     v.cpu().contiguous()) == 0
        cache.end_append(batch)
    assert backend.launches <= launches + 2 * chunks        # per chunk: one append kernel (+ one table scatter)
    cache.check_device_status()
    assert torch.equal(S.bits(cache.pools[0, 0]), S.bits(ref_k)), "K pool differs"
    assert torch.equal(S.bits(cache.pools[0, 1]), S.bits(ref_v)), "V pool differs"
    gb = cache.begin_gather(slots)
    want_k = torch.zeros(gb.total, H, D, dtype=dtype)
    want_v = torch.zeros_like(want_k)
    assert c_oracle.gather_paged(ref_k, ref_v, cache.table_host.clone(), None,
                                 torch.full((B,), chunk * chunks, dtype=torch.int32),
                                 torch.tensor(gb.cu[:-1], dtype=torch.int32), want_k, want_v) == 0
    kn, vn = cache.gather(0, gb, "NHD")
    assert torch.equal(S.bits(kn), S.bits(want_k)) and torch.equal(S.bits(vn), S.bits(want_v))
    cache.check_device_status()


def test_bounded_wait_gives_up_flags_and_leaves_the_context_usable(backend):
    """``barqkv_gather_wait_selftest``: one CTA of the bulk gather whose ring stages expect bytes that never
    arrive, every wait bounded by about a millisecond.  The kernel must return on its own, report
    ``BARQKV_S_TIMEOUT`` through the status word, take no longer than a few bounds, and leave the device in
    working order: the same gather run normally afterwards is bit-exact."""
    import ctypes
    import time

    from barqtrain_b200 import BlockTableKVCache, _ffi

    H, D, ps, dtype = 2, 128, 16, torch.bfloat16
    lens = [100, 37, 260]
    g = torch.Generator().manual_seed(77)
    cache = BlockTableKVCache(1, H, D, page_size=ps, num_pages=40, max_seqs=3, max_blocks_per_seq=20, dtype=dtype,
                              device=DEV, seed=2)
    slots = [cache.open(i) for i in range(3)]
    k = S.randn(g, (sum(lens), H, D), dtype).to(DEV)
    v = S.randn(g, (sum(lens), H, D), dtype).to(DEV)
    cache.append_step(slots, lens, [k], [v])
    gb = cache.begin_gather(slots)
    want_k, want_v = cache.gather(0, gb, "HND", mode="bulk")
    torch.cuda.synchronize()
    assert backend.read_status(DEV) == 0

    out_k, out_v = torch.zeros_like(want_k), torch.zeros_like(want_v)
    rows = _ffi.RowsLayout(0, D, gb.total * D, 1, 0)
    status = backend.status_word(DEV)
    cycles = 2_000_000                                       # about 1 ms at the SM clock
    t0 = time.perf_counter()
    rc = backend.lib.barqkv_gather_wait_selftest(ctypes.byref(cache._pool_layout), cache._k_ptr[0], cache._v_ptr[0],
                                                 gb.table_ref, gb.p_first, gb.p_cu, gb.n, out_k.data_ptr(),
                                                 out_v.data_ptr(), ctypes.byref(rows), cycles, status.data_ptr(), gb.stream)
    assert rc == 0, backend.lib.barqkv_last_error()
    torch.cuda.synchronize()                                 # returns: the kernel did not spin past its bound
    elapsed = time.perf_counter() - t0
    assert elapsed < 1.0, f"the give-up took {elapsed:.3f} s for a 1 ms bound"
    assert backend.read_status(DEV) == _ffi.S_TIMEOUT        # reported, and cleared by the read
    # the context still works and the data are untouched
    got_k, got_v = cache.gather(0, gb, "HND", mode="bulk")
    torch.cuda.synchronize()
    assert torch.equal(S.bits(got_k), S.bits(want_k)) and torch.equal(S.bits(got_v), S.bits(want_v))
    assert backend.read_status(DEV) == 0


def test_continuous_batching_churn_at_full_width_reads_back_exactly(backend):
    """The churn configuration at full width (256 live sequences, 8 heads, head_dim 128, fp16, page 16;
    two layers, 150 steps, about 380 sequences finished, released and replaced): after all the page
    recycling every live sequence must gather to exactly the rows that were appended to it."""
    from barqtrain_b200.benchmarks.workloads import churn

    res = churn(1, 0, torch.device("cuda", 0), steps=150, warmup=2, layers=2, verify=True,
                sync=lambda: torch.cuda.synchronize())
    assert res["verified"] is True
    assert res["extra"]["sequences_released"] > 200
    assert res["extra"]["pages_peak"] >= res["extra"]["pages_resident"] > 0


def test_continuous_batching_with_attention_from_a_graph_reads_back_exactly(backend):
    """The churn configuration with every decode step run as recorded launches that store the token and attend
    over the pages, the batch's rows re-pointed at the replacement sequences between replays
    (``DecodeGraphs``): after 80 steps of releases and replacements every live sequence still gathers to
    exactly the rows that were appended to it."""
    from barqtrain_b200.benchmarks.workloads import churn

    res = churn(1, 0, torch.device("cuda", 0), steps=80, warmup=2, layers=2, verify=True, attend=True,
                sync=lambda: torch.cuda.synchronize())
    assert res["verified"] is True
    assert res["extra"]["sequences_released"] > 100
    assert res["launches"] >= 80 * 2


@pytest.mark.parametrize("dtype_name", ["fp32", "fp16", "bf16"])
def test_rope_fused_into_append_against_the_reference_helper(backend, golden_dir, dtype_name):
    """A prefill appended with ``rope=(cos, sin)`` leaves in the pages exactly the K rows the reference's
    ``apply_rope_to_qk`` (ops.py:376-428) returns for it - compared with the helper's stored output bit for
    bit, using the helper's own cos / sin tables - and the V rows unchanged."""
    from barqtrain_b200 import BlockTableKVCache

    gold = np.load(golden_dir / "rope_prefill.npz")
    k, v = S.rope_prefill(dtype_name)                          # [B, H, T, D]
    B, H, T, D = k.shape
    cos = torch.from_numpy(gold[f"cos_{dtype_name}"]).view(k.dtype)       # [T, D/2]
    sin = torch.from_numpy(gold[f"sin_{dtype_name}"]).view(k.dtype)
    want_k = torch.from_numpy(gold[f"k_rope_{dtype_name}"]).view(k.dtype)  # [B, H, T, D]
    ps = 16
    cache = BlockTableKVCache(1, H, D, page_size=ps, num_pages=2 * B * (-(-T // ps)), max_seqs=B,
                              max_blocks_per_seq=-(-T // ps), dtype=k.dtype, device=DEV, seed=3)
    slots = [cache.open(i) for i in range(B)]
    rows = lambda t: t.permute(0, 2, 1, 3).reshape(B * T, H, D).to(DEV)   # packed [B*T, H, D]
    full = lambda t: torch.cat([t, t], dim=-1).repeat(B, 1).to(DEV)       # per packed token, halves duplicated
    batch = cache.begin_append(slots, [T] * B)
    cache.append(0, batch, rows(k), rows(v), rope=(full(cos), full(sin)))
    cache.end_append(batch)
    gk, gv = cache.gather(0, cache.begin_gather(slots), "HND")            # [H, B*T, D]
    cache.check_device_status()
    got_k = gk.view(H, B, T, D).permute(1, 0, 2, 3)
    got_v = gv.view(H, B, T, D).permute(1, 0, 2, 3)
    assert torch.equal(S.bits(got_k), S.bits(want_k))
    assert torch.equal(S.bits(got_v), S.bits(v))


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float16, 64), (torch.float32, 32)])
def test_rope_fused_into_append_equals_rotate_then_append(backend, dtype, D):
    """``append(..., rope=(cos, sin))`` stores ``k*cos + rotate_half(k)*sin`` - the reference helper's
    formula (ops.py:376-428) with per-token tables - bit for bit what rotating with tensor expressions
    in the same dtype and appending afterwards stores; V is untouched."""
    from barqtrain_b200 import BlockTableKVCache

    H, ps = 3, 16
    g = torch.Generator().manual_seed(41)
    order = torch.randperm(40, generator=g).tolist()

    def make():
        c = BlockTableKVCache(1, H, D, page_size=ps, num_pages=40, max_seqs=3, max_blocks_per_seq=12, dtype=dtype,
                              device=DEV, free_order=order)
        return c, [c.open(i) for i in range(3)]

    fused, fs = make()
    plain, pl = make()
    lens = [0, 0, 0]
    for counts in ((37, 5, 100), (1, 1, 1), (0, 20, 3)):
        total = sum(counts)
        k = S.randn(g, (total, H, D), dtype).to(DEV)
        v = S.randn(g, (total, H, D), dtype).to(DEV)
        pos = torch.cat([torch.arange(lens[i], lens[i] + c) for i, c in enumerate(counts)]).float()
        freqs = 1.0 / torch.pow(10000.0, torch.arange(D // 2).float() / (D // 2))
        ang = pos[:, None] * freqs[None, :]
        cos = torch.cat([ang.cos(), ang.cos()], dim=-1).to(dtype).to(DEV)         # [total, D], halves duplicated
        sin = torch.cat([ang.sin(), ang.sin()], dim=-1).to(dtype).to(DEV)
        rotated = k * cos[:, None, :] + torch.cat([-k[..., D // 2:], k[..., :D // 2]], dim=-1) * sin[:, None, :]
        b1 = fused.begin_append(fs, counts)
        fused.append(0, b1, k, v, rope=(cos, sin))
        fused.end_append(b1)
        b2 = plain.begin_append(pl, counts)
        plain.append(0, b2, rotated, v)
        plain.end_append(b2)
        lens = [n + c for n, c in zip(lens, counts)]
        assert torch.equal(S.bits_dev(fused.pools), S.bits_dev(plain.pools))
    fused.check_device_status()


def test_more_sequences_than_one_launch_scans(backend):
    from barqtrain_b200 import BlockTableKVCache

    """9000 short sequences in one batch: a gather launch scans at most 8192, so the cache slices the
    batch; the result must still be every sequence's rows back to back, in both layouts and through
    update()."""
    H, D, ps, n = 1, 16, 4, 9000
    g = torch.Generator().manual_seed(77)
    lens = torch.randint(1, 10, (n,), generator=g).tolist()
    pages = sum(-(-(x + 1) // ps) for x in lens)
    cache = BlockTableKVCache(1, H, D, page_size=ps, num_pages=pages, max_seqs=n, max_blocks_per_seq=3,
                              dtype=torch.float16, device=DEV, seed=77)
    slots = [cache.open(i) for i in range(n)]
    total = sum(lens)
    k = torch.randn(total, H, D, generator=g, dtype=torch.float32).to(torch.float16).to(DEV)
    v = torch.randn(total, H, D, generator=g, dtype=torch.float32).to(torch.float16).to(DEV)
    batch = cache.begin_append(slots, lens)
    cache.append(0, batch, k, v)
    cache.end_append(batch)
    gb = cache.begin_gather(slots)
    kn, vn = cache.gather(0, gb, "NHD")
    assert torch.equal(kn, k) and torch.equal(vn, v)
    kh, vh = cache.gather(0, gb, "HND")
    assert torch.equal(kh, k.transpose(0, 1)) and torch.equal(vh, v.transpose(0, 1))
    # one more token each through update(): old rows then the new row, per sequence
    k1 = torch.randn(n, H, D, generator=g, dtype=torch.float32).to(torch.float16).to(DEV)
    new = cache.begin_append(slots, [1] * n)
    cache.end_append(new)
    full = cache.begin_gather(slots)
    ku, vu = cache.update(0, new, full, k1, k1, "NHD")
    cu_old = torch.tensor(gb.cu[:-1])
    at_new = torch.tensor(full.cu[1:]) - 1
    assert torch.equal(ku[at_new.to(DEV)], k1)
    keep = torch.ones(full.total, dtype=torch.bool)
    keep[at_new] = False
    assert torch.equal(ku[keep.to(DEV)], k) and torch.equal(vu[keep.to(DEV)], v)
    assert cu_old.numel() == n and backend.read_status(DEV) == 0


@pytest.mark.parametrize("layout", ["HND", "NHD"])
def test_all_layers_in_one_gather_launch(backend, layout):
    """gather_layers() against gather() per layer: ragged lengths, shuffled pool, partial last pages."""
    from barqtrain_b200 import BlockTableKVCache

    L, H, D, ps = 5, 2, 64, 16
    lens = [37, 1, 16, 250, 33, 64, 129]
    g = torch.Generator().manual_seed(91)
    pages = sum(-(-x // ps) for x in lens) + 2
    cache = BlockTableKVCache(L, H, D, page_size=ps, num_pages=pages, max_seqs=len(lens), max_blocks_per_seq=16,
                              dtype=torch.bfloat16, device=DEV, seed=91)
    slots = [cache.open(i) for i in range(len(lens))]
    total = sum(lens)
    batch = cache.begin_append(slots, lens)
    for layer in range(L):
        k = torch.randn(total, H, D, generator=g, dtype=torch.float32).to(torch.bfloat16).to(DEV)
        v = torch.randn(total, H, D, generator=g, dtype=torch.float32).to(torch.bfloat16).to(DEV)
        cache.append(layer, batch, k, v)
    cache.end_append(batch)
    order = [3, 0, 6, 2, 5]                                     # a subset, in another order
    gb = cache.begin_gather([slots[i] for i in order])
    before = backend.launches
    k_all, v_all = cache.gather_layers(gb, layout)
    assert backend.launches - before == 1
    assert k_all.shape[0] == L
    for layer in range(L):
        k1, v1 = cache.gather(layer, gb, layout)
        assert torch.equal(S.bits(k_all[layer]), S.bits(k1)) and torch.equal(S.bits(v_all[layer]), S.bits(v1))
    assert backend.read_status(DEV) == 0


def test_crop_on_an_exhausted_pool_raises_and_changes_nothing(backend):
    """``crop`` of a sequence that shares its last kept page needs one fresh page for its private copy; when the
    pool has none the call must fail before anything was given back or edited."""
    from barqtrain_b200 import BlockTableKVCache
    from barqtrain_b200.block_table import PagePoolExhausted

    H, D, ps, dtype = 2, 64, 16, torch.float16
    g = torch.Generator().manual_seed(5)
    cache = BlockTableKVCache(1, H, D, page_size=ps, num_pages=8, max_seqs=3, max_blocks_per_seq=6, dtype=dtype,
                              device=DEV, seed=1)
    a = cache.open("a")
    k = S.randn(g, (64, H, D), dtype).to(DEV)
    cache.append_step([a], [64], [k], [k])                      # 4 full pages
    cache.fork("a", "b")                                        # shares all four
    filler = cache.open("c")
    cache.append_step([filler], [64], [k], [k])                 # the other 4 pages: the pool is empty
    assert cache.allocator.pages_free == 0
    before = (cache.pages_of[cache.slot("b")], int(cache.lengths[cache.slot("b")]),
              [cache.allocator.holders(p) for p in range(8)])
    with pytest.raises(PagePoolExhausted):
        cache.crop("b", 40)                                     # keeps 3 pages, the third partly: needs a copy
    after = (cache.pages_of[cache.slot("b")], int(cache.lengths[cache.slot("b")]),
             [cache.allocator.holders(p) for p in range(8)])
    assert after == before
    cache.release("c")
    cache.crop("b", 40)                                         # with room it goes through
    assert int(cache.lengths[cache.slot("b")]) == 40 and len(cache.pages_of[cache.slot("b")]) == 3
    gk, _ = cache.gather_sequence(0, "b", "NHD")
    assert torch.equal(S.bits(gk), S.bits(k[:40]))
    cache.check_device_status()


def test_padded_output_of_a_batch_gathered_in_slices(backend, monkeypatch):
    """Batches beyond one launch's scan limit are gathered in slices; with the padded ``[n, H, S, D]`` layout
    every slice must land on its own batch rows (the limit is lowered here so that a small batch needs three)."""
    from barqtrain_b200 import BlockTableKVCache, block_table

    monkeypatch.setattr(block_table, "_GATHER_MAX_ENTRIES", 4)
    H, D, ps, dtype = 2, 128, 16, torch.bfloat16
    lens = [5, 33, 16, 1, 40, 17, 2, 31, 9, 20]
    g = torch.Generator().manual_seed(6)
    cache = BlockTableKVCache(1, H, D, page_size=ps, num_pages=40, max_seqs=len(lens), max_blocks_per_seq=4, dtype=dtype,
                              device=DEV, seed=4)
    slots = [cache.open(i) for i in range(len(lens))]
    k = S.randn(g, (sum(lens), H, D), dtype).to(DEV)
    v = S.randn(g, (sum(lens), H, D), dtype).to(DEV)
    cache.append_step(slots, lens, [k], [v])
    gb = cache.begin_gather(slots)
    out = (torch.zeros(len(lens), H, max(lens), D, dtype=dtype, device=DEV),
           torch.zeros(len(lens), H, max(lens), D, dtype=dtype, device=DEV))
    cache.gather(0, gb, "BHSD", out=out)
    at = 0
    for i, n in enumerate(lens):
        assert torch.equal(S.bits(out[0][i, :, :n]), S.bits(k[at:at + n].transpose(0, 1))), i
        assert torch.equal(S.bits(out[1][i, :, :n]), S.bits(v[at:at + n].transpose(0, 1))), i
        assert not out[0][i, :, n:].any()
        at += n
    kn, _ = cache.gather(0, gb, "NHD")                           # packed outputs go in slices too
    assert torch.equal(S.bits(kn), S.bits(k))
    cache.check_device_status()


def test_a_description_overwritten_by_a_later_one_is_refused(backend):
    from barqtrain_b200 import BlockTableKVCache

    H, D, dtype = 1, 128, torch.bfloat16
    cache = BlockTableKVCache(1, H, D, num_pages=8, max_seqs=2, max_blocks_per_seq=4, dtype=dtype, device=DEV)
    a, b = cache.open(0), cache.open(1)
    k = torch.zeros(3, H, D, dtype=dtype, device=DEV)
    first = cache.begin_append([a], [3])
    second = cache.begin_append([b], [3])                       # rewrites the device words `first` points to
    with pytest.raises(RuntimeError, match="stale"):
        cache.append(0, first, k, k)
    cache.append(0, second, k, k)
    cache.end_append(second)
    cache.check_device_status()


def test_table_changes_beyond_one_staging_slot_go_in_several_uploads(backend):
    """``barqkv_host_begin`` sends the description and the changed block-table entries in one upload; when more
    entries changed than the attached buffers hold beside the description, the rest travel in further uploads
    ahead of it.  Re-attached here with room for four entries per upload."""
    import ctypes

    from barqtrain_b200 import BlockTableKVCache

    H, D, ps, dtype = 1, 128, 16, torch.bfloat16
    lens = [200, 150, 90]
    g = torch.Generator().manual_seed(8)
    cache = BlockTableKVCache(1, H, D, page_size=ps, num_pages=40, max_seqs=3, max_blocks_per_seq=16, dtype=dtype,
                              device=DEV, seed=9)
    slots = [cache.open(i) for i in range(3)]
    n = len(slots)
    small = 3 * n + 1 + 8                                        # the description and four (index, page) pairs
    dev = [torch.zeros(small, dtype=torch.int32, device=DEV) for _ in range(2)]
    staging = torch.zeros(8 * small, dtype=torch.int32).pin_memory()
    assert backend.lib.barqkv_host_attach(cache._host, cache.table_dev.data_ptr(), dev[0].data_ptr(), dev[1].data_ptr(),
                                          small, staging.data_ptr(), staging.numel()) == 0
    cache._step_dev, cache._staging = dev, staging
    cache._staging_np, cache._staging_ptr = staging.numpy(), staging.data_ptr()
    cache._tables.clear()
    k = S.randn(g, (sum(lens), H, D), dtype).to(DEV)
    batch = cache.begin_append(slots, lens)                      # 13 + 10 + 6 = 29 new table entries: 8 uploads
    assert int(cache._info[3]) == 29 and int(cache._info[6]) == 8 + 8
    cache.append(0, batch, k, k)
    cache.end_append(batch)
    torch.cuda.synchronize()
    assert torch.equal(cache.table_dev.cpu(), cache.table_host)
    gk, _ = cache.gather(0, cache.begin_gather(slots), "NHD")
    assert torch.equal(S.bits(gk), S.bits(k))
    cache.check_device_status()
