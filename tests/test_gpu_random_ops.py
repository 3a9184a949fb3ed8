"""Model-based test: a seeded random program of cache operations against reference layers.

Every live sequence is mirrored by one oracle layer per cache layer (the reference's CPU semantics,
deep-copied on fork).  After every operation all live sequences are gathered - random layout, random
gather kernel - and must equal the oracle bit for bit; the allocator's holder counts must match the
tables.  Small pages (4 or 8 rows) make page boundaries, partial pages and recycling frequent."""

import copy
import random

import pytest
import torch

from tests import scenarios as S

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.mark.parametrize("seed,ps,dtype,H,D", [(0, 4, torch.float16, 2, 64), (1, 8, torch.bfloat16, 3, 32),
                                               (2, 16, torch.float32, 1, 16)])
def test_random_programs_match_reference_layers(seed, ps, dtype, H, D):
    from barqtrain_b200 import BlockTableKVCache, _ffi
    from oracle.paged_kv_oracle import OracleLayer

    backend = _ffi.require_cuda_backend()
    rnd = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    L, max_seqs, max_blocks, pages = 2, 6, 12, 48
    cap = max_blocks * ps
    cache = BlockTableKVCache(L, H, D, page_size=ps, num_pages=pages, max_seqs=max_seqs, max_blocks_per_seq=max_blocks,
                              dtype=dtype, device=DEV, seed=seed)
    truth = {}
    next_id = 0

    def length(sid):
        return truth[sid][0].get_seq_length()

    def room(extra_pages):
        return cache.allocator.pages_free >= extra_pages

    def append(ids, counts, fused):
        slots = [cache.slot(i) for i in ids]
        new = cache.begin_append(slots, counts)
        cache.end_append(new)
        full = cache.begin_gather(slots)
        total = sum(counts)
        for l in range(L):
            k, v = S.randn(g, (total, H, D), dtype), S.randn(g, (total, H, D), dtype)
            if fused:
                cache.update(l, new, full, k.to(DEV), v.to(DEV), rnd.choice(["HND", "NHD"]))
            else:
                cache.append(l, new, k.to(DEV), v.to(DEV))
            at = 0
            for i, c in zip(ids, counts):
                if c:
                    truth[i][l].append(k[at:at + c].transpose(0, 1).unsqueeze(0), v[at:at + c].transpose(0, 1).unsqueeze(0))
                at += c

    def check():
        ids = sorted(truth, key=str)
        rnd.shuffle(ids)
        if not ids:
            return
        layout, mode = rnd.choice(["HND", "NHD"]), rnd.choice(["vector", "bulk", "auto"])
        gb = cache.begin_gather([cache.slot(i) for i in ids])
        for l in range(L):
            k, v = cache.gather(l, gb, layout, mode=mode)
            if layout == "NHD":
                k, v = k.transpose(0, 1), v.transpose(0, 1)
            for row, i in enumerate(ids):
                a, b = gb.cu[row], gb.cu[row + 1]
                assert b - a == length(i)
                if b > a:
                    wk, wv = truth[i][l].current_tensors()
                    assert torch.equal(S.bits(k[:, a:b]), S.bits(wk[0])), (layout, mode, l, i)
                    assert torch.equal(S.bits(v[:, a:b]), S.bits(wv[0])), (layout, mode, l, i)
        held = {}
        for i in ids:
            for p in cache.pages_of[cache.slot(i)]:
                held[p] = held.get(p, 0) + 1
        assert all(cache.allocator.holders(p) == c for p, c in held.items())
        assert cache.stats().pages_resident == len(held)

    for step in range(160):
        op = rnd.choice(["open", "append", "append", "append", "decode", "decode", "fork", "crop", "release"])
        live = sorted(truth, key=str)
        if op == "open" and len(live) < max_seqs:
            sid = next_id
            next_id += 1
            cache.open(sid)
            truth[sid] = [OracleLayer(1, cap, ps) for _ in range(L)]
        elif op in ("append", "decode") and live:
            ids = rnd.sample(live, rnd.randint(1, len(live)))
            counts = [1 if op == "decode" else rnd.randint(0, 2 * ps + 1) for _ in ids]
            counts = [min(c, cap - length(i)) for i, c in zip(ids, counts)]
            if room(sum(-(-c // ps) + 1 for c in counts)):
                append(ids, counts, fused=rnd.random() < 0.5)
        elif op == "fork" and live and len(live) < max_seqs and room(1):
            src = rnd.choice(live)
            dst = cache.fork(src)
            truth[dst] = copy.deepcopy(truth[src])
        elif op == "crop" and live and room(1):
            sid = rnd.choice(live)
            keep = rnd.randint(0, length(sid)) if rnd.random() < 0.7 else -rnd.randint(0, 3)
            cache.crop(sid, keep)
            for lay in truth[sid]:
                if lay.is_initialized:
                    lay.crop(keep)
        elif op == "release" and live:
            sid = rnd.choice(live)
            cache.release(sid)
            del truth[sid]
        check()
    cache.check_device_status()
    assert backend.read_status(DEV) == 0
