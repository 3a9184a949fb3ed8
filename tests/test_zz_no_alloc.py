"""``barqkv_gather_noalloc``: the gather for callers that cannot allocate device memory.

A server that has handed all free HBM to its own arena, or a plugin host that forbids
allocation inside an operator call, cannot give ``barqkv_gather`` the small ``work`` buffer
it wants for its page hand-out counters.  This entry point keeps those counters in an array
built into the library.  The test drives it through the C ABI (raw pointers, ctypes) and
requires its output to be bit-identical to ``barqkv_gather``'s on two calls in a row that
share a scratch slot - the second with a different batch, so state left by the first call
would show - and checks that a slot beyond the built-in array is refused.

Collected last on purpose (file name), so a run that stops at the first failure has already
run every other test.  It depends on no other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

E_LIMIT = -3


def _bind(lib):
    from barqtrain_b200._ffi import BlockTable, PoolLayout, RowsLayout

    i32, i64, ptr, P = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.POINTER
    fn = lib.barqkv_gather_noalloc
    fn.restype = i32
    fn.argtypes = [P(PoolLayout), ptr, ptr, P(BlockTable), ptr, ptr, i32, i64, ptr, ptr, P(RowsLayout), i32, ptr, i32, ptr]
    return fn


def test_gather_noalloc_matches_gather_on_two_calls_in_a_row():
    from barqtrain_b200 import BlockTableKVCache, _ffi

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    backend = _ffi.require_cuda_backend()
    gather_noalloc = _bind(backend.lib)

    g = torch.Generator().manual_seed(404)
    H, D, ps, dtype = 4, 128, 16, torch.bfloat16
    lens = [700, 33, 1, 512, 1290, 16, 255]
    pages = sum(-(-n // ps) for n in lens) + 5
    cache = BlockTableKVCache(1, H, D, page_size=ps, num_pages=pages, max_seqs=len(lens),
                              max_blocks_per_seq=-(-max(lens) // ps), dtype=dtype, device=dev, seed=8)
    slots = [cache.open(i) for i in range(len(lens))]
    k = torch.randn(sum(lens), H, D, generator=g).to(dtype).to(dev)
    v = torch.randn(sum(lens), H, D, generator=g).to(dtype).to(dev)
    cache.append_step(slots, lens, [k], [v])
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = backend.status_word(dev)

    def both(batch_slots, layout, work_slot):
        gb = cache.begin_gather(batch_slots)
        want_k, want_v = cache.gather(0, gb, layout, mode="bulk")          # the existing entry point
        got_k = torch.full_like(want_k, float("nan"))
        got_v = torch.full_like(want_v, float("nan"))
        total = gb.total
        rows = _ffi.RowsLayout(0, D, total * D, 1, 0) if layout == "HND" else _ffi.RowsLayout(0, H * D, D, 1, 0)
        cache._table.slots = gb.p_slots
        rc = gather_noalloc(ctypes.byref(cache._pool_layout), cache._k_ptr[0], cache._v_ptr[0],
                            ctypes.byref(cache._table), gb.p_first, gb.p_cu, gb.n, total,
                            got_k.data_ptr(), got_v.data_ptr(), ctypes.byref(rows), _ffi.MODE_BULK,
                            status.data_ptr(), work_slot, stream)
        assert rc == 0, backend.lib.barqkv_last_error()
        torch.cuda.synchronize(dev)
        view = {2: torch.int16}[want_k.element_size()]
        assert torch.equal(got_k.view(view), want_k.view(view))            # bit-exact, as everywhere on this path
        assert torch.equal(got_v.view(view), want_v.view(view))
        return total

    # First call on this device: performs the one-time address look-up of the built-in scratch.  The library's
    # device code is loaded already (the appends above ran its kernels), so even this call must not take device
    # memory: the array it uses came with the code image.  Output tensors are made before the reading.
    warm = cache.gather(0, cache.begin_gather(slots), "HND", mode="bulk")
    spare = [torch.full_like(warm[0], float("nan")) for _ in range(2)]
    del warm, spare                                        # torch keeps the blocks cached for the calls below
    torch.cuda.synchronize(dev)
    free_before_first = torch.cuda.mem_get_info(dev)[0]
    assert both(slots, "HND", work_slot=3) == sum(lens)
    free_after_first = torch.cuda.mem_get_info(dev)[0]
    assert free_after_first >= free_before_first - (1 << 20)
    # second call, same slot, a different and smaller batch in another layout: leftovers would corrupt it
    assert both([slots[4], slots[0], slots[2]], "NHD", work_slot=3) == 1290 + 700 + 1
    assert both(slots, "HND", work_slot=31) == sum(lens)
    # the entry point itself took no device memory (the tensors above come from torch's cached blocks)
    assert torch.cuda.mem_get_info(dev)[0] >= free_after_first - (1 << 20)

    # a slot beyond the built-in array is refused with a clear message and nothing is launched
    gb = cache.begin_gather(slots)
    out_k = torch.zeros(H, gb.total, D, dtype=dtype, device=dev)
    out_v = torch.zeros_like(out_k)
    rows = _ffi.RowsLayout(0, D, gb.total * D, 1, 0)
    cache._table.slots = gb.p_slots
    for bad in (32, -1, 1000):
        rc = gather_noalloc(ctypes.byref(cache._pool_layout), cache._k_ptr[0], cache._v_ptr[0],
                            ctypes.byref(cache._table), gb.p_first, gb.p_cu, gb.n, gb.total,
                            out_k.data_ptr(), out_v.data_ptr(), ctypes.byref(rows), _ffi.MODE_BULK,
                            status.data_ptr(), bad, stream)
        assert rc == E_LIMIT
        assert b"work_slot" in backend.lib.barqkv_last_error()
    torch.cuda.synchronize(dev)
    assert not out_k.any() and not out_v.any()
    assert backend.read_status(dev) == 0
