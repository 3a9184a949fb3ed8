"""Host-side logic that needs no GPU: loader contract, C-ABI exports, page allocator, cache
factory and generate() kwargs injection, memory helpers, and the "no CPU fallback" rule."""

import re
import types
from pathlib import Path

import pytest
import torch

from barqtrain_b200 import _build, _ffi
from barqtrain_b200.block_table import PageAllocator, PagePoolExhausted
from barqtrain_b200.kv_cache import (
    BarqPagedKVCache,
    BarqPagedKVCacheLayer,
    create_paged_kv_cache,
    maybe_prepare_paged_kv_generate_kwargs,
)
from barqtrain_b200.memory import CudaMemorySnapshot, cuda_memory_snapshot, generation_overhead_mb

ROOT = Path(__file__).resolve().parent.parent


# ---------------------------------------------------------------------------
# loader (the contract of the reference's tests/test_ffi.py:12-39)
# ---------------------------------------------------------------------------
def test_detect_cuda_home_prefers_environment(monkeypatch, tmp_path):
    home = tmp_path / "cuda"
    home.mkdir()
    monkeypatch.setenv("CUDA_HOME", str(home))
    assert _ffi._detect_cuda_home() == str(home)


def test_loader_retries_after_late_install_and_honours_auto_build_off(monkeypatch):
    fake = object()
    calls = {"n": 0}

    def open_library():
        calls["n"] += 1
        if calls["n"] == 1:
            raise OSError("not built yet")
        return fake

    built = {"n": 0}
    monkeypatch.setattr(_ffi, "_CUDA_BACKEND", None)
    monkeypatch.setattr(_ffi, "_CUDA_BUILD_FAILED", False)
    monkeypatch.setattr(_ffi, "_env_enabled", lambda name, default="1": False)      # auto-build off
    monkeypatch.setattr(_ffi, "_open_library", open_library)
    monkeypatch.setattr(_ffi, "_wrap", lambda lib: lib)
    monkeypatch.setattr(_build, "build_native", lambda **kw: built.__setitem__("n", built["n"] + 1))
    assert _ffi.load_cuda_backend() is None
    assert _ffi.load_cuda_backend() is fake
    assert _ffi.load_cuda_backend() is fake and calls["n"] == 2                      # cached afterwards
    assert built["n"] == 0


def test_loader_builds_once_and_latches_failure(monkeypatch):
    attempts = {"n": 0}

    def failing_build(**kw):
        attempts["n"] += 1
        raise RuntimeError("nvcc exploded")

    monkeypatch.setattr(_ffi, "_CUDA_BACKEND", None)
    monkeypatch.setattr(_ffi, "_CUDA_BUILD_FAILED", False)
    monkeypatch.setattr(_build, "is_stale", lambda: True)
    monkeypatch.setattr(_build, "build_native", failing_build)
    monkeypatch.setattr(_ffi, "_open_library", lambda: (_ for _ in ()).throw(OSError("missing")))
    with pytest.warns(UserWarning, match="auto-build failed"):
        assert _ffi.load_cuda_backend() is None
    assert _ffi.load_cuda_backend() is None
    assert attempts["n"] == 1
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _ffi.require_cuda_backend()


def test_library_exports_every_symbol_the_header_declares():
    """Loads the built library (no compute call) and checks the header's functions are all there."""
    header = (ROOT / "include" / "barqkv.h").read_text()
    declared = set(re.findall(r"\b(barqkv_[a-z_]+)\s*\(", header))
    assert {"barqkv_append", "barqkv_append_legacy", "barqkv_gather", "barqkv_version",
            "barqkv_last_error"} <= declared
    backend = _ffi.load_cuda_backend()
    assert backend is not None, "libbarqkv.so must be built (python -c 'import __graft_entry__ as g; g.build()')"
    for name in sorted(declared):
        assert hasattr(backend.lib, name), name
    assert declared <= set(_ffi.EXPORTS), declared - set(_ffi.EXPORTS)     # and the loader insists on each of them
    assert backend.version == int(re.search(r"#define BARQKV_VERSION (\d+)", header).group(1))
    # struct mirrors have the C sizes
    import ctypes
    assert ctypes.sizeof(_ffi.PoolLayout) == 40 and ctypes.sizeof(_ffi.BlockTable) == 32
    assert ctypes.sizeof(_ffi.RowsLayout) == 32


def test_argument_errors_come_back_as_codes_with_messages():
    """Validation happens before any CUDA call, so it can be exercised without a device."""
    import ctypes

    backend = _ffi.load_cuda_backend()
    pool = _ffi.PoolLayout(0, 128, 16, 2, 10, 0, 0, 0)                    # zero heads
    table = _ffi.BlockTable(None, None, 1, 1, 0, 0)
    rows = _ffi.RowsLayout(0, 0, 0, 1, 0)
    rc = backend.lib.barqkv_gather(ctypes.byref(pool), 1, 1, ctypes.byref(table), 1, 1, 1, 0, 1, 1,
                                   ctypes.byref(rows), 0, None, None, None)
    assert rc == -1 and b"must be positive" in backend.lib.barqkv_last_error()
    pool.num_heads, pool.page_stride = 8, 16 * 128
    rc = backend.lib.barqkv_gather(ctypes.byref(pool), 1, 1, ctypes.byref(table), 1, 1, 9000, 0, 1, 1,
                                   ctypes.byref(rows), 0, None, None, None)
    assert rc == -3 and b"8192" in backend.lib.barqkv_last_error()
    # the serving library has no tuning knobs: no mutable process-wide settings behind the ABI
    assert not hasattr(backend.lib, "barqkv_set_tuning") and not backend.tunable
    with pytest.raises(_ffi.BarqKVError, match="no tuning knobs"):
        backend.set_tuning(stages=4)
    # the no-allocation gather refuses a slot outside its built-in scratch before touching the device
    rc = backend.lib.barqkv_gather_noalloc(ctypes.byref(pool), 1, 1, ctypes.byref(table), 1, 1, 1, 0, 1, 1,
                                           ctypes.byref(rows), 0, None, _ffi.STATIC_WORK_SLOTS, None)
    assert rc == -3 and b"work_slot" in backend.lib.barqkv_last_error()
    rc = backend.lib.barqkv_gather_wait_selftest(ctypes.byref(pool), 1, 1, ctypes.byref(table), 1, 1, 1, 1, 1,
                                                 ctypes.byref(rows), 0, None, None)
    assert rc == -1 and b"wait_cycles" in backend.lib.barqkv_last_error()
    # decode-attention workspace: none while one split per sequence suffices, else counters + partial results
    ws = backend.lib.barqkv_paged_decode_workspace_bytes
    assert ws(64, 8, 64, 0, 16) == 0 and ws(0, 8, 4096, 0, 16) == 0
    big = ws(64, 8, 4096, 0, 16)
    assert big > 0 and big % 16 == 0 and big == ws(64, 8, 4096, 0, 16)
    # the sum of the lengths is an optional hint; with it the answer is still a whole number of 16-byte units
    assert ws(4, 1, 4096, 4 * 4096, 16) > 0 and ws(4, 1, 4096, 4 * 4096, 16) % 16 == 0
    out = ctypes.c_int32(7)
    assert backend.lib.barqkv_max_length(None, 0, ctypes.byref(out), None) == 0 and out.value == 0   # empty: no device work
    assert backend.lib.barqkv_max_length(None, 4, ctypes.byref(out), None) == -1
    assert backend.lib.barqkv_max_length(1, -1, ctypes.byref(out), None) == -1


# ---------------------------------------------------------------------------
# page allocator
# ---------------------------------------------------------------------------
def test_allocator_order_accounting_and_reuse():
    a = PageAllocator(8, order=[5, 2, 7, 0, 1, 3, 4, 6])
    assert a.take(3).tolist() == [5, 2, 7] and a.pages_resident == 3 and a.pages_free == 5
    assert a.take(2).tolist() == [0, 1] and a.pages_peak == 5
    a.give_back([2, 5])
    assert a.pages_resident == 3 and a.pages_peak == 5
    assert a.take(4).tolist() == [3, 4, 6, 2]                       # released pages queue up behind the initial order
    with pytest.raises(PagePoolExhausted):
        a.take(2)
    assert a.pages_resident == 7                           # a refused request changes nothing
    with pytest.raises(AssertionError):
        a.give_back([5, 5])                                # never owned twice
    assert a.pages_resident == 7 and a.free_pages() == [5]
    a.give_back([6, 3, 0])                                 # the ring wraps: freed pages keep their order
    assert a.free_pages() == [5, 6, 3, 0] and a.take(3).tolist() == [5, 6, 3]
    a.share([1, 4]); a.give_back([1, 4, 1])                # a shared page goes back once both holders let go
    assert a.free_pages() == [0, 1] and a.holders(4) == 1
    with pytest.raises(AssertionError):
        a.give_back([7, 0])                                # 0 is free
    seeded = PageAllocator(64, seed=1235)
    assert sorted(seeded.free_pages()) == list(range(64)) and seeded.free_pages() != list(range(64))
    with pytest.raises(ValueError):
        PageAllocator(4, order=[0, 1, 1, 2])


def test_allocator_random_operations_match_a_plain_model():
    """Seeded random take / share / give_back sequences against a dict-and-list model: same pages in the
    same order, same holder counts, same resident and free figures, and the ring never loses a page."""
    import random

    for seed in range(6):
        rng = random.Random(seed)
        num = rng.choice([1, 7, 64, 257])
        order = list(range(num))
        rng.shuffle(order)
        a = PageAllocator(num, order=order)
        free, refs, held = list(order), {}, []          # model: free list, holders per page, one entry per holding
        for _ in range(400):
            op = rng.random()
            if op < 0.45:
                count = rng.randint(0, max(1, num // 3))
                if count > len(free):
                    with pytest.raises(PagePoolExhausted):
                        a.take(count)
                    continue
                want, free = free[:count], free[count:]
                assert a.take(count).tolist() == want
                for p in want:
                    refs[p] = 1
                    held.append(p)
            elif op < 0.6 and held:
                some = rng.sample(sorted(set(held)), k=min(len(set(held)), rng.randint(1, 4)))
                a.share(some)
                for p in some:
                    refs[p] += 1
                    held.append(p)
            elif held:
                k = rng.randint(1, min(len(held), 9))
                rng.shuffle(held)
                back, held = held[:k], held[k:]
                a.give_back(back)
                for p in back:
                    refs[p] -= 1
                free += [p for p in dict.fromkeys(back) if refs[p] == 0]     # in the order first mentioned
            assert a.free_pages() == free
            assert a.pages_free == len(free) and a.pages_resident == num - len(free)
            assert all(a.holders(p) == refs.get(p, 0) for p in range(num))
        assert sorted(a.free_pages() + sorted(set(held))) == list(range(num))


# ---------------------------------------------------------------------------
# reference API: factory, kwargs injection (reference tests/test_kv_cache.py:50-107), no CPU path
# ---------------------------------------------------------------------------
class _DecoderConfig:
    num_hidden_layers = 3


class _Config:
    def get_text_config(self, decoder=True):
        return _DecoderConfig()


def test_factory_builds_one_layer_per_decoder_layer():
    cache = create_paged_kv_cache(_Config(), max_batch_size=2, max_cache_len=64, page_size=16)
    assert isinstance(cache, BarqPagedKVCache) and len(cache.layers) == 3
    assert (cache.barqtrain_max_batch_size, cache.barqtrain_max_cache_len, cache.page_size) == (2, 64, 16)
    layer = cache.layers[0]
    assert layer.max_blocks == 4 and layer.get_seq_length() == 0 and layer.get_max_cache_shape() == 64
    assert layer.get_mask_sizes(5) == (5, 0) and layer.get_mask_sizes(torch.arange(3)) == (3, 0)

    class Shared(_DecoderConfig):
        num_kv_shared_layers = 1

    assert len(BarqPagedKVCache(Shared(), 1, 16).layers) == 2


def _model(max_length=32):
    return types.SimpleNamespace(config=_Config(), _barqtrain_paged_kv_supported=True,
                                 generation_config=types.SimpleNamespace(max_new_tokens=None, max_length=max_length))


def test_generate_kwargs_injection_gates(monkeypatch):
    monkeypatch.setattr("barqtrain_b200.kv_cache._get_cuda_backend", lambda: object())
    monkeypatch.setenv("BARQTRAIN_PAGED_KV_MIN_CACHE_LEN", "0")
    ids = types.SimpleNamespace(shape=(2, 8), device=torch.device("cuda"))

    kwargs, used = maybe_prepare_paged_kv_generate_kwargs(_model(), (), {"input_ids": ids, "max_new_tokens": 4})
    assert used and kwargs["use_cache"] is True
    cache = kwargs["past_key_values"]
    assert isinstance(cache, BarqPagedKVCache)
    assert (cache.barqtrain_max_batch_size, cache.barqtrain_max_cache_len) == (2, 12)

    # positional input_ids, length from generation_config.max_length
    kwargs, used = maybe_prepare_paged_kv_generate_kwargs(_model(40), (ids,), {})
    assert used and kwargs["past_key_values"].barqtrain_max_cache_len == 40

    monkeypatch.setenv("BARQTRAIN_PAGED_KV_PAGE_SIZE", "32")
    kwargs, _ = maybe_prepare_paged_kv_generate_kwargs(_model(), (), {"input_ids": ids, "max_new_tokens": 4})
    assert kwargs["past_key_values"].page_size == 32

    def refused(model, kw):
        out, used = maybe_prepare_paged_kv_generate_kwargs(model, (), kw)
        return (not used) and "past_key_values" not in {k: v for k, v in out.items() if k not in kw}

    assert refused(_model(), {"input_ids": ids, "past_key_values": "mine"})          # caller's cache wins
    assert refused(_model(), {"input_ids": types.SimpleNamespace(shape=(2, 8), device=torch.device("cpu")),
                              "max_new_tokens": 4})                                  # not on a GPU
    assert refused(types.SimpleNamespace(config=_Config()), {"input_ids": ids, "max_new_tokens": 4})
    assert refused(_model(None), {"input_ids": ids})                                  # no length known
    assert refused(_model(), {"max_new_tokens": 4})                                   # no inputs
    monkeypatch.setenv("BARQTRAIN_PAGED_KV_MIN_CACHE_LEN", "256")
    assert refused(_model(), {"input_ids": ids, "max_new_tokens": 16})               # too short to pay off
    monkeypatch.setenv("BARQTRAIN_PAGED_KV_MIN_CACHE_LEN", "0")
    monkeypatch.setenv("BARQTRAIN_ENABLE_PAGED_KV", "off")
    assert refused(_model(), {"input_ids": ids, "max_new_tokens": 4})
    monkeypatch.setenv("BARQTRAIN_ENABLE_PAGED_KV", "1")
    monkeypatch.setattr("barqtrain_b200.kv_cache._get_cuda_backend", lambda: None)
    assert refused(_model(), {"input_ids": ids, "max_new_tokens": 4})                # library missing


def test_layer_has_no_cpu_fallback():
    layer = BarqPagedKVCacheLayer(max_batch_size=1, max_cache_len=8, page_size=4)
    k = torch.zeros(1, 2, 3, 4)
    with pytest.raises(RuntimeError, match="no CPU append"):
        layer.update(k, k)
    with pytest.raises(ValueError):
        layer.lazy_initialization(torch.zeros(2, 3, 4))
    with pytest.raises(ValueError, match="exceeds max_batch_size"):
        layer.lazy_initialization(torch.zeros(2, 2, 3, 4))
    layer.crop(3)
    layer.reset()                                                                   # no-ops before first use
    assert layer.get_seq_length() == 0


def test_product_never_imports_the_oracle():
    for path in (ROOT / "barqtrain_b200").rglob("*.py"):
        text = path.read_text()
        assert "oracle" not in text.replace("the oracle", ""), path
    assert "oracle" not in (ROOT / "barqtrain_b200" / "csrc" / "barqkv.cu").read_text()


# ---------------------------------------------------------------------------
# memory helpers (reference tests/test_memory.py:16-29)
# ---------------------------------------------------------------------------
def test_memory_snapshot_and_overhead(monkeypatch):
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert cuda_memory_snapshot() == CudaMemorySnapshot()
    resident, peak = CudaMemorySnapshot(allocated_mb=256.0), CudaMemorySnapshot(max_allocated_mb=384.0)
    assert generation_overhead_mb(resident, peak) == 128.0
    assert generation_overhead_mb(peak, resident) == 0.0
