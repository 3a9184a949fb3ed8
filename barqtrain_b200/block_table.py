"""Block-table paged KV cache: page pool, free list, append, gather, release.

The reference's layer gives every (sequence, head) a private run of
``max_blocks`` adjacent pages (``python/barqtrain/kv_cache.py:66-70,84-89``) -
a block table fixed at ``table[b][j] = j``.  This module is the general form
its roadmap describes: one pool of pages per layer shared by all sequences, an
explicit ``[slot, logical page] -> physical page`` table, a free list pages are
drawn from and returned to, and a gather that turns a sequence's scattered
pages back into contiguous K/V.  Logical content is defined by the reference:
logical page ``j`` of a sequence equals the reference's ``keys[b, :, j]`` and a
gathered sequence equals its ``current_tensors()`` slice.

Layout in device memory, per layer: ``K`` and ``V`` pools of shape
``[kv_heads, num_pages, page_size, head_dim]`` (a page of one head is
contiguous - 4 KiB at page 16, head_dim 128, 2-byte elements - and a KV-head
shard is a contiguous slice).  All layers share one block table and one set of
lengths; the host owns both and mirrors them to the device.

All device work goes through ``libbarqkv.so``; there is no CPU path.
"""

from __future__ import annotations

import ctypes
import gc
from dataclasses import dataclass

import numpy as np
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from . import _ffi


class PagePoolExhausted(RuntimeError):
    """The free list cannot satisfy an allocation; nothing was changed."""


E_INVALID, E_LIMIT, E_CAPACITY = -1, -3, -4


def _i32(values) -> np.ndarray:
    return np.ascontiguousarray(values, dtype=np.int32).reshape(-1)


class PageAllocator:
    """Host-side free list with resident/peak accounting (native: ``barqkv_host_*`` in ``libbarqkv.so``).

    ``order`` fixes the initial free list (e.g. a seeded permutation, so tests
    and benchmarks get fragmented but reproducible tables); pages are handed
    out from its front and released pages go to its back.  A page may have
    several holders (forked sequences share their full pages).
    """

    def __init__(self, num_pages: int, order: Optional[Sequence[int]] = None, seed: Optional[int] = None, *,
                 _handle=None, _backend=None):
        self.backend = _backend or _ffi.require_cuda_backend()
        self._lib = self.backend.lib
        self.num_pages = num_pages
        if _handle is not None:                 # the free list of a BlockTableKVCache's native table
            self._h, self._owns = _handle, False
            return
        self._h = _create_host_table(self.backend, num_pages, order, seed, 0, 0, 1, None, None, None)
        self._owns = True

    def __del__(self):
        if getattr(self, "_owns", False) and self._h:
            self._lib.barqkv_host_destroy(self._h)
            self._h = None

    def _stats(self) -> List[int]:
        out = (ctypes.c_int64 * 6)()
        self._lib.barqkv_host_stats(self._h, out)
        return list(out)

    pages_free = property(lambda self: self._stats()[0])
    pages_resident = property(lambda self: self._stats()[1])
    pages_peak = property(lambda self: self._stats()[2])
    alloc_calls = property(lambda self: self._stats()[3])
    release_calls = property(lambda self: self._stats()[4])

    def free_pages(self) -> List[int]:
        """The free list, front first."""
        out = np.empty(self.num_pages, dtype=np.int32)
        count = self._lib.barqkv_host_free_list(self._h, out.ctypes.data, self.num_pages)
        return out[:count].tolist()

    def take(self, count: int) -> np.ndarray:
        """``count`` pages from the front of the free list, as an int32 array."""
        out = np.empty(max(count, 0), dtype=np.int32)
        rc = self._lib.barqkv_host_take(self._h, count, out.ctypes.data)
        if rc == E_LIMIT:
            raise PagePoolExhausted(self.backend.last_error())
        if rc:
            raise AssertionError(self.backend.last_error())
        return out

    def share(self, pages: Iterable[int]) -> None:
        """One more holder for pages that are already held (a forked sequence)."""
        idx = _i32(list(pages) if not isinstance(pages, np.ndarray) else pages)
        if idx.size and self._lib.barqkv_host_share(self._h, idx.ctypes.data, idx.size):
            raise AssertionError(self.backend.last_error())

    def holders(self, page: int) -> int:
        return int(self._lib.barqkv_host_holders(self._h, int(page)))

    def give_back(self, pages: Iterable[int]) -> None:
        """Drop one holder of each page; pages nobody holds any more join the back of the free list."""
        idx = _i32(list(pages) if not isinstance(pages, np.ndarray) else pages)
        if self._lib.barqkv_host_give_back(self._h, idx.ctypes.data if idx.size else None, idx.size):
            raise AssertionError(self.backend.last_error())


def _create_host_table(backend, num_pages, order, seed, max_seqs, max_blocks, page_size, table_ptr, lengths_ptr, count_ptr):
    if order is None and seed is not None:
        g = torch.Generator().manual_seed(seed)
        order = torch.randperm(num_pages, generator=g).numpy()
    order_ptr = None
    if order is not None:
        order = _i32(order)
        if order.size != num_pages:
            raise ValueError("free-list order must be a permutation of range(num_pages)")
        order_ptr = order.ctypes.data
    handle = backend.lib.barqkv_host_create(num_pages, order_ptr, max_seqs, max_blocks, page_size, table_ptr, lengths_ptr,
                                            count_ptr)
    if not handle:
        raise ValueError(backend.last_error())
    return handle


@dataclass(frozen=True)
class PoolStats:
    pages_total: int
    pages_resident: int
    pages_peak: int
    bytes_per_page: int          # all layers, K and V, all local heads
    bytes_resident: int
    bytes_peak: int
    sequences_live: int


_GATHER_MAX_ENTRIES = 8192      # sequences one gather launch can scan (the library's limit)


class _PagesOf:
    """``cache.pages_of[slot]``: the slot's page ids in logical order (read from the host block table)."""

    def __init__(self, cache):
        self._cache = cache

    def __getitem__(self, slot: int) -> List[int]:
        c = self._cache
        return c._table_np[slot, :int(c._page_count[slot])].tolist()

    def __len__(self) -> int:
        return self._cache.max_seqs


class _Descriptor:
    """Per-step int32 batch description on the device:
    ``[slots(n) | first(n) | cu(n + 1)]`` where ``first`` is the start position
    (append) or the length (gather) and ``cu`` the packed row offsets."""

    def __init__(self, n: int, dev: torch.Tensor, total: int, host_first, host_cu, slots, table_ref=None,
                 stream: int = 0, work: int = 0):
        self.kind, self.generation = None, 0     # set by the cache: which shared device buffer holds it, and its turn
        self.used_at = -1               # the cache's upload count when a kernel last used this description
        self.table_ref = table_ref      # ctypes reference to a barqkv_block_table whose `slots` points into `dev`
        self.stream = stream            # the CUDA stream the description was uploaded on
        self.work = work                # the stream's hand-out counters (bulk gather, bulk append)
        self.n = n
        self.dev = dev
        self.total = total
        # host copies, as lists or numpy arrays; the list views below are made when somebody asks
        self._first, self._cu, self._slots = host_first, host_cu, slots
        base = dev.data_ptr()
        self.p_slots = base
        self.p_first = base + 4 * n
        self.p_cu = base + 8 * n

    @staticmethod
    def _as_list(values) -> List[int]:
        return values if isinstance(values, list) else values.tolist()

    @property
    def first(self) -> List[int]:
        """Start positions (append) or lengths (gather), one per entry."""
        self._first = self._as_list(self._first)
        return self._first

    @property
    def cu(self) -> List[int]:
        """Packed row offsets: entry ``i`` owns rows ``cu[i]:cu[i + 1]``."""
        self._cu = self._as_list(self._cu)
        return self._cu

    @property
    def slots(self) -> List[int]:
        self._slots = self._as_list(self._slots)
        return self._slots


# Native host tables whose owner is gone.  Destroying one waits for its last uploads and frees pinned memory -
# neither is allowed while a stream of this thread records a CUDA graph, and the garbage collector may well run
# a cache's finaliser in the middle of a recording - so the handles wait here until no recording is under way.
_PENDING_DESTROY: list = []


def _destroy_pending() -> None:
    try:
        if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
            return
    except Exception:  # noqa: BLE001 - interpreter or context already going down
        return
    while _PENDING_DESTROY:
        backend, host, device = _PENDING_DESTROY.pop()
        try:
            torch.cuda.synchronize(device)                # uploads out of the staging memory must have run
        except Exception:  # noqa: BLE001
            pass
        backend.lib.barqkv_host_destroy(host)


class BlockTableKVCache:
    """Paged K/V for ``num_layers`` layers over a shared block table.

    ``num_kv_heads`` is the number of heads THIS device holds (the full count
    divided by the tensor-parallel size when the cache is sharded by KV head).
    """

    def __init__(self, num_layers: int, num_kv_heads: int, head_dim: int, *, page_size: int = 16, num_pages: int,
                 max_seqs: int, max_blocks_per_seq: int, dtype: torch.dtype = torch.bfloat16,
                 device="cuda", free_order: Optional[Sequence[int]] = None, seed: Optional[int] = None,
                 zero_pages: bool = True, gather_mode: str = "auto"):
        self.backend = _ffi.require_cuda_backend()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("BlockTableKVCache needs a CUDA device: this build has no CPU path")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.num_layers, self.num_kv_heads, self.head_dim = num_layers, num_kv_heads, head_dim
        self.page_size, self.num_pages = page_size, num_pages
        self.max_seqs, self.max_blocks = max_seqs, max_blocks_per_seq
        self.dtype = dtype
        self.gather_mode = gather_mode

        shape = (num_layers, 2, num_kv_heads, num_pages, page_size, head_dim)
        self.pools = (torch.zeros if zero_pages else torch.empty)(shape, dtype=dtype, device=self.device)
        self.elem = self.pools.element_size()
        page_elems = page_size * head_dim
        self._pool_layout = _ffi.PoolLayout(num_kv_heads, head_dim, page_size, self.elem, num_pages, 0,
                                            num_pages * page_elems, page_elems)
        self._k_ptr = [self.pools[l, 0].data_ptr() for l in range(num_layers)]
        self._v_ptr = [self.pools[l, 1].data_ptr() for l in range(num_layers)]

        # block table: pinned host copy is authoritative, device copy follows.  The free list, the table rows and
        # the per-step descriptions are kept by native code (barqkv_host_*); the arrays below are shared with it.
        self.table_host = torch.full((max_seqs, max_blocks_per_seq), -1, dtype=torch.int32).pin_memory()
        self.table_dev = torch.full((max_seqs, max_blocks_per_seq), -1, dtype=torch.int32, device=self.device)
        self._table_np = self.table_host.numpy()
        self._table = _ffi.BlockTable(self.table_dev.data_ptr(), None, max_seqs, max_blocks_per_seq, 0, 0)
        self.lengths = np.zeros(max_seqs, dtype=np.int64)      # tokens held, per slot
        self._page_count = np.zeros(max_seqs, dtype=np.int64)  # pages owned, per slot
        _destroy_pending()
        self._host = _create_host_table(self.backend, num_pages, free_order, seed, max_seqs, max_blocks_per_seq, page_size,
                                        self.table_host.data_ptr(), self.lengths.ctypes.data,
                                        self._page_count.ctypes.data)
        self.allocator = PageAllocator(num_pages, _handle=self._host, _backend=self.backend)
        # A step's upload is its description (at most 5 * max_seqs + 2 words) followed by the table entries that
        # changed (two words each); more entries than fit go in several uploads.
        self._step_words = 5 * max_seqs + 2 + 2 * min(max(max_seqs * max_blocks_per_seq, 1024), 1 << 18)
        self._step_dev = [torch.zeros(self._step_words, dtype=torch.int32, device=self.device) for _ in range(2)]
        # staging ring: up to 32 steps for small tables (the host may run that far ahead of the device), 4 MiB at most
        ring = max(2, min(32, (1 << 20) // self._step_words))
        self._staging = torch.zeros(ring * self._step_words, dtype=torch.int32).pin_memory()
        rc = self.backend.lib.barqkv_host_attach(self._host, self.table_dev.data_ptr(), self._step_dev[0].data_ptr(),
                                                 self._step_dev[1].data_ptr(), self._step_words,
                                                 self._staging.data_ptr(), self._staging.numel())
        if rc:
            self.backend._check(rc)
        self._c_begin = self.backend.lib.barqkv_host_begin
        self._info = (ctypes.c_int64 * 8)()
        self._staging_np, self._staging_ptr = self._staging.numpy(), self._staging.data_ptr()
        self._work_bases: Dict[int, int] = {}
        self.pages_of = _PagesOf(self)                         # pages_of[slot] -> list of page ids, in order
        self._free_slots: List[int] = list(range(max_seqs - 1, -1, -1))
        self._slot_of: Dict[object, int] = {}
        self._fork_counter = 0
        self._attn_ws, self._attn_ws_bytes = None, 0

        self._desc_turn: Dict[str, int] = {}
        self._uploads = 0               # descriptions uploaded + table scatters enqueued so far
        self._tables: Dict[str, _ffi.BlockTable] = {}
        self._status = self.backend.status_word(self.device)
        # per-call constants of the native calls, resolved once
        self._status_ptr = self._status.data_ptr()
        self._pool_ref = ctypes.byref(self._pool_layout)
        self._c_append = self.backend.lib.barqkv_append
        self._c_gather = self.backend.lib.barqkv_gather
        self._c_update = self.backend.lib.barqkv_update
        self._rows: Dict[Tuple[int, ...], object] = {}
        self._new_shape = (0, num_kv_heads, head_dim)

    # -- sequences and pages ----------------------------------------------------
    def open(self, seq_id=None) -> int:
        """Claim a table row for a new sequence; returns its slot."""
        if not self._free_slots:
            raise RuntimeError(f"all {self.max_seqs} sequence slots are in use")
        slot = self._free_slots.pop()
        self._slot_of[slot if seq_id is None else seq_id] = slot
        self.lengths[slot] = 0
        return slot

    def slot(self, seq_id) -> int:
        return self._slot_of[seq_id]

    def close(self) -> None:
        """Give the pools and every other buffer back now.  The cache object sits in reference cycles (its page
        views, its allocator), so without this its device memory waits for the garbage collector; after it the
        object must not be used any more."""
        host, backend = getattr(self, "_host", None), getattr(self, "backend", None)
        if host and backend is not None:
            self._host = None
            if getattr(self, "allocator", None) is not None:
                self.allocator._h = None
            _PENDING_DESTROY.append((backend, host, self.device))
            _destroy_pending()
        self.pools = self.table_dev = self._attn_ws = None
        self._step_dev, self._staging, self._staging_np = [], None, None
        self._k_ptr, self._v_ptr = [], []

    def __del__(self):
        self.close()

    def _raise_host(self, rc: int):
        msg = self.backend.last_error()
        if rc == E_CAPACITY:
            raise ValueError(msg)
        if rc == E_LIMIT and msg.startswith("need "):
            raise PagePoolExhausted(msg)
        if rc == E_INVALID and msg.startswith("page "):
            raise AssertionError(msg)
        raise _ffi.BarqKVError(msg)

    def release(self, seq_id) -> None:
        """Return a sequence's pages to the free list and free its slot (data stays in the pages; the row is
        cleared in the host table only - kernels never read entries beyond a sequence's length, so the device
        copy keeps the stale ids until a new owner of the row overwrites them)."""
        slot = self._slot_of.pop(seq_id)
        rc = self.backend.lib.barqkv_host_release(self._host, slot)
        if rc:
            self._raise_host(rc)
        self._free_slots.append(slot)

    def reserve(self, slot: int, new_length: int) -> None:
        """Make sure the slot owns pages for ``new_length`` tokens."""
        rc = self.backend.lib.barqkv_host_reserve(self._host, slot, int(new_length))
        if rc:
            self._raise_host(rc)

    # -- forks, crops, beam reordering: table edits plus at most one page copy per sequence --------
    def _copy_pages(self, pairs: List[Tuple[int, int]]) -> None:
        if not pairs:
            return
        ids = torch.tensor([p[0] for p in pairs] + [p[1] for p in pairs], dtype=torch.int32, device=self.device)
        n = len(pairs)
        rc = self.backend.lib.barqkv_copy_pages(self._pool_ref, self._k_ptr[0], self._v_ptr[0], self.num_layers,
                                                self.pools.stride(0), ids.data_ptr(), ids.data_ptr() + 4 * n, n,
                                                self._status_ptr, torch.cuda.current_stream(self.device).cuda_stream)
        if rc:
            self.backend._check(rc)

    def _set_pages(self, slot: int, pages: List[int]) -> None:
        arr = _i32(pages)
        rc = self.backend.lib.barqkv_host_set_pages(self._host, slot, arr.ctypes.data if arr.size else None, arr.size)
        if rc:
            self._raise_host(rc)

    def fork(self, seq_id, new_seq_id=None):
        """A new sequence with the same contents as ``seq_id`` (the block-table form of the reference's
        ``batch_repeat_interleave``, ``kv_cache.py:166-173``, which copies the whole cache row).

        Full pages are shared between the two sequences; only a partial last page - the one both will
        append into - is copied, in every layer.  Returns the new sequence's id.
        """
        src = self.slot(seq_id)
        if new_seq_id is None:
            new_seq_id = ("fork", self._fork_counter)
            self._fork_counter += 1
        dst = self.open(new_seq_id)
        length = int(self.lengths[src])
        full, partial = divmod(length, self.page_size)
        pages = list(self.pages_of[src][:full])
        self.allocator.share(pages)
        if partial:
            try:
                fresh = int(self.allocator.take(1)[0])
            except PagePoolExhausted:
                self.allocator.give_back(pages)
                self._slot_of.pop(new_seq_id)
                self._free_slots.append(dst)
                raise
            self._copy_pages([(self.pages_of[src][full], fresh)])
            pages.append(fresh)
        self._set_pages(dst, pages)
        self.lengths[dst] = length
        return new_seq_id

    def crop(self, seq_id, max_length: int) -> None:
        """Shorten a sequence to ``max_length`` tokens (negative: that many fewer), as the reference's
        ``crop`` does for a layer (``kv_cache.py:158-164``).  Pages no longer needed go back to the free
        list; rows beyond the new length in the last kept page stay as they are."""
        slot = self.slot(seq_id)
        length = int(self.lengths[slot])
        if max_length < 0:
            max_length = length - abs(max_length)
        new_length = min(length, max(max_length, 0))
        keep = -(-new_length // self.page_size)
        pages = self.pages_of[slot]
        fresh = None
        if new_length % self.page_size and self.allocator.holders(pages[keep - 1]) > 1:
            # The sequence will append into a page it shares: it gets a copy of its own.  That page is taken
            # before anything is given back, so an exhausted pool raises with the cache unchanged.
            fresh = int(self.allocator.take(1)[0])
        if keep < len(pages):
            self.allocator.give_back(pages[keep:])
            pages = pages[:keep]
        if fresh is not None:
            self._copy_pages([(pages[-1], fresh)])
            self.allocator.give_back([pages[-1]])
            pages = pages[:-1] + [fresh]
        self._set_pages(slot, list(pages))
        self.lengths[slot] = new_length

    def reorder(self, seq_ids: Sequence, beam_idx: Sequence[int]) -> List:
        """Beam-search reordering: entry ``i`` of the new batch continues ``seq_ids[beam_idx[i]]``
        (the reference's ``batch_select_indices`` / ``reorder_cache``, ``kv_cache.py:175-186``).
        Returns the new batch's sequence ids; sequences no beam continues are released."""
        chosen = [seq_ids[int(b)] for b in beam_idx]
        kept = set(chosen)
        for sid in seq_ids:                      # dropped beams first: their slots and pages serve the forks
            if sid not in kept:
                self.release(sid)
        seen = set()
        out = []
        for sid in chosen:
            if sid in seen:
                out.append(self.fork(sid))
            else:
                seen.add(sid)
                out.append(sid)
        return out

    # -- a step's host work: pages, table entries, description - one native call ------------------------
    def _begin(self, kind: str, slots, counts) -> _Descriptor:
        slots32 = slots if (type(slots) is np.ndarray and slots.dtype == np.int32 and slots.ndim == 1
                            and slots.flags.c_contiguous) else _i32(slots)
        n = slots32.size
        code = 0 if kind == "append" else 1
        counts_ptr = None
        if code == 0:
            counts32 = counts if (type(counts) is np.ndarray and counts.dtype == np.int32 and counts.ndim == 1
                                  and counts.flags.c_contiguous) else _i32(counts)
            if counts32.size != n:
                raise ValueError("slots and counts must have the same length")
            counts_ptr = counts32.ctypes.data if n else None
        stream = torch.cuda.current_stream(self.device).cuda_stream
        info = self._info
        rc = self._c_begin(self._host, code, slots32.ctypes.data if n else None, counts_ptr, n, 0, stream, info)
        if rc:
            self._raise_host(rc)
        self._uploads += 1
        # host copy of the description the native side just wrote into the staging ring: [slots | first | cu]
        at = (info[4] - self._staging_ptr) >> 2
        host = self._staging_np[at:at + 3 * n + 1].copy()
        first, cu = host[n:2 * n], host[2 * n:]
        table = self._tables.get(kind)
        if table is None:
            table = _ffi.BlockTable(self.table_dev.data_ptr(), self._step_dev[code].data_ptr(), self.max_seqs,
                                    self.max_blocks, 0, 0)
            self._tables[kind] = (table, ctypes.byref(table))
            table = self._tables[kind]
        desc = _Descriptor(n, self._step_dev[code], info[0], first, cu, host[:n], table[1], stream, self._work_base(stream))
        desc.slots_np = host[:n]
        desc.after_np = cu[1:] - cu[:-1]
        desc.after_np += first
        desc.max_first = info[1]
        # The device buffer of a kind is rewritten by the next begin_* of that kind: an older description
        # would silently address the newer one's contents, so every use checks that it is still current.
        turn = self._desc_turn.get(kind, 0) + 1
        self._desc_turn[kind] = turn
        desc.kind, desc.generation = kind, turn
        return desc

    def _work_base(self, stream: int) -> int:
        base = self._work_bases.get(stream)
        if base is None:
            base = self._work_bases[stream] = self.backend.work_words(self.device).data_ptr()
        return base

    def _launch_terms(self, desc: _Descriptor) -> Tuple[int, int]:
        """(work pointer, flag) for the next kernel that uses ``desc``.  The flag says that nothing the kernel
        reads besides K/V has been uploaded or scattered since an earlier kernel used the same description -
        true from the second layer of a step on - which lets the kernel's prologue overlap its predecessor."""
        flag = _ffi.FLAG_DESC_STABLE if desc.used_at == self._uploads else 0
        desc.used_at = self._uploads
        return self.backend.take_work(self.device.index, desc.stream), flag

    def _current(self, desc: _Descriptor) -> _Descriptor:
        if desc.kind is not None and desc.generation != self._desc_turn.get(desc.kind):
            raise RuntimeError(f"this {desc.kind} description is stale: a later begin_{desc.kind} of this cache "
                               f"has rewritten the device buffer it points to")
        return desc

    # -- append -------------------------------------------------------------------
    def begin_append(self, slots: Sequence[int], counts: Sequence[int]) -> _Descriptor:
        """Reserve pages for ``counts[i]`` new tokens of ``slots[i]`` and upload the step description.

        Use the returned batch for every layer's ``append`` of this step, then ``end_append``.
        """
        return self._begin("append", slots, counts)

    def append(self, layer: int, batch: _Descriptor, k_new: torch.Tensor, v_new: torch.Tensor,
               rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> None:
        """Scatter packed new rows ``[total_tokens, kv_heads, head_dim]`` (any strides with a
        contiguous last dimension; ``[H, T, D].transpose(0, 1)`` works) into the layer's pages.

        ``rope=(cos, sin)``, each ``[total_tokens, head_dim]`` in the cache dtype: the K rows are stored as
        ``k * cos + rotate_half(k) * sin`` (bit-identical to rotating first), saving that separate pass."""
        total = self._current(batch).total
        if total == 0:
            return
        shape = k_new.shape
        if shape != v_new.shape or len(shape) != 3:
            raise ValueError("k_new and v_new must both be [total_tokens, kv_heads, head_dim]")
        if shape[0] != total or shape[1] != self.num_kv_heads or shape[2] != self.head_dim:
            raise ValueError(f"new rows have shape {tuple(shape)}, expected "
                             f"{(total, self.num_kv_heads, self.head_dim)}")
        if k_new.dtype != self.dtype or v_new.dtype != self.dtype:
            raise ValueError("new rows must be in the cache dtype")
        if k_new.device != self.device or v_new.device != self.device:
            raise ValueError("new rows must be on the cache device")
        strides = k_new.stride()
        if strides[2] != 1 or v_new.stride() != strides:
            k_new, v_new = k_new.contiguous(), v_new.contiguous()
            strides = k_new.stride()
        rows_ref = self._rows.get(strides)
        if rows_ref is None:
            rows_ref = self._rows[strides] = self._rows_ref(0, strides[0], strides[1])
        if rope is not None:
            cos, sin = rope
            want = (total, self.head_dim)
            if cos.shape != want or sin.shape != want or cos.dtype != self.dtype or sin.dtype != self.dtype \
                    or cos.device != self.device or sin.device != self.device:
                raise ValueError(f"rope cos and sin must be {want} in the cache dtype on the cache device")
            if cos.stride(1) != 1 or sin.stride() != cos.stride():
                cos, sin = cos.contiguous(), sin.contiguous()
            code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}.get(self.dtype)
            if code is None:
                raise ValueError("rope needs a bf16, fp16 or fp32 cache")
            rc = self.backend.lib.barqkv_append_rope(
                self._pool_ref, self._k_ptr[layer], self._v_ptr[layer], batch.table_ref, batch.p_first, batch.p_cu,
                batch.n, 0, total, k_new.data_ptr(), v_new.data_ptr(), rows_ref, cos.data_ptr(), sin.data_ptr(),
                cos.stride(0), code, self._status_ptr, batch.stream)
            if rc:
                self.backend._check(rc)
            return
        work, flag = self._launch_terms(batch)
        rc = self._c_append(self._pool_ref, self._k_ptr[layer], self._v_ptr[layer], batch.table_ref,
                            batch.p_first, batch.p_cu, batch.n, 0, total, k_new.data_ptr(), v_new.data_ptr(),
                            rows_ref, self._status_ptr, work, flag, batch.stream)
        if rc:
            self.backend._check(rc)

    def append_layers(self, batch: _Descriptor, k_all: torch.Tensor, v_all: torch.Tensor) -> None:
        """All layers' appends of a step in one launch: ``k_all`` / ``v_all`` are
        ``[num_layers, total_tokens, kv_heads, head_dim]`` (any layer and token strides, contiguous
        last dimension)."""
        total = self._current(batch).total
        if total == 0:
            return
        shape = k_all.shape
        if shape != v_all.shape or len(shape) != 4 or shape[0] != self.num_layers or shape[1] != total \
                or shape[2] != self.num_kv_heads or shape[3] != self.head_dim:
            raise ValueError(f"new rows must both be {(self.num_layers, total, self.num_kv_heads, self.head_dim)}")
        if k_all.dtype != self.dtype or v_all.dtype != self.dtype or k_all.device != self.device \
                or v_all.device != self.device:
            raise ValueError("new rows must be in the cache dtype on the cache device")
        strides = k_all.stride()
        if strides[3] != 1 or v_all.stride() != strides:
            k_all, v_all = k_all.contiguous(), v_all.contiguous()
            strides = k_all.stride()
        rows_ref = self._rows.get(strides[1:])
        if rows_ref is None:
            rows_ref = self._rows[strides[1:]] = self._rows_ref(0, strides[1], strides[2])
        rc = self.backend.lib.barqkv_append_layers(
            self._pool_ref, self._k_ptr[0], self._v_ptr[0], self.num_layers, self.pools.stride(0), batch.table_ref,
            batch.p_first, batch.p_cu, batch.n, 0, total, k_all.data_ptr(), v_all.data_ptr(), rows_ref, strides[0],
            self._status_ptr, self.backend.take_work(self.device.index, batch.stream), 0, batch.stream)
        if rc:
            self.backend._check(rc)

    def _rows_ref(self, seq_stride: int, tok_stride: int, head_stride: int, packed: int = 1):
        """A cached ctypes reference to a ``barqkv_rows_layout`` (packed unless told otherwise)."""
        layout = _ffi.RowsLayout(seq_stride, tok_stride, head_stride, packed, 0)
        self._keep = getattr(self, "_keep", [])
        self._keep.append(layout)               # byref() does not own the structure
        return ctypes.byref(layout)

    def end_append(self, batch: _Descriptor) -> None:
        self.lengths[batch.slots_np] = batch.after_np

    def append_each_layer(self, batch: _Descriptor, k_layers, v_layers) -> None:
        """Every layer's append of a step from one native call, one launch per layer: ``k_layers[l]`` /
        ``v_layers[l]`` are layer ``l``'s packed rows ``[total_tokens, kv_heads, head_dim]``, separate tensors of
        one shape, dtype and stride pattern (``barqkv_append_each_layer``).  Same result as ``append`` layer by
        layer, without the host's share of every call between the launches; layers whose tensors differ in their
        strides are appended one by one."""
        total = self._current(batch).total
        if total == 0:
            return
        if len(k_layers) != self.num_layers or len(v_layers) != self.num_layers:
            raise ValueError(f"need the rows of all {self.num_layers} layers")
        first = k_layers[0]
        want = (total, self.num_kv_heads, self.head_dim)
        strides = first.stride()
        same = strides[2] == 1
        for k, v in zip(k_layers, v_layers):
            if tuple(k.shape) != want or v.shape != k.shape or k.dtype != self.dtype or v.dtype != self.dtype \
                    or k.device != self.device or v.device != self.device:
                raise ValueError(f"every layer's new rows must be {want} in the cache dtype on the cache device")
            same = same and k.stride() == strides and v.stride() == strides
        if not same:
            for layer in range(self.num_layers):
                self.append(layer, batch, k_layers[layer], v_layers[layer])
            return
        rows_ref = self._rows.get(strides)
        if rows_ref is None:
            rows_ref = self._rows[strides] = self._rows_ref(0, strides[0], strides[1])
        pointers = ctypes.c_void_p * self.num_layers
        k_ptrs = pointers(*[k.data_ptr() for k in k_layers])
        v_ptrs = pointers(*[v.data_ptr() for v in v_layers])
        batch.used_at = self._uploads
        # the first launch waits for whatever precedes it (a launch of this cache that still hands out pages from
        # the first counter pair, say); the chain behind it is the library's
        rc = self.backend.lib.barqkv_append_each_layer(
            self._pool_ref, self._k_ptr[0], self._v_ptr[0], self.num_layers, self.pools.stride(0), batch.table_ref,
            batch.p_first, batch.p_cu, batch.n, 0, total, k_ptrs, v_ptrs, rows_ref, self._status_ptr,
            self._work_base(batch.stream), 0, batch.stream)
        # the launches alternated between the stream's two counter pairs starting with the first: the next launch on
        # this stream takes the pair the last layer did not use
        self.backend._work_turn[(self.device.index, batch.stream)] = self.num_layers & 1
        if rc:
            self.backend._check(rc)

    def append_step(self, slots: Sequence[int], counts: Sequence[int], k_layers, v_layers) -> None:
        """All layers of one step: ``k_layers[l]`` / ``v_layers[l]`` are that layer's packed rows."""
        batch = self.begin_append(slots, counts)
        self.append_each_layer(batch, k_layers, v_layers)
        self.end_append(batch)

    # -- gather -------------------------------------------------------------------
    def begin_gather(self, slots: Sequence[int]) -> _Descriptor:
        return self._begin("gather", slots, None)

    def _output(self, layout: str, total: int, out, n: int = 0):
        """Output buffers, their row addressing and the views holding exactly ``total`` tokens.

        ``out`` may be larger than needed along the token dimension (``[H, cap, D]`` or
        ``[cap, H, D]`` with ``cap >= total``, contiguous): the rows are written at the front and
        the returned views are cut to ``total``.  A fixed-capacity buffer keeps every address and
        stride of the call constant from step to step, which a recorded CUDA graph needs.
        """
        H, D = self.num_kv_heads, self.head_dim
        if layout == "BHSD":
            return self._output_padded(total, out, n)
        if layout not in ("HND", "NHD"):
            raise ValueError("layout must be 'HND', 'NHD' or 'BHSD'")
        if out is None:
            shape = (H, total, D) if layout == "HND" else (total, H, D)
            out = (torch.empty(shape, dtype=self.dtype, device=self.device),
                   torch.empty(shape, dtype=self.dtype, device=self.device))
        k_out, v_out = out
        shape = k_out.shape
        tok_dim = 1 if layout == "HND" else 0
        ok = (len(shape) == 3 and shape[2] == D and shape[1 - tok_dim] == H and shape[tok_dim] >= total
              and v_out.shape == shape and k_out.is_contiguous() and v_out.is_contiguous()
              and k_out.dtype == self.dtype and v_out.dtype == self.dtype
              and k_out.device == self.device and v_out.device == self.device)
        if not ok:
            want = "[H, >=total, D]" if layout == "HND" else "[>=total, H, D]"
            raise ValueError(f"out tensors must be contiguous {want} = H {H}, total {total}, D {D} in the cache "
                             f"dtype on the cache device")
        cap = shape[tok_dim]
        key = (layout, cap)
        rows_ref = self._rows.get(key)
        if rows_ref is None:
            if len(self._rows) > 4096:
                self._rows.clear()
                self._keep = []
            rows_ref = self._rows[key] = (self._rows_ref(0, D, cap * D) if layout == "HND"
                                          else self._rows_ref(0, H * D, D))
        if cap != total:
            views = (k_out[:, :total], v_out[:, :total]) if layout == "HND" else (k_out[:total], v_out[:total])
        else:
            views = (k_out, v_out)
        return k_out, v_out, rows_ref, views

    def _output_padded(self, total: int, out, n: int = 0):
        """``[n, H, S, D]`` batch-major outputs (what Hugging Face attention takes): sequence ``i`` fills
        ``[i, :, :len_i]``; rows beyond a sequence's length are left as they are."""
        H, D = self.num_kv_heads, self.head_dim
        if out is None:
            raise ValueError("layout 'BHSD' needs out tensors [n, H, S, D] (S = longest sequence or more)")
        k_out, v_out = out
        shape = k_out.shape
        ok = (len(shape) == 4 and shape[0] >= n and shape[1] == H and shape[3] == D and v_out.shape == shape
              and k_out.is_contiguous() and v_out.is_contiguous() and k_out.dtype == self.dtype
              and v_out.dtype == self.dtype and k_out.device == self.device and v_out.device == self.device)
        if not ok:
            raise ValueError("out tensors must be contiguous [n, H, S, D] in the cache dtype on the cache device")
        S = shape[2]
        key = ("BHSD", S)
        rows_ref = self._rows.get(key)
        if rows_ref is None:
            rows_ref = self._rows[key] = self._rows_ref(H * S * D, D, S * D, packed=0)
        return k_out, v_out, rows_ref, (k_out, v_out)

    def gather(self, layer: int, batch: _Descriptor, layout: str = "HND",
               out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
               mode: Optional[str] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Materialise the batch's sequences back to back.

        ``layout="HND"``: ``[kv_heads, total_tokens, head_dim]`` (sequence ``i`` is
        ``[:, cu[i]:cu[i+1]]``, each head's rows contiguous: the SDPA operand).
        ``layout="NHD"``: ``[total_tokens, kv_heads, head_dim]`` (the varlen
        flash-attention operand).  ``batch.cu`` holds the offsets.  ``out`` may be a pair of
        larger fixed-capacity buffers (see ``_output``); views of the filled part are returned.
        """
        total = self._current(batch).total
        k_out, v_out, rows_ref, views = self._output(layout, total, out, batch.n)
        if total == 0:
            return views
        if batch.n > _GATHER_MAX_ENTRIES:
            # a launch scans at most 8192 sequences: larger batches go in slices of the same description.
            # Packed outputs: the offsets in ``cu`` are absolute, so every slice writes to its own part.
            # Padded [n, H, S, D] outputs are addressed by the entry's index within the launch, so a
            # slice's output pointers start at its first batch row.
            row_bytes = k_out.stride(0) * self.elem if layout == "BHSD" else 0
            for lo in range(0, batch.n, _GATHER_MAX_ENTRIES):
                count = min(_GATHER_MAX_ENTRIES, batch.n - lo)
                table = _ffi.BlockTable(self.table_dev.data_ptr(), batch.p_slots + 4 * lo, self.max_seqs,
                                        self.max_blocks, 0, 0)
                rc = self._c_gather(self._pool_ref, self._k_ptr[layer], self._v_ptr[layer], ctypes.byref(table),
                                    batch.p_first + 4 * lo, batch.p_cu + 4 * lo, count,
                                    batch.cu[lo + count] - batch.cu[lo], k_out.data_ptr() + lo * row_bytes,
                                    v_out.data_ptr() + lo * row_bytes,
                                    rows_ref, _ffi.MODES[mode or self.gather_mode], self._status_ptr,
                                    self.backend.take_work(self.device.index, batch.stream), batch.stream)
                if rc:
                    self.backend._check(rc)
            return views
        work, flag = self._launch_terms(batch)
        rc = self._c_gather(self._pool_ref, self._k_ptr[layer], self._v_ptr[layer], batch.table_ref,
                            batch.p_first, batch.p_cu, batch.n, total, k_out.data_ptr(), v_out.data_ptr(),
                            rows_ref, _ffi.MODES[mode or self.gather_mode] | flag, self._status_ptr, work,
                            batch.stream)
        if rc:
            self.backend._check(rc)
        return views

    def gather_layers(self, batch: _Descriptor, layout: str = "HND",
                      out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Every layer's ``gather`` of the batch in one launch: ``[num_layers, kv_heads, total_tokens,
        head_dim]`` (``"HND"``) or ``[num_layers, total_tokens, kv_heads, head_dim]`` (``"NHD"``) for K and V.

        For callers that want all layers at once (exporting a cache, re-laying it out for another attention
        backend); the launch's fixed cost is paid once instead of once per layer.  A decode step cannot use
        it: a layer's new rows depend on the layer before.
        """
        if layout not in ("HND", "NHD"):
            raise ValueError("layout must be 'HND' or 'NHD'")
        total, L, H, D = self._current(batch).total, self.num_layers, self.num_kv_heads, self.head_dim
        shape = (L, H, total, D) if layout == "HND" else (L, total, H, D)
        if out is None:
            out = (torch.empty(shape, dtype=self.dtype, device=self.device),
                   torch.empty(shape, dtype=self.dtype, device=self.device))
        k_out, v_out = out
        if tuple(k_out.shape) != shape or v_out.shape != k_out.shape or not k_out.is_contiguous() \
                or not v_out.is_contiguous() or k_out.dtype != self.dtype or v_out.dtype != self.dtype \
                or k_out.device != self.device or v_out.device != self.device:
            raise ValueError(f"out tensors must be contiguous {shape} in the cache dtype on the cache device")
        if total == 0:
            return k_out, v_out
        if batch.n > _GATHER_MAX_ENTRIES:
            for layer in range(L):
                self.gather(layer, batch, layout, out=(k_out[layer], v_out[layer]))
            return k_out, v_out
        key = ("layers", layout, total)
        rows_ref = self._rows.get(key)
        if rows_ref is None:
            if len(self._rows) > 4096:
                self._rows.clear()
                self._keep = []
            rows_ref = self._rows[key] = (self._rows_ref(0, D, total * D) if layout == "HND"
                                          else self._rows_ref(0, H * D, D))
        rc = self.backend.lib.barqkv_gather_layers(
            self._pool_ref, self._k_ptr[0], self._v_ptr[0], L, self.pools.stride(0), batch.table_ref, batch.p_first,
            batch.p_cu, batch.n, total, k_out.data_ptr(), v_out.data_ptr(), rows_ref, k_out.stride(0),
            self._status_ptr, self.backend.take_work(self.device.index, batch.stream), batch.stream)
        if rc:
            self.backend._check(rc)
        return k_out, v_out

    # -- append + gather in one call ------------------------------------------------
    def update(self, layer: int, new: _Descriptor, full: _Descriptor, k_new: torch.Tensor, v_new: torch.Tensor,
               layout: str = "HND", out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
               mode: Optional[str] = None, tokens_hint: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Append this step's rows and return every sequence gathered, new rows included - the
        block-table form of the reference layer's ``update`` (``kv_cache.py:135-142``).

        ``new`` comes from ``begin_append`` (followed by ``end_append``) and ``full`` from a
        ``begin_gather`` of the same slots made after it.  For decode-sized appends this is one
        kernel launch instead of two.
        """
        self._current(new), self._current(full)
        if full.n != new.n or not np.array_equal(full.slots_np, new.slots_np):
            raise ValueError("update: the append and gather descriptions must list the same slots")
        if full.n > _GATHER_MAX_ENTRIES:             # beyond one launch's scan: append, then gather in slices
            self.append(layer, new, k_new, v_new)
            return self.gather(layer, full, layout, out=out, mode=mode)
        total, H, D = full.total, self.num_kv_heads, self.head_dim
        k_out, v_out, out_ref, views = self._output(layout, total, out, full.n)
        if new.total:
            nshape = k_new.shape
            if nshape != v_new.shape or len(nshape) != 3 or nshape[0] != new.total or nshape[1] != H or nshape[2] != D:
                raise ValueError(f"new rows must both be {(new.total, H, D)}")
            if k_new.dtype != self.dtype or v_new.dtype != self.dtype or k_new.device != self.device \
                    or v_new.device != self.device:
                raise ValueError("new rows must be in the cache dtype on the cache device")
            strides = k_new.stride()
            if strides[2] != 1 or v_new.stride() != strides:
                k_new, v_new = k_new.contiguous(), v_new.contiguous()
                strides = k_new.stride()
            new_ref = self._rows.get(strides)
            if new_ref is None:
                new_ref = self._rows[strides] = self._rows_ref(0, strides[0], strides[1])
            k_ptr, v_ptr = k_new.data_ptr(), v_new.data_ptr()
        else:
            new_ref, k_ptr, v_ptr = self._rows_ref(0, H * D, D), None, None
        if total == 0:
            return views
        work, flag = self._launch_terms(full)
        if new.used_at != self._uploads:          # both descriptions must be unchanged since their last use
            flag = 0
        new.used_at = self._uploads
        rc = self._c_update(self._pool_ref, self._k_ptr[layer], self._v_ptr[layer], new.table_ref,
                            new.p_first, new.p_cu, new.n, 0, new.total, k_ptr, v_ptr, new_ref,
                            full.p_cu, tokens_hint or total, k_out.data_ptr(), v_out.data_ptr(), out_ref,
                            _ffi.MODES[mode or self.gather_mode] | flag, self._status_ptr, work, full.p_first,
                            full.stream)
        if rc:
            self.backend._check(rc)
        return views

    def update_layers(self, new: _Descriptor, full: _Descriptor, k_all: torch.Tensor, v_all: torch.Tensor,
                      outs: Sequence[Tuple[torch.Tensor, torch.Tensor]], layout: str = "HND",
                      mode: Optional[str] = None, tokens_hint: Optional[int] = None, one_stream: bool = False) -> None:
        """``update`` of every layer with one native call (``barqkv_update_layers``): ``k_all`` / ``v_all`` are
        ``[num_layers, new_tokens, kv_heads, head_dim]``; layer ``l`` writes its gathered rows to
        ``outs[l % len(outs)]`` (pairs of fixed-capacity buffers as ``update`` takes them).  For callers that
        hold every layer's new rows before the first launch - a recorded decode step.  With an even number of
        distinct output pairs the library runs odd layers on a second stream of its own beside the even ones
        (joined back before the call returns); ``one_stream=True`` keeps every layer on the caller's stream."""
        self._current(new), self._current(full)
        if full.n != new.n or not np.array_equal(full.slots_np, new.slots_np):
            raise ValueError("update_layers: the append and gather descriptions must list the same slots")
        L, H, D = self.num_layers, self.num_kv_heads, self.head_dim
        shape = k_all.shape
        if shape != v_all.shape or len(shape) != 4 or shape[0] != L or shape[1] != new.total or shape[2] != H \
                or shape[3] != D:
            raise ValueError(f"new rows must both be {(L, new.total, H, D)}")
        if k_all.dtype != self.dtype or v_all.dtype != self.dtype or k_all.device != self.device \
                or v_all.device != self.device:
            raise ValueError("new rows must be in the cache dtype on the cache device")
        strides = k_all.stride()
        if strides[3] != 1 or v_all.stride() != strides:
            k_all, v_all = k_all.contiguous(), v_all.contiguous()
            strides = k_all.stride()
        if full.n > _GATHER_MAX_ENTRIES or full.total == 0 or new.total == 0:
            for layer in range(L):
                self.update(layer, new, full, k_all[layer], v_all[layer], layout, out=outs[layer % len(outs)], mode=mode,
                            tokens_hint=tokens_hint)
            return
        new_ref = self._rows.get(strides[1:])
        if new_ref is None:
            new_ref = self._rows[strides[1:]] = self._rows_ref(0, strides[1], strides[2])
        out_ref = None
        k_ptrs, v_ptrs = (ctypes.c_void_p * len(outs))(), (ctypes.c_void_p * len(outs))()
        for i, out in enumerate(outs):
            k_out, v_out, ref, _ = self._output(layout, full.total, out, full.n)
            if out_ref is not None and ref is not out_ref:
                raise ValueError("update_layers: all output pairs must have the same shape")
            out_ref = ref
            k_ptrs[i], v_ptrs[i] = k_out.data_ptr(), v_out.data_ptr()
        rc = self.backend.lib.barqkv_update_layers(
            self._pool_ref, self._k_ptr[0], self._v_ptr[0], L, self.pools.stride(0), new.table_ref, new.p_first, new.p_cu,
            new.n, 0, new.total, k_all.data_ptr(), v_all.data_ptr(), new_ref, strides[0], full.p_cu,
            tokens_hint or full.total, k_ptrs, v_ptrs, len(outs), out_ref,
            _ffi.MODES[mode or self.gather_mode] | (_ffi.FLAG_ONE_STREAM if one_stream else 0),
            self._status_ptr, full.work, full.p_first, full.stream)
        # on one stream the layers alternated between the first two counter pairs starting with the first, so the
        # next launch on this stream takes the pair the last layer did not use (after a call that used the second
        # stream every layer is complete before the next launch starts, and either pair will do)
        self.backend._work_turn[(self.device.index, full.stream)] = (L & 1)
        if rc:
            self.backend._check(rc)

    def gather_each_layer(self, full: _Descriptor, outs: Sequence[Tuple[torch.Tensor, torch.Tensor]], layout: str = "HND",
                          mode: Optional[str] = None, tokens_hint: Optional[int] = None, one_stream: bool = False) -> None:
        """``gather`` of every layer with one native call, one launch per layer (``barqkv_update_layers`` with
        nothing to append): layer ``l`` writes to ``outs[l % len(outs)]``.  The launches are chained and, with an
        even number of distinct output pairs, neighbouring layers run side by side on two streams, as in
        ``update_layers``; work queued on the caller's stream afterwards sees every layer done."""
        self._current(full)
        L = self.num_layers
        if full.n > _GATHER_MAX_ENTRIES or full.total == 0:
            for layer in range(L):
                self.gather(layer, full, layout, out=outs[layer % len(outs)], mode=mode)
            return
        out_ref = None
        k_ptrs, v_ptrs = (ctypes.c_void_p * len(outs))(), (ctypes.c_void_p * len(outs))()
        for i, out in enumerate(outs):
            k_out, v_out, ref, _ = self._output(layout, full.total, out, full.n)
            if out_ref is not None and ref is not out_ref:
                raise ValueError("gather_each_layer: all output pairs must have the same shape")
            out_ref = ref
            k_ptrs[i], v_ptrs[i] = k_out.data_ptr(), v_out.data_ptr()
        rc = self.backend.lib.barqkv_update_layers(
            self._pool_ref, self._k_ptr[0], self._v_ptr[0], L, self.pools.stride(0), full.table_ref, full.p_first, None,
            full.n, 0, 0, None, None, None, 0, full.p_cu, tokens_hint or full.total, k_ptrs, v_ptrs, len(outs), out_ref,
            _ffi.MODES[mode or self.gather_mode] | (_ffi.FLAG_ONE_STREAM if one_stream else 0),
            self._status_ptr, full.work, full.p_first, full.stream)
        self.backend._work_turn[(self.device.index, full.stream)] = (L & 1)
        if rc:
            self.backend._check(rc)

    # -- attention straight from the pages (decode) ---------------------------------------
    def decode_attention(self, layer: int, full: _Descriptor, q: torch.Tensor, scale: Optional[float] = None,
                         out: Optional[torch.Tensor] = None, new_rows: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                         max_len: Optional[int] = None, total_len: Optional[int] = None) -> torch.Tensor:
        """``softmax(q k^T * scale) v`` for one query token per sequence, reading K/V from the pages.

        ``full`` is a ``begin_gather`` description (lengths include the token appended this step);
        ``q`` is ``[n, num_q_heads, head_dim]`` in the cache dtype, ``num_q_heads`` a multiple (<= 8x) of
        the KV heads on this device.  Returns ``[n, num_q_heads, head_dim]``.  No gather is involved.

        ``new_rows=(k_new, v_new)``, each ``[n, kv_heads, head_dim]``: the step's token has NOT been appended
        yet (its page is reserved, the lengths already count it); the same launch stores the rows into the
        pages and attends them - a decode layer in one call (``decode_update``).  ``max_len`` /
        ``total_len`` override the description's longest length and sum of lengths (they fix the launch
        shape and the workspace size; a recorded CUDA graph passes bounds that hold for all its replays).
        """
        self._current(full)
        if q.dim() != 3 or q.shape[0] != full.n or q.shape[2] != self.head_dim or q.stride(2) != 1:
            raise ValueError(f"q must be [{full.n}, num_q_heads, {self.head_dim}] with a contiguous last dimension")
        if q.dtype != self.dtype or q.device != self.device or self.dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("q must be bf16 or fp16, in the cache dtype, on the cache device")
        if out is None:
            out = torch.empty_like(q, memory_format=torch.contiguous_format)
        elif out.shape != q.shape or out.dtype != q.dtype or out.device != q.device or out.stride(2) != 1:
            raise ValueError("out must match q")
        if full.n == 0:
            return out
        if max_len is None:
            max_len = full.max_first
        if total_len is None:
            total_len = full.total          # the sum of the lengths: sizes the splits for small batches
        need = int(self.backend.lib.barqkv_paged_decode_workspace_bytes(full.n, self.num_kv_heads, max_len, total_len,
                                                                        self.page_size))
        if need > self._attn_ws_bytes:
            # allocated on the stream the kernels will run on (the description's), so that the workspace it
            # replaces is not reused under a kernel that still runs there
            with torch.cuda.stream(torch.cuda.ExternalStream(full.stream, device=self.device)):
                self._attn_ws = torch.empty(need, dtype=torch.uint8, device=self.device)
            self._attn_ws_bytes = need
        ws_ptr = self._attn_ws.data_ptr() if need else None
        if scale is None:
            scale = self.head_dim ** -0.5
        is_bf16 = 1 if self.dtype == torch.bfloat16 else 0
        lib = self.backend.lib
        if new_rows is None:
            rc = lib.barqkv_paged_decode_attention(
                self._pool_ref, self._k_ptr[layer], self._v_ptr[layer], full.table_ref, full.p_first, full.n,
                q.data_ptr(), q.stride(0), q.stride(1), out.data_ptr(), out.stride(0), out.stride(1), q.shape[1],
                float(scale), is_bf16, max_len, total_len, ws_ptr, need, self._status_ptr, full.stream)
        else:
            k_new, v_new = new_rows
            want = (full.n, self.num_kv_heads, self.head_dim)
            if tuple(k_new.shape) != want or v_new.shape != k_new.shape or k_new.dtype != self.dtype \
                    or v_new.dtype != self.dtype or k_new.device != self.device or v_new.device != self.device:
                raise ValueError(f"new rows must both be {want} in the cache dtype on the cache device")
            if k_new.stride(2) != 1 or v_new.stride() != k_new.stride():
                k_new, v_new = k_new.contiguous(), v_new.contiguous()
            flag = _ffi.FLAG_DESC_STABLE if full.used_at == self._uploads else 0
            full.used_at = self._uploads
            rc = lib.barqkv_paged_decode_update(
                self._pool_ref, self._k_ptr[layer], self._v_ptr[layer], full.table_ref, full.p_first, full.n,
                k_new.data_ptr(), v_new.data_ptr(), k_new.stride(0), k_new.stride(1),
                q.data_ptr(), q.stride(0), q.stride(1), out.data_ptr(), out.stride(0), out.stride(1), q.shape[1],
                float(scale), is_bf16, max_len, total_len, ws_ptr, need, flag, self._status_ptr, full.stream)
        if rc:
            self.backend._check(rc)
        return out

    def decode_update(self, layer: int, full: _Descriptor, k_new: torch.Tensor, v_new: torch.Tensor, q: torch.Tensor,
                      scale: Optional[float] = None, out: Optional[torch.Tensor] = None, **bounds) -> torch.Tensor:
        """A decode layer in one call: store the step's K/V rows into the pages and attend over the pages,
        new token included (``barqkv_paged_decode_update``).  Call ``begin_append`` / ``end_append`` /
        ``begin_gather`` for the step first, as for ``update``; skip the layer's ``append``."""
        return self.decode_attention(layer, full, q, scale=scale, out=out, new_rows=(k_new, v_new), **bounds)

    def gather_sequence(self, layer: int, seq_id, layout: str = "HND") -> Tuple[torch.Tensor, torch.Tensor]:
        """One sequence as contiguous ``[H, len, D]`` (or ``[len, H, D]``)."""
        return self.gather(layer, self.begin_gather([self.slot(seq_id)]), layout)

    # -- inspection ---------------------------------------------------------------
    def logical_page(self, layer: int, seq_id, j: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """``[kv_heads, page_size, head_dim]`` views of logical page ``j`` of a sequence."""
        page = self.pages_of[self.slot(seq_id)][j]
        return self.pools[layer, 0, :, page], self.pools[layer, 1, :, page]

    def check_device_status(self) -> None:
        """Synchronise and raise if any kernel guard fired since the last check."""
        self.backend.raise_on_status(self.device)

    def stats(self) -> PoolStats:
        per_page = self.num_layers * 2 * self.num_kv_heads * self.page_size * self.head_dim * self.elem
        a = self.allocator
        return PoolStats(a.num_pages, a.pages_resident, a.pages_peak, per_page, a.pages_resident * per_page,
                         a.pages_peak * per_page, len(self._slot_of))


class DecodeStepGraph:
    """One decode step of a fixed batch recorded into a CUDA graph and replayed.

    A decode step is, for every layer, ``update`` of the same slots with one new token each: append
    the token's K/V rows and gather every sequence for attention.  From step to step only the
    contents of small device buffers change (start positions, lengths, offsets, block-table rows, the
    new rows themselves); every address, stride and launch shape stays the same once the outputs are
    fixed-capacity buffers.  So the per-layer launches are recorded once and replayed with one graph
    launch per step, which removes the host's per-call cost and the gaps between the kernels - the
    difference between 47 us and 31 us per layer when a GPU holds a single KV head.

    Usage: fill ``k_in`` / ``v_in`` (``[layers, batch, kv_heads, head_dim]``) with the step's new rows
    on ``stream`` (or any stream ordered before it), call ``step()``, then read ``outputs(layer)``
    - views ``[kv_heads, total, head_dim]`` into two alternating buffer pairs (a layer's output is
    overwritten by the layer after next).  ``step()`` runs eagerly until ``record()`` has been called
    (after at least one eager step); from then on it replays the graph.
    """

    def __init__(self, cache: BlockTableKVCache, slots: Sequence[int], capacity_tokens: int,
                 mode: Optional[str] = None, what: str = "update", q_heads: int = 0, max_len: int = 0,
                 one_stream: bool = False):
        """``what``: ``"update"`` (append + gather per layer, the default), ``"append"`` (the append alone, one
        launch per layer), ``"append_layers"`` (the append alone, one launch for all layers) or ``"attention"``
        (append fused into attention over the pages, one call per layer, no gather: fill ``q_in``
        ``[batch, q_heads, head_dim]``, read ``attn_out``; ``max_len`` bounds the longest sequence over all
        replays and ``capacity_tokens`` the sum of the lengths).  Only ``"update"`` needs output buffers."""
        if what not in ("update", "append", "append_layers", "attention"):
            raise ValueError("what must be 'update', 'append', 'append_layers' or 'attention'")
        # "update" only: keep every layer's launch on one stream (see ``update_layers``); takes effect at the
        # next eager step or ``record()``
        self.one_stream = one_stream
        self.cache, self.slots, self.mode, self.what = cache, list(slots), mode, what
        c = cache
        B = len(self.slots)
        self.capacity = int(capacity_tokens)
        self.stream = torch.cuda.Stream(c.device)
        self.k_in = torch.zeros(c.num_layers, B, c.num_kv_heads, c.head_dim, dtype=c.dtype, device=c.device)
        self.v_in = torch.zeros_like(self.k_in)
        self._k_rows, self._v_rows = self.k_in.unbind(0), self.v_in.unbind(0)
        self.bufs = [(torch.empty(c.num_kv_heads, self.capacity, c.head_dim, dtype=c.dtype, device=c.device),
                      torch.empty(c.num_kv_heads, self.capacity, c.head_dim, dtype=c.dtype, device=c.device))
                     for _ in range(2)] if what == "update" else []
        self.q_in = self.attn_out = None
        self.max_len = int(max_len)
        if what == "attention":
            if q_heads <= 0 or self.max_len <= 0 or self.capacity <= 0:
                raise ValueError("what='attention' needs q_heads, max_len and capacity_tokens")
            self.q_in = torch.zeros(B, q_heads, c.head_dim, dtype=c.dtype, device=c.device)
            self.attn_out = torch.zeros_like(self.q_in)
        self.total = 0
        self.steps = 0
        self.launches_per_replay = 0
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        # Both descriptions of a step live at the start of the cache's append step buffer, at fixed addresses:
        # [slots(n) | start(n) | cu_new(n+1) | lengths_after(n) | cu_out(n+1)], rewritten by one upload per step.
        n = B
        self._slots_np = np.asarray(self.slots, dtype=np.int64)
        self._slots32 = _i32(self.slots)
        self._ones32 = np.ones(n, dtype=np.int32)
        self._desc = c._step_dev[0]
        self._table = _ffi.BlockTable(c.table_dev.data_ptr(), self._desc.data_ptr(), c.max_seqs, c.max_blocks, 0, 0)
        base = self._desc.data_ptr()
        ones_cu = list(range(n + 1))
        with torch.cuda.stream(self.stream):
            work = c.backend.work_words(c.device).data_ptr()
        ref = ctypes.byref(self._table)
        self._new = _Descriptor(n, self._desc, n, [0] * n, ones_cu, self.slots, ref, self.stream.cuda_stream, 0)
        self._full = _Descriptor(n, self._desc, 0, [0] * n, [0] * (n + 1), self.slots, ref, self.stream.cuda_stream, work)
        self._new.slots_np = self._full.slots_np = self._slots_np
        self._full.p_first = base + 4 * (3 * n + 1)
        self._full.p_cu = base + 4 * (4 * n + 1)

    def set_slots(self, slots: Sequence[int]) -> None:
        """Continue with other sequences in the batch's rows (continuous batching: a finished sequence's row is
        taken by its replacement).  The recorded launches read the slots from the step's description on the
        device, so the graph stays valid as long as the batch size does; a different size needs another graph
        (``DecodeGraphs`` keeps one per size)."""
        slots = list(slots)
        if len(slots) != len(self.slots):
            raise ValueError(f"this graph was recorded for {len(self.slots)} sequences, not {len(slots)}")
        self.slots = slots
        self._slots_np = np.asarray(slots, dtype=np.int64)
        self._slots32 = _i32(slots)
        self._new.slots_np = self._full.slots_np = self._slots_np
        self._new._slots = self._full._slots = slots

    def _launch_layers(self) -> None:
        c = self.cache
        if self.what == "append":
            for layer in range(c.num_layers):
                c.append(layer, self._new, self._k_rows[layer], self._v_rows[layer])
            return
        if self.what == "append_layers":
            c.append_layers(self._new, self.k_in, self.v_in)
            return
        if self.what == "attention":
            # the launch shape and the workspace come from the bounds, so every replay fits the recording
            self._full.n = len(self.slots)
            for layer in range(c.num_layers):
                c.decode_update(layer, self._full, self._k_rows[layer], self._v_rows[layer], self.q_in, out=self.attn_out,
                                max_len=self.max_len, total_len=self.capacity)
            return
        # one native call issues every layer's launch; from the second layer on each is a programmatic
        # dependent of the one before (its prologue overlaps that layer's tail)
        self.cache.update_layers(self._new, self._full, self.k_in, self.v_in, self.bufs, "HND", mode=self.mode,
                                 tokens_hint=self.capacity, one_stream=self.one_stream)

    def _describe_step(self) -> int:
        """Host side of a step: pages for the new tokens, new lengths, one upload of both descriptions
        (one native call: ``barqkv_host_begin`` with the decode-step layout)."""
        c, n = self.cache, len(self.slots)
        info = c._info
        rc = c._c_begin(c._host, 0, self._slots32.ctypes.data, self._ones32.ctypes.data, n, 1, self.stream.cuda_stream, info)
        if rc:
            c._raise_host(rc)
        total = int(info[0])
        if total > self.capacity and self.what in ("update", "attention"):
            raise ValueError(f"decode graph capacity {self.capacity} tokens exceeded by {total}")
        if self.what == "attention" and int(info[1]) + 1 > self.max_len:
            raise ValueError(f"decode graph max_len {self.max_len} exceeded by a sequence of {int(info[1]) + 1} tokens")
        c.lengths[self._slots_np] += 1
        c._uploads += 1
        # any description made by begin_append meanwhile now points at this step's words
        c._desc_turn["append"] = c._desc_turn.get("append", 0) + 1
        self._full.total = total
        return total

    def step(self) -> int:
        """Append one token per sequence in every layer and gather; returns the total tokens gathered."""
        c = self.cache
        caller = torch.cuda.current_stream(c.device)
        self.stream.wait_stream(caller)
        with torch.cuda.stream(self.stream):
            total = self._describe_step()
            if self.graph is not None:
                # the recorded launches read the descriptions uploaded just above: same buffer, new contents
                self.graph.replay()
            else:
                self._launch_layers()                         # eager; the first one also sets kernel attributes
            self.total = total
        self.steps += 1
        caller.wait_stream(self.stream)
        return self.total

    def record(self) -> None:
        """Record the per-layer launches into a graph.  Recording does not execute them: call it
        between steps, after at least one eager ``step()``; the next ``step()`` replays."""
        c = self.cache
        if self.steps == 0:
            raise RuntimeError("run one eager step() before record(): the first launch sets kernel attributes")
        gc.collect()                                     # finalisers of dead caches run now, not inside the recording
        _destroy_pending()
        torch.cuda.synchronize(c.device)
        self._new.used_at = self._full.used_at = -1      # the first recorded launch waits for whatever precedes a replay
        with torch.cuda.stream(self.stream):
            graph = torch.cuda.CUDAGraph()
            counted = c.backend.launches
            with torch.cuda.graph(graph, stream=self.stream):
                self._launch_layers()
            self.launches_per_replay = c.backend.launches - counted     # kernel nodes in the graph
        self.graph = graph

    def outputs(self, layer: int) -> Tuple[torch.Tensor, torch.Tensor]:
        k, v = self.bufs[layer & 1]
        return k[:, :self.total], v[:, :self.total]


class DecodeGraphs:
    """Decode steps of a batch whose membership and size change (continuous batching): one recorded
    ``DecodeStepGraph`` per batch size, made and recorded the first time that size shows up (one eager step,
    then the recording), replayed from then on with whatever slots the step names."""

    def __init__(self, cache: BlockTableKVCache, capacity_tokens: int, **graph_options):
        self.cache, self.capacity, self.options = cache, int(capacity_tokens), graph_options
        self.graphs: Dict[int, DecodeStepGraph] = {}

    def graph_for(self, slots: Sequence[int]) -> DecodeStepGraph:
        graph = self.graphs.get(len(slots))
        if graph is None:
            graph = self.graphs[len(slots)] = DecodeStepGraph(self.cache, slots, self.capacity, **self.options)
        else:
            graph.set_slots(slots)
        return graph

    def step(self, slots: Sequence[int]) -> DecodeStepGraph:
        """One decode step for ``slots``; returns the graph that ran it (its ``k_in`` / ``v_in`` / ``q_in`` must hold
        the step's inputs before the call: fill them through ``graph_for(slots)``)."""
        graph = self.graph_for(slots)
        graph.step()
        if graph.graph is None and graph.steps >= 1:
            graph.record()
        return graph
