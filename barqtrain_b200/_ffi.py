"""Native loading for the paged KV-cache path.

Mirrors the loader contract of the reference (``python/barqtrain/_ffi.py:104-183``):
``load_cuda_backend()`` returns a cached backend object, or ``None`` when the
native library cannot be had; it retries the plain load on every call until it
succeeds, builds at most once per process, and honours ``BARQTRAIN_AUTO_BUILD``
(``0/false/no/off`` disable building, ``_ffi.py:36-38,126``).

What differs: the backend is ``libbarqkv.so`` - a C-ABI library of hand-written
sm_100a kernels opened with ``ctypes`` - not a pybind11/ATen extension, and it
is built by one ``nvcc`` command, not by ``torch.utils.cpp_extension``.  The
returned object keeps the reference's entry point ``paged_kv_append_(key_cache,
value_cache, seq_lens, key_states, value_states)`` (``csrc/src/bindings.cpp:74-75``)
and adds the block-table calls ``append`` and ``gather``.

There is no CPU implementation behind this object: callers that get ``None``
must fail, not fall back.
"""

from __future__ import annotations

import ctypes
import os
import warnings
from typing import Dict, Optional, Tuple

from . import _build

_CUDA_BACKEND: Optional["CudaBackend"] = None
_CUDA_BUILD_FAILED = False

# status bits the kernels may set (include/barqkv.h)
S_BAD_PAGE, S_CAPACITY, S_TIMEOUT, S_BAD_SLOT = 1, 2, 4, 8
MODE_AUTO, MODE_VECTOR, MODE_BULK = 0, 1, 2
MODES = {"auto": MODE_AUTO, "vector": MODE_VECTOR, "bulk": MODE_BULK}
FLAG_DESC_STABLE = 0x100
FLAG_ONE_STREAM = 0x200       # barqkv_update_layers: no second stream

_i32, _i64, _ptr = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p


class PoolLayout(ctypes.Structure):
    """``barqkv_pool_layout``"""

    _fields_ = [("num_heads", _i32), ("head_dim", _i32), ("page_size", _i32), ("elem_bytes", _i32),
                ("num_pages", _i32), ("reserved", _i32), ("head_stride", _i64), ("page_stride", _i64)]


class BlockTable(ctypes.Structure):
    """``barqkv_block_table``"""

    _fields_ = [("table", _ptr), ("slots", _ptr), ("table_rows", _i32), ("table_stride", _i32),
                ("implicit_pages_per_slot", _i32), ("reserved", _i32)]


class RowsLayout(ctypes.Structure):
    """``barqkv_rows_layout``"""

    _fields_ = [("seq_stride", _i64), ("tok_stride", _i64), ("head_stride", _i64), ("packed", _i32), ("reserved", _i32)]


EXPORTS = ("barqkv_version", "barqkv_last_error", "barqkv_sm_count", "barqkv_launch_count",
           "barqkv_append", "barqkv_append_layers", "barqkv_append_each_layer", "barqkv_append_rope", "barqkv_upload",
           "barqkv_max_length", "barqkv_table_scatter", "barqkv_copy_pages", "barqkv_append_legacy",
           "barqkv_gather", "barqkv_gather_layers", "barqkv_update", "barqkv_paged_decode_attention",
           "barqkv_paged_decode_workspace_bytes", "barqkv_update_layers", "barqkv_gather_wait_selftest",
           "barqkv_gather_noalloc", "barqkv_host_create", "barqkv_host_destroy", "barqkv_host_take", "barqkv_host_share",
           "barqkv_host_give_back", "barqkv_host_holders", "barqkv_host_stats", "barqkv_host_free_list",
           "barqkv_host_reserve", "barqkv_host_set_pages", "barqkv_host_release", "barqkv_host_pending_changes",
           "barqkv_host_attach", "barqkv_host_begin", "barqkv_paged_decode_update")
# experiment knobs: only a library built with -DBARQKV_TUNING exports barqkv_set_tuning (include/barqkv_experimental.h)
KNOBS = {"stages": 1, "ctas": 2, "vctas": 3, "interleave": 4, "group": 5, "static": 6, "pdl": 7, "fixed": 8, "tensor_store": 9,
         "attn_promotion": 10, "attn_split": 11, "append_bulk": 12, "attn_wide": 13, "layer_overlap": 14, "attn_page_box": 15, "attn_compact": 16, "attn_probe": 17, "zero_ahead": 18}
STATIC_WORK_SLOTS = 32


def _env_enabled(name: str, default: str = "1") -> bool:
    value = os.environ.get(name, default).strip().lower()
    return value not in {"0", "false", "no", "off"}


def _detect_cuda_home() -> Optional[str]:
    return _build.detect_cuda_home()


def _open_library() -> ctypes.CDLL:
    """Open the prebuilt library; raises ``OSError`` when it is not there.  ``BARQKV_TUNING_LIB=1``
    opens the experiment build (with ``barqkv_set_tuning``) instead, for parameter sweeps."""
    path = _build.TUNING_LIBRARY if _env_enabled("BARQKV_TUNING_LIB", "0") else _build.LIBRARY
    if not path.exists():
        raise OSError(f"{path} has not been built")
    return ctypes.CDLL(str(path))


class BarqKVError(RuntimeError):
    """A native call returned a non-zero code."""


class CudaBackend:
    """ctypes binding of ``libbarqkv.so`` plus tensor-level convenience calls."""

    __name__ = "barqkv"

    def __init__(self, lib: ctypes.CDLL):
        self.lib = lib
        lib.barqkv_version.restype = _i32
        lib.barqkv_last_error.restype = ctypes.c_char_p
        lib.barqkv_sm_count.restype = _i32
        self.tunable = hasattr(lib, "barqkv_set_tuning")
        if self.tunable:
            lib.barqkv_set_tuning.restype = _i32
            lib.barqkv_set_tuning.argtypes = [_i32, _i32]
        P = ctypes.POINTER
        lib.barqkv_append.restype = _i32
        lib.barqkv_append.argtypes = [P(PoolLayout), _ptr, _ptr, P(BlockTable), _ptr, _ptr, _i32, _i32, _i32,
                                      _ptr, _ptr, P(RowsLayout), _ptr, _ptr, _i32, _ptr]
        lib.barqkv_append_legacy.restype = _i32
        lib.barqkv_append_legacy.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, P(RowsLayout),
                                             _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _ptr, _ptr, _ptr]
        lib.barqkv_gather.restype = _i32
        lib.barqkv_gather.argtypes = [P(PoolLayout), _ptr, _ptr, P(BlockTable), _ptr, _ptr, _i32, _i64,
                                      _ptr, _ptr, P(RowsLayout), _i32, _ptr, _ptr, _ptr]
        lib.barqkv_gather_layers.restype = _i32
        lib.barqkv_gather_layers.argtypes = [P(PoolLayout), _ptr, _ptr, _i32, _i64, P(BlockTable), _ptr, _ptr, _i32, _i64,
                                             _ptr, _ptr, P(RowsLayout), _i64, _ptr, _ptr, _ptr]
        lib.barqkv_append_layers.restype = _i32
        lib.barqkv_append_layers.argtypes = [P(PoolLayout), _ptr, _ptr, _i32, _i64, P(BlockTable), _ptr, _ptr,
                                             _i32, _i32, _i32, _ptr, _ptr, P(RowsLayout), _i64, _ptr, _ptr, _i32, _ptr]
        lib.barqkv_append_each_layer.restype = _i32
        lib.barqkv_append_each_layer.argtypes = [P(PoolLayout), _ptr, _ptr, _i32, _i64, P(BlockTable), _ptr, _ptr,
                                                 _i32, _i32, _i32, _ptr, _ptr, P(RowsLayout), _ptr, _ptr, _i32, _ptr]
        lib.barqkv_append_rope.restype = _i32
        lib.barqkv_append_rope.argtypes = [P(PoolLayout), _ptr, _ptr, P(BlockTable), _ptr, _ptr, _i32, _i32, _i32,
                                           _ptr, _ptr, P(RowsLayout), _ptr, _ptr, _i64, _i32, _ptr, _ptr]
        lib.barqkv_upload.restype = _i32
        lib.barqkv_upload.argtypes = [_ptr, _ptr, _i64, _ptr]
        lib.barqkv_table_scatter.restype = _i32
        lib.barqkv_table_scatter.argtypes = [_ptr, _i64, _ptr, _i32, _ptr]
        lib.barqkv_copy_pages.restype = _i32
        lib.barqkv_copy_pages.argtypes = [P(PoolLayout), _ptr, _ptr, _i32, _i64, _ptr, _ptr, _i32, _ptr, _ptr]
        lib.barqkv_paged_decode_workspace_bytes.restype = _i64
        lib.barqkv_paged_decode_workspace_bytes.argtypes = [_i32, _i32, _i64, _i64, _i32]
        lib.barqkv_paged_decode_attention.restype = _i32
        lib.barqkv_paged_decode_attention.argtypes = [P(PoolLayout), _ptr, _ptr, P(BlockTable), _ptr, _i32,
                                                      _ptr, _i64, _i64, _ptr, _i64, _i64, _i32, ctypes.c_float, _i32,
                                                      _i64, _i64, _ptr, _i64, _ptr, _ptr]
        lib.barqkv_paged_decode_update.restype = _i32
        lib.barqkv_paged_decode_update.argtypes = [P(PoolLayout), _ptr, _ptr, P(BlockTable), _ptr, _i32, _ptr, _ptr, _i64,
                                                   _i64, _ptr, _i64, _i64, _ptr, _i64, _i64, _i32, ctypes.c_float, _i32,
                                                   _i64, _i64, _ptr, _i64, _i32, _ptr, _ptr]
        lib.barqkv_update.restype = _i32
        lib.barqkv_update.argtypes = [P(PoolLayout), _ptr, _ptr, P(BlockTable), _ptr, _ptr, _i32, _i32, _i32,
                                      _ptr, _ptr, P(RowsLayout), _ptr, _i64, _ptr, _ptr, P(RowsLayout),
                                      _i32, _ptr, _ptr, _ptr, _ptr]
        lib.barqkv_update_layers.restype = _i32
        lib.barqkv_update_layers.argtypes = [P(PoolLayout), _ptr, _ptr, _i32, _i64, P(BlockTable), _ptr, _ptr, _i32, _i32,
                                             _i32, _ptr, _ptr, P(RowsLayout), _i64, _ptr, _i64, P(_ptr), P(_ptr), _i32,
                                             P(RowsLayout), _i32, _ptr, _ptr, _ptr, _ptr]
        lib.barqkv_gather_wait_selftest.restype = _i32
        lib.barqkv_gather_wait_selftest.argtypes = [P(PoolLayout), _ptr, _ptr, P(BlockTable), _ptr, _ptr, _i32, _ptr, _ptr,
                                                    P(RowsLayout), _i64, _ptr, _ptr]
        lib.barqkv_gather_noalloc.restype = _i32
        lib.barqkv_gather_noalloc.argtypes = [P(PoolLayout), _ptr, _ptr, P(BlockTable), _ptr, _ptr, _i32, _i64,
                                              _ptr, _ptr, P(RowsLayout), _i32, _ptr, _i32, _ptr]
        lib.barqkv_host_create.restype = _ptr
        lib.barqkv_host_create.argtypes = [_i32, _ptr, _i32, _i32, _i32, _ptr, _ptr, _ptr]
        lib.barqkv_host_destroy.restype = None
        lib.barqkv_host_destroy.argtypes = [_ptr]
        for name, args in (("take", [_ptr, _i32, _ptr]), ("share", [_ptr, _ptr, _i32]), ("give_back", [_ptr, _ptr, _i32]),
                           ("holders", [_ptr, _i32]), ("stats", [_ptr, _ptr]), ("free_list", [_ptr, _ptr, _i32]),
                           ("reserve", [_ptr, _i32, _i64]), ("set_pages", [_ptr, _i32, _ptr, _i32]),
                           ("release", [_ptr, _i32]), ("attach", [_ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64]),
                           ("begin", [_ptr, _i32, _ptr, _ptr, _i32, _i32, _ptr, _ptr])):
            fn = getattr(lib, "barqkv_host_" + name)
            fn.restype = _i32
            fn.argtypes = args
        lib.barqkv_host_pending_changes.restype = _i64
        lib.barqkv_host_pending_changes.argtypes = [_ptr]
        self.version = int(lib.barqkv_version())
        lib.barqkv_launch_count.restype = _i64
        self._status: Dict[int, "object"] = {}
        self._tickets: Dict[Tuple[int, int], "object"] = {}
        self._work: Dict[Tuple[int, int], "object"] = {}
        self._work_turn: Dict[Tuple[int, int], int] = {}
        self._legacy_sig, self._legacy_plan, self._legacy_rows = None, None, None
        lib.barqkv_max_length.restype = _i32
        lib.barqkv_max_length.argtypes = [_ptr, _i32, ctypes.POINTER(_i32), _ptr]

    @property
    def launches(self) -> int:
        """Kernels the library has enqueued in this process (counted in C at every launch)."""
        return int(self.lib.barqkv_launch_count())

    # -- plumbing -----------------------------------------------------------
    def _check(self, rc: int) -> None:
        if rc != 0:
            msg = self.lib.barqkv_last_error().decode("utf-8", "replace")
            raise BarqKVError(msg or f"barqkv call failed with code {rc}")

    def last_error(self) -> str:
        return self.lib.barqkv_last_error().decode("utf-8", "replace")

    @staticmethod
    def _stream(device) -> int:
        import torch

        return torch.cuda.current_stream(device).cuda_stream

    def status_word(self, device):
        """Device int32[1] the kernels OR their guard bits into (one per device)."""
        import torch

        index = torch.device(device).index
        if index is None:
            index = torch.cuda.current_device()
        word = self._status.get(index)
        if word is None:
            word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
            self._status[index] = word
        return word

    def read_status(self, device, clear: bool = True) -> int:
        """Synchronises; returns the guard bits set since the last clear."""
        word = self.status_word(device)
        bits = int(word.item())
        if clear and bits:
            word.zero_()
        return bits

    def raise_on_status(self, device) -> None:
        bits = self.read_status(device)
        if bits:
            names = [n for b, n in ((S_BAD_PAGE, "block-table entry out of range"),
                                    (S_CAPACITY, "paged KV cache capacity exceeded, or decode attention given a sum of lengths below the real one"),
                                    (S_TIMEOUT, "bulk-copy wait timed out"),
                                    (S_BAD_SLOT, "sequence slot out of range")) if bits & b]
            raise BarqKVError("device-side guard: " + ", ".join(names))

    def work_words(self, device):
        """Device int32[8] scratch of the bulk kernels' page hand-out (four counter pairs), one per (device, current stream)."""
        import torch

        device = torch.device(device)
        index = device.index if device.index is not None else torch.cuda.current_device()
        key = (index, self._stream(torch.device("cuda", index)))
        words = self._work.get(key)
        if words is None:
            # four counter pairs: single launches alternate between the first two, barqkv_update_layers uses all
            words = torch.zeros(8, dtype=torch.int32, device=torch.device("cuda", index))
            self._work[key] = words
        return words

    def take_work(self, index: int, stream: int) -> int:
        """Address of the counter pair the next bulk launch on ``stream`` should use.  The first four of
        the stream's words hold two pairs handed out in turn, so that two launches adjacent in the stream never share
        one (a launch flagged ``FLAG_DESC_STABLE`` takes its first pages while its predecessor still runs)."""
        import torch

        key = (index, stream)
        words = self._work.get(key)
        if words is None:
            words = torch.zeros(8, dtype=torch.int32, device=torch.device("cuda", index))
            self._work[key] = words
        turn = self._work_turn.get(key, 0)
        self._work_turn[key] = turn ^ 1
        return words.data_ptr() + 8 * turn

    def sm_count(self) -> int:
        return int(self.lib.barqkv_sm_count())

    def set_tuning(self, **knobs: int) -> None:
        """Experiment knobs (process-wide; the ``BARQKV_KNOB_*`` values of ``barqkv_experimental.h``); only a
        library built with ``-DBARQKV_TUNING`` has them (``BARQKV_TUNING_LIB=1`` selects that build).  Gather:
        ``stages``, ``ctas``, ``vctas``, ``interleave``, ``group``, ``static``, ``fixed``, ``pdl``, ``tensor_store``;
        append: ``append_bulk``; decode attention: ``attn_promotion``, ``attn_split``."""
        if not self.tunable:
            raise BarqKVError("this libbarqkv.so has no tuning knobs: build the experiment library "
                              "(barqtrain_b200._build.build_native(tuning=True)) and set BARQKV_TUNING_LIB=1")
        for name, value in knobs.items():
            self._check(self.lib.barqkv_set_tuning(KNOBS[name], int(value)))

    # -- raw calls (pointers as ints) -----------------------------------------
    def append_raw(self, pool: PoolLayout, k_pool: int, v_pool: int, table: BlockTable, seq_start: int,
                   cu_new: Optional[int], n: int, tokens_per_entry: int, total_tokens: int,
                   k_new: int, v_new: int, rows: RowsLayout, status: Optional[int], stream: int,
                   work: Optional[int] = None) -> None:
        self._check(self.lib.barqkv_append(ctypes.byref(pool), k_pool, v_pool, ctypes.byref(table), seq_start, cu_new,
                                           n, tokens_per_entry, total_tokens, k_new, v_new, ctypes.byref(rows),
                                           status, work, 0, stream))

    def gather_noalloc_raw(self, pool: PoolLayout, k_pool: int, v_pool: int, table: BlockTable, seq_lens: int,
                           cu_out: Optional[int], n: int, total_tokens_hint: int, k_out: int, v_out: int,
                           rows: RowsLayout, mode: int, status: Optional[int], work_slot: int, stream: int) -> None:
        """``barqkv_gather_noalloc``: the gather whose hand-out counters live in the library's built-in array
        (``work_slot`` in ``range(STATIC_WORK_SLOTS)``), for callers that cannot allocate device memory."""
        self._check(self.lib.barqkv_gather_noalloc(ctypes.byref(pool), k_pool, v_pool, ctypes.byref(table), seq_lens,
                                                   cu_out, n, total_tokens_hint, k_out, v_out, ctypes.byref(rows), mode,
                                                   status, work_slot, stream))

    def gather_raw(self, pool: PoolLayout, k_pool: int, v_pool: int, table: BlockTable, seq_lens: int,
                   cu_out: Optional[int], n: int, total_tokens_hint: int, k_out: int, v_out: int,
                   rows: RowsLayout, mode: int, status: Optional[int], work: Optional[int], stream: int) -> None:
        self._check(self.lib.barqkv_gather(ctypes.byref(pool), k_pool, v_pool, ctypes.byref(table), seq_lens, cu_out,
                                           n, total_tokens_hint, k_out, v_out, ctypes.byref(rows), mode,
                                           status, work, stream))

    # -- the reference's native entry point -----------------------------------
    def paged_kv_append_(self, key_cache, value_cache, seq_lens, key_states, value_states, *,
                         max_start: Optional[int] = None) -> None:
        """In-place append in the reference layout; same checks and messages as
        ``paged_kv_append_cuda`` (``csrc/kernels/paged_kv_cache.cu:58-128``).

        ``max_start``: the caller's host-side copy of ``seq_lens[:batch].max()``.
        With it the capacity check needs no device read; without it this call
        reads the lengths back like the reference launcher does
        (``paged_kv_cache.cu:93``).  ``key_states``/``value_states`` may be any
        view whose last dimension is contiguous - no copy is made.
        """
        import torch

        # Same tensors, shapes, strides and types as the previous call: its validation still holds.
        stream = torch.cuda.current_stream(key_cache.device).cuda_stream if key_cache.is_cuda else None
        sig = (stream, key_cache.data_ptr(), value_cache.data_ptr(), seq_lens.data_ptr(), key_cache.shape, value_cache.shape,
               key_cache.stride(), value_cache.stride(), key_states.shape, value_states.shape, key_states.stride(),
               value_states.stride(), key_cache.dtype, value_cache.dtype, key_states.dtype, value_states.dtype,
               seq_lens.dtype, seq_lens.shape, seq_lens.stride(), key_states.device, value_states.device)
        plan = self._legacy_plan if sig == self._legacy_sig else None
        if plan is None:
            plan = self._validate_legacy(key_cache, value_cache, seq_lens, key_states, value_states)
            if plan is None:
                return
            if plan[-1]:                       # cacheable: nothing had to be converted or copied
                self._legacy_sig, self._legacy_plan = sig, plan
        batch, max_batch, heads, tokens, head_dim, max_blocks, page_size, elem, rows_ref, device, ticket, status, _ = plan

        lens, k_new, v_new = seq_lens, key_states, value_states
        if not plan[-1]:
            if lens.dtype != torch.int32 or not lens.is_contiguous():
                lens = seq_lens.to(torch.int32).contiguous()
            if k_new.stride(3) != 1 and k_new.size(3) > 1:
                k_new = k_new.contiguous()
            if v_new.stride() != k_new.stride():
                k_new, v_new = k_new.contiguous(), v_new.contiguous()
            rows_ref = ctypes.byref(RowsLayout(k_new.stride(0), k_new.stride(2), k_new.stride(1), 0, 0))
        if max_start is None:
            out = ctypes.c_int32(0)
            self._check(self.lib.barqkv_max_length(lens.data_ptr(), batch, ctypes.byref(out), stream))
            max_start = out.value
        capacity = max_blocks * page_size
        if max_start + tokens > capacity:
            raise RuntimeError(
                f"paged KV cache capacity exceeded: requested {max_start + tokens} tokens, max_cache_len={capacity}")
        if tokens == 0:
            return
        self._check(self.lib.barqkv_append_legacy(
            key_cache.data_ptr(), value_cache.data_ptr(), lens.data_ptr(), k_new.data_ptr(), v_new.data_ptr(),
            rows_ref, batch, max_batch, heads, tokens, head_dim, max_blocks, page_size, elem,
            ticket.data_ptr(), status.data_ptr(), stream))
        if lens is not seq_lens:
            seq_lens[:batch].add_(tokens)

    def _validate_legacy(self, key_cache, value_cache, seq_lens, key_states, value_states):
        """The reference launcher's argument checks, in its order and with its messages
        (``paged_kv_cache.cu:64-90``).  Returns the call's constants, or ``None`` for an empty batch."""
        import torch

        def need(cond, msg):
            if not cond:
                raise RuntimeError(msg)

        need(key_cache.is_cuda, "key_cache must be a CUDA tensor")
        need(value_cache.is_cuda, "value_cache must be a CUDA tensor")
        need(seq_lens.is_cuda, "seq_lens must be a CUDA tensor")
        need(key_states.is_cuda, "key_states must be a CUDA tensor")
        need(value_states.is_cuda, "value_states must be a CUDA tensor")
        need(key_cache.dim() == 5, "key_cache must have shape [batch, kv_heads, max_blocks, page_size, head_dim]")
        need(value_cache.shape == key_cache.shape, "value_cache must match key_cache")
        need(seq_lens.dim() == 1, "seq_lens must have shape [batch]")
        need(key_states.dim() == 4, "key_states must have shape [batch, kv_heads, seq, head_dim]")
        need(value_states.shape == key_states.shape, "value_states must match key_states")
        need(key_cache.dtype == key_states.dtype, "key_cache and key_states must share dtype")
        need(value_cache.dtype == value_states.dtype, "value_cache and value_states must share dtype")
        need(key_cache.is_contiguous(), "key_cache must be contiguous")
        need(value_cache.is_contiguous(), "value_cache must be contiguous")

        batch, heads, tokens, head_dim = key_states.shape
        max_batch, _, max_blocks, page_size, _ = key_cache.shape
        need(batch <= max_batch, "key_cache batch dimension is too small")
        need(heads == key_cache.size(1), "key_cache kv_heads dimension does not match key_states")
        need(head_dim == key_cache.size(4), "key_cache head_dim dimension does not match key_states")
        need(batch <= seq_lens.size(0), "seq_lens batch dimension is too small")
        if batch == 0:
            return None

        device = key_cache.device
        direct = (seq_lens.dtype == torch.int32 and seq_lens.is_contiguous()
                  and (key_states.stride(3) == 1 or key_states.size(3) <= 1)
                  and value_states.stride() == key_states.stride())
        rows_ref = None
        if direct:
            rows = RowsLayout(key_states.stride(0), key_states.stride(2), key_states.stride(1), 0, 0)
            self._legacy_rows = rows                      # keeps the struct behind the reference alive
            rows_ref = ctypes.byref(rows)
        stream = self._stream(device)
        ticket = self._tickets.get((device.index, stream))
        if ticket is None:
            ticket = torch.zeros(1, dtype=torch.int32, device=device)
            self._tickets[(device.index, stream)] = ticket
        status = self.status_word(device)
        return (batch, max_batch, heads, tokens, head_dim, max_blocks, page_size, key_cache.element_size(), rows_ref,
                device, ticket, status, direct)


def _wrap(lib: ctypes.CDLL) -> CudaBackend:
    missing = [name for name in EXPORTS if not hasattr(lib, name)]
    if missing:
        raise OSError("libbarqkv.so lacks symbols: " + ", ".join(missing))
    return CudaBackend(lib)


def load_cuda_backend() -> Optional[CudaBackend]:
    """Load the native backend.

    The reference loader's contract: return the cached backend; otherwise
    (re)build when auto-build is enabled, the library is missing or older than
    its source, and no build has failed in this process; then open the
    library; ``None`` when it cannot be opened.
    """
    global _CUDA_BACKEND, _CUDA_BUILD_FAILED
    if _CUDA_BACKEND is not None:
        return _CUDA_BACKEND

    auto_build = _env_enabled("BARQTRAIN_AUTO_BUILD", "1")
    if auto_build and not _CUDA_BUILD_FAILED and _build.is_stale():
        if not _build.SOURCE.exists():
            warnings.warn(f"BarqTrain CUDA source missing, skipping CUDA build: {_build.SOURCE}")
        elif _detect_cuda_home() is None:
            warnings.warn(
                "BarqTrain CUDA auto-build skipped because a CUDA toolkit was not found. Set CUDA_HOME."
            )
        else:
            try:
                _build.build_native(verbose=_env_enabled("BARQTRAIN_VERBOSE_BUILD", "0"))
            except Exception as exc:  # noqa: BLE001 - same soft-fail contract as the reference loader
                _CUDA_BUILD_FAILED = True
                warnings.warn(f"BarqTrain CUDA auto-build failed: {exc}")

    try:
        _CUDA_BACKEND = _wrap(_open_library())
    except OSError:
        return None
    return _CUDA_BACKEND


def require_cuda_backend() -> CudaBackend:
    """The backend, or a loud failure: this package has no CPU path."""
    backend = load_cuda_backend()
    if backend is None:
        raise RuntimeError(
            "the barqkv CUDA library is not available (build it with `python -c 'import __graft_entry__ as g; "
            "g.build()'` or set BARQTRAIN_AUTO_BUILD=1 with nvcc on PATH); there is no CPU fallback"
        )
    return backend
