"""CPU oracle for the paged KV-cache path.  TEST INFRASTRUCTURE ONLY.

This module restates, on CPU torch tensors, what the reference's paged cache
computes when its native backend is absent.  Nothing in the product imports
it: only the tests, the smoke check and the benchmark's CPU-baseline leg do,
and there only as the checker or as the timed baseline.

Parity status: PINNED.  ``tests/golden/make_golden.py`` runs the unmodified
reference (``python/barqtrain/kv_cache.py``) on seeded inputs and stores its
outputs; ``tests/test_oracle_golden.py`` replays the same inputs through this
file and compares raw bit patterns.  The reference's only known-answer test
for the path (``tests/test_kv_cache.py:24-47``) is replayed there as well.

What is restated, with the reference lines each part follows:

* ``OracleLayer``            - ``BarqPagedKVCacheLayer``  (kv_cache.py:37-194)
* ``OracleLayer.append``     - ``_python_append``         (kv_cache.py:75-91)
  plus the argument checks of ``append``                  (kv_cache.py:93-104)
* ``OracleLayer.current_tensors`` - ``_flatten_pages`` / ``current_tensors``
                                                           (kv_cache.py:120-133)
* ``OraclePagedCache``       - the composition rule for ragged batches and
  explicit block tables: one reference layer per (layer, sequence) with
  ``max_batch_size=1``.  Logical page ``j`` of a sequence is
  ``layer.keys[0, :, j]``; the gathered sequence is ``current_tensors()[.][0]``.
* ``rope_rotate_keys``       - the K half of ``apply_rope_to_qk``  (ops.py:376-428),
  pinned by ``tests/golden/rope_prefill.npz`` (the helper's own output).
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch


class OracleLayer:
    """One fixed-capacity paged cache layer, reference CPU semantics.

    Storage is ``[max_batch, kv_heads, max_blocks, page_size, head_dim]`` for
    keys and for values (kv_cache.py:66-71), zero-filled on first use, with an
    int32 length per batch row.
    """

    def __init__(self, max_batch_size: int, max_cache_len: int, page_size: int = 16):
        self.max_batch_size = int(max_batch_size)
        self.max_cache_len = int(max_cache_len)
        self.page_size = int(page_size)
        # ceil division, as math.ceil(max_cache_len / page_size) at kv_cache.py:47
        self.max_blocks = -(-self.max_cache_len // self.page_size)
        self.keys: Optional[torch.Tensor] = None
        self.values: Optional[torch.Tensor] = None
        self.seq_lens: Optional[torch.Tensor] = None
        self.dtype: Optional[torch.dtype] = None
        self.current_batch_size = 0
        self.is_initialized = False

    # -- allocation (kv_cache.py:53-73) ------------------------------------
    def _allocate(self, key_states: torch.Tensor) -> None:
        if key_states.dim() != 4:
            raise ValueError("key_states must have shape [batch, kv_heads, seq, head_dim]")
        rows, heads, _, dim = key_states.shape
        if rows > self.max_batch_size:
            raise ValueError(
                f"batch_size={rows} exceeds max_batch_size={self.max_batch_size} for paged KV cache"
            )
        shape = (self.max_batch_size, heads, self.max_blocks, self.page_size, dim)
        self.dtype = key_states.dtype
        self.keys = torch.zeros(shape, dtype=self.dtype)
        self.values = torch.zeros(shape, dtype=self.dtype)
        self.seq_lens = torch.zeros(self.max_batch_size, dtype=torch.int32)
        self.current_batch_size = rows
        self.is_initialized = True

    # -- append (kv_cache.py:75-118) ---------------------------------------
    def append(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        if not self.is_initialized:
            self._allocate(key_states)
        if key_states.shape != value_states.shape:
            raise ValueError("key_states and value_states must have identical shapes")
        if key_states.dtype != self.dtype or value_states.dtype != self.dtype:
            raise ValueError("key_states and value_states must stay in the cache dtype")
        if key_states.size(0) > self.max_batch_size:
            raise ValueError("batch size exceeds the configured paged KV cache capacity")

        k = key_states.contiguous()
        v = value_states.contiguous()
        rows, _, new_tokens, _ = k.shape
        ps = self.page_size
        # One sequence at a time; a sequence that does not fit raises AFTER the
        # sequences before it were written (kv_cache.py:77-83).
        for row in range(rows):
            first = int(self.seq_lens[row].item())
            last = first + new_tokens
            if last > self.max_cache_len:
                raise ValueError(
                    f"paged KV cache capacity exceeded: requested {last}, max_cache_len={self.max_cache_len}"
                )
            for t in range(new_tokens):
                block, slot = divmod(first + t, ps)
                self.keys[row, :, block, slot, :] = k[row, :, t, :]
                self.values[row, :, block, slot, :] = v[row, :, t, :]
            self.seq_lens[row] = last
        self.current_batch_size = rows

    # -- "gather": the flattened view (kv_cache.py:120-133) -----------------
    def get_seq_length(self) -> int:
        if not self.is_initialized or self.current_batch_size == 0:
            return 0
        return int(self.seq_lens[: self.current_batch_size].max().item())

    def current_tensors(self) -> Tuple[torch.Tensor, torch.Tensor]:
        longest = self.get_seq_length()
        rows = self.current_batch_size or self.keys.size(0)

        def flat(cache: torch.Tensor) -> torch.Tensor:
            merged = cache[:rows].view(rows, cache.size(1), self.max_blocks * self.page_size, cache.size(-1))
            return merged[..., :longest, :]

        return flat(self.keys), flat(self.values)

    def update(self, key_states, value_states, cache_kwargs=None):
        self.append(key_states, value_states)
        return self.current_tensors()

    # -- bookkeeping operations (kv_cache.py:155-194) -----------------------
    def get_max_cache_shape(self) -> int:
        return self.max_cache_len

    def crop(self, max_length: int) -> None:
        if not self.is_initialized:
            return
        if max_length < 0:
            max_length = self.get_seq_length() - abs(max_length)
        max_length = max(max_length, 0)
        self.seq_lens[: self.current_batch_size].clamp_(max=max_length)

    def batch_select_indices(self, indices: torch.Tensor) -> None:
        if not self.is_initialized or self.current_batch_size == 0:
            return
        n = self.current_batch_size
        self.keys = self.keys[:n].index_select(0, indices)
        self.values = self.values[:n].index_select(0, indices)
        self.seq_lens = self.seq_lens[:n].index_select(0, indices)
        self.current_batch_size = self.keys.size(0)
        self.max_batch_size = self.current_batch_size

    def batch_repeat_interleave(self, repeats: int) -> None:
        if not self.is_initialized or self.current_batch_size == 0:
            return
        n = self.current_batch_size
        self.keys = self.keys[:n].repeat_interleave(repeats, dim=0)
        self.values = self.values[:n].repeat_interleave(repeats, dim=0)
        self.seq_lens = self.seq_lens[:n].repeat_interleave(repeats, dim=0)
        self.current_batch_size = self.keys.size(0)
        self.max_batch_size = self.current_batch_size

    def reset(self) -> None:
        if not self.is_initialized:
            return
        self.keys.zero_()
        self.values.zero_()
        self.seq_lens.zero_()
        self.current_batch_size = 0


class OraclePagedCache:
    """Ragged batches and block tables expressed with reference layers.

    The reference has one implicit block table (page ``j`` of a sequence is its
    ``j``-th block), so a cache with an explicit table is checked on LOGICAL
    content: for every layer ``l`` and sequence ``s`` a private
    ``OracleLayer(max_batch_size=1)`` holds what the reference would hold.
    """

    def __init__(self, num_layers: int, page_size: int):
        self.num_layers = int(num_layers)
        self.page_size = int(page_size)
        self._layers: List[Dict[int, OracleLayer]] = [dict() for _ in range(num_layers)]

    def open(self, seq_id: int, capacity_tokens: int) -> None:
        cap = -(-int(capacity_tokens) // self.page_size) * self.page_size
        for per_layer in self._layers:
            per_layer[seq_id] = OracleLayer(1, cap, self.page_size)

    def release(self, seq_id: int) -> None:
        for per_layer in self._layers:
            per_layer.pop(seq_id, None)

    def append(self, layer: int, seq_id: int, k: torch.Tensor, v: torch.Tensor) -> None:
        """``k``/``v``: ``[kv_heads, new_tokens, head_dim]`` for one sequence."""
        self._layers[layer][seq_id].append(k.unsqueeze(0), v.unsqueeze(0))

    def length(self, layer: int, seq_id: int) -> int:
        return self._layers[layer][seq_id].get_seq_length()

    def gather(self, layer: int, seq_id: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Contiguous ``[kv_heads, len, head_dim]`` keys and values."""
        k, v = self._layers[layer][seq_id].current_tensors()
        return k[0].contiguous(), v[0].contiguous()

    def logical_page(self, layer: int, seq_id: int, j: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """``[kv_heads, page_size, head_dim]`` of logical page ``j`` (zero tail included)."""
        ref = self._layers[layer][seq_id]
        return ref.keys[0, :, j], ref.values[0, :, j]


def bits(t: torch.Tensor) -> torch.Tensor:
    """Reinterpret a floating tensor as same-width integers for bit-exact comparison."""
    width = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()]
    return t.contiguous().view(width)


def rope_rotate_keys(k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding of ``k`` ``[..., T, D]`` with tables ``[T, D/2]``: the reference helper's
    expressions (ops.py:409-427) - real half ``k1*cos - k2*sin``, imaginary half ``k1*sin + k2*cos``,
    every product and sum rounded to the tensor's dtype as torch's CPU kernels round them."""
    half = k.shape[-1] // 2
    k1, k2 = k[..., :half], k[..., half:]
    return torch.cat([k1 * cos - k2 * sin, k1 * sin + k2 * cos], dim=-1)
