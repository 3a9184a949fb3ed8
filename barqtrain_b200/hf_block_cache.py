"""The block-table cache under Hugging Face ``generate()``.

``BarqBlockTableCache`` is a ``transformers`` ``Cache`` like the reference's ``BarqPagedKVCache``
(``python/barqtrain/kv_cache.py:197-223``), but all layers share one ``BlockTableKVCache``: pages come
from a pool, a batch row is a block-table row, and ``update`` is one fused append + gather launch per
layer that returns contiguous ``[batch, kv_heads, length, head_dim]`` K/V.

With ``attention_from_pages=True`` and the attention function of this module selected
(``use_paged_attention(model)``), single-token decode steps skip the gather altogether: ``update`` hands
the attention function a tag carrying the new rows, and the attention function stores them and reads K/V
from the pages in one call (``BlockTableKVCache.decode_update``).  Prefill and multi-token steps keep using the gathered tensors
with the stock SDPA path.  From-pages decoding attends every cached token of a row, so it is for batches
without padding: a decode step whose attention mask hides any position is refused with an error.
"""

from __future__ import annotations

from typing import Any, Optional, Tuple

import torch

from .block_table import BlockTableKVCache
from .kv_cache import _decoder_config

try:
    from transformers.cache_utils import Cache, CacheLayerMixin
except ImportError:  # pragma: no cover
    Cache = object  # type: ignore[assignment,misc]
    CacheLayerMixin = object  # type: ignore[assignment,misc]

ATTENTION_NAME = "barq_paged"


class BarqBlockTableLayer(CacheLayerMixin):
    """One decoder layer's view of the shared block-table cache."""

    is_sliding = False

    def __init__(self, owner: "BarqBlockTableCache", layer_idx: int):
        super().__init__()
        self.owner = owner
        self.layer_idx = layer_idx
        self.length = 0                      # tokens this layer holds per batch row

    def lazy_initialization(self, key_states: torch.Tensor, value_states: Optional[torch.Tensor] = None) -> None:
        self.owner._ensure_store(key_states)
        self.is_initialized = True

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor,
               cache_kwargs: Optional[dict[str, Any]] = None, *args, **kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
        if key_states.dim() != 4 or key_states.shape != value_states.shape:
            raise ValueError("key_states and value_states must both be [batch, kv_heads, seq, head_dim]")
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        owner = self.owner
        batch, heads, tokens, dim = key_states.shape
        new, full = owner._step(self, batch, tokens)
        store = owner.store

        def rows(t):   # [B, H, T, D] -> packed [B*T, H, D]; a view when the memory is [B, T, H, D] (HF projections)
            return t.transpose(1, 2).reshape(batch * tokens, heads, dim)

        self.length += tokens
        if self.length == tokens and tokens > 1:
            # a prompt entering an empty cache: the gathered result would be the new rows themselves
            store.append(self.layer_idx, new, rows(key_states), rows(value_states))
            return key_states, value_states
        if owner.attention_from_pages and tokens == 1:
            # nothing is launched here: the attention function stores these rows and attends in one kernel
            tag = key_states.new_empty(0)
            tag._barq_paged = (owner, self.layer_idx, rows(key_states), rows(value_states))
            return tag, tag
        # Gathered rows go into one of two cache-owned buffers of the full capacity (consecutive layers
        # alternate), so a decode step allocates nothing; the views returned are cut to the current length.
        k_buf, v_buf = owner._gather_buffers(self.layer_idx, key_states)
        store.update(self.layer_idx, new, full, rows(key_states), rows(value_states), "BHSD",
                     out=(k_buf[:batch], v_buf[:batch]))
        return k_buf[:batch, :, :self.length], v_buf[:batch, :, :self.length]

    def get_seq_length(self) -> int:
        return self.length

    def get_mask_sizes(self, cache_position) -> Tuple[int, int]:
        query_length = cache_position if isinstance(cache_position, int) else cache_position.shape[0]
        return self.length + query_length, 0

    def get_max_cache_shape(self) -> int:
        return self.owner.barqtrain_max_cache_len

    def reset(self) -> None:
        self.length = 0
        self.owner._reset_store()


class BarqBlockTableCache(Cache):
    """Paged K/V for every decoder layer over one page pool and one block table."""

    def __init__(self, config, max_batch_size: int, max_cache_len: int, page_size: int = 16,
                 attention_from_pages: bool = False):
        text_config = _decoder_config(config)
        count = text_config.num_hidden_layers - getattr(text_config, "num_kv_shared_layers", 0)
        super().__init__(layers=[BarqBlockTableLayer(self, i) for i in range(count)])
        self.num_layers = count
        self.barqtrain_max_batch_size = max_batch_size
        self.barqtrain_max_cache_len = max_cache_len
        self.page_size = page_size
        self.attention_from_pages = attention_from_pages
        self.store: Optional[BlockTableKVCache] = None
        self.slots = []
        self._new = self._full = None
        self._step_tokens = 0
        self._bufs = []

    def _ensure_store(self, key_states: torch.Tensor) -> None:
        if self.store is not None:
            return
        batch, heads, _, dim = key_states.shape
        if batch > self.barqtrain_max_batch_size:
            raise ValueError(f"batch_size={batch} exceeds max_batch_size={self.barqtrain_max_batch_size} for paged KV cache")
        blocks = -(-self.barqtrain_max_cache_len // self.page_size)
        self.store = BlockTableKVCache(self.num_layers, heads, dim, page_size=self.page_size,
                                       num_pages=self.barqtrain_max_batch_size * blocks, max_seqs=self.barqtrain_max_batch_size,
                                       max_blocks_per_seq=blocks, dtype=key_states.dtype, device=key_states.device)
        self.slots = [self.store.open(row) for row in range(self.barqtrain_max_batch_size)]

    def _gather_buffers(self, layer_idx: int, like: torch.Tensor):
        if not self._bufs:
            shape = (self.barqtrain_max_batch_size, like.shape[1], self.barqtrain_max_cache_len, like.shape[3])
            self._bufs = [(torch.empty(shape, dtype=like.dtype, device=like.device),
                           torch.empty(shape, dtype=like.dtype, device=like.device)) for _ in range(2)]
        return self._bufs[layer_idx & 1]

    def release_memory(self) -> None:
        """Drop the page pool and the gather buffers now (the cache object sits in reference cycles with its
        layers, so otherwise the memory would wait for the garbage collector)."""
        if self.store is not None:
            self.store.close()
        self.store, self._bufs, self.slots = None, [], []
        self._new = self._full = None

    def _reset_store(self) -> None:
        if self.store is not None and any(int(self.store.lengths[s]) for s in self.slots):
            for row in range(self.barqtrain_max_batch_size):
                self.store.release(row)
            self.slots = [self.store.open(row) for row in range(self.barqtrain_max_batch_size)]
        self._new = self._full = None

    def _step(self, layer: BarqBlockTableLayer, batch: int, tokens: int):
        """The step's descriptions, made when the first layer of a forward pass arrives and shared by the rest."""
        store = self.store
        held = int(store.lengths[self.slots[0]]) if batch else 0
        if layer.length == held:                     # this layer is the first to see the step
            slots = self.slots[:batch]
            self._new = store.begin_append(slots, [tokens] * batch)
            store.end_append(self._new)
            self._full = store.begin_gather(slots)
            self._step_tokens = tokens
        elif layer.length + tokens != held or tokens != self._step_tokens or batch != self._new.n:
            raise RuntimeError("layers of one forward pass must append the same number of tokens in order")
        return self._new, self._full


def paged_attention_forward(module, query, key, value, attention_mask, dropout: float = 0.0,
                            scaling: Optional[float] = None, **kwargs):
    """Attention function for ``transformers``: decode steps tagged by ``BarqBlockTableCache`` read K/V
    from the pages; everything else goes to the stock SDPA function."""
    tag = getattr(key, "_barq_paged", None)
    if tag is None:
        from transformers.integrations.sdpa_attention import sdpa_attention_forward

        return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout, scaling=scaling,
                                      **kwargs)
    owner, layer_idx, k_rows, v_rows = tag
    if attention_mask is not None and layer_idx == 0:
        # The kernel attends every cached token of a row.  transformers hands a mask to a one-token step only
        # when something is hidden (padding), so this read of the mask runs once per step at most, and only then.
        hidden = (~attention_mask).any() if attention_mask.dtype == torch.bool else (attention_mask != 0).any()
        if bool(hidden):
            raise ValueError("attention_from_pages=True cannot serve a padded batch: the attention mask hides cached "
                             "positions, and attention over the pages attends all of them; use the gathered path "
                             "(attention_from_pages=False) or batch sequences of equal length")
    q = query[:, :, 0, :]                                        # [batch, q_heads, head_dim]
    out = owner.store.decode_update(layer_idx, owner._full, k_rows, v_rows, q, scale=scaling)
    return out.unsqueeze(1), None                                # [batch, 1, q_heads, head_dim]


def use_paged_attention(model) -> None:
    """Register ``paged_attention_forward`` with ``transformers`` and select it for ``model``."""
    from transformers import AttentionInterface
    from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS, AttentionMaskInterface

    AttentionInterface.register(ATTENTION_NAME, paged_attention_forward)
    AttentionMaskInterface.register(ATTENTION_NAME, ALL_MASK_ATTENTION_FUNCTIONS["sdpa"])   # masks as for SDPA
    model.config._attn_implementation = ATTENTION_NAME


__all__ = ["BarqBlockTableCache", "paged_attention_forward", "use_paged_attention"]
