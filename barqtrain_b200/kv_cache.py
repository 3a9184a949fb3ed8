"""Drop-in for the reference's paged KV-cache API, backed by the sm_100a kernels.

Same classes, methods and argument meaning as ``python/barqtrain/kv_cache.py``
of the reference:

* ``BarqPagedKVCacheLayer``  (kv_cache.py:37-194) - fixed-capacity layer with
  storage ``[max_batch, kv_heads, max_blocks, page_size, head_dim]``
* ``BarqPagedKVCache``       (kv_cache.py:197-223) - one layer per decoder layer
* ``create_paged_kv_cache``  (kv_cache.py:226-240)
* ``maybe_prepare_paged_kv_generate_kwargs`` (kv_cache.py:243-303)
* ``paged_kv_supported_for_model``           (kv_cache.py:306-308)

What is different underneath:

* ``append`` always runs the native kernel.  There is no Python loop to fall
  back to: CPU tensors or a missing library raise.
* New rows are read through their strides, so the transposed ``[B, H, T, D]``
  view Hugging Face attention hands over is not copied first
  (the reference calls ``.contiguous()`` on both, kv_cache.py:112-113).
* Sequence lengths are mirrored on the host, so ``get_seq_length`` and the
  capacity check do not read the device (the reference synchronises in both:
  kv_cache.py:153, paged_kv_cache.cu:93).  The device tensor ``seq_lens`` is
  still advanced by the kernel and stays authoritative for device consumers.
* ``gather_contiguous`` is an addition: it materialises the sequences as
  contiguous tensors with the gather kernel (the reference only offers the
  strided view ``current_tensors``, which is kept unchanged).
"""

from __future__ import annotations

import os
from typing import Any, List, Optional, Tuple

import torch

from . import _ffi

try:  # transformers supplies only the base classes; no arithmetic lives there
    from transformers.cache_utils import Cache, CacheLayerMixin
except ImportError:  # pragma: no cover
    Cache = object  # type: ignore[assignment,misc]
    CacheLayerMixin = object  # type: ignore[assignment,misc]


def _get_cuda_backend():
    return _ffi.load_cuda_backend()


def _env_enabled(name: str, default: str = "1") -> bool:
    return _ffi._env_enabled(name, default)


def _decoder_config(config):
    getter = getattr(config, "get_text_config", None)
    return getter(decoder=True) if callable(getter) else config


def _min_paged_kv_cache_len() -> int:
    return int(os.environ.get("BARQTRAIN_PAGED_KV_MIN_CACHE_LEN", "256"))


class BarqPagedKVCacheLayer(CacheLayerMixin):
    """A fixed-capacity paged KV-cache layer; the append runs on the GPU."""

    is_sliding = False

    def __init__(self, max_batch_size: int, max_cache_len: int, page_size: int = 16):
        super().__init__()
        self.max_batch_size = max_batch_size
        self.max_cache_len = max_cache_len
        self.page_size = page_size
        self.max_blocks = -(-max_cache_len // page_size)
        self.seq_lens: Optional[torch.Tensor] = None
        self.device: Optional[torch.device] = None
        self.dtype: Optional[torch.dtype] = None
        self.current_batch_size = 0
        self._host_lens: List[int] = []

    # -- allocation -----------------------------------------------------------
    def lazy_initialization(self, key_states: torch.Tensor, value_states: Optional[torch.Tensor] = None) -> None:
        if key_states.dim() != 4:
            raise ValueError("key_states must have shape [batch, kv_heads, seq, head_dim]")
        batch, heads, _, head_dim = key_states.shape
        if batch > self.max_batch_size:
            raise ValueError(
                f"batch_size={batch} exceeds max_batch_size={self.max_batch_size} for paged KV cache"
            )
        if not key_states.is_cuda:
            raise RuntimeError("BarqPagedKVCacheLayer needs CUDA tensors: this build has no CPU append")
        self.device = key_states.device
        self.dtype = key_states.dtype
        self.current_batch_size = batch
        shape = (self.max_batch_size, heads, self.max_blocks, self.page_size, head_dim)
        self.keys = torch.zeros(shape, dtype=self.dtype, device=self.device)
        self.values = torch.zeros_like(self.keys)
        self.seq_lens = torch.zeros((self.max_batch_size,), dtype=torch.int32, device=self.device)
        self._host_lens = [0] * self.max_batch_size
        self.is_initialized = True

    # -- append ---------------------------------------------------------------
    def append(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        if key_states.shape != value_states.shape:
            raise ValueError("key_states and value_states must have identical shapes")
        if key_states.device != self.device or value_states.device != self.device:
            raise ValueError("key_states and value_states must stay on the cache device")
        if key_states.dtype != self.dtype or value_states.dtype != self.dtype:
            raise ValueError("key_states and value_states must stay in the cache dtype")
        batch = key_states.size(0)
        if batch > self.max_batch_size:
            raise ValueError("batch size exceeds the configured paged KV cache capacity")

        backend = _ffi.require_cuda_backend()
        longest = max(self._host_lens[:batch], default=0)
        backend.paged_kv_append_(self.keys, self.values, self.seq_lens, key_states, value_states, max_start=longest)
        tokens = key_states.size(2)
        for row in range(batch):
            self._host_lens[row] += tokens
        self.current_batch_size = batch

    # -- read-back ------------------------------------------------------------
    def _flatten_pages(self, cache_tensor: torch.Tensor) -> torch.Tensor:
        rows = self.current_batch_size or cache_tensor.size(0)
        return cache_tensor[:rows].view(rows, cache_tensor.size(1), self.max_blocks * self.page_size,
                                        cache_tensor.size(-1))

    def current_tensors(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Zero-copy ``[B, H, longest, D]`` views, cut at the longest sequence (reference semantics)."""
        longest = self.get_seq_length()
        return (self._flatten_pages(self.keys)[..., :longest, :],
                self._flatten_pages(self.values)[..., :longest, :])

    def gather_contiguous(self, mode: str = "auto") -> Tuple[torch.Tensor, torch.Tensor]:
        """Contiguous ``[B, H, longest, D]`` copies made by the gather kernel.

        Rows at and beyond a sequence's own length are zero (the strided view
        of ``current_tensors`` exposes whatever the pages hold there).
        """
        backend = _ffi.require_cuda_backend()
        rows = self.current_batch_size
        longest = self.get_seq_length()
        heads, head_dim = self.keys.size(1), self.keys.size(4)
        k_out = torch.zeros((rows, heads, longest, head_dim), dtype=self.dtype, device=self.device)
        v_out = torch.zeros_like(k_out)
        if rows == 0 or longest == 0:
            return k_out, v_out
        page_elems = self.page_size * head_dim
        pool = _ffi.PoolLayout(heads, head_dim, self.page_size, self.keys.element_size(),
                               self.keys.size(0) * heads * self.max_blocks, 0,
                               self.max_blocks * page_elems, page_elems)
        table = _ffi.BlockTable(None, None, self.keys.size(0), self.max_blocks, heads * self.max_blocks, 0)
        out_rows = _ffi.RowsLayout(heads * longest * head_dim, head_dim, longest * head_dim, 0, 0)
        backend.gather_raw(pool, self.keys.data_ptr(), self.values.data_ptr(), table, self.seq_lens.data_ptr(), None,
                           rows, sum(self._host_lens[:rows]), k_out.data_ptr(), v_out.data_ptr(), out_rows,
                           _ffi.MODES[mode], backend.status_word(self.device).data_ptr(),
                           backend.work_words(self.device).data_ptr(), backend._stream(self.device))
        return k_out, v_out

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor,
               cache_kwargs: Optional[dict[str, Any]] = None, *args, **kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
        self.append(key_states, value_states)
        return self.current_tensors()

    # -- sizes ------------------------------------------------------------------
    def get_seq_length(self) -> int:
        if not self.is_initialized or self.seq_lens is None or self.current_batch_size == 0:
            return 0
        return max(self._host_lens[: self.current_batch_size])

    def get_mask_sizes(self, cache_position) -> Tuple[int, int]:
        """``(kv_length, kv_offset)``; accepts a position tensor (reference signature,
        kv_cache.py:144-148) or a plain query length (newer ``transformers``)."""
        query_length = cache_position if isinstance(cache_position, int) else cache_position.shape[0]
        return self.get_seq_length() + query_length, 0

    def get_max_cache_shape(self) -> int:
        return self.max_cache_len

    # -- bookkeeping ------------------------------------------------------------
    def crop(self, max_length: int) -> None:
        if not self.is_initialized or self.seq_lens is None:
            return
        if max_length < 0:
            max_length = self.get_seq_length() - abs(max_length)
        max_length = max(max_length, 0)
        rows = self.current_batch_size
        self.seq_lens[:rows].clamp_(max=max_length)
        self._host_lens[:rows] = [min(n, max_length) for n in self._host_lens[:rows]]

    def _take_rows(self, row_ids: List[int], keys: torch.Tensor, values: torch.Tensor, lens: torch.Tensor) -> None:
        self.keys, self.values, self.seq_lens = keys, values, lens
        self._host_lens = [self._host_lens[r] for r in row_ids]
        self.current_batch_size = keys.size(0)
        self.max_batch_size = self.current_batch_size

    def batch_repeat_interleave(self, repeats: int) -> None:
        if not self.is_initialized or self.current_batch_size == 0:
            return
        rows = self.current_batch_size
        self._take_rows([r for r in range(rows) for _ in range(repeats)],
                        self.keys[:rows].repeat_interleave(repeats, dim=0),
                        self.values[:rows].repeat_interleave(repeats, dim=0),
                        self.seq_lens[:rows].repeat_interleave(repeats, dim=0))

    def batch_select_indices(self, indices: torch.Tensor) -> None:
        if not self.is_initialized or self.current_batch_size == 0:
            return
        rows = self.current_batch_size
        on_device = indices.to(self.keys.device)
        self._take_rows([int(i) for i in indices.tolist()],
                        self.keys[:rows].index_select(0, on_device),
                        self.values[:rows].index_select(0, on_device),
                        self.seq_lens[:rows].index_select(0, on_device))

    def reorder_cache(self, beam_idx: torch.LongTensor) -> None:
        self.batch_select_indices(beam_idx)

    def reset(self) -> None:
        if not self.is_initialized:
            return
        self.keys.zero_()
        self.values.zero_()
        self.seq_lens.zero_()
        self._host_lens = [0] * len(self._host_lens)
        self.current_batch_size = 0


class BarqPagedKVCache(Cache):
    """A paged KV cache that preallocates decode storage for each decoder layer."""

    def __init__(self, config, max_batch_size: int, max_cache_len: int, page_size: int = 16):
        text_config = _decoder_config(config)
        count = text_config.num_hidden_layers - getattr(text_config, "num_kv_shared_layers", 0)
        super().__init__(layers=[
            BarqPagedKVCacheLayer(max_batch_size=max_batch_size, max_cache_len=max_cache_len, page_size=page_size)
            for _ in range(count)
        ])
        self.page_size = page_size
        self.barqtrain_max_cache_len = max_cache_len
        self.barqtrain_max_batch_size = max_batch_size


def create_paged_kv_cache(model_or_config, *, max_batch_size: int, max_cache_len: int,
                          page_size: int = 16) -> BarqPagedKVCache:
    """Create a paged KV cache for a model or decoder config."""
    config = getattr(model_or_config, "config", model_or_config)
    return BarqPagedKVCache(config=config, max_batch_size=max_batch_size, max_cache_len=max_cache_len,
                            page_size=page_size)


def _prompt_geometry(args, kwargs):
    """(batch, prompt_length, device) from input_ids / inputs_embeds / attention_mask, or None."""
    candidates = [kwargs.get("input_ids")]
    if candidates[0] is None and args:
        candidates[0] = args[0]
    candidates += [kwargs.get("inputs_embeds"), kwargs.get("attention_mask")]
    for tensor in candidates:
        if tensor is not None:
            batch, length = tensor.shape[:2]
            return batch, length, tensor.device
    return None


def _requested_cache_len(model, kwargs, prompt_length: int) -> Optional[int]:
    generation_config = kwargs.get("generation_config") or getattr(model, "generation_config", None)

    def setting(name):
        value = kwargs.get(name)
        if value is None and generation_config is not None:
            value = getattr(generation_config, name, None)
        return value

    new_tokens = setting("max_new_tokens")
    if new_tokens is not None:
        return prompt_length + int(new_tokens)
    max_length = setting("max_length")
    if max_length is None:
        return None
    return int(max(max_length, prompt_length))


def maybe_prepare_paged_kv_generate_kwargs(model: torch.nn.Module, args, kwargs):
    """Inject a paged KV cache into ``generate()`` kwargs when the native path can run.

    Returns ``(kwargs, used)``.  The gates and their order are the reference's:
    caller already passed a cache; ``BARQTRAIN_ENABLE_PAGED_KV``; the model flag
    ``_barqtrain_paged_kv_supported``; backend loaded; inputs on a CUDA device;
    ``prompt + max_new_tokens`` (or ``max_length``) at least
    ``BARQTRAIN_PAGED_KV_MIN_CACHE_LEN``.  Page size from
    ``BARQTRAIN_PAGED_KV_PAGE_SIZE`` (16).
    """
    if kwargs.get("past_key_values") is not None:
        return kwargs, False
    if not _env_enabled("BARQTRAIN_ENABLE_PAGED_KV", "1"):
        return kwargs, False
    if not getattr(model, "_barqtrain_paged_kv_supported", False):
        return kwargs, False
    if _get_cuda_backend() is None:
        return kwargs, False

    geometry = _prompt_geometry(args, kwargs)
    if geometry is None:
        return kwargs, False
    batch, prompt_length, device = geometry
    if device.type != "cuda":
        return kwargs, False

    max_cache_len = _requested_cache_len(model, kwargs, prompt_length)
    if max_cache_len is None or max_cache_len < _min_paged_kv_cache_len():
        return kwargs, False

    cache = create_paged_kv_cache(
        model,
        max_batch_size=batch,
        max_cache_len=max_cache_len,
        page_size=int(os.environ.get("BARQTRAIN_PAGED_KV_PAGE_SIZE", "16")),
    )
    return {**kwargs, "past_key_values": cache, "use_cache": True}, True


def paged_kv_supported_for_model(model: torch.nn.Module) -> bool:
    """True when paged KV-cache injection can run for this model."""
    return torch.cuda.is_available() and _get_cuda_backend() is not None and hasattr(model, "generate")


__all__ = [
    "BarqPagedKVCache",
    "BarqPagedKVCacheLayer",
    "create_paged_kv_cache",
    "maybe_prepare_paged_kv_generate_kwargs",
    "paged_kv_supported_for_model",
]
