"""barqtrain_b200: BarqTrain's paged KV-cache path (append + gather) on NVIDIA B200.

Public surface mirrors the reference package for this path
(``python/barqtrain/__init__.py:42-48``): the paged-cache classes, the
``create_paged_kv_cache`` factory and the memory snapshot helpers, plus the
block-table cache that generalises the reference's arithmetic paging.
"""

__version__ = "0.1.0"

from .memory import CudaMemorySnapshot, cuda_memory_snapshot, generation_overhead_mb
from .kv_cache import (
    BarqPagedKVCache,
    BarqPagedKVCacheLayer,
    create_paged_kv_cache,
    maybe_prepare_paged_kv_generate_kwargs,
    paged_kv_supported_for_model,
)
from .block_table import (BlockTableKVCache, DecodeGraphs, DecodeStepGraph, PageAllocator, PagePoolExhausted,
                          PoolStats)
from .hf_block_cache import BarqBlockTableCache, use_paged_attention
from ._ffi import load_cuda_backend

__all__ = [
    "BarqBlockTableCache",
    "BarqPagedKVCache",
    "BarqPagedKVCacheLayer",
    "BlockTableKVCache",
    "CudaMemorySnapshot",
    "DecodeGraphs",
    "DecodeStepGraph",
    "PageAllocator",
    "PagePoolExhausted",
    "PoolStats",
    "create_paged_kv_cache",
    "cuda_memory_snapshot",
    "generation_overhead_mb",
    "load_cuda_backend",
    "maybe_prepare_paged_kv_generate_kwargs",
    "paged_kv_supported_for_model",
    "use_paged_attention",
    "__version__",
]
