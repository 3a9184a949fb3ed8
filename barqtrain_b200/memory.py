"""Resident / peak accounting for generation benchmarks.

Same names and meaning as the reference's helpers
(``python/barqtrain/memory.py:13-46``): a snapshot of the CUDA allocator in MiB
and the overhead a generation run added on top of the resident model.  The
block-table cache additionally reports page-pool occupancy through
``BlockTableKVCache.stats()``; ``pool_overhead_mb`` expresses that in the same
unit.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

_MIB = float(1 << 20)


@dataclass(frozen=True)
class CudaMemorySnapshot:
    allocated_mb: float = 0.0
    reserved_mb: float = 0.0
    max_allocated_mb: float = 0.0
    max_reserved_mb: float = 0.0


def cuda_memory_snapshot(reset_peak: bool = False) -> CudaMemorySnapshot:
    """Current CUDA allocator state in MiB; all zeros when no CUDA device is usable."""
    if not torch.cuda.is_available():
        return CudaMemorySnapshot()
    if reset_peak:
        torch.cuda.reset_peak_memory_stats()
    readings = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved(),
                torch.cuda.max_memory_allocated(), torch.cuda.max_memory_reserved())
    return CudaMemorySnapshot(*(r / _MIB for r in readings))


def generation_overhead_mb(resident_snapshot: CudaMemorySnapshot, peak_snapshot: CudaMemorySnapshot) -> float:
    """Peak allocation during generation beyond the resident footprint, never negative."""
    return max(peak_snapshot.max_allocated_mb - resident_snapshot.allocated_mb, 0.0)


def pool_overhead_mb(stats) -> float:
    """Peak page-pool occupancy of a ``BlockTableKVCache`` (its ``stats()``) in MiB."""
    return stats.bytes_peak / _MIB


__all__ = ["CudaMemorySnapshot", "cuda_memory_snapshot", "generation_overhead_mb", "pool_overhead_mb"]
