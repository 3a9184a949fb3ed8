"""KV-head sharding of the paged cache across the GPUs of one node.

The reference is single-GPU.  The path shards without any exchange: every
(layer, KV head) is an independent copy problem, so rank ``r`` of ``world``
owns a contiguous run of heads of every layer's pools (the tensor-parallel
layout), new K/V rows arrive already split by head, and gathered K/V stay on
the owning GPU.  Block tables, lengths and the free list are small host-side
metadata computed identically on every rank from the same seed or the same
scheduler decisions - replicated, never communicated on the data path.
"""

from __future__ import annotations

import hashlib
from typing import Iterable, Sequence, Tuple


def kv_head_shard(total_heads: int, world: int, rank: int) -> Tuple[int, int]:
    """``(first_head, count)`` owned by ``rank``; ``world`` must divide ``total_heads``."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is not in a world of {world}")
    if total_heads % world:
        raise ValueError(f"{world} GPUs do not divide {total_heads} KV heads")
    count = total_heads // world
    return rank * count, count


def shard_heads(tensor, head_dim_index: int, world: int, rank: int):
    """The slice of ``tensor`` along its head dimension that ``rank`` owns (a view)."""
    first, count = kv_head_shard(tensor.shape[head_dim_index], world, rank)
    return tensor.narrow(head_dim_index, first, count)


def metadata_digest(lengths: Sequence[int], free_order: Iterable[int]) -> str:
    """Fingerprint of the replicated metadata; ranks compare it to prove they agree."""
    h = hashlib.sha256()
    h.update(",".join(str(int(x)) for x in lengths).encode())
    h.update(b"|")
    h.update(",".join(str(int(x)) for x in free_order).encode())
    return h.hexdigest()
