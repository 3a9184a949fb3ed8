"""Seeded input scenarios shared by the golden-vector generator and the tests.

Every scenario draws on a CPU ``torch.Generator`` in a fixed order (lengths ->
free-list permutation -> K/V per step per layer), so the reference, the oracle
and the CUDA path all see identical bits.  K/V are N(0,1) drawn in fp32 and
cast to the scenario's dtype.
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Dict, List, Tuple

import torch

DTYPES = {"fp32": torch.float32, "fp64": torch.float64, "fp16": torch.float16, "bf16": torch.bfloat16}
_INT_VIEW = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}


def bits(t: torch.Tensor) -> torch.Tensor:
    """Same-width integer view of a tensor (contiguous copy) for bit-exact comparison."""
    return t.detach().cpu().contiguous().view(_INT_VIEW[t.element_size()])


def bits_dev(t: torch.Tensor) -> torch.Tensor:
    """Integer view on the tensor's own device (no host copy), for large comparisons."""
    return t.contiguous().view(_INT_VIEW[t.element_size()])


def digest(*tensors: torch.Tensor) -> str:
    """sha256 over shapes and raw bytes of the given tensors."""
    h = hashlib.sha256()
    for t in tensors:
        b = bits(t)
        h.update(str(tuple(b.shape)).encode())
        h.update(b.numpy().tobytes())
    return h.hexdigest()


def randn(g: torch.Generator, shape, dtype: torch.dtype) -> torch.Tensor:
    return torch.randn(shape, generator=g, dtype=torch.float32).to(dtype)


# --------------------------------------------------------------------------
# Scenario 1: the reference's own known-answer case (tests/test_kv_cache.py:24-47)
# --------------------------------------------------------------------------
def ref_known_answer():
    k0 = torch.arange(24, dtype=torch.float32).view(1, 2, 3, 4)
    v0 = k0 + 100.0
    k1 = torch.arange(16, dtype=torch.float32).view(1, 2, 2, 4) + 1000.0
    v1 = k1 + 100.0
    return dict(max_batch_size=1, max_cache_len=8, page_size=4), [(k0, v0), (k1, v1)]


# --------------------------------------------------------------------------
# Scenario 2: small paged cache, ragged batch, prefill then decode
# (2 layers, 4 KV heads, head_dim 64, fp32, page 16, 64-page pool; prefill 37
#  and 50 tokens; 32 single-token decode steps; gather after every step)
# --------------------------------------------------------------------------
@dataclass
class SmallPagedScenario:
    num_layers: int = 2
    kv_heads: int = 4
    head_dim: int = 64
    dtype: torch.dtype = torch.float32
    page_size: int = 16
    num_pages: int = 64
    prefill: Tuple[int, ...] = (37, 50)
    decode_steps: int = 32
    seed: int = 1235
    free_list: List[int] = field(default_factory=list)
    # steps[i] = list over layers of list over sequences of (k, v) with shape [H, T, D]
    steps: List[List[List[Tuple[torch.Tensor, torch.Tensor]]]] = field(default_factory=list)

    def final_lengths(self) -> Tuple[int, ...]:
        return tuple(p + self.decode_steps for p in self.prefill)


def small_paged(**overrides) -> SmallPagedScenario:
    sc = SmallPagedScenario(**overrides)
    g = torch.Generator().manual_seed(sc.seed)
    sc.free_list = torch.randperm(sc.num_pages, generator=g).tolist()
    H, D = sc.kv_heads, sc.head_dim
    step0 = []
    for _layer in range(sc.num_layers):
        per_seq = []
        for T in sc.prefill:
            per_seq.append((randn(g, (H, T, D), sc.dtype), randn(g, (H, T, D), sc.dtype)))
        step0.append(per_seq)
    sc.steps.append(step0)
    for _step in range(sc.decode_steps):
        one = []
        for _layer in range(sc.num_layers):
            per_seq = []
            for _s in sc.prefill:
                per_seq.append((randn(g, (H, 1, D), sc.dtype), randn(g, (H, 1, D), sc.dtype)))
            one.append(per_seq)
        sc.steps.append(one)
    return sc


# --------------------------------------------------------------------------
# Scenario 3: reference layout (identity block table), uniform T per call,
# several dtypes, with the bookkeeping operations mixed in.
# --------------------------------------------------------------------------
def legacy_script(dtype_name: str, seed: int = 4321):
    """Returns (ctor kwargs, list of operations).

    Operations: ("append", k, v) with k/v ``[B, H, T, D]``; ("crop", n);
    ("select", LongTensor); ("repeat", n); ("reset",).
    """
    dtype = DTYPES[dtype_name]
    g = torch.Generator().manual_seed(seed)
    H, D = 2, 8
    ops = []

    def app(B, T):
        ops.append(("append", randn(g, (B, H, T, D), dtype), randn(g, (B, H, T, D), dtype)))

    app(2, 3)      # two of three rows, 3 tokens: lengths (3, 3, 0)
    app(3, 2)      # all three rows -> (5, 5, 2); rows 0, 1 cross a page boundary
    app(3, 1)      # decode step -> (6, 6, 3)
    app(3, 1)      # (7, 7, 4)
    ops.append(("crop", 5))                        # lengths (5, 5, 4); data stays
    app(3, 7)      # bulk append over stale slots, ends at (12, 12, 11)
    ops.append(("select", torch.tensor([2, 0, 1])))  # lengths (11, 12, 12)
    app(3, 4)      # (15, 16, 16)
    ops.append(("crop", -2))                       # clamp to longest - 2 = 14
    app(2, 6)      # rows 0, 1 -> (20, 20, 14)
    ops.append(("reset",))
    app(1, 9)
    ops.append(("repeat", 2))                      # beam expansion: row 0 twice, lengths (9, 9), batch capacity 2
    app(2, 3)      # both copies grow on their own -> (12, 12)
    ops.append(("select", torch.tensor([1, 1, 0])))  # reorder with a duplicate: batch capacity 3
    app(3, 2)      # (14, 14, 14)
    return dict(max_batch_size=3, max_cache_len=22, page_size=4), ops


def legacy_overflow_script(seed: int = 99):
    """Lengths (2, 5, 5) then a 4-token append into capacity 8: row 0 fits, row 1 does not."""
    g = torch.Generator().manual_seed(seed)
    H, D = 2, 8
    dt = torch.float32
    ops = [
        ("append", randn(g, (2, H, 3, D), dt), randn(g, (2, H, 3, D), dt)),
        ("append", randn(g, (3, H, 2, D), dt), randn(g, (3, H, 2, D), dt)),
        ("select", torch.tensor([2, 0, 1])),
        ("append", randn(g, (3, H, 4, D), dt), randn(g, (3, H, 4, D), dt)),  # raises
    ]
    return dict(max_batch_size=3, max_cache_len=8, page_size=4), ops


def run_legacy_script(layer, ops, record):
    """Drive any object with the reference layer's methods; ``record(layer, i, op)`` after each op."""
    for i, op in enumerate(ops):
        kind = op[0]
        if kind == "append":
            layer.append(op[1], op[2])
        elif kind == "crop":
            layer.crop(op[1])
        elif kind == "select":
            layer.batch_select_indices(op[1])
        elif kind == "repeat":
            layer.batch_repeat_interleave(op[1])
        elif kind == "reset":
            layer.reset()
        else:  # pragma: no cover
            raise ValueError(kind)
        record(layer, i, op)


# --------------------------------------------------------------------------
# Scenario 4: scaled-down shapes of the large configurations (bf16 / fp16)
# --------------------------------------------------------------------------
def ragged_lengths(g: torch.Generator, n: int, lo: int, hi: int, log_uniform: bool = False) -> List[int]:
    if log_uniform:
        u = torch.rand(n, generator=g, dtype=torch.float64)
        import math
        return [int(round(math.exp(math.log(lo) + float(x) * (math.log(hi) - math.log(lo))))) for x in u]
    return torch.randint(lo, hi + 1, (n,), generator=g).tolist()


# --------------------------------------------------------------------------
# Scenario 5: rotary embedding of a prefill's K rows, the reference helper's formula
# (python/barqtrain/ops.py:376-428: positions 0..T-1, base 10000, halves convention)
# --------------------------------------------------------------------------
def rope_prefill(dtype_name: str, seed: int = 777):
    """``k`` and ``v`` ``[B, H, T, D]`` of one prefill in the given dtype."""
    dtype = DTYPES[dtype_name]
    g = torch.Generator().manual_seed(seed)
    B, H, T, D = 2, 3, 45, 64
    return randn(g, (B, H, T, D), dtype), randn(g, (B, H, T, D), dtype)


def rope_tables(T: int, D: int, dtype: torch.dtype):
    """cos / sin ``[T, D/2]`` exactly as the reference helper forms them (ops.py:394-407)."""
    positions = torch.arange(T, dtype=dtype)
    half = D // 2
    freqs = torch.arange(half, dtype=torch.float32)
    freqs = 1.0 / torch.pow(10000.0, freqs / half)
    angles = positions[:, None] * freqs[None, :]
    return torch.cos(angles).to(dtype), torch.sin(angles).to(dtype)
