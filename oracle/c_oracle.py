"""Build recipe and ctypes binding for the C restatement (``paged_kv_ref.c``).

TEST INFRASTRUCTURE ONLY: imported by the tests, the smoke check and the
benchmark's CPU-baseline leg, never by the product package.

``build()`` compiles ``paged_kv_ref.c`` with gcc (+OpenMP) into
``oracle/_build/libbarqkv_ref.so``.  The functions take torch CPU tensors and
pass raw pointers and byte strides to C.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path
from typing import Optional

import torch

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "paged_kv_ref.c"
_OUT = _HERE / "_build" / "libbarqkv_ref.so"
_LIB: Optional[ctypes.CDLL] = None


def build(force: bool = False) -> Path:
    """Compile the C oracle if the shared object is missing or older than its source."""
    if not force and _OUT.exists() and _OUT.stat().st_mtime >= _SRC.stat().st_mtime:
        return _OUT
    _OUT.parent.mkdir(parents=True, exist_ok=True)
    cmd = ["gcc", "-O3", "-fPIC", "-shared", "-fopenmp", "-std=c11", "-o", str(_OUT), str(_SRC)]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return _OUT


def _lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = _OUT if _OUT.exists() and not _SRC.exists() else build()
        lib = ctypes.CDLL(str(path))
        i32, i64, p = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p
        lib.barqkv_ref_threads.restype = i32
        lib.barqkv_ref_append_legacy.restype = i32
        lib.barqkv_ref_append_legacy.argtypes = [p, p, p, p, p, i32, i32, i32, i32, i32, i32, i64]
        lib.barqkv_ref_append_paged.restype = i32
        lib.barqkv_ref_append_paged.argtypes = [p, p, i64, i64, i32, p, i32, p, p, p, i32, p, p, i64, i64, i32, i32, i64]
        lib.barqkv_ref_gather_paged.restype = i32
        lib.barqkv_ref_gather_paged.argtypes = [p, p, i64, i64, i32, p, i32, p, p, p, i32, p, p, i64, i64, i32, i32, i64]
        _LIB = lib
    return _LIB


def threads() -> int:
    return int(_lib().barqkv_ref_threads())


def set_threads(n: int) -> None:
    os.environ["OMP_NUM_THREADS"] = str(int(n))


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _cpu(*tensors):
    for t in tensors:
        if t is not None and (t.device.type != "cpu"):
            raise ValueError("the C oracle works on CPU tensors only")


def append_legacy(keys, values, seq_lens, k_new, v_new, max_cache_len: int) -> int:
    """In-place reference-layout append; returns 0 or 1 + first sequence that does not fit."""
    _cpu(keys, values, seq_lens, k_new, v_new)
    assert keys.is_contiguous() and values.is_contiguous() and k_new.is_contiguous() and v_new.is_contiguous()
    assert seq_lens.dtype == torch.int32
    B, H, T, D = k_new.shape
    max_blocks, ps = keys.shape[2], keys.shape[3]
    return int(_lib().barqkv_ref_append_legacy(
        _ptr(keys), _ptr(values), _ptr(seq_lens), _ptr(k_new), _ptr(v_new),
        B, H, T, max_blocks, ps, int(max_cache_len), D * k_new.element_size()))


def append_paged(k_pool, v_pool, table, slots, start, cu_new, k_new, v_new) -> int:
    """``k_pool``/``v_pool``: ``[H, P, ps, D]``; ``k_new``/``v_new``: packed ``[N, H, D]``."""
    _cpu(k_pool, v_pool, table, slots, start, cu_new, k_new, v_new)
    H, P, ps, D = k_pool.shape
    e = k_pool.element_size()
    assert k_pool.is_contiguous() and v_pool.is_contiguous() and table.is_contiguous()
    assert k_new.stride(2) == 1 and v_new.stride() == k_new.stride()
    n = cu_new.numel() - 1
    return int(_lib().barqkv_ref_append_paged(
        _ptr(k_pool), _ptr(v_pool), P * ps * D * e, ps * D * e, P,
        _ptr(table), table.stride(0), _ptr(slots), _ptr(start), _ptr(cu_new), n,
        _ptr(k_new), _ptr(v_new), k_new.stride(0) * e, k_new.stride(1) * e, H, ps, D * e))


def gather_paged(k_pool, v_pool, table, slots, lens, cu_out, k_out, v_out) -> int:
    """Writes ``k_out``/``v_out`` (any layout with unit stride on the last dim, indexed [token, head, dim])."""
    _cpu(k_pool, v_pool, table, slots, lens, cu_out, k_out, v_out)
    H, P, ps, D = k_pool.shape
    e = k_pool.element_size()
    assert k_out.stride(2) == 1 and v_out.stride() == k_out.stride()
    n = lens.numel()
    return int(_lib().barqkv_ref_gather_paged(
        _ptr(k_pool), _ptr(v_pool), P * ps * D * e, ps * D * e, P,
        _ptr(table), table.stride(0), _ptr(slots), _ptr(lens), _ptr(cu_out), n,
        _ptr(k_out), _ptr(v_out), k_out.stride(0) * e, k_out.stride(1) * e, H, ps, D * e))
