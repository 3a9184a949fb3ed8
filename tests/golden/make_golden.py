"""Generate the golden vectors in this folder by running the UNMODIFIED reference.

Run where the reference checkout is available:

    BARQTRAIN_REFERENCE=/path/to/BarqTrain python tests/golden/make_golden.py

It imports ``barqtrain.kv_cache.BarqPagedKVCacheLayer`` from the reference's
``python/`` folder with the native backend disabled (``BARQTRAIN_AUTO_BUILD=0``,
so ``append`` takes ``_python_append``, kv_cache.py:75-91), drives it with the
seeded scenarios of ``tests/scenarios.py`` and stores what it produced:
whole tensors as integer bit patterns where they are small, sha256 digests
where they are not.  The tests replay the scenarios through the oracle and the
CUDA path and compare with these files; nothing at test time needs the
reference itself.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

if "BARQTRAIN_REFERENCE" not in os.environ:
    raise SystemExit("set BARQTRAIN_REFERENCE to a checkout of YASSERRMD/BarqTrain")
REF = Path(os.environ["BARQTRAIN_REFERENCE"])
os.environ["BARQTRAIN_AUTO_BUILD"] = "0"
sys.dont_write_bytecode = True
sys.path.insert(0, str(REF / "python"))

from barqtrain.kv_cache import BarqPagedKVCacheLayer  # noqa: E402  (the reference)
from barqtrain.ops import apply_rope_to_qk  # noqa: E402  (the reference)

from tests import scenarios as S  # noqa: E402


def npbits(t: torch.Tensor) -> np.ndarray:
    return S.bits(t).numpy().copy()  # copy: the layer keeps mutating its storage


def gen_known_answer():
    ctor, steps = S.ref_known_answer()
    layer = BarqPagedKVCacheLayer(**ctor)
    out = {}
    for i, (k, v) in enumerate(steps):
        ks, vs = layer.update(k, v)
        out[f"ret_k_{i}"] = npbits(ks)
        out[f"ret_v_{i}"] = npbits(vs)
        out[f"keys_{i}"] = npbits(layer.keys)
        out[f"values_{i}"] = npbits(layer.values)
        out[f"lens_{i}"] = layer.seq_lens.numpy().copy()
        out[f"seq_length_{i}"] = np.int64(layer.get_seq_length())
    np.savez_compressed(HERE / "ref_known_answer.npz", **out)


def gen_small_paged(name: str, **overrides):
    sc = S.small_paged(**overrides)
    ps = sc.page_size
    finals = sc.final_lengths()
    refs = [[BarqPagedKVCacheLayer(1, -(-n // ps) * ps, ps) for n in finals] for _ in range(sc.num_layers)]
    out = {"free_list": np.asarray(sc.free_list, dtype=np.int32)}
    gather_digests = []
    inputs = []
    for step in sc.steps:
        row = []
        for l, per_seq in enumerate(step):
            for s, (k, v) in enumerate(per_seq):
                inputs += [k, v]
                refs[l][s].append(k.unsqueeze(0), v.unsqueeze(0))
                gk, gv = refs[l][s].current_tensors()
                # digest of the contiguous [H, len, D] gather of this sequence
                row.append(S.digest(gk[0], gv[0]))
        gather_digests.append(row)
    out["gather_digests"] = np.asarray(gather_digests)  # [steps, L*S]
    out["input_digest"] = np.asarray(S.digest(*inputs))
    for l in range(sc.num_layers):
        for s in range(len(finals)):
            out[f"keys_l{l}_s{s}"] = npbits(refs[l][s].keys[0])      # [H, blocks, ps, D]
            out[f"values_l{l}_s{s}"] = npbits(refs[l][s].values[0])
            out[f"len_l{l}_s{s}"] = np.int64(refs[l][s].get_seq_length())
    np.savez_compressed(HERE / f"{name}.npz", **out)


def gen_legacy(dtype_name: str):
    ctor, ops = S.legacy_script(dtype_name)
    layer = BarqPagedKVCacheLayer(**ctor)
    out = {}

    def record(lay, i, op):
        out[f"keys_{i}"] = npbits(lay.keys)
        out[f"values_{i}"] = npbits(lay.values)
        out[f"lens_{i}"] = lay.seq_lens.numpy().copy()
        out[f"batch_{i}"] = np.int64(lay.current_batch_size)
        out[f"seq_length_{i}"] = np.int64(lay.get_seq_length())
        if lay.current_batch_size:
            ks, vs = lay.current_tensors()
            out[f"cur_k_{i}"] = npbits(ks)
            out[f"cur_v_{i}"] = npbits(vs)

    S.run_legacy_script(layer, ops, record)
    out["num_ops"] = np.int64(len(ops))
    np.savez_compressed(HERE / f"legacy_{dtype_name}.npz", **out)


def gen_overflow():
    ctor, ops = S.legacy_overflow_script()
    layer = BarqPagedKVCacheLayer(**ctor)
    raised = ""
    try:
        S.run_legacy_script(layer, ops, lambda *a: None)
    except ValueError as exc:
        raised = str(exc)
    out = dict(
        raised=np.asarray(raised),
        keys=npbits(layer.keys),
        values=npbits(layer.values),
        lens=layer.seq_lens.numpy().copy(),
    )
    np.savez_compressed(HERE / "legacy_overflow.npz", **out)


def gen_rope():
    """The reference's rotary helper on a seeded prefill, per dtype: its rotated K rows, plus the cos / sin
    tables formed with the helper's own expressions - stored so that a test does not depend on the host's
    libm - after checking that they reproduce the helper's output bit for bit."""
    out = {}
    for name in ("fp32", "fp16", "bf16"):
        k, _v = S.rope_prefill(name)
        _, k_rope = apply_rope_to_qk(k, k)
        T, D = k.shape[2], k.shape[3]
        cos, sin = S.rope_tables(T, D, k.dtype)
        half = D // 2
        again = torch.cat([k[..., :half] * cos - k[..., half:] * sin, k[..., :half] * sin + k[..., half:] * cos], dim=-1)
        assert torch.equal(S.bits(again), S.bits(k_rope)), name
        out[f"k_rope_{name}"] = npbits(k_rope)
        out[f"cos_{name}"] = npbits(cos)
        out[f"sin_{name}"] = npbits(sin)
    np.savez_compressed(HERE / "rope_prefill.npz", **out)


def main():
    gen_known_answer()
    gen_rope()
    gen_small_paged("small_paged_fp32")
    gen_small_paged("small_paged_bf16", dtype=torch.bfloat16, kv_heads=2, head_dim=128,
                    prefill=(21, 64, 90), decode_steps=5, num_pages=40, seed=2001)
    gen_small_paged("small_paged_fp16_ps32", dtype=torch.float16, kv_heads=8, head_dim=128, page_size=32,
                    prefill=(100, 33), decode_steps=3, num_pages=16, seed=2002, num_layers=1)
    for name in ("fp32", "fp64", "fp16", "bf16"):
        gen_legacy(name)
    gen_overflow()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
