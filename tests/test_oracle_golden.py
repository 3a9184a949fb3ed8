"""The Python oracle against golden vectors produced by the unmodified reference."""

import numpy as np
import pytest
import torch

from oracle.paged_kv_oracle import OracleLayer, OraclePagedCache, rope_rotate_keys
from tests import scenarios as S


def _np(t):
    return S.bits(t).numpy()


def test_reference_known_answer(golden_dir):
    """The reference's own test case (tests/test_kv_cache.py:24-47), values included."""
    gold = np.load(golden_dir / "ref_known_answer.npz")
    ctor, steps = S.ref_known_answer()
    layer = OracleLayer(**ctor)
    seen = []
    for i, (k, v) in enumerate(steps):
        ks, vs = layer.update(k, v)
        seen.append((k, v))
        assert np.array_equal(_np(ks), gold[f"ret_k_{i}"])
        assert np.array_equal(_np(vs), gold[f"ret_v_{i}"])
        assert np.array_equal(_np(layer.keys), gold[f"keys_{i}"])
        assert np.array_equal(_np(layer.values), gold[f"values_{i}"])
        assert np.array_equal(layer.seq_lens.numpy(), gold[f"lens_{i}"])
        assert layer.get_seq_length() == int(gold[f"seq_length_{i}"])
    # the assertions the reference test makes, restated
    assert ks.shape == (1, 2, 5, 4)
    assert torch.equal(ks[:, :, :3], seen[0][0]) and torch.equal(ks[:, :, 3:], seen[1][0])
    assert torch.equal(vs[:, :, :3], seen[0][1]) and torch.equal(vs[:, :, 3:], seen[1][1])
    assert layer.get_seq_length() == 5


SMALL = {
    "small_paged_fp32": {},
    "small_paged_bf16": dict(dtype=torch.bfloat16, kv_heads=2, head_dim=128, prefill=(21, 64, 90),
                             decode_steps=5, num_pages=40, seed=2001),
    "small_paged_fp16_ps32": dict(dtype=torch.float16, kv_heads=8, head_dim=128, page_size=32,
                                  prefill=(100, 33), decode_steps=3, num_pages=16, seed=2002, num_layers=1),
}


@pytest.mark.parametrize("name", sorted(SMALL))
def test_small_paged_against_reference(golden_dir, name):
    gold = np.load(golden_dir / f"{name}.npz")
    sc = S.small_paged(**SMALL[name])
    assert sc.free_list == gold["free_list"].tolist()
    inputs = [t for step in sc.steps for per_seq in step for kv in per_seq for t in kv]
    assert S.digest(*inputs) == str(gold["input_digest"]), "seeded inputs differ from the ones the fixtures were made with"

    finals = sc.final_lengths()
    cache = OraclePagedCache(sc.num_layers, sc.page_size)
    for s, n in enumerate(finals):
        cache.open(s, n)
    for i, step in enumerate(sc.steps):
        col = 0
        for l, per_seq in enumerate(step):
            for s, (k, v) in enumerate(per_seq):
                cache.append(l, s, k, v)
                gk, gv = cache.gather(l, s)
                assert S.digest(gk, gv) == str(gold["gather_digests"][i][col]), (i, l, s)
                col += 1
    for l in range(sc.num_layers):
        for s, n in enumerate(finals):
            assert cache.length(l, s) == int(gold[f"len_l{l}_s{s}"]) == n
            pages = -(-n // sc.page_size)
            k_all = torch.stack([cache.logical_page(l, s, j)[0] for j in range(pages)], dim=1)
            v_all = torch.stack([cache.logical_page(l, s, j)[1] for j in range(pages)], dim=1)
            assert np.array_equal(_np(k_all), gold[f"keys_l{l}_s{s}"])
            assert np.array_equal(_np(v_all), gold[f"values_l{l}_s{s}"])


@pytest.mark.parametrize("dtype_name", ["fp32", "fp64", "fp16", "bf16"])
def test_legacy_script_against_reference(golden_dir, dtype_name):
    gold = np.load(golden_dir / f"legacy_{dtype_name}.npz")
    ctor, ops = S.legacy_script(dtype_name)
    layer = OracleLayer(**ctor)

    def check(lay, i, op):
        assert np.array_equal(_np(lay.keys), gold[f"keys_{i}"]), (i, op[0])
        assert np.array_equal(_np(lay.values), gold[f"values_{i}"]), (i, op[0])
        assert np.array_equal(lay.seq_lens.numpy(), gold[f"lens_{i}"]), (i, op[0])
        assert lay.current_batch_size == int(gold[f"batch_{i}"])
        assert lay.get_seq_length() == int(gold[f"seq_length_{i}"])
        if lay.current_batch_size:
            ks, vs = lay.current_tensors()
            assert np.array_equal(_np(ks), gold[f"cur_k_{i}"])
            assert np.array_equal(_np(vs), gold[f"cur_v_{i}"])

    S.run_legacy_script(layer, ops, check)
    assert int(gold["num_ops"]) == len(ops)


def test_capacity_overflow_matches_reference(golden_dir):
    """The CPU loop raises at the first sequence that does not fit; earlier ones stay written."""
    gold = np.load(golden_dir / "legacy_overflow.npz")
    ctor, ops = S.legacy_overflow_script()
    layer = OracleLayer(**ctor)
    with pytest.raises(ValueError) as err:
        S.run_legacy_script(layer, ops, lambda *a: None)
    assert str(err.value) == str(gold["raised"])
    assert np.array_equal(_np(layer.keys), gold["keys"])
    assert np.array_equal(_np(layer.values), gold["values"])
    assert np.array_equal(layer.seq_lens.numpy(), gold["lens"])


def test_argument_checks():
    layer = OracleLayer(2, 8, 4)
    k = torch.zeros(2, 1, 1, 4)
    with pytest.raises(ValueError):
        layer.append(torch.zeros(3, 1, 1, 4), torch.zeros(3, 1, 1, 4))   # batch too large
    layer.append(k, k)
    with pytest.raises(ValueError):
        layer.append(k, torch.zeros(2, 1, 2, 4))                          # shape mismatch
    with pytest.raises(ValueError):
        layer.append(k.double(), k.double())                              # dtype change
    empty = OracleLayer(2, 8, 4)
    assert empty.get_seq_length() == 0


@pytest.mark.parametrize("dtype_name", ["fp32", "fp16", "bf16"])
def test_rope_restatement_against_the_reference_helper(golden_dir, dtype_name):
    """``rope_rotate_keys`` equals the K output of the reference's ``apply_rope_to_qk`` (ops.py:376-428) on
    the seeded prefill, with the helper's own cos / sin tables (stored beside the output)."""
    gold = np.load(golden_dir / "rope_prefill.npz")
    k, _ = S.rope_prefill(dtype_name)
    view = S._INT_VIEW[k.element_size()]
    cos = torch.from_numpy(gold[f"cos_{dtype_name}"]).view(k.dtype)
    sin = torch.from_numpy(gold[f"sin_{dtype_name}"]).view(k.dtype)
    assert cos.shape == (k.shape[2], k.shape[3] // 2) and view is not None
    assert np.array_equal(_np(rope_rotate_keys(k, cos, sin)), gold[f"k_rope_{dtype_name}"])


def test_byte_compiled_reference_runs_the_known_answer_case(golden_dir):
    """``oracle/ref_python.py`` byte-compiles the reference's own CPU path into ``oracle/_ref``; where that
    build exists it must be the code the golden files were made with (the benchmark's reference arm times it)."""
    from oracle import ref_python

    module = ref_python.load() if ref_python.built() else None
    if module is None:
        pytest.skip("no byte-compiled reference under oracle/_ref (no checkout on this machine)")
    gold = np.load(golden_dir / "ref_known_answer.npz")
    ctor, steps = S.ref_known_answer()
    layer = module.BarqPagedKVCacheLayer(**ctor)
    for i, (k, v) in enumerate(steps):
        ks, vs = layer.update(k, v)
        assert np.array_equal(_np(ks), gold[f"ret_k_{i}"]) and np.array_equal(_np(vs), gold[f"ret_v_{i}"])
        assert np.array_equal(_np(layer.keys), gold[f"keys_{i}"])
        assert layer.get_seq_length() == int(gold[f"seq_length_{i}"])
