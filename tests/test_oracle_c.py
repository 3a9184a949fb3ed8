"""The C restatement against the Python oracle (which is pinned to the reference)."""

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle.paged_kv_oracle import OracleLayer, OraclePagedCache
from tests import scenarios as S


@pytest.mark.parametrize("dtype_name", ["fp32", "fp64", "fp16", "bf16"])
def test_c_legacy_append_matches_python_oracle(dtype_name):
    ctor, ops = S.legacy_script(dtype_name)
    ref = OracleLayer(**ctor)
    state = {}

    def mirror(lay, i, op):
        # replay appends through C on a private copy taken before the append
        if op[0] != "append":
            state["k"], state["v"], state["n"] = lay.keys.clone(), lay.values.clone(), lay.seq_lens.clone()
            return
        k, v = op[1], op[2]
        if "k" not in state or state["k"].shape != lay.keys.shape:
            state["k"] = torch.zeros_like(lay.keys)
            state["v"] = torch.zeros_like(lay.values)
            state["n"] = torch.zeros_like(lay.seq_lens)
        rc = c_oracle.append_legacy(state["k"], state["v"], state["n"], k.contiguous(), v.contiguous(), lay.max_cache_len)
        assert rc == 0
        assert torch.equal(S.bits(state["k"]), S.bits(lay.keys)), i
        assert torch.equal(S.bits(state["v"]), S.bits(lay.values)), i
        assert torch.equal(state["n"], lay.seq_lens), i

    S.run_legacy_script(ref, ops, mirror)


def test_c_legacy_overflow_reports_first_failing_row(golden_dir):
    gold = np.load(golden_dir / "legacy_overflow.npz")
    ctor, ops = S.legacy_overflow_script()
    ref = OracleLayer(**ctor)
    S.run_legacy_script(ref, ops[:3], lambda *a: None)
    k, v, n = ref.keys.clone(), ref.values.clone(), ref.seq_lens.clone()
    rc = c_oracle.append_legacy(k, v, n, ops[3][1], ops[3][2], ref.max_cache_len)
    assert rc == 2                                  # 1 + row 1
    assert np.array_equal(S.bits(k).numpy(), gold["keys"])
    assert np.array_equal(S.bits(v).numpy(), gold["values"])
    assert np.array_equal(n.numpy(), gold["lens"])


@pytest.mark.parametrize("layout", ["token_major", "head_major"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_c_block_table_forms_match_composed_reference_layers(dtype, layout):
    g = torch.Generator().manual_seed(7)
    H, D, ps, P, L = 3, 16, 4, 48, 1
    lens0 = [5, 0, 13, 8]
    n = len(lens0)
    free = torch.randperm(P, generator=g).tolist()
    max_blocks = 8
    table = torch.full((n, max_blocks), -1, dtype=torch.int32)
    k_pool = torch.zeros(H, P, ps, D, dtype=dtype)
    v_pool = torch.zeros_like(k_pool)
    ora = OraclePagedCache(L, ps)
    lens = [0] * n
    for s in range(n):
        ora.open(s, max_blocks * ps)

    def step(counts):
        total = sum(counts)
        k_new = S.randn(g, (total, H, D), dtype)
        v_new = S.randn(g, (total, H, D), dtype)
        cu = [0]
        for s, c in enumerate(counts):
            need = -(-(lens[s] + c) // ps)
            have = -(-lens[s] // ps)
            for j in range(have, need):
                table[s, j] = free.pop()
            cu.append(cu[-1] + c)
        start = torch.tensor(lens, dtype=torch.int32)
        rc = c_oracle.append_paged(k_pool, v_pool, table, None, start, torch.tensor(cu, dtype=torch.int32), k_new, v_new)
        assert rc == 0
        for s, c in enumerate(counts):
            if c:
                ora.append(0, s, k_new[cu[s]:cu[s + 1]].transpose(0, 1), v_new[cu[s]:cu[s + 1]].transpose(0, 1))
            lens[s] += c

    step(lens0)
    step([1, 1, 1, 1])
    step([7, 3, 0, 2])

    total = sum(lens)
    cu_out = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    if layout == "token_major":
        k_out = torch.zeros(total, H, D, dtype=dtype)
        v_out = torch.zeros_like(k_out)
        ko, vo = k_out, v_out
    else:
        k_out = torch.zeros(H, total, D, dtype=dtype)
        v_out = torch.zeros_like(k_out)
        ko, vo = k_out.transpose(0, 1), v_out.transpose(0, 1)
    rc = c_oracle.gather_paged(k_pool, v_pool, table, None, torch.tensor(lens, dtype=torch.int32), cu_out[:-1].contiguous(), ko, vo)
    assert rc == 0
    for s in range(n):
        gk, gv = ora.gather(0, s)                  # [H, len, D]
        a, b = int(cu_out[s]), int(cu_out[s + 1])
        assert torch.equal(S.bits(ko[a:b].transpose(0, 1)), S.bits(gk))
        assert torch.equal(S.bits(vo[a:b].transpose(0, 1)), S.bits(gv))
        for j in range(-(-lens[s] // ps)):
            pk, pv = ora.logical_page(0, s, j)
            assert torch.equal(S.bits(k_pool[:, int(table[s, j])]), S.bits(pk))
            assert torch.equal(S.bits(v_pool[:, int(table[s, j])]), S.bits(pv))


def test_c_rejects_bad_table_entry():
    H, D, ps, P = 1, 4, 2, 4
    pool = torch.zeros(H, P, ps, D)
    table = torch.tensor([[9]], dtype=torch.int32)
    one = torch.ones(1, H, D)
    rc = c_oracle.append_paged(pool, pool.clone(), table, None, torch.zeros(1, dtype=torch.int32),
                               torch.tensor([0, 1], dtype=torch.int32), one, one)
    assert rc == -1
    assert pool.abs().sum() == 0
