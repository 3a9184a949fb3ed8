"""KV-head sharding with world_size 2 over gloo on CPU: the ranks' shards are disjoint, cover all
heads, agree on the replicated metadata, and concatenating the per-rank gathers (C oracle standing
in for the device) gives the unsharded gather.  The max-over-ranks timing reduction is checked too."""

import os
import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from barqtrain_b200.sharding import kv_head_shard, metadata_digest, shard_heads
        from oracle import c_oracle

        H, D, ps, P = 4, 16, 4, 40
        g = torch.Generator().manual_seed(2024)                 # same seed on every rank
        lens = torch.randint(1, 30, (5,), generator=g).tolist()
        order = torch.randperm(P, generator=g).tolist()
        k_full = torch.randn(sum(lens), H, D, generator=g)
        v_full = torch.randn(sum(lens), H, D, generator=g)

        # replicated metadata must agree
        digests = [None] * world
        dist.all_gather_object(digests, metadata_digest(lens, order))
        assert len(set(digests)) == 1

        first, count = kv_head_shard(H, world, rank)
        owned = [None] * world
        dist.all_gather_object(owned, (first, count))
        covered = sorted(h for f, c in owned for h in range(f, f + c))
        assert covered == list(range(H)), "shards must be disjoint and cover every head"

        # this rank's pools hold only its heads; table identical everywhere
        table = torch.full((len(lens), 8), -1, dtype=torch.int32)
        at = 0
        for s, n in enumerate(lens):
            nb = -(-n // ps)
            table[s, :nb] = torch.tensor(order[at:at + nb], dtype=torch.int32)
            at += nb
        k_pool = torch.zeros(count, P, ps, D)
        v_pool = torch.zeros_like(k_pool)
        cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
        start = torch.zeros(len(lens), dtype=torch.int32)
        k_mine = shard_heads(k_full, 1, world, rank)
        v_mine = shard_heads(v_full, 1, world, rank)
        assert c_oracle.append_paged(k_pool, v_pool, table, None, start, cu, k_mine, v_mine) == 0
        k_out = torch.zeros(sum(lens), count, D)
        v_out = torch.zeros_like(k_out)
        lens_t = torch.tensor(lens, dtype=torch.int32)
        assert c_oracle.gather_paged(k_pool, v_pool, table, None, lens_t, cu[:-1].contiguous(), k_out, v_out) == 0
        assert torch.equal(k_out, k_mine) and torch.equal(v_out, v_mine)

        # concatenating the shards along the head dimension gives the unsharded result
        parts = [torch.zeros(sum(lens), count, D) for _ in range(world)]
        dist.all_gather(parts, k_out)
        assert torch.equal(torch.cat(parts, dim=1), k_full)

        # timing reduction used by the benchmark: the slowest rank defines the step
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert float(t) == float(world)
        Path(out_dir, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_by_kv_head(tmp_path):
    from oracle import c_oracle

    c_oracle.build()                       # compile once, before the ranks race for it
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(p.name for p in tmp_path.iterdir()) == ["ok0", "ok1"]


def test_shard_arithmetic():
    import pytest

    from barqtrain_b200.sharding import kv_head_shard

    assert [kv_head_shard(8, 4, r) for r in range(4)] == [(0, 2), (2, 2), (4, 2), (6, 2)]
    assert kv_head_shard(8, 8, 7) == (7, 1) and kv_head_shard(8, 1, 0) == (0, 8)
    with pytest.raises(ValueError):
        kv_head_shard(8, 3, 0)
    with pytest.raises(ValueError):
        kv_head_shard(8, 2, 2)
