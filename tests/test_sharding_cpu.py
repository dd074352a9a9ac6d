"""KV-head sharding across ranks, exercised with world_size-2 gloo processes on CPU."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tq_local_b200.runtime.sharding import HeadShard

        shard = HeadShard.from_process_group()
        assert (shard.world_size, shard.rank) == (world, rank)
        B, Hq, Hkv, D = 3, 8, 4, 128
        shard.check(Hkv, Hq)
        g = torch.Generator().manual_seed(7)  # same tensors on every rank
        k = torch.randn(B, Hkv, 5, D, generator=g)
        q = torch.randn(B, Hq, 1, D, generator=g)
        lo, hi = shard.kv_range(Hkv)
        assert (lo, hi) == (rank * 2, rank * 2 + 2) and shard.q_range(Hkv, Hq) == (rank * 4, rank * 4 + 4)
        assert torch.equal(shard.local_kv(k), k[:, lo:hi])
        ql = shard.local_q(q, Hkv)
        assert torch.equal(ql, q[:, rank * 4:rank * 4 + 4])
        # a per-head "attention" stand-in: the gather must restore global head order
        full = shard.gather_heads(ql * 2.0)
        assert torch.equal(full, q * 2.0)
        with pytest.raises(ValueError):
            shard.check(3, 6)  # 3 KV heads and 2 ranks: neither count divides the other
        # one KV head, two ranks: both serve the head, each stores a part of its tokens
        shard.check(1, 4)
        assert shard.seq_parts(1) == 2 and shard.seq_parts(4) == 1 and shard.kv_range(1) == (0, 1)
        assert shard.q_range(1, 4) == (0, 4)
        k1 = torch.randn(B, 1, 7, D, generator=g)
        piece = shard.local_tokens(shard.local_kv(k1), 1, 0)
        assert torch.equal(piece, k1[:, :, :4] if rank == 0 else k1[:, :, 4:])
        for seen in (7, 8):  # decoded tokens go to the parts in turn
            one = shard.local_tokens(k1[:, :, :1], 1, seen)
            assert one.shape[2] == (1 if seen % 2 == rank else 0)
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_head_shard_two_ranks_gloo():
    world = 2
    with mp.Manager() as manager:
        ret = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert dict(ret) == {0: "ok", 1: "ok"}


def test_single_rank_is_identity():
    from tq_local_b200.runtime.sharding import HeadShard

    s = HeadShard()
    x = torch.randn(2, 4, 3, 128)
    assert s.local_kv(x) is x and s.local_q(x, 2) is x and s.gather_heads(x) is x
    assert s.kv_range(8) == (0, 8) and s.q_range(8, 32) == (0, 32)
    assert s.seq_parts(8) == 1 and s.local_tokens(x, 4, 3) is x
    eight = [HeadShard(8, r) for r in range(8)]  # Qwen2.5-7B: 4 KV heads on 8 ranks
    assert [sh.seq_parts(4) for sh in eight] == [2] * 8
    assert [sh.kv_range(4) for sh in eight] == [(0, 1), (0, 1), (1, 2), (1, 2), (2, 3), (2, 3), (3, 4), (3, 4)]
    assert [sh.q_range(4, 28) for sh in eight][:3] == [(0, 7), (0, 7), (7, 14)]
    t = torch.arange(9.0).view(1, 1, 9, 1)
    pieces = [eight[r].local_tokens(t, 4, 0) for r in (0, 1)]
    assert torch.equal(torch.cat(pieces, dim=2), t)  # a disjoint cover of the prompt
    with pytest.raises(ValueError):
        HeadShard(2, 5).check(8, 32)
