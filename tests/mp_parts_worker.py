"""Worker of the 2-GPU sequence-split test (one process per GPU, launched by torchrun): one KV head
shared by two ranks, each holding a part of its tokens.  The cache layer under a ``HeadShard`` must
give, on every rank, the attention of an unsharded layer over all tokens, through prefill, appends
that alternate between the ranks, and decode steps."""

from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    from tq_local_b200.runtime.packed_qmse_cache import PackedMSELayer
    from tq_local_b200.runtime.sharding import HeadShard, PeerGather

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    shard = HeadShard.from_process_group()
    for Hq, Hkv in ((8, 1), (7, 1)):  # four heads per KV head; seven (the wide kernel variant)
        B, N, steps = 3, 1001, 5
        g = torch.Generator().manual_seed(11)  # identical on every rank
        k = torch.randn(B, Hkv, N + steps, 128, generator=g).to(torch.bfloat16).to(dev)
        v = torch.randn(B, Hkv, N + steps, 128, generator=g).to(torch.bfloat16).to(dev)
        qs = torch.randn(steps, B, Hq, 1, 128, generator=g).to(torch.bfloat16).to(dev)
        kw = dict(bits=4, use_qjl_keys=True, quantize_decode=True, reserve_tokens=steps + 4)
        whole = PackedMSELayer(**kw)  # every rank also keeps an unsharded copy as the reference
        split = PackedMSELayer(shard=shard, **kw)
        whole.initialize_from_dense(k[:, :, :N], v[:, :, :N])
        split.initialize_from_dense(k[:, :, :N], v[:, :, :N])
        whole._lazy_update = split._lazy_update = True
        assert split.seq_parts == 2 and split.get_seq_length() == N
        assert split.store.length == (501 if rank == 0 else 500)
        for t in range(steps):
            kt, vt = k[:, :, N + t:N + t + 1], v[:, :, N + t:N + t + 1]
            whole.update(kt, vt)
            split.update(kt, vt)
            want = whole.attend(qs[t])
            got = split.attend(qs[t])
            torch.cuda.synchronize()
            assert tuple(got.shape) == (B, Hq, 1, 128) and split.get_seq_length() == N + t + 1
            err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
            assert err <= 2.0 ** -7, f"rank {rank} heads {Hq}/{Hkv} step {t}: {err}"
        # the five appended tokens alternate between the parts (token N + t goes to part (N + t) % 2)
        assert split.store.length == (501 + 2 if rank == 0 else 500 + 3)
        assert split.codec.device_status() == 0
        # both ranks hold the same bytes of output
        mine = got.contiguous()
        theirs = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(theirs, mine)
        assert torch.equal(theirs[0], theirs[1])
    PeerGather.close_shared()
    if rank == 0:
        print("PARTS_OK")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
