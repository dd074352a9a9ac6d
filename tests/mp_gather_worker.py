"""Worker of the 2-GPU gather test (one process per GPU, launched by torchrun): KV-head sharded
decode attention with the fused peer gather must equal the NCCL all-gather of the same outputs."""

from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    from tq_local_b200.runtime.codec import Codec
    from tq_local_b200.runtime.packed_store import PackedStore
    from tq_local_b200.runtime.sharding import HeadShard, PeerGather

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    shard = HeadShard.from_process_group()
    B, Hq, Hkv, N, steps = 3, 16, 4, 1500, 5
    g = torch.Generator().manual_seed(7)  # identical on every rank
    k = torch.randn(B, Hkv, N, 128, generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn(B, Hkv, N, 128, generator=g).to(torch.bfloat16).to(dev)
    qs = torch.randn(steps, B, Hq, 1, 128, generator=g).to(torch.bfloat16).to(dev)
    codec = Codec.get(dev, 4, True, 0)
    store = PackedStore(codec, B, Hkv // world, capacity=N + 8)
    store.pack(shard.local_kv(k), shard.local_kv(v))
    gather = PeerGather(shard, B, Hq, torch.bfloat16, dev)
    try:
        for t in range(steps):
            q_local = shard.local_q(qs[t], Hkv)
            want = shard.gather_heads(store.decode_attn(q_local))  # NCCL all-gather
            got = store.decode_attn_gather(q_local, gather)
            torch.cuda.synchronize()
            assert torch.equal(got, want), f"rank {rank} step {t}"
        assert codec.device_status() == 0
    finally:
        gather.close()

    # host buffers in, gathered output into a host buffer (append + attend + exchange in one call)
    host_store = PackedStore(codec, B, Hkv // world, capacity=N + 8)
    ref2 = PackedStore(codec, B, Hkv // world, capacity=N + 8)
    for st in (host_store, ref2):
        st.pack(shard.local_kv(k[:, :, :N - 4]), shard.local_kv(v[:, :, :N - 4]))
    gather = PeerGather(shard, B, Hq, torch.bfloat16, dev)
    try:
        h_out = torch.empty(B, Hq, 1, 128, dtype=torch.bfloat16).pin_memory()
        for t in range(3):
            pos = N - 4 + t
            kt, vt = shard.local_kv(k[:, :, pos:pos + 1]), shard.local_kv(v[:, :, pos:pos + 1])
            ref2.pack(kt, vt)
            want = shard.gather_heads(ref2.decode_attn(shard.local_q(qs[t], Hkv)))
            host_store.decode_step_host_gather(shard.local_q(qs[t], Hkv).contiguous().cpu().pin_memory(),
                                               kt.contiguous().cpu().pin_memory(), vt.contiguous().cpu().pin_memory(),
                                               h_out, gather)
            torch.cuda.synchronize()
            assert torch.equal(h_out, want.cpu()), f"rank {rank} host step {t}"
    finally:
        gather.close()

    # the same exchange inside the device-length step, numbered on the device and replayed from a
    # CUDA graph; the reference is the un-sharded result of the NCCL path
    N0 = N - 4
    dev_store = PackedStore(codec, B, Hkv // world, capacity=N + 8)
    ref_store = PackedStore(codec, B, Hkv // world, capacity=N + 8)
    for st in (dev_store, ref_store):
        st.pack(shard.local_kv(k[:, :, :N0]), shard.local_kv(v[:, :, :N0]))
    gather = PeerGather(shard, B, Hq, torch.bfloat16, dev, device_sequence=True)
    try:
        pos = torch.tensor([N0], dtype=torch.int32, device=dev)
        sq = torch.empty(B, Hq // world, 1, 128, dtype=torch.bfloat16, device=dev)
        sk = torch.empty(B, Hkv // world, 1, 128, dtype=torch.bfloat16, device=dev)
        sv = torch.empty_like(sk)
        sout = torch.empty(B, Hq, 1, 128, dtype=torch.bfloat16, device=dev)
        graph = None
        for t in range(4):
            kt, vt = shard.local_kv(k[:, :, N0 + t:N0 + t + 1]), shard.local_kv(v[:, :, N0 + t:N0 + t + 1])
            ref_store.pack(kt, vt)
            want = shard.gather_heads(ref_store.decode_attn(shard.local_q(qs[t], Hkv),
                                                            splits=dev_store.suggest_splits(dev_store.capacity)))
            sq.copy_(shard.local_q(qs[t], Hkv)), sk.copy_(kt), sv.copy_(vt)
            if t == 0:
                dev_store.decode_step_dev(sq, sk, sv, pos, out=sout, gather=gather)
                pos.add_(1)
            else:
                if graph is None:
                    torch.cuda.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                        dev_store.decode_step_dev(sq, sk, sv, pos, out=sout, gather=gather)
                        pos.add_(1)
                graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(sout, want), f"rank {rank} device-length step {t}"
        assert codec.device_status() == 0
    finally:
        gather.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("GATHER_OK")


if __name__ == "__main__":
    main()
