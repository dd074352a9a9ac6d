"""GPU: the fused peer gather of KV-head sharded decode attention (tq_decode_attn_gather)."""

from __future__ import annotations

import os
import subprocess
import sys

import pytest
import torch

from helpers import make_codec
from oracle import tq_oracle as O

pytestmark = pytest.mark.gpu


def test_gather_of_one_rank_equals_plain_decode(setup_golden):
    """world = 1: same kernels, the combine writes into the gathered buffer and raises its own
    flag, the wait kernel sees it.  Must equal tq_decode_attn bit for bit on every step (the two
    output buffers alternate)."""
    from tq_local_b200.runtime.packed_store import PackedStore
    from tq_local_b200.runtime.sharding import HeadShard, PeerGather

    codec = make_codec(4, True, setup_golden)
    B, Hq, Hkv, N = 2, 14, 2, 900
    k, v, _ = O.synth_kvq(B, Hq, Hkv, N, 128, seed=31, dtype=torch.bfloat16)
    store = PackedStore(codec, B, Hkv, capacity=N)
    store.pack(k.cuda(), v.cuda())
    gather = PeerGather(HeadShard(), B, Hq, torch.bfloat16, codec.device)
    try:
        g = torch.Generator().manual_seed(1)
        for step in range(4):
            q = torch.randn(B, Hq, 1, 128, generator=g).to(torch.bfloat16).cuda()
            want = store.decode_attn(q)
            got = store.decode_attn_gather(q, gather)
            torch.cuda.synchronize()
            assert tuple(got.shape) == (B, Hq, 1, 128) and torch.equal(got, want), step
    finally:
        gather.close()
    assert codec.device_status() == 0


def test_device_sequenced_gather_in_the_device_length_step_and_in_a_graph(setup_golden):
    """world = 1: decode_step_dev with a PeerGather whose step numbers live on the device equals
    the plain device-length step, eagerly and replayed from a CUDA graph (both gathered buffers
    get used: the step number advances on the device)."""
    from tq_local_b200.runtime.packed_store import PackedStore
    from tq_local_b200.runtime.sharding import HeadShard, PeerGather

    codec = make_codec(4, True, setup_golden)
    B, Hq, Hkv, N0, steps = 2, 8, 2, 600, 6
    k, v, _ = O.synth_kvq(B, Hq, Hkv, N0 + steps, 128, seed=33, dtype=torch.bfloat16)
    k, v = k.cuda(), v.cuda()
    g = torch.Generator().manual_seed(2)
    qs = torch.randn(steps, B, Hq, 1, 128, generator=g).to(torch.bfloat16).cuda()
    plain, fused = (PackedStore(codec, B, Hkv, capacity=1024) for _ in range(2))
    for st in (plain, fused):
        st.pack(k[:, :, :N0], v[:, :, :N0])
    gather = PeerGather(HeadShard(), B, Hq, torch.bfloat16, codec.device, device_sequence=True)
    try:
        pos_a = torch.tensor([N0], dtype=torch.int32, device="cuda")
        pos_b = pos_a.clone()
        want = []
        for t in range(steps):
            want.append(plain.decode_step_dev(qs[t], k[:, :, N0 + t:N0 + t + 1], v[:, :, N0 + t:N0 + t + 1], pos_a).clone())
            pos_a.add_(1)
        sq, sk, sv = torch.empty_like(qs[0]), torch.empty_like(k[:, :, :1]), torch.empty_like(v[:, :, :1])
        sout = torch.empty_like(qs[0])

        def load(t):
            sq.copy_(qs[t]), sk.copy_(k[:, :, N0 + t:N0 + t + 1]), sv.copy_(v[:, :, N0 + t:N0 + t + 1])

        load(0)
        fused.decode_step_dev(sq, sk, sv, pos_b, out=sout, gather=gather)
        pos_b.add_(1)
        assert torch.equal(sout, want[0])
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        load(1)
        with torch.cuda.graph(graph):
            fused.decode_step_dev(sq, sk, sv, pos_b, out=sout, gather=gather)
            pos_b.add_(1)
        for t in range(1, steps):
            load(t)
            graph.replay()
            assert torch.equal(sout, want[t]), t
        assert int(gather.seq_dev.item()) == steps
    finally:
        gather.close()
    assert codec.device_status() == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_gather_between_two_gpus_equals_nccl_all_gather():
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mp_gather_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29611", worker],
                         capture_output=True, text=True, timeout=240, env=env)
    assert out.returncode == 0 and "GATHER_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_generation_on_two_gpus_eager_and_recorded():
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mp_generate_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29613", worker],
                         capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0 and "GENERATE_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-3000:]
