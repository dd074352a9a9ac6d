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


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_gather_between_two_gpus_equals_nccl_all_gather():
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mp_gather_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29611", worker],
                         capture_output=True, text=True, timeout=240, env=env)
    assert out.returncode == 0 and "GATHER_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
