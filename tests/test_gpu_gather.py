"""GPU: the fused peer gather of KV-head sharded decode attention (tq_decode_attn_gather)."""

from __future__ import annotations

import os
import subprocess
import sys

import pytest
import torch

from helpers import make_codec, oracle_params
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


def _parts_desc(rank, world, q_heads_total, exch, flags, counters, seq):
    from tq_local_b200.runtime import ffi

    d = ffi.GatherDesc()
    d.world, d.rank, d.q_heads_total, d.seq = world, rank, q_heads_total, seq
    d.out_stride = exch[0].stride(0) * 4
    for r in range(world):
        d.out[r] = exch[r].data_ptr()
        d.flags[r] = flags[r].data_ptr()
    d.counter = counters[rank].data_ptr()
    d.seq_dev = None
    return d


@pytest.mark.parametrize("Hq,Hkv,parts,lens", [
    (8, 1, 2, (700, 333)),      # one KV head shared by two ranks
    (7, 1, 2, (512, 0)),        # the wide kernel variant; the second part holds no token yet
    (8, 2, 2, (100, 1)),        # two KV heads per group
    (16, 2, 4, (300, 301, 0, 77)),  # four ranks share a group of two KV heads
])
def test_sequence_split_on_one_gpu_matches_the_undivided_cache(setup_golden, Hq, Hkv, parts, lens):
    """More ranks than KV heads: `parts` ranks hold disjoint parts of a KV-head group's tokens and
    exchange unfinished partials.  Emulated on one GPU: the ranks' calls run one after the other on
    one stream (all scatters, then all finishes, so no wait depends on a later launch), with plain
    device tensors as exchange buffers.  Every rank's result must equal attention over the
    undivided cache (oracle, 2e-3 + output rounding) and all ranks must agree bit for bit."""
    import ctypes as C

    from tq_local_b200.runtime import ffi
    from tq_local_b200.runtime.codec import tq_dtype
    from tq_local_b200.runtime.packed_store import PackedStore

    codec = make_codec(4, True, setup_golden)
    p = oracle_params(4, True, setup_golden)
    world, B, dtype = parts, 2, torch.bfloat16  # one head group: world = parts
    n_total = sum(lens)
    k, v, q = O.synth_kvq(B, Hq, Hkv, n_total, 128, seed=61, dtype=dtype)
    whole = PackedStore(codec, B, Hkv, capacity=n_total)
    whole.pack(k.cuda(), v.cuda())
    stores, lo = [], 0
    for n in lens:
        st = PackedStore(codec, B, Hkv, capacity=max(n, 8))
        if n:
            st.pack(k[:, :, lo:lo + n].cuda(), v[:, :, lo:lo + n].cuda())
        stores.append(st)
        lo += n
    L = ffi.lib()
    nbytes = int(L.tq_parts_exchange_bytes(B, Hq, parts))
    assert nbytes >= B * Hq * parts * 130 * 4
    exch = [torch.zeros(2, nbytes // 4, dtype=torch.float32, device="cuda") for _ in range(world)]
    flags = [torch.zeros(ffi.TQ_MAX_PEERS, dtype=torch.int32, device="cuda") for _ in range(world)]
    counters = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(world)]
    qd = q.cuda().reshape(B, Hq, 128).contiguous()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    dt = tq_dtype(dtype)
    for seq in (1, 2, 3):  # both exchange buffers get used
        outs = [torch.empty(B, Hq, 1, 128, dtype=dtype, device="cuda") for _ in range(world)]
        descs = [_parts_desc(r, world, Hq, exch, flags, counters, seq) for r in range(world)]
        for r in range(world):
            st = stores[r]
            ws = st._get_workspace(Hq, 2)
            rc = L.tq_decode_attn_parts(codec.handle, qd.data_ptr(), dt, Hq, C.byref(st._desc), st.length, 2,
                                        ws.data_ptr(), ws.numel(), C.byref(descs[r]), parts, stream)
            assert rc == 0, rc
        for r in range(world):
            rc = L.tq_decode_parts_finish(codec.handle, C.byref(descs[r]), B, dt, parts, Hq // Hkv, outs[r].data_ptr(),
                                          stream)
            assert rc == 0, rc
        torch.cuda.synchronize()
        for r in range(1, world):
            assert torch.equal(outs[0], outs[r])
        # the oracle wants (k_codes, k_norms, v_codes, v_norms, k_signs, k_rnorms) in its own order
        layer = O.PackedLayer(p, dtype, whole.k_codes[:, :, :n_total].cpu(), whole.k_norms[:, :, :n_total].cpu(),
                              whole.v_codes[:, :, :n_total].cpu(), whole.v_norms[:, :, :n_total].cpu(),
                              whole.k_signs[:, :, :n_total].cpu(), whole.k_rnorms[:, :, :n_total].cpu())
        want = O.attend_rotated_space(q, layer, Hq // Hkv)
        err = float((outs[0].float().cpu() - want).abs().max() / want.abs().max())
        assert err <= 2e-3 + 2.0 ** -9, (seq, err)
        err2 = float((outs[0].float() - whole.decode_attn(q.cuda()).float()).abs().max() / want.abs().max())
        assert err2 <= 2.0 ** -7
    assert codec.device_status() == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_split_between_two_gpus_through_the_cache_layer():
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mp_parts_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29617", worker],
                         capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0 and "PARTS_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-3000:]
