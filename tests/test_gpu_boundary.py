"""GPU: the C ABI's argument checks, its bounded waits and its per-device state.

Nothing here faults, traps or hangs a GPU: bad descriptors are rejected on the host before any
launch, and the one wait that runs out is a flag poll with a short time limit that returns
a status code."""

from __future__ import annotations

import ctypes as C
import time

import pytest
import torch

from helpers import make_codec
from oracle import tq_oracle as O
from tq_local_b200.runtime import ffi
from tq_local_b200.runtime.codec import tq_dtype

pytestmark = pytest.mark.gpu

TQ_ERR_ARG, TQ_ERR_UNSUPPORTED, TQ_ERR_WORKSPACE = -1, -2, -4


def _small_store(codec, B=1, Hkv=2, N=64, seed=3):
    from tq_local_b200.runtime.packed_store import PackedStore

    k, v, _ = O.synth_kvq(B, 4 * Hkv, Hkv, N, 128, seed=seed, dtype=torch.bfloat16)
    store = PackedStore(codec, B, Hkv, capacity=N + 8)
    store.pack(k.cuda(), v.cuda())
    return store


def _local_gather_desc(world=1, rank=0, q_heads_total=8, seq=1, batch=1):
    """A gather descriptor over plain device tensors of this process (world = 1 needs no peers)."""
    out = torch.zeros(2, batch * q_heads_total * 128, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(ffi.TQ_MAX_PEERS, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    d = ffi.GatherDesc()
    d.world, d.rank, d.q_heads_total, d.seq = world, rank, q_heads_total, seq
    d.out_stride = out.stride(0) * 2
    for r in range(world):
        d.out[r] = out.data_ptr()
        d.flags[r] = flags.data_ptr()
    d.counter = counter.data_ptr()
    d.seq_dev = None
    return d, (out, flags, counter)


def test_gather_wait_runs_out_reports_status_5_and_returns(setup_golden):
    """A wait for a step number that nobody raises gives up after the limit set with
    tq_set_wait_limit_ms: the call returns, the status word reads 5, the output is untouched,
    and a fresh context on the same device works afterwards."""
    codec = make_codec(4, True, setup_golden)
    codec.set_wait_limit_ms(50)
    B, Hq = 1, 8
    desc, keep = _local_gather_desc(q_heads_total=Hq, seq=7, batch=B)  # the row counts are all zero: step 7 never arrives
    final = torch.full((B, Hq, 1, 128), 3.0, dtype=torch.bfloat16, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.perf_counter()
    rc = ffi.lib().tq_gather_wait(codec.handle, C.byref(desc), B, tq_dtype(torch.bfloat16), final.data_ptr(), stream)
    assert rc == 0
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.03 < waited < 1.5, waited  # about the 50 ms limit, far from the 2 s default
    assert codec.device_status() == 5
    with pytest.raises(ffi.TQError):
        codec.raise_on_device_status("test")
    assert bool((final == 3.0).all()), "a wait that ran out must not copy the gathered output"
    # the word is sticky for that context only: a new context decodes normally
    fresh = make_codec(4, True, setup_golden)
    store = _small_store(fresh)
    q = torch.randn(1, 8, 1, 128, dtype=torch.bfloat16, device="cuda")
    store.decode_attn(q)
    torch.cuda.synchronize()
    assert fresh.device_status() == 0
    # limits outside 1 .. 60000 ms are refused
    assert ffi.lib().tq_set_wait_limit_ms(fresh.handle, 0) == TQ_ERR_ARG
    assert ffi.lib().tq_set_wait_limit_ms(fresh.handle, 600000) == TQ_ERR_ARG


def test_gather_wait_passes_when_the_flag_is_there(setup_golden):
    codec = make_codec(4, True, setup_golden)
    codec.set_wait_limit_ms(50)
    desc, (out, flags, counter) = _local_gather_desc(q_heads_total=8, seq=2, batch=1)
    flags[0] = 2 * 1 * 8  # this rank's rows of steps 1 and 2 (batch 1 x 8 heads each) are in
    out[0].fill_(1.5)  # step 2 uses buffer 2 & 1 = 0
    final = torch.zeros(1, 8, 1, 128, dtype=torch.bfloat16, device="cuda")
    rc = ffi.lib().tq_gather_wait(codec.handle, C.byref(desc), 1, tq_dtype(torch.bfloat16), final.data_ptr(),
                                  C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert codec.device_status() == 0 and bool((final == 1.5).all())


def test_bad_descriptors_are_rejected_before_any_launch(setup_golden):
    """Misaligned stream pointers, overlapping strides, a missing counter, a missing peer buffer
    and an out-of-range rank all come back as TQ_ERR_ARG from every entry point that takes the
    descriptor; the device never sees them (its status stays 0 and the cache is unchanged)."""
    codec = make_codec(4, True, setup_golden)
    store = _small_store(codec)
    L = ffi.lib()
    B, Hq, Hkv = 1, 8, 2
    q = torch.randn(B, Hq, 128, dtype=torch.bfloat16, device="cuda")
    knew = torch.randn(B, Hkv, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(q)
    ws = torch.empty(int(L.tq_decode_step_workspace_bytes(B, Hq, Hkv, 2)), dtype=torch.uint8, device="cuda")
    pos = torch.tensor([store.length], dtype=torch.int32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    n_stored = store.length
    before = [t[:, :, :n_stored].clone() for t in store.streams()]
    dt = tq_dtype(torch.bfloat16)

    def cache_variant(**kw):
        d = ffi.CacheDesc.from_buffer_copy(store._desc)
        for k_, v_ in kw.items():
            setattr(d, k_, v_)
        return d

    bad_caches = [
        cache_variant(k_codes=store.k_codes.data_ptr() + 1),     # odd pointer
        cache_variant(v_norms=store.v_norms.data_ptr() + 8),     # 8-byte, not 16-byte aligned
        cache_variant(stride_b=store.capacity),                  # rows of a batch entry overlap
        cache_variant(stride_h=store.capacity + 4),              # not a multiple of 8 tokens
        cache_variant(k_signs=None),                             # Q_prod context without a sign stream
    ]
    for bad in bad_caches:
        ref = C.byref(bad)
        assert L.tq_decode_attn(codec.handle, q.data_ptr(), dt, Hq, ref, store.length, None, None, 0, 2,
                                ws.data_ptr(), ws.numel(), out.data_ptr(), stream) == TQ_ERR_ARG
        assert L.tq_decode_attn_static(codec.handle, q.data_ptr(), dt, Hq, ref, store.length, 2, out.data_ptr(),
                                       stream) == TQ_ERR_ARG
        gd, keep = _local_gather_desc(q_heads_total=Hq)
        assert L.tq_decode_attn_gather(codec.handle, q.data_ptr(), dt, Hq, ref, store.length, 2, ws.data_ptr(),
                                       ws.numel(), C.byref(gd), stream) == TQ_ERR_ARG
        assert L.tq_decode_step_dev(codec.handle, q.data_ptr(), knew.data_ptr(), knew.data_ptr(), dt, Hq, ref,
                                    pos.data_ptr(), 2, ws.data_ptr(), ws.numel(), out.data_ptr(), None,
                                    stream) == TQ_ERR_ARG

    good = C.byref(store._desc)
    seq_dev = torch.zeros(1, dtype=torch.int32, device="cuda")
    for breaker in ("counter", "out", "flags", "rank", "world"):
        gd, keep = _local_gather_desc(q_heads_total=Hq)
        gd.seq_dev = seq_dev.data_ptr()
        if breaker == "counter":
            gd.counter = None
        elif breaker == "out":
            gd.out[0] = None
        elif breaker == "flags":
            gd.flags[0] = None
        elif breaker == "rank":
            gd.rank = 1
        else:
            gd.world = ffi.TQ_MAX_PEERS + 1
        assert L.tq_decode_attn_gather(codec.handle, q.data_ptr(), dt, Hq, good, store.length, 2, ws.data_ptr(),
                                       ws.numel(), C.byref(gd), stream) == TQ_ERR_ARG, breaker
        assert L.tq_decode_step_dev(codec.handle, q.data_ptr(), knew.data_ptr(), knew.data_ptr(), dt, Hq, good,
                                    pos.data_ptr(), 2, ws.data_ptr(), ws.numel(), out.data_ptr(), C.byref(gd),
                                    stream) == TQ_ERR_ARG, breaker
        assert L.tq_gather_wait(codec.handle, C.byref(gd), B, dt, None, stream) == TQ_ERR_ARG, breaker

    # the host step checks everything before its first copy or append
    qh, kh, oh = (torch.zeros(B, n, 128, dtype=torch.bfloat16).pin_memory() for n in (Hq, Hkv, Hq))
    step = lambda n_splits, heads, ws_bytes=ws.numel(): L.tq_decode_step_host(
        codec.handle, qh.data_ptr(), kh.data_ptr(), kh.data_ptr(), dt, heads, good, store.length, n_splits,
        ws.data_ptr(), ws_bytes, oh.data_ptr(), stream)
    assert step(0, Hq) == TQ_ERR_ARG              # no splits: the workspace formula has no answer
    assert step(2, 7) == TQ_ERR_ARG               # query heads not a multiple of the KV heads
    assert step(2, Hkv * 16) == TQ_ERR_UNSUPPORTED  # too many query heads per KV head
    assert step(2, Hq, 64) == TQ_ERR_WORKSPACE
    torch.cuda.synchronize()
    assert codec.device_status() == 0
    for a, b in zip(before, store.streams()):
        assert torch.equal(a, b[:, :, :n_stored]), "a rejected call must leave the cache untouched"


def test_device_length_step_with_more_rows_than_sms_and_one_partial_per_row(setup_golden):
    """batch * kv_heads = 2 x the SM count makes tq_decode_suggest_splits answer 1 (whole rows per
    CTA); the device-length step must then launch one CTA per row, not one per SM."""
    from tq_local_b200.runtime.packed_store import PackedStore

    codec = make_codec(4, True, setup_golden)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    Hkv, G = 4, 2
    B = 2 * sms // Hkv
    assert B * Hkv == 2 * sms
    N = 512  # one kernel step per row
    k, v, _ = O.synth_kvq(B, Hkv * G, Hkv, N + 1, 128, seed=17, dtype=torch.bfloat16)
    k, v = k.cuda(), v.cuda()
    plain = PackedStore(codec, B, Hkv, capacity=1024)
    dev = PackedStore(codec, B, Hkv, capacity=1024)
    for st in (plain, dev):
        st.pack(k[:, :, :N], v[:, :, :N])
    assert dev.suggest_splits(dev.capacity) == 1
    q = torch.randn(B, Hkv * G, 1, 128, dtype=torch.bfloat16, device="cuda")
    plain.pack(k[:, :, N:], v[:, :, N:])
    want = plain.decode_attn(q, splits=4)
    pos = torch.tensor([N], dtype=torch.int32, device="cuda")
    got = dev.decode_step_dev(q, k[:, :, N:], v[:, :, N:], pos)
    torch.cuda.synchronize()
    err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
    assert err < 2.0 ** -7, err  # same arithmetic, different split of the rows: one bf16 ulp at most
    assert codec.device_status() == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_two_devices(setup_golden):
    """One process that holds a context on each of two GPUs (the reference's device_map='auto'
    case): both encode and decode; the kernel attributes are set per device."""
    from tq_local_b200.runtime.codec import Codec
    from tq_local_b200.runtime.packed_store import PackedStore

    import gc

    outs = []
    current = torch.cuda.current_device()
    k, v, q = O.synth_kvq(2, 8, 2, 700, 128, seed=5, dtype=torch.bfloat16)
    for idx in (0, 1):
        dev = torch.device("cuda", idx)
        with torch.cuda.device(dev):
            codec = Codec(dev, 4, True, seed=0, rot_v=setup_golden.z["rotation_s0"], rot_k=setup_golden.z["rotation_s1"])
            store = PackedStore(codec, 2, 2, capacity=704)
            store.pack(k.to(dev), v.to(dev))
            outs.append(store.decode_attn(q.to(dev)).cpu())
            torch.cuda.synchronize(dev)
            assert codec.device_status() == 0
    assert torch.equal(outs[0], outs[1])
    # creating a context on another device, and destroying it whenever the collector gets to it,
    # leaves the process's current device alone
    created = Codec(torch.device("cuda", 1), 4, True, seed=0, rot_v=setup_golden.z["rotation_s0"],
                    rot_k=setup_golden.z["rotation_s1"])
    assert torch.cuda.current_device() == current
    del created, codec, store
    gc.collect()
    assert torch.cuda.current_device() == current


def test_a_sample_of_the_suite_on_the_bounds_checked_build():
    """The same sources built with -DTQ_DEBUG_BOUNDS check every bulk-copy request and every stored
    partial of the decode kernel against the buffers' extents (a violation is recorded as status 6
    and the access dropped).  The ragged-length, many-rows and left-padding cases run on that build
    in a child process; they assert a clean status word themselves."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib = os.path.join(root, "tq_local_b200", "libtq_b200_checked.so")
    assert os.path.isfile(lib), "build it with `python -m tq_local_b200.build --checked`"
    env = dict(os.environ, TQ_B200_LIBRARY=lib)
    out = subprocess.run([sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_gpu_parity.py"), "-m", "gpu",
                          "-x", "-q", "-k", "ragged or seeded or left_padded"], capture_output=True, text=True,
                         timeout=900, env=env, cwd=root)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-2000:]
    assert " passed" in out.stdout and "failed" not in out.stdout
