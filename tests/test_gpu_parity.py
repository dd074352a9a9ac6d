"""GPU parity: the CUDA path (through the C ABI) against the golden vectors of the
reference and against the CPU oracle on the same seeded inputs."""

from __future__ import annotations

import math

import pytest
import torch

from conftest import LAYER_CASES, load_layer_case
from helpers import (assert_codes_match, check_packed, fp16_ulp_diff, load_into_store, make_codec, oracle_params, rel_inf,
                     store_to_layer)
from oracle import tq_oracle as O

pytestmark = pytest.mark.gpu

# Output tolerances, relative to the largest reference magnitude (inf-norm): 1e-5 for fp32 and
# 2e-3 for 16-bit caches.  For 16-bit caches the bound is asserted, with nothing added, on the
# kernels' UNROUNDED result (tq_decode_attn_f32out: same kernels, final cast left out), and the
# usual output must be exactly that result rounded to the query dtype.  Where the ROUNDED output
# is compared with an fp32 reference, the half-ulp of that last rounding (2^-9 for bf16, 2^-12
# for fp16) comes on top (TOL).
KERNEL_TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-3, torch.float16: 2e-3}
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-3 + 2.0 ** -9, torch.float16: 2e-3 + 2.0 ** -12}
WORST = {}  # (variant, dtype) -> worst unrounded error seen in this run (printed by the last test)


def check_unrounded(store, q_dev, got, fused32, groups, **kw):
    """The kernels' own error, apart from the rounding of the output: <= 2e-3, nothing added."""
    if q_dev.dtype == torch.float32:
        return
    raw = store.decode_attn_f32(q_dev, **kw)
    err = rel_inf(raw, fused32)
    key = ("wide" if groups > 4 else "narrow", str(q_dev.dtype).replace("torch.", ""))
    WORST[key] = max(WORST.get(key, 0.0), err)
    assert err <= KERNEL_TOL[q_dev.dtype], (key, err)
    assert torch.equal(raw.to(q_dev.dtype), got), "the usual output is the unrounded one, rounded once"


def _golden_layer(g, p, tag) -> O.PackedLayer:
    f16 = torch.float16
    return O.PackedLayer(p, g.dtype, g.t(f"{tag}_k_codes"), g.t(f"{tag}_k_norms", f16), g.t(f"{tag}_v_codes"),
                         g.t(f"{tag}_v_norms", f16),
                         g.t(f"{tag}_k_signs") if p.use_qjl else None,
                         g.t(f"{tag}_k_rnorms", f16) if p.use_qjl else None)


@pytest.mark.parametrize("case", LAYER_CASES)
def test_pack_and_append_match_reference(setup_golden, case):
    from tq_local_b200.runtime.packed_store import PackedStore

    g = load_layer_case(case)
    bits, qjl = g.i("bits"), bool(g.i("qjl"))
    p = oracle_params(bits, qjl, setup_golden)
    codec = make_codec(bits, qjl, setup_golden)
    S, n_app = g.i("S"), g.i("n_append")
    k, v = g.t("k"), g.t("v")
    kd, vd = k.cuda(), v.cuda()
    store = PackedStore(codec, g.i("B"), g.i("Hkv"), capacity=S)  # forces a capacity growth on append
    store.pack(kd[:, :, :S], vd[:, :, :S])
    check_packed(store, _golden_layer(g, p, "prefill"), k, v, p, case + " prefill")
    assert store.storage_bytes() == g.i("prefill_storage_bytes")
    for t in range(n_app):
        store.pack(kd[:, :, S + t:S + t + 1], vd[:, :, S + t:S + t + 1])
    check_packed(store, _golden_layer(g, p, "appended"), k, v, p, case + " appended")
    assert store.storage_bytes() == g.i("appended_storage_bytes")


@pytest.mark.parametrize("case", LAYER_CASES)
def test_dequant_matches_reference(setup_golden, case):
    from tq_local_b200.runtime.packed_store import PackedStore

    g = load_layer_case(case)
    bits, qjl = g.i("bits"), bool(g.i("qjl"))
    p = oracle_params(bits, qjl, setup_golden)
    codec = make_codec(bits, qjl, setup_golden)
    ref = _golden_layer(g, p, "appended")
    store = PackedStore(codec, g.i("B"), g.i("Hkv"), capacity=ref.seq_len)
    load_into_store(store, ref)
    for which, key in (("keys", "appended_k_dequant"), ("values", "appended_v_dequant")):
        got = store.dequant(which, dtype=g.dtype).cpu().float()
        want = g.t(key).float()
        scale = float(want.abs().max())
        if g.dtype == torch.float32:
            assert float((got - want).abs().max()) <= 2e-6 * scale
        else:
            # at most one 16-bit ulp, and only on a small fraction of elements
            ulp = 2.0 ** (-7 if g.dtype == torch.bfloat16 else -10)
            assert float(((got - want).abs() / want.abs().clamp(min=1e-3)).max()) <= 2.1 * ulp
            assert float((got != want).float().mean()) < 0.02
    # range decode
    part = store.dequant("values", 3, 11, dtype=g.dtype).cpu().float()
    assert torch.equal(part, store.dequant("values", dtype=g.dtype).cpu().float()[:, :, 3:11])


@pytest.mark.parametrize("case", LAYER_CASES)
@pytest.mark.parametrize("tag", ["prefill", "appended"])
def test_decode_attention_matches_reference(setup_golden, case, tag):
    from tq_local_b200.runtime.packed_store import PackedStore

    g = load_layer_case(case)
    bits, qjl = g.i("bits"), bool(g.i("qjl"))
    p = oracle_params(bits, qjl, setup_golden)
    codec = make_codec(bits, qjl, setup_golden)
    ref = _golden_layer(g, p, tag)
    store = PackedStore(codec, g.i("B"), g.i("Hkv"), capacity=64)
    load_into_store(store, ref)
    q = g.t("q")
    groups = g.i("Hq") // g.i("Hkv")
    want32 = g.t(f"{tag}_attn_dequant_f32")
    fused32 = O.attend_rotated_space(q, ref, groups)
    for splits in (1, 2, 5):
        got = store.decode_attn(q.cuda(), splits=splits)
        assert got.dtype == q.dtype and tuple(got.shape) == (g.i("B"), g.i("Hq"), 1, 128)
        # (1) against the reference's fused identity, at the headline tolerance
        assert rel_inf(got, fused32) <= TOL[g.dtype]
        check_unrounded(store, q.cuda(), got, fused32, groups, splits=splits)
        # (2) against dequantise-then-attend: exact-to-tolerance for fp32 caches; for 16-bit caches
        # the reference rounds the dequantised K/V to the cache dtype, which no rotated-space
        # kernel (its own Triton one included) reproduces, so allow that measured gap on top.
        gap = rel_inf(fused32, want32) if g.dtype != torch.float32 else 0.0
        assert rel_inf(got, want32) <= TOL[g.dtype] + gap
    # the reference's own chunked output (query dtype)
    chunked = g.t(f"{tag}_attn_chunked")
    # (both sides are rounded to the query dtype here, hence one more half-ulp)
    half_ulp = {torch.float32: 0.0, torch.bfloat16: 2.0 ** -9, torch.float16: 2.0 ** -12}[g.dtype]
    assert rel_inf(got, chunked) <= TOL[g.dtype] + gap + half_ulp


@pytest.mark.parametrize("case", LAYER_CASES)
def test_dense_tail_attention_matches_reference(setup_golden, case):
    from tq_local_b200.runtime.packed_store import PackedStore

    g = load_layer_case(case)
    bits, qjl = g.i("bits"), bool(g.i("qjl"))
    p = oracle_params(bits, qjl, setup_golden)
    codec = make_codec(bits, qjl, setup_golden)
    S, n_app = g.i("S"), g.i("n_append")
    ref = _golden_layer(g, p, "prefill")
    store = PackedStore(codec, g.i("B"), g.i("Hkv"), capacity=64)
    load_into_store(store, ref)
    k, v, q = g.t("k"), g.t("v"), g.t("q")
    groups = g.i("Hq") // g.i("Hkv")
    got = store.decode_attn(q.cuda(), tail_k=k[:, :, S:S + n_app].cuda(), tail_v=v[:, :, S:S + n_app].cuda(), splits=3)
    want = g.t("densetail_attn_chunked")
    # oracle of the same computation without the 16-bit rounding of dequantised K/V
    kd = O.dequant_keys(ref)
    gap = 0.0
    if g.dtype != torch.float32:
        # gap between the reference's two formulations on the packed part
        gap = rel_inf(O.attend_rotated_space(q, ref, groups), O.attend_dequant(q, ref, groups))
    assert rel_inf(got, want) <= TOL[g.dtype] + gap
    del kd


@pytest.mark.parametrize("bits,qjl,dtype,B,Hq,Hkv,N", [
    (4, True, torch.bfloat16, 2, 8, 2, 1500),
    (4, False, torch.float32, 1, 32, 8, 1027),
    (3, True, torch.bfloat16, 1, 14, 2, 2049),
    (3, False, torch.float16, 2, 4, 4, 513),
    (2, True, torch.bfloat16, 1, 8, 1, 777),
    (2, False, torch.float32, 1, 6, 2, 300),
    (4, True, torch.float32, 1, 16, 2, 640),
    (2, True, torch.bfloat16, 2, 8, 2, 600),
    (3, True, torch.float16, 1, 4, 4, 300),
    # more than four query heads per KV head (the kernel's wide variant)
    (4, True, torch.float16, 1, 10, 2, 1100),
    (4, False, torch.bfloat16, 2, 16, 2, 900),
    (3, False, torch.bfloat16, 1, 12, 2, 1300),
    (4, True, torch.bfloat16, 2, 28, 4, 2100),
    # more (batch, KV head) rows than SMs: a CTA's chunk spans several rows
    (4, True, torch.bfloat16, 40, 8, 4, 600),
    (3, True, torch.float16, 23, 14, 7, 200),
])
def test_seeded_layer_against_oracle(setup_golden, bits, qjl, dtype, B, Hq, Hkv, N):
    """Larger seeded inputs: encode on the GPU, compare codes with the oracle, then
    decode from the GPU's own cache and compare with the oracle's attention over it."""
    from tq_local_b200.runtime.packed_store import PackedStore

    torch.set_num_threads(max(1, torch.get_num_threads()))
    p = oracle_params(bits, qjl, setup_golden)
    codec = make_codec(bits, qjl, setup_golden)
    k, v, q = O.synth_kvq(B, Hq, Hkv, N, 128, seed=100 + N, dtype=dtype)
    store = PackedStore(codec, B, Hkv, capacity=N + 8)
    # K/V arrive as transposed views, like HF attention modules hand them over
    kd = k.cuda().transpose(1, 2).contiguous().transpose(1, 2)
    vd = v.cuda().transpose(1, 2).contiguous().transpose(1, 2)
    assert Hkv == 1 or not kd.is_contiguous()
    store.pack(kd, vd)
    ref = O.pack_layer(k, v, p)
    check_packed(store, ref, k, v, p, f"seeded b{bits} qjl{qjl}")
    mine = store_to_layer(store, p, dtype)  # attention parity is judged on the GPU's own codes
    groups = Hq // Hkv
    fused32 = O.attend_rotated_space(q, mine, groups)
    want32 = O.attend_dequant(q, mine, groups)
    got = store.decode_attn(q.cuda())
    assert rel_inf(got, fused32) <= TOL[dtype]
    check_unrounded(store, q.cuda(), got, fused32, groups)
    gap = rel_inf(fused32, want32) if dtype != torch.float32 else 0.0
    assert rel_inf(got, want32) <= TOL[dtype] + gap
    # split count must not change the answer beyond rounding
    a = store.decode_attn(q.cuda(), splits=1).float()
    b = store.decode_attn(q.cuda(), splits=7).float()
    assert rel_inf(a, b.cpu()) <= TOL[dtype]
    assert codec.device_status() == 0  # no bounded wait inside a kernel ever ran out


@pytest.mark.parametrize("n", [1, 2, 31, 32, 33, 63, 64, 65, 127, 129])
def test_ragged_lengths(setup_golden, n):
    from tq_local_b200.runtime.packed_store import PackedStore

    p = oracle_params(4, True, setup_golden)
    codec = make_codec(4, True, setup_golden)
    k, v, q = O.synth_kvq(1, 8, 2, n, 128, seed=n, dtype=torch.float32)
    store = PackedStore(codec, 1, 2, capacity=n)
    store.pack(k.cuda(), v.cuda())
    mine = store_to_layer(store, p, torch.float32)
    for splits in (1, 3, 9):
        got = store.decode_attn(q.cuda(), splits=splits)
        assert rel_inf(got, O.attend_dequant(q, mine, 4)) <= 1e-5


def test_zero_vectors_and_append_equivalence(setup_golden):
    """A zero vector keeps norm 1.0 (reference: safe_norm) and packing S tokens at once
    equals packing them one at a time."""
    from tq_local_b200.runtime.packed_store import PackedStore

    codec = make_codec(3, True, setup_golden)
    p = oracle_params(3, True, setup_golden)
    k, v, _ = O.synth_kvq(2, 4, 2, 20, 128, seed=9, dtype=torch.bfloat16)
    k[0, 1, 5] = 0
    v[1, 0, 7] = 0
    a = PackedStore(codec, 2, 2, capacity=32)
    a.pack(k.cuda(), v.cuda())
    b = PackedStore(codec, 2, 2, capacity=8)
    for t in range(20):
        b.pack(k[:, :, t:t + 1].cuda(), v[:, :, t:t + 1].cuda())
    for x, y in zip(a.streams(), b.streams()):
        assert torch.equal(x[:, :, :20], y[:, :, :20])
    assert float(a.k_norms[0, 1, 5]) == 1.0 and float(a.v_norms[1, 0, 7]) == 1.0
    ref = O.pack_layer(k, v, p)
    check_packed(a, ref, k, v, p, "zero-vector case")


def test_argument_errors(setup_golden):
    from tq_local_b200.runtime import ffi
    from tq_local_b200.runtime.packed_store import PackedStore

    codec = make_codec(4, False, setup_golden)
    store = PackedStore(codec, 1, 2, capacity=16)
    k = torch.zeros(1, 2, 4, 128, device="cuda")
    with pytest.raises(ValueError):
        store.pack(k, k[:, :1])
    with pytest.raises(ValueError):
        store.pack(torch.zeros(1, 3, 4, 128, device="cuda"), torch.zeros(1, 3, 4, 128, device="cuda"))
    store.pack(k, k)
    with pytest.raises(ffi.TQError):  # 5 query heads do not divide over 2 KV heads
        store.decode_attn(torch.zeros(1, 5, 1, 128, device="cuda"))
    with pytest.raises(ffi.TQError):  # more than 8 query heads per KV head
        store.decode_attn(torch.zeros(1, 18, 1, 128, device="cuda"))
    with pytest.raises(NotImplementedError):
        make_codec(5, False, setup_golden)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_host_buffer_decode_step_matches_device_calls(setup_golden, dtype):
    """tq_decode_step_host (host tensors in, host tensor out) == append + decode on device tensors."""
    from tq_local_b200.runtime.packed_store import PackedStore

    codec = make_codec(4, True, setup_golden)
    k, v, q = O.synth_kvq(2, 8, 2, 130, 128, seed=77, dtype=dtype)
    a = PackedStore(codec, 2, 2, capacity=160)
    b = PackedStore(codec, 2, 2, capacity=160)
    a.pack(k[:, :, :128].cuda(), v[:, :, :128].cuda())
    b.pack(k[:, :, :128].cuda(), v[:, :, :128].cuda())
    for t in (128, 129):
        kn, vn = k[:, :, t:t + 1].contiguous(), v[:, :, t:t + 1].contiguous()
        out_h = torch.empty(2, 8, 1, 128, dtype=dtype).pin_memory()
        a.decode_step_host(q.contiguous().pin_memory(), kn.pin_memory(), vn.pin_memory(), out_h)
        b.pack(kn.cuda(), vn.cuda())
        want = b.decode_attn(q.cuda())
        torch.cuda.synchronize()
        assert a.length == b.length == t + 1
        assert torch.equal(out_h, want.cpu())
    for x, y in zip(a.streams(), b.streams()):
        assert torch.equal(x[:, :, :130], y[:, :, :130])


def test_bound_host_step_reuses_buffers_across_capacity_growth(setup_golden):
    """bind_host_step: buffers checked once, one call per token, including a step that has to grow
    the cache; pageable (not page-locked) buffers take the staged-copy route."""
    from tq_local_b200.runtime.packed_store import PackedStore

    codec = make_codec(3, True, setup_golden)
    k, v, _ = O.synth_kvq(1, 4, 2, 40, 128, seed=78, dtype=torch.float16)
    g = torch.Generator().manual_seed(3)
    for pinned in (True, False):
        a = PackedStore(codec, 1, 2, capacity=32)
        b = PackedStore(codec, 1, 2, capacity=64)
        a.pack(k[:, :, :30].cuda(), v[:, :, :30].cuda())
        b.pack(k[:, :, :30].cuda(), v[:, :, :30].cuda())
        bufs = [torch.empty(1, 4, 1, 128, dtype=torch.float16), torch.empty(1, 2, 1, 128, dtype=torch.float16),
                torch.empty(1, 2, 1, 128, dtype=torch.float16), torch.empty(1, 4, 1, 128, dtype=torch.float16)]
        if pinned:
            bufs = [t.pin_memory() for t in bufs]
        hq, hk, hv, hout = bufs
        step = a.bind_host_step(hq, hk, hv, hout)
        for t in range(30, 40):  # crosses the capacity of 32
            q = torch.randn(1, 4, 1, 128, generator=g).to(torch.float16)
            hq.copy_(q), hk.copy_(k[:, :, t:t + 1]), hv.copy_(v[:, :, t:t + 1])
            step()
            b.pack(k[:, :, t:t + 1].cuda(), v[:, :, t:t + 1].cuda())
            want = b.decode_attn(q.cuda())
            torch.cuda.synchronize()
            assert torch.equal(hout, want.cpu()), (pinned, t)
        assert a.length == 40 and a.capacity >= 40


@pytest.mark.parametrize("Hq", [8, 14])
def test_decode_step_with_device_length_matches_and_replays_from_a_cuda_graph(setup_golden, Hq):
    """tq_decode_step_dev: the append position / sequence length is a device scalar, so one
    recorded launch sequence serves every token.  Results must equal the host-length path bit
    for bit, eagerly and when replayed from a CUDA graph."""
    from tq_local_b200.runtime.packed_store import PackedStore

    codec = make_codec(4, True, setup_golden)
    B, Hkv, N0, steps = 2, 2, 700, 6
    k, v, _ = O.synth_kvq(B, Hq, Hkv, N0 + steps, 128, seed=21, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(5)
    qs = torch.randn(steps, B, Hq, 1, 128, generator=g).to(torch.bfloat16).cuda()
    k, v = k.cuda(), v.cuda()
    ref = PackedStore(codec, B, Hkv, capacity=1024)
    dev = PackedStore(codec, B, Hkv, capacity=1024)
    ref.pack(k[:, :, :N0], v[:, :, :N0])
    dev.pack(k[:, :, :N0], v[:, :, :N0])
    want = []
    for t in range(steps):
        ref.pack(k[:, :, N0 + t:N0 + t + 1], v[:, :, N0 + t:N0 + t + 1])
        want.append(ref.decode_attn(qs[t], splits=dev.suggest_splits(dev.capacity)).clone())

    pos = torch.tensor([N0], dtype=torch.int32, device="cuda")
    sq = torch.empty_like(qs[0])
    sk = torch.empty(B, Hkv, 1, 128, dtype=torch.bfloat16, device="cuda")
    sv = torch.empty_like(sk)
    sout = torch.empty_like(qs[0])

    def load(t):
        sq.copy_(qs[t]), sk.copy_(k[:, :, N0 + t:N0 + t + 1]), sv.copy_(v[:, :, N0 + t:N0 + t + 1])

    load(0)
    dev.decode_step_dev(sq, sk, sv, pos, out=sout)  # eager
    pos.add_(1)
    assert torch.equal(sout, want[0])
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    load(1)
    with torch.cuda.graph(graph):
        dev.decode_step_dev(sq, sk, sv, pos, out=sout)
        pos.add_(1)
    for t in range(1, steps):
        load(t)
        graph.replay()
        assert torch.equal(sout, want[t]), f"step {t}"
    assert int(pos.item()) == N0 + steps
    dev.length = N0 + steps
    for a, b in zip(ref.streams(), dev.streams()):
        assert torch.equal(a[:, :, :N0 + steps], b[:, :, :N0 + steps])
    assert codec.device_status() == 0


def test_decode_step_dev_drops_appends_past_capacity_and_reports_it(setup_golden):
    from tq_local_b200.runtime.packed_store import PackedStore

    codec = make_codec(4, True, setup_golden)
    B, Hq, Hkv = 1, 4, 1
    k, v, q = O.synth_kvq(B, Hq, Hkv, 64, 128, seed=22, dtype=torch.bfloat16)
    store = PackedStore(codec, B, Hkv, capacity=64)
    store.pack(k.cuda(), v.cuda())
    before = [t.clone() for t in store.streams()]
    pos = torch.tensor([store.capacity], dtype=torch.int32, device="cuda")  # no room left
    out = store.decode_step_dev(q.cuda(), k[:, :, :1].cuda(), v[:, :, :1].cuda(), pos)
    torch.cuda.synchronize()
    assert codec.device_status() == 4
    for a, b in zip(before, store.streams()):
        assert torch.equal(a, b)  # nothing was written
    assert torch.isfinite(out.float()).all()
    # the status word is sticky by design; a fresh context starts clean


def test_zz_report_worst_unrounded_error():
    """Runs last in this file: the worst error of the unrounded outputs seen above, per kernel
    variant (G <= 4 "narrow", G > 4 "wide") and dtype, all of which passed the 2e-3 bound."""
    assert WORST, "no 16-bit case ran"
    for key in sorted(WORST):
        print(f"worst unrounded attention error {key}: {WORST[key]:.3e}")
        assert WORST[key] <= 2e-3


@pytest.mark.parametrize("bits,qjl,dtype,Hq,Hkv", [
    (4, True, torch.bfloat16, 8, 2),    # tensor-core kernel, four heads per KV head
    (4, True, torch.bfloat16, 14, 2),   # wide variant
    (3, True, torch.float16, 4, 2),
    (4, False, torch.float32, 8, 2),    # fp32-exact kernel
])
def test_left_padded_rows_attend_from_their_first_real_token(setup_golden, bits, qjl, dtype, Hq, Hkv):
    """``seq_start``: row b attends tokens [start_b, N).  Checked against the oracle's attention
    over each row's own slice of the cache; starts fall on, next to and far from the kernel's
    512-token steps, and one row has no padding."""
    from tq_local_b200.runtime.packed_store import PackedStore

    p = oracle_params(bits, qjl, setup_golden)
    codec = make_codec(bits, qjl, setup_golden)
    starts = [0, 5, 511, 512, 700, 1499]
    B, N = len(starts), 1500
    k, v, q = O.synth_kvq(B, Hq, Hkv, N, 128, seed=77, dtype=dtype)
    store = PackedStore(codec, B, Hkv, capacity=N + 8)
    store.pack(k.cuda(), v.cuda())
    groups = Hq // Hkv
    for splits in (1, 4):
        store.set_seq_start(None)
        unmasked = store.decode_attn(q.cuda(), splits=splits).clone()
        store.set_seq_start(torch.tensor(starts, dtype=torch.int32, device="cuda"))
        got = store.decode_attn(q.cuda(), splits=splits)
        raw = got if dtype == torch.float32 else store.decode_attn_f32(q.cuda(), splits=splits)
        for b, s0 in enumerate(starts):
            sl = lambda t: None if t is None else t[b:b + 1, :, s0:N].contiguous().cpu()
            mine = O.PackedLayer(p, dtype, sl(store.k_codes), sl(store.k_norms), sl(store.v_codes), sl(store.v_norms),
                                 sl(store.k_signs), sl(store.k_rnorms))
            want = O.attend_rotated_space(q[b:b + 1], mine, groups)
            assert rel_inf(raw[b:b + 1], want) <= KERNEL_TOL[dtype], (b, s0, splits)
        assert torch.equal(got[0], unmasked[0])  # the unpadded row is untouched by the others' offsets
    store.set_seq_start(None)
    assert torch.equal(store.decode_attn(q.cuda(), splits=4), unmasked)
    # the device-length step honours the offsets too
    if dtype != torch.float32:
        store.set_seq_start(torch.tensor(starts, dtype=torch.int32, device="cuda"))
        ref_store = PackedStore(codec, B, Hkv, capacity=N + 8)
        ref_store.pack(k.cuda(), v.cuda())
        ref_store.set_seq_start(torch.tensor(starts, dtype=torch.int32, device="cuda"))
        k1, v1, _ = O.synth_kvq(B, Hq, Hkv, 1, 128, seed=78, dtype=dtype)
        ref_store.pack(k1.cuda(), v1.cuda())
        want = ref_store.decode_attn(q.cuda())
        pos = torch.tensor([N], dtype=torch.int32, device="cuda")
        got = store.decode_step_dev(q.cuda(), k1.cuda(), v1.cuda(), pos)
        assert rel_inf(got, want.float().cpu()) <= 2.0 ** -7
    assert codec.device_status() == 0
