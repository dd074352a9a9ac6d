"""GPU: the benchmark's five workload shapes at their full stated sizes (batch, heads, context),
checked against the CPU oracle on whole sequences and through size-independent properties."""

from __future__ import annotations

import math

import pytest
import torch

from helpers import StoreView, check_packed, make_codec, oracle_params, rel_inf, store_to_layer
from oracle import tq_oracle as O

pytestmark = pytest.mark.gpu


def _synth_gpu(shape, seed, dtype, lognormal=True, norm_range=None):
    """iid N(0,1) coordinates with lognormal(0, 0.5) per-token norms, or (``norm_range``) unit
    directions times a uniform norm, generated on the device."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(shape, device="cuda", generator=g)
    if norm_range is not None:
        lo, hi = norm_range
        x = x / x.norm(dim=-1, keepdim=True)
        x = x * (lo + (hi - lo) * torch.rand(*shape[:-1], 1, device="cuda", generator=g))
    elif lognormal:
        x = x * torch.exp(0.5 * torch.randn(*shape[:-1], 1, device="cuda", generator=g))
    return x.to(dtype)


def _slice_layer(store, p, dtype, b, n=None):
    """Batch entry ``b`` (all KV heads) of the GPU's packed cache as an oracle layer."""
    n = store.length if n is None else n
    sl = lambda t: None if t is None else t[b:b + 1, :, :n].contiguous().cpu()
    return O.PackedLayer(p, dtype, sl(store.k_codes), sl(store.k_norms), sl(store.v_codes), sl(store.v_norms),
                         sl(store.k_signs), sl(store.k_rnorms))


def _check_sequence_codes(store, p, k, v, b, lo, hi, what):
    """Codes, norms, sign sketches and residual norms of tokens [lo, hi) of batch entry ``b`` (every
    KV head) against the oracle's encoding of the same vectors, by the same rules as the small
    cases: identical outside the 1e-6 boundary band."""
    kc, vc = k[b:b + 1, :, lo:hi].cpu().contiguous(), v[b:b + 1, :, lo:hi].cpu().contiguous()
    check_packed(StoreView(store, b, lo, hi), O.pack_layer(kc, vc, p), kc, vc, p, what)


def _dense_attention(q, k, v, groups):
    kf = k.float().repeat_interleave(groups, dim=1)
    vf = v.float().repeat_interleave(groups, dim=1)
    w = torch.softmax((q.float() @ kf.transpose(-1, -2)) / math.sqrt(128), dim=-1)
    return w @ vf


def test_config1_fp32_4bit_mse_full_shape(setup_golden):
    """Config 1: batch 1, 32 / 8 heads, 4096 tokens, fp32, Q_mse 4-bit, seed 0."""
    from tq_local_b200.runtime.packed_store import PackedStore

    p = oracle_params(4, False, setup_golden)
    codec = make_codec(4, False, setup_golden)
    k, v, q = O.synth_kvq(1, 32, 8, 4096, 128, seed=0, dtype=torch.float32)
    store = PackedStore(codec, 1, 8, capacity=4096)
    store.pack(k.cuda(), v.cuda())
    assert store.storage_bytes() == 4_325_376
    ref = O.pack_layer(k, v, p)
    # tensor-core encoder vs the reference quantiser: identical outside the 1e-6 boundary band
    from helpers import assert_codes_match
    assert_codes_match(store.k_codes, ref.k_codes, k, p.rot_k, p.bnd_k, 4, "config 1 keys")
    assert_codes_match(store.v_codes, ref.v_codes, v, p.rot_v, p.bnd_v, 4, "config 1 values")
    mine = store_to_layer(store, p, torch.float32)
    got = store.decode_attn(q.cuda())
    assert rel_inf(got, O.attend_dequant(q, mine, 4)) <= 1e-5
    assert rel_inf(got, O.attend_chunked(q, mine, 4)) <= 1e-5


def test_config2_full_shape_codes_and_attention(setup_golden):
    """The headline workload at its full size: bf16, batch 8, 32 / 8 heads, 32768 tokens, 4-bit
    Q_prod.  One whole sequence (all 8 KV heads x 32768 tokens) is compared code for code with the
    oracle, and the attention output of all 32 heads of that sequence with the oracle's
    attention over the GPU's own codes."""
    from tq_local_b200.runtime.packed_store import PackedStore

    codec = make_codec(4, True, setup_golden)
    p = oracle_params(4, True, setup_golden)
    B, Hq, Hkv, N = 8, 32, 8, 32768
    k = _synth_gpu((B, Hkv, N, 128), 1, torch.bfloat16)
    v = _synth_gpu((B, Hkv, N, 128), 2, torch.bfloat16)
    q = _synth_gpu((B, Hq, 1, 128), 3, torch.bfloat16, lognormal=False)
    store = PackedStore(codec, B, Hkv, capacity=N + 8)
    store.pack(k, v)
    assert store.storage_bytes() == 134 * B * Hkv * N == 281_018_368
    _check_sequence_codes(store, p, k, v, 5, 0, N, "full-size sequence 5")
    # reconstruction quality gates of the reference's smoke test (4-bit: cosine >= 0.990 for
    # Q_mse values; Q_prod keys ~0.975 by the reference's own account)
    cos = torch.nn.functional.cosine_similarity
    vd = store.dequant("values", 0, 4096, dtype=torch.bfloat16).float()
    kd = store.dequant("keys", 0, 4096, dtype=torch.bfloat16).float()
    assert float(cos(vd.reshape(-1, 128), v[:, :, :4096].float().reshape(-1, 128), dim=-1).mean()) >= 0.990
    assert float(cos(kd.reshape(-1, 128), k[:, :, :4096].float().reshape(-1, 128), dim=-1).mean()) >= 0.970
    del vd, kd
    out = store.decode_attn(q)
    raw = store.decode_attn_f32(q)
    assert torch.equal(raw.to(torch.bfloat16), out)
    # quantised attention tracks dense attention (loose sanity bound: iid Gaussian keys with
    # lognormal norms give a peaked softmax, the hardest case for a 3-bit key quantiser)
    dense = torch.cat([_dense_attention(q[b:b + 1], k[b:b + 1], v[b:b + 1], Hq // Hkv) for b in range(B)])
    assert float(cos(out.float().reshape(-1, 128), dense.reshape(-1, 128), dim=-1).mean()) > 0.8
    # split invariance at full length
    assert rel_inf(store.decode_attn_f32(q, splits=2), store.decode_attn_f32(q, splits=9).cpu()) <= 2e-3
    # every head of two sequences against the oracle on the GPU's own codes: 2e-3, nothing added
    for b in (5, 0):
        want = O.attend_rotated_space(q[b:b + 1].cpu(), _slice_layer(store, p, torch.bfloat16, b), 4)
        assert rel_inf(raw[b:b + 1], want) <= 2e-3, b
        assert rel_inf(out[b:b + 1], want) <= 2e-3 + 2.0 ** -9, b
    assert codec.device_status() == 0


def test_config3_full_shape_three_bit_long_context_256_appends(setup_golden):
    """3-bit Q_prod (2-bit keys + QJL, 3-bit values) at batch 4 x 8 KV heads x 131072 tokens, then 256
    decode steps that each re-quantise the new token into the cache.  Earlier tokens must not
    move (O(1) append), the appended tokens must equal the oracle's encoding of the same vectors,
    and the last step's attention must match the oracle over the GPU's codes."""
    from tq_local_b200.runtime.packed_store import PackedStore

    codec = make_codec(3, True, setup_golden)
    p = oracle_params(3, True, setup_golden)
    B, Hq, Hkv, N, steps = 4, 32, 8, 131072, 256
    store = PackedStore(codec, B, Hkv, capacity=N + steps)
    k = _synth_gpu((B, Hkv, N + steps, 128), 4, torch.bfloat16)
    v = _synth_gpu((B, Hkv, N + steps, 128), 5, torch.bfloat16)
    q = _synth_gpu((B, Hq, 1, 128), 6, torch.bfloat16, lognormal=False)
    store.pack(k[:, :, :N], v[:, :, :N])
    assert store.storage_bytes() == 102 * B * Hkv * N == 427_819_008
    # fingerprints of the history instead of a full copy: byte sums per stream and row
    fingerprint = lambda: [t[:, :, :N].reshape(B, Hkv, -1).view(torch.uint8).to(torch.int64).sum(-1) for t in store.streams()]
    before, sample = fingerprint(), [t[2, 3, 1000:1064].clone() for t in store.streams()]
    ptrs = [t.data_ptr() for t in store.streams()]
    pos = torch.tensor([N], dtype=torch.int32, device="cuda")
    half = steps // 2
    for t in range(half):  # host-numbered appends ...
        store.pack(k[:, :, N + t:N + t + 1], v[:, :, N + t:N + t + 1])
        out = store.decode_attn(q)
    pos.fill_(N + half)
    for t in range(half, steps):  # ... and the device-length step that a recorded decode loop replays
        out = store.decode_step_dev(q, k[:, :, N + t:N + t + 1], v[:, :, N + t:N + t + 1], pos)
        pos.add_(1)
    store.length = N + steps
    assert [t.data_ptr() for t in store.streams()] == ptrs  # no reallocation, no copy of history
    for a, b in zip(before, fingerprint()):
        assert torch.equal(a, b)
    for a, t in zip(sample, store.streams()):
        assert torch.equal(a, t[2, 3, 1000:1064])
    assert store.storage_bytes() == 102 * B * Hkv * (N + steps)
    # all 256 appended tokens of every row against the oracle's encoding of the same vectors
    for b in range(B):
        _check_sequence_codes(store, p, k, v, b, N, N + steps, f"appended tokens of sequence {b}")
    # the last step attended over N + steps tokens: all heads of one sequence against the oracle
    raw = store.decode_attn_f32(q)
    assert torch.equal(raw.to(torch.bfloat16), out)
    want = O.attend_rotated_space(q[1:2].cpu(), _slice_layer(store, p, torch.bfloat16, 1), 4)
    assert rel_inf(raw[1:2], want) <= 2e-3
    assert codec.device_status() == 0


def test_config4_full_shape_qwen_seven_heads_per_kv_head_and_norm_guard(setup_golden):
    """28 / 4 heads (7 query heads per KV head), batch 8, 32768 tokens, asymmetric norms: the norm
    guard keeps the layer with key norms U[100, 400] dense and packs the ordinary one, which goes
    through the wide-group kernel."""
    from tq_local_b200.runtime.packed_qmse_cache import build_packed_mse_cache

    B, Hq, Hkv, N = 8, 28, 4, 32768
    k_hi = _synth_gpu((B, Hkv, N, 128), 8, torch.bfloat16, norm_range=(100.0, 400.0))
    v_hi = _synth_gpu((B, Hkv, N, 128), 9, torch.bfloat16, norm_range=(1.0, 10.0))
    k_lo = _synth_gpu((B, Hkv, N, 128), 10, torch.bfloat16)
    v_lo = _synth_gpu((B, Hkv, N, 128), 11, torch.bfloat16)
    q = _synth_gpu((B, Hq, 1, 128), 12, torch.bfloat16, lognormal=False)
    cache = build_packed_mse_cache([(k_hi, v_hi), (k_lo, v_lo)], bits=4, use_qjl_keys=True,
                                   quantize_decode=True, norm_guard=True)
    dense_layer, packed_layer = cache.layers
    assert dense_layer._force_dense and not packed_layer._force_dense
    assert dense_layer.storage_bytes() == 2 * B * Hkv * N * 128 * 2 == 536_870_912
    assert packed_layer.storage_bytes() == 134 * B * Hkv * N == 140_509_184
    out = packed_layer.attend(q)
    codec = packed_layer.codec
    p = O.QuantParams.build(128, 4, True, seed=0, rot_v=codec.rot_v, rot_k=codec.rot_k)
    _check_sequence_codes(packed_layer.store, p, k_lo, v_lo, 3, 0, N, "packed layer, sequence 3")
    raw = packed_layer.store.decode_attn_f32(q)
    assert torch.equal(raw.to(torch.bfloat16), out)
    for b in (3, 7):
        want = O.attend_rotated_space(q[b:b + 1].cpu(), _slice_layer(packed_layer.store, p, torch.bfloat16, b), 7)
        assert rel_inf(raw[b:b + 1], want) <= 2e-3, b
    # dense layer: the attention backend falls back to SDPA with the full dense K/V
    from tq_local_b200.runtime.attention import turboquant_attention_forward

    class Mod:
        num_key_value_groups = 7
        _tq_cache_layer = dense_layer
    o, _ = turboquant_attention_forward(Mod(), q, k_hi, v_hi, None)
    want_d = torch.cat([_dense_attention(q[b:b + 1], k_hi[b:b + 1], v_hi[b:b + 1], 7) for b in range(B)])
    assert rel_inf(o.transpose(1, 2), want_d.cpu()) < 2e-2
    assert codec.device_status() == 0
