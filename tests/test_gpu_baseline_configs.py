"""GPU: the BASELINE configurations at (near) full size, checked through size-independent
properties and against the CPU oracle on the GPU's own packed codes."""

from __future__ import annotations

import math

import pytest
import torch

from helpers import make_codec, oracle_params, rel_inf, store_to_layer
from oracle import tq_oracle as O

pytestmark = pytest.mark.gpu


def _synth_gpu(shape, seed, dtype, lognormal=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(shape, device="cuda", generator=g)
    if lognormal:
        x = x * torch.exp(0.5 * torch.randn(*shape[:-1], 1, device="cuda", generator=g))
    return x.to(dtype)


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


def test_config2_shape_properties(setup_golden):
    """Config 2 (bf16, 32 / 8 heads, 32768 tokens, 4-bit Q_prod) at batch 2."""
    from tq_local_b200.runtime.packed_store import PackedStore

    codec = make_codec(4, True, setup_golden)
    p = oracle_params(4, True, setup_golden)
    B, Hq, Hkv, N = 2, 32, 8, 32768
    k = _synth_gpu((B, Hkv, N, 128), 1, torch.bfloat16)
    v = _synth_gpu((B, Hkv, N, 128), 2, torch.bfloat16)
    q = _synth_gpu((B, Hq, 1, 128), 3, torch.bfloat16, lognormal=False)
    store = PackedStore(codec, B, Hkv, capacity=N + 8)
    store.pack(k, v)
    assert store.storage_bytes() == 134 * B * Hkv * N
    # reconstruction quality gates of the reference's smoke test (4-bit: cosine >= 0.990 for
    # Q_mse values; Q_prod keys ~0.975 by the reference's own account)
    cos = torch.nn.functional.cosine_similarity
    vd = store.dequant("values", 0, 4096, dtype=torch.bfloat16).float()
    kd = store.dequant("keys", 0, 4096, dtype=torch.bfloat16).float()
    assert float(cos(vd.reshape(-1, 128), v[:, :, :4096].float().reshape(-1, 128), dim=-1).mean()) >= 0.990
    assert float(cos(kd.reshape(-1, 128), k[:, :, :4096].float().reshape(-1, 128), dim=-1).mean()) >= 0.970
    out = store.decode_attn(q)
    dense = _dense_attention(q, k, v, Hq // Hkv)
    # quantised attention tracks dense attention (loose sanity bound: iid Gaussian keys with
    # lognormal norms give a peaked softmax, the hardest case for a 3-bit key quantiser)
    assert float(cos(out.float().reshape(-1, 128), dense.reshape(-1, 128), dim=-1).mean()) > 0.8
    # split invariance at full length
    assert rel_inf(store.decode_attn(q, splits=2), store.decode_attn(q, splits=9).float().cpu()) <= 2e-3 + 2.0 ** -8
    # oracle on the GPU's own codes for one (batch, KV head) slice
    sl = lambda t: None if t is None else t[1:2, 3:4, :N].contiguous().cpu()
    mine = O.PackedLayer(p, torch.bfloat16, sl(store.k_codes), sl(store.k_norms), sl(store.v_codes), sl(store.v_norms),
                         sl(store.k_signs), sl(store.k_rnorms))
    q_sl = q[1:2, 12:16].cpu()
    want = O.attend_rotated_space(q_sl, mine, 4)
    assert rel_inf(out[1:2, 12:16], want) <= 2e-3 + 2.0 ** -9
    assert codec.device_status() == 0


def test_config3_three_bit_long_context_with_appends(setup_golden):
    """Config 3 shape at batch 1 x 2 KV heads: 3-bit Q_prod (2-bit keys + QJL, 3-bit values),
    131072 tokens, then quantised appends; earlier tokens must not move (O(1) append)."""
    from tq_local_b200.runtime.packed_store import PackedStore

    codec = make_codec(3, True, setup_golden)
    p = oracle_params(3, True, setup_golden)
    B, Hq, Hkv, N, steps = 1, 8, 2, 131072, 16
    k = _synth_gpu((B, Hkv, N + steps, 128), 4, torch.bfloat16)
    v = _synth_gpu((B, Hkv, N + steps, 128), 5, torch.bfloat16)
    q = _synth_gpu((B, Hq, 1, 128), 6, torch.bfloat16, lognormal=False)
    store = PackedStore(codec, B, Hkv, capacity=N + steps)
    store.pack(k[:, :, :N], v[:, :, :N])
    assert store.storage_bytes() == 102 * B * Hkv * N
    before = [t[:, :, :N].clone() for t in store.streams()]
    ptrs = [t.data_ptr() for t in store.streams()]
    for t in range(steps):
        store.pack(k[:, :, N + t:N + t + 1], v[:, :, N + t:N + t + 1])
        out = store.decode_attn(q)
    assert [t.data_ptr() for t in store.streams()] == ptrs  # no reallocation, no copy of history
    for a, b in zip(before, store.streams()):
        assert torch.equal(a, b[:, :, :N])
    assert store.storage_bytes() == 102 * B * Hkv * (N + steps)
    mine = store_to_layer(store, p, torch.bfloat16)
    want = O.attend_rotated_space(q.cpu(), mine, 4)
    assert rel_inf(out, want) <= 2e-3 + 2.0 ** -9
    # the appended tokens equal a one-shot encode of the same vectors, up to the boundary band
    ref_tail = O.pack_layer(k[:, :, N:].cpu(), v[:, :, N:].cpu(), p)
    from helpers import assert_codes_match
    assert_codes_match(store.v_codes[:, :, N:N + steps], ref_tail.v_codes, v[:, :, N:].cpu(), p.rot_v, p.bnd_v, 3, "tail")
    assert codec.device_status() == 0


def test_config4_qwen_shape_seven_heads_per_kv_head_and_norm_guard(setup_golden):
    """Config 4: 28 / 4 heads (7 query heads per KV head), asymmetric norms; the norm guard keeps
    the high-norm layer dense and the packed layer goes through the wide-group kernel."""
    from tq_local_b200.runtime.packed_qmse_cache import build_packed_mse_cache

    B, Hq, Hkv, N = 2, 28, 4, 4096
    k_hi, v_hi, _ = O.synth_kvq(B, Hq, Hkv, N, 128, seed=8, dtype=torch.bfloat16, norm_mode="asym")
    k_lo, v_lo, q = O.synth_kvq(B, Hq, Hkv, N, 128, seed=9, dtype=torch.bfloat16)
    cache = build_packed_mse_cache([(k_hi.cuda(), v_hi.cuda()), (k_lo.cuda(), v_lo.cuda())], bits=4, use_qjl_keys=True,
                                   quantize_decode=True, norm_guard=True)
    dense_layer, packed_layer = cache.layers
    assert dense_layer._force_dense and not packed_layer._force_dense
    assert dense_layer.storage_bytes() == 2 * B * Hkv * N * 128 * 2
    out = packed_layer.attend(q.cuda())
    codec = packed_layer.codec
    p = O.QuantParams.build(128, 4, True, seed=0, rot_v=codec.rot_v, rot_k=codec.rot_k)
    mine = store_to_layer(packed_layer.store, p, torch.bfloat16)
    want = O.attend_rotated_space(q, mine, 7)
    assert rel_inf(out, want) <= 2e-3 + 2.0 ** -9
    # dense layer: the attention backend falls back to SDPA with the full dense K/V
    from tq_local_b200.runtime.attention import turboquant_attention_forward

    class Mod:
        num_key_value_groups = 7
        _tq_cache_layer = dense_layer
    o, _ = turboquant_attention_forward(Mod(), q.cuda(), k_hi.cuda(), v_hi.cuda(), None)
    want_d = _dense_attention(q.cuda(), k_hi.cuda(), v_hi.cuda(), 7)
    assert rel_inf(o.transpose(1, 2), want_d.cpu()) < 2e-2
