"""GPU: the reference-facing API end to end on a tiny random Llama, against the golden run
of the reference (tests/golden/e2e_tiny_llama.npz), plus cache-layer behaviour on device."""

from __future__ import annotations

import pytest
import torch

from conftest import Golden
from oracle import tq_oracle as O

pytestmark = pytest.mark.gpu


class StubTokenizer:
    eos_token_id = None

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(int(i)) for i in ids)

    def encode(self, text, add_special_tokens=False):
        return [int(t) for t in text.split()]


def _tiny_model(dtype=torch.float32):
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=512)
    return LlamaForCausalLM(cfg).eval().to("cuda", dtype)


@pytest.mark.parametrize("tag,kw", [
    ("prod4", dict(bits=4, use_qjl_keys=True, quantize_decode=True)),
    ("mse3_densetail", dict(bits=3, use_qjl_keys=False, quantize_decode=False)),
])
def test_activate_generate_matches_reference_run(tag, kw):
    import turboquant

    g = Golden("e2e_tiny_llama")
    model = _tiny_model()
    ids = torch.from_numpy(g.z["input_ids"]).cuda()
    turboquant.activate(model, StubTokenizer(), quiet=True, **kw)
    assert turboquant.is_active(model)
    out = model.generate(ids, max_new_tokens=8)
    again = model.generate(ids, max_new_tokens=8)
    tel = turboquant.last_telemetry(model)
    met = turboquant.last_metrics(model)
    assert model.config._attn_implementation != "turboquant"  # restored after the call
    turboquant.deactivate(model, quiet=True)

    want = torch.from_numpy(g.z[f"{tag}_output_ids"])
    assert tuple(out.shape) == tuple(want.shape)
    assert torch.equal(out, again)  # reproducible (the reference's own smoke criterion)
    assert torch.equal(out.cpu()[:, :48], want[:, :48])
    # Greedy tokens of a random-init model: the first new token comes from the dense prefill and
    # must match; later ones go through quantised attention on both sides and are compared too.
    assert int(out[0, 48]) == int(want[0, 48])
    assert (out.cpu() == want).float().mean() >= 0.95
    for key in ("dense_kv_bytes", "packed_estimate_bytes", "packed_actual_bytes", "prompt_tokens",
                "completion_tokens", "qmse_bits"):
        assert tel[key] == int(g.z[f"{tag}_tel_{key}"]), key
    assert sorted(tel.keys()) == list(g.z[f"{tag}_tel_keys"])
    assert sorted(met.keys()) == list(g.z[f"{tag}_metrics_keys"])
    rq = met["reconstruction_quality"]
    assert sorted(rq[0].keys()) == list(g.z[f"{tag}_recon_keys"])
    for layer, (kc, vc) in enumerate(zip(g.z[f"{tag}_recon_key_cos"], g.z[f"{tag}_recon_val_cos"])):
        assert abs(rq[layer]["key_cosine_sim"] - kc) < 2e-4 and abs(rq[layer]["val_cosine_sim"] - vc) < 2e-4
    # the reference's quality gates (key cosine >= 0.990 at 4 bits, 0.970 at 3 bits)
    gate = {4: 0.990, 3: 0.970}[kw["bits"]]
    if not kw["use_qjl_keys"]:
        assert all(r["key_cosine_sim"] >= gate for r in rq)


def test_batched_generate_and_bf16():
    import turboquant

    model = _tiny_model(torch.bfloat16)
    ids = torch.randint(0, 512, (3, 40), device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    turboquant.activate(model, StubTokenizer(), quiet=True, bits=4, verify=False)
    out = model.generate(ids, max_new_tokens=6)
    assert tuple(out.shape) == (3, 46) and torch.equal(out[:, :40], ids)
    tel = turboquant.last_telemetry(model)
    assert tel["packed_actual_bytes"] < tel["dense_kv_bytes"] and 0.7 < tel["payload_savings_fraction"] < 0.76
    assert turboquant.last_metrics(model)["reconstruction_quality"] is None
    turboquant.deactivate(model, quiet=True)


def test_norm_guard_keeps_high_norm_layers_dense(setup_golden, capsys):
    from tq_local_b200.runtime.packed_qmse_cache import build_packed_mse_cache

    g = Golden("norm_guard")
    k_hi, v_hi, _ = O.synth_kvq(1, 4, 4, 64, 128, seed=11, norm_mode="asym")
    k_lo, v_lo, _ = O.synth_kvq(1, 4, 4, 64, 128, seed=12)
    layers = [(k_hi.cuda(), v_hi.cuda()), (k_lo.cuda(), v_lo.cuda()), ((k_lo * 9.0).cuda(), v_lo.cuda())]
    cache = build_packed_mse_cache(layers, bits=4, use_qjl_keys=True, quantize_decode=True, norm_guard=True)
    assert [int(layer._force_dense) for layer in cache.layers] == list(g.z["dense_flags"])
    assert [layer.storage_bytes() for layer in cache.layers] == list(g.z["storage_bytes"])
    assert "norm_guard: 1/3 layers kept dense" in capsys.readouterr().err
    off = build_packed_mse_cache(layers, bits=4, use_qjl_keys=True, norm_guard=False)
    assert not any(layer._force_dense for layer in off.layers)


def test_cache_layer_views_and_multi_token_queries(setup_golden):
    """keys_packed / values_packed / _keys_qjl expose the reference's tensors; a 3-token query
    is served with causal visibility."""
    from helpers import oracle_params
    from tq_local_b200.runtime.packed_qmse_cache import PackedMSELayer

    k, v, _ = O.synth_kvq(2, 8, 2, 50, 128, seed=21, dtype=torch.float32)
    layer = PackedMSELayer(bits=4, use_qjl_keys=True, quantize_decode=True, reserve_tokens=4)
    layer.initialize_from_dense(k[:, :, :47].cuda(), v[:, :, :47].cuda())
    layer._lazy_update = True
    kk, vv = layer.update(k[:, :, 47:].cuda(), v[:, :, 47:].cuda())  # three tokens at once
    assert kk.shape[2] == 3 and layer.get_seq_length() == 50 and layer.packed_seq_length() == 50
    assert tuple(layer.keys_packed.packed_indices.shape) == (2, 2, 50, 48)
    assert tuple(layer.values_packed.packed_indices.shape) == (2, 2, 50, 64)
    assert tuple(layer._keys_qjl.packed_signs.shape) == (2, 2, 50, 16)
    assert layer.keys_packed.norms.dtype == torch.float16 and layer.keys_packed.bits == 3
    assert layer.storage_bytes() == 2 * 2 * 50 * (48 + 2 + 16 + 2 + 64 + 2)
    q = torch.randn(2, 8, 3, 128, generator=torch.Generator().manual_seed(3))
    got = layer.attend(q.cuda()).cpu()
    p = O.QuantParams.build(128, 4, True, seed=0, rot_v=layer.codec.rot_v, rot_k=layer.codec.rot_k)
    for i in range(3):
        n = 48 + i
        c = lambda t: t[:, :, :n].contiguous().cpu()
        s = layer.store
        mine = O.PackedLayer(p, torch.float32, c(s.k_codes), c(s.k_norms), c(s.v_codes), c(s.v_norms),
                             c(s.k_signs), c(s.k_rnorms))
        want = O.attend_dequant(q[:, :, i:i + 1], mine, 4)
        assert float((got[:, :, i:i + 1] - want).abs().max() / want.abs().max()) < 1e-5


def test_generate_with_recorded_decode_step_matches_eager_stepping(monkeypatch):
    """``cuda_graph=True``: the model's decode step is recorded once and replayed per token with
    the cache length on the device.  Replay must give exactly the tokens of the same steps run
    eagerly, and (up to near-ties of a random-init model) those of the host-length path."""
    import turboquant
    from tq_local_b200.runtime import generation

    model = _tiny_model(torch.bfloat16)
    ids = torch.randint(0, 512, (2, 40), device="cuda", generator=torch.Generator("cuda").manual_seed(3))
    new = 24

    def run(**kw):
        turboquant.activate(model, StubTokenizer(), quiet=True, bits=4, verify=False, **kw)
        try:
            out = model.generate(ids, max_new_tokens=new)
            tel = turboquant.last_telemetry(model)
        finally:
            turboquant.deactivate(model, quiet=True)
        return out, tel

    import warnings

    with warnings.catch_warnings():
        warnings.simplefilter("error")  # a step that could not be recorded warns; here it must record
        graphed, tel_g = run(cuda_graph=True)
    host_len, tel_h = run(cuda_graph=False)
    monkeypatch.setattr(generation, "_GRAPH_WARMUP_STEPS", 10 ** 9)  # same device-length steps, never recorded
    stepped, _ = run(cuda_graph=True)
    assert tuple(graphed.shape) == (2, 40 + new)
    assert torch.equal(graphed, stepped)
    assert (graphed == host_len).float().mean() >= 0.9 and torch.equal(graphed[:, :42], host_len[:, :42])
    assert tel_g["completion_tokens"] == tel_h["completion_tokens"] == new
    assert tel_g["packed_actual_bytes"] == tel_h["packed_actual_bytes"]


def test_streaming_prefill_packs_layer_by_layer_with_the_same_result(setup_golden, capsys):
    """Without the reconstruction report the prompt pass packs each layer as the model produces
    it (no dense cache of the whole model).  Tokens, telemetry and norm-guard decisions must equal
    the pack-after-prefill path."""
    import turboquant
    from tq_local_b200.runtime.packed_qmse_cache import build_packed_mse_cache, build_streaming_prefill_cache

    model = _tiny_model()
    ids = torch.from_numpy(Golden("e2e_tiny_llama").z["input_ids"]).cuda()

    def run(verify):
        turboquant.activate(model, StubTokenizer(), quiet=True, bits=4, verify=verify)
        try:
            return model.generate(ids, max_new_tokens=8), turboquant.last_telemetry(model)
        finally:
            turboquant.deactivate(model, quiet=True)

    streamed, tel_s = run(False)
    packed_after, tel_p = run(True)
    assert torch.equal(streamed, packed_after)
    for key in ("dense_kv_bytes", "packed_estimate_bytes", "packed_actual_bytes", "prompt_tokens", "completion_tokens"):
        assert tel_s[key] == tel_p[key], key

    # norm guard inside the streaming cache: same decisions and bytes as the batch builder
    k_hi, v_hi, _ = O.synth_kvq(1, 4, 4, 64, 128, seed=11, norm_mode="asym")
    k_lo, v_lo, _ = O.synth_kvq(1, 4, 4, 64, 128, seed=12)
    pairs = [(k_hi.cuda(), v_hi.cuda()), (k_lo.cuda(), v_lo.cuda())]
    want = build_packed_mse_cache(pairs, bits=4, use_qjl_keys=True, quantize_decode=True, norm_guard=True)
    capsys.readouterr()
    cache = build_streaming_prefill_cache(2, 4, use_qjl_keys=True, quantize_decode=True, norm_guard=True)
    for layer, (k, v) in zip(cache.layers, pairs):
        rk, rv = layer.update(k, v)
        assert rk is k and rv is v
    assert [l._force_dense for l in cache.layers] == [l._force_dense for l in want.layers] == [True, False]
    assert [l.storage_bytes() for l in cache.layers] == [l.storage_bytes() for l in want.layers]
    assert torch.equal(cache.layers[1].store.k_codes[:, :, :64], want.layers[1].store.k_codes[:, :, :64])
    assert cache.layers[1].get_seq_length() == 64


def test_prompt_pass_in_row_blocks_equals_the_single_pass(capsys):
    """``prefill_block_tokens``: a streaming prompt pass that takes the batch two sequences at a
    time must leave exactly the packed cache, the norm-guard decisions and the tokens of the pass
    that takes the whole batch at once."""
    import turboquant

    model = _tiny_model(torch.bfloat16)
    ids = torch.randint(0, 512, (5, 64), device="cuda", generator=torch.Generator("cuda").manual_seed(5))
    captured, outs = {}, {}
    for name, block in (("single", 1 << 30), ("blocks", 128)):  # 128 tokens = two 64-token sequences per block
        turboquant.activate(model, StubTokenizer(), quiet=True, bits=4, verify=False, cuda_graph=False,
                            prefill_block_tokens=block)
        outs[name] = model.generate(ids, max_new_tokens=6)
        captured[name] = turboquant.last_telemetry(model)
        turboquant.deactivate(model, quiet=True)
    assert torch.equal(outs["single"], outs["blocks"])
    for key in ("dense_kv_bytes", "packed_actual_bytes", "prompt_tokens", "completion_tokens"):
        assert captured["single"][key] == captured["blocks"][key], key


def test_row_block_prefill_fills_the_same_cache_and_keeps_norm_guard_layers_dense():
    """Layer level: K/V handed over in row blocks give byte-identical packed streams (packed layer)
    and the same dense tensors (norm-guarded layer) as one hand-over of the whole batch."""
    from tq_local_b200.runtime.packed_qmse_cache import _auto_norm_threshold, build_streaming_prefill_cache

    B, Hkv, S = 5, 2, 96
    k_lo, v_lo, _ = O.synth_kvq(B, 4, Hkv, S, 128, seed=41, dtype=torch.bfloat16)
    k_hi, v_hi, _ = O.synth_kvq(B, 4, Hkv, S, 128, seed=42, dtype=torch.bfloat16, norm_mode="asym")
    thr = _auto_norm_threshold(4, 128)
    kw = dict(bits=4, use_qjl_keys=True, quantize_decode=True, norm_guard=True, reserve_tokens=8)
    whole = build_streaming_prefill_cache(2, **kw)
    whole.layers[0].update(k_lo.cuda(), v_lo.cuda())
    whole.layers[1].update(k_hi.cuda(), v_hi.cuda())
    blocks = build_streaming_prefill_cache(2, **kw)
    for b0 in range(0, B, 2):
        for layer, (k, v) in zip(blocks.layers, ((k_lo, v_lo), (k_hi, v_hi))):
            assert layer.get_seq_length() == 0  # every block's prompt starts at position 0
            layer.begin_prefill_block(b0, B, thr)
            layer.update(k[b0:b0 + 2].cuda(), v[b0:b0 + 2].cuda())
    assert all(layer.finish_prefill(S, thr) for layer in blocks.layers)
    a, b = whole.layers[0], blocks.layers[0]
    assert not a._force_dense and not b._force_dense and b.get_seq_length() == S
    for x, y in zip(a.store.streams(), b.store.streams()):
        assert torch.equal(x[:, :, :S], y[:, :, :S])
    a, b = whole.layers[1], blocks.layers[1]
    assert a._force_dense and b._force_dense and b.get_seq_length() == S
    assert torch.equal(a._dense_keys, b._dense_keys) and torch.equal(a._dense_values, b._dense_values)
    assert a.storage_bytes() == b.storage_bytes()


def test_long_prompt_batch_16_by_32768_through_activate_on_two_layers():
    """The full-model workload's prompt shape (batch 16 x 32768 random token ids, Llama-3.1-8B layer
    dimensions, vocabulary 128256) through ``activate()`` -> ``generate()`` on a two-layer model:
    the prompt pass runs in row blocks, so neither [16, 32768, vocab] logits (134 GB) nor the
    activations of the whole batch are ever held; then greedy tokens through the recorded step."""
    import turboquant
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=2,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=131072,
                      tie_word_embeddings=False)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device("cuda"):
            model = LlamaForCausalLM(cfg).eval()
    finally:
        torch.set_default_dtype(old)
    B, S, new = 16, 32768, 12
    ids = torch.randint(0, 128256, (B, S), device="cuda", generator=torch.Generator("cuda").manual_seed(7))
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    turboquant.activate(model, StubTokenizer(), quiet=True, bits=4, use_qjl_keys=True, verify=False)
    out = model.generate(ids, max_new_tokens=new)
    tel = turboquant.last_telemetry(model)
    turboquant.deactivate(model, quiet=True)
    assert tuple(out.shape) == (B, S + new) and torch.equal(out[:, :S], ids)
    assert tel["prompt_tokens"] == S and tel["packed_actual_bytes"] == 2 * 134 * B * 8 * S
    # four sequences (131072 tokens) per block: activations of a block stay far below what the
    # whole batch would need (the MLP intermediates alone would be 45 GB)
    assert torch.cuda.max_memory_allocated() - base < 40e9


def test_attention_masks_on_the_packed_path():
    """The cache layer turns a left-padding mask (2-D, 4-D boolean or 4-D additive) into per-row
    start offsets; ``chunked_turboquant_attention`` accepts the mask and un-stored new tokens."""
    from tq_local_b200.runtime.attention import chunked_turboquant_attention
    from tq_local_b200.runtime.packed_qmse_cache import PackedMSELayer, is_left_padding_mask, leading_masked_tokens

    B, Hq, Hkv, N = 3, 8, 2, 90
    k, v, q = O.synth_kvq(B, Hq, Hkv, N + 2, 128, seed=51, dtype=torch.bfloat16)
    layer = PackedMSELayer(bits=4, use_qjl_keys=True, quantize_decode=True, reserve_tokens=4)
    layer.initialize_from_dense(k[:, :, :N].cuda(), v[:, :, :N].cuda())
    pads = [0, 7, 33]
    m2 = torch.ones(B, N, dtype=torch.long)
    for b, n in enumerate(pads):
        m2[b, :n] = 0
    assert is_left_padding_mask(m2.cuda()) and not is_left_padding_mask(torch.flip(m2, dims=[1]).cuda())
    assert leading_masked_tokens(m2.cuda()).tolist() == pads
    m4_bool = m2.bool()[:, None, None, :].cuda()
    m4_add = torch.where(m4_bool, 0.0, torch.finfo(torch.bfloat16).min).to(torch.bfloat16)
    assert leading_masked_tokens(m4_bool).tolist() == pads and leading_masked_tokens(m4_add).tolist() == pads
    qd = q.cuda()
    plain = layer.attend(qd).clone()
    masked = [layer.attend(qd, m).clone() for m in (m2.cuda(), m4_bool, m4_add)]
    assert torch.equal(masked[0], masked[1]) and torch.equal(masked[0], masked[2])
    assert torch.equal(masked[0][0], plain[0]) and not torch.equal(masked[0][2], plain[2])
    assert torch.equal(layer.attend(qd), plain)  # a call without a mask is unrestricted again
    assert torch.equal(chunked_turboquant_attention(qd, layer, n_kv_groups=4, attention_mask=m4_bool), masked[0])
    # per-row oracle: row b attends tokens [pad_b, N)
    p = O.QuantParams.build(128, 4, True, seed=0, rot_v=layer.codec.rot_v, rot_k=layer.codec.rot_k)
    s = layer.store
    for b, n in enumerate(pads):
        c = lambda t: t[b:b + 1, :, n:N].contiguous().cpu()
        mine = O.PackedLayer(p, torch.bfloat16, c(s.k_codes), c(s.k_norms), c(s.v_codes), c(s.v_norms),
                             c(s.k_signs), c(s.k_rnorms))
        want = O.attend_rotated_space(q[b:b + 1], mine, 4)
        assert float((masked[0][b:b + 1].float().cpu() - want).abs().max() / want.abs().max()) <= 2e-3 + 2.0 ** -9
    # un-stored new tokens are attended dense, after the cache, and nothing is stored
    before = [t[:, :, :N].clone() for t in s.streams()]
    got = chunked_turboquant_attention(qd, layer, new_key=k[:, :, N:].cuda(), new_value=v[:, :, N:].cuda(), n_kv_groups=4)
    want = s.decode_attn(qd, tail_k=k[:, :, N:].cuda(), tail_v=v[:, :, N:].cuda())
    assert torch.equal(got, want) and s.length == N and not torch.equal(got, plain)
    for a, b_ in zip(before, s.streams()):
        assert torch.equal(a, b_[:, :, :N])
    # a bound mask stays in force for calls without one (the generation loop binds the prompt's mask)
    layer.bind_attention_mask(m2.cuda())
    assert torch.equal(layer.attend(qd), masked[0])
    layer.bind_attention_mask(None)
    assert torch.equal(layer.attend(qd), plain)


def test_generate_with_a_left_padded_batch_matches_the_unpadded_prompt():
    """A short prompt left-padded into a batch must generate what it generates alone: the padding is
    masked in the prompt pass (the model's own attention) and in every packed decode step, eager
    and recorded.  (RoPE is relative, so the shifted positions of the padded row do not matter.)"""
    import turboquant

    model = _tiny_model(torch.float32)
    gen = torch.Generator("cuda").manual_seed(9)
    long_ids = torch.randint(1, 512, (1, 48), device="cuda", generator=gen)
    short_ids = torch.randint(1, 512, (1, 29), device="cuda", generator=gen)
    batch = torch.cat((long_ids, torch.cat((torch.zeros(1, 19, dtype=torch.long, device="cuda"), short_ids), dim=1)))
    mask = torch.ones_like(batch)
    mask[1, :19] = 0
    for graph in (False, True):
        turboquant.activate(model, StubTokenizer(), quiet=True, bits=4, use_qjl_keys=False, verify=False, cuda_graph=graph)
        alone = model.generate(short_ids, max_new_tokens=12)[:, 29:]
        both = model.generate(batch, attention_mask=mask, max_new_tokens=12)
        unmasked = model.generate(batch, max_new_tokens=12)
        turboquant.deactivate(model, quiet=True)
        assert int(both[1, 48]) == int(alone[0, 0])  # first token: dense prompt pass with the mask
        assert (both[1, 48:] == alone[0]).float().mean() >= 0.9, (graph, both[1, 48:], alone[0])
        assert not torch.equal(unmasked[1, 48:], both[1, 48:])  # attending the padding changes the text
    with pytest.raises(ValueError):
        turboquant.activate(model, StubTokenizer(), quiet=True, bits=4, verify=False)
        try:
            model.generate(batch, attention_mask=torch.flip(mask, dims=[1]), max_new_tokens=4)
        finally:
            turboquant.deactivate(model, quiet=True)


class _CallableTokenizer(StubTokenizer):
    """The stub plus what ``TurboQuantSession.generate`` uses: a call that tokenises a prompt
    ("12 7 300" -> ids) and a chat template that joins the messages' contents."""

    def __call__(self, text, return_tensors="pt"):
        ids = torch.tensor([[int(t) for t in text.split()]], dtype=torch.long)
        return {"input_ids": ids, "attention_mask": torch.ones_like(ids)}

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True):
        return " ".join(m["content"] for m in messages) + (" 1" if add_generation_prompt else "")


def test_session_generate_telemetry_and_errors():
    """``TurboQuantSession`` (reference: adapters/transformers.py:180-311): prompt and chat-message
    input, text or full output, metrics / telemetry / compatibility report, and its error cases;
    it must produce what ``activate`` + ``generate`` produces with the same settings."""
    import turboquant
    from turboquant import TurboQuantSession

    model = _tiny_model()
    tok = _CallableTokenizer()
    prompt = " ".join(str(3 + 5 * i % 500) for i in range(40))
    session = TurboQuantSession(model=model, tokenizer=tok, bits=4, use_qjl_keys=True, quantize_decode=True)
    assert session.last_metrics() is None and session.last_telemetry() is None
    text = session.generate(prompt=prompt, max_new_tokens=6)
    assert isinstance(text, str) and len(text.split()) == 6
    full = session.generate(prompt=prompt, max_new_tokens=6, return_output=True)
    assert full.text == text  # reproducible
    tel, met = session.last_telemetry(), session.last_metrics()
    assert tel["prompt_tokens"] == 40 and tel["completion_tokens"] == 6 and tel["qmse_bits"] == 4
    assert tel["packed_actual_bytes"] < tel["dense_kv_bytes"] and met["variant"] == "qmse_packed"
    assert met["reconstruction_quality"] is not None  # the session verifies like the reference's
    assert session.compatibility_report()["compatible"] is True
    # the same settings through activate() give the same tokens
    ids = tok(prompt)["input_ids"].cuda()
    turboquant.activate(model, tok, quiet=True, bits=4, use_qjl_keys=True, quantize_decode=True)
    out = model.generate(ids, max_new_tokens=6)
    turboquant.deactivate(model, quiet=True)
    assert " ".join(str(int(t)) for t in out[0, 40:]) == text
    # chat messages go through the tokenizer's template
    chat = session.generate(messages=[{"role": "user", "content": prompt}], max_new_tokens=3)
    assert len(chat.split()) == 3
    with pytest.raises(ValueError):
        session.generate(max_new_tokens=3)  # neither prompt nor messages
    with pytest.raises(ValueError):
        TurboQuantSession(model=model, tokenizer=StubTokenizer()).generate(messages=[{"role": "user", "content": "1"}])
    # the uncompressed comparison run the reference's CLI offers
    base = TurboQuantSession(model=model, tokenizer=tok, variant="baseline").generate(prompt=prompt, max_new_tokens=6,
                                                                                     return_output=True)
    assert base.metrics.variant == "baseline" and base.metrics.turboquant_mse_packed_actual is None
    assert base.text.split()[0] == text.split()[0]  # the first token comes from the same dense prompt pass
