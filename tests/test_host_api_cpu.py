"""Host-side behaviour of the reference-facing API (no GPU needed)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import Golden


def _tiny_model():
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=512)
    return LlamaForCausalLM(cfg).eval()


class StubTokenizer:
    eos_token_id = None

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(int(i)) for i in ids)

    def encode(self, text, add_special_tokens=False):
        return [int(t) for t in text.split()]


def test_public_names_match_reference():
    import tq_local_b200
    import turboquant

    expected = {"__version__", "CompatibilityReport", "TelemetrySummary", "TransformersLoadConfig",
                "TurboQuantSession", "activate", "deactivate", "inspect_transformers_model_compatibility",
                "is_active", "last_metrics", "last_telemetry", "load_transformers_model", "print_telemetry",
                "summarize_generation_metrics"}
    assert set(turboquant.__all__) == expected == set(tq_local_b200.__all__)
    for name in expected:
        assert getattr(turboquant, name) is getattr(tq_local_b200, name)


def test_activate_signature_and_defaults():
    import inspect

    import turboquant

    sig = inspect.signature(turboquant.activate)
    want = dict(bits=4, rotation_seed=0, num_outlier_channels=0, outlier_extra_bits=1, use_qjl_keys=True,
                quantize_decode=True, norm_guard=True, quiet=False)
    for name, default in want.items():
        p = sig.parameters[name]
        assert p.kind is inspect.Parameter.KEYWORD_ONLY and p.default == default
    assert list(sig.parameters)[:2] == ["model", "tokenizer"]


def test_activate_deactivate_state_machine(capsys):
    import turboquant

    model = _tiny_model()
    original = model.generate
    assert not turboquant.is_active(model)
    assert turboquant.last_telemetry(model) is None and turboquant.last_metrics(model) is None
    turboquant.deactivate(model)  # no-op with a message
    assert "nothing to deactivate" in capsys.readouterr().out
    turboquant.activate(model, StubTokenizer(), quiet=True)
    assert turboquant.is_active(model) and model.generate is not original
    assert model._tq_state.bits == 4 and model._tq_state.use_qjl_keys is True
    with pytest.raises(RuntimeError, match="already active"):
        turboquant.activate(model, StubTokenizer(), quiet=True)
    with pytest.raises(ValueError, match="input_ids"):
        model.generate()
    turboquant.print_telemetry(model)
    assert "No generation data" in capsys.readouterr().out
    turboquant.deactivate(model, quiet=True)
    assert not turboquant.is_active(model) and model.generate == original
    for attr in ("_tq_state", "_tq_tokenizer", "_tq_last_output"):
        assert not hasattr(model, attr)


def test_activate_rejects_bad_models():
    import turboquant

    model = _tiny_model()
    model.config._name_or_path = ""
    with pytest.raises(ValueError, match="tokenizer"):
        turboquant.activate(model, None, quiet=True)
    model.config.use_cache = False
    with pytest.raises(ValueError, match="not compatible"):
        turboquant.activate(model, StubTokenizer(), quiet=True)
    model.config.use_cache = True
    turboquant.activate(model, StubTokenizer(), quiet=True, num_outlier_channels=8)
    assert model._tq_state.num_outlier_channels == 8
    turboquant.deactivate(model)
    report = turboquant.inspect_transformers_model_compatibility(model)
    assert report.compatible and report.backend == "transformers" and report.details["num_key_value_heads"] == 2


def test_generate_without_gpu_fails_loudly():
    """No CPU fallback: on a machine without CUDA the packed path raises."""
    import turboquant
    from tq_local_b200.runtime import ffi

    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    model = _tiny_model()
    turboquant.activate(model, StubTokenizer(), quiet=True)
    with pytest.raises(ffi.TQError):
        model.generate(torch.randint(0, 512, (1, 8)), max_new_tokens=2)
    assert model.config._attn_implementation != "turboquant"  # wiring never left half-enabled
    turboquant.deactivate(model, quiet=True)


def test_telemetry_schema_and_numbers_match_reference():
    from tq_local_b200.runtime.generation import GenerationMetrics
    from tq_local_b200.runtime.memory_accounting import turboquant_mse_packed_bytes
    from tq_local_b200.telemetry import summarize_generation_metrics

    g = Golden("e2e_tiny_llama")
    est = turboquant_mse_packed_bytes(num_vectors_per_kind=2 * 1 * 2 * 48, vector_dimension=128, bits=4)
    assert est["packed_kv_bytes"] == int(g.z["prod4_tel_packed_estimate_bytes"])
    m = GenerationMetrics(
        variant="qmse_packed", qmse_bits=4, quantization_seconds=0.5, generation_seconds=2.0, prompt_tokens=48,
        completion_tokens=8,
        prefill_cache={"dense_kv_bytes": int(g.z["prod4_tel_dense_kv_bytes"])},
        turboquant_mse_packed_estimate=est,
        turboquant_mse_packed_actual={"packed_total_bytes": int(g.z["prod4_tel_packed_actual_bytes"])},
        post_cache_setup_gpu_memory={"allocated_bytes": None, "reserved_bytes": None},
        gpu_peak_memory={"peak_allocated_bytes": 10, "peak_reserved_bytes": 20},
    )
    assert sorted(m.to_dict().keys()) == list(g.z["prod4_metrics_keys"])
    tel = summarize_generation_metrics(m)
    d = tel.to_dict()
    assert sorted(d.keys()) == list(g.z["prod4_tel_keys"])
    assert d["payload_savings_fraction"] == pytest.approx(1 - d["packed_actual_bytes"] / d["dense_kv_bytes"])
    assert d["peak_allocated_bytes"] == 10 and d["post_cache_setup_allocated_bytes"] is None
    assert "KV" in tel.format(compact=True) and "TurboQuant Telemetry" in tel.format()
    assert summarize_generation_metrics(m.to_dict()) == tel


def test_memory_breakdown_on_dynamic_cache_and_tuples():
    from transformers import DynamicCache

    from tq_local_b200.runtime.memory_accounting import past_key_values_memory_breakdown

    k, v = torch.zeros(2, 2, 5, 128, dtype=torch.bfloat16), torch.zeros(2, 2, 5, 128, dtype=torch.bfloat16)
    out = past_key_values_memory_breakdown([(k, v), (k, v)])
    assert out["num_layers"] == 2 and out["dense_kv_bytes"] == 4 * k.numel() * 2
    assert out["num_key_value_vectors_per_kind"] == 2 * 2 * 2 * 5 and out["vector_dimension"] == 128
    cache = DynamicCache()
    cache.update(k, v, 0)
    assert past_key_values_memory_breakdown(cache)["dense_kv_bytes"] == 2 * k.numel() * 2


def test_norm_threshold_and_layer_interface():
    from tq_local_b200.runtime.packed_qmse_cache import PackedMSELayer, _auto_norm_threshold

    g = Golden("setup")
    for b in (2, 3, 4, 5):
        assert _auto_norm_threshold(b, 128) == float(g.z[f"norm_threshold_b{b}"])
    layer = PackedMSELayer(bits=4, use_qjl_keys=True, quantize_decode=True)
    assert layer.get_seq_length() == 0 and layer.get_max_cache_shape() == -1 and layer.is_sliding is False
    assert layer.get_mask_sizes(3) == (3, 0) and layer.get_mask_sizes(torch.arange(2)) == (2, 0)
    assert layer.keys_packed is None and layer.storage_bytes() == 0
    split = PackedMSELayer(bits=4, num_outlier_channels=4)
    assert not split._outlier_enabled and split.keys_packed is None  # (decided with the first tensors it sees)
    # force-dense layers never touch the GPU
    k = torch.randn(1, 2, 6, 128)
    layer.initialize_from_dense(k, k, force_dense=True)
    assert layer._force_dense and layer.get_seq_length() == 6
    kk, vv = layer.update(k[:, :, :1], k[:, :, :1])
    assert kk.shape[2] == 7 and torch.equal(kk[:, :, :6], k) and layer.storage_bytes() == 2 * 7 * 2 * 128 * 4


def test_generation_variant_validation():
    from tq_local_b200.runtime.generation import validate_generation_variant

    validate_generation_variant("baseline")
    validate_generation_variant("qmse_packed")
    validate_generation_variant("qmse")
    with pytest.raises(ValueError):
        validate_generation_variant("nope")


def test_unpacked_qmse_variant_matches_the_reference():
    """The unpacked ``qmse`` variant (quantise-dequantise in place; reference turboquant_mse.py:124-217,
    generation.py:104-113,170-178) against the reference's own outputs: per-vector reconstruction and
    indices, in-place treatment of a cache (whole, and last token only), and a greedy generation
    on the tiny Llama.  Plain tensor arithmetic on the tensors' device, so it runs here on the CPU."""
    import numpy as np
    import torch
    from transformers import LlamaConfig, LlamaForCausalLM

    from conftest import Golden
    from tq_local_b200.quantization.turboquant_mse import quantize_past_key_values_mse, quantize_vectors_mse
    from tq_local_b200.runtime.generation import greedy_decode_with_prefill_cache

    g = Golden("qmse")
    vec = g.z["vectors"]
    for bits, seed in ((3, 0), (4, 5)):
        rec, idx = quantize_vectors_mse(vec, bits=bits, seed=seed)
        assert isinstance(rec, np.ndarray) and rec.dtype == np.float32 and idx.dtype == np.int16
        want_idx, want_rec = g.z[f"idx_b{bits}_s{seed}"], g.z[f"rec_b{bits}_s{seed}"]
        # (BLAS summation order may move a value across a boundary it sits on: at most a few codes)
        assert (idx != want_idx).mean() < 1e-4 and np.abs(idx.astype(int) - want_idx).max() <= 1
        same = (idx == want_idx).all(axis=1)
        assert np.abs(rec[same] - want_rec[same]).max() <= 2e-6 * np.abs(want_rec).max()
    kv = torch.from_numpy(g.z["kv"])
    as_tuple = lambda t: tuple((t[i, 0], t[i, 1]) for i in range(t.shape[0]))
    for key, sl in (("kv_full", None), ("kv_last", slice(-1, None))):
        got = quantize_past_key_values_mse(as_tuple(kv), bits=4, seed=0, token_slice=sl)
        want = torch.from_numpy(g.z[key])
        for i, (k_, v_) in enumerate(got):
            assert float((k_ - want[i, 0]).abs().max()) <= 1e-5 and float((v_ - want[i, 1]).abs().max()) <= 1e-5
    assert torch.equal(quantize_past_key_values_mse(as_tuple(kv), 4, token_slice=slice(-1, None))[0][0][:, :, :-1],
                       kv[0, 0][:, :, :-1])  # earlier tokens untouched

    class Tok:
        eos_token_id = None

        def decode(self, ids, skip_special_tokens=True):
            return " ".join(str(int(i)) for i in ids)

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=512)
    model = LlamaForCausalLM(cfg).eval()
    ids = torch.from_numpy(Golden("e2e_tiny_llama").z["input_ids"])
    out = greedy_decode_with_prefill_cache(model=model, tokenizer=Tok(), inputs={"input_ids": ids}, max_new_tokens=8,
                                           variant="qmse", qmse_bits=4)
    got_ids = [int(t) for t in out.text.split()]
    want_ids = list(g.z["gen_text_ids"])
    assert got_ids[0] == want_ids[0] and sum(a == b for a, b in zip(got_ids, want_ids)) >= 7
    assert out.metrics.variant == "qmse" and out.metrics.qmse_bits == int(g.z["gen_qmse_bits"])
    assert sorted(out.metrics.to_dict().keys()) == list(g.z["gen_metrics_keys"])
    assert out.metrics.turboquant_mse_packed_actual is None and out.metrics.reconstruction_quality is None
