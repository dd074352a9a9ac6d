"""Generate the golden fixtures in this folder from the UNMODIFIED reference.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py --reference /path/to/reference

The script imports ``turboquant`` from ``<reference>/src`` (never from this
repository), runs the reference's own CPU code on small seeded inputs and
stores inputs + outputs as ``.npz`` files.  The test-suite only reads the
``.npz`` files, so it runs on machines without the reference.

bf16 / fp16 tensors are stored as their 16-bit patterns (``*_bits16`` keys).
"""

from __future__ import annotations

import argparse
import math
import os
import sys

import numpy as np


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the unmodified reference project (its root)")
    ap.add_argument("--out", default=None, help="folder to write the fixtures to (default: beside this script)")
    args = ap.parse_args()
    here = os.path.dirname(os.path.abspath(__file__))
    # The reference must shadow any other package called ``turboquant``.
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != os.path.dirname(os.path.dirname(here))]
    sys.path.insert(0, os.path.join(args.reference, "src"))

    script_dir = here
    if args.out:
        here = os.path.abspath(args.out)
        os.makedirs(here, exist_ok=True)
    del script_dir

    import torch
    import turboquant  # noqa: F401  (the reference)
    assert os.path.abspath(turboquant.__file__).startswith(os.path.abspath(args.reference)), turboquant.__file__
    from turboquant.quantization.turboquant_mse import build_scalar_codebook, random_rotation_matrix
    from turboquant.runtime import packed_qmse_cache as pc
    from turboquant.runtime.attention import chunked_turboquant_attention

    torch.set_num_threads(1)  # fixed reduction order for the stored matmuls

    def bits16(t: torch.Tensor) -> np.ndarray:
        return t.contiguous().view(torch.int16).numpy().copy()

    def store(t: torch.Tensor, name: str, out: dict) -> None:
        if t.dtype in (torch.bfloat16, torch.float16):
            out[name + "_bits16"] = bits16(t)
        else:
            out[name] = t.numpy().copy()

    # ---------------- set-up data: codebooks, rotations, QJL, packing KAT -------------
    setup: dict[str, np.ndarray] = {}
    for b in (1, 2, 3, 4):
        cb = build_scalar_codebook(128, b)
        setup[f"centers_b{b}"] = cb.centers
        setup[f"boundaries_b{b}"] = cb.boundaries
    cb64 = build_scalar_codebook(64, 3)
    setup["centers_d64_b3"] = cb64.centers
    for seed in (0, 1, 7):
        setup[f"rotation_s{seed}"] = random_rotation_matrix(128, seed)
    setup["qjl_s31337"] = pc._generate_qjl_matrix(128, 31337).numpy()
    setup["qjl_s31344"] = pc._generate_qjl_matrix(128, 31344).numpy()
    g = torch.Generator().manual_seed(123)
    for b in (1, 2, 3, 4):
        idx = torch.randint(0, 2 ** b, (5, 128), generator=g)
        setup[f"packkat_idx_b{b}"] = idx.numpy()
        setup[f"packkat_bytes_b{b}"] = pc._pack_indices(idx, b).numpy()
        assert torch.equal(pc._unpack_indices(pc._pack_indices(idx, b), b, 128), idx)
    # ragged row length (dim*bits not a multiple of 8)
    idx = torch.randint(0, 8, (3, 13), generator=g)
    setup["packkat_idx_ragged"] = idx.numpy()
    setup["packkat_bytes_ragged"] = pc._pack_indices(idx, 3).numpy()
    setup["packkat_0to7_b3"] = pc._pack_indices(torch.arange(8).view(1, 8), 3).numpy()
    for b in (2, 3, 4, 5):
        setup[f"norm_threshold_b{b}"] = np.float64(pc._auto_norm_threshold(b, 128))
    np.savez_compressed(os.path.join(here, "setup.npz"), **setup)

    # ---------------- layer cases ---------------------------------------------------
    def synth(batch, hq, hkv, seq, seed, dtype, mode="lognormal"):
        gg = torch.Generator().manual_seed(seed)

        def draw(lo=None, hi=None):
            x = torch.randn(batch, hkv, seq, 128, generator=gg)
            if mode == "lognormal":
                return x * torch.exp(0.5 * torch.randn(batch, hkv, seq, 1, generator=gg))
            u = x / x.norm(dim=-1, keepdim=True)
            return u * (lo + (hi - lo) * torch.rand(batch, hkv, seq, 1, generator=gg))

        k = draw(100.0, 400.0)
        v = draw(1.0, 10.0)
        q = torch.randn(batch, hq, 1, 128, generator=gg)
        return k.to(dtype), v.to(dtype), q.to(dtype)

    cases = [
        # name, bits, qjl, dtype, B, Hq, Hkv, S, n_append, seed
        ("mse4_f32", 4, False, torch.float32, 2, 8, 2, 40, 3, 0),
        ("prod4_bf16", 4, True, torch.bfloat16, 2, 8, 2, 40, 3, 1),
        ("prod3_bf16", 3, True, torch.bfloat16, 1, 14, 2, 37, 2, 2),
        ("mse3_f32", 3, False, torch.float32, 1, 4, 4, 33, 1, 3),
        ("prod2_f16", 2, True, torch.float16, 1, 8, 2, 35, 2, 4),
        ("mse2_bf16", 2, False, torch.bfloat16, 2, 4, 2, 31, 1, 5),
        ("prod4_f32", 4, True, torch.float32, 1, 8, 2, 48, 2, 6),
    ]
    for name, bits, qjl, dtype, B, Hq, Hkv, S, n_app, seed in cases:
        k, v, q = synth(B, Hq, Hkv, S + n_app, seed, dtype)
        out: dict[str, np.ndarray] = {
            "bits": np.int64(bits), "qjl": np.int64(qjl), "B": np.int64(B), "Hq": np.int64(Hq),
            "Hkv": np.int64(Hkv), "S": np.int64(S), "n_append": np.int64(n_app),
            "seed": np.int64(seed), "dtype": np.array(str(dtype).replace("torch.", "")),
        }
        store(k, "k", out)
        store(v, "v", out)
        store(q, "q", out)
        layer = pc.PackedMSELayer(bits=bits, seed=0, use_qjl_keys=qjl, quantize_decode=True)
        layer.initialize_from_dense(k[:, :, :S].contiguous(), v[:, :, :S].contiguous())
        groups = Hq // Hkv

        def dump(tag):
            out[f"{tag}_k_codes"] = layer.keys_packed.packed_indices.numpy().copy()
            out[f"{tag}_k_norms_bits16"] = bits16(layer.keys_packed.norms)
            out[f"{tag}_v_codes"] = layer.values_packed.packed_indices.numpy().copy()
            out[f"{tag}_v_norms_bits16"] = bits16(layer.values_packed.norms)
            if qjl:
                out[f"{tag}_k_signs"] = layer._keys_qjl.packed_signs.numpy().copy()
                out[f"{tag}_k_rnorms_bits16"] = bits16(layer._keys_qjl.residual_norms)
            out[f"{tag}_storage_bytes"] = np.int64(layer.storage_bytes())
            kd = layer._decode_keys_full()
            vd = layer._decode_values_full()
            store(kd, f"{tag}_k_dequant", out)
            store(vd, f"{tag}_v_dequant", out)
            att = chunked_turboquant_attention(q, layer, n_kv_groups=groups, chunk_size=16)
            store(att, f"{tag}_attn_chunked", out)
            kf = kd.float().repeat_interleave(groups, dim=1)
            vf = vd.float().repeat_interleave(groups, dim=1)
            ref = torch.softmax((q.float() @ kf.transpose(-1, -2)) / math.sqrt(128), -1) @ vf
            out[f"{tag}_attn_dequant_f32"] = ref.numpy().copy()

        dump("prefill")
        layer._lazy_update = True
        for t in range(n_app):
            layer.update(k[:, :, S + t:S + t + 1].contiguous(), v[:, :, S + t:S + t + 1].contiguous())
        dump("appended")
        # quantize_decode=False tail: packed prefill + dense tail attention
        layer2 = pc.PackedMSELayer(bits=bits, seed=0, use_qjl_keys=qjl, quantize_decode=False)
        layer2.initialize_from_dense(k[:, :, :S].contiguous(), v[:, :, :S].contiguous())
        layer2._lazy_update = True
        for t in range(n_app):
            layer2.update(k[:, :, S + t:S + t + 1].contiguous(), v[:, :, S + t:S + t + 1].contiguous())
        att = chunked_turboquant_attention(q, layer2, n_kv_groups=groups, chunk_size=16)
        store(att, "densetail_attn_chunked", out)
        np.savez_compressed(os.path.join(here, f"layer_{name}.npz"), **out)
        print(name, "ok", {k_: v_.shape for k_, v_ in out.items() if hasattr(v_, "shape") and v_.ndim > 1 and "codes" in k_})

    # ---------------- outlier-channel split (num_outlier_channels > 0) ----------------------------
    ocases = [
        # name, bits, qjl, dtype, n_outlier, extra_bits, B, Hq, Hkv, S, n_append, seed
        ("mse3_o8_f32", 3, False, torch.float32, 8, 1, 2, 4, 2, 21, 2, 11),
        ("prod4_o16_bf16", 4, True, torch.bfloat16, 16, 1, 1, 8, 2, 26, 2, 12),
        ("prod3_o32_f16", 3, True, torch.float16, 32, 2, 1, 4, 2, 19, 1, 13),
    ]
    for name, bits, qjl, dtype, n_out, extra, B, Hq, Hkv, S, n_app, seed in ocases:
        k, v, q = synth(B, Hq, Hkv, S + n_app, seed, dtype)
        # a few channels carry more energy, as outlier channels of a real model do
        gg = torch.Generator().manual_seed(1000 + seed)
        boost = torch.ones(128)
        boost[torch.randperm(128, generator=gg)[:n_out]] = 4.0
        k, v = (k.float() * boost).to(dtype), (v.float() * boost).to(dtype)
        out = {"bits": np.int64(bits), "qjl": np.int64(qjl), "n_outlier": np.int64(n_out), "extra_bits": np.int64(extra),
               "B": np.int64(B), "Hq": np.int64(Hq), "Hkv": np.int64(Hkv), "S": np.int64(S), "n_append": np.int64(n_app),
               "dtype": np.array(str(dtype).replace("torch.", ""))}
        store(k, "k", out)
        store(v, "v", out)
        store(q, "q", out)
        layer = pc.PackedMSELayer(bits=bits, seed=0, num_outlier_channels=n_out, outlier_extra_bits=extra,
                                  use_qjl_keys=qjl, quantize_decode=True)
        layer.initialize_from_dense(k[:, :, :S].contiguous(), v[:, :, :S].contiguous())
        out["outlier_indices"] = layer._outlier_indices.numpy().copy()
        out["normal_indices"] = layer._normal_indices.numpy().copy()
        groups = Hq // Hkv

        def odump(tag):
            for part, kp, vp, kq in (("n", layer.keys_packed, layer.values_packed, layer._keys_qjl),
                                     ("o", layer._keys_outlier, layer._values_outlier, layer._keys_outlier_qjl)):
                out[f"{tag}_{part}_k_codes"] = kp.packed_indices.numpy().copy()
                out[f"{tag}_{part}_k_norms_bits16"] = bits16(kp.norms)
                out[f"{tag}_{part}_v_codes"] = vp.packed_indices.numpy().copy()
                out[f"{tag}_{part}_v_norms_bits16"] = bits16(vp.norms)
                if qjl:
                    out[f"{tag}_{part}_k_signs"] = kq.packed_signs.numpy().copy()
                    out[f"{tag}_{part}_k_rnorms_bits16"] = bits16(kq.residual_norms)
            out[f"{tag}_storage_bytes"] = np.int64(layer.storage_bytes())
            store(layer._decode_keys_full(), f"{tag}_k_dequant", out)
            store(layer._decode_values_full(), f"{tag}_v_dequant", out)
            store(chunked_turboquant_attention(q, layer, n_kv_groups=groups, chunk_size=8), f"{tag}_attn_chunked", out)

        odump("prefill")
        # (the reference's lazy update does not serve a split layer; its eager update does and
        # hands back the dequantised history followed by the new token)
        for t in range(n_app):
            ret_k, ret_v = layer.update(k[:, :, S + t:S + t + 1].contiguous(), v[:, :, S + t:S + t + 1].contiguous())
        store(ret_k, "update_ret_k", out)
        store(ret_v, "update_ret_v", out)
        odump("appended")
        np.savez_compressed(os.path.join(here, f"outlier_{name}.npz"), **out)
        print("outlier", name, "ok")

    # ---------------- norm guard -----------------------------------------------------
    ng: dict[str, np.ndarray] = {}
    k, v, _ = synth(1, 4, 4, 64, 11, torch.float32, mode="asym")
    k2, v2, _ = synth(1, 4, 4, 64, 12, torch.float32)
    cache = pc.build_packed_mse_cache([(k, v), (k2, v2), (k2 * 9.0, v2)], bits=4, use_qjl_keys=True,
                                      quantize_decode=True, norm_guard=True)
    ng["dense_flags"] = np.array([int(l._force_dense) for l in cache.layers])
    ng["mean_key_norms"] = np.array([float(t.float().norm(dim=-1).mean()) for t in (k, k2, k2 * 9.0)])
    ng["storage_bytes"] = np.array([l.storage_bytes() for l in cache.layers])
    np.savez_compressed(os.path.join(here, "norm_guard.npz"), **ng)

    # ---------------- end-to-end activate() on a tiny random Llama -----------------
    from transformers import LlamaConfig, LlamaForCausalLM

    def _mask_sizes(self, q):
        ql = q if isinstance(q, int) else q.shape[0]
        return self.get_seq_length() + ql, 0

    # Harness shim only: newer transformers pass an int query length here.
    pc.PackedMSELayer.get_mask_sizes = _mask_sizes

    class Tok:
        eos_token_id = None

        def decode(self, ids, skip_special_tokens=True):
            return " ".join(str(int(i)) for i in ids)

        def encode(self, text, add_special_tokens=False):
            return [int(t) for t in text.split()]

    e2e: dict[str, np.ndarray] = {}
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                      max_position_embeddings=512)
    model = LlamaForCausalLM(cfg).eval()
    ids = torch.randint(0, 512, (1, 48), generator=torch.Generator().manual_seed(5))
    e2e["input_ids"] = ids.numpy()
    for tag, kw in (("prod4", dict(bits=4, use_qjl_keys=True, quantize_decode=True)),
                    ("mse3_densetail", dict(bits=3, use_qjl_keys=False, quantize_decode=False))):
        turboquant.activate(model, Tok(), quiet=True, **kw)
        out_ids = model.generate(ids, max_new_tokens=8)
        tel = turboquant.last_telemetry(model)
        met = turboquant.last_metrics(model)
        turboquant.deactivate(model, quiet=True)
        e2e[f"{tag}_output_ids"] = out_ids.numpy()
        for key in ("dense_kv_bytes", "packed_estimate_bytes", "packed_actual_bytes",
                    "prompt_tokens", "completion_tokens", "qmse_bits"):
            e2e[f"{tag}_tel_{key}"] = np.int64(tel[key])
        e2e[f"{tag}_tel_keys"] = np.array(sorted(tel.keys()))
        e2e[f"{tag}_metrics_keys"] = np.array(sorted(met.keys()))
        e2e[f"{tag}_recon_keys"] = np.array(sorted(met["reconstruction_quality"][0].keys()))
        e2e[f"{tag}_recon_key_cos"] = np.array([r["key_cosine_sim"] for r in met["reconstruction_quality"]])
        e2e[f"{tag}_recon_val_cos"] = np.array([r["val_cosine_sim"] for r in met["reconstruction_quality"]])
    np.savez_compressed(os.path.join(here, "e2e_tiny_llama.npz"), **e2e)

    # ---------------- the unpacked "qmse" variant (quantise-dequantise in place) -----------------
    from turboquant.quantization.turboquant_mse import quantize_past_key_values_mse, quantize_vectors_mse
    from turboquant.runtime.generation import greedy_decode_with_prefill_cache

    qm: dict[str, np.ndarray] = {}
    g = torch.Generator().manual_seed(17)
    vec = torch.randn(257, 128, generator=g) * torch.exp(0.5 * torch.randn(257, 1, generator=g))
    vec[5] = 0.0  # a zero vector keeps norm 1
    qm["vectors"] = vec.numpy().copy()
    for bits, seed in ((3, 0), (4, 5)):
        rec, idx = quantize_vectors_mse(vec.numpy(), bits=bits, seed=seed)
        qm[f"rec_b{bits}_s{seed}"], qm[f"idx_b{bits}_s{seed}"] = rec, idx
    kv = tuple((torch.randn(1, 2, 9, 128, generator=g), torch.randn(1, 2, 9, 128, generator=g)) for _ in range(2))
    qm["kv"] = torch.stack([torch.stack(pair) for pair in kv]).numpy().copy()
    full = quantize_past_key_values_mse(kv, bits=4, seed=0)
    last = quantize_past_key_values_mse(kv, bits=4, seed=0, token_slice=slice(-1, None))
    qm["kv_full"] = torch.stack([torch.stack(list(pair)) for pair in full]).numpy().copy()
    qm["kv_last"] = torch.stack([torch.stack(list(pair)) for pair in last]).numpy().copy()
    out = greedy_decode_with_prefill_cache(model=model, tokenizer=Tok(), inputs={"input_ids": ids}, max_new_tokens=8,
                                           variant="qmse", qmse_bits=4)
    qm["gen_text_ids"] = np.array([int(t) for t in out.text.split()])
    qm["gen_metrics_keys"] = np.array(sorted(out.metrics.to_dict().keys()))
    qm["gen_qmse_bits"] = np.int64(out.metrics.qmse_bits)
    qm["gen_packed_estimate_total"] = np.int64(out.metrics.turboquant_mse_packed_estimate["total_bytes"]
                                               if "total_bytes" in out.metrics.turboquant_mse_packed_estimate
                                               else sum(v for v in out.metrics.turboquant_mse_packed_estimate.values()
                                                        if isinstance(v, (int, np.integer))))
    np.savez_compressed(os.path.join(here, "qmse.npz"), **qm)
    print("golden fixtures written to", here)


if __name__ == "__main__":
    main()
