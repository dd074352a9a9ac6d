"""Outlier-channel split (``num_outlier_channels > 0``): the product's tensor-arithmetic path and
the oracle's restatement against fixtures produced by the unmodified reference
(``tests/golden/make_golden.py``, files ``outlier_*.npz``)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import Golden
from oracle import tq_oracle as O

CASES = ("mse3_o8_f32", "prod4_o16_bf16", "prod3_o32_f16")


def _load(name: str):
    g = Golden(f"outlier_{name}")
    z = g.z
    dt = getattr(torch, str(z["dtype"]))

    def t(key: str) -> torch.Tensor:
        if key + "_bits16" in z:
            return torch.from_numpy(z[key + "_bits16"].copy()).view(dt)
        return torch.from_numpy(z[key].copy())

    cfg = dict(bits=int(z["bits"]), n_out=int(z["n_outlier"]), extra=int(z["extra_bits"]), qjl=bool(z["qjl"]),
               S=int(z["S"]), n_app=int(z["n_append"]), groups=int(z["Hq"]) // int(z["Hkv"]))
    return z, dt, t, cfg


def _bits16(x: torch.Tensor) -> np.ndarray:
    return x.contiguous().view(torch.int16).cpu().numpy()


@pytest.mark.parametrize("name", CASES)
def test_oracle_split_matches_reference(name):
    z, dt, t, c = _load(name)
    k, v, q = t("k"), t("v"), t("q")
    S = c["S"]
    layer = O.pack_layer_split(k[:, :, :S].contiguous(), v[:, :, :S].contiguous(), c["bits"], c["n_out"], c["extra"], c["qjl"])
    assert np.array_equal(layer.idx_o.numpy(), z["outlier_indices"])
    assert np.array_equal(layer.idx_n.numpy(), z["normal_indices"])

    def check(tag: str, layer) -> None:
        for part, pl in (("n", layer.normal), ("o", layer.outlier)):
            assert np.array_equal(pl.k_codes.numpy(), z[f"{tag}_{part}_k_codes"])
            assert np.array_equal(pl.v_codes.numpy(), z[f"{tag}_{part}_v_codes"])
            assert np.array_equal(_bits16(pl.k_norms), z[f"{tag}_{part}_k_norms_bits16"])
            assert np.array_equal(_bits16(pl.v_norms), z[f"{tag}_{part}_v_norms_bits16"])
            if c["qjl"]:
                assert np.array_equal(pl.k_signs.numpy(), z[f"{tag}_{part}_k_signs"])
                assert np.array_equal(_bits16(pl.k_rnorms), z[f"{tag}_{part}_k_rnorms_bits16"])
        assert layer.storage_bytes() == int(z[f"{tag}_storage_bytes"])
        assert torch.equal(O.dequant_keys(layer), t(f"{tag}_k_dequant"))
        assert torch.equal(O.dequant_values(layer), t(f"{tag}_v_dequant"))
        assert torch.equal(O.attend_chunked(q, layer, c["groups"], chunk=8), t(f"{tag}_attn_chunked"))

    check("prefill", layer)
    for i in range(c["n_app"]):
        layer = O.append_tokens_split(layer, k[:, :, S + i:S + i + 1].contiguous(), v[:, :, S + i:S + i + 1].contiguous())
    check("appended", layer)


def test_bit_fields_round_trip_and_known_bytes(setup_golden):
    from tq_local_b200.runtime.outlier_split import pack_bit_fields, unpack_bit_fields

    g = torch.Generator().manual_seed(3)
    for bits in (1, 2, 3, 4, 5, 6):
        for dim in (8, 13, 96, 120, 128):
            codes = torch.randint(0, 2 ** bits, (7, dim), generator=g)
            packed = pack_bit_fields(codes, bits)
            assert packed.shape == (7, -(-dim * bits // 8)) and packed.dtype == torch.uint8
            assert np.array_equal(packed.numpy(), O.pack_codes(codes.numpy(), bits))
            assert torch.equal(unpack_bit_fields(packed, bits, dim), codes)
    # the reference's own bytes (known-answer vectors)
    for bits in (1, 2, 3, 4):
        idx = torch.from_numpy(setup_golden.z[f"packkat_idx_b{bits}"])
        assert np.array_equal(pack_bit_fields(idx, bits).numpy(), setup_golden.z[f"packkat_bytes_b{bits}"])
    idx = torch.from_numpy(setup_golden.z["packkat_idx_ragged"])
    assert np.array_equal(pack_bit_fields(idx, 3).numpy(), setup_golden.z["packkat_bytes_ragged"])


def _run_product(name: str, device: str, exact: bool) -> None:
    """The product's layer on ``device`` against the reference's outputs.  On the CPU (where the
    reference ran) everything is bit-identical; on a GPU the matrix products are summed in another
    order, so codes may differ for coordinates on a decision boundary and the comparison goes
    through the dequantised tensors and the attention output."""
    from tq_local_b200.runtime.attention import chunked_turboquant_attention
    from tq_local_b200.runtime.packed_qmse_cache import PackedMSELayer

    z, dt, t, c = _load(name)
    k, v, q = t("k").to(device), t("v").to(device), t("q").to(device)
    S = c["S"]
    layer = PackedMSELayer(bits=c["bits"], seed=0, num_outlier_channels=c["n_out"], outlier_extra_bits=c["extra"],
                           use_qjl_keys=c["qjl"], quantize_decode=True)
    layer.initialize_from_dense(k[:, :, :S].contiguous(), v[:, :, :S].contiguous())
    assert layer._outlier_enabled and not layer.supports_static_decode(int(z["Hq"]))
    assert np.array_equal(layer._outlier_indices.cpu().numpy(), z["outlier_indices"])
    assert np.array_equal(layer._normal_indices.cpu().numpy(), z["normal_indices"])
    tol = 1e-5 if dt == torch.float32 else 4e-3

    def check(tag: str) -> None:
        views = (("n", layer.keys_packed, layer.values_packed, layer._keys_qjl),
                 ("o", layer._keys_outlier, layer._values_outlier, layer._keys_outlier_qjl))
        for part, kp, vp, kq in views:
            ref_k, ref_v = z[f"{tag}_{part}_k_codes"], z[f"{tag}_{part}_v_codes"]
            assert kp.packed_indices.shape == ref_k.shape and vp.packed_indices.shape == ref_v.shape
            same_k = kp.packed_indices.cpu().numpy() == ref_k
            same_v = vp.packed_indices.cpu().numpy() == ref_v
            if exact:
                assert same_k.all() and same_v.all()
                assert np.array_equal(_bits16(kp.norms), z[f"{tag}_{part}_k_norms_bits16"])
                assert np.array_equal(_bits16(vp.norms), z[f"{tag}_{part}_v_norms_bits16"])
                if c["qjl"]:
                    assert np.array_equal(kq.packed_signs.cpu().numpy(), z[f"{tag}_{part}_k_signs"])
                    assert np.array_equal(_bits16(kq.residual_norms), z[f"{tag}_{part}_k_rnorms_bits16"])
            else:
                assert same_k.mean() > 0.995 and same_v.mean() > 0.995
        assert layer.storage_bytes() == int(z[f"{tag}_storage_bytes"])
        for got, key in ((layer._decode_keys_full(), f"{tag}_k_dequant"), (layer._decode_values_full(), f"{tag}_v_dequant")):
            ref = t(key).float()
            if exact:
                assert torch.equal(got.cpu().float(), ref)
            else:  # a code on a boundary moves one coordinate by one bin: bounded, and rare
                diff = (got.cpu().float() - ref).abs()
                assert float(diff.max()) <= 0.5 * float(ref.abs().max()) and float((diff > 1e-2 * ref.abs().max()).float().mean()) < 5e-3
        att = chunked_turboquant_attention(q, layer, n_kv_groups=c["groups"]).cpu().float()
        ref = t(f"{tag}_attn_chunked").float()
        assert float((att - ref).abs().max()) <= (tol if exact else 2e-2) * float(ref.abs().max())

    check("prefill")
    for i in range(c["n_app"]):
        ret_k, ret_v = layer.update(k[:, :, S + i:S + i + 1].contiguous(), v[:, :, S + i:S + i + 1].contiguous())
    if exact:  # the eager update hands back the dequantised history followed by the new token
        assert torch.equal(ret_k.cpu(), t("update_ret_k")) and torch.equal(ret_v.cpu(), t("update_ret_v"))
    check("appended")

    # lazy updates (what the attention backend uses) store the same bytes as eager ones
    lazy = PackedMSELayer(bits=c["bits"], seed=0, num_outlier_channels=c["n_out"], outlier_extra_bits=c["extra"],
                          use_qjl_keys=c["qjl"], quantize_decode=True)
    lazy.initialize_from_dense(k[:, :, :S].contiguous(), v[:, :, :S].contiguous())
    lazy._lazy_update = True
    for i in range(c["n_app"]):
        out_k, _ = lazy.update(k[:, :, S + i:S + i + 1].contiguous(), v[:, :, S + i:S + i + 1].contiguous())
        assert out_k.shape[2] == 1
    assert torch.equal(lazy.keys_packed.packed_indices, layer.keys_packed.packed_indices)
    assert torch.equal(lazy._values_outlier.packed_indices, layer._values_outlier.packed_indices)
    assert lazy.get_seq_length() == S + c["n_app"]

    # a left-padded batch attends only the tokens after its padding
    B = int(k.shape[0])
    start = torch.tensor([3] + [0] * (B - 1), dtype=torch.int32, device=device)
    mask2d = (torch.arange(S + c["n_app"], device=device).view(1, -1) >= start.view(-1, 1)).to(torch.int64)
    got = chunked_turboquant_attention(q, layer, n_kv_groups=c["groups"], attention_mask=mask2d).cpu().float()
    kd, vd = layer._decode_keys_full().cpu().float(), layer._decode_values_full().cpu().float()
    kd[0, :, :3] = 0
    logits = (q.cpu().float() @ kd.repeat_interleave(c["groups"], 1).transpose(-1, -2)) / np.sqrt(128)
    logits[0, :, :, :3] = float("-inf")
    want = torch.softmax(logits, -1) @ vd.repeat_interleave(c["groups"], 1)
    assert float((got - want).abs().max()) <= (2e-5 if dt == torch.float32 else 4e-3) * float(want.abs().max())


@pytest.mark.parametrize("name", CASES)
def test_product_split_matches_reference_on_host_tensors(name, monkeypatch):
    from tq_local_b200.runtime import ffi, outlier_split
    from tq_local_b200.runtime.packed_qmse_cache import PackedMSELayer

    layer = PackedMSELayer(bits=4, num_outlier_channels=8)
    with pytest.raises(ffi.TQError):  # the library itself serves CUDA tensors only
        layer.initialize_from_dense(torch.randn(1, 2, 4, 128), torch.randn(1, 2, 4, 128))
    monkeypatch.setattr(outlier_split, "HOST_TENSORS_FOR_TESTS", True)
    _run_product(name, "cpu", exact=True)


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_product_split_on_gpu(name):
    _run_product(name, "cuda", exact=False)


@pytest.mark.gpu
def test_generate_with_outlier_split():
    """activate(num_outlier_channels=...) -> generate(): eager decode steps through the split layers;
    same tokens as the run without the split for nearly every position (both quantise the same
    random-init model's cache at 4 bits)."""
    import turboquant
    from test_gpu_adapter import StubTokenizer, _tiny_model  # the tiny random Llama of the adapter tests

    model = _tiny_model().cuda()
    ids = torch.randint(0, 512, (2, 40), generator=torch.Generator().manual_seed(5)).cuda()
    turboquant.activate(model, StubTokenizer(), quiet=True, bits=4, use_qjl_keys=True, verify=False)
    base = model.generate(ids, max_new_tokens=8)
    turboquant.deactivate(model, quiet=True)
    turboquant.activate(model, StubTokenizer(), quiet=True, bits=4, use_qjl_keys=True, num_outlier_channels=16, verify=False)
    out = model.generate(ids, max_new_tokens=8)
    tel = turboquant.last_telemetry(model)
    turboquant.deactivate(model, quiet=True)
    assert out.shape == base.shape and torch.equal(out[:, :40], ids)
    assert tel is not None
    assert float((out[:, 40:] == base[:, 40:]).float().mean()) >= 0.5
