"""Helpers shared by the GPU parity tests (test infrastructure; may use the oracle)."""

from __future__ import annotations

import numpy as np
import torch

from oracle import tq_oracle as O


def make_codec(bits, qjl, setup_golden, device="cuda"):
    from tq_local_b200.runtime.codec import Codec

    return Codec(torch.device(device, torch.cuda.current_device()), bits, qjl, seed=0,
                 rot_v=setup_golden.z["rotation_s0"], rot_k=setup_golden.z["rotation_s1"])


def oracle_params(bits, qjl, setup_golden):
    return O.QuantParams.build(128, bits, qjl, seed=0, rot_v=setup_golden.z["rotation_s0"],
                               rot_k=setup_golden.z["rotation_s1"])


def load_into_store(store, layer: O.PackedLayer):
    """Copy an oracle/golden packed layer into a device store (bypasses the encoder)."""
    n = layer.seq_len
    store.reserve(n)
    store.k_codes[:, :, :n].copy_(layer.k_codes)
    store.k_norms[:, :, :n].copy_(layer.k_norms)
    store.v_codes[:, :, :n].copy_(layer.v_codes)
    store.v_norms[:, :, :n].copy_(layer.v_norms)
    if layer.k_signs is not None:
        store.k_signs[:, :, :n].copy_(layer.k_signs)
        store.k_rnorms[:, :, :n].copy_(layer.k_rnorms)
    store.length = n


def store_to_layer(store, p, dtype) -> O.PackedLayer:
    n = store.length
    c = lambda t: None if t is None else t[:, :, :n].contiguous().cpu()
    return O.PackedLayer(p, dtype, c(store.k_codes), c(store.k_norms), c(store.v_codes), c(store.v_norms),
                         c(store.k_signs), c(store.k_rnorms))


def fp16_ulp_diff(a: torch.Tensor, b: torch.Tensor) -> int:
    """Largest distance in fp16 ulps (positive finite values)."""
    ai = a.contiguous().view(torch.int16).to(torch.int32)
    bi = b.contiguous().view(torch.int16).to(torch.int32)
    return int((ai - bi).abs().max()) if ai.numel() else 0


def assert_codes_match(got: torch.Tensor, ref: torch.Tensor, x: torch.Tensor, rot, bnd, bits: int, what: str):
    """Codes must be bit-exact except elements whose rotated fp32 value lies within 1e-6
    of a decision boundary.  Returns the boolean mask [vectors] of fully exact vectors."""
    got2 = got.reshape(-1, got.shape[-1]).cpu().numpy()
    ref2 = ref.reshape(-1, ref.shape[-1]).cpu().numpy()
    gi = O.unpack_codes(got2, bits, 128)
    ri = O.unpack_codes(ref2, bits, 128)
    diff = gi != ri
    if diff.any():
        z, _ = O.rotate_unit(x, rot)
        dist = (z.unsqueeze(-1) - bnd).abs().min(-1).values.numpy()
        bad = diff & (dist >= 1e-6)
        assert not bad.any(), f"{what}: {int(bad.sum())} code mismatches outside the 1e-6 boundary band"
        assert (np.abs(gi - ri)[diff] == 1).all(), f"{what}: mismatching codes are not neighbouring bins"
    return torch.from_numpy(~diff.any(axis=1))


def rel_inf(a: torch.Tensor, ref: torch.Tensor) -> float:
    return float((a.float().cpu() - ref.float().cpu()).abs().max() / ref.float().abs().max())
