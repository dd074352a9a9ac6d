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


class StoreView:
    """Tokens [lo, hi) of batch entry ``b`` of a PackedStore, shaped like a store of its own."""

    def __init__(self, store, b: int, lo: int, hi: int):
        sl = lambda t: None if t is None else t[b:b + 1, :, lo:hi]
        self.k_codes, self.k_norms, self.v_codes, self.v_norms = (sl(t) for t in (store.k_codes, store.k_norms,
                                                                                  store.v_codes, store.v_norms))
        self.k_signs, self.k_rnorms = sl(store.k_signs), sl(store.k_rnorms)
        self.length = hi - lo


def check_packed(store, ref: O.PackedLayer, k, v, p, what):
    """Codes, norms, QJL signs and residual norms of ``store`` (a PackedStore or a StoreView of
    one) against the oracle's layer ``ref`` built from the same ``k`` / ``v``."""
    n = ref.seq_len
    assert store.length == n
    k, v = k[:, :, :n], v[:, :, :n]
    exact_k = assert_codes_match(store.k_codes[:, :, :n], ref.k_codes, k, p.rot_k, p.bnd_k, p.key_bits, what + " keys")
    assert_codes_match(store.v_codes[:, :, :n], ref.v_codes, v, p.rot_v, p.bnd_v, p.bits, what + " values")
    assert fp16_ulp_diff(store.k_norms[:, :, :n].cpu(), ref.k_norms) <= 1
    assert fp16_ulp_diff(store.v_norms[:, :, :n].cpu(), ref.v_norms) <= 1
    if p.use_qjl:
        # Signs and residual norms are compared on vectors whose codes match exactly.  The residual
        # is taken against the reconstruction ROUNDED to the cache dtype (packed_qmse_cache.py:
        # 295-297), so two things decide how far fp32 summation order can move it:
        #  * an element of the fp32 reconstruction that sits on a rounding edge of that dtype
        #    becomes the other neighbour, a jump of one ulp of that element ("rounding edge", the
        #    same rule as "within 1e-6 of a decision boundary" for the codes);
        #  * a vector whose fp16 norm landed on the other side of an fp16 rounding edge (allowed
        #    above) is reconstructed 2^-11 larger or smaller, which re-rounds many elements.
        # Sign flips are accepted where the reference's projected residual is within 5e-3 of zero
        # plus what the vector's rounding edges can move it; residual norms may differ by one fp16
        # ulp plus the same reach.  Norm-edge vectors only get loose bounds.
        *_, proj = O.encode_keys_prod(k.contiguous(), p)
        proj = proj.reshape(-1, 128).abs()
        got = torch.from_numpy(O.unpack_codes(store.k_signs[:, :, :n].reshape(-1, 16).cpu().numpy(), 1, 128))
        want = torch.from_numpy(O.unpack_codes(ref.k_signs.reshape(-1, 16).numpy(), 1, 128))
        same_norm = (store.k_norms[:, :, :n].cpu().reshape(-1).view(torch.int16) ==
                     ref.k_norms.reshape(-1).view(torch.int16))
        rnorm = ref.k_rnorms.reshape(-1).float()
        if ref.dtype == torch.float32:
            edge_ulp = torch.zeros_like(proj)
        else:
            idx = torch.from_numpy(O.unpack_codes(ref.k_codes.reshape(-1, ref.k_codes.shape[-1]).numpy(),
                                                  p.key_bits, 128))
            norm = ref.k_norms.reshape(-1).float().unsqueeze(1)
            rec = (p.cen_k[idx] @ p.rot_k) * norm
            q = rec.to(ref.dtype).float()
            ulp = (torch.nextafter(q.to(ref.dtype), torch.tensor(float("inf"), dtype=ref.dtype)).float() - q).abs()
            on_edge = ((rec - q).abs() - ulp / 2).abs() < 1e-6 * norm  # fp32 summation error ~ 1e-7 |k|
            edge_ulp = on_edge * ulp
        reach = (edge_ulp @ p.qjl.abs().T) / rnorm.unsqueeze(1)  # how far each projection can move
        flips = (got != want) & exact_k.unsqueeze(1)
        judged = flips & same_norm.unsqueeze(1)
        assert (proj[judged] <= 5e-3 + 1.05 * reach[judged]).all(), what + ": QJL sign flips away from zero"
        assert (proj[flips] < 0.1).all() and flips.float().mean() < 1e-3
        rn_got = store.k_rnorms[:, :, :n].cpu().reshape(-1).float()
        ok = exact_k & same_norm
        fp16_ulp = torch.maximum(rnorm, torch.tensor(2.0 ** -14)).log2().floor().exp2() * 2.0 ** -10
        assert ((rn_got - rnorm).abs()[ok] <= (1.01 * fp16_ulp + 1.05 * edge_ulp.sum(dim=1))[ok]).all()
        edge = exact_k & ~same_norm
        assert ((rn_got - rnorm).abs()[edge] <= 1e-2 * rnorm[edge]).all()
        assert (~same_norm).float().mean() < 2e-3
