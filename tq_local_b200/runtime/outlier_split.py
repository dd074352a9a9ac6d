"""Outlier-channel split of the packed cache (``num_outlier_channels > 0``).

The reference (``src/turboquant/runtime/packed_qmse_cache.py:95-114,237-283,437-515``) picks the
``num_outlier_channels`` channels with the largest combined key + value energy on the prompt and
quantises them as a vector of their own with ``outlier_extra_bits`` more bits; the remaining
channels form a second vector quantised with ``bits``.  Each group has its own rotation, codebook
and - for Q_prod keys - QJL matrix, built for the group's dimension.

Neither group has 128 coordinates, and the sm_100a kernels of this library are written for
128-coordinate vectors, so this mode is served by tensor arithmetic on the cache's device: a
functional path with the reference's numbers (same tables, same rounding points), not a tuned
one.  ``SplitStore`` offers the part of ``PackedStore``'s interface that ``PackedMSELayer`` uses,
so the layer logic (lazy updates, dense tail, left-padding offsets, streaming prefill) is shared.
"""

from __future__ import annotations

from dataclasses import dataclass
from math import pi, sqrt

import torch

from tq_local_b200.quantization.turboquant_mse import build_scalar_codebook, random_rotation_matrix
from tq_local_b200.runtime.codec import QJL_SEED_OFFSET, generate_qjl_matrix

OUTLIER_SEED_OFFSET = 7919  # reference: packed_qmse_cache.py:117

# The library serves CUDA tensors only (``PackedMSELayer`` refuses anything else).  The arithmetic
# below is device-agnostic, which the CPU part of the test-suite uses to compare it bit for bit
# with fixtures the reference produced on a CPU: tests, and only tests, set this.
HOST_TENSORS_FOR_TESTS = False


def detect_outlier_channels(key_states: torch.Tensor, value_states: torch.Tensor,
                            num_outlier_channels: int) -> tuple[torch.Tensor, torch.Tensor]:
    """``(outlier_indices, normal_indices)``, both ascending: the channels ranked by the sum of
    squares of keys plus values over batch, heads and tokens (packed_qmse_cache.py:95-114)."""
    energy = key_states.float().square().sum(dim=(0, 1, 2)) + value_states.float().square().sum(dim=(0, 1, 2))
    top = torch.topk(energy, int(num_outlier_channels)).indices.sort().values
    keep = torch.ones(int(key_states.shape[-1]), dtype=torch.bool, device=key_states.device)
    keep[top] = False
    return top, torch.nonzero(keep).flatten()


# ---------------------------------------------------------------------------- bit streams
def pack_bit_fields(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """[T, D] integer codes -> uint8 [T, ceil(D * bits / 8)]: field j occupies bits
    [j * bits, (j + 1) * bits) of the row's little-endian bitstream, rows padded with zero bits
    (the layout of packed_qmse_cache.py:13-43).  A field spans at most two bytes (bits <= 8): its
    low part is added into byte ``j * bits // 8``, what overflows into the next one."""
    t, d = codes.shape
    row_bytes = -(-d * bits // 8)
    pos = torch.arange(d, device=codes.device) * bits
    shifted = codes.to(torch.int32) << (pos % 8).to(torch.int32)
    out = torch.zeros(t, row_bytes + 1, dtype=torch.int32, device=codes.device)
    out.index_add_(1, pos // 8, shifted & 0xFF)
    out.index_add_(1, pos // 8 + 1, shifted >> 8)
    return out[:, :row_bytes].to(torch.uint8)


def unpack_bit_fields(packed: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    """Inverse of ``pack_bit_fields``: uint8 [T, row_bytes] -> int64 [T, dim]."""
    t = packed.shape[0]
    padded = torch.cat((packed.to(torch.int32), torch.zeros(t, 1, dtype=torch.int32, device=packed.device)), dim=1)
    pos = torch.arange(dim, device=packed.device) * bits
    word = padded[:, pos // 8] | (padded[:, pos // 8 + 1] << 8)
    return ((word >> (pos % 8).to(torch.int32)) & ((1 << bits) - 1)).to(torch.int64)


# ---------------------------------------------------------------------------- one channel group
@dataclass
class GroupTables:
    """Rotation / codebook / QJL tables of one channel group, on the cache's device."""

    index: torch.Tensor   # int64 [dim]: the group's channels in the full vector
    dim: int
    bits: int             # value bits
    key_bits: int         # bits - 1 with QJL keys, else bits
    rot_v: torch.Tensor
    cen_v: torch.Tensor
    bnd_v: torch.Tensor
    rot_k: torch.Tensor
    cen_k: torch.Tensor
    bnd_k: torch.Tensor
    qjl: torch.Tensor | None

    @classmethod
    def build(cls, index: torch.Tensor, bits: int, use_qjl: bool, value_seed: int, qjl_seed: int, grid_size: int,
              device: torch.device) -> "GroupTables":
        dim = int(index.numel())

        def tables(b: int, seed: int):
            book = build_scalar_codebook(dimension=dim, bits=b, grid_size=grid_size)
            f32 = dict(dtype=torch.float32, device=device)
            return (torch.from_numpy(random_rotation_matrix(dimension=dim, seed=seed)).to(**f32),
                    torch.from_numpy(book.centers.astype("float32")).to(**f32),
                    torch.from_numpy(book.boundaries.astype("float32")).to(**f32))

        rot_v, cen_v, bnd_v = tables(bits, value_seed)
        if use_qjl:  # keys: their own rotation (seed + 1) and a codebook of one bit less (packed_qmse_cache.py:262-272)
            rot_k, cen_k, bnd_k = tables(bits - 1, value_seed + 1)
            qjl = generate_qjl_matrix(dim, qjl_seed).to(device)
        else:
            rot_k, cen_k, bnd_k, qjl = rot_v, cen_v, bnd_v, None
        return cls(index, dim, bits, bits - 1 if use_qjl else bits, rot_v, cen_v, bnd_v, rot_k, cen_k, bnd_k, qjl)


def _encode(x: torch.Tensor, rot: torch.Tensor, bnd: torch.Tensor, bits: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Rows of ``x`` [T, d] -> (bitstreams uint8 [T, row_bytes], fp16 norms [T]); norm 0 is stored
    as 1, a value equal to a boundary takes the lower bin (packed_qmse_cache.py:376-402)."""
    flat = x.float()
    norm = torch.linalg.norm(flat, dim=1)
    safe = torch.where(norm > 0, norm, torch.ones_like(norm))
    idx = torch.bucketize((flat / safe.unsqueeze(1)) @ rot.T, bnd)
    return pack_bit_fields(idx, bits), safe.to(torch.float16)


def _decode(codes: torch.Tensor, norms: torch.Tensor, rot: torch.Tensor, cen: torch.Tensor, bits: int, dim: int,
            dtype: torch.dtype) -> torch.Tensor:
    """(bitstreams [T, row_bytes], fp16 norms [T]) -> [T, dim] in ``dtype`` (packed_qmse_cache.py:404-435)."""
    idx = unpack_bit_fields(codes, bits, dim)
    return ((cen[idx] @ rot) * norms.float().unsqueeze(1)).to(dtype)


class _GroupStreams:
    """The packed streams of one channel group of one layer: [B, H, capacity, ...] with spare
    capacity, so that appending a token is an in-place write."""

    def __init__(self, g: GroupTables, batch: int, heads: int, capacity: int, use_qjl: bool, device: torch.device):
        self.g, self.use_qjl = g, use_qjl
        self.batch, self.heads = batch, heads
        self.device = device
        self.capacity = 0
        self.k_codes = self.k_norms = self.k_signs = self.k_rnorms = self.v_codes = self.v_norms = None
        self.reserve(capacity, 0)

    def _names(self) -> list[str]:
        return ["k_codes", "k_norms", "v_codes", "v_norms"] + (["k_signs", "k_rnorms"] if self.use_qjl else [])

    def reserve(self, capacity: int, length: int) -> None:
        if capacity <= self.capacity:
            return
        g, b, h = self.g, self.batch, self.heads
        widths = {"k_codes": -(-g.dim * g.key_bits // 8), "v_codes": -(-g.dim * g.bits // 8), "k_signs": -(-g.dim // 8)}
        for name in self._names():
            old = getattr(self, name)
            if name in widths:
                new = torch.zeros(b, h, capacity, widths[name], dtype=torch.uint8, device=self.device)
            else:
                new = torch.ones(b, h, capacity, dtype=torch.float16, device=self.device)
            if old is not None and length:
                new[:, :, :length] = old[:, :, :length]
            setattr(self, name, new)
        self.capacity = capacity

    def write(self, k: torch.Tensor, v: torch.Tensor, rows: slice, pos0: int) -> None:
        """Quantise this group's channels of ``k`` / ``v`` [b, H, T, D_full] into tokens
        [pos0, pos0 + T) of the batch rows ``rows``."""
        g = self.g
        b, h, t, _ = k.shape
        kg, vg = k[..., g.index].reshape(-1, g.dim), v[..., g.index].reshape(-1, g.dim)
        span = slice(pos0, pos0 + t)
        codes, norms = _encode(kg, g.rot_k, g.bnd_k, g.key_bits)
        self.k_codes[rows, :, span] = codes.view(b, h, t, -1)
        self.k_norms[rows, :, span] = norms.view(b, h, t)
        if self.use_qjl:
            # residual against the reconstruction rounded to the cache dtype; its norm (0 -> 1) and
            # the signs (0 -> +) of the unit residual's projection (packed_qmse_cache.py:285-310)
            rec = _decode(codes, norms, g.rot_k, g.cen_k, g.key_bits, g.dim, k.dtype)
            res = kg.float() - rec.float()
            rn = torch.linalg.norm(res, dim=1)
            rsafe = torch.where(rn > 0, rn, torch.ones_like(rn))
            proj = (res / rsafe.unsqueeze(1)) @ g.qjl.T
            self.k_signs[rows, :, span] = pack_bit_fields((proj >= 0).to(torch.int64), 1).view(b, h, t, -1)
            self.k_rnorms[rows, :, span] = rsafe.to(torch.float16).view(b, h, t)
        codes, norms = _encode(vg, g.rot_v, g.bnd_v, g.bits)
        self.v_codes[rows, :, span] = codes.view(b, h, t, -1)
        self.v_norms[rows, :, span] = norms.view(b, h, t)

    def read(self, which: str, lo: int, hi: int, dtype: torch.dtype) -> torch.Tensor:
        """Dequantised keys or values of tokens [lo, hi): [B, H, hi - lo, dim] in ``dtype``."""
        g = self.g
        b, h, t = self.batch, self.heads, hi - lo
        if which == "values":
            out = _decode(self.v_codes[:, :, lo:hi].reshape(b * h * t, -1), self.v_norms[:, :, lo:hi].reshape(-1),
                          g.rot_v, g.cen_v, g.bits, g.dim, dtype)
            return out.view(b, h, t, g.dim)
        out = _decode(self.k_codes[:, :, lo:hi].reshape(b * h * t, -1), self.k_norms[:, :, lo:hi].reshape(-1),
                      g.rot_k, g.cen_k, g.key_bits, g.dim, dtype)
        if self.use_qjl:  # packed_qmse_cache.py:312-330
            signs = 2.0 * unpack_bit_fields(self.k_signs[:, :, lo:hi].reshape(b * h * t, -1), 1, g.dim).float() - 1.0
            corr = (signs @ g.qjl) * self.k_rnorms[:, :, lo:hi].reshape(-1).float().unsqueeze(1) * (sqrt(pi / 2) / g.dim)
            out = out + corr.to(out.dtype)
        return out.view(b, h, t, g.dim)

    def nbytes(self, length: int) -> int:
        return sum(int(getattr(self, n)[:, :, :length].numel()) * getattr(self, n).element_size() for n in self._names())


class SplitStore:
    """Packed storage of one layer with the outlier-channel split; the subset of
    ``PackedStore``'s interface that ``PackedMSELayer`` calls."""

    ATTEND_CHUNK = 4096  # tokens dequantised at a time by ``decode_attn``

    def __init__(self, key_states: torch.Tensor, value_states: torch.Tensor, bits: int, num_outlier_channels: int,
                 outlier_extra_bits: int, use_qjl: bool, seed: int, grid_size: int, batch: int, capacity: int):
        device = key_states.device
        self.device, self.dtype = device, key_states.dtype
        self.full_dim = int(key_states.shape[-1])
        self.batch, self.kv_heads = int(batch), int(key_states.shape[1])
        self.use_qjl = bool(use_qjl)
        out_idx, norm_idx = detect_outlier_channels(key_states, value_states, num_outlier_channels)
        qjl_seed = seed + QJL_SEED_OFFSET
        out_seed = seed + OUTLIER_SEED_OFFSET
        self.normal = GroupTables.build(norm_idx, bits, use_qjl, seed, qjl_seed, grid_size, device)
        self.outlier = GroupTables.build(out_idx, bits + outlier_extra_bits, use_qjl, out_seed, qjl_seed + 1, grid_size, device)
        self.length = 0
        self._seq_start: torch.Tensor | None = None
        cap = max(8, int(capacity))
        self.groups = [_GroupStreams(g, self.batch, self.kv_heads, cap, self.use_qjl, device) for g in (self.normal, self.outlier)]
        self.capacity = cap

    # ------------------------------------------------------------------ storage
    def reserve(self, capacity: int) -> None:
        if capacity > self.capacity:
            capacity = max(int(capacity), 2 * self.capacity)
            for gs in self.groups:
                gs.reserve(capacity, self.length)
            self.capacity = capacity

    def set_seq_start(self, seq_start: torch.Tensor | None) -> None:
        self._seq_start = seq_start

    def storage_bytes(self) -> int:
        return sum(gs.nbytes(self.length) for gs in self.groups)

    def pack(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """Append ``k`` / ``v`` [B, H, T, D] at the end of every row."""
        t = int(k.shape[2])
        self.reserve(self.length + t)
        for gs in self.groups:
            gs.write(k, v, slice(0, self.batch), self.length)
        self.length += t

    def pack_rows(self, k: torch.Tensor, v: torch.Tensor, b0: int, pos0: int = 0) -> None:
        """Write ``k`` / ``v`` [b, H, T, D] into batch rows [b0, b0 + b) at tokens [pos0, pos0 + T)
        (a prompt pass that runs the batch a few rows at a time); the caller sets ``length``."""
        self.reserve(pos0 + int(k.shape[2]))
        for gs in self.groups:
            gs.write(k, v, slice(b0, b0 + int(k.shape[0])), pos0)

    def dequant(self, which: str, lo: int = 0, hi: int | None = None, dtype: torch.dtype | None = None) -> torch.Tensor:
        """Dequantised keys or values of tokens [lo, hi) with the two groups' channels put back in
        place: [B, H, hi - lo, D] (packed_qmse_cache.py:456-515)."""
        hi = self.length if hi is None else hi
        dtype = dtype or self.dtype
        full = torch.zeros(self.batch, self.kv_heads, hi - lo, self.full_dim, dtype=dtype, device=self.device)
        for gs in self.groups:
            full[..., gs.g.index] = gs.read(which, lo, hi, dtype)
        return full

    # ------------------------------------------------------------------ attention
    def decode_attn(self, q: torch.Tensor, *, seq_len: int | None = None, tail_k: torch.Tensor | None = None,
                    tail_v: torch.Tensor | None = None) -> torch.Tensor:
        """Attention of ``q`` [B, Hq, 1, D] over tokens [seq_start[b], seq_len) of the packed cache
        followed by the dense tail, chunk by chunk with a running maximum and sum in fp32: what the
        reference's chunked path computes for such a layer (attention.py:215-304)."""
        n = self.length if seq_len is None else int(seq_len)
        b, hq, _, d = q.shape
        groups = hq // self.kv_heads
        qf = q.float().view(b, self.kv_heads, groups, d) * (1.0 / sqrt(d))
        m = torch.full((b, self.kv_heads, groups), float("-inf"), device=q.device)
        l = torch.zeros_like(m)
        acc = torch.zeros(b, self.kv_heads, groups, d, device=q.device)

        def step(k: torch.Tensor, v: torch.Tensor, first_token: int | None) -> None:
            nonlocal m, l, acc
            logits = torch.einsum("bhgd,bhtd->bhgt", qf, k.float())
            if first_token is not None and self._seq_start is not None:
                tok = torch.arange(first_token, first_token + k.shape[2], device=q.device)
                hidden = tok.view(1, -1) < self._seq_start.view(-1, 1)
                logits = logits.masked_fill(hidden.view(b, 1, 1, -1), float("-inf"))
            m_new = torch.maximum(m, logits.amax(dim=-1))
            m_safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
            scale = torch.exp(m - m_safe)
            p = torch.exp(logits - m_safe.unsqueeze(-1))
            l = l * scale + p.sum(dim=-1)
            acc = acc * scale.unsqueeze(-1) + torch.einsum("bhgt,bhtd->bhgd", p, v.float())
            m = m_new

        for lo in range(0, n, self.ATTEND_CHUNK):
            hi = min(n, lo + self.ATTEND_CHUNK)
            step(self.dequant("keys", lo, hi, q.dtype), self.dequant("values", lo, hi, q.dtype), lo)
        if tail_k is not None and tail_k.shape[2]:
            step(tail_k, tail_v, None)
        return (acc / l.clamp(min=1e-8).unsqueeze(-1)).to(q.dtype).view(b, hq, 1, d)  # (clamp: attention.py:303)
