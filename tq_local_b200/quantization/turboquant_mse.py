"""Host-side codec set-up: Lloyd-Max scalar codebook and the seeded rotation.

These run once per (head_dim, bits, seed) on the CPU in float64 and are passed
to the CUDA library as data.  They reproduce, number for number, what the
reference builds in ``src/turboquant/quantization/turboquant_mse.py:37-121``
(``build_scalar_codebook`` and ``random_rotation_matrix``): the same numpy
calls in the same order, so the float32 tables are bit-identical on the same
host.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from functools import lru_cache

import numpy as np


@dataclass(frozen=True)
class ScalarCodebook:
    dimension: int
    bits: int
    centers: np.ndarray
    boundaries: np.ndarray
    grid_size: int


class _SphereCoordinateLaw:
    """Density of one coordinate of a uniform point on the unit sphere in R^dimension,
    tabulated on a uniform grid over [-1, 1] (reference ``_sphere_coordinate_density``,
    ``_cdf_from_density``, ``_conditional_mean``: turboquant_mse.py:37-67)."""

    def __init__(self, dimension: int, grid_size: int) -> None:
        self.grid = np.linspace(-1.0, 1.0, grid_size, dtype=np.float64)
        norm_const = math.gamma(dimension / 2.0) / (math.sqrt(np.pi) * math.gamma((dimension - 1.0) / 2.0))
        pdf = np.zeros_like(self.grid, dtype=np.float64)
        support = np.abs(self.grid) <= 1.0
        pdf[support] = norm_const * np.power(1.0 - np.square(self.grid[support]), (dimension - 3.0) / 2.0)
        self.pdf = pdf

    def cdf(self) -> np.ndarray:
        step = self.grid[1] - self.grid[0]
        total = np.cumsum(self.pdf) * step
        total /= total[-1]
        total[0] = 0.0
        total[-1] = 1.0
        return total

    def mean_between(self, lo: float, hi: float) -> float:
        midpoint = (lo + hi) / 2.0
        if hi <= lo:
            return midpoint
        window = (self.grid >= lo) & (self.grid <= hi)
        xs = self.grid[window]
        if xs.size == 0:
            return midpoint
        ws = self.pdf[window]
        mass = np.trapezoid(ws, xs)
        if mass <= 0:
            return midpoint
        return float(np.trapezoid(xs * ws, xs) / mass)


@lru_cache(maxsize=32)
def build_scalar_codebook(
    dimension: int,
    bits: int,
    grid_size: int = 32769,
    max_iters: int = 200,
    tol: float = 1e-10,
) -> ScalarCodebook:
    """Lloyd-Max quantiser with ``2**bits`` levels for the sphere-coordinate law."""
    if bits <= 0:
        raise ValueError("bits must be positive for TurboQuant_mse.")
    n_levels = 2 ** bits
    law = _SphereCoordinateLaw(dimension, grid_size)
    probs = np.linspace(0.0, 1.0, n_levels + 2, dtype=np.float64)[1:-1]
    centers = np.interp(probs, law.cdf(), law.grid)

    for _ in range(max_iters):
        cuts = (centers[:-1] + centers[1:]) / 2.0
        edges = np.concatenate(([-1.0], cuts, [1.0]))
        moved = np.array([law.mean_between(edges[i], edges[i + 1]) for i in range(n_levels)], dtype=np.float64)
        converged = np.max(np.abs(moved - centers)) < tol
        centers = moved
        if converged:
            break

    return ScalarCodebook(
        dimension=dimension,
        bits=bits,
        centers=centers,
        boundaries=(centers[:-1] + centers[1:]) / 2.0,
        grid_size=grid_size,
    )


@lru_cache(maxsize=16)
def random_rotation_matrix(dimension: int, seed: int) -> np.ndarray:
    """Haar-ish random orthogonal matrix: QR of a seeded Gaussian with the sign of
    diag(R) folded into Q, as float32."""
    gauss = np.random.default_rng(seed).standard_normal((dimension, dimension))
    q, r = np.linalg.qr(gauss)
    flip = np.sign(np.diag(r))
    flip[flip == 0.0] = 1.0
    return (q * flip).astype(np.float32)


# ---------------------------------------------------------------------------------------------
# The unpacked "qmse" variant: quantise and dequantise in place, nothing is packed (reference:
# turboquant_mse.py:124-217).  It exists to look at quantisation error without the packed cache;
# it saves no memory and is not on the accelerated path, so it is written with plain tensor
# operations on whatever device the tensors live on (the reference moves them to the CPU and
# uses numpy; the arithmetic - float32, same operations in the same order - is the same).

def quantize_vectors_mse(vectors, bits: int, seed: int = 0, grid_size: int = 32769):
    """``[num_vectors, dimension]`` -> (reconstruction float32, indices int16); reference
    ``quantize_vectors_mse`` (turboquant_mse.py:124-147).  A value equal to a boundary goes to the
    UPPER bin here (``np.digitize(right=False)``), unlike the packed path's ``bucketize``."""
    import torch

    t = torch.as_tensor(vectors)
    if t.dim() != 2:
        raise ValueError(f"Expected shape [num_vectors, dimension], got {tuple(t.shape)}.")
    x = t.to(torch.float32)
    dimension = int(x.shape[1])
    codebook = build_scalar_codebook(dimension=dimension, bits=bits, grid_size=grid_size)
    rotation = torch.from_numpy(random_rotation_matrix(dimension=dimension, seed=seed)).to(x.device)
    centers = torch.from_numpy(codebook.centers.astype(np.float32)).to(x.device)
    bounds = torch.from_numpy(codebook.boundaries.astype(np.float32)).to(x.device)
    norms = torch.linalg.vector_norm(x, dim=1, keepdim=True)
    safe = torch.where(norms > 0, norms, torch.ones_like(norms))
    rotated = (x / safe) @ rotation.T
    indices = torch.bucketize(rotated, bounds, right=True)  # == np.digitize(rotated, bounds, right=False)
    reconstructed = (centers[indices] @ rotation) * safe
    if isinstance(vectors, np.ndarray):
        return reconstructed.numpy(), indices.to(torch.int16).numpy()
    return reconstructed, indices.to(torch.int16)


def reconstruct_tensor_mse(tensor, bits: int, seed: int = 0, grid_size: int = 32769):
    """Quantise-dequantise a ``[..., dimension]`` tensor, keeping its device and dtype
    (reference: turboquant_mse.py:150-166)."""
    shape = tensor.shape
    rec, _ = quantize_vectors_mse(tensor.detach().reshape(-1, shape[-1]), bits=bits, seed=seed, grid_size=grid_size)
    return rec.reshape(shape).to(dtype=tensor.dtype)


def quantize_past_key_values_mse(past_key_values, bits: int, seed: int = 0, grid_size: int = 32769,
                                 token_slice: slice | None = None):
    """Replace every layer's keys and values (or the tokens of ``token_slice``) of an HF cache, or of
    a tuple / list of per-layer (key, value, ...) entries, by their quantise-dequantise
    reconstruction (reference: turboquant_mse.py:169-217)."""
    import torch

    def selected(t):
        if token_slice is None:
            return reconstruct_tensor_mse(t, bits=bits, seed=seed, grid_size=grid_size)
        updated = t.clone()
        updated[:, :, token_slice, :] = reconstruct_tensor_mse(t[:, :, token_slice, :], bits=bits, seed=seed,
                                                               grid_size=grid_size)
        return updated

    if hasattr(past_key_values, "layers"):
        for layer in past_key_values.layers:
            if getattr(layer, "keys", None) is None or getattr(layer, "values", None) is None:
                continue
            layer.keys, layer.values = selected(layer.keys), selected(layer.values)
        return past_key_values
    if isinstance(past_key_values, (tuple, list)):
        out = []
        for entry in past_key_values:
            if not isinstance(entry, (tuple, list)):
                raise TypeError(f"Unsupported layer cache type: {type(entry)!r}")
            items = list(entry)
            where = [i for i, item in enumerate(items) if torch.is_tensor(item)]
            if len(where) < 2:
                raise ValueError(f"Expected at least two tensor entries in a layer cache, got {len(where)}.")
            items[where[0]], items[where[1]] = selected(items[where[0]]), selected(items[where[1]])
            out.append(tuple(items) if isinstance(entry, tuple) else items)
        return tuple(out) if isinstance(past_key_values, tuple) else out
    raise TypeError(f"Unsupported past_key_values type: {type(past_key_values)!r}")
