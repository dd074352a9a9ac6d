"""CPU-side checks of the C-ABI boundary: the library builds, loads, and exports every
symbol the public header declares (no compute calls: there is no GPU here)."""

from __future__ import annotations

import ctypes
import os
import re

import pytest

from conftest import ROOT


def _declared_functions() -> list[str]:
    text = open(os.path.join(ROOT, "include", "tq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tq_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_agree():
    from tq_local_b200.runtime import ffi

    assert sorted(ffi.EXPORTS) == _declared_functions()


def test_library_builds_and_exports_every_symbol():
    import __graft_entry__ as entry
    from tq_local_b200.runtime import ffi

    entry.build()
    lib = ctypes.CDLL(ffi.LIB_PATH)
    for name in _declared_functions():
        assert hasattr(lib, name), name
    assert ffi.lib().tq_abi_version() == 1


def test_workspace_size_contract():
    from tq_local_b200.runtime import ffi

    L = ffi.lib()
    assert L.tq_decode_workspace_bytes(0, 32, 4) == 0
    small, big = L.tq_decode_workspace_bytes(1, 32, 1), L.tq_decode_workspace_bytes(8, 32, 16)
    assert small % 256 == 0 and big > small
    # rotated + projected query, and (max, sum, acc[128]) per split, in fp32
    assert big >= 8 * 32 * (2 * 128 + 16 * 130) * 4


def test_no_cpu_fallback():
    """Without a CUDA device the product refuses to run instead of falling back."""
    import torch

    from tq_local_b200.runtime import ffi
    from tq_local_b200.runtime.codec import Codec

    with pytest.raises(ffi.TQError):
        Codec(torch.device("cpu"), 4, True)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from tq_local_b200.runtime import ffi

    monkeypatch.setattr(ffi, "_lib", None)
    monkeypatch.setattr(ffi, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ffi.TQError, match="missing"):
        ffi.lib()


def test_host_tables_match_reference_golden(setup_golden):
    """The product's own host set-up (not the oracle) reproduces the reference tables."""
    import numpy as np

    from tq_local_b200.quantization import build_scalar_codebook, random_rotation_matrix
    from tq_local_b200.runtime.codec import generate_qjl_matrix

    for bits in (1, 2, 3, 4):
        cb = build_scalar_codebook(128, bits)
        np.testing.assert_array_equal(cb.centers, setup_golden.z[f"centers_b{bits}"])
        np.testing.assert_array_equal(cb.boundaries, setup_golden.z[f"boundaries_b{bits}"])
    for seed in (0, 1, 7):
        np.testing.assert_allclose(random_rotation_matrix(128, seed), setup_golden.z[f"rotation_s{seed}"], atol=2e-6)
    np.testing.assert_array_equal(generate_qjl_matrix(128, 31337).numpy(), setup_golden.z["qjl_s31337"])
    with pytest.raises(ValueError):
        build_scalar_codebook(128, 0)
