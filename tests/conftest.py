"""Shared pytest set-up: the ``gpu`` marker, import path and golden-fixture loader."""

from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}

LAYER_CASES = ["mse4_f32", "prod4_bf16", "prod3_bf16", "mse3_f32", "prod2_f16", "mse2_bf16", "prod4_f32"]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class Golden:
    """One ``.npz`` fixture; 16-bit float tensors come back in their real dtype."""

    def __init__(self, name: str):
        self.z = np.load(os.path.join(GOLDEN, name + ".npz"))
        self.dtype = _DTYPES[str(self.z["dtype"])] if "dtype" in self.z else torch.float32

    def __contains__(self, key):
        return key in self.z or key + "_bits16" in self.z

    def t(self, key: str, dtype: torch.dtype | None = None) -> torch.Tensor:
        if key in self.z:
            return torch.from_numpy(self.z[key].copy())
        raw = torch.from_numpy(self.z[key + "_bits16"].copy())
        return raw.view(dtype or self.dtype)

    def i(self, key: str) -> int:
        return int(self.z[key])


@pytest.fixture(scope="session")
def setup_golden():
    return Golden("setup")


def load_layer_case(name: str) -> Golden:
    return Golden("layer_" + name)
