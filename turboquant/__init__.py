"""Drop-in alias: ``import turboquant`` resolves to the B200 implementation.

Code written against the reference package (``turboquant.activate(model, tokenizer, bits=...,
use_qjl_keys=..., quantize_decode=..., norm_guard=...)``, ``deactivate``, ``last_telemetry`` ...)
runs unchanged; the sub-modules ``turboquant.runtime.*``, ``turboquant.adapters.*``,
``turboquant.quantization.*`` and ``turboquant.telemetry`` are aliases of the matching
``tq_local_b200`` modules.
"""

from __future__ import annotations

import importlib
import sys

import tq_local_b200 as _impl

__version__ = _impl.__version__
__all__ = list(_impl.__all__)

_ALIASES = (
    "api", "constants", "telemetry", "quantization", "quantization.turboquant_mse", "runtime",
    "runtime.attention", "runtime.generation", "runtime.memory_accounting", "runtime.packed_qmse_cache",
    "adapters", "adapters.transformers",
)


class _AliasFinder:
    """Resolve ``turboquant.x.y`` to ``tq_local_b200.x.y`` on first import."""

    def find_spec(self, name, path=None, target=None):
        if not name.startswith("turboquant.") or name[len("turboquant."):] not in _ALIASES:
            return None
        real = "tq_local_b200." + name[len("turboquant."):]
        module = importlib.import_module(real)
        sys.modules[name] = module
        return importlib.util.spec_from_loader(name, loader=_AliasLoader(module))


class _AliasLoader:
    def __init__(self, module):
        self.module = module

    def create_module(self, spec):
        return self.module

    def exec_module(self, module):
        pass


import importlib.util  # noqa: E402

sys.meta_path.insert(0, _AliasFinder())


def __getattr__(name: str):
    if name in _impl.__all__:
        return getattr(_impl, name)
    if name in {a.split(".")[0] for a in _ALIASES}:
        return importlib.import_module("turboquant." + name)
    raise AttributeError(f"module 'turboquant' has no attribute {name!r}")
