"""TurboQuant packed-KV hot path for NVIDIA B200 (sm_100a).

Public surface mirrors the reference package (``src/turboquant/__init__.py``):
``activate`` / ``deactivate`` / ``is_active`` / ``last_metrics`` /
``last_telemetry`` / ``print_telemetry`` / ``TurboQuantSession`` and friends.
Attributes are resolved lazily so that the low-level runtime modules can be
imported without pulling in ``transformers``.
"""

from __future__ import annotations

__version__ = "0.1.0"

__all__ = [
    "__version__",
    "CompatibilityReport",
    "TelemetrySummary",
    "TransformersLoadConfig",
    "TurboQuantSession",
    "activate",
    "deactivate",
    "inspect_transformers_model_compatibility",
    "is_active",
    "last_metrics",
    "last_telemetry",
    "load_transformers_model",
    "print_telemetry",
    "summarize_generation_metrics",
]


def __getattr__(name: str):
    if name in __all__:
        from tq_local_b200 import api

        return getattr(api, name)
    raise AttributeError(f"module 'tq_local_b200' has no attribute {name!r}")
