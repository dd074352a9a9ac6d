"""Public API surface (same names as the reference's ``src/turboquant/api.py``)."""

from __future__ import annotations

from tq_local_b200.adapters.transformers import (
    CompatibilityReport,
    TransformersLoadConfig,
    TurboQuantSession,
    activate,
    deactivate,
    inspect_transformers_model_compatibility,
    is_active,
    last_metrics,
    last_telemetry,
    load_transformers_model,
    print_telemetry,
)
from tq_local_b200.telemetry import TelemetrySummary, summarize_generation_metrics

__all__ = [
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
