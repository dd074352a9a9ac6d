"""Byte accounting for telemetry (host only).

Produces the same dictionaries as the reference's
``src/turboquant/runtime/memory_accounting.py`` (keys and meaning), which
``summarize_generation_metrics`` and ``last_telemetry`` consume.
"""

from __future__ import annotations

from typing import Any

import torch


def _kv_tensors(layer) -> list[torch.Tensor]:
    """Key, value (and any extra) tensors of one layer of an HF cache or a legacy tuple."""
    if isinstance(layer, (tuple, list)):
        return [t for t in layer if torch.is_tensor(t)]
    found = [getattr(layer, name, None) for name in ("keys", "values")]
    found = [t for t in found if t is not None]
    extra = getattr(layer, "_sliding_window_tensor", None)
    if torch.is_tensor(extra):
        found.append(extra)
    return found


def _nbytes(t: torch.Tensor) -> int:
    return int(t.numel() * t.element_size())


def past_key_values_memory_breakdown(past_key_values) -> dict[str, Any]:
    """Dense KV bytes of a prefill cache (reference: memory_accounting.py:34-64)."""
    layers = past_key_values.layers if hasattr(past_key_values, "layers") else past_key_values
    totals = dict(key=0, value=0, extra=0, layers=0, vectors=0)
    dim = None
    for layer in layers:
        tensors = _kv_tensors(layer)
        if len(tensors) < 2:
            continue
        k, v, *rest = tensors
        totals["key"] += _nbytes(k)
        totals["value"] += _nbytes(v)
        totals["extra"] += sum(_nbytes(t) for t in rest)
        totals["layers"] += 1
        totals["vectors"] += int(k.shape[0] * k.shape[1] * k.shape[2])
        if dim is None:
            dim = int(k.shape[-1])
    dense = totals["key"] + totals["value"]
    return {
        "num_layers": totals["layers"],
        "vector_dimension": dim,
        "num_key_value_vectors_per_kind": totals["vectors"],
        "key_bytes": totals["key"],
        "value_bytes": totals["value"],
        "dense_kv_bytes": dense,
        "extra_tensor_bytes": totals["extra"],
        "total_cache_tensor_bytes": dense + totals["extra"],
    }


def turboquant_mse_packed_bytes(*, num_vectors_per_kind: int, vector_dimension: int, bits: int,
                                norm_bytes: int = 2) -> dict[str, int | str]:
    """Size estimate of a Q_mse packed cache: codes + one norm per vector, keys and values
    (reference: memory_accounting.py:67-85)."""
    code_bytes = -(-(num_vectors_per_kind * vector_dimension * bits) // 8)
    norm_total = num_vectors_per_kind * norm_bytes
    return {
        "bits": bits,
        "norm_bytes_per_vector": norm_bytes,
        "norm_dtype_assumption": "float16" if norm_bytes == 2 else f"{norm_bytes * 8}-bit",
        "packed_kv_bytes": 2 * (code_bytes + norm_total),
        "packed_index_bytes": 2 * code_bytes,
        "packed_norm_bytes": 2 * norm_total,
    }


def gpu_peak_memory_bytes() -> dict[str, int | None]:
    if not torch.cuda.is_available():
        return {"peak_allocated_bytes": None, "peak_reserved_bytes": None}
    return {"peak_allocated_bytes": int(torch.cuda.max_memory_allocated()),
            "peak_reserved_bytes": int(torch.cuda.max_memory_reserved())}


def gpu_current_memory_bytes() -> dict[str, int | None]:
    if not torch.cuda.is_available():
        return {"allocated_bytes": None, "reserved_bytes": None}
    return {"allocated_bytes": int(torch.cuda.memory_allocated()),
            "reserved_bytes": int(torch.cuda.memory_reserved())}
