"""Telemetry summary of one ``generate()`` call (host only).

Same fields, dictionary schema and text layout as the reference's
``src/turboquant/telemetry.py`` (``TelemetrySummary``, ``summarize_generation_metrics``), which
is what ``turboquant.last_telemetry(model)`` returns.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any


def _human_bytes(n: int | float | None) -> str:
    if n is None:
        return "n/a"
    x = float(n)
    for unit in ("B", "KB", "MB", "GB"):
        if x < 1024.0:
            return f"{x:.2f} {unit}"
        x /= 1024.0
    return f"{x:.2f} TB"


@dataclass(frozen=True)
class TelemetrySummary:
    variant: str
    qmse_bits: int | None
    prompt_tokens: int
    completion_tokens: int
    dense_kv_bytes: int
    packed_estimate_bytes: int | None
    packed_actual_bytes: int | None
    payload_savings_fraction: float | None
    payload_savings_percent: float | None
    post_cache_setup_allocated_bytes: int | None
    post_cache_setup_reserved_bytes: int | None
    peak_allocated_bytes: int | None
    peak_reserved_bytes: int | None
    generation_seconds: float
    quantization_seconds: float

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)

    def _packed(self) -> int | None:
        return self.packed_actual_bytes or self.packed_estimate_bytes

    def format(self, compact: bool = False) -> str:
        return self._one_line() if compact else self._block()

    def _one_line(self) -> str:
        mb = 1024 * 1024
        packed = self._packed()
        saved = f"{self.payload_savings_percent:.0f}% saved" if self.payload_savings_percent else ""
        peak = f" | peak {self.peak_allocated_bytes / 1e9:.1f} GB" if self.peak_allocated_bytes else ""
        return (f"[TurboQuant] {self.prompt_tokens}→{self.completion_tokens} tok"
                f" | KV {self.dense_kv_bytes / mb:.0f}→{(packed / mb if packed else 0):.0f} MB ({saved}){peak}")

    def _block(self) -> str:
        mode = f"{self.qmse_bits}-bit {self.variant}" if self.qmse_bits else self.variant
        saved = f"{self.payload_savings_percent:.1f}%" if self.payload_savings_percent else "n/a"
        rate = (f"{self.completion_tokens / self.generation_seconds:.1f}" if self.generation_seconds > 0 else "n/a")
        out = ["", "  TurboQuant Telemetry", "  " + "─" * 50, "",
               f"    Mode:               {mode}",
               f"    KV savings:         {saved}",
               f"    Generation:         {self.generation_seconds:.2f}s  ({rate} tok/s)",
               f"    Quantization:       {self.quantization_seconds:.3f}s", "",
               f"    Prompt tokens:      {self.prompt_tokens}",
               f"    Completion tokens:  {self.completion_tokens}", "",
               f"    Dense KV cache:     {_human_bytes(self.dense_kv_bytes)}",
               f"    Packed KV cache:    {_human_bytes(self._packed())}"]
        if self.post_cache_setup_allocated_bytes is not None:
            out += ["", f"    GPU after setup:    {_human_bytes(self.post_cache_setup_allocated_bytes)}"]
        if self.peak_allocated_bytes is not None:
            out.append(f"    GPU peak:           {_human_bytes(self.peak_allocated_bytes)}")
        out.append("")
        return "\n".join(out)


def _opt_int(d: dict | None, key: str) -> int | None:
    if d is None or d.get(key) is None:
        return None
    return int(d[key])


def summarize_generation_metrics(metrics) -> TelemetrySummary:
    """Accepts a ``GenerationMetrics`` or its ``to_dict()``."""
    m = metrics if isinstance(metrics, dict) else metrics.to_dict()
    dense = int(m["prefill_cache"]["dense_kv_bytes"])
    estimate = _opt_int(m.get("turboquant_mse_packed_estimate"), "packed_kv_bytes")
    actual = _opt_int(m.get("turboquant_mse_packed_actual"), "packed_total_bytes")
    packed = actual if actual is not None else estimate
    fraction = percent = None
    if packed is not None and dense > 0:
        fraction = 1.0 - packed / dense
        percent = fraction * 100.0
    return TelemetrySummary(
        variant=str(m["variant"]),
        qmse_bits=m.get("qmse_bits"),
        prompt_tokens=int(m["prompt_tokens"]),
        completion_tokens=int(m["completion_tokens"]),
        dense_kv_bytes=dense,
        packed_estimate_bytes=estimate,
        packed_actual_bytes=actual,
        payload_savings_fraction=fraction,
        payload_savings_percent=percent,
        post_cache_setup_allocated_bytes=_opt_int(m.get("post_cache_setup_gpu_memory"), "allocated_bytes"),
        post_cache_setup_reserved_bytes=_opt_int(m.get("post_cache_setup_gpu_memory"), "reserved_bytes"),
        peak_allocated_bytes=_opt_int(m.get("gpu_peak_memory"), "peak_allocated_bytes"),
        peak_reserved_bytes=_opt_int(m.get("gpu_peak_memory"), "peak_reserved_bytes"),
        generation_seconds=float(m["generation_seconds"]),
        quantization_seconds=float(m["quantization_seconds"]),
    )
