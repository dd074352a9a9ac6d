"""HuggingFace Transformers adapter: the public switch of the library.

Mirror of the reference's ``src/turboquant/adapters/transformers.py``: ``activate`` patches
``model.generate`` so that every call runs greedy decoding over the packed cache (now served by
the sm_100a kernels), ``deactivate`` restores it, ``last_metrics`` / ``last_telemetry`` /
``print_telemetry`` report on the last call, ``TurboQuantSession`` is the object-style entry
point.  Names, keyword arguments, defaults, the attributes stashed on the model
(``_tq_state``, ``_tq_tokenizer``, ``_tq_last_output``) and the exceptions raised are the
reference's.

Host-side extensions: ``activate(..., verify=..., shard=..., cuda_graph=..., prefill_block_tokens=...)`` (skip the
per-call reconstruction report; shard KV heads over a process group; record the decode step in a
CUDA graph and replay it per token — on by default when every layer qualifies), and the patched
``generate`` returns every batch row (``[B, prompt + new]``) instead of row 0 only.
"""

from __future__ import annotations

import functools
from dataclasses import asdict, dataclass, field
from typing import Any

import torch
from transformers.cache_utils import Cache

from tq_local_b200.constants import DEFAULT_MAX_NEW_TOKENS
from tq_local_b200.runtime.generation import GenerationOutput, greedy_decode_with_prefill_cache
from tq_local_b200.telemetry import summarize_generation_metrics


@dataclass(frozen=True)
class TransformersLoadConfig:
    model_id_or_path: str
    revision: str | None = None
    dtype: str | torch.dtype = "auto"
    device_map: str | dict[str, Any] = "auto"
    attn_implementation: str = "sdpa"
    trust_remote_code: bool = False
    token: str | None = None
    cache_dir: str | None = None


@dataclass(frozen=True)
class CompatibilityReport:
    compatible: bool
    backend: str
    reasons: list[str] = field(default_factory=list)
    warnings: list[str] = field(default_factory=list)
    details: dict[str, Any] = field(default_factory=dict)

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


def load_transformers_model(config: TransformersLoadConfig):
    """``(tokenizer, model.eval())`` from a hub id or local path."""
    from transformers import AutoModelForCausalLM, AutoTokenizer

    common = dict(revision=config.revision, token=config.token, cache_dir=config.cache_dir,
                  trust_remote_code=config.trust_remote_code)
    tokenizer = AutoTokenizer.from_pretrained(config.model_id_or_path, **common)
    dtype = config.dtype
    if isinstance(dtype, str) and dtype != "auto":
        dtype = getattr(torch, dtype, dtype)
    model = AutoModelForCausalLM.from_pretrained(
        config.model_id_or_path, torch_dtype=dtype, device_map=config.device_map,
        attn_implementation=config.attn_implementation, low_cpu_mem_usage=True, **common)
    model.eval()
    return tokenizer, model


def inspect_transformers_model_compatibility(model) -> CompatibilityReport:
    cfg = model.config
    details = {
        "model_type": getattr(cfg, "model_type", None),
        "is_encoder_decoder": bool(getattr(cfg, "is_encoder_decoder", False)),
        "num_hidden_layers": getattr(cfg, "num_hidden_layers", None),
        "num_attention_heads": getattr(cfg, "num_attention_heads", None),
        "num_key_value_heads": getattr(cfg, "num_key_value_heads", None),
        "sliding_window": getattr(cfg, "sliding_window", None),
        "attention_chunk_size": getattr(cfg, "attention_chunk_size", None),
        "has_generate": hasattr(model, "generate"),
        "has_model_layers": bool(hasattr(model, "model") and hasattr(model.model, "layers")),
        "use_cache": getattr(cfg, "use_cache", True),
    }
    reasons, warnings = [], []
    if not details["has_generate"]:
        reasons.append("Model does not expose a generate() method.")
    if details["is_encoder_decoder"]:
        reasons.append("Encoder-decoder models are not supported in v1.")
    if not details["use_cache"]:
        reasons.append("Model config disables use_cache.")
    if details["num_hidden_layers"] is None or details["num_attention_heads"] is None:
        reasons.append("Model is missing standard decoder attention metadata.")
    if details["sliding_window"] is not None:
        warnings.append("Sliding-window attention is not explicitly supported in v1.")
    if details["attention_chunk_size"] is not None:
        warnings.append("Chunked attention is not explicitly supported in v1.")
    if getattr(cfg, "num_kv_shared_layers", None) is not None:
        warnings.append("Shared-KV-layer models are not explicitly supported in v1.")
    return CompatibilityReport(compatible=not reasons, backend="transformers", reasons=reasons,
                               warnings=warnings, details=details)


def _get_model_layers(model):
    inner = getattr(model, "model", None)
    return None if inner is None else getattr(inner, "layers", None)


def enable_turboquant_attention(model, packed_cache: Cache) -> str | None:
    """Route the model's attention through the packed cache: set the attention implementation
    to ``"turboquant"``, hang each ``PackedMSELayer`` on its ``self_attn._tq_cache_layer`` and
    switch the layers to lazy updates.  Returns the previous implementation name."""
    from tq_local_b200.runtime.attention import _register_attention_backend

    _register_attention_backend()  # (again on every switch: another package may have taken the name since import)
    layers = _get_model_layers(model)
    if layers is None:
        raise RuntimeError("Cannot locate model decoder layers for TurboQuant attention wiring.")
    previous = getattr(model.config, "_attn_implementation", None)
    model.config._attn_implementation = "turboquant"
    for idx, block in enumerate(layers):
        cache_layer = packed_cache.layers[idx]
        block.self_attn._tq_cache_layer = cache_layer
        cache_layer._lazy_update = True
    return previous


def disable_turboquant_attention(model, packed_cache: Cache, old_impl: str | None = "sdpa") -> None:
    layers = _get_model_layers(model)
    if layers is None:
        return
    model.config._attn_implementation = old_impl or "sdpa"
    for idx, block in enumerate(layers):
        if hasattr(block.self_attn, "_tq_cache_layer"):
            del block.self_attn._tq_cache_layer
        if idx < len(packed_cache.layers):
            packed_cache.layers[idx]._lazy_update = False


def _render_inputs(*, tokenizer, prompt, messages, add_generation_prompt):
    if messages is not None:
        if not hasattr(tokenizer, "apply_chat_template"):
            raise ValueError("Tokenizer does not support apply_chat_template, so messages input is unavailable.")
        prompt = tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt)
    elif prompt is None:
        raise ValueError("Either prompt or messages must be provided.")
    return tokenizer(prompt, return_tensors="pt")


class TurboQuantSession:
    """Object-style entry point: holds a model + tokenizer + settings, ``generate`` returns text."""

    def __init__(self, *, model, tokenizer, variant: str = "qmse_packed", bits: int = 3, rotation_seed: int = 0,
                 num_outlier_channels: int = 0, outlier_extra_bits: int = 1, use_qjl_keys: bool = False,
                 quantize_decode: bool = False, norm_guard: bool = True) -> None:
        report = inspect_transformers_model_compatibility(model)
        if not report.compatible:
            raise ValueError(f"Incompatible model for TurboQuantSession: {report.reasons}")
        self.model, self.tokenizer, self.variant = model, tokenizer, variant
        self.bits, self.rotation_seed = bits, rotation_seed
        self.num_outlier_channels, self.outlier_extra_bits = num_outlier_channels, outlier_extra_bits
        self.use_qjl_keys, self.quantize_decode, self.norm_guard = use_qjl_keys, quantize_decode, norm_guard
        self.compatibility = report
        self._last_output: GenerationOutput | None = None

    @classmethod
    def from_pretrained(cls, model_id_or_path: str, *, revision=None, dtype="auto", device_map="auto",
                        attn_implementation="sdpa", trust_remote_code=False, token=None, cache_dir=None,
                        **session_kwargs) -> "TurboQuantSession":
        tokenizer, model = load_transformers_model(TransformersLoadConfig(
            model_id_or_path=model_id_or_path, revision=revision, dtype=dtype, device_map=device_map,
            attn_implementation=attn_implementation, trust_remote_code=trust_remote_code, token=token,
            cache_dir=cache_dir))
        return cls(model=model, tokenizer=tokenizer, **session_kwargs)

    def generate(self, *, prompt=None, messages=None, max_new_tokens: int = DEFAULT_MAX_NEW_TOKENS,
                 add_generation_prompt: bool = True, return_output: bool = False):
        inputs = _render_inputs(tokenizer=self.tokenizer, prompt=prompt, messages=messages,
                                add_generation_prompt=add_generation_prompt)
        device = next(self.model.parameters()).device
        inputs = {name: t.to(device) for name, t in inputs.items()}
        output = greedy_decode_with_prefill_cache(
            model=self.model, tokenizer=self.tokenizer, inputs=inputs, max_new_tokens=max_new_tokens,
            variant=self.variant, qmse_bits=self.bits, rotation_seed=self.rotation_seed,
            num_outlier_channels=self.num_outlier_channels, outlier_extra_bits=self.outlier_extra_bits,
            use_qjl_keys=self.use_qjl_keys, quantize_decode=self.quantize_decode, norm_guard=self.norm_guard)
        self._last_output = output
        return output if return_output else output.text

    def last_metrics(self):
        return None if self._last_output is None else self._last_output.metrics.to_dict()

    def last_telemetry(self):
        if self._last_output is None:
            return None
        return summarize_generation_metrics(self._last_output.metrics).to_dict()

    def print_telemetry(self) -> None:
        if self._last_output is None:
            print("[TurboQuant] No generation data yet.")
            return
        print(summarize_generation_metrics(self._last_output.metrics).format(compact=False))

    def compatibility_report(self) -> dict[str, Any]:
        return self.compatibility.to_dict()


@dataclass
class _TurboQuantState:
    """What ``activate`` remembers on the model."""

    bits: int
    rotation_seed: int
    num_outlier_channels: int
    outlier_extra_bits: int
    use_qjl_keys: bool
    quantize_decode: bool
    norm_guard: bool
    original_generate: Any = None
    call_count: int = 0
    verify: bool = True
    shard: Any = None
    use_cuda_graph: bool | None = None
    prefill_block_tokens: int | None = None


def activate(model, tokenizer=None, *, bits: int = 4, rotation_seed: int = 0, num_outlier_channels: int = 0,
             outlier_extra_bits: int = 1, use_qjl_keys: bool = True, quantize_decode: bool = True,
             norm_guard: bool = True, quiet: bool = False, verify: bool = True, shard=None,
             cuda_graph: bool | None = None, prefill_block_tokens: int | None = None) -> None:
    """Make ``model.generate()`` decode greedily over a TurboQuant packed KV cache.

    ``bits`` 2-4; ``use_qjl_keys`` selects Q_prod keys (``bits-1`` Lloyd-Max bits + a 1-bit QJL
    residual sketch); ``quantize_decode`` re-quantises generated tokens into the cache;
    ``norm_guard`` keeps layers with very large key norms dense.  Raises ``RuntimeError`` when
    already active, ``ValueError`` for an incompatible model or a missing tokenizer."""
    if hasattr(model, "_tq_state"):
        raise RuntimeError("TurboQuant is already active on this model. Call turboquant.deactivate(model) first.")
    report = inspect_transformers_model_compatibility(model)
    if not report.compatible:
        raise ValueError(f"Model is not compatible with TurboQuant: {report.reasons}")
    if tokenizer is None:
        name = getattr(model.config, "_name_or_path", None)
        if not name:
            raise ValueError("Cannot auto-detect tokenizer. Pass tokenizer= explicitly.")
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(name)

    state = _TurboQuantState(bits=bits, rotation_seed=rotation_seed, num_outlier_channels=num_outlier_channels,
                             outlier_extra_bits=outlier_extra_bits, use_qjl_keys=use_qjl_keys,
                             quantize_decode=quantize_decode, norm_guard=norm_guard,
                             original_generate=model.generate, verify=verify, shard=shard,
                             use_cuda_graph=cuda_graph, prefill_block_tokens=prefill_block_tokens)
    model._tq_state = state
    model._tq_tokenizer = tokenizer

    @functools.wraps(state.original_generate)
    def _tq_generate(input_ids=None, **kwargs):
        tq: _TurboQuantState = model._tq_state
        max_new = kwargs.pop("max_new_tokens", None) or kwargs.pop("max_length", None) or 20
        attention_mask = kwargs.pop("attention_mask", None)
        if input_ids is None:
            raise ValueError("input_ids is required for TurboQuant generate().")
        inputs = {"input_ids": input_ids}
        if attention_mask is not None:
            inputs["attention_mask"] = attention_mask
        tq.call_count += 1
        output = greedy_decode_with_prefill_cache(
            model=model, tokenizer=model._tq_tokenizer, inputs=inputs, max_new_tokens=max_new,
            variant="qmse_packed", qmse_bits=tq.bits, rotation_seed=tq.rotation_seed,
            num_outlier_channels=tq.num_outlier_channels, outlier_extra_bits=tq.outlier_extra_bits,
            use_qjl_keys=tq.use_qjl_keys, quantize_decode=tq.quantize_decode, norm_guard=tq.norm_guard,
            verify=tq.verify, shard=tq.shard, use_cuda_graph=tq.use_cuda_graph,
            prefill_block_tokens=tq.prefill_block_tokens)
        model._tq_last_output = output
        return torch.cat([input_ids, output.completion_ids.to(input_ids.device)], dim=1)

    model.generate = _tq_generate

    if not quiet:
        mode = "Q_prod" if use_qjl_keys else "Q_mse"
        print()
        print("  TurboQuant activated")
        print(f"    Model:      {getattr(model.config, 'model_type', 'unknown')} "
              f"({getattr(model.config, 'num_hidden_layers', '?')} layers)")
        print(f"    Bits:       {bits}-bit {mode}")
        print(f"    Norm guard: {'on' if norm_guard else 'off'}")
        print(f"    Decode:     {'quantized' if quantize_decode else 'dense'}")
        print()
        print("  model.generate() now uses TurboQuant compression.")
        print("  Call turboquant.deactivate(model) to restore original behavior.")
        print()


def deactivate(model, quiet: bool = False) -> None:
    state: _TurboQuantState | None = getattr(model, "_tq_state", None)
    if state is None:
        if not quiet:
            print("[TurboQuant] Not active on this model, nothing to deactivate.")
        return
    model.generate = state.original_generate
    for attr in ("_tq_state", "_tq_tokenizer", "_tq_last_output"):
        if hasattr(model, attr):
            delattr(model, attr)
    if not quiet:
        print(f"[TurboQuant] Deactivated after {state.call_count} calls.")


def is_active(model) -> bool:
    return hasattr(model, "_tq_state")


def last_metrics(model) -> dict[str, Any] | None:
    output = getattr(model, "_tq_last_output", None)
    return None if output is None else output.metrics.to_dict()


def last_telemetry(model) -> dict[str, Any] | None:
    output = getattr(model, "_tq_last_output", None)
    return None if output is None else summarize_generation_metrics(output.metrics).to_dict()


def print_telemetry(model, *, verbose: bool = False) -> None:
    output = getattr(model, "_tq_last_output", None)
    if output is None:
        print("[TurboQuant] No generation data yet.")
        return
    print(summarize_generation_metrics(output.metrics).format(compact=not verbose))
