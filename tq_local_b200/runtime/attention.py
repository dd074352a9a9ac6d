"""HF ``AttentionInterface`` backend that attends straight from the packed cache.

Mirror of the reference's ``src/turboquant/runtime/attention.py``: the function registered
under the name ``"turboquant"`` has the same signature and routing —

* no packed layer on the module, or a norm-guarded dense layer -> ``F.scaled_dot_product_attention``
  (``_sdpa_fallback``, reference lines 75-99);
* otherwise the fused CUDA decode kernel (``PackedMSELayer.attend``), which replaces both the
  reference's Triton ``fused_attention`` (batch 1 only) and its chunked PyTorch fallback
  (lines 215-304) for every batch size and query length.

As in the reference's fused path, the softmax scale is 1/sqrt(head_dim), the ``scaling``
argument is not applied on the packed path, and the current token is attended through its own
quantised copy because it was appended before attention.  An attention mask is honoured in the
one form a decoder-only generation loop produces - left padding: every batch row attends the
tokens after its padding (the kernels take a per-row start offset), which is what the reference's
chunked path computes when it adds the additive mask to its logits (lines 253-255, 278-283).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def _sdpa_fallback(module, query, key, value, attention_mask, scaling):
    """Dense attention for prefill and for layers the norm guard kept dense."""
    groups = getattr(module, "num_key_value_groups", 1)
    out = F.scaled_dot_product_attention(
        query, key, value,
        attn_mask=attention_mask,
        dropout_p=0.0,
        is_causal=attention_mask is None and query.shape[-2] > 1,
        scale=scaling,
        enable_gqa=groups > 1,
    )
    return out.transpose(1, 2).contiguous(), None


def chunked_turboquant_attention(query_states, packed_layer, new_key=None, new_value=None, n_kv_groups: int = 1,
                                 attention_mask=None, chunk_size: int = 1024) -> torch.Tensor:
    """Attention over a packed layer, ``[B, Hq, Sq, D]`` in and out (reference:
    attention.py:215-304).  The work is done by the fused kernel, so ``chunk_size`` has no effect:
    there is nothing to chunk on the host.  ``attention_mask`` ([B, 1, Sq, Skv] additive or boolean,
    or [B, Skv]) is honoured for left-padded batches.  ``new_key`` / ``new_value`` [B, Hkv, T, D]
    (tokens the caller has not stored yet, which the reference attends un-quantised after the
    cache) are attended as a dense tail and the cache is left unchanged."""
    if (new_key is None) != (new_value is None):
        raise ValueError("new_key and new_value come together")
    if new_key is not None:
        return packed_layer.attend_with_new_tokens(query_states, new_key, new_value, attention_mask)
    return packed_layer.attend(query_states, attention_mask)


def turboquant_attention_forward(module, query, key, value, attention_mask, dropout: float = 0.0,
                                 scaling: float | None = None, is_causal: bool | None = None, **kwargs):
    """``(module, query[B,Hq,Sq,D], key, value, mask, ...) -> (out[B,Sq,Hq,D], None)``."""
    layer = getattr(module, "_tq_cache_layer", None)
    if layer is None or layer._force_dense:
        return _sdpa_fallback(module, query, key, value, attention_mask, scaling)
    out = layer.attend(query, attention_mask)
    return out.transpose(1, 2).contiguous(), None


def _register_attention_backend() -> None:
    """Register ``"turboquant"`` (and the SDPA mask builder under the same key); idempotent.
    The name is claimed for THIS function even when something else registered it before (the
    reference package uses the same name): a model switched to ``"turboquant"`` by this library
    must reach this library's kernels."""
    try:
        from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    except ImportError:
        return
    try:
        current = ALL_ATTENTION_FUNCTIONS["turboquant"] if "turboquant" in ALL_ATTENTION_FUNCTIONS else None
    except KeyError:
        current = None
    if current is not turboquant_attention_forward:
        ALL_ATTENTION_FUNCTIONS.register("turboquant", turboquant_attention_forward)
    try:
        from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS

        if "turboquant" not in ALL_MASK_ATTENTION_FUNCTIONS:
            ALL_MASK_ATTENTION_FUNCTIONS.register("turboquant", ALL_MASK_ATTENTION_FUNCTIONS["sdpa"])
    except (ImportError, KeyError):
        pass


_register_attention_backend()
