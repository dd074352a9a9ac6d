"""HF ``AttentionInterface`` backend that attends straight from the packed cache.

Mirror of the reference's ``src/turboquant/runtime/attention.py``: the function registered
under the name ``"turboquant"`` has the same signature and routing —

* no packed layer on the module, or a norm-guarded dense layer -> ``F.scaled_dot_product_attention``
  (``_sdpa_fallback``, reference lines 75-99);
* otherwise the fused CUDA decode kernel (``PackedMSELayer.attend``), which replaces both the
  reference's Triton ``fused_attention`` (batch 1 only) and its chunked PyTorch fallback
  (lines 215-304) for every batch size and query length.

As in the reference's fused path, the softmax scale is 1/sqrt(head_dim), the ``scaling``
argument and the attention mask are not applied on the packed path, and the current token
is attended through its own quantised copy because it was appended before attention.
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
    """Attention over a packed layer, ``[B, Hq, Sq, D]`` in and out.

    Kept under the reference's name for callers that import it; the work is done by the fused
    kernel, so ``chunk_size`` has no effect and there is nothing to chunk on the host.  A
    not-yet-stored ``new_key`` / ``new_value`` is not supported (append it with
    ``packed_layer.update`` first, which is what the HF forward pass does)."""
    if new_key is not None or new_value is not None:
        raise NotImplementedError("pass new tokens through PackedMSELayer.update() before attending")
    return packed_layer.attend(query_states)


def turboquant_attention_forward(module, query, key, value, attention_mask, dropout: float = 0.0,
                                 scaling: float | None = None, is_causal: bool | None = None, **kwargs):
    """``(module, query[B,Hq,Sq,D], key, value, mask, ...) -> (out[B,Sq,Hq,D], None)``."""
    layer = getattr(module, "_tq_cache_layer", None)
    if layer is None or layer._force_dense:
        return _sdpa_fallback(module, query, key, value, attention_mask, scaling)
    out = layer.attend(query)
    return out.transpose(1, 2).contiguous(), None


def _register_attention_backend() -> None:
    """Register ``"turboquant"`` (and the SDPA mask builder under the same key); idempotent."""
    try:
        from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    except ImportError:
        return
    if "turboquant" not in ALL_ATTENTION_FUNCTIONS:
        ALL_ATTENTION_FUNCTIONS.register("turboquant", turboquant_attention_forward)
    try:
        from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS

        if "turboquant" not in ALL_MASK_ATTENTION_FUNCTIONS:
            ALL_MASK_ATTENTION_FUNCTIONS.register("turboquant", ALL_MASK_ATTENTION_FUNCTIONS["sdpa"])
    except (ImportError, KeyError):
        pass


_register_attention_backend()
