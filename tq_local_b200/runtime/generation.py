"""Greedy generation over a packed prefill cache.

Mirror of the reference's ``src/turboquant/runtime/generation.py``
(``greedy_decode_with_prefill_cache``, ``GenerationMetrics``, ``GenerationOutput``): dense
prefill with the model's own attention, pack the prefill cache, switch the model to the
``"turboquant"`` attention backend, then one forward pass per new token.  Differences, all
on the host side of the hot path:

* the packed cache is allocated once with room for ``max_new_tokens`` (no per-token
  ``torch.cat``);
* only the last position's logits are requested from the prefill;
* the EOS test reads the device every few steps instead of every step and the result is
  trimmed afterwards, so the returned text is the same;
* all batch rows are kept (``GenerationOutput.completion_ids``); ``text`` is row 0 as in
  the reference.
"""

from __future__ import annotations

import time
from dataclasses import asdict, dataclass
from typing import Any

from tq_local_b200.runtime.memory_accounting import (
    gpu_current_memory_bytes,
    gpu_peak_memory_bytes,
    past_key_values_memory_breakdown,
    turboquant_mse_packed_bytes,
)
from tq_local_b200.runtime.packed_qmse_cache import (
    _auto_norm_threshold,
    is_left_padding_mask,
    build_packed_mse_cache,
    build_streaming_prefill_cache,
    packed_cache_storage_breakdown,
    report_streamed_norm_guard,
    streamed_prefill_memory_breakdown,
    verify_packed_reconstruction,
)

_EOS_POLL_STEPS = 8
# A streaming prompt pass runs at most this many prompt tokens through the model at a time (whole
# sequences: batch rows are taken in blocks), which bounds the activations of a long-prompt batch.
PREFILL_BLOCK_TOKENS = 131072
_GRAPH_WARMUP_STEPS = 2  # eager steps in static mode before the decode step is recorded


@dataclass(frozen=True)
class GenerationMetrics:
    variant: str
    qmse_bits: int | None
    quantization_seconds: float
    generation_seconds: float
    prompt_tokens: int
    completion_tokens: int
    prefill_cache: dict[str, Any]
    turboquant_mse_packed_estimate: dict[str, Any] | None
    turboquant_mse_packed_actual: dict[str, Any] | None
    post_cache_setup_gpu_memory: dict[str, Any] | None
    gpu_peak_memory: dict[str, Any] | None
    reconstruction_quality: list[dict[str, Any]] | None = None

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


@dataclass(frozen=True)
class GenerationOutput:
    text: str
    metrics: GenerationMetrics
    completion_ids: Any = None  # LongTensor [batch, new_tokens]; rows padded with EOS after their end


def validate_generation_variant(variant: str) -> None:
    if variant not in {"baseline", "qmse", "qmse_packed"}:
        raise ValueError(
            f"Unsupported generation variant={variant!r}. Choose from ['baseline', 'qmse', 'qmse_packed']."
        )


def eos_token_ids(model, tokenizer) -> set[int]:
    eos = getattr(getattr(model, "generation_config", None), "eos_token_id", None)
    if eos is None:
        eos = getattr(tokenizer, "eos_token_id", None)
    if eos is None:
        return set()
    return {int(eos)} if isinstance(eos, int) else {int(x) for x in eos}


def _prefill(model, inputs, cache=None):
    """Dense prefill; ask for the last position's logits only when the model supports it."""
    extra = {} if cache is None else {"past_key_values": cache}
    try:
        return model(**inputs, use_cache=True, logits_to_keep=1, **extra)
    except TypeError:
        if cache is not None and any(layer.is_initialized for layer in cache.layers):
            raise  # the cache already holds part of the prompt: a second pass would store it twice
        return model(**inputs, use_cache=True, **extra)


def raise_on_device_status(layers, where: str) -> None:
    """The kernels' bounded waits only set a status word when they give up (a peer that never
    raised its flag, a bulk copy that never landed); what was computed after that is not valid.
    Called wherever the generation loops synchronise anyway: reads the word of every codec the
    layers use, agrees on it across the ranks of a sharded run (so that all of them raise, and
    none is left waiting in a collective), and raises ``TQError`` if any kernel gave up."""
    import torch

    from tq_local_b200.runtime.ffi import TQError

    codecs, shard = {}, None
    for layer in layers:
        codec = getattr(layer, "codec", None)
        if codec is not None and getattr(codec, "handle", None):
            codecs[id(codec)] = codec
            shard = shard or getattr(layer, "shard", None)
    status = max((c.device_status() for c in codecs.values()), default=0)
    if shard is not None and shard.world_size > 1:
        import torch.distributed as dist

        device = next(iter(codecs.values())).device
        if dist.get_backend(shard.group) == "gloo":
            device = torch.device("cpu")
        word = torch.tensor([status], dtype=torch.int32, device=device)
        dist.all_reduce(word, op=dist.ReduceOp.MAX, group=shard.group)
        status = int(word.item())
    if status:
        from tq_local_b200.runtime.codec import Codec

        raise TQError(f"{where}: device status {status} ({Codec._STATUS_TEXT.get(status, 'unknown')}); "
                      "the generated tokens are not valid")


def _prefill_in_row_blocks(model, inputs, packed_cache, threshold: float, rows_per_block: int):
    """The prompt pass of a streaming prefill, ``rows_per_block`` sequences at a time: every block
    runs the whole model with its own dense attention (exactly what the reference's single prompt
    pass computes for those rows, generation.py:91) while each layer packs the block's K/V into its
    rows of the packed cache.  Neither the logits of the whole prompt ([B, S, vocab]) nor a dense
    cache of the whole model nor the activations of the whole batch ever exist.  Returns the last
    position's logits [B, vocab]."""
    import sys

    import torch

    ids = inputs["input_ids"]
    batch, n_tokens = int(ids.shape[0]), int(ids.shape[1])
    last = []
    for b0 in range(0, batch, rows_per_block):
        block = {k: (v[b0:b0 + rows_per_block] if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == batch else v)
                 for k, v in inputs.items()}
        for layer in packed_cache.layers:
            layer.begin_prefill_block(b0, batch, threshold)
        out = _prefill(model, block, packed_cache)
        last.append(out.logits[:, -1, :].clone())
        del out
    agree = [layer.finish_prefill(n_tokens, threshold) for layer in packed_cache.layers]
    if not all(agree):
        odd = [i for i, ok in enumerate(agree) if not ok]
        print(f"[TurboQuant] norm_guard: layers {odd} were decided on the first block of sequences; the mean key "
              "norm of the whole batch falls on the other side of the threshold", file=sys.stderr)
    return torch.cat(last, dim=0)


def _static_decode_eligible(model, packed_cache) -> bool:
    """The replayable (CUDA-graph) decode loop needs every layer packed with quantised appends and
    a tensor-core shape.  (A left-padded prompt is fine: the layers carry the per-row start
    offsets that ``bind_attention_mask`` derived from the prompt's mask.)"""
    import torch

    if packed_cache is None or not torch.cuda.is_available():
        return False
    q_heads = int(getattr(model.config, "num_attention_heads", 0))
    return bool(q_heads) and all(layer.supports_static_decode(q_heads) for layer in packed_cache.layers)


class RecordedDecoder:
    """Greedy decode steps with the whole model step recorded once in a CUDA graph and replayed
    per token.  The cache length, the position ids, the current token and the output cursor all
    live on the device, so the host only launches the graph.  The first steps run eagerly (they
    are real steps) and the next one is recorded; if the model's forward pass cannot be recorded,
    all steps run eagerly with a warning.  Use as a context manager, or call ``close``: it hands
    the layers back to their normal bookkeeping."""

    def __init__(self, model, cache, first_token, max_steps: int, eager_steps: int | None = None):
        import torch

        self.model, self.cache = model, cache
        self.layers = cache.layers
        device = first_token.device
        self.length0 = self.layers[0].store.length
        self.pos32 = torch.tensor([self.length0], dtype=torch.int32, device=device)
        self.pos_ids = torch.full((1, 1), self.length0, dtype=torch.long, device=device)
        self.token = first_token.clone()
        self.produced = torch.zeros((first_token.shape[0], max(max_steps, 1)), dtype=first_token.dtype,
                                    device=device)
        self.cursor = torch.zeros(1, dtype=torch.long, device=device)
        self.max_steps = int(max_steps)
        self.eager_steps = _GRAPH_WARMUP_STEPS if eager_steps is None else int(eager_steps)
        self.done = 0
        self.graph = None  # None: not recorded yet; False: cannot be recorded
        # KV-head shards exchange their outputs through one shared set of peer buffers whose step
        # numbers live on the device (created and closed collectively by all ranks)
        self.gather = None
        shard = self.layers[0].shard
        if shard.world_size > 1:
            from tq_local_b200.runtime.sharding import PeerGather

            self.gather = PeerGather(shard, int(first_token.shape[0]), int(model.config.num_attention_heads),
                                     self.layers[0].dtype, device, device_sequence=True)
        for layer in self.layers:
            layer.begin_static_decode(self.pos32, max_steps, gather=self.gather)

    def _forward_once(self) -> None:
        import torch

        out = self.model(input_ids=self.token, past_key_values=self.cache, use_cache=True, position_ids=self.pos_ids)
        nxt = torch.argmax(out.logits[:, -1, :], dim=-1, keepdim=True)
        self.token.copy_(nxt)
        self.produced.index_copy_(1, self.cursor, nxt)
        self.cursor.add_(1), self.pos32.add_(1), self.pos_ids.add_(1)

    def step(self) -> None:
        """Queue one more token (asynchronous; read ``tokens`` after a synchronise)."""
        import torch

        if self.done >= self.max_steps:
            raise RuntimeError("RecordedDecoder: no room left for another token")
        if self.done >= self.eager_steps and self.graph is None:
            torch.cuda.synchronize()
            try:
                recorded = torch.cuda.CUDAGraph()
                with torch.cuda.graph(recorded, capture_error_mode="thread_local"):
                    self._forward_once()
                self.graph = recorded
            except Exception as exc:
                import warnings

                warnings.warn(f"decode step not recorded in a CUDA graph ({exc!r}); running it eagerly")
                self.graph = False
        if self.graph:
            self.graph.replay()
        else:
            self._forward_once()
        self.done += 1

    @property
    def tokens(self):
        """The tokens produced so far, [B, done] (a view; synchronise first)."""
        return self.produced[:, :self.done]

    def close(self) -> None:
        import torch

        if self.layers is not None:
            torch.cuda.synchronize()
            layers = self.layers
            for layer in layers:
                layer.end_static_decode(self.length0 + self.done)
            self.layers = None
            if self.gather is not None:
                self.gather.close()
                self.gather = None
            raise_on_device_status(layers, "RecordedDecoder.close")

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def _graphed_greedy_steps(model, cache, first_token, n_steps, eos_tensor):
    """Up to ``n_steps`` greedy tokens after ``first_token`` through a ``RecordedDecoder``, looking
    at the produced tokens every few steps for the EOS test.  Returns them as [B, <= n_steps]."""
    import torch

    with RecordedDecoder(model, cache, first_token, n_steps) as dec:
        while dec.done < n_steps:
            if eos_tensor is not None and dec.done and dec.done % _EOS_POLL_STEPS == 0:
                so_far = torch.cat((first_token, dec.tokens), dim=-1)
                if bool(torch.isin(so_far, eos_tensor).any(dim=-1).all()):
                    break
                raise_on_device_status(cache.layers, "recorded decode")  # (the EOS test synchronised already)
            dec.step()
        torch.cuda.synchronize()
        return dec.tokens.clone()


def greedy_decode_with_prefill_cache(
    *,
    model,
    tokenizer,
    inputs,
    max_new_tokens: int,
    variant: str,
    qmse_bits: int,
    rotation_seed: int = 0,
    num_outlier_channels: int = 0,
    outlier_extra_bits: int = 1,
    use_qjl_keys: bool = False,
    quantize_decode: bool = False,
    norm_guard: bool = True,
    verify: bool = True,
    shard=None,
    use_cuda_graph: bool | None = None,
    prefill_block_tokens: int | None = None,
) -> GenerationOutput:
    import torch

    validate_generation_variant(variant)
    if max_new_tokens <= 0:
        raise ValueError("max_new_tokens must be positive.")

    started = time.monotonic()
    quant_seconds = 0.0
    eos_ids = eos_token_ids(model, tokenizer)
    packed_cache = None
    old_impl = None

    with torch.inference_mode():
        cfg = getattr(model, "config", None)
        n_layers = getattr(cfg, "num_hidden_layers", None)
        heads = getattr(cfg, "num_attention_heads", None)
        head_dim = getattr(cfg, "head_dim", None) or (cfg.hidden_size // heads if heads else None)
        # Without the reconstruction report nothing needs the dense prompt cache: every layer packs
        # its K/V while the prompt pass runs.
        streaming = variant == "qmse_packed" and not verify and bool(n_layers) and bool(head_dim)
        if streaming:
            t0 = time.monotonic()
            packed_cache = build_streaming_prefill_cache(
                n_layers, qmse_bits, head_dim=head_dim, seed=rotation_seed, num_outlier_channels=num_outlier_channels,
                outlier_extra_bits=outlier_extra_bits, use_qjl_keys=use_qjl_keys, quantize_decode=quantize_decode,
                norm_guard=norm_guard, reserve_tokens=max_new_tokens, shard=shard)
            quant_seconds += time.monotonic() - t0
            ids = inputs["input_ids"]
            block_tokens = PREFILL_BLOCK_TOKENS if prefill_block_tokens is None else int(prefill_block_tokens)
            rows_per_block = max(1, block_tokens // max(int(ids.shape[1]), 1))
            if rows_per_block < int(ids.shape[0]):
                threshold = _auto_norm_threshold(qmse_bits, head_dim) if norm_guard else float("inf")
                last_logits = _prefill_in_row_blocks(model, inputs, packed_cache, threshold, rows_per_block)
                cache = packed_cache
            else:
                outputs = _prefill(model, inputs, packed_cache)
                cache, last_logits = outputs.past_key_values, outputs.logits[:, -1, :]
                del outputs
        else:
            outputs = _prefill(model, inputs)
            cache, last_logits = outputs.past_key_values, outputs.logits[:, -1, :]
            del outputs
        next_token = torch.argmax(last_logits, dim=-1, keepdim=True)
        del last_logits
        estimate = actual = recon = None
        if streaming:
            report_streamed_norm_guard(packed_cache, qmse_bits, head_dim)
            dense_breakdown = streamed_prefill_memory_breakdown(packed_cache)
        else:
            dense_breakdown = past_key_values_memory_breakdown(cache)
        if variant == "qmse":
            # unpacked variant (reference: generation.py:104-113): the prompt's dense cache is replaced by
            # its quantise-dequantise reconstruction; nothing is packed, attention stays the model's own
            from tq_local_b200.quantization.turboquant_mse import quantize_past_key_values_mse

            t0 = time.monotonic()
            cache = quantize_past_key_values_mse(cache, bits=qmse_bits, seed=rotation_seed)
            quant_seconds += time.monotonic() - t0
        if variant in ("qmse", "qmse_packed"):
            estimate = turboquant_mse_packed_bytes(
                num_vectors_per_kind=dense_breakdown["num_key_value_vectors_per_kind"],
                vector_dimension=dense_breakdown["vector_dimension"],
                bits=qmse_bits,
            )
        if variant == "qmse_packed":
            t0 = time.monotonic()
            if not streaming:
                packed_cache = build_packed_mse_cache(
                    cache, bits=qmse_bits, seed=rotation_seed, num_outlier_channels=num_outlier_channels,
                    outlier_extra_bits=outlier_extra_bits, use_qjl_keys=use_qjl_keys, quantize_decode=quantize_decode,
                    norm_guard=norm_guard, reserve_tokens=max_new_tokens, shard=shard, release_dense=not verify,
                )
            if verify:
                recon = verify_packed_reconstruction(cache, packed_cache)
            actual = packed_cache_storage_breakdown(packed_cache)
            cache = packed_cache
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            quant_seconds += time.monotonic() - t0

            # Padding: a decoder-only batch is padded on the left.  The packed layers take the
            # per-row start offset from the prompt's mask once (it does not change while decoding).
            prompt_mask = inputs.get("attention_mask")
            if prompt_mask is not None and bool(prompt_mask.all()):
                prompt_mask = None
            if prompt_mask is not None and not is_left_padding_mask(prompt_mask):
                raise ValueError("TurboQuant attends left-padded batches only: every row of attention_mask "
                                 "must be zeros followed by ones (tokenizer.padding_side = 'left')")
            for layer in packed_cache.layers:
                layer.bind_attention_mask(prompt_mask, lock=True)

            from tq_local_b200.adapters.transformers import enable_turboquant_attention

            old_impl = enable_turboquant_attention(model, packed_cache)

        try:
            if torch.cuda.is_available():
                torch.cuda.empty_cache()
            post_setup = gpu_current_memory_bytes()
            if torch.cuda.is_available():
                torch.cuda.reset_peak_memory_stats()

            eos_tensor = (torch.tensor(sorted(eos_ids), device=next_token.device) if eos_ids else None)
            generated = [next_token]
            mask = inputs.get("attention_mask")
            if use_cuda_graph is None:
                use_cuda_graph = variant == "qmse_packed" and max_new_tokens > 8
            graphed = False
            if use_cuda_graph and max_new_tokens > 1 and _static_decode_eligible(model, packed_cache):
                if eos_tensor is None or not bool(torch.isin(next_token, eos_tensor).any(dim=-1).all()):
                    generated.append(_graphed_greedy_steps(model, cache, next_token, max_new_tokens - 1, eos_tensor))
                graphed = True
            for step in range(0 if graphed else max_new_tokens - 1):
                if eos_tensor is not None and step % _EOS_POLL_STEPS == 0:
                    seen = torch.isin(torch.cat(generated, dim=-1), eos_tensor).any(dim=-1)
                    if bool(seen.all()):
                        break
                if mask is not None:
                    mask = torch.cat((mask, mask.new_ones((mask.shape[0], 1))), dim=-1)
                out = model(input_ids=next_token, attention_mask=mask, past_key_values=cache, use_cache=True)
                cache = out.past_key_values
                if variant == "qmse":  # the token just appended gets quantised in place (generation.py:170-178)
                    t0 = time.monotonic()
                    cache = quantize_past_key_values_mse(cache, bits=qmse_bits, seed=rotation_seed,
                                                         token_slice=slice(-1, None))
                    quant_seconds += time.monotonic() - t0
                next_token = torch.argmax(out.logits[:, -1, :], dim=-1, keepdim=True)
                generated.append(next_token)
            if packed_cache is not None and torch.cuda.is_available():
                torch.cuda.synchronize()
                raise_on_device_status(packed_cache.layers, "greedy decode")
        finally:
            if packed_cache is not None:
                from tq_local_b200.adapters.transformers import disable_turboquant_attention

                disable_turboquant_attention(model, packed_cache, old_impl)

        completion = torch.cat(generated, dim=-1)
        if eos_tensor is not None:
            # Cut every row after its first EOS (which is kept, as in the reference); the batch
            # is as long as its longest row and shorter rows are padded with their EOS.
            hit = torch.isin(completion, eos_tensor)
            steps = torch.arange(completion.shape[1], device=completion.device).expand_as(completion)
            first = torch.where(hit, steps, torch.full_like(steps, completion.shape[1] - 1)).min(dim=-1).values
            keep = int(first.max().item()) + 1
            completion = completion[:, :keep].clone()
            for row in range(completion.shape[0]):
                end = int(first[row])
                completion[row, end + 1:] = completion[row, end]
            row0_len = int(first[0]) + 1
        else:
            row0_len = completion.shape[1]

    text = tokenizer.decode(completion[0, :row0_len], skip_special_tokens=True).strip()
    metrics = GenerationMetrics(
        variant=variant,
        qmse_bits=qmse_bits if variant in ("qmse", "qmse_packed") else None,
        quantization_seconds=round(quant_seconds, 4),
        generation_seconds=round(time.monotonic() - started, 4),
        prompt_tokens=int(inputs["input_ids"].shape[-1]),
        completion_tokens=int(row0_len),
        prefill_cache=dense_breakdown,
        turboquant_mse_packed_estimate=estimate,
        turboquant_mse_packed_actual=actual,
        post_cache_setup_gpu_memory=post_setup,
        gpu_peak_memory=gpu_peak_memory_bytes(),
        reconstruction_quality=recon,
    )
    return GenerationOutput(text=text, metrics=metrics, completion_ids=completion)
