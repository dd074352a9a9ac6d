"""Packed TurboQuant cache layer backed by the sm_100a kernels.

Host-side mirror of the reference's ``src/turboquant/runtime/packed_qmse_cache.py``:
the same class / function names, constructor arguments, attributes and error behaviour,
so code written against the reference (its attention backend, its generation loop, its
telemetry) works unchanged — but every tensor operation of the hot path is one call into
``libtq_b200.so``:

===========================================  ==========================================
reference                                    here
===========================================  ==========================================
``_encode_group`` / ``_encode_keys_qjl_group``  ``tq_pack`` (rotate, quantise, bit-pack, QJL)
``PackedTensorMSE.append`` (``torch.cat``)      in-place write at the current length
``_decode_group`` / ``triton_decode_group``     ``tq_dequant``
``fused_attention`` / chunked fallback          ``tq_decode_attn`` (:meth:`PackedMSELayer.attend`)
===========================================  ==========================================

Outlier-channel splitting (``num_outlier_channels > 0``) is served by ``outlier_split.SplitStore``
(tensor arithmetic on the cache's device; the kernels handle 128-coordinate vectors only).
"""

from __future__ import annotations

import sys
from dataclasses import dataclass
from math import sqrt
from typing import Any

import torch
from transformers.cache_utils import Cache, CacheLayerMixin

from tq_local_b200.runtime.codec import Codec
from tq_local_b200.runtime.packed_store import PackedStore, key_norm_mean
from tq_local_b200.runtime.sharding import HeadShard


@dataclass
class PackedTensorMSE:
    """View of the stored tokens of one packed stream pair (reference: packed_qmse_cache.py:58-92)."""

    packed_indices: torch.Tensor  # uint8 [B, H, N, 16*bits]
    norms: torch.Tensor           # fp16  [B, H, N]
    original_shape: tuple[int, int, int, int]
    original_dtype: torch.dtype
    bits: int

    @property
    def num_vectors(self) -> int:
        b, h, n, _ = self.original_shape
        return int(b * h * n)

    @property
    def dimension(self) -> int:
        return int(self.original_shape[-1])

    def storage_bytes(self) -> int:
        return int(self.packed_indices.numel() * self.packed_indices.element_size()
                   + self.norms.numel() * self.norms.element_size())


@dataclass
class PackedQJL:
    """View of the 1-bit QJL sign sketch and residual norms (packed_qmse_cache.py:121-140)."""

    packed_signs: torch.Tensor    # uint8 [B, H, N, 16]
    residual_norms: torch.Tensor  # fp16  [B, H, N]
    dimension: int

    def storage_bytes(self) -> int:
        return int(self.packed_signs.numel() * self.packed_signs.element_size()
                   + self.residual_norms.numel() * self.residual_norms.element_size())


def leading_masked_tokens(mask: torch.Tensor) -> torch.Tensor:
    """Per batch row, how many key positions are masked before the first kept one (int32 [B], no
    host synchronisation).  ``mask`` is [B, S] (non-zero / True = keep) or [B, 1, Sq, S] (bool
    keep-mask, or additive float where kept positions are 0 and masked ones very negative; the
    last query row is looked at)."""
    if mask.dim() == 4:
        row = mask[:, 0, -1, :]
        keep = row if row.dtype == torch.bool else row > -1.0
    elif mask.dim() == 2:
        keep = mask if mask.dtype == torch.bool else mask != 0
    else:
        raise ValueError(f"expected a [B, S] or [B, 1, Sq, S] attention mask, got {tuple(mask.shape)}")
    return (torch.cumsum(keep.to(torch.int32), dim=-1) == 0).sum(dim=-1, dtype=torch.int32).contiguous()


def is_left_padding_mask(mask: torch.Tensor) -> bool:
    """Whether a 2-D mask [B, S] is zeros followed by ones in every row with at least one kept
    position (one host synchronisation; the generation loop asks once per call)."""
    keep = mask if mask.dtype == torch.bool else mask != 0
    seen = torch.cumsum(keep.to(torch.int32), dim=-1) > 0
    return bool(((seen == keep).all(dim=-1) & keep.any(dim=-1)).all())


class _GrowingDense:
    """Dense [B, H, T, D] buffer with spare capacity: amortised O(1) append along T."""

    def __init__(self) -> None:
        self.buf: torch.Tensor | None = None
        self.length = 0

    def append(self, x: torch.Tensor, reserve: int = 0) -> torch.Tensor:
        n = int(x.shape[2])
        if self.buf is None:
            cap = max(self.length + n + reserve, 16)
            self.buf = torch.empty(x.shape[0], x.shape[1], cap, x.shape[3], dtype=x.dtype, device=x.device)
        elif self.length + n > self.buf.shape[2]:
            cap = max(2 * self.buf.shape[2], self.length + n + reserve)
            grown = torch.empty(*self.buf.shape[:2], cap, self.buf.shape[3], dtype=self.buf.dtype,
                                device=self.buf.device)
            grown[:, :, :self.length] = self.buf[:, :, :self.length]
            self.buf = grown
        self.buf[:, :, self.length:self.length + n] = x
        self.length += n
        return self.view()

    def write_rows(self, x: torch.Tensor, b0: int, total_batch: int, reserve: int = 0) -> None:
        """Batch rows ``[b0, b0 + x.shape[0])`` of a buffer for ``total_batch`` rows, tokens
        ``[0, x.shape[2])``; ``length`` is left for the caller to set once every row is in."""
        n = int(x.shape[2])
        if self.buf is None:
            self.buf = torch.empty(total_batch, x.shape[1], max(n + reserve, 16), x.shape[3], dtype=x.dtype,
                                   device=x.device)
        self.buf[b0:b0 + x.shape[0], :, :n] = x

    def view(self) -> torch.Tensor | None:
        return None if self.buf is None else self.buf[:, :, :self.length]


class PackedMSELayer(CacheLayerMixin):
    """One layer of the packed cache (reference: packed_qmse_cache.py:163-885)."""

    is_sliding = False

    def __init__(
        self,
        bits: int,
        seed: int = 0,
        grid_size: int = 32769,
        num_outlier_channels: int = 0,
        outlier_extra_bits: int = 1,
        use_qjl_keys: bool = False,
        quantize_decode: bool = False,
        reserve_tokens: int = 0,
        shard: HeadShard | None = None,
    ):
        super().__init__()
        if num_outlier_channels and shard is not None and shard.world_size > 1:
            raise NotImplementedError("the outlier-channel split is not available for a sharded cache")
        self.is_initialized = False
        self.bits = bits
        self.seed = seed
        self.grid_size = grid_size
        self.num_outlier_channels = num_outlier_channels
        self.outlier_extra_bits = outlier_extra_bits
        self.use_qjl_keys = use_qjl_keys
        self.quantize_decode = quantize_decode
        self.reserve_tokens = int(reserve_tokens)
        self.shard = shard or HeadShard()

        self.device: torch.device | None = None
        self.dtype: torch.dtype | None = None
        self.codec: Codec | None = None
        self.store: PackedStore | None = None
        self._force_dense = False
        self._lazy_update = False
        self._dense_k = _GrowingDense()
        self._dense_v = _GrowingDense()
        self._kv_heads_total: int | None = None
        self._static_pos: torch.Tensor | None = None  # see begin_static_decode
        self._stream_threshold: float | None = None   # see build_streaming_prefill_cache
        self._mask_bound = False                      # see bind_attention_mask
        self._tokens_seen = 0                         # tokens handed to this layer (sequence split: not all are stored here)
        self._window: tuple[int, int] | None = None   # (first batch row, total batch) of a prompt pass run in row blocks
        self._window_dense: bool | None = None        # the norm-guard decision of such a pass (taken on its first block)
        self._window_norm = [0.0, 0]                  # running (sum of block means x rows, rows) of such a pass
        self._prefill_shape: tuple[int, ...] | None = None
        self._static_kv: tuple[torch.Tensor, torch.Tensor] | None = None
        self._static_gather = None
        self._split = False  # outlier-channel split in use (see lazy_initialization)

    # ---------------------------------------------------------------- reference attributes
    @property
    def _outlier_enabled(self) -> bool:
        """Whether this layer splits off outlier channels (decided with the first tensors it sees:
        the reference needs ``0 < num_outlier_channels < head_dim``, packed_qmse_cache.py:243)."""
        return self._split

    def _table(self, name: str, key_side: bool = False):
        if key_side and not self.use_qjl_keys:
            return None
        if self._split:
            return getattr(self.store.normal, name) if self.store is not None else None
        return self.codec.table(name) if self.codec else None

    @property
    def rotation(self):
        return self._table("rot_v")

    @property
    def centers(self):
        return self._table("cen_v")

    @property
    def boundaries(self):
        return self._table("bnd_v")

    @property
    def _key_rotation(self):
        return self._table("rot_k", True)

    @property
    def _key_centers(self):
        return self._table("cen_k", True)

    @property
    def _key_boundaries(self):
        return self._table("bnd_k", True)

    @property
    def _qjl_matrix(self):
        return self._table("qjl", True)

    @property
    def _outlier_indices(self):
        return self.store.outlier.index if self._split and self.store is not None else None

    @property
    def _normal_indices(self):
        return self.store.normal.index if self._split and self.store is not None else None

    @property
    def _dense_keys(self):
        return self._dense_k.view()

    @property
    def _dense_values(self):
        return self._dense_v.view()

    def _shape(self) -> tuple[int, int, int, int]:
        s = self.store
        return (s.batch, s.kv_heads, s.length, 128)

    def _group_view(self, group: int, which: str):
        """The reference's view of one channel group of a split layer (0: the normal channels,
        1: the outlier channels; packed_qmse_cache.py:199-213,351-358)."""
        s = self.store
        if not self._split or s is None or s.length == 0 or (which == "qjl" and not self.use_qjl_keys):
            return None
        gs, n = s.groups[group], s.length
        shape = (s.batch, s.kv_heads, n, gs.g.dim)
        if which == "keys":
            return PackedTensorMSE(gs.k_codes[:, :, :n], gs.k_norms[:, :, :n], shape, self.dtype, gs.g.key_bits)
        if which == "values":
            return PackedTensorMSE(gs.v_codes[:, :, :n], gs.v_norms[:, :, :n], shape, self.dtype, gs.g.bits)
        return PackedQJL(gs.k_signs[:, :, :n], gs.k_rnorms[:, :, :n], gs.g.dim)

    @property
    def keys_packed(self) -> PackedTensorMSE | None:
        if self._split:
            return self._group_view(0, "keys")
        s = self.store
        if s is None or s.length == 0:
            return None
        n = s.length
        return PackedTensorMSE(s.k_codes[:, :, :n], s.k_norms[:, :, :n], self._shape(), self.dtype, s.codec.key_bits)

    @property
    def values_packed(self) -> PackedTensorMSE | None:
        if self._split:
            return self._group_view(0, "values")
        s = self.store
        if s is None or s.length == 0:
            return None
        n = s.length
        return PackedTensorMSE(s.v_codes[:, :, :n], s.v_norms[:, :, :n], self._shape(), self.dtype, s.codec.bits)

    @property
    def _keys_qjl(self) -> PackedQJL | None:
        if self._split:
            return self._group_view(0, "qjl")
        s = self.store
        if s is None or s.length == 0 or not self.use_qjl_keys:
            return None
        n = s.length
        return PackedQJL(s.k_signs[:, :, :n], s.k_rnorms[:, :, :n], 128)

    @property
    def _keys_outlier(self) -> PackedTensorMSE | None:
        return self._group_view(1, "keys")

    @property
    def _values_outlier(self) -> PackedTensorMSE | None:
        return self._group_view(1, "values")

    @property
    def _keys_outlier_qjl(self) -> PackedQJL | None:
        return self._group_view(1, "qjl")

    # ---------------------------------------------------------------- set-up
    def lazy_initialization(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        """Bind to the tensors' device and dtype and fetch the shared codec context
        (reference: packed_qmse_cache.py:237-283)."""
        self.dtype = key_states.dtype
        self.device = key_states.device
        self._split = 0 < self.num_outlier_channels < int(key_states.shape[-1])
        if not self._split:  # (a split layer is served by tensor arithmetic: it needs no kernel context)
            self.codec = Codec.get(self.device, self.bits, self.use_qjl_keys, self.seed, self.grid_size,
                                   int(key_states.shape[-1]))
        self.is_initialized = True

    def _new_store(self, key_states: torch.Tensor, value_states: torch.Tensor, batch: int, heads: int, capacity: int):
        if self._split:
            # the outlier channels are chosen on these very tensors: the first K/V the layer sees
            # (packed_qmse_cache.py:243-247)
            from tq_local_b200.runtime import ffi, outlier_split
            from tq_local_b200.runtime.outlier_split import SplitStore

            if key_states.device.type != "cuda" and not outlier_split.HOST_TENSORS_FOR_TESTS:
                raise ffi.TQError("TurboQuant-B200 runs on CUDA devices only; there is no CPU path")
            return SplitStore(key_states, value_states, self.bits, self.num_outlier_channels, self.outlier_extra_bits,
                              self.use_qjl_keys, self.seed, self.grid_size, batch, capacity)
        return PackedStore(self.codec, batch, heads, capacity)

    def _ensure_store(self, key_states: torch.Tensor, value_states: torch.Tensor | None = None) -> None:
        if self.store is None:
            local = self.shard.local_tokens(self.shard.local_kv(key_states), int(key_states.shape[1]), self._tokens_seen)
            cap = int(local.shape[2]) + self.reserve_tokens
            self.store = self._new_store(key_states, value_states, int(local.shape[0]), int(local.shape[1]), cap)
            self._kv_heads_total = int(key_states.shape[1])

    @property
    def seq_parts(self) -> int:
        """Ranks that share the tokens of each of this layer's KV heads (1: plain head sharding)."""
        return 1 if self._kv_heads_total is None else self.shard.seq_parts(self._kv_heads_total)

    def _local(self, key_states: torch.Tensor, value_states: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """This rank's share of new K/V [B, Hkv, T, D]: its KV heads and, when several ranks share
        a head, its tokens.  Counts the tokens as seen."""
        heads = int(key_states.shape[1])
        k = self.shard.local_tokens(self.shard.local_kv(key_states), heads, self._tokens_seen)
        v = self.shard.local_tokens(self.shard.local_kv(value_states), heads, self._tokens_seen)
        self._tokens_seen += int(key_states.shape[2])
        return k, v

    def initialize_from_dense(self, key_states: torch.Tensor, value_states: torch.Tensor, *,
                              force_dense: bool = False) -> None:
        """Pack a dense prefill cache (reference: packed_qmse_cache.py:332-374)."""
        if force_dense:
            self.device, self.dtype = key_states.device, key_states.dtype
            self._dense_k.append(key_states, self.reserve_tokens)
            self._dense_v.append(value_states, self.reserve_tokens)
            self._force_dense = True
            self.is_initialized = True
            return
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        self._ensure_store(key_states, value_states)
        self.store.pack(*self._local(key_states, value_states))

    # ---------------------------------------------------------------- replayable decode
    def supports_static_decode(self, q_heads: int) -> bool:
        """Whether this layer can serve decode steps whose length lives on the device (packed,
        quantised appends, 16-bit cache, at most 8 query heads per KV head).  A sharded layer
        additionally needs a device-sequenced ``PeerGather`` (see ``begin_static_decode``)."""
        return (self.store is not None and not self._split and not self._force_dense and self.quantize_decode
                and self.seq_parts == 1
                and self._dense_k.length == 0 and self.dtype in (torch.float16, torch.bfloat16)
                and q_heads // self._kv_heads_total <= 8)

    def begin_static_decode(self, pos: torch.Tensor, max_new_tokens: int, gather=None) -> None:
        """Switch to decode steps that read the cache length from the int32 device scalar ``pos``
        (shared by all layers of a model and advanced by the caller once per step).  From here on
        ``update`` only remembers the new token and ``attend`` appends it and attends in one fused
        call, neither touching host-side state: the whole model step can be recorded in a CUDA
        graph.  ``end_static_decode`` returns to the normal bookkeeping."""
        if self.shard.world_size > 1 and gather is None:
            raise RuntimeError("a sharded layer needs a PeerGather(device_sequence=True) for static decode")
        self.store.reserve(self.store.length + int(max_new_tokens))
        self._static_pos = pos
        self._static_gather = gather if self.shard.world_size > 1 else None

    def end_static_decode(self, new_length: int) -> None:
        self._static_pos, self._static_kv, self._static_gather = None, None, None
        self.store.length = int(new_length)

    # ---------------------------------------------------------------- decode-time update
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor,
               cache_kwargs: dict[str, Any] | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """HF cache hook (reference: packed_qmse_cache.py:600-624)."""
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        if self._static_pos is not None:
            if key_states.shape[2] != 1:
                raise RuntimeError("static decode serves one new token per step")
            self._static_kv = (key_states, value_states)
            return key_states, value_states
        if self._stream_threshold is not None:
            # Streaming prefill: this is the prompt's K/V of this layer.  Pack it now (or keep it
            # dense under the norm guard) and hand the dense tensors back for the prompt's own
            # attention; nothing dense outlives the layer's forward pass.
            threshold, self._stream_threshold = self._stream_threshold, None
            if self._window is not None:
                self._update_prefill_block(key_states, value_states, threshold)
                return key_states, value_states
            self._prefill_shape = tuple(key_states.shape)
            dense = threshold != float("inf") and float(key_norm_mean(key_states).item()) > threshold
            self.initialize_from_dense(key_states, value_states, force_dense=dense)
            return key_states, value_states
        if self._force_dense:
            return self._update_dense_decode(key_states, value_states)
        if self._lazy_update:
            return self._update_lazy(key_states, value_states)
        if not self.quantize_decode:
            return self._update_dense_decode(key_states, value_states)
        # Eager path: hand back the dequantised history plus the new token, then store it.
        prev_k, prev_v = self._decode_keys_full(), self._decode_values_full()
        self._ensure_store(key_states, value_states)
        if self.seq_parts > 1:
            raise NotImplementedError("a sequence-split cache serves attention through the 'turboquant' backend only "
                                      "(enable_turboquant_attention); it cannot hand back dequantised history")
        self.store.pack(*self._local(key_states, value_states))
        if prev_k is None:
            return key_states, value_states
        return (torch.cat((prev_k, self.shard.local_kv(key_states)), dim=-2),
                torch.cat((prev_v, self.shard.local_kv(value_states)), dim=-2))

    def _update_prefill_block(self, key_states, value_states, threshold: float) -> None:
        """Streaming prefill of a prompt pass that runs the batch a few rows at a time: this is the
        prompt's K/V of rows ``[b0, b0 + kb)``.  The norm-guard decision of the layer is taken on
        the first block (the reference takes it on the whole batch at once,
        packed_qmse_cache.py:918-929; key norms are a property of the layer, not of the sequence)
        and the running mean over all blocks is kept so that ``finish_prefill`` can tell if the
        whole-batch rule would have decided otherwise."""
        b0, total = self._window
        kb, _, n, _ = key_states.shape
        if threshold != float("inf"):
            mean = float(key_norm_mean(key_states).item())
            self._window_norm[0] += mean * kb
            self._window_norm[1] += kb
            if self._window_dense is None:
                self._window_dense = mean > threshold
        elif self._window_dense is None:
            self._window_dense = False
        self._prefill_shape = (total, *key_states.shape[1:])
        if self._window_dense:
            self.device, self.dtype = key_states.device, key_states.dtype
            self._dense_k.write_rows(key_states, b0, total, self.reserve_tokens)
            self._dense_v.write_rows(value_states, b0, total, self.reserve_tokens)
            self._force_dense = True
            self.is_initialized = True
            return
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        self._kv_heads_total = int(key_states.shape[1])
        seen = self._tokens_seen
        local_k, local_v = self._local(key_states, value_states)
        self._tokens_seen = seen  # (every row block brings the same token positions; finish_prefill counts them once)
        if self.store is None:  # (a split layer chooses its outlier channels on this first block)
            self.store = self._new_store(key_states, value_states, total, int(local_k.shape[1]),
                                         int(local_k.shape[2]) + self.reserve_tokens)
        self.store.pack_rows(local_k, local_v, b0, 0)
        self._window_local = int(local_k.shape[2])

    def begin_prefill_block(self, b0: int, total_batch: int, threshold: float) -> None:
        """Arm the layer for the prompt K/V of batch rows starting at ``b0`` (of ``total_batch``)."""
        self._window = (int(b0), int(total_batch))
        self._stream_threshold = threshold

    def finish_prefill(self, n_tokens: int, threshold: float) -> bool:
        """All row blocks are in: the cache now holds ``n_tokens`` tokens per row.  Returns whether
        the whole-batch norm-guard rule agrees with the decision taken on the first block."""
        self._window, self._stream_threshold = None, None
        if self._force_dense:
            self._dense_k.length = self._dense_v.length = int(n_tokens)
        elif self.store is not None:
            self.store.length = int(getattr(self, "_window_local", n_tokens))  # (a sequence split stores a piece)
        self._tokens_seen = int(n_tokens)
        s, rows = self._window_norm
        return rows == 0 or ((s / rows) > threshold) == bool(self._window_dense)

    def _update_lazy(self, key_states, value_states):
        """Store the new token without touching history (reference: packed_qmse_cache.py:626-679):
        quantised in place when ``quantize_decode``, otherwise appended to the dense tail."""
        if self.quantize_decode:
            self._ensure_store(key_states, value_states)
            self.store.pack(*self._local(key_states, value_states))
        else:
            if self.seq_parts > 1:
                raise NotImplementedError("quantize_decode=False is not available when several ranks share a KV head")
            self._dense_k.append(self.shard.local_kv(key_states), self.reserve_tokens)
            self._dense_v.append(self.shard.local_kv(value_states), self.reserve_tokens)
            self._tokens_seen += int(key_states.shape[2])
        return key_states, value_states

    def _update_dense_decode(self, key_states, value_states):
        """Keep generated tokens dense and return the full K/V (packed_qmse_cache.py:681-705)."""
        if not self._force_dense:
            key_states, value_states = self.shard.local_kv(key_states), self.shard.local_kv(value_states)
        dk = self._dense_k.append(key_states, self.reserve_tokens)
        dv = self._dense_v.append(value_states, self.reserve_tokens)
        pk, pv = self._decode_keys_full(), self._decode_values_full()
        if pk is None:
            return dk, dv
        return torch.cat((pk, dk), dim=-2), torch.cat((pv, dv), dim=-2)

    # ---------------------------------------------------------------- attention
    def bind_attention_mask(self, mask: torch.Tensor | None, lock: bool | None = None) -> None:
        """Fix which cached tokens every batch row attends for the decode steps that follow: ``mask``
        is the prompt's 2-D mask [B, S] (1 / True = attend) of a LEFT-padded batch, or a 4-D mask
        [B, 1, Sq, Skv] (bool keep-mask or additive float) of the same shape of padding; row ``b``
        then attends tokens from its first kept position on.  ``None`` removes the restriction.
        While the binding is locked (``lock``; default: locked exactly when a mask is given),
        per-call masks handed to ``attend`` are not looked at: the padding of a batch does not
        change during generation, so a generation loop binds once - also for an unpadded batch -
        and spares every layer and step the look at the mask the model passes down."""
        if self.store is None or self._force_dense:
            return
        if mask is not None and self.seq_parts > 1:
            raise NotImplementedError("padded batches are not available when several ranks share a KV head")
        self.store.set_seq_start(None if mask is None else leading_masked_tokens(mask))
        self._mask_bound = (mask is not None) if lock is None else bool(lock)

    def attend(self, query_states: torch.Tensor, attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        """Decode attention of ``query_states`` [B, Hq, Sq, D] over this layer's cache, returning
        [B, Hq, Sq, D] in the query dtype.  ``Sq > 1`` is served one query position at a
        time with causal visibility (the new tokens were appended before attention).  An
        ``attention_mask`` (see ``bind_attention_mask`` for the accepted forms) restricts every
        row to the tokens after its left padding, which is what the reference's chunked path does
        by adding the mask to its logits (attention.py:253-255,278-283)."""
        if self.store is None or self._force_dense:
            raise RuntimeError("attend() needs a packed (non-dense) layer")
        if not self._mask_bound and self._static_pos is None:  # (a recorded step keeps the offsets it was given)
            if attention_mask is not None:
                self.store.set_seq_start(leading_masked_tokens(attention_mask))
            elif self.store._seq_start is not None:
                self.store.set_seq_start(None)
        if self._static_pos is not None:
            k_new, v_new = self._static_kv
            # (sharded: the combine kernel writes every rank's gathered buffer, the result is complete)
            return self.store.decode_step_dev(self.shard.local_q(query_states, self._kv_heads_total),
                                              self.shard.local_kv(k_new), self.shard.local_kv(v_new), self._static_pos,
                                              gather=self._static_gather)
        b, hq, sq, d = query_states.shape
        q_local = self.shard.local_q(query_states, self._kv_heads_total)
        if self.seq_parts > 1:
            # Several ranks share each KV head: every rank attends its part of the tokens, the partials
            # are exchanged and every rank finishes the whole output (no gather of outputs afterwards).
            if sq != 1:
                raise NotImplementedError("a sequence-split cache serves one query token per step")
            from tq_local_b200.runtime.sharding import PeerGather

            gather = PeerGather.shared(self.shard, b, hq, query_states.dtype, query_states.device, self.seq_parts)
            return self.store.decode_attn_parts(q_local, gather)
        tail_k, tail_v = self._dense_k.view(), self._dense_v.view()
        n_tail = 0 if tail_k is None else int(tail_k.shape[2])
        outs = []
        for i in range(sq):
            behind = sq - 1 - i  # tokens of this very call that position i must not see
            if self.quantize_decode or n_tail == 0:
                out = self.store.decode_attn(q_local[:, :, i:i + 1], seq_len=self.store.length - behind,
                                             tail_k=tail_k, tail_v=tail_v)
            else:
                out = self.store.decode_attn(q_local[:, :, i:i + 1], tail_k=tail_k[:, :, :n_tail - behind],
                                             tail_v=tail_v[:, :, :n_tail - behind])
            outs.append(out)
        out = outs[0] if sq == 1 else torch.cat(outs, dim=2)
        return self.shard.gather_heads(out)

    def attend_with_new_tokens(self, query_states: torch.Tensor, new_key: torch.Tensor, new_value: torch.Tensor,
                               attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        """``attend`` over the cache plus ``new_key`` / ``new_value`` [B, Hkv, T, D], tokens that are
        not stored (and are not stored by this call): they are attended un-quantised after the
        cached ones, as the reference's chunked path does with its ``new_key`` argument
        (attention.py:286-297).  Every query position sees all T new tokens."""
        if self.store is None or self._force_dense:
            raise RuntimeError("attend_with_new_tokens() needs a packed (non-dense) layer")
        if attention_mask is not None and not self._mask_bound:
            self.store.set_seq_start(leading_masked_tokens(attention_mask))
        q_local = self.shard.local_q(query_states, self._kv_heads_total)
        tail_k, tail_v = self.shard.local_kv(new_key), self.shard.local_kv(new_value)
        if self._dense_k.length:
            tail_k = torch.cat((self._dense_k.view(), tail_k), dim=2)
            tail_v = torch.cat((self._dense_v.view(), tail_v), dim=2)
        tail_k, tail_v = tail_k.to(query_states.dtype), tail_v.to(query_states.dtype)
        outs = [self.store.decode_attn(q_local[:, :, i:i + 1], tail_k=tail_k, tail_v=tail_v)
                for i in range(int(query_states.shape[2]))]
        out = outs[0] if len(outs) == 1 else torch.cat(outs, dim=2)
        return self.shard.gather_heads(out)

    # ---------------------------------------------------------------- dequantisation
    def _decode_keys_full(self) -> torch.Tensor | None:
        if self.store is None or self.store.length == 0:
            return None
        return self.store.dequant("keys", dtype=self.dtype)

    def _decode_values_full(self) -> torch.Tensor | None:
        if self.store is None or self.store.length == 0:
            return None
        return self.store.dequant("values", dtype=self.dtype)

    def _decode_keys_range(self, start: int, end: int) -> torch.Tensor:
        return self.store.dequant("keys", start, end, dtype=self.dtype)

    def _decode_values_range(self, start: int, end: int) -> torch.Tensor:
        return self.store.dequant("values", start, end, dtype=self.dtype)

    # ---------------------------------------------------------------- bookkeeping
    def packed_seq_length(self) -> int:
        return 0 if self.store is None else int(self.store.length)

    def get_seq_length(self) -> int:
        if self.seq_parts > 1:
            return self._tokens_seen  # (this rank stores only its part of them)
        return self.packed_seq_length() + self._dense_k.length

    def get_mask_sizes(self, cache_position) -> tuple[int, int]:
        """(kv_length, kv_offset); newer ``transformers`` pass the query length as an int,
        older ones a position tensor (reference: packed_qmse_cache.py:860-864)."""
        q_len = cache_position if isinstance(cache_position, int) else int(cache_position.shape[0])
        return self.get_seq_length() + q_len, 0

    def get_max_cache_shape(self) -> int:
        return -1

    def storage_bytes(self) -> int:
        """Bytes held for the stored tokens (reference: packed_qmse_cache.py:874-885)."""
        total = 0 if self.store is None else self.store.storage_bytes()
        for dense in (self._dense_k.view(), self._dense_v.view()):
            if dense is not None:
                total += dense.numel() * dense.element_size()
        return int(total)


_APPROX_DMSE_UNIT: dict[int, float] = {2: 0.079, 3: 0.030, 4: 0.009, 5: 0.003, 6: 0.0008, 7: 0.0002, 8: 0.00005}


def _auto_norm_threshold(bits: int, head_dim: int, mse_budget: float = 1.0) -> float:
    """Largest mean key norm a layer may have before it is kept dense:
    ``norm^2 * D_mse(bits) / head_dim < mse_budget`` (reference: packed_qmse_cache.py:888-900)."""
    return sqrt(mse_budget * head_dim / _APPROX_DMSE_UNIT.get(bits, 0.03))


def _layer_kv(layer) -> tuple[torch.Tensor, torch.Tensor]:
    if isinstance(layer, (tuple, list)):
        return layer[0], layer[1]
    return layer.keys, layer.values


def build_packed_mse_cache(
    past_key_values,
    bits: int,
    seed: int = 0,
    grid_size: int = 32769,
    num_outlier_channels: int = 0,
    outlier_extra_bits: int = 1,
    use_qjl_keys: bool = False,
    quantize_decode: bool = False,
    norm_guard: bool = True,
    reserve_tokens: int = 0,
    shard: HeadShard | None = None,
    release_dense: bool = False,
) -> Cache:
    """Pack every layer of a dense prefill cache (reference: packed_qmse_cache.py:903-951).

    A layer whose MEAN key norm exceeds ``sqrt(head_dim / D_mse(bits))`` stays dense when
    ``norm_guard`` is on.  The per-layer means are computed on the device and fetched with a
    single host synchronisation.  ``release_dense`` drops each dense layer from a
    ``DynamicCache`` right after it has been packed, so peak memory is one dense layer.
    """
    source_layers = past_key_values.layers if hasattr(past_key_values, "layers") else list(past_key_values)
    pairs = [_layer_kv(layer) for layer in source_layers]
    head_dim = int(pairs[0][0].shape[-1]) if pairs else 128
    threshold = _auto_norm_threshold(bits, head_dim) if norm_guard else float("inf")
    if norm_guard and pairs:
        means = torch.stack([key_norm_mean(k) for k, _ in pairs]).tolist()
    else:
        means = [0.0] * len(pairs)

    layers: list[PackedMSELayer] = []
    for idx, (k, v) in enumerate(pairs):
        layer = PackedMSELayer(bits=bits, seed=seed, grid_size=grid_size, num_outlier_channels=num_outlier_channels,
                               outlier_extra_bits=outlier_extra_bits, use_qjl_keys=use_qjl_keys,
                               quantize_decode=quantize_decode, reserve_tokens=reserve_tokens, shard=shard)
        layer.initialize_from_dense(k, v, force_dense=means[idx] > threshold)
        layers.append(layer)
        if release_dense and hasattr(source_layers[idx], "keys") and not layer._force_dense:
            source_layers[idx].keys = source_layers[idx].values = None
    dense_ids = [i for i, m in enumerate(means) if m > threshold]
    if dense_ids:
        print(f"[TurboQuant] norm_guard: {len(dense_ids)}/{len(layers)} layers kept dense "
              f"(threshold={threshold:.1f}, layers={dense_ids})", file=sys.stderr)
    return Cache(layers=layers)


def build_streaming_prefill_cache(
    num_layers: int,
    bits: int,
    head_dim: int = 128,
    seed: int = 0,
    grid_size: int = 32769,
    num_outlier_channels: int = 0,
    outlier_extra_bits: int = 1,
    use_qjl_keys: bool = False,
    quantize_decode: bool = False,
    norm_guard: bool = True,
    reserve_tokens: int = 0,
    shard: HeadShard | None = None,
) -> Cache:
    """An empty packed cache to run the PROMPT pass with: each layer packs its keys / values the
    moment the model hands them over (``update``), applying the same norm-guard rule as
    ``build_packed_mse_cache``, so the dense cache of the whole model (the reference's
    generation.py:91-129) never exists — peak memory holds one layer's dense K/V."""
    threshold = _auto_norm_threshold(bits, head_dim) if norm_guard else float("inf")
    layers = []
    for _ in range(num_layers):
        layer = PackedMSELayer(bits=bits, seed=seed, grid_size=grid_size, num_outlier_channels=num_outlier_channels,
                               outlier_extra_bits=outlier_extra_bits, use_qjl_keys=use_qjl_keys,
                               quantize_decode=quantize_decode, reserve_tokens=reserve_tokens, shard=shard)
        layer._stream_threshold = threshold
        layers.append(layer)
    return Cache(layers=layers)


def report_streamed_norm_guard(cache: Cache, bits: int, head_dim: int = 128) -> None:
    """The norm-guard notice of ``build_packed_mse_cache`` for a cache filled by a streaming prefill."""
    dense_ids = [i for i, layer in enumerate(cache.layers) if layer._force_dense]
    if dense_ids:
        print(f"[TurboQuant] norm_guard: {len(dense_ids)}/{len(cache.layers)} layers kept dense "
              f"(threshold={_auto_norm_threshold(bits, head_dim):.1f}, layers={dense_ids})", file=sys.stderr)


def streamed_prefill_memory_breakdown(cache: Cache) -> dict[str, Any]:
    """What ``past_key_values_memory_breakdown`` reports for the dense prompt cache, computed
    from the shapes the layers saw (the dense tensors themselves were never kept)."""
    shapes = [(layer._prefill_shape, layer.dtype) for layer in cache.layers if layer._prefill_shape is not None]
    per_kind = sum(b * h * s * d * torch.empty((), dtype=dt).element_size() for (b, h, s, d), dt in shapes)
    return {
        "num_layers": len(shapes),
        "vector_dimension": shapes[0][0][3] if shapes else None,
        "num_key_value_vectors_per_kind": sum(b * h * s for (b, h, s, _), _ in shapes),
        "key_bytes": per_kind,
        "value_bytes": per_kind,
        "dense_kv_bytes": 2 * per_kind,
        "extra_tensor_bytes": 0,
        "total_cache_tensor_bytes": 2 * per_kind,
    }


def verify_packed_reconstruction(original_cache, packed_cache: Cache) -> list[dict[str, Any]]:
    """Per-layer reconstruction quality against the dense cache (reference:
    packed_qmse_cache.py:954-1009; same keys, same rounding)."""
    source_layers = original_cache.layers if hasattr(original_cache, "layers") else list(original_cache)
    report: list[dict[str, Any]] = []
    for idx, src in enumerate(source_layers):
        k0, v0 = _layer_kv(src)
        layer: PackedMSELayer = packed_cache.layers[idx]
        dense = layer._force_dense
        if dense:
            k1, v1 = layer._dense_keys, layer._dense_values
        else:
            heads = int(k0.shape[1])  # (a sequence split holds a piece of the prompt's tokens on this rank)
            k0 = layer.shard.local_tokens(layer.shard.local_kv(k0), heads, 0)
            v0 = layer.shard.local_tokens(layer.shard.local_kv(v0), heads, 0)
            k1, v1 = layer._decode_keys_full(), layer._decode_values_full()
        k0, v0, k1, v1 = k0.float(), v0.float(), k1.float(), v1.float()
        dk, dv = k0 - k1, v0 - v1
        cos = torch.nn.functional.cosine_similarity
        stats = torch.stack([
            (dk ** 2).mean(), cos(k0.reshape(-1, k0.shape[-1]), k1.reshape(-1, k1.shape[-1]), dim=-1).mean(),
            dk.abs().max(), k0.norm(dim=-1).mean(),
            (dv ** 2).mean(), cos(v0.reshape(-1, v0.shape[-1]), v1.reshape(-1, v1.shape[-1]), dim=-1).mean(),
            dv.abs().max(), v0.norm(dim=-1).mean(),
        ]).tolist()
        report.append({
            "layer": idx, "dense": dense,
            "key_mse": round(stats[0], 6), "key_cosine_sim": round(stats[1], 6),
            "key_max_abs_error": round(stats[2], 6), "key_mean_norm": round(stats[3], 4),
            "val_mse": round(stats[4], 6), "val_cosine_sim": round(stats[5], 6),
            "val_max_abs_error": round(stats[6], 6), "val_mean_norm": round(stats[7], 4),
        })
    return report


def packed_cache_storage_bytes(cache: Cache) -> int:
    return int(sum(layer.storage_bytes() for layer in cache.layers if hasattr(layer, "storage_bytes")))


def packed_cache_storage_breakdown(cache: Cache) -> dict[str, int]:
    per_layer = [int(layer.storage_bytes()) for layer in cache.layers if hasattr(layer, "storage_bytes")]
    return {
        "packed_total_bytes": int(sum(per_layer)),
        "packed_layer_mean_bytes": int(sum(per_layer) / len(per_layer)) if per_layer else 0,
        "packed_num_layers": len(per_layer),
    }
