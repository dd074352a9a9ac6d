"""Device storage of one layer's packed KV cache and the calls that touch it.

Layout in HBM (all streams row-major, token axis second to last):

    k_codes  uint8 [B, Hkv, capacity, 16*key_bits]   LSB-first bitstream per token
    k_norms  fp16  [B, Hkv, capacity]
    k_signs  uint8 [B, Hkv, capacity, 16]            (Q_prod only) 1 bit per coordinate
    k_rnorms fp16  [B, Hkv, capacity]                (Q_prod only)
    v_codes  uint8 [B, Hkv, capacity, 16*bits]
    v_norms  fp16  [B, Hkv, capacity]

``[:, :, :length]`` of each stream is byte-for-byte what the reference keeps in
``PackedTensorMSE.packed_indices`` / ``.norms`` and ``PackedQJL.packed_signs`` /
``.residual_norms`` (``src/turboquant/runtime/packed_qmse_cache.py:58-92,121-140``).
The spare capacity makes the append of a decoded token an in-place write
instead of the reference's ``torch.cat`` of the whole cache.
"""

from __future__ import annotations

import ctypes as C

import torch

from tq_local_b200.runtime import ffi
from tq_local_b200.runtime.codec import Codec, dense_desc, tq_dtype


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class PackedStore:
    def __init__(self, codec: Codec, batch: int, kv_heads: int, capacity: int):
        self.codec = codec
        self.batch, self.kv_heads = int(batch), int(kv_heads)
        self.length = 0
        self._seq_start: torch.Tensor | None = None  # see set_seq_start
        self._alloc(max(8, _round_up(int(capacity), 8)))
        self._workspace: torch.Tensor | None = None
        self._step_plan = None

    # ------------------------------------------------------------------ storage
    def _alloc(self, capacity: int) -> None:
        dev, b, h = self.codec.device, self.batch, self.kv_heads
        u8 = dict(dtype=torch.uint8, device=dev)
        f16 = dict(dtype=torch.float16, device=dev)
        self.capacity = capacity
        self.k_codes = torch.empty(b, h, capacity, 16 * self.codec.key_bits, **u8)
        self.k_norms = torch.empty(b, h, capacity, **f16)
        self.v_codes = torch.empty(b, h, capacity, 16 * self.codec.bits, **u8)
        self.v_norms = torch.empty(b, h, capacity, **f16)
        if self.codec.use_qjl:
            self.k_signs = torch.empty(b, h, capacity, 16, **u8)
            self.k_rnorms = torch.empty(b, h, capacity, **f16)
        else:
            self.k_signs = self.k_rnorms = None
        self._desc = ffi.CacheDesc(
            self.k_codes.data_ptr(), self.k_norms.data_ptr(),
            self.k_signs.data_ptr() if self.k_signs is not None else None,
            self.k_rnorms.data_ptr() if self.k_rnorms is not None else None,
            self.v_codes.data_ptr(), self.v_norms.data_ptr(),
            b, h, capacity, h * capacity, capacity,
            self._seq_start.data_ptr() if self._seq_start is not None else None,
        )
        self._desc_ref = C.byref(self._desc)
        self._step_plan = None

    def set_seq_start(self, seq_start: torch.Tensor | None) -> None:
        """Per-row first attended token (int32 [batch] on the cache's device): the decode calls then
        attend tokens ``[seq_start[b], length)`` of batch entry ``b`` - a left-padded batch.  ``None``
        (the default) attends every row from token 0."""
        if seq_start is not None:
            if seq_start.dtype != torch.int32 or seq_start.device != self.codec.device or \
                    tuple(seq_start.shape) != (self.batch,) or not seq_start.is_contiguous():
                raise ValueError(f"seq_start must be a contiguous int32 tensor [{self.batch}] on {self.codec.device}")
        self._seq_start = seq_start
        self._desc.seq_start = seq_start.data_ptr() if seq_start is not None else None

    def streams(self) -> list[torch.Tensor]:
        return [t for t in (self.k_codes, self.k_norms, self.k_signs, self.k_rnorms, self.v_codes, self.v_norms)
                if t is not None]

    def reserve(self, capacity: int) -> None:
        """Grow to at least ``capacity`` tokens per row, keeping the stored tokens."""
        if capacity <= self.capacity:
            return
        old = self.streams()
        n = self.length
        self._alloc(_round_up(max(capacity, 2 * self.capacity), 8))
        for src, dst in zip(old, self.streams()):
            dst[:, :, :n].copy_(src[:, :, :n])

    def storage_bytes(self) -> int:
        """Bytes of the ``length`` stored tokens (what the reference's ``storage_bytes`` counts)."""
        per_token = sum(t[0, 0, 0].numel() * t.element_size() for t in self.streams())
        return int(per_token * self.batch * self.kv_heads * self.length)

    # ------------------------------------------------------------------ kernels
    def _stream_ptr(self):
        return C.c_void_p(torch.cuda.current_stream(self.codec.device).cuda_stream)

    def pack(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """Quantise ``k``/``v`` [B, Hkv, T, 128] and append them at the current length."""
        if k.shape != v.shape or k.dtype != v.dtype:
            raise ValueError("key and value tensors must have the same shape and dtype")
        if k.shape[0] != self.batch or k.shape[1] != self.kv_heads:
            raise ValueError("Packed tensor append requires matching batch, head, and dimension shape.")
        if k.device != self.codec.device:
            raise ffi.TQError(f"tensor on {k.device}, cache on {self.codec.device}")
        n = int(k.shape[2])
        if n == 0:
            return
        if k.stride(-1) != 1:
            k = k.contiguous()
        if v.stride(-1) != 1:
            v = v.contiguous()
        self.reserve(self.length + n)
        kd, vd = dense_desc(k), dense_desc(v)
        with torch.cuda.device(self.codec.device):
            ffi.check(ffi.lib().tq_pack(self.codec.handle, C.byref(kd), C.byref(vd), n, C.byref(self._desc),
                                        self.length, self._stream_ptr()), "tq_pack")
        self.length += n

    def pack_rows(self, k: torch.Tensor, v: torch.Tensor, b0: int, pos0: int = 0) -> None:
        """Quantise ``k`` / ``v`` [kb, Hkv, T, 128] into batch rows ``[b0, b0 + kb)`` at token positions
        ``[pos0, pos0 + T)`` without touching ``length``: a prompt pass that runs a few sequences
        at a time fills the cache row block by row block and sets ``length`` when it is done."""
        kb, n = int(k.shape[0]), int(k.shape[2])
        if k.shape != v.shape or k.dtype != v.dtype or k.shape[1] != self.kv_heads:
            raise ValueError("key and value tensors must have the same shape and dtype and this cache's KV heads")
        if b0 < 0 or b0 + kb > self.batch or pos0 < 0 or pos0 + n > self.capacity:
            raise ValueError(f"rows [{b0}, {b0 + kb}) x tokens [{pos0}, {pos0 + n}) do not fit a cache of "
                             f"{self.batch} rows x {self.capacity} tokens")
        if n == 0 or kb == 0:
            return
        if k.stride(-1) != 1:
            k = k.contiguous()
        if v.stride(-1) != 1:
            v = v.contiguous()
        ptr = lambda t: None if t is None else t[b0:].data_ptr()
        desc = ffi.CacheDesc(ptr(self.k_codes), ptr(self.k_norms), ptr(self.k_signs), ptr(self.k_rnorms),
                             ptr(self.v_codes), ptr(self.v_norms), kb, self.kv_heads, self.capacity,
                             self.kv_heads * self.capacity, self.capacity, None)
        kd, vd = dense_desc(k), dense_desc(v)
        with torch.cuda.device(self.codec.device):
            ffi.check(ffi.lib().tq_pack(self.codec.handle, C.byref(kd), C.byref(vd), n, C.byref(desc), pos0,
                                        self._stream_ptr()), "tq_pack")

    def suggest_splits(self, seq_len: int | None = None) -> int:
        n = self.length if seq_len is None else seq_len
        return int(ffi.lib().tq_decode_suggest_splits(self.codec.handle, self.batch, self.kv_heads, max(n, 1)))

    def _get_workspace(self, q_heads: int, splits: int) -> torch.Tensor:
        need = int(ffi.lib().tq_decode_workspace_bytes(self.batch, q_heads, splits))
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = torch.empty(need, dtype=torch.uint8, device=self.codec.device)
            self._step_plan = None  # (it remembers the scratch address)
        return self._workspace

    def decode_attn(self, q: torch.Tensor, *, seq_len: int | None = None, tail_k: torch.Tensor | None = None,
                    tail_v: torch.Tensor | None = None, splits: int | None = None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
        """One decode step: ``q`` [B, Hq, 1, 128] (or [B, Hq, 128]) -> [B, Hq, 1, 128]."""
        b, hq = int(q.shape[0]), int(q.shape[1])
        if q.shape[-1] != 128 or q.numel() != b * hq * 128 or b != self.batch:
            raise ValueError(f"expected a single-token query [B={self.batch}, Hq, 1, 128], got {tuple(q.shape)}")
        qc = q.reshape(b, hq, 128)
        if not qc.is_contiguous():
            qc = qc.contiguous()
        n = self.length if seq_len is None else int(seq_len)
        n_tail = 0 if tail_k is None else int(tail_k.shape[2])
        if n_tail:
            tkd, tvd = dense_desc(tail_k), dense_desc(tail_v)
            tk_ref, tv_ref = C.byref(tkd), C.byref(tvd)
        else:
            tk_ref = tv_ref = None
        splits = self.suggest_splits(n) if splits is None else int(splits)
        ws = self._get_workspace(hq, splits)
        if out is None:
            out = torch.empty(b, hq, 1, 128, dtype=q.dtype, device=q.device)
        with torch.cuda.device(self.codec.device):
            ffi.check(ffi.lib().tq_decode_attn(self.codec.handle, qc.data_ptr(), tq_dtype(q.dtype), hq,
                                               C.byref(self._desc), n, tk_ref, tv_ref, n_tail, splits,
                                               ws.data_ptr(), ws.numel(), out.data_ptr(), self._stream_ptr()),
                      "tq_decode_attn")
        return out

    def decode_attn_f32(self, q: torch.Tensor, *, seq_len: int | None = None, splits: int | None = None) -> torch.Tensor:
        """``decode_attn`` for a 16-bit query with the result left unrounded: float32
        [B, Hq, 1, 128] (``tq_decode_attn_f32out``)."""
        b, hq = int(q.shape[0]), int(q.shape[1])
        if q.shape[-1] != 128 or q.numel() != b * hq * 128 or b != self.batch:
            raise ValueError(f"expected a single-token query [B={self.batch}, Hq, 1, 128], got {tuple(q.shape)}")
        qc = q.reshape(b, hq, 128)
        if not qc.is_contiguous():
            qc = qc.contiguous()
        n = self.length if seq_len is None else int(seq_len)
        splits = self.suggest_splits(n) if splits is None else int(splits)
        ws = self._get_workspace(hq, splits)
        out = torch.empty(b, hq, 1, 128, dtype=torch.float32, device=q.device)
        with torch.cuda.device(self.codec.device):
            ffi.check(ffi.lib().tq_decode_attn_f32out(self.codec.handle, qc.data_ptr(), tq_dtype(q.dtype), hq,
                                                      C.byref(self._desc), n, splits, ws.data_ptr(), ws.numel(),
                                                      out.data_ptr(), self._stream_ptr()), "tq_decode_attn_f32out")
        return out

    def decode_attn_gather(self, q: torch.Tensor, gather, *, seq_len: int | None = None,
                           splits: int | None = None) -> torch.Tensor:
        """``decode_attn`` for a KV-head shard with the exchange fused in: ``q`` holds this rank's
        query heads [B, Hq_local, 1, 128]; the result is the gathered output of ALL ranks
        [B, Hq_total, 1, 128] (a view of ``gather``'s buffer for this step, valid until the
        step after next).  ``gather`` is a ``PeerGather``; every rank must make the same calls."""
        b, hq = int(q.shape[0]), int(q.shape[1])
        if q.shape[-1] != 128 or q.numel() != b * hq * 128 or b != self.batch:
            raise ValueError(f"expected a single-token query [B={self.batch}, Hq, 1, 128], got {tuple(q.shape)}")
        qc = q.reshape(b, hq, 128)
        if not qc.is_contiguous():
            qc = qc.contiguous()
        n = self.length if seq_len is None else int(seq_len)
        splits = self.suggest_splits(n) if splits is None else int(splits)
        ws = self._get_workspace(hq, splits)
        desc, view = gather.next_desc()
        stream = self._stream_ptr()
        with torch.cuda.device(self.codec.device):
            ffi.check(ffi.lib().tq_decode_attn_gather(self.codec.handle, qc.data_ptr(), tq_dtype(q.dtype), hq,
                                                      C.byref(self._desc), n, splits, ws.data_ptr(), ws.numel(),
                                                      C.byref(desc), stream), "tq_decode_attn_gather")
            ffi.check(ffi.lib().tq_gather_wait(self.codec.handle, C.byref(desc), b, tq_dtype(q.dtype), None, stream),
                      "tq_gather_wait")
        return view

    def decode_attn_parts(self, q: torch.Tensor, gather, *, seq_len: int | None = None, splits: int | None = None,
                          out: torch.Tensor | None = None) -> torch.Tensor:
        """Decode attention when more ranks than KV heads share the cache: ``gather.parts`` ranks
        hold disjoint parts of the tokens of one group of KV heads (this store holds this rank's
        part, possibly no token at all), ``q`` [B, Hq_group, 1, 128] holds the group's query heads.
        The kernels exchange unfinished partials through ``gather`` (a ``PeerGather`` created with
        ``parts=``) and every rank finishes all rows: the result is the output of the whole model
        [B, Hq_total, 1, 128].  Every rank must make the same calls."""
        b, hq = int(q.shape[0]), int(q.shape[1])
        if q.shape[-1] != 128 or q.numel() != b * hq * 128 or b != self.batch:
            raise ValueError(f"expected a single-token query [B={self.batch}, Hq, 1, 128], got {tuple(q.shape)}")
        if not gather.parts:
            raise ValueError("decode_attn_parts needs a PeerGather created with parts=")
        qc = q.reshape(b, hq, 128)
        if not qc.is_contiguous():
            qc = qc.contiguous()
        n = self.length if seq_len is None else int(seq_len)
        splits = self.suggest_splits(max(n, 1)) if splits is None else int(splits)
        ws = self._get_workspace(hq, splits)
        desc, _ = gather.next_desc()
        if out is None:
            out = torch.empty(gather.shape, dtype=q.dtype, device=q.device)
        stream = self._stream_ptr()
        with torch.cuda.device(self.codec.device):
            ffi.check(ffi.lib().tq_decode_attn_parts(self.codec.handle, qc.data_ptr(), tq_dtype(q.dtype), hq,
                                                     C.byref(self._desc), n, splits, ws.data_ptr(), ws.numel(),
                                                     C.byref(desc), gather.parts, stream), "tq_decode_attn_parts")
            ffi.check(ffi.lib().tq_decode_parts_finish(self.codec.handle, C.byref(desc), b, tq_dtype(q.dtype),
                                                       gather.parts, hq // self.kv_heads, out.data_ptr(), stream),
                      "tq_decode_parts_finish")
        return out

    def decode_step_host(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, out: torch.Tensor,
                         splits: int | None = None) -> torch.Tensor:
        """One decode step with HOST tensors (pinned memory keeps the copies asynchronous): append
        ``k_new`` / ``v_new`` [B, Hkv, 1, 128], attend with ``q`` [B, Hq, 1, 128], write ``out``
        [B, Hq, 1, 128] on the host.  Queued on the current stream; synchronise it before reading
        ``out``."""
        for t in (q, k_new, v_new, out):
            if t.device.type != "cpu" or not t.is_contiguous():
                raise ValueError("decode_step_host takes contiguous host tensors")
        b, hq = int(q.shape[0]), int(q.shape[1])
        if b != self.batch or k_new.shape[1] != self.kv_heads or q.dtype != k_new.dtype or out.dtype != q.dtype:
            raise ValueError("shape or dtype mismatch")
        self.reserve(self.length + 1)
        # the split count and the scratch size only change when the length crosses a kernel step
        key = (hq, splits, (self.length + 1) >> 9, self.capacity)
        if self._step_plan is None or self._step_plan[0] != key:
            n_splits = self.suggest_splits(self.length + 1) if splits is None else int(splits)
            need = int(ffi.lib().tq_decode_step_workspace_bytes(b, hq, self.kv_heads, n_splits))
            if self._workspace is None or self._workspace.numel() < need:
                self._workspace = torch.empty(need, dtype=torch.uint8, device=self.codec.device)
            self._step_plan = (key, n_splits, self._workspace.data_ptr(), self._workspace.numel(), tq_dtype(q.dtype))
        _, n_splits, ws_ptr, ws_bytes, dt = self._step_plan
        dev = self.codec.device
        if torch.cuda.current_device() == dev.index:
            rc = ffi.lib().tq_decode_step_host(self.codec.handle, q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), dt,
                                               hq, self._desc_ref, self.length, n_splits, ws_ptr, ws_bytes,
                                               out.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
        else:
            with torch.cuda.device(dev):
                rc = ffi.lib().tq_decode_step_host(self.codec.handle, q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(),
                                                   dt, hq, self._desc_ref, self.length, n_splits, ws_ptr, ws_bytes,
                                                   out.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
        if rc:
            ffi.check(rc, "tq_decode_step_host")
        self.length += 1
        return out

    def decode_step_host_gather(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, out: torch.Tensor,
                                gather, splits: int | None = None) -> torch.Tensor:
        """``decode_step_host`` for a KV-head shard: ``q`` / ``k_new`` / ``v_new`` hold this rank's
        heads, ``out`` [B, Hq_total, 1, 128] receives the gathered output of all ranks, or, when it
        has this rank's shape [B, Hq, 1, 128], this rank's heads only (the device-side gathered
        buffer ``gather.last_view()`` is complete either way).  All four must be pinned host
        tensors; ``gather`` is a host-sequenced ``PeerGather``."""
        for t in (q, k_new, v_new, out):
            if t.device.type != "cpu" or not t.is_contiguous() or not t.is_pinned():
                raise ValueError("decode_step_host_gather takes contiguous pinned host tensors")
        b, hq = int(q.shape[0]), int(q.shape[1])
        if b != self.batch or k_new.shape[1] != self.kv_heads or q.dtype != k_new.dtype or out.dtype != q.dtype:
            raise ValueError("shape or dtype mismatch")
        local_shape = (b, hq, 1, 128)
        if tuple(out.shape) not in (tuple(gather.shape), local_shape):
            raise ValueError(f"out must have the gathered shape {gather.shape} or this rank's shape {local_shape}")
        self.reserve(self.length + 1)
        splits = self.suggest_splits(self.length + 1) if splits is None else int(splits)
        ws = self._get_workspace(hq, splits)
        desc, _ = gather.next_desc()
        # (an `out` of this rank's shape asks for this rank's heads only; every rank's gathered
        # device buffer is complete either way)
        desc.out_local_only = int(tuple(out.shape) == local_shape and tuple(gather.shape) != local_shape)
        with torch.cuda.device(self.codec.device):
            ffi.check(ffi.lib().tq_decode_step_host_gather(
                self.codec.handle, q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), tq_dtype(q.dtype), hq,
                C.byref(self._desc), self.length, splits, ws.data_ptr(), ws.numel(), C.byref(desc), out.data_ptr(),
                self._stream_ptr()), "tq_decode_step_host_gather")
        self.length += 1
        return out

    def bind_host_step(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, out: torch.Tensor):
        """``decode_step_host`` for a serving loop that reuses the same four host buffers every
        step: checks them once and returns a function that runs one step per call (append the
        buffers' current K/V, attend with the current query, write ``out``; queued on the current
        stream).  The buffers must stay alive and unmoved while the function is in use."""
        for t in (q, k_new, v_new, out):
            if t.device.type != "cpu" or not t.is_contiguous():
                raise ValueError("bind_host_step takes contiguous host tensors")
        b, hq = int(q.shape[0]), int(q.shape[1])
        if b != self.batch or k_new.shape[1] != self.kv_heads or q.dtype != k_new.dtype or out.dtype != q.dtype:
            raise ValueError("shape or dtype mismatch")
        fn = ffi.lib().tq_decode_step_host
        handle, dt, dev = self.codec.handle, tq_dtype(q.dtype), self.codec.device
        ptrs = (q.data_ptr(), k_new.data_ptr(), v_new.data_ptr())
        out_ptr, keep = out.data_ptr(), (q, k_new, v_new, out)
        state = {"bucket": None}

        def step() -> None:
            n = self.length + 1
            if n > self.capacity or state["bucket"] != (n >> 9, self.capacity):
                self.reserve(n)
                splits = self.suggest_splits(n)
                need = int(ffi.lib().tq_decode_step_workspace_bytes(b, hq, self.kv_heads, splits))
                if self._workspace is None or self._workspace.numel() < need:
                    self._workspace = torch.empty(need, dtype=torch.uint8, device=dev)
                    self._step_plan = None
                state.update(bucket=(n >> 9, self.capacity), splits=splits, ws=self._workspace,
                             ws_ptr=self._workspace.data_ptr(), ws_bytes=self._workspace.numel())
            rc = fn(handle, ptrs[0], ptrs[1], ptrs[2], dt, hq, self._desc_ref, self.length, state["splits"],
                    state["ws_ptr"], state["ws_bytes"], out_ptr, torch.cuda.current_stream(dev).cuda_stream)
            if rc:
                ffi.check(rc, "tq_decode_step_host")
            self.length = n

        step.buffers = keep
        return step

    def decode_step_dev(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, pos: torch.Tensor,
                        out: torch.Tensor | None = None, splits: int | None = None, gather=None) -> torch.Tensor:
        """One decode step whose cache length is the int32 DEVICE scalar ``pos``: append ``k_new`` /
        ``v_new`` [B, Hkv, 1, 128] at token ``pos`` and attend with ``q`` [B, Hq, 1, 128] over
        ``pos + 1`` tokens.  Nothing here depends on the value of ``pos`` on the host, so the call
        can be recorded in a CUDA graph and replayed; the caller advances ``pos`` and, when it is
        done, sets ``self.length``.  The cache must already have room (``reserve``).  With ``gather``
        (a ``PeerGather`` created with ``device_sequence=True``) this store is a KV-head shard and
        the result is the gathered output of all ranks [B, Hq_total, 1, 128]."""
        b, hq = int(q.shape[0]), int(q.shape[1])
        if b != self.batch or k_new.shape[1] != self.kv_heads or q.dtype != k_new.dtype:
            raise ValueError("shape or dtype mismatch")
        if pos.dtype != torch.int32 or pos.device != self.codec.device or pos.numel() != 1:
            raise ValueError("pos must be an int32 scalar tensor on the cache's device")
        qc, kc, vc = (t if t.is_contiguous() else t.contiguous() for t in (q, k_new, v_new))
        splits = self.suggest_splits(self.capacity) if splits is None else int(splits)
        ws = self._get_workspace(hq, splits)
        gdesc = None if gather is None else gather.static_desc()
        if out is None:
            out = torch.empty(b, hq if gather is None else gather.shape[1], 1, 128, dtype=q.dtype, device=q.device)
        with torch.cuda.device(self.codec.device):
            ffi.check(ffi.lib().tq_decode_step_dev(self.codec.handle, qc.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                                   tq_dtype(q.dtype), hq, C.byref(self._desc), pos.data_ptr(), splits,
                                                   ws.data_ptr(), ws.numel(), out.data_ptr(),
                                                   None if gdesc is None else C.byref(gdesc), self._stream_ptr()),
                      "tq_decode_step_dev")
        return out

    def dequant(self, which: str, lo: int = 0, hi: int | None = None,
                dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """Dequantise tokens [lo, hi) of ``which`` in {'keys', 'values'} -> [B, Hkv, hi-lo, 128]."""
        hi = self.length if hi is None else hi
        n = hi - lo
        out = torch.empty(self.batch, self.kv_heads, n, 128, dtype=dtype, device=self.codec.device)
        if n > 0:
            od = dense_desc(out)
            with torch.cuda.device(self.codec.device):
                ffi.check(ffi.lib().tq_dequant(self.codec.handle, C.byref(self._desc), 0 if which == "keys" else 1,
                                               lo, n, C.byref(od), self._stream_ptr()), "tq_dequant")
        return out


def key_norm_mean(k: torch.Tensor) -> torch.Tensor:
    """Mean L2 norm over all vectors of ``k`` [B, H, T, 128] as a 0-dim float64 device tensor
    (no host sync); the norm-guard statistic of ``build_packed_mse_cache``
    (packed_qmse_cache.py:918-920)."""
    if k.device.type != "cuda":
        raise ffi.TQError("TurboQuant-B200 runs on CUDA devices only; there is no CPU path")
    acc = torch.zeros((), dtype=torch.float64, device=k.device)
    if k.stride(-1) != 1:
        k = k.contiguous()
    kd = dense_desc(k)
    b, h, t = int(k.shape[0]), int(k.shape[1]), int(k.shape[2])
    with torch.cuda.device(k.device):
        ffi.check(ffi.lib().tq_key_norm_sum(C.byref(kd), b, h, t, acc.data_ptr(),
                                            C.c_void_p(torch.cuda.current_stream(k.device).cuda_stream)),
                  "tq_key_norm_sum")
    return acc / (b * h * t)
