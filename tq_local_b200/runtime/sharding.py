"""KV-head sharding of the packed cache across the GPUs of one box.

Heads are independent through packing, append and decode attention, so rank ``r`` of
``W`` owns KV heads ``[r*Hkv/W, (r+1)*Hkv/W)`` and the query heads that attend to them.
The only exchange per layer and decode step is one all-gather of the per-head attention
outputs ``[B, Hq/W, D]`` (model dtype) before the output projection.  The reference has no
multi-GPU path; this module is the whole of it.  Works with any ``torch.distributed``
backend (NCCL on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class HeadShard:
    """Which slice of the KV (and query) heads this rank serves."""

    world_size: int = 1
    rank: int = 0
    group: "dist.ProcessGroup | None" = None

    @classmethod
    def from_process_group(cls, group: "dist.ProcessGroup | None" = None) -> "HeadShard":
        if not (dist.is_available() and dist.is_initialized()):
            return cls()
        return cls(dist.get_world_size(group), dist.get_rank(group), group)

    def check(self, kv_heads: int, q_heads: int) -> None:
        if self.world_size < 1 or not 0 <= self.rank < self.world_size:
            raise ValueError(f"bad shard: rank {self.rank} of {self.world_size}")
        if kv_heads % self.world_size and self.world_size % kv_heads:
            raise ValueError(
                f"{kv_heads} KV heads and {self.world_size} ranks: one count must divide the other "
                "(heads are sharded over the ranks, or several ranks share the tokens of each head)")
        if q_heads % kv_heads:
            raise ValueError(f"{q_heads} query heads are not a multiple of {kv_heads} KV heads")

    def seq_parts(self, kv_heads: int) -> int:
        """How many ranks share the tokens of one KV head: 1 while there are at least as many KV
        heads as ranks, else ``world_size // kv_heads`` (Qwen2.5-7B's 4 KV heads on 8 GPUs: 2)."""
        return self.world_size // kv_heads if kv_heads < self.world_size else 1

    def kv_range(self, kv_heads: int) -> tuple[int, int]:
        parts = self.seq_parts(kv_heads)
        if parts > 1:
            head = self.rank // parts
            return head, head + 1
        per = kv_heads // self.world_size
        return self.rank * per, (self.rank + 1) * per

    def local_tokens(self, t: torch.Tensor, kv_heads: int, seen: int) -> torch.Tensor:
        """The tokens of ``t`` [B, H, T, D] this rank stores when ``seq_parts`` ranks share a head:
        a prompt (T > 1) is cut into ``parts`` contiguous pieces, single decoded tokens go to the
        parts in turn (``seen`` = tokens the cache has been handed so far).  Attention over a set
        of tokens does not depend on their order, so any disjoint cover works."""
        parts = self.seq_parts(kv_heads)
        if parts == 1:
            return t
        part, n = self.rank % parts, int(t.shape[2])
        if n == 1:
            return t if seen % parts == part else t[:, :, :0]
        piece = (n + parts - 1) // parts
        return t[:, :, part * piece:(part + 1) * piece]

    def q_range(self, kv_heads: int, q_heads: int) -> tuple[int, int]:
        lo, hi = self.kv_range(kv_heads)
        groups = q_heads // kv_heads
        return lo * groups, hi * groups

    def local_kv(self, t: torch.Tensor) -> torch.Tensor:
        """Slice ``[B, Hkv, T, D]`` down to this rank's KV heads (a view)."""
        if self.world_size == 1:
            return t
        lo, hi = self.kv_range(t.shape[1])
        return t[:, lo:hi]

    def local_q(self, q: torch.Tensor, kv_heads: int) -> torch.Tensor:
        """Slice ``[B, Hq, Sq, D]`` down to the query heads of this rank's KV heads."""
        if self.world_size == 1:
            return q
        lo, hi = self.q_range(kv_heads, q.shape[1])
        return q[:, lo:hi]

    def gather_heads(self, out_local: torch.Tensor) -> torch.Tensor:
        """All-gather per-head outputs ``[B, Hq/W, Sq, D]`` into ``[B, Hq, Sq, D]`` (head order
        = rank order, which is the global head order because shards are contiguous)."""
        if self.world_size == 1:
            return out_local
        out_local = out_local.contiguous()
        b, hl = out_local.shape[0], out_local.shape[1]
        # rank-major concatenation along dim 0 (the layout every backend agrees on)
        parts = torch.empty((self.world_size * b, *out_local.shape[1:]), dtype=out_local.dtype,
                            device=out_local.device)
        dist.all_gather_into_tensor(parts, out_local, group=self.group)
        parts = parts.view(self.world_size, b, *out_local.shape[1:])
        return parts.permute(1, 0, 2, 3, 4).reshape(b, self.world_size * hl, *out_local.shape[2:])


class _DeviceBytes:
    """Lets torch alias device memory that the library allocated."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerGather:
    """Buffers for the fused gather of ``PackedStore.decode_attn_gather``: every rank owns two
    gathered-output buffers ``[batch, q_heads_total, 1, 128]`` (steps alternate between them) and
    a flag block, all in memory that the other ranks of the box map through CUDA IPC, so a rank's
    combine kernel stores its rows straight into every rank's buffer over NVLink and no
    collective library call is on the path.  Set-up exchanges the 64-byte handles with
    ``all_gather_object``; ``world_size`` 1 works too (nothing is mapped).

    ``device_sequence=True`` keeps the step number in device memory (advanced by the kernels), for
    launch sequences that are recorded once and replayed (``PackedStore.decode_step_dev``); such a
    gather must not be used through ``next_desc``."""

    def __init__(self, shard: HeadShard, batch: int, q_heads_total: int, dtype: torch.dtype, device: torch.device,
                 device_sequence: bool = False, parts: int = 0):
        from tq_local_b200.runtime import ffi

        if shard.world_size > ffi.TQ_MAX_PEERS:
            raise ValueError(f"at most {ffi.TQ_MAX_PEERS} ranks")
        self.shard, self.device, self.dtype = shard, torch.device(device), dtype
        self.shape = (int(batch), int(q_heads_total), 1, 128)
        # parts > 0: the buffers exchange unfinished fp32 partials of a sequence split (every rank
        # finishes all rows itself, see PackedStore.decode_attn_parts) instead of finished outputs
        self.parts = int(parts)
        if self.parts:
            if device_sequence or shard.world_size % self.parts:
                raise ValueError("a sequence split needs host-numbered steps and a world size that is a multiple of parts")
            self.out_bytes = int(ffi.lib().tq_parts_exchange_bytes(batch, q_heads_total, self.parts))
        else:
            self.out_bytes = (batch * q_heads_total * 128 * torch.empty((), dtype=dtype).element_size() + 255) // 256 * 256
        self.total = 2 * self.out_bytes + 256
        self.seq = 0
        self.seq_dev = torch.zeros(1, dtype=torch.int32, device=self.device) if device_sequence else None
        self._lib = ffi.lib()
        self._views = None
        # Set-up is collective: every rank takes part in every exchange below even when a step failed
        # locally, and all ranks then fail together, so nobody is left waiting in a collective.
        base, handle, problem = C.c_void_p(), (C.c_uint8 * 64)(), None
        with torch.cuda.device(self.device):
            rc = self._lib.tq_peer_buffer_create(self.total, C.byref(base), handle)
        if rc:
            problem = f"tq_peer_buffer_create: status {rc}"
        self.bases = [0] * shard.world_size
        self.bases[shard.rank] = int(base.value or 0)
        if shard.world_size > 1:
            handles = [None] * shard.world_size
            dist.all_gather_object(handles, None if problem else bytes(handle), group=shard.group)
            if problem is None and any(h is None for h in handles):
                problem = "a peer could not create its buffer"
            if problem is None:
                for r, h in enumerate(handles):
                    if r == shard.rank:
                        continue
                    ptr = C.c_void_p()
                    with torch.cuda.device(self.device):
                        rc = self._lib.tq_peer_buffer_open((C.c_uint8 * 64).from_buffer_copy(h), C.byref(ptr))
                    if rc:
                        problem = f"tq_peer_buffer_open(rank {r}): status {rc}"
                        break
                    self.bases[r] = int(ptr.value)
            states = [None] * shard.world_size  # also the barrier: nobody writes before everybody has mapped
            dist.all_gather_object(states, problem, group=shard.group)
            problem = problem or next((f"rank {r}: {p}" for r, p in enumerate(states) if p), None)
        if problem:
            self._release()
            raise ffi.TQError(f"peer buffers unavailable: {problem}")
        raw = torch.as_tensor(_DeviceBytes(self.bases[shard.rank], 2 * self.out_bytes), device=self.device)
        self._views = None if self.parts else [
            raw[i * self.out_bytes:i * self.out_bytes + self._numel_bytes()].view(dtype).view(self.shape) for i in range(2)]

    def _numel_bytes(self) -> int:
        b, h, _, d = self.shape
        return b * h * d * torch.empty((), dtype=self.dtype).element_size()

    def _desc(self):
        from tq_local_b200.runtime import ffi

        d = ffi.GatherDesc()
        d.world, d.rank, d.q_heads_total, d.seq = self.shard.world_size, self.shard.rank, self.shape[1], 0
        d.out_stride = self.out_bytes
        for r, base in enumerate(self.bases):
            d.out[r] = base
            d.flags[r] = base + 2 * self.out_bytes
        d.counter = self.bases[self.shard.rank] + 2 * self.out_bytes + 64
        d.seq_dev = self.seq_dev.data_ptr() if self.seq_dev is not None else None
        return d

    def next_desc(self):
        """Descriptor of the next step (advances the host-side sequence number) and the view of this
        rank's gathered output for it."""
        if self.seq_dev is not None:
            raise RuntimeError("this PeerGather takes its step numbers from the device")
        self.seq += 1
        d = self._desc()
        d.seq = self.seq
        return d, (None if self._views is None else self._views[self.seq & 1])

    def last_view(self) -> torch.Tensor:
        """This rank's gathered output [batch, q_heads_total, 1, 128] of the latest host-numbered step."""
        return self._views[self.seq & 1]

    _shared: dict = {}

    @classmethod
    def shared(cls, shard: HeadShard, batch: int, q_heads_total: int, dtype: torch.dtype, device: torch.device,
               parts: int) -> "PeerGather":
        """One partial-exchange ``PeerGather`` per (group, shape) for all layers of a model whose
        KV heads are fewer than its ranks.  Created on first use, collectively (every rank reaches
        its first sequence-split attention call at the same point of the model)."""
        key = (id(shard.group), shard.rank, int(batch), int(q_heads_total), dtype, str(device), int(parts))
        if key not in cls._shared:
            cls._shared[key] = cls(shard, batch, q_heads_total, dtype, device, parts=parts)
        return cls._shared[key]

    @classmethod
    def close_shared(cls) -> None:
        """Collective: release every shared partial-exchange buffer."""
        for gather in list(cls._shared.values()):
            gather.close()
        cls._shared.clear()

    def static_desc(self):
        """Descriptor for steps numbered on the device (the same for every step)."""
        if self.seq_dev is None:
            raise RuntimeError("create the PeerGather with device_sequence=True")
        return self._desc()

    def _release(self) -> None:
        with torch.cuda.device(self.device):
            for r, base in enumerate(self.bases):
                if r != self.shard.rank and base:
                    self._lib.tq_peer_buffer_close(C.c_void_p(base))
            self._views = None
            if self.bases[self.shard.rank]:
                self._lib.tq_peer_buffer_destroy(C.c_void_p(self.bases[self.shard.rank]))
        self._lib = None

    def close(self) -> None:
        """Collective: unmap the peers' buffers and free this rank's."""
        if self._lib is None:
            return
        torch.cuda.synchronize(self.device)
        if self.shard.world_size > 1:
            dist.barrier(group=self.shard.group)  # peers are done writing into this rank's memory
        self._release()
