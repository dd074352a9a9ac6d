"""KV-head sharding of the packed cache across the GPUs of one box.

Heads are independent through packing, append and decode attention, so rank ``r`` of
``W`` owns KV heads ``[r*Hkv/W, (r+1)*Hkv/W)`` and the query heads that attend to them.
The only exchange per layer and decode step is one all-gather of the per-head attention
outputs ``[B, Hq/W, D]`` (model dtype) before the output projection.  The reference has no
multi-GPU path; this module is the whole of it.  Works with any ``torch.distributed``
backend (NCCL on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

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
        if kv_heads % self.world_size:
            raise ValueError(
                f"{kv_heads} KV heads do not divide over {self.world_size} ranks; "
                "use a world size that divides the KV-head count")
        if q_heads % kv_heads:
            raise ValueError(f"{q_heads} query heads are not a multiple of {kv_heads} KV heads")

    def kv_range(self, kv_heads: int) -> tuple[int, int]:
        per = kv_heads // self.world_size
        return self.rank * per, (self.rank + 1) * per

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
