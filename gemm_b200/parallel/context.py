"""Context parallelism for decode: the KV positions of every sequence are sharded block-cyclically over the ranks.

Rank r stores the K/V of the position blocks b with ``b % world == r`` (block = 128 positions) in its own paged cache; every
rank holds the same queries, runs the flash kernel over its local shard only and gets partials (O normalised by its own
sum, base-2 log-sum-exp); the partials are exchanged with peer stores into every rank's heap and merged with the rule of
the split-KV decode, so all ranks end with identical outputs.  This is the reference's scheme for its long-context decode
(a64fx/m3/m3_ep_runner.c:121-140, common/glm5.h:285-298: all-reduce-MAX of the per-head maxima followed by an
all-reduce-SUM of the rescaled [sumexp | out]); here the two all-reduces are one all-gather of ``Hq * (D + 1)`` floats per
token and rank plus the merge kernel.  As in the reference, tensor-parallel attention is off under context parallelism.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import attention as att
from .fabric import Fabric


class ContextParallel:
    def __init__(self, group, device: torch.device, block: int = 128, fused: bool = True, max_tokens: int = 256, hq: int = 32,
                 head_dim: int = 128):
        self.group, self.device, self.block = group, device, block
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.fused = fused and device.type == "cuda"
        self.max_tokens, self.hq, self.d = max_tokens, hq, head_dim
        self.fab: Optional[Fabric] = None
        if self.fused:
            per = max_tokens * hq * (head_dim + 1) * 4
            self.fab = Fabric(group, device, self.world * per + (1 << 20))
            self.ag = self.fab.make_exchange(per, chunks=8)

    # ------------------------------------------------------------------------------------------ layout
    def owner(self, pos: int) -> int:
        return (pos // self.block) % self.world

    def local_index(self, pos: int) -> int:
        """Index of global position ``pos`` inside its owner's shard."""
        return (pos // (self.block * self.world)) * self.block + pos % self.block

    def local_len(self, kv_len: int, rank: Optional[int] = None) -> int:
        """How many of the positions ``[0, kv_len)`` the rank owns."""
        r = self.rank if rank is None else rank
        full, rem = divmod(kv_len, self.block * self.world)
        return full * self.block + min(max(rem - r * self.block, 0), self.block)

    def shard_positions(self, kv_len: int, rank: Optional[int] = None) -> Sequence[int]:
        r = self.rank if rank is None else rank
        return [p for p in range(kv_len) if self.owner(p) == r]

    # ------------------------------------------------------------------------------------------ attention
    def attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: torch.Tensor, local_kv_len: torch.Tensor,
                  block_table: torch.Tensor, page_size: int, work: torch.Tensor) -> torch.Tensor:
        """``q`` bf16 [T, Hq, D] (the same on every rank, pre-scaled as the flash kernel expects; one decode token per sequence);
        caches, ``local_kv_len`` and ``block_table`` describe THIS rank's shard.  Returns bf16 [T, Hq, D], identical on all ranks."""
        t, hq, d = q.shape
        po, pl = att.attention_partial(q, k_cache, v_cache, cu_q, local_kv_len, block_table, page_size, work, causal=False)
        mine = torch.cat([po[0].reshape(t, hq * d), pl[0].reshape(t, hq)], dim=1).contiguous()      # [T, Hq * (D + 1)] f32
        if self.fused:
            assert t <= self.max_tokens and hq == self.hq and d == self.d
            buf = torch.zeros(self.max_tokens, hq * (d + 1), dtype=torch.float32, device=q.device)
            buf[:t] = mine
            allp = self.ag.all_gather(buf).view(torch.float32).view(self.world, self.max_tokens, hq * (d + 1))[:, :t]
        else:
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine, group=self.group)
            allp = torch.stack(parts)
        part_o = allp[:, :, : hq * d].reshape(self.world, t * hq, d).contiguous()
        part_lse = allp[:, :, hq * d:].reshape(self.world, t * hq).contiguous()
        out, _ = att.combine_partials(part_o, part_lse)
        return out.reshape(t, hq, d)

    def close(self) -> None:
        if self.fab is not None:
            self.fab.close()
