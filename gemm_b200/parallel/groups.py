"""Process-group layout for tensor / pipeline / data parallelism.

Rank decomposition is the reference's (common/parallel.h:117-123): ``tp_rank = r % tp``, ``pp_rank = (r // tp) % pp``,
``dp_rank = r // (tp * pp)``; one communicator per dimension (colours as in parallel.h:231-242).  Groups are
``torch.distributed`` process groups (NCCL on GPUs, gloo on CPU); the NVLink fabric is built on top of the TP / EP group.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch.distributed as dist


@dataclass
class ParallelLayout:
    tp: int = 1
    pp: int = 1
    dp: int = 1

    @property
    def world(self) -> int:
        return self.tp * self.pp * self.dp

    def coords(self, rank: int) -> Tuple[int, int, int]:
        """(tp_rank, pp_rank, dp_rank) of a global rank."""
        return rank % self.tp, (rank // self.tp) % self.pp, rank // (self.tp * self.pp)

    def rank_of(self, tp_rank: int, pp_rank: int, dp_rank: int) -> int:
        return tp_rank + self.tp * (pp_rank + self.pp * dp_rank)

    def tp_group_ranks(self, rank: int) -> List[int]:
        _, p, d = self.coords(rank)
        return [self.rank_of(t, p, d) for t in range(self.tp)]

    def pp_group_ranks(self, rank: int) -> List[int]:
        t, _, d = self.coords(rank)
        return [self.rank_of(t, p, d) for p in range(self.pp)]

    def dp_group_ranks(self, rank: int) -> List[int]:
        t, p, _ = self.coords(rank)
        return [self.rank_of(t, p, d) for d in range(self.dp)]


def pp_layer_range(n_layers: int, pp: int, pp_rank: int) -> Tuple[int, int]:
    """Contiguous layer range of a pipeline stage, remainder to the low ranks (common/parallel.h:125-133)."""
    q, r = divmod(n_layers, pp)
    lo = pp_rank * q + min(pp_rank, r)
    return lo, lo + q + (1 if pp_rank < r else 0)


@dataclass
class ParallelGroups:
    layout: ParallelLayout
    rank: int
    tp_rank: int
    pp_rank: int
    dp_rank: int
    tp_group: Optional[object]
    pp_group: Optional[object]
    dp_group: Optional[object]


def init_parallel(layout: ParallelLayout) -> ParallelGroups:
    """Create the three families of process groups.  Every rank must call this (``new_group`` is collective)."""
    world, rank = dist.get_world_size(), dist.get_rank()
    if world != layout.world:
        raise ValueError(f"world size {world} != tp*pp*dp = {layout.world}")
    mine = {"tp": None, "pp": None, "dp": None}
    seen = {"tp": set(), "pp": set(), "dp": set()}
    for r in range(world):
        for kind, ranks in (("tp", layout.tp_group_ranks(r)), ("pp", layout.pp_group_ranks(r)), ("dp", layout.dp_group_ranks(r))):
            key = tuple(ranks)
            if key in seen[kind]:
                continue
            seen[kind].add(key)
            g = dist.new_group(ranks)
            if rank in ranks:
                mine[kind] = g
    t, p, d = layout.coords(rank)
    return ParallelGroups(layout, rank, t, p, d, mine["tp"], mine["pp"], mine["dp"])
