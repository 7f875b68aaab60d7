"""Data parallelism: independent replicas of the model serving disjoint requests.

The reference's DP mode runs every replica on the same prompt and compares the last token against rank 0's
(cpu/llm/test_transformer_parallel.c:216-281, "WARNING: output diverged!"); ``check_agreement`` is that check,
``shard`` is what a real deployment does instead — split the requests."""
from __future__ import annotations

from typing import List, Sequence, TypeVar

import torch
import torch.distributed as dist

T = TypeVar("T")


class DataParallel:
    def __init__(self, group):
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def shard(self, items: Sequence[T]) -> List[T]:
        """Round-robin share of a request list for this replica."""
        return [x for i, x in enumerate(items) if i % self.size == self.rank]

    def check_agreement(self, tokens: torch.Tensor) -> bool:
        """True when this replica produced the same tokens as replica 0 (collective)."""
        ref = tokens.clone()
        dist.broadcast(ref, src=dist.get_process_group_ranks(self.group)[0], group=self.group)
        same = torch.tensor([1 if torch.equal(ref, tokens) else 0], dtype=torch.int32, device=tokens.device)
        dist.all_reduce(same, op=dist.ReduceOp.MIN, group=self.group)
        return bool(same.item())

    def gather_outputs(self, local: List[List[int]], total: int) -> List[List[int]]:
        """Collect every replica's outputs back into request order (collective, via object gather)."""
        parts: List = [None] * self.size
        dist.all_gather_object(parts, local, group=self.group)
        out: List[List[int]] = [[] for _ in range(total)]
        for r, lst in enumerate(parts):
            for j, o in enumerate(lst):
                out[r + j * self.size] = o
        return out
