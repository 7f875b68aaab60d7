"""Pipeline parallelism: contiguous layer ranges per stage, hidden states handed from stage to stage.

Reference behaviour (common/parallel.h:125-133,254-270; cpu/llm/test_transformer_parallel.c:110-213): layers are split
evenly with the remainder to the low ranks; per step a stage receives the hidden state, runs its layers
(``transformer_forward_partial``), sends it on; the last stage computes the logits and the next token, which is
broadcast to every stage.  Here a step carries a whole packed batch ``[T, hidden]`` (bf16) instead of one token.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..models.transformer import ForwardBatch, Transformer
from ..ops import sampling
from .groups import pp_layer_range


class PipelineStage:
    def __init__(self, model: Transformer, group, n_layers_total: int):
        self.model, self.group = model, group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.ranks = dist.get_process_group_ranks(group)
        self.first, self.last = self.rank == 0, self.rank == self.size - 1
        self.layer_range = pp_layer_range(n_layers_total, self.size, self.rank)

    @torch.no_grad()
    def step(self, fb: ForwardBatch) -> torch.Tensor:
        """Run this stage's share of one forward pass; returns the greedy next tokens (int32, on every stage)."""
        hidden = self.model.cfg.hidden
        dev = fb.positions.device
        x: Optional[torch.Tensor] = None
        if not self.first:
            x = torch.empty(fb.n_tokens, hidden, dtype=torch.bfloat16, device=dev)
            dist.recv(x, src=self.ranks[self.rank - 1], group=self.group)
        x = self.model.forward_hidden(fb, x=x)
        if not self.last:
            dist.send(self.model.final_hidden(x).contiguous(), dst=self.ranks[self.rank + 1], group=self.group)
            tok = torch.empty(fb.logit_rows.numel(), dtype=torch.int32, device=dev)
        else:
            logits = self.model.head(x, fb)
            tok = sampling.argmax(logits, idx_offset=self.model.w.vocab_start).to(torch.int32)
        dist.broadcast(tok, src=self.ranks[-1], group=self.group)
        return tok
