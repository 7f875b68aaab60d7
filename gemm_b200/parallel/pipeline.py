"""Pipeline parallelism: contiguous layer ranges per stage, hidden states handed from stage to stage.

Reference behaviour (common/parallel.h:125-133,254-270; cpu/llm/test_transformer_parallel.c:110-213): layers are split
evenly with the remainder to the low ranks; per step a stage receives the hidden state, runs its layers
(``transformer_forward_partial``), sends it on; the last stage computes the logits and the next token, which is
broadcast to every stage.  Here a step carries a whole packed batch ``[T, hidden]`` (bf16) instead of one token.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

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

    @torch.no_grad()
    def step_many(self, fbs: Sequence[ForwardBatch]) -> List[torch.Tensor]:
        """One forward pass over several micro-batches (disjoint groups of sequences) with the stages overlapped: the receives of
        all micro-batches are posted up front, every hidden state is sent on without waiting for it to arrive, so stage ``r + 1``
        works on micro-batch ``i`` while stage ``r`` runs ``i + 1`` (with ``m`` micro-batches over ``p`` stages the idle share of a
        stage drops from ``(p - 1) / p`` to ``(p - 1) / (m + p - 1)``).  The last stage broadcasts all tokens once.  Returns the
        greedy next tokens per micro-batch, on every stage; equal to ``step`` called per micro-batch."""
        hidden = self.model.cfg.hidden
        dev = fbs[0].positions.device
        prev = None if self.first else self.ranks[self.rank - 1]
        nxt = None if self.last else self.ranks[self.rank + 1]
        bufs, recvs = [], []
        if prev is not None:
            for i, fb in enumerate(fbs):
                buf = torch.empty(fb.n_tokens, hidden, dtype=torch.bfloat16, device=dev)
                bufs.append(buf)
                recvs.append(dist.irecv(buf, src=prev, group=self.group, tag=i))
        sends, toks = [], []
        for i, fb in enumerate(fbs):
            x = None
            if prev is not None:
                recvs[i].wait()
                x = bufs[i]
            x = self.model.forward_hidden(fb, x=x)
            if nxt is not None:
                out = self.model.final_hidden(x).contiguous()
                sends.append((dist.isend(out, dst=nxt, group=self.group, tag=i), out))      # the tensor stays alive until the send is done
            else:
                toks.append(sampling.argmax(self.model.head(x, fb), idx_offset=self.model.w.vocab_start).to(torch.int32))
        for req, _ in sends:
            req.wait()
        sizes = [fb.logit_rows.numel() for fb in fbs]
        tok = torch.cat(toks) if self.last else torch.empty(sum(sizes), dtype=torch.int32, device=dev)
        dist.broadcast(tok, src=self.ranks[-1], group=self.group)
        return list(torch.split(tok, sizes))
