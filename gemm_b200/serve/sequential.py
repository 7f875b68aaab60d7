"""Serving adapter for the model families that run as tensor-op forward passes (``models.gemma4``, ``models.m3``, ``models.glm5``):
the interface ``serve.server`` and the ``generate`` command expect from ``serve.llm.LLM``, over a model object with
``reset(batch, max_pos)`` and ``forward(ids [1, T]) -> logits [1, V]``.

Requests are served one at a time in arrival order: the prompt is prefilled in chunks, then one token per step, greedy or sampled
on the host.  This is the reference server's own discipline (one model, one request at a time: server/server_llm.c:422-632); the
Qwen families go through the continuous-batching engine of ``serve.llm`` instead.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

import torch

from .engine import SamplingParams


@dataclass
class _Req:
    prompt: List[int]
    sp: SamplingParams
    out: List[int] = field(default_factory=list)
    done: bool = False
    error: str = ""
    logits: Optional[torch.Tensor] = None


class _Counts:
    def __init__(self):
        self.num_waiting = 0
        self.num_running = 0


class SequentialLLM:
    def __init__(self, model, tokenizer=None, max_seq_len: int = 4096, prefill_chunk: int = 512):
        self.model, self.tokenizer = model, tokenizer
        self.max_seq_len, self.prefill_chunk = max_seq_len, prefill_chunk
        self._reqs: Dict[int, _Req] = {}
        self._queue: Deque[int] = deque()
        self._active: Optional[int] = None
        self._next_id = 0
        self.produced_all: Dict[int, List[int]] = {}
        self.sched = _Counts()
        self.steps = 0

    # ------------------------------------------------------------------------------------------ requests
    def add_request(self, prompt_ids: Sequence[int], sp: Optional[SamplingParams] = None) -> int:
        sp = sp or SamplingParams()
        if len(prompt_ids) == 0 or len(prompt_ids) + sp.max_new_tokens + 1 > self.max_seq_len:
            raise ValueError(f"the request needs {len(prompt_ids) + sp.max_new_tokens + 1} positions, the cache holds {self.max_seq_len}")
        rid = self._next_id
        self._next_id += 1
        self._reqs[rid] = _Req(list(prompt_ids), sp)
        self._queue.append(rid)
        self._count()
        return rid

    def _count(self) -> None:
        self.sched.num_waiting = len(self._queue)
        self.sched.num_running = 0 if self._active is None else 1

    def has_work(self) -> bool:
        return self._active is not None or len(self._queue) > 0

    def _pick(self, logits: torch.Tensor, sp: SamplingParams, step: int) -> int:
        row = logits[0].float()
        if sp.temperature <= 0:
            return int(row.argmax())
        row = row / sp.temperature
        if sp.top_k > 0:
            kth = torch.topk(row, min(sp.top_k, row.numel())).values[-1]
            row = row.masked_fill(row < kth, float("-inf"))
        p = torch.softmax(row, dim=-1)
        if sp.top_p < 1.0:
            sp_, idx = torch.sort(p, descending=True)
            cut = (torch.cumsum(sp_, 0) - sp_) > sp.top_p
            sp_[cut] = 0.0
            p = torch.zeros_like(p).scatter_(0, idx, sp_)
            p = p / p.sum()
        g = torch.Generator(device="cpu").manual_seed(sp.seed * 1000003 + step)
        return int(torch.multinomial(p.cpu(), 1, generator=g))

    @torch.no_grad()
    def step(self) -> Dict[int, int]:
        """Prefill of the next waiting request (it yields its first token), or one more token of the active one."""
        self.produced_all = {}
        if self._active is None:
            if not self._queue:
                return {}
            rid = self._queue.popleft()
            r = self._reqs[rid]
            self._active = rid
            self.model.reset(1, len(r.prompt) + r.sp.max_new_tokens + 1)
            ids = torch.tensor([r.prompt])
            for i in range(0, ids.shape[1], self.prefill_chunk):
                r.logits = self.model.forward(ids[:, i: i + self.prefill_chunk])
        else:
            rid = self._active
            r = self._reqs[rid]
            r.logits = self.model.forward(torch.tensor([[r.out[-1]]]))
        tok = self._pick(r.logits, r.sp, len(r.out))
        r.out.append(tok)
        self.produced_all[rid] = [tok]
        self.steps += 1
        if tok in r.sp.stop_token_ids or len(r.out) >= r.sp.max_new_tokens:
            r.done = True
            self._active = None
        self._count()
        return {rid: tok}

    # ------------------------------------------------------------------------------------------ whole prompts
    def generate(self, prompts: Sequence[Sequence[int]], sp: Optional[SamplingParams] = None) -> List[List[int]]:
        rids = [self.add_request(p, sp) for p in prompts]
        while self.has_work():
            self.step()
        return [self._reqs.pop(r).out for r in rids]

    def decode(self, ids: Sequence[int]) -> str:
        return self.tokenizer.decode(ids) if self.tokenizer is not None else " ".join(str(i) for i in ids)
