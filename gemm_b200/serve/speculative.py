"""Speculative greedy decoding with batched verification.

A drafter proposes up to ``gamma`` tokens per sequence; ONE forward over ``1 + len(draft)`` query positions per sequence
(the chunked-prefill path of the engine: paged KV, causal inside the chunk) returns the target model's arg-max token after
every position, and the longest prefix of the draft that the target agrees with is kept, plus the target's own next token.
Every verify step therefore yields between 1 and ``gamma + 1`` tokens per sequence and the output equals plain greedy
decoding token for token.  Rejected positions need no cache roll-back: their K/V sit beyond the sequence's committed
length, attention never reads past ``kv_len``, and the next step overwrites them (slots are a function of the position).
That holds for attention layers only: recurrent (Delta-Net) state cannot be rewound, so hybrid models are refused.

Three drafters are provided: ``NgramDrafter`` (prompt lookup: continue the most recent earlier occurrence of the current
suffix; needs no second model), ``ModelDrafter`` (a smaller model of the same vocabulary with its own paged cache, batched
over the live sequences) and ``CallableDrafter`` (wraps any function).

Counterpart in the reference: the multi-token-prediction draft of depth 1 with batched verification of the DeepSeek engine
(a64fx/ds4f/DS4P_DECODE_PERF_FINDINGS.md:43-61), generalised to any draft source and depth.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from ..models.transformer import ForwardBatch, KvCache, Transformer
from .scheduler import KvBlockManager


class NgramDrafter:
    """Prompt-lookup drafts: find the latest earlier occurrence of the last ``n`` tokens (``n`` from ``max_ngram`` down to
    ``min_ngram``) and propose the ``gamma`` tokens that followed it."""

    def __init__(self, gamma: int = 4, max_ngram: int = 3, min_ngram: int = 1):
        self.gamma, self.max_ngram, self.min_ngram = gamma, max_ngram, min_ngram

    def propose(self, tokens: Sequence[int]) -> List[int]:
        n_tok = len(tokens)
        for n in range(min(self.max_ngram, n_tok - 1), self.min_ngram - 1, -1):
            suffix = list(tokens[n_tok - n:])
            for start in range(n_tok - n - 1, -1, -1):
                if list(tokens[start:start + n]) == suffix:
                    cont = list(tokens[start + n:start + n + self.gamma])
                    if cont:
                        return cont
        return []


class CallableDrafter:
    def __init__(self, fn: Callable[[Sequence[int]], Sequence[int]], gamma: int = 4):
        self.fn, self.gamma = fn, gamma

    def propose(self, tokens: Sequence[int]) -> List[int]:
        return list(self.fn(tokens))[: self.gamma]


class ModelDrafter:
    """Drafts from a (smaller) model of the same vocabulary, decoded greedily with its own paged cache, for all live sequences
    at once: one catch-up step over the tokens the draft cache does not hold yet (the tokens the target accepted or produced
    since the last call), then ``gamma - 1`` single-token steps.  The draft cache follows the target's decisions the same way
    the target's does: positions beyond the common prefix of what it was fed and what was kept are overwritten."""

    def __init__(self, model: Transformer, kv: KvCache, page_size: int, num_pages: int, gamma: int = 4):
        if model.cfg.is_hybrid:
            raise ValueError("a draft model with recurrent layers cannot drop rejected positions")
        self.model, self.kv, self.page, self.gamma = model, kv, page_size, gamma
        self.blocks = KvBlockManager(num_pages, page_size)
        self.device = model.w.embed.device
        self._seq = {}                # key -> sequence handle of the block manager
        self._held = {}               # key -> tokens whose K/V the draft cache holds, in position order
        self.steps = 0

    def _step(self, keys, q_lens, ctx, ids) -> List[int]:
        pages = [self.blocks.pages(self._seq[k]) for k in keys]
        bt = torch.zeros(len(keys), max(len(p) for p in pages), dtype=torch.int32)
        for i, p in enumerate(pages):
            bt[i, : len(p)] = torch.tensor(p, dtype=torch.int32)
        m = self.model
        fb = ForwardBatch.build(q_lens, ctx, ids, bt, self.page, m.hq_local, m.hkv_local, self.device)
        self.steps += 1
        return [int(t) for t in m.forward_greedy(fb).cpu()]

    @torch.no_grad()
    def propose_batch(self, keys: Sequence[int], tokens: Sequence[Sequence[int]], limits: Sequence[int]) -> List[List[int]]:
        drafts: List[List[int]] = [[] for _ in keys]
        act = [i for i in range(len(keys)) if limits[i] > 0]
        if not act:
            return drafts
        q_lens, ctx, ids = [], [], []
        for i in act:
            k, t = keys[i], list(tokens[i])
            if k not in self._seq:
                self._seq[k], self._held[k] = self.blocks.new_sequence(), []
            self.blocks.reserve(self._seq[k], len(t) + self.gamma + 1)
            held = self._held[k]
            c = 0
            while c < len(held) and c < len(t) - 1 and held[c] == t[c]:
                c += 1
            q_lens.append(len(t) - c)
            ctx.append(c)
            ids.extend(t[c:])
            self._held[k] = t
        nxt = self._step([keys[i] for i in act], q_lens, ctx, ids)
        for i, d in zip(act, nxt):
            drafts[i].append(d)
        for j in range(1, self.gamma):
            act = [i for i in act if limits[i] > j]
            if not act:
                break
            ctx = [len(tokens[i]) + j - 1 for i in act]
            ids = [drafts[i][-1] for i in act]
            for i in act:
                self._held[keys[i]] = self._held[keys[i]] + [drafts[i][-1]]
            nxt = self._step([keys[i] for i in act], [1] * len(act), ctx, ids)
            for i, d in zip(act, nxt):
                drafts[i].append(d)
        return drafts

    def finish(self, keys: Sequence[int]) -> None:
        for k in keys:
            if k in self._seq:
                self.blocks.release(self._seq.pop(k))
                self._held.pop(k, None)


def accept_greedy(draft: Sequence[int], target: Sequence[int]) -> Tuple[int, int]:
    """``target[i]`` is the model's arg-max after the inputs ``[last, draft[0], ..., draft[i-1]]``.  Returns (number of
    draft tokens kept, the token that follows them)."""
    assert len(target) == len(draft) + 1
    n = 0
    while n < len(draft) and int(draft[n]) == int(target[n]):
        n += 1
    return n, int(target[n])


@dataclass
class SpecStats:
    verify_steps: int = 0
    drafted: int = 0
    accepted: int = 0
    produced: int = 0
    per_step: List[int] = field(default_factory=list)

    @property
    def acceptance(self) -> float:
        return self.accepted / self.drafted if self.drafted else 0.0

    @property
    def tokens_per_step(self) -> float:
        return self.produced / self.verify_steps if self.verify_steps else 0.0


class SpeculativeDecoder:
    """Greedy generation for a fixed group of prompts over a ``Transformer`` and its paged cache (CPU or GPU tensors)."""

    def __init__(self, model: Transformer, kv: KvCache, page_size: int, num_pages: int, drafter=None):
        if model.cfg.is_hybrid:
            raise ValueError("speculative decoding needs a cache that can drop rejected positions: recurrent layers cannot")
        if model.w.tp_size > 1 and model.w.lm_head.w.shape[0] != model.cfg.vocab:
            raise ValueError("speculative decoding takes the arg-max of the local logits: it needs an unsharded LM head")
        self.model, self.kv, self.page = model, kv, page_size
        self.blocks = KvBlockManager(num_pages, page_size)
        self.drafter = drafter
        self.device = model.w.embed.device
        self.stats = SpecStats()

    def _table(self, seqs: Sequence[int]) -> torch.Tensor:
        pages = [self.blocks.pages(s) for s in seqs]
        bt = torch.zeros(len(seqs), max(len(p) for p in pages), dtype=torch.int32)
        for i, p in enumerate(pages):
            bt[i, : len(p)] = torch.tensor(p, dtype=torch.int32)
        return bt

    def _forward(self, q_lens, ctx, ids, seqs, all_logits: bool) -> List[int]:
        m = self.model
        fb = ForwardBatch.build(q_lens, ctx, ids, self._table(seqs), self.page, m.hq_local, m.hkv_local, self.device, all_logits=all_logits)
        return [int(t) for t in m.forward_greedy(fb).cpu()]

    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, stop_token_ids: Sequence[int] = ()) -> List[List[int]]:
        gamma = self.drafter.gamma if self.drafter is not None else 0
        n_seq = len(prompts)
        seqs = [self.blocks.new_sequence() for _ in range(n_seq)]
        toks = [list(p) for p in prompts]
        for s, p in zip(seqs, prompts):
            self.blocks.reserve(s, len(p) + max_new_tokens + gamma + 1)
        # prefill: the last position's arg-max is the first new token
        first = self._forward([len(p) for p in prompts], [0] * n_seq, [t for p in prompts for t in p], seqs, all_logits=False)
        out: List[List[int]] = [[f] for f in first]
        ctx = [len(p) for p in prompts]                      # positions whose K/V are committed
        for i in range(n_seq):
            toks[i].append(first[i])
        stop = set(int(t) for t in stop_token_ids)
        done = [len(o) >= max_new_tokens or o[-1] in stop for o in out]
        while not all(done):
            live = [i for i in range(n_seq) if not done[i]]
            rooms = [max(0, min(gamma, max_new_tokens - len(out[i]) - 1)) for i in live]   # drafts that may follow the sure token
            if hasattr(self.drafter, "propose_batch"):
                drafts = [[int(t) for t in d][:r] for d, r in zip(self.drafter.propose_batch(live, [toks[i] for i in live], rooms), rooms)]
            else:
                drafts = [[int(t) for t in self.drafter.propose(toks[i])][:r] if self.drafter is not None and r > 0 else []
                          for i, r in zip(live, rooms)]
            q_lens = [1 + len(d) for d in drafts]
            ids = []
            for i, d in zip(live, drafts):
                ids.extend([toks[i][-1]] + d)
            target = self._forward(q_lens, [ctx[i] for i in live], ids, [seqs[i] for i in live], all_logits=True)
            p0 = 0
            step_tokens = 0
            for i, d, q in zip(live, drafts, q_lens):
                n_keep, nxt = accept_greedy(d, target[p0:p0 + q])
                p0 += q
                new = d[:n_keep] + [nxt]
                self.stats.drafted += len(d)
                self.stats.accepted += n_keep
                for t in new:
                    out[i].append(t)
                    toks[i].append(t)
                    step_tokens += 1
                    if t in stop or len(out[i]) >= max_new_tokens:
                        done[i] = True
                        break
                ctx[i] += 1 + n_keep                          # the last input and the kept drafts are now committed
            self.stats.verify_steps += 1
            self.stats.produced += step_tokens
            self.stats.per_step.append(step_tokens)
        for s in seqs:
            self.blocks.release(s)
        if hasattr(self.drafter, "finish"):
            self.drafter.finish(range(n_seq))
        return out
