"""``LLM``: the user-facing object.  Loads a checkpoint (GGUF, HF safetensors or synthetic), owns the tokenizer and
serves requests with continuous batching: every engine step mixes one decode token per running sequence with
prompt chunks of waiting ones (scheduler and block manager in C++, csrc/host/runtime.cc).

The reference serves one request at a time with token-by-token prefill (server/server_llm.c:422-632); its batched
engines refill finished slots immediately (a64fx/glm5/glm5_ep_runner.c:294-376) — that behaviour is what the
scheduler reproduces, for any number of sequences and with a paged cache.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Iterator, List, Optional, Sequence

import torch

from ..models import loader
from ..models.config import ModelConfig, get_config
from ..models.transformer import ForwardBatch, KvCache, Transformer
from ..models.weights import ModelWeights, synthetic_weights
from ..ops import attention as att
from ..ops import elementwise as ew
from ..ops import sampling
from ..utils.tokenizer import Tokenizer
from .engine import SamplingParams
from .scheduler import KvBlockManager, Scheduler


@dataclass
class _Req:
    tokens: List[int]
    prompt_len: int
    sp: SamplingParams
    out: List[int] = field(default_factory=list)
    done: bool = False
    error: Optional[str] = None      # set when the scheduler had to drop the request (the cache can never hold it)
    embeds: Optional[torch.Tensor] = None       # bf16 [prompt_len, hidden]: input rows of a multimodal prompt (replace the token embeddings)
    deepstack: Optional[torch.Tensor] = None    # bf16 [n_deepstack, prompt_len, hidden]: rows added after the first layers, zero on text


class LLM:
    def __init__(self, weights: ModelWeights, tokenizer: Optional[Tokenizer] = None, max_running: int = 64, max_batch_tokens: int = 8192,
                 num_pages: int = 512, page_size: int = 128, par=None):
        self.w = weights
        self.cfg: ModelConfig = weights.cfg
        self.tokenizer = tokenizer
        self.device = weights.embed.device
        self.page_size = page_size
        self.num_pages = num_pages
        hkv_local = max(1, self.cfg.n_kv_heads // weights.tp_size)
        self.kv = KvCache.allocate(self.cfg, num_pages, page_size, self.device, hkv_local, n_layers=len(weights.layers), n_seq_slots=max_running)
        self._free_slots = list(range(max_running))       # recurrent-state slots of the hybrid models, one per running request
        self._slot_of: Dict[int, int] = {}
        self.blocks = KvBlockManager(num_pages, page_size)
        self.sched = Scheduler(self.blocks, max_running, max_batch_tokens)
        self.model = Transformer(weights, self.kv, par)
        if weights.lm_head.w.shape[0] != self.cfg.vocab and weights.tp_size > 1:
            # this loop samples from the local logits; with a vocabulary-sharded head every rank would pick a different token.
            # serve.engine.Engine merges the shards (arg-max all-reduce); here the head must be whole.
            raise ValueError("LLM (continuous batching) needs an unsharded LM head: build the weights with shard_vocab=False, "
                             "or use serve.engine.Engine, which merges the vocabulary shards")
        self._reqs: Dict[int, _Req] = {}
        self._next_id = 0
        self.steps = 0
        self.drafter = None                                 # speculative decoding of greedy requests inside the batching loop
        self.produced_all: Dict[int, List[int]] = {}        # every token of the last step, per request (several after accepted drafts)
        self.spec_drafted = 0
        self.spec_accepted = 0

    # ------------------------------------------------------------------------------------------ constructors
    @classmethod
    def from_gguf(cls, path: str, fmt: str = "bf16", device="cuda", **kw) -> "LLM":
        from ..utils import gguf as G
        with G.GGUFFile(path) as f:
            tok = Tokenizer.from_gguf(f) if "tokenizer.ggml.tokens" in f.metadata else None
        return cls(loader.load_gguf(path, fmt, device), tok, **kw)

    @classmethod
    def from_safetensors(cls, path: str, fmt: str = "bf16", device="cuda", tokenizer: Optional[Tokenizer] = None, **kw) -> "LLM":
        return cls(loader.load_safetensors(path, fmt, device), tokenizer, **kw)

    @classmethod
    def from_synthetic(cls, model: str, fmt: str = "bf16", device="cuda", seed: int = 0, **kw) -> "LLM":
        return cls(synthetic_weights(get_config(model), fmt, device, seed), None, **kw)

    # ------------------------------------------------------------------------------------------ requests
    def add_request(self, prompt_ids: Sequence[int], sp: Optional[SamplingParams] = None, embeds: Optional[torch.Tensor] = None,
                    deepstack: Optional[torch.Tensor] = None) -> int:
        """``embeds`` / ``deepstack`` (multimodal prompts, ``models.vision.prompt_inputs``): input rows of the prompt positions; the
        ids at image positions are placeholders.  Generated tokens are embedded from the table as usual."""
        sp = sp or SamplingParams()
        if embeds is not None and (embeds.shape[0] != len(prompt_ids) or (deepstack is not None and deepstack.shape[1] != len(prompt_ids))):
            raise ValueError("embeds / deepstack must have one row per prompt position")
        rid = self._next_id
        self._next_id += 1
        self.sched.add(rid, len(prompt_ids), sp.max_new_tokens)      # raises ValueError for a request the cache can never hold
        self._reqs[rid] = _Req(list(prompt_ids), len(prompt_ids), sp, embeds=embeds, deepstack=deepstack)
        return rid

    def set_drafter(self, drafter) -> None:
        """Speculative decoding inside continuous batching: decode items of greedy requests carry up to ``drafter.gamma`` draft
        tokens (``drafter.propose(tokens)``, e.g. ``serve.speculative.NgramDrafter``), verified in the same step; the scheduler
        reserves the extra positions and counts them against the token budget.  ``None`` switches it off."""
        if drafter is not None and self.cfg.is_hybrid:
            raise ValueError("speculative decoding needs a cache that can drop rejected positions: recurrent layers cannot")
        self.drafter = drafter
        self.sched.set_lookahead(drafter.gamma if drafter is not None else 0)

    def has_work(self) -> bool:
        return self.sched.num_waiting > 0 or self.sched.num_running > 0

    @torch.no_grad()
    def step(self) -> Dict[int, int]:
        """One engine step.  Returns ``{request id: new token}`` for the requests that produced a token."""
        plan = self.sched.plan()
        for rid in self.sched.take_aborted():               # dropped by the scheduler: finish them with an error instead of spinning
            r = self._reqs.get(rid)
            if r is not None:
                r.done, r.error = True, "request dropped: the KV cache cannot hold it"
            if rid in self._slot_of:
                self._free_slots.append(self._slot_of.pop(rid))
        if not plan:
            if self.has_work():
                self._idle_steps = getattr(self, "_idle_steps", 0) + 1
                if self._idle_steps > 2:
                    raise RuntimeError("scheduler made no progress: requests are queued but no step can be planned")
            return {}
        self._idle_steps = 0
        q_lens, ctx, ids, drafts = [], [], [], []
        max_pages = max(len(self.blocks.pages(it.seq)) for it in plan)
        bt = torch.zeros(len(plan), max_pages, dtype=torch.int32)
        draft_of: Dict[int, List[int]] = {}
        if self.drafter is not None:                        # drafts for the decode items of greedy requests, batched if the drafter can
            cand = [(it, self._reqs[it.req_id]) for it in plan if not it.is_prefill and self._reqs[it.req_id].sp.temperature <= 0]
            rooms = [max(0, min(self.drafter.gamma, r.sp.max_new_tokens - len(r.out) - 1)) for _, r in cand]
            if hasattr(self.drafter, "propose_batch"):
                ds = self.drafter.propose_batch([it.req_id for it, _ in cand], [r.tokens for _, r in cand], rooms) if cand else []
            else:
                ds = [self.drafter.propose(r.tokens) if room > 0 else [] for (_, r), room in zip(cand, rooms)]
            for (it, _), d, room in zip(cand, ds, rooms):
                draft_of[it.req_id] = [int(t) for t in d][:room]
        for i, it in enumerate(plan):
            r = self._reqs[it.req_id]
            pages = self.blocks.pages(it.seq)
            bt[i, : len(pages)] = torch.tensor(pages, dtype=torch.int32)
            draft = draft_of.get(it.req_id, [])
            drafts.append(draft)
            q_lens.append(it.q_len + len(draft))
            ctx.append(it.ctx_len)
            ids.extend(r.tokens[it.ctx_len: it.ctx_len + it.q_len] + draft)
            if it.req_id not in self._slot_of:              # first chunk of this request: take a state slot
                self._slot_of[it.req_id] = self._free_slots.pop()
            if it.is_prefill and it.ctx_len == 0:
                # a sequence starts (or restarts after a recompute-preemption) from an empty recurrent state: unlike K/V, which the
                # re-prefill overwrites, the conv / Delta-Net state of the first pass would otherwise leak into the second
                self.kv.reset_slots([self._slot_of[it.req_id]])
        fb = ForwardBatch.build(q_lens, ctx, ids, bt, self.page_size, self.model.hq_local, self.model.hkv_local, self.device,
                                seq_slots=[self._slot_of[it.req_id] for it in plan])
        if any(self._reqs[it.req_id].embeds is not None and it.ctx_len < self._reqs[it.req_id].prompt_len for it in plan):
            # a prefill chunk of a multimodal prompt is in the batch: every row of the step enters as an embedding
            rows_in = ew.embed(fb.ids, self.w.embed).clone()
            ds_in, p0 = None, 0
            for it, q in zip(plan, q_lens):
                r = self._reqs[it.req_id]
                lo, hi = it.ctx_len, min(it.ctx_len + q, r.prompt_len)
                if r.embeds is not None and hi > lo:
                    rows_in[p0: p0 + hi - lo] = r.embeds[lo:hi].to(self.device, torch.bfloat16)
                    if r.deepstack is not None:
                        if ds_in is None:
                            ds_in = torch.zeros(r.deepstack.shape[0], rows_in.shape[0], rows_in.shape[1], dtype=torch.bfloat16, device=self.device)
                        ds_in[:, p0: p0 + hi - lo] = r.deepstack[:, lo:hi].to(self.device, torch.bfloat16)
                p0 += q
            fb.embeds, fb.deepstack = rows_in, ds_in
        # logits: one row per plan item (its last token); an item with draft tokens gets a row for each of its positions
        row0, rows, p0 = [], [], 0
        for q, d in zip(q_lens, drafts):
            row0.append(len(rows))
            rows.extend(range(p0 + q - 1 - len(d), p0 + q))
            p0 += q
        if any(drafts):
            fb.logit_rows = torch.tensor(rows, dtype=torch.int64, device=self.device)
        logits = self.model.forward(fb)
        greedy_rows = sampling.argmax(logits).cpu().tolist() if any(drafts) else None     # one device read for all drafted items
        produced: Dict[int, int] = {}
        self.produced_all = {}
        finished, advance = [], []
        for i, it in enumerate(plan):
            r = self._reqs[it.req_id]
            fin = False
            new: List[int] = []
            if it.emits_token:
                sp = r.sp
                if drafts[i]:
                    from .speculative import accept_greedy
                    target = greedy_rows[row0[i]: row0[i] + len(drafts[i]) + 1]
                    n_keep, nxt = accept_greedy(drafts[i], target)
                    new = drafts[i][:n_keep] + [nxt]
                    self.spec_drafted += len(drafts[i])
                    self.spec_accepted += n_keep
                else:
                    j = row0[i]
                    new = [int(sampling.sample(logits[j:j + 1], sp.temperature, sp.top_k, sp.top_p, sp.seed + it.req_id, len(r.out))[0])]
                kept = []
                for tok in new:
                    r.tokens.append(tok)
                    r.out.append(tok)
                    kept.append(tok)
                    if tok in sp.stop_token_ids or len(r.out) >= sp.max_new_tokens:
                        fin = True
                        break
                new = kept
                produced[it.req_id] = new[-1]
                self.produced_all[it.req_id] = new
                r.done = fin
            finished.append(fin)
            advance.append(max(1, len(new)))
            if fin and it.req_id in self._slot_of:
                self._free_slots.append(self._slot_of.pop(it.req_id))
            if fin and hasattr(self.drafter, "finish"):
                self.drafter.finish([it.req_id])
        self.sched.commit(finished, advance if any(a > 1 for a in advance) else None)
        self.steps += 1
        return produced

    # ------------------------------------------------------------------------------------------ convenience
    def generate(self, prompts: Sequence, sp: Optional[SamplingParams] = None) -> List[List[int]]:
        """Token ids generated for every prompt (lists of ids, or strings when a tokenizer is loaded)."""
        rids = []
        for p in prompts:
            ids = self.tokenizer.encode(p) if isinstance(p, str) else list(p)
            rids.append(self.add_request(ids, sp))
        while self.has_work():
            self.step()
        reqs = [self._reqs.pop(r) for r in rids]
        bad = [q.error for q in reqs if q.error]
        if bad:
            raise RuntimeError(bad[0])
        return [q.out for q in reqs]

    def generate_speculative(self, prompts: Sequence, max_new_tokens: int = 64, gamma: int = 4, drafter=None,
                             stop_token_ids: Sequence[int] = ()):
        """Greedy generation with speculative decoding (``serve/speculative.py``): same tokens as greedy ``generate``, fewer
        model steps when the drafts hit.  Uses the whole cache, so no request may be in flight.  Returns (outputs, statistics)."""
        from .speculative import NgramDrafter, SpeculativeDecoder
        if self.has_work():
            raise RuntimeError("speculative generation needs an idle engine")
        if self.blocks.num_free != self.num_pages:
            raise RuntimeError("speculative generation needs an empty cache")
        dec = SpeculativeDecoder(self.model, self.kv, self.page_size, self.num_pages, drafter or NgramDrafter(gamma=gamma))
        enc = [self.tokenizer.encode(p) if isinstance(p, str) else list(p) for p in prompts]
        return dec.generate(enc, max_new_tokens, stop_token_ids), dec.stats

    def stream(self, prompt, sp: Optional[SamplingParams] = None) -> Iterator[int]:
        """Yield the tokens of one request as they are produced (other queued requests keep being served)."""
        ids = self.tokenizer.encode(prompt) if isinstance(prompt, str) else list(prompt)
        rid = self.add_request(ids, sp)
        while not self._reqs[rid].done and self.has_work():
            self.step()
            for tok in self.produced_all.get(rid, ()):
                yield tok
        r = self._reqs.pop(rid, None)
        if r is not None and r.error:
            raise RuntimeError(r.error)

    def decode(self, ids: Sequence[int]) -> str:
        if self.tokenizer is None:
            raise RuntimeError("no tokenizer loaded")
        return self.tokenizer.decode(ids)
