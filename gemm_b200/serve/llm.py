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
        self._reqs: Dict[int, _Req] = {}
        self._next_id = 0
        self.steps = 0

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
    def add_request(self, prompt_ids: Sequence[int], sp: Optional[SamplingParams] = None) -> int:
        sp = sp or SamplingParams()
        rid = self._next_id
        self._next_id += 1
        self._reqs[rid] = _Req(list(prompt_ids), len(prompt_ids), sp)
        self.sched.add(rid, len(prompt_ids), sp.max_new_tokens)
        return rid

    def has_work(self) -> bool:
        return self.sched.num_waiting > 0 or self.sched.num_running > 0

    @torch.no_grad()
    def step(self) -> Dict[int, int]:
        """One engine step.  Returns ``{request id: new token}`` for the requests that produced a token."""
        plan = self.sched.plan()
        if not plan:
            return {}
        q_lens, ctx, ids, emit_rows = [], [], [], []
        max_pages = max(len(self.blocks.pages(it.seq)) for it in plan)
        bt = torch.zeros(len(plan), max_pages, dtype=torch.int32)
        for i, it in enumerate(plan):
            r = self._reqs[it.req_id]
            pages = self.blocks.pages(it.seq)
            bt[i, : len(pages)] = torch.tensor(pages, dtype=torch.int32)
            q_lens.append(it.q_len)
            ctx.append(it.ctx_len)
            ids.extend(r.tokens[it.ctx_len: it.ctx_len + it.q_len])
            if it.req_id not in self._slot_of:              # first chunk of this request: take a state slot and clear it
                self._slot_of[it.req_id] = self._free_slots.pop()
                self.kv.reset_slots([self._slot_of[it.req_id]])
        fb = ForwardBatch.build(q_lens, ctx, ids, bt, self.page_size, self.model.hq_local, self.model.hkv_local, self.device,
                                seq_slots=[self._slot_of[it.req_id] for it in plan])
        logits = self.model.forward(fb)                     # one row per plan item (its last token)
        produced: Dict[int, int] = {}
        finished = []
        for i, it in enumerate(plan):
            r = self._reqs[it.req_id]
            fin = False
            if it.emits_token:
                sp = r.sp
                tok = int(sampling.sample(logits[i:i + 1], sp.temperature, sp.top_k, sp.top_p, sp.seed + it.req_id, len(r.out))[0])
                r.tokens.append(tok)
                r.out.append(tok)
                produced[it.req_id] = tok
                fin = tok in sp.stop_token_ids or len(r.out) >= sp.max_new_tokens
                r.done = fin
            finished.append(fin)
            if fin and it.req_id in self._slot_of:
                self._free_slots.append(self._slot_of.pop(it.req_id))
        self.sched.commit(finished)
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
        return [self._reqs.pop(r).out for r in rids]

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
            out = self.step()
            if rid in out:
                yield out[rid]
        self._reqs.pop(rid, None)

    def decode(self, ids: Sequence[int]) -> str:
        if self.tokenizer is None:
            raise RuntimeError("no tokenizer loaded")
        return self.tokenizer.decode(ids)
