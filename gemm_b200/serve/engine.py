"""Inference engine: paged KV cache, chunked batched prefill, CUDA-graph decode, sampling.

This is the public entry point of the framework (``gemm_b200.LLM`` re-exports it).  It replaces the
reference's ``transformer_load -> forward -> sample`` loop (cpu/llm/test_transformer.c:209-345) and the CUDA
runner's ``cuda_llm_prefill / cuda_llm_forward_logits`` (cuda/llm/cuda_llm_runner.h:24-137), adding what
those lack: batches of sequences, a paged cache, and a decode step that is one graph launch with the
bookkeeping (positions, cache slots, token feedback) kept on the device.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import ctypes
import os

import torch

from .. import _native
from ..utils import profiler

from ..models.config import ModelConfig
from ..models.transformer import ForwardBatch, KvCache, Transformer
from ..models.weights import ModelWeights
from ..ops import attention as att
from ..ops import elementwise as ew
from ..ops import sampling


@dataclass
class SamplingParams:
    max_new_tokens: int = 16
    temperature: float = 0.0          # 0 = greedy
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0
    stop_token_ids: Sequence[int] = ()


class PageAllocator:
    """Free list of KV pages (host side)."""

    def __init__(self, num_pages: int):
        self.free = list(range(num_pages - 1, -1, -1))
        self.num_pages = num_pages

    def alloc(self, n: int) -> List[int]:
        if n > len(self.free):
            raise MemoryError(f"KV cache exhausted: want {n} pages, {len(self.free)} free")
        return [self.free.pop() for _ in range(n)]

    def release(self, pages: Sequence[int]) -> None:
        self.free.extend(pages)


class Engine:
    def __init__(self, weights: ModelWeights, max_batch: int, max_seq_len: int, page_size: int = 128, par=None,
                 max_prefill_tokens: int = 16384, num_pages: Optional[int] = None, kv_dtype: str = "bf16"):
        self.w = weights
        self.cfg: ModelConfig = weights.cfg
        if weights.embed.is_cuda and "GB_PDL" not in os.environ:
            # Programmatic dependent launch (every kernel starts its prologue under the tail of the one before): chosen by what was
            # measured on the decode step.  Dense stacks gain (Qwen3-8B, 2 GPUs: 7.67 against 7.95 ms).  The MoE step, whose layer is
            # two long persistent kernels and a few short ones, loses on 1, 2 and 4 GPUs (Qwen3-30B-A3B: 11.56 against 11.14 ms,
            # 9.86 against 9.47, 7.92 against 7.85) and gains on 8, where every kernel is short (7.41 against 7.62).
            ep = getattr(par, "ep_size", 1) if par is not None else 1
            _native.cuda().gb_set_pdl(ctypes.c_int(0 if (self.cfg.is_moe and ep <= 4) else 1))
        self.device = weights.embed.device
        self.page_size = page_size
        self.max_batch = max_batch
        self.max_pages_per_seq = (max_seq_len + page_size - 1) // page_size
        # context parallelism (parallel.context.ContextParallel as ``par``): this rank's cache holds every world-th page of a sequence
        self.cp = par if getattr(par, "cp_world", 1) > 1 else None
        if self.cp is not None:
            if self.cp.block != page_size:
                raise ValueError("context parallelism deals the positions out by pages: ContextParallel(block=...) must equal page_size")
            if kv_dtype != "bf16" or self.cfg.sliding_window or any(l.ssm is not None for l in weights.layers) or weights.tp_size > 1:
                raise NotImplementedError("context parallelism: bf16 KV cache, full attention in every layer, replicated weights")
            self.max_pages_per_seq = (self.max_pages_per_seq + self.cp.world - 1) // self.cp.world
        n_pages = num_pages if num_pages is not None else max_batch * self.max_pages_per_seq
        hkv_local = max(1, self.cfg.n_kv_heads // weights.tp_size)
        # one recurrent-state slot per sequence plus a scratch slot (hybrid models; used by the warm-up run before graph capture)
        # kv_dtype "int8": pages of int8 + scales read directly by the decode attention kernel (half the bytes per step and per
        # sequence); a prompt must then fit one prefill chunk (max_prefill_tokens)
        self.kv = KvCache.allocate(self.cfg, n_pages, page_size, self.device, hkv_local, n_layers=len(weights.layers), n_seq_slots=max_batch + 1,
                                   kv_dtype=kv_dtype, stage_pages=(max_prefill_tokens + page_size - 1) // page_size + max_batch)
        self.pages = PageAllocator(n_pages)
        self.model = Transformer(weights, self.kv, par)
        self.par = self.model.par
        self.max_prefill_tokens = max_prefill_tokens
        self.hq_local = self.model.hq_local
        self.hkv_local = self.model.hkv_local
        self._graph = None
        self._static: Dict[str, torch.Tensor] = {}
        self.seq_pages: List[List[int]] = []
        self.seq_len: List[int] = []
        self.step_count = 0
        self.kernels_per_step = 0

    # ------------------------------------------------------------------------------------------ sequences
    def reset(self) -> None:
        """Drop every sequence and return its pages (the reference's cuda_llm_reset_state)."""
        for p in self.seq_pages:
            self.pages.release(p)
        self.seq_pages, self.seq_len = [], []
        self._graph = None

    def _ensure_pages(self, s: int, length: int) -> None:
        need = (length + self.page_size - 1) // self.page_size
        if self.cp is not None:
            need = self.cp.local_pages(need)
        have = len(self.seq_pages[s])
        if need > have:
            self.seq_pages[s].extend(self.pages.alloc(need - have))

    def _block_table(self, seqs: Sequence[int]) -> torch.Tensor:
        bt = torch.zeros(len(seqs), self.max_pages_per_seq, dtype=torch.int32)
        for i, s in enumerate(seqs):
            p = self.seq_pages[s]
            bt[i, : len(p)] = torch.tensor(p, dtype=torch.int32)
        return bt

    # ------------------------------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, prompts: Sequence[torch.Tensor], reserve: int = 0, embeds: Optional[Sequence[torch.Tensor]] = None,
                deepstack: Optional[Sequence[Optional[torch.Tensor]]] = None) -> torch.Tensor:
        """Batched, chunked prefill of new sequences (token id tensors, host or device).  Returns the logits of
        the last prompt token of every sequence, ``f32 [B, V_local]``.  ``reserve`` extra positions are paged in.
        ``embeds`` (multimodal prompts): per sequence a bf16 ``[len, hidden]`` tensor of input rows that replace the token
        embeddings (text rows embedded by the caller, vision rows from the encoder; ``models.vision.prompt_inputs`` builds
        them); ``deepstack``: per sequence bf16 ``[n_deepstack, len, hidden]`` (zero on text rows) or None."""
        base = len(self.seq_pages)
        if base + len(prompts) > self.max_batch:
            raise ValueError(f"{base + len(prompts)} sequences exceed max_batch = {self.max_batch}")
        self.kv.reset_slots(range(base, base + len(prompts)))
        for pr in prompts:
            self.seq_pages.append([])
            self.seq_len.append(0)
            self._ensure_pages(len(self.seq_pages) - 1, pr.numel() + reserve)
        b = len(prompts)
        if embeds is not None and self.cp is not None:
            raise NotImplementedError("multimodal prompts under context parallelism")
        if self.cp is not None:
            # sequence-parallel prefill of whole prompts: this rank runs the tokens of its own pages
            # (whole sequences per forward pass, as many as keep every rank within max_prefill_tokens: the same groups on all ranks)
            cp, ps = self.cp, self.page_size
            share = [max(min(cp.local_pages((p.numel() + ps - 1) // ps, r) * ps, p.numel()) for r in range(cp.world)) for p in prompts]
            if max(share) > self.max_prefill_tokens:
                raise ValueError(f"context-parallel prefill: a prompt puts {max(share)} tokens on one rank, max_prefill_tokens is "
                                 f"{self.max_prefill_tokens}")
            i0, parts = 0, []
            while i0 < b:
                i1, room = i0, self.max_prefill_tokens
                while i1 < b and share[i1] <= room:
                    room -= share[i1]
                    i1 += 1
                fb, owned = cp.build_prefill(prompts[i0:i1], self.seq_pages[base + i0: base + i1], self.hq_local, self.hkv_local, self.device,
                                             seq_slots=range(base + i0, base + i1))
                with profiler.region("prefill_chunk", "step", "engine"):
                    logits = self.model.forward(fb)
                parts.append(cp.merge_logits(logits, owned, i1 - i0))
                i0 = i1
            for i in range(b):
                self.seq_len[base + i] = prompts[i].numel()
            return torch.cat(parts)
        done = [0] * b
        last_logits: List[Optional[torch.Tensor]] = [None] * b
        budget = self.max_prefill_tokens
        while any(done[i] < prompts[i].numel() for i in range(b)):
            q_lens, ctx, ids, seqs = [], [], [], []
            room = budget
            for i in range(b):
                left = prompts[i].numel() - done[i]
                if left == 0 or room == 0:
                    continue
                take = min(left, room)
                q_lens.append(take); ctx.append(done[i]); seqs.append(i)
                ids.append(prompts[i][done[i]:done[i] + take])
                room -= take
            fb = ForwardBatch.build(q_lens, ctx, torch.cat([x.to(self.device) for x in ids]), self._block_table([base + i for i in seqs]),
                                    self.page_size, self.hq_local, self.hkv_local, self.device, seq_slots=[base + i for i in seqs],
                                    stage=self.kv.quantized)
            if embeds is not None:
                fb.embeds = torch.cat([embeds[i][c: c + q].to(self.device, torch.bfloat16) for i, c, q in zip(seqs, ctx, q_lens)])
                if deepstack is not None and any(d is not None for d in deepstack):
                    n_ds = next(d.shape[0] for d in deepstack if d is not None)
                    fb.deepstack = torch.cat([deepstack[i][:, c: c + q].to(self.device, torch.bfloat16) if deepstack[i] is not None else
                                              torch.zeros(n_ds, q, self.cfg.hidden, dtype=torch.bfloat16, device=self.device)
                                              for i, c, q in zip(seqs, ctx, q_lens)], dim=1)
            with profiler.region("prefill_chunk", "step", "engine"):
                logits = self.model.forward(fb)
            for j, i in enumerate(seqs):
                done[i] += q_lens[j]
                if done[i] == prompts[i].numel():
                    last_logits[i] = logits[j]
        for i in range(b):
            self.seq_len[base + i] = prompts[i].numel()
        return torch.stack(last_logits)

    # ------------------------------------------------------------------------------------------ decode
    def _sample(self, logits: torch.Tensor, sp: SamplingParams, step: int, step_ctr: Optional[torch.Tensor] = None) -> torch.Tensor:
        tok = sampling.sample(logits, sp.temperature, sp.top_k, sp.top_p, sp.seed, step, step_ctr) if sp.temperature > 0 else \
            sampling.argmax(logits, idx_offset=self.w.vocab_start)
        return self.par.merge_sampled(tok, logits) if hasattr(self.par, "merge_sampled") else tok

    @torch.no_grad()
    def begin_decode(self, first_tokens: torch.Tensor, sp: Optional[SamplingParams] = None, max_new_tokens: int = 256,
                     use_graph: bool = True) -> None:
        """Set up the static decode state for all current sequences: the next input token of each, positions,
        slots, block table (pages for ``max_new_tokens`` more positions are reserved now), then capture one step."""
        sp = sp or SamplingParams()
        self._sp = sp
        b = len(self.seq_pages)
        for s in range(b):
            self._ensure_pages(s, self.seq_len[s] + max_new_tokens + 1)
        bt = self._block_table(range(b)).to(self.device)
        pos = torch.tensor(self.seq_len, dtype=torch.int32, device=self.device)
        slots = None if self.cp is not None else torch.tensor(
            [self.seq_pages[s][self.seq_len[s] // self.page_size] * self.page_size + self.seq_len[s] % self.page_size for s in range(b)],
            dtype=torch.int32, device=self.device)
        max_kv = max(self.seq_len) + max_new_tokens + 1
        splits = att.pick_splits(b, self.hkv_local, max_kv) if self.device.type == "cuda" else 1
        kv_len = pos + 1
        if self.cp is not None:
            cp, ps = self.cp, self.page_size
            # KV ranges per rank: by the rank's share of the longest sequence, the same on every rank (the merge gathers them all)
            splits = min(att.pick_splits(b, self.hkv_local, (max_kv + cp.world - 1) // cp.world), cp.max_splits) if self.device.type == "cuda" else 1
            kv_len = torch.tensor([cp.local_len(n + 1) for n in self.seq_len], dtype=torch.int32, device=self.device)
            slots = torch.tensor([self.seq_pages[s][n // ps // cp.world] * ps + n % ps if cp.owner(n) == cp.rank else -1
                                  for s, n in enumerate(self.seq_len)], dtype=torch.int32, device=self.device)
        st = self._static
        st["ids"] = first_tokens.to(device=self.device, dtype=torch.int32).clone()
        st["positions"], st["slots"] = pos, slots
        st["kv_len"] = kv_len
        st["block_table"] = bt
        st["cu_q"] = torch.arange(b + 1, dtype=torch.int32, device=self.device)
        st["work"] = att.build_work([1] * b, self.hq_local, self.hkv_local, splits).to(self.device)
        st["rows"] = torch.arange(b, dtype=torch.int64, device=self.device)
        st["tokens"] = torch.zeros(b, dtype=torch.int32, device=self.device)
        st["seq_slots"] = torch.arange(b, dtype=torch.int32, device=self.device)
        st["stage_slots"] = torch.arange(b, dtype=torch.int32, device=self.device) if self.kv.quantized else None
        # decode step number on the device: the sampler reads it and the bookkeeping kernel advances it, so graph replays and
        # eager steps draw the same random numbers
        st["step"] = torch.ones(1, dtype=torch.int64, device=self.device)       # step 0 sampled the first token after the prefill
        self._splits = splits
        self._graph = None
        self.step_count = 0
        if use_graph and self.device.type == "cuda":
            # warm up on a side stream (lazy initialisations must not happen during capture), restoring state after
            saved = {k: st[k].clone() for k in ("ids", "positions", "slots", "kv_len", "step")}
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            n0 = _native.launch_count()
            st["seq_slots"].fill_(self.max_batch)          # the warm-up run must not advance any sequence's recurrent state
            with torch.cuda.stream(side):
                self._decode_body()
            self.kernels_per_step = _native.launch_count() - n0
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            for k, v in saved.items():
                st[k].copy_(v)
            st["seq_slots"].copy_(torch.arange(b, dtype=torch.int32, device=self.device))
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._decode_body()
            for k, v in saved.items():
                st[k].copy_(v)
            self._graph = g

    def _decode_body(self) -> None:
        st = self._static
        fb = ForwardBatch(ids=st["ids"], positions=st["positions"], slots=st["slots"], cu_q=st["cu_q"], kv_len=st["kv_len"],
                          block_table=st["block_table"], work=st["work"], logit_rows=st["rows"], num_splits=self._splits,
                          n_tokens=st["ids"].numel(), seq_slots=st["seq_slots"], is_decode=True, stage_slots=st["stage_slots"])
        if self._sp.temperature <= 0 and not hasattr(self.par, "merge_sampled"):
            tok = self.model.forward_greedy(fb)
        else:
            logits = self.model.forward(fb)
            tok = self._sample(logits, self._sp, 0, st["step"])
        st["tokens"].copy_(tok)
        st["ids"].copy_(tok)
        ew.decode_advance(st["positions"], st["kv_len"], st["slots"], st["block_table"], self.page_size, step_ctr=st["step"],
                          cp_world=self.cp.world if self.cp is not None else 1, cp_rank=self.cp.rank if self.cp is not None else 0)

    @torch.no_grad()
    def decode_step(self) -> torch.Tensor:
        """One token for every sequence; returns the device tensor of sampled ids (valid until the next step)."""
        with profiler.region("decode_step", "step", "engine"):
            if self._graph is not None:
                self._graph.replay()
            else:
                self._decode_body()
        self.step_count += 1
        for s in range(len(self.seq_len)):
            self.seq_len[s] += 1
        return self._static["tokens"]

    def set_next_tokens(self, ids: torch.Tensor) -> None:
        """Override the tokens fed to the next decode step (H2D copy when ``ids`` is a pinned host tensor)."""
        self._static["ids"].copy_(ids, non_blocking=True)

    # ------------------------------------------------------------------------------------------ generate
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], sp: Optional[SamplingParams] = None, use_graph: bool = True) -> List[List[int]]:
        """Static-batch generation: prefill all prompts, then decode until every sequence stopped or hit the limit."""
        sp = sp or SamplingParams()
        self.reset()
        pts = [torch.tensor(list(p), dtype=torch.int32) for p in prompts]
        logits = self.prefill(pts, reserve=sp.max_new_tokens + 1)
        first = self._sample(logits, sp, 0)
        out = [[int(t)] for t in first.tolist()]
        alive = [t[0] not in sp.stop_token_ids for t in out]
        if sp.max_new_tokens > 1:
            self.begin_decode(first, sp, sp.max_new_tokens, use_graph)
            for _ in range(sp.max_new_tokens - 1):
                if not any(alive):
                    break
                toks = self.decode_step().tolist()
                for i, t in enumerate(toks):
                    if alive[i]:
                        out[i].append(int(t))
                        if t in sp.stop_token_ids:
                            alive[i] = False
        return out
