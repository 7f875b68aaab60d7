"""Baseline: the benchmark models in plain PyTorch + NCCL — ``torch.matmul`` / ``torch.bmm`` (cuBLAS), ``scaled_dot_product_attention``,
``torch.distributed`` collectives, CUDA graphs for the decode step.  No kernel of ``gemm_b200`` is used anywhere in this file.

It is the comparison the product has to beat: "a path that only calls NCCL (and cuBLAS) is the baseline".  Same architecture,
same random-init weights (``gemm_b200.models.weights.RandomSource`` is only used as the tensor source), same sharding:

* dense models, N GPUs: Megatron tensor parallelism (q/k/v/gate/up by rows, o/down by columns + ``all_reduce``); KV heads are
  replicated when there are fewer of them than ranks;
* MoE models, N GPUs: data-parallel attention + expert parallelism in the reference's own formulation — replicate the tokens
  (``all_gather``), every rank evaluates the experts it owns on all tokens, ``reduce_scatter`` of the partial sums
  (common/m3_impl.h:699-714, 924-950).

Weights are bf16 (the MXFP8 checkpoints of the product are compared against bf16 cuBLAS: PyTorch has no block-scaled fp8 expert
GEMM to call).  KV cache: one contiguous ``[B, Hkv, S_max, D]`` buffer per layer, as in the reference (no paging).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F


def _rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(torch.bfloat16)


def _rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """NeoX rotation (pairs j, j + d/2); x [T, H, D], pos [T]."""
    d = x.shape[-1]
    inv = theta ** (-torch.arange(0, d // 2, device=x.device, dtype=torch.float32) * 2.0 / d)
    ang = pos.float()[:, None] * inv[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    a, b = xf[..., : d // 2], xf[..., d // 2:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1).to(torch.bfloat16)


class _Layer:
    pass


class BaselineModel:
    def __init__(self, cfg, device, seed: int = 0, n_layers: Optional[int] = None, group=None, layout: str = "single"):
        from gemm_b200.models.weights import RandomSource, shard_range
        self.cfg, self.device, self.group = cfg, device, group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.layout = layout if self.world > 1 else "single"          # "tp" | "ep" | "single"
        tp = self.world if self.layout == "tp" else 1
        ep = self.world if self.layout == "ep" else 1
        src = RandomSource(cfg, seed, device)
        h, d = cfg.hidden, cfg.head_dim
        self.hq = cfg.n_heads // tp
        if cfg.n_kv_heads >= tp:
            self.hkv = cfg.n_kv_heads // tp
            kv_lo = (self.rank if tp > 1 else 0) * self.hkv
        else:
            self.hkv, kv_lo = 1, self.rank // (tp // cfg.n_kv_heads)
        r = self.rank if tp > 1 else 0
        q0, q1 = r * self.hq * d, (r + 1) * self.hq * d
        k0, k1 = kv_lo * d, (kv_lo + self.hkv) * d
        self.layers: List[_Layer] = []
        bf = torch.bfloat16
        for li in range(n_layers if n_layers is not None else cfg.n_layers):
            pre = f"blk.{li}."
            L = _Layer()
            L.attn_norm = src.get(pre + "attn_norm.weight", (h,)).to(bf)
            L.ffn_norm = src.get(pre + "ffn_norm.weight", (h,)).to(bf)
            L.wqkv = torch.cat([src.get(pre + "attn_q.weight", (cfg.q_dim, h))[q0:q1], src.get(pre + "attn_k.weight", (cfg.kv_dim, h))[k0:k1],
                                src.get(pre + "attn_v.weight", (cfg.kv_dim, h))[k0:k1]]).to(bf).contiguous()
            L.wo = src.get(pre + "attn_output.weight", (h, cfg.q_dim))[:, q0:q1].to(bf).contiguous()
            L.q_norm = src.get(pre + "attn_q_norm.weight", (d,)).to(bf) if cfg.qk_norm else None
            L.k_norm = src.get(pre + "attn_k_norm.weight", (d,)).to(bf) if cfg.qk_norm else None
            if cfg.is_moe:
                e_l = cfg.n_experts // ep
                e0 = (self.rank if ep > 1 else 0) * e_l
                L.router = src.get(pre + "ffn_gate_inp.weight", (cfg.n_experts, h)).to(bf)
                inter = cfg.expert_ffn
                L.w13 = torch.empty(e_l, 2 * inter, h, dtype=bf, device=device)
                L.w2 = torch.empty(e_l, h, inter, dtype=bf, device=device)
                for j in range(e_l):
                    L.w13[j, :inter] = src.get_expert(pre + "ffn_gate_exps.weight", e0 + j, (inter, h))
                    L.w13[j, inter:] = src.get_expert(pre + "ffn_up_exps.weight", e0 + j, (inter, h))
                    L.w2[j] = src.get_expert(pre + "ffn_down_exps.weight", e0 + j, (h, inter))
                L.e0, L.e_l = e0, e_l
            else:
                f0, f1 = shard_range(cfg.ffn, tp, r) if cfg.ffn % tp else (r * (cfg.ffn // tp), (r + 1) * (cfg.ffn // tp))
                L.wgu = torch.cat([src.get(pre + "ffn_gate.weight", (cfg.ffn, h))[f0:f1], src.get(pre + "ffn_up.weight", (cfg.ffn, h))[f0:f1]]).to(bf).contiguous()
                L.wd = src.get(pre + "ffn_down.weight", (h, cfg.ffn))[:, f0:f1].to(bf).contiguous()
            self.layers.append(L)
        self.embed = src.get("token_embd.weight", (cfg.vocab, h)).to(bf)
        self.head = self.embed if cfg.tie_embeddings else src.get("output.weight", (cfg.vocab, h)).to(bf)
        self.final_norm = src.get("output_norm.weight", (h,)).to(bf)
        self.k_cache: List[torch.Tensor] = []
        self.v_cache: List[torch.Tensor] = []
        self._graph = None

    # ------------------------------------------------------------------------------------------ pieces
    def alloc_kv(self, batch: int, max_len: int) -> None:
        d = self.cfg.head_dim
        self.k_cache = [torch.zeros(batch, self.hkv, max_len, d, dtype=torch.bfloat16, device=self.device) for _ in self.layers]
        self.v_cache = [torch.zeros(batch, self.hkv, max_len, d, dtype=torch.bfloat16, device=self.device) for _ in self.layers]
        self.max_len = max_len

    def _all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.layout == "tp":
            dist.all_reduce(x, group=self.group)
        return x

    def _qkv(self, L, h: torch.Tensor, pos: torch.Tensor):
        cfg, d = self.cfg, self.cfg.head_dim
        qkv = h @ L.wqkv.t()
        t = h.shape[0]
        q = qkv[:, : self.hq * d].reshape(t, self.hq, d)
        k = qkv[:, self.hq * d: (self.hq + self.hkv) * d].reshape(t, self.hkv, d)
        v = qkv[:, (self.hq + self.hkv) * d:].reshape(t, self.hkv, d)
        if L.q_norm is not None:
            q, k = _rmsnorm(q, L.q_norm, cfg.rms_eps), _rmsnorm(k, L.k_norm, cfg.rms_eps)
        return _rope(q, pos, cfg.rope_theta), _rope(k, pos, cfg.rope_theta), v

    def _moe(self, L, h: torch.Tensor) -> torch.Tensor:
        """Experts owned by this rank over the tokens ``h`` (all tokens of the step under expert parallelism): padded batched GEMMs."""
        cfg = self.cfg
        t, k = h.shape[0], cfg.n_experts_used
        logits = (h @ L.router.t()).float()
        p = torch.softmax(logits, dim=-1)
        w, ids = torch.topk(p, k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        local = ids - L.e0
        ok = (local >= 0) & (local < L.e_l)
        flat_e = torch.where(ok, local, torch.full_like(local, L.e_l)).reshape(-1)                 # dropped pairs -> bucket e_l
        onehot = F.one_hot(flat_e, L.e_l + 1)
        slot = (onehot.cumsum(0) - 1).gather(1, flat_e[:, None]).squeeze(1)                        # position inside the expert's bucket
        cap = min(t, self._cap)
        keep = ok.reshape(-1) & (slot < cap)
        tok = torch.arange(t, device=h.device).repeat_interleave(k)
        buf = torch.zeros(L.e_l + 1, cap, h.shape[1], dtype=h.dtype, device=h.device)
        buf[torch.where(keep, flat_e, torch.full_like(flat_e, L.e_l)), torch.where(keep, slot, torch.zeros_like(slot))] = h[tok]
        x = buf[: L.e_l]
        gu = torch.bmm(x, L.w13.transpose(1, 2))
        inter = cfg.expert_ffn
        act = F.silu(gu[..., :inter].float()).to(h.dtype) * gu[..., inter:]
        y = torch.bmm(act, L.w2.transpose(1, 2))                                                   # [e_l, cap, H]
        yp = y[flat_e.clamp_max(L.e_l - 1), slot.clamp_max(cap - 1)].float() * (w.reshape(-1, 1) * keep[:, None])
        return yp.reshape(t, k, -1).sum(1)

    def _ffn(self, L, h: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        if not cfg.is_moe:
            gu = h @ L.wgu.t()
            inter = gu.shape[1] // 2
            act = F.silu(gu[:, :inter].float()).to(h.dtype) * gu[:, inter:]
            return self._all_reduce(act @ L.wd.t())
        if self.layout != "ep":
            return self._moe(L, h).to(torch.bfloat16)
        t = h.shape[0]
        allh = torch.empty(self.world * t, h.shape[1], dtype=h.dtype, device=h.device)
        dist.all_gather_into_tensor(allh, h.contiguous(), group=self.group)
        part = self._moe(L, allh)
        out = torch.empty(t, h.shape[1], dtype=torch.float32, device=h.device)
        dist.reduce_scatter_tensor(out, part, group=self.group)
        return out.to(torch.bfloat16)

    # ------------------------------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, seqs_per_chunk: int = 8) -> torch.Tensor:
        """``tokens`` int [B, S] (this rank's sequences; the whole batch under TP).  Fills the cache, returns the last-token logits."""
        b, s = tokens.shape
        cfg = self.cfg
        self._cap = 1 << 30
        outs = []
        for b0 in range(0, b, seqs_per_chunk):
            ids = tokens[b0: b0 + seqs_per_chunk].to(self.device)
            nb = ids.shape[0]
            x = self.embed[ids.reshape(-1).long()]
            pos = torch.arange(s, device=self.device).repeat(nb)
            for li, L in enumerate(self.layers):
                h = _rmsnorm(x, L.attn_norm, cfg.rms_eps)
                q, k, v = self._qkv(L, h, pos)
                q = q.reshape(nb, s, self.hq, -1).transpose(1, 2)
                k = k.reshape(nb, s, self.hkv, -1).transpose(1, 2)
                v = v.reshape(nb, s, self.hkv, -1).transpose(1, 2)
                self.k_cache[li][b0: b0 + nb, :, :s] = k
                self.v_cache[li][b0: b0 + nb, :, :s] = v
                a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
                a = a.transpose(1, 2).reshape(nb * s, -1)
                x = x + self._all_reduce(a @ L.wo.t())
                h = _rmsnorm(x, L.ffn_norm, cfg.rms_eps)
                x = x + self._ffn_prefill(L, h)
            last = x.reshape(nb, s, -1)[:, -1]
            outs.append(_rmsnorm(last, self.final_norm, cfg.rms_eps) @ self.head.t())
        self.pos = torch.full((b,), s, dtype=torch.long, device=self.device)
        self._prompt_len, self._steps_done = s, 0
        return torch.cat(outs).float()

    def _ffn_prefill(self, L, h: torch.Tensor) -> torch.Tensor:
        """Prefill-sized MoE: tokens sorted by expert, one GEMM pair per owned expert (split sizes read on the host)."""
        cfg = self.cfg
        if not cfg.is_moe:
            return self._ffn(L, h)
        if self.layout == "ep":
            t = h.shape[0]
            allh = torch.empty(self.world * t, h.shape[1], dtype=h.dtype, device=h.device)
            dist.all_gather_into_tensor(allh, h.contiguous(), group=self.group)
            part = self._moe_sorted(L, allh)
            out = torch.empty(t, h.shape[1], dtype=torch.float32, device=h.device)
            dist.reduce_scatter_tensor(out, part, group=self.group)
            return out.to(torch.bfloat16)
        return self._moe_sorted(L, h).to(torch.bfloat16)

    def _moe_sorted(self, L, h: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        t, k, inter = h.shape[0], cfg.n_experts_used, cfg.expert_ffn
        p = torch.softmax((h @ L.router.t()).float(), dim=-1)
        w, ids = torch.topk(p, k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        local = (ids - L.e0).reshape(-1)
        ok = (local >= 0) & (local < L.e_l)
        key = torch.where(ok, local, torch.full_like(local, L.e_l))
        order = torch.argsort(key, stable=True)
        counts = torch.bincount(key, minlength=L.e_l + 1)[: L.e_l].tolist()
        tok = torch.arange(t, device=h.device).repeat_interleave(k)[order]
        xs = h[tok[: sum(counts)]]
        ys = torch.empty(xs.shape[0], h.shape[1], dtype=h.dtype, device=h.device)
        o = 0
        for e, c in enumerate(counts):
            if c == 0:
                continue
            gu = xs[o:o + c] @ L.w13[e].t()
            ys[o:o + c] = (F.silu(gu[:, :inter].float()).to(h.dtype) * gu[:, inter:]) @ L.w2[e].t()
            o += c
        out = torch.zeros(t, h.shape[1], dtype=torch.float32, device=h.device)
        wsel = w.reshape(-1)[order][: sum(counts)]
        out.index_add_(0, tok[: sum(counts)], ys.float() * wsel[:, None])
        return out

    # ------------------------------------------------------------------------------------------ decode
    @torch.no_grad()
    def _decode_body(self) -> None:
        cfg = self.cfg
        ids, pos = self._ids, self.pos
        b = ids.shape[0]
        x = self.embed[ids.long()]
        bidx = torch.arange(b, device=self.device)
        mask = (torch.arange(self.max_len, device=self.device)[None, :] <= pos[:, None])[:, None, None, :]
        for li, L in enumerate(self.layers):
            h = _rmsnorm(x, L.attn_norm, cfg.rms_eps)
            q, k, v = self._qkv(L, h, pos)
            self.k_cache[li][bidx, :, pos] = k
            self.v_cache[li][bidx, :, pos] = v
            a = F.scaled_dot_product_attention(q[:, :, None, :], self.k_cache[li], self.v_cache[li], attn_mask=mask, enable_gqa=True)
            x = x + self._all_reduce(a.reshape(b, -1) @ L.wo.t())
            h = _rmsnorm(x, L.ffn_norm, cfg.rms_eps)
            x = x + self._ffn(L, h)
        logits = _rmsnorm(x, self.final_norm, cfg.rms_eps) @ self.head.t()
        self._ids.copy_(logits.argmax(-1).to(self._ids.dtype))
        self.pos += 1

    def begin_decode(self, first_tokens: torch.Tensor, use_graph: bool = True) -> None:
        self._ids = first_tokens.to(self.device).clone()
        b = self._ids.shape[0]
        self._cap = min(64, b * self.world) if self.cfg.is_moe else 0
        self._graph = None
        if use_graph:
            saved_pos, saved_ids = self.pos.clone(), self._ids.clone()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._decode_body()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.pos.copy_(saved_pos); self._ids.copy_(saved_ids)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._decode_body()
            self.pos.copy_(saved_pos); self._ids.copy_(saved_ids)
            self._graph = g

    def decode_step(self) -> torch.Tensor:
        self._steps_done = getattr(self, "_steps_done", 0) + 1
        if self._prompt_len + self._steps_done >= self.max_len:      # checked on the host: the cache write must never leave the buffer
            raise RuntimeError(f"KV cache of {self.max_len} positions is full")
        if self._graph is not None:
            self._graph.replay()
        else:
            self._decode_body()
        return self._ids
