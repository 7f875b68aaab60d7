"""MiniMax-M3 style engine as a PyTorch-op forward pass (CPU or CUDA): GQA attention with partial RoPE and per-head QK norm, MiniMax
sparse attention (MSA) on the MoE layers, sigmoid-router MoE with score-correction bias, top-k, routed scale and a shared expert,
SwiGLU-OAI activations, Gemma-style RMSNorm, bf16 or int4 KV cache, expert parallelism.

Reference: common/m3.h:75-124 (configuration), common/m3_impl.h:643-732 (one token through the stack), :593-640 (MSA block
selection), :66-90 (int4 KV codec), :113-127 (norms, SwiGLU-OAI, RoPE).  What the pieces do:

* norms multiply by ``1 + w``; q / k heads are normalised the same way, then the first ``rotary_dim`` features of a head are rotated
  (pairs ``(k, k + rotary_dim / 2)``), the rest pass through;
* layers ``< n_dense_layers``: full causal attention + dense FFN; the others: MSA + MoE.  MSA keeps an index key per position (one
  MQA head of ``msa_index_dim``) and projects ``msa_n_index_heads`` index queries per token; a block of ``msa_block_size`` positions
  scores ``max_t sum_h q_h . k_t``; the token attends the first ``msa_init_block`` blocks, the last ``msa_local_block`` blocks and
  the ``msa_topk_blocks`` best of the rest (all causal positions while there are no more blocks than that);
* K / V rows (and index keys) are stored rounded to bf16, or as int4 with one bf16 scale (absmax / 7) per position and head;
* router: ``sigmoid(gate x)``; experts are picked by ``score + bias``, weighted by ``score / sum(scores of the picked) *
  routed_scale``; the shared expert is always added; ``swiglu_oai(g, u) = min(g, lim) * sigmoid(alpha * min(g, lim)) *
  (clamp(u, -lim, lim) + 1)``;
* expert parallelism: expert ``e`` lives on rank ``e % ep_size``; every rank sees every token, evaluates its own experts and the
  partial sums are all-reduced (common/m3_impl.h:699-714).

Like the reference's bring-up path the weights are bf16 (router in fp32); matrix products are library tensor ops.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch


@dataclass
class M3Config:
    n_layers: int = 60
    n_dense_layers: int = 3
    hidden: int = 6144
    vocab: int = 200064
    norm_eps: float = 1e-6
    n_heads: int = 64
    n_kv_heads: int = 4
    head_dim: int = 128
    rotary_dim: int = 64
    rope_theta: float = 5e6
    msa_index_dim: int = 128
    msa_n_index_heads: int = 4
    msa_block_size: int = 128
    msa_topk_blocks: int = 16
    msa_init_block: int = 0
    msa_local_block: int = 1
    n_experts: int = 128
    n_active: int = 4
    moe_inter: int = 3072
    dense_inter: int = 12288
    routed_scale: float = 2.0
    swiglu_alpha: float = 1.702
    swiglu_limit: float = 7.0
    max_pos: int = 8192

    def is_moe(self, li: int) -> bool:
        return li >= self.n_dense_layers


def random_tensors(cfg: M3Config, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    u = lambda amp, *s: ((torch.rand(*s, generator=g) * 2 - 1) * amp)
    bf = lambda amp, *s: u(amp, *s).to(torch.bfloat16)
    h, qd, kvd, hd = cfg.hidden, cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim, cfg.head_dim
    t = {"embed": bf(0.05, cfg.vocab, h), "head": bf(0.05, cfg.vocab, h), "out_norm": bf(0.1, h)}
    for li in range(cfg.n_layers):
        p = f"l{li}."
        t.update({p + "input_norm": bf(0.1, h), p + "post_norm": bf(0.1, h), p + "wq": bf(0.03, qd, h), p + "wk": bf(0.03, kvd, h),
                  p + "wv": bf(0.03, kvd, h), p + "wo": bf(0.03, h, qd), p + "q_norm": bf(0.1, hd), p + "k_norm": bf(0.1, hd)})
        if cfg.is_moe(li):
            iqd, idim, e, it = cfg.msa_n_index_heads * cfg.msa_index_dim, cfg.msa_index_dim, cfg.n_experts, cfg.moe_inter
            t.update({p + "idx_wq": bf(0.03, iqd, h), p + "idx_wk": bf(0.03, idim, h), p + "idx_q_norm": bf(0.1, idim), p + "idx_k_norm": bf(0.1, idim),
                      p + "gate": u(0.03, e, h), p + "gate_bias": u(0.1, e), p + "sh_w1": bf(0.03, it, h), p + "sh_w3": bf(0.03, it, h),
                      p + "sh_w2": bf(0.03, h, it), p + "ex_w1": bf(0.03, e, it, h), p + "ex_w3": bf(0.03, e, it, h), p + "ex_w2": bf(0.03, e, h, it)})
        else:
            t.update({p + "ff_gate": bf(0.03, cfg.dense_inter, h), p + "ff_up": bf(0.03, cfg.dense_inter, h), p + "ff_down": bf(0.03, h, cfg.dense_inter)})
    return t


def q4_quant(x: torch.Tensor):
    """Per last-dimension group: signed int4 codes (int8 tensor in [-7, 7]) and the bf16 scale absmax / 7 (round half to even, like lrintf)."""
    amax = x.float().abs().amax(-1, keepdim=True)
    inv = torch.where(amax > 0, 7.0 / amax, torch.zeros_like(amax))
    codes = torch.round(x.float() * inv).clamp_(-7, 7).to(torch.int8)
    return codes, (amax / 7.0).to(torch.bfloat16)


def q4_dequant(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return codes.float() * scale.float()


class M3Model:
    def __init__(self, cfg: M3Config, tensors: Dict[str, torch.Tensor], device="cpu", dtype=torch.float32, ep_rank: int = 0, ep_size: int = 1,
                 group=None, int4_kv: bool = False, msa: bool = True):
        """``dtype``: the type the bf16 weights are widened to for the products (fp32 reproduces the reference's arithmetic,
        bf16 is the fast path on a GPU).  ``group``: the process group of the expert-parallel ranks (None: single process)."""
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.ep_rank, self.ep_size, self.group, self.int4_kv, self.msa = ep_rank, ep_size, group, int4_kv, msa
        self.t: Dict[str, torch.Tensor] = {}
        for k, v in tensors.items():
            if ".ex_w" in k and ep_size > 1:
                v = v[ep_rank::ep_size]                                # this rank's experts: e % ep_size == ep_rank, slot e // ep_size
            keep32 = k.rsplit(".", 1)[-1] in ("gate", "gate_bias") or v.dim() == 1          # the router and every vector stay fp32
            self.t[k] = v.to(self.device, torch.float32 if keep32 else dtype)
        half = cfg.rotary_dim // 2
        self.inv_freq = (cfg.rope_theta ** (-2.0 * torch.arange(half, dtype=torch.float64) / cfg.rotary_dim)).to(self.device)
        self.pos, self.batch = 0, 0
        self.cache: List[Dict[str, torch.Tensor]] = []

    # ------------------------------------------------------------------------------------------ state
    def clone_runtime(self):
        """Another runtime over the SAME weights with caches and position of its own: several sequences (or streams of a server)
        advance independently at one copy of the parameters (common/glm5_impl.h:640-660 ``glm5_clone_runtime``; the subclasses
        inherit it).  The clone starts empty; call ``reset`` on it."""
        import copy
        other = copy.copy(self)                                  # shares self.t, the tables and the configuration
        other.pos, other.batch, other.cache = 0, 0, []
        for name in ("comp", "icomp", "mtp_cache", "trace", "last_hc"):
            if hasattr(other, name):
                setattr(other, name, {} if name in ("comp", "icomp") else None)
        return other

    def reset(self, batch: int = 1, max_pos: Optional[int] = None) -> None:
        cfg = self.cfg
        n = max_pos or cfg.max_pos
        self.pos, self.batch, self.cache = 0, batch, []
        for li in range(cfg.n_layers):
            c: Dict[str, torch.Tensor] = {}
            shape = (batch, n, cfg.n_kv_heads, cfg.head_dim)
            names = [("k", shape), ("v", shape)] + ([("ik", (batch, n, 1, cfg.msa_index_dim))] if cfg.is_moe(li) else [])
            for nm, shp in names:
                if self.int4_kv:
                    c[nm + "_q"] = torch.zeros(shp, dtype=torch.int8, device=self.device)
                    c[nm + "_s"] = torch.zeros(shp[:-1] + (1,), dtype=torch.bfloat16, device=self.device)
                else:
                    c[nm] = torch.zeros(shp, dtype=torch.bfloat16, device=self.device)
            self.cache.append(c)

    def kv_bytes(self) -> int:
        """Bytes of the caches as they would be packed (two int4 codes per byte)."""
        tot = 0
        for c in self.cache:
            for k, v in c.items():
                tot += v.numel() // 2 if k.endswith("_q") else v.numel() * v.element_size()
        return tot

    def _store(self, c, name: str, rows: torch.Tensor, p0: int) -> None:
        t = rows.shape[1]
        if self.int4_kv:
            q, s = q4_quant(rows)
            c[name + "_q"][:, p0: p0 + t] = q
            c[name + "_s"][:, p0: p0 + t] = s
        else:
            c[name][:, p0: p0 + t] = rows.to(torch.bfloat16)

    def _load(self, c, name: str, n: int) -> torch.Tensor:
        if self.int4_kv:
            return q4_dequant(c[name + "_q"][:, :n], c[name + "_s"][:, :n])
        return c[name][:, :n].float()

    # ------------------------------------------------------------------------------------------ pieces
    def _norm(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.norm_eps) * (1.0 + w.float())).to(x.dtype)

    def _rope(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """``x`` [B, T, H, D]: the first ``rotary_dim`` features turn, the rest pass through."""
        rd = self.cfg.rotary_dim
        half = rd // 2
        ang = positions.double()[:, None] * self.inv_freq[None, :]
        cos, sin = ang.cos().float()[None, :, None, :], ang.sin().float()[None, :, None, :]
        a, b = x[..., :half].float(), x[..., half:rd].float()
        return torch.cat([a * cos - b * sin, a * sin + b * cos, x[..., rd:].float()], dim=-1).to(x.dtype)

    def _swiglu(self, g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
        lim, al = self.cfg.swiglu_limit, self.cfg.swiglu_alpha
        gf, uf = g.float().clamp(max=lim), u.float().clamp(-lim, lim)
        return (gf * torch.sigmoid(al * gf) * (uf + 1.0)).to(g.dtype)

    def _msa_mask(self, li: int, hn: torch.Tensor, positions: torch.Tensor, p0: int, q_lat: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Boolean ``[B, T, p0 + T]``: which cached positions every query token of a sparse layer attends.  Also stores the step's
        index keys.  The index queries come from the normalised hidden rows (``idx_wq``) or, where the checkpoint has ``idx_wq_b``,
        from the low-rank query latent ``q_lat``."""
        cfg, tt, p = self.cfg, self.t, f"l{li}."
        b, t, _ = hn.shape
        ih, idim, blk = cfg.msa_n_index_heads, cfg.msa_index_dim, cfg.msa_block_size
        iq = (q_lat @ tt[p + "idx_wq_b"].t() if (p + "idx_wq_b") in tt else hn @ tt[p + "idx_wq"].t()).reshape(b, t, ih, idim)
        if (p + "idx_q_norm") in tt:
            iq = self._norm(iq, tt[p + "idx_q_norm"])
        iq = self._rope(iq, positions)
        ik = self._rope(self._norm((hn @ tt[p + "idx_wk"].t()).reshape(b, t, 1, idim), tt[p + "idx_k_norm"]), positions)
        self._store(self.cache[li], "ik", ik, p0)
        n = p0 + t
        kpos = torch.arange(n, device=self.device)
        causal = kpos[None, :] <= positions[:, None]                                                  # [T, n]
        keep = cfg.msa_topk_blocks + cfg.msa_local_block + cfg.msa_init_block
        nblk = positions // blk + 1                                                                   # [T] blocks a token can see
        if not self.msa or int(nblk.max()) <= keep:
            return causal[None].expand(b, t, n)
        keys = self._load(self.cache[li], "ik", n)[:, :, 0]                                           # [B, n, idim]
        sc = torch.einsum("bqhd,bkd->bqhk", iq.float(), keys).sum(2)                                  # sum over the index heads
        sc = sc.masked_fill(~causal[None], float("-inf"))
        nb = (n + blk - 1) // blk
        sc = torch.nn.functional.pad(sc, (0, nb * blk - n), value=float("-inf")).reshape(b, t, nb, blk).amax(-1)   # [B, T, nb]
        bidx = torch.arange(nb, device=self.device)
        visible = bidx[None, :] < nblk[:, None]                                                       # [T, nb]
        forced = (bidx[None, :] < cfg.msa_init_block) | (bidx[None, :] >= (nblk[:, None] - cfg.msa_local_block))
        forced = forced & visible
        cand = sc.masked_fill(~(visible & ~forced)[None], float("-inf"))
        k = min(cfg.msa_topk_blocks, nb)
        top = torch.topk(cand, k, dim=-1)
        picked = torch.zeros(b, t, nb, dtype=torch.bool, device=self.device)
        picked.scatter_(2, top.indices, torch.isfinite(top.values))
        sel_blocks = picked | forced[None]
        dense = (nblk <= keep)[None, :, None]                                                         # tokens that still see everything
        sel_blocks = sel_blocks | (dense & visible[None])
        return sel_blocks.repeat_interleave(blk, dim=2)[:, :, :n] & causal[None]

    def _moe(self, li: int, h2: torch.Tensor) -> torch.Tensor:
        cfg, tt, p = self.cfg, self.t, f"l{li}."
        b, t, h = h2.shape
        x = h2.reshape(b * t, h)
        score = torch.sigmoid(x.float() @ tt[p + "gate"].t())                                         # [N, E] fp32 router
        pick = torch.topk(score + tt[p + "gate_bias"][None, :], cfg.n_active, dim=-1).indices
        w = torch.gather(score, 1, pick)
        ws = w.sum(-1, keepdim=True)
        w = w / torch.where(ws > 0, ws, torch.ones_like(ws)) * cfg.routed_scale
        route = torch.zeros(b * t, h, dtype=torch.float32, device=self.device)
        for slot in range(tt[p + "ex_w1"].shape[0]):
            e = slot * self.ep_size + self.ep_rank
            hit = pick == e
            rows = hit.any(-1).nonzero(as_tuple=True)[0]
            if rows.numel() == 0:
                continue
            xe = x[rows]
            act = self._swiglu(xe @ tt[p + "ex_w1"][slot].t(), xe @ tt[p + "ex_w3"][slot].t())
            ye = (act @ tt[p + "ex_w2"][slot].t()).float()
            route.index_add_(0, rows, ye * (w * hit)[rows].sum(-1, keepdim=True))
        pending = None
        if self.ep_size > 1 and self.group is not None:          # the sum over the ranks runs while this rank computes the shared
            import torch.distributed as dist                     # expert (a64fx/m3/m3_ep_runner.c:143-169 does the same with its
            pending = dist.all_reduce(route, group=self.group, async_op=True)     # asynchronous reduce)
        sh = self._swiglu(x @ tt[p + "sh_w1"].t(), x @ tt[p + "sh_w3"].t()) @ tt[p + "sh_w2"].t()
        if pending is not None:
            pending.wait()
        return (route + sh.float()).reshape(b, t, h).to(h2.dtype)

    # ------------------------------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, ids: torch.Tensor, all_logits: bool = False) -> torch.Tensor:
        """``ids`` int [B, T]: the next T tokens of every sequence; f32 logits [B, V] of the last token (``all_logits``: [B, T, V])."""
        cfg, tt = self.cfg, self.t
        ids = ids.to(self.device).long()
        b, t = ids.shape
        if not self.cache or b != self.batch:
            self.reset(b)
        p0 = self.pos
        positions = torch.arange(p0, p0 + t, device=self.device)
        hd, nh, kvh = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
        x = tt["embed"][ids].float()                                                                   # the stream is fp32, like the reference's
        for li in range(cfg.n_layers):
            p, c = f"l{li}.", self.cache[li]
            hn = self._norm(x, tt[p + "input_norm"]).to(self.dtype)
            q = self._rope(self._norm((hn @ tt[p + "wq"].t()).reshape(b, t, nh, hd), tt[p + "q_norm"]), positions)
            k = self._rope(self._norm((hn @ tt[p + "wk"].t()).reshape(b, t, kvh, hd), tt[p + "k_norm"]), positions)
            v = (hn @ tt[p + "wv"].t()).reshape(b, t, kvh, hd)
            self._store(c, "k", k, p0)
            self._store(c, "v", v, p0)
            n = p0 + t
            if cfg.is_moe(li):
                mask = self._msa_mask(li, hn, positions, p0)[:, None]                                  # [B, 1, T, n]
            else:
                mask = (torch.arange(n, device=self.device)[None, :] <= positions[:, None])[None, None]
            g = nh // kvh
            kf = self._load(c, "k", n).repeat_interleave(g, dim=2)
            vf = self._load(c, "v", n).repeat_interleave(g, dim=2)
            sc = torch.einsum("bqhd,bkhd->bhqk", q.float(), kf) / math.sqrt(hd)
            sc = sc.masked_fill(~mask, float("-inf"))
            a = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, dim=-1), vf).reshape(b, t, nh * hd).to(self.dtype)
            x = x + (a @ tt[p + "wo"].t()).float()
            h2 = self._norm(x, tt[p + "post_norm"]).to(self.dtype)
            if cfg.is_moe(li):
                x = x + self._moe(li, h2).float()
            else:
                f = self._swiglu(h2 @ tt[p + "ff_gate"].t(), h2 @ tt[p + "ff_up"].t()) @ tt[p + "ff_down"].t()
                x = x + f.float()
        self.pos = p0 + t
        xo = self._norm(x if all_logits else x[:, -1:], tt["out_norm"]).to(self.dtype)
        logits = (xo @ tt["head"].t()).float()
        return logits if all_logits else logits[:, 0]

    @torch.no_grad()
    def generate(self, prompt: Sequence[int], max_new_tokens: int = 16, chunk: int = 512) -> List[int]:
        self.reset(1, len(prompt) + max_new_tokens + 1)
        ids = torch.tensor([list(prompt)])
        logits = None
        for i in range(0, ids.shape[1], chunk):
            logits = self.forward(ids[:, i: i + chunk])
        out = []
        for _ in range(max_new_tokens):
            out.append(int(logits[0].argmax()))
            logits = self.forward(torch.tensor([[out[-1]]]))
        return out


# ---------------------------------------------------------------------------------------------------- checkpoints
# tensor names of the MiniMax-M3 checkpoints, as the reference's loader reads them (common/m3_impl.h:463-560): per layer under
# "language_model.model.layers.<l>.", experts under ".block_sparse_moe.experts.<e>."
_HF_LAYER = {"input_norm": "input_layernorm.weight", "post_norm": "post_attention_layernorm.weight", "wq": "self_attn.q_proj.weight",
             "wk": "self_attn.k_proj.weight", "wv": "self_attn.v_proj.weight", "wo": "self_attn.o_proj.weight", "q_norm": "self_attn.q_norm.weight",
             "k_norm": "self_attn.k_norm.weight", "idx_wq": "self_attn.index_q_proj.weight", "idx_wk": "self_attn.index_k_proj.weight",
             "idx_q_norm": "self_attn.index_q_norm.weight", "idx_k_norm": "self_attn.index_k_norm.weight", "gate": "block_sparse_moe.gate.weight",
             "gate_bias": "block_sparse_moe.e_score_correction_bias", "sh_w1": "block_sparse_moe.shared_experts.gate_proj.weight",
             "sh_w3": "block_sparse_moe.shared_experts.up_proj.weight", "sh_w2": "block_sparse_moe.shared_experts.down_proj.weight",
             "ff_gate": "mlp.gate_proj.weight", "ff_up": "mlp.up_proj.weight", "ff_down": "mlp.down_proj.weight"}
_HF_EXPERT = {"ex_w1": "w1.weight", "ex_w3": "w3.weight", "ex_w2": "w2.weight"}
_HF_GLOBAL = {"embed": "language_model.model.embed_tokens.weight", "head": "language_model.lm_head.weight", "out_norm": "language_model.model.norm.weight"}
_HF_PREFIX, _HF_EXPERTS = "language_model.model.layers.{l}.", "block_sparse_moe.experts.{e}."


def checkpoint_names(tensors: Dict[str, torch.Tensor], layer: Dict[str, str], expert: Dict[str, str], glob: Dict[str, str], prefix: str,
                     experts: str) -> Dict[str, torch.Tensor]:
    """Our tensor dictionary under checkpoint names (stacked expert tensors become one entry per expert)."""
    out: Dict[str, torch.Tensor] = {}
    for k, v in tensors.items():
        if k in glob:
            out[glob[k]] = v
            continue
        li, key = int(k[1:k.index(".")]), k[k.index(".") + 1:]
        if key in expert:
            for e in range(v.shape[0]):
                out[prefix.format(l=li) + experts.format(e=e) + expert[key]] = v[e]
        else:
            out[prefix.format(l=li) + layer[key]] = v
    return out


def read_checkpoint(path: str, shapes: Dict[str, torch.Tensor], layer, expert, glob, prefix, experts) -> Dict[str, torch.Tensor]:
    """The tensors named by ``shapes`` (a dictionary of the wanted names, e.g. ``random_tensors(cfg)``) from an HF safetensors
    directory: bf16 as stored; FP8 with E8M0 or 128 x 128 fp32 block scales and MXFP4 dequantised (``loader.SafetensorsSource``)."""
    from .loader import SafetensorsSource
    src = SafetensorsSource(path)
    out: Dict[str, torch.Tensor] = {}
    for k, like in shapes.items():
        if k in glob:
            t = src._raw(glob[k])
        else:
            li, key = int(k[1:k.index(".")]), k[k.index(".") + 1:]
            if key in expert:
                t = torch.stack([src._raw(prefix.format(l=li) + experts.format(e=e) + expert[key]) for e in range(like.shape[0])])
            else:
                name = prefix.format(l=li) + layer[key]
                if name not in src.where:
                    continue                                    # optional tensors (a checkpoint without an indexer norm, ...)
                t = src._raw(name)
        if tuple(t.shape) != tuple(like.shape):
            raise ValueError(f"{k}: checkpoint has shape {tuple(t.shape)}, the configuration wants {tuple(like.shape)}")
        out[k] = t.to(like.dtype, copy=True)            # a copy: the file's mapping goes away with ``src``
    return out


def save_checkpoint(cfg: M3Config, tensors: Dict[str, torch.Tensor], path: str) -> None:
    """An HF-layout directory (``model.safetensors`` + ``config.json`` holding the fields of ``M3Config``)."""
    import dataclasses
    import json
    import os
    from .loader import save_safetensors
    os.makedirs(path, exist_ok=True)
    save_safetensors(checkpoint_names(tensors, _HF_LAYER, _HF_EXPERT, _HF_GLOBAL, _HF_PREFIX, _HF_EXPERTS), os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump({"model_type": "minimax_m3", "gemm_b200": dataclasses.asdict(cfg)}, fh)


def load_checkpoint(path: str, device="cpu", dtype=torch.float32, cfg: Optional[M3Config] = None, **kw) -> "M3Model":
    import json
    import os
    if cfg is None:
        with open(os.path.join(path, "config.json")) as fh:
            cfg = M3Config(**json.load(fh)["gemm_b200"])
    wanted = {k: torch.empty(v.shape, dtype=v.dtype, device="meta") for k, v in _shapes(cfg).items()}
    t = read_checkpoint(path, wanted, _HF_LAYER, _HF_EXPERT, _HF_GLOBAL, _HF_PREFIX, _HF_EXPERTS)
    return M3Model(cfg, t, device, dtype, **kw)


def _shapes(cfg: M3Config) -> Dict[str, torch.Tensor]:
    """Names, shapes and dtypes of a checkpoint of ``cfg`` without allocating it."""
    with torch.device("meta"):
        h, qd, kvd, hd = cfg.hidden, cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim, cfg.head_dim
        bf = lambda *s: torch.empty(*s, dtype=torch.bfloat16)
        f32 = lambda *s: torch.empty(*s, dtype=torch.float32)
        t = {"embed": bf(cfg.vocab, h), "head": bf(cfg.vocab, h), "out_norm": bf(h)}
        for li in range(cfg.n_layers):
            p = f"l{li}."
            t.update({p + "input_norm": bf(h), p + "post_norm": bf(h), p + "wq": bf(qd, h), p + "wk": bf(kvd, h), p + "wv": bf(kvd, h),
                      p + "wo": bf(h, qd), p + "q_norm": bf(hd), p + "k_norm": bf(hd)})
            if cfg.is_moe(li):
                iqd, idim, e, it = cfg.msa_n_index_heads * cfg.msa_index_dim, cfg.msa_index_dim, cfg.n_experts, cfg.moe_inter
                t.update({p + "idx_wq": bf(iqd, h), p + "idx_wk": bf(idim, h), p + "idx_q_norm": bf(idim), p + "idx_k_norm": bf(idim),
                          p + "gate": f32(e, h), p + "gate_bias": f32(e), p + "sh_w1": bf(it, h), p + "sh_w3": bf(it, h), p + "sh_w2": bf(h, it),
                          p + "ex_w1": bf(e, it, h), p + "ex_w3": bf(e, it, h), p + "ex_w2": bf(e, h, it)})
            else:
                t.update({p + "ff_gate": bf(cfg.dense_inter, h), p + "ff_up": bf(cfg.dense_inter, h), p + "ff_down": bf(h, cfg.dense_inter)})
    return t
