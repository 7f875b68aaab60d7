"""DeepSeek-V4-Flash style engine as a PyTorch-op forward pass (CPU or CUDA), after the "exact" mode of the reference's harness
(common/ds4f.h:60-135 configuration; common/ds4f_impl.h:4781-5018 one token through the stack; :3916-4110 hyper-connections;
:3426-3470 attention; :3691-3708 router; :872-925 RoPE / YaRN tables).  What sets it apart from the other engines here:

* **hyper-connections (mHC)**: the residual is ``hc_mult`` streams ``[hc, hidden]``.  In front of attention and of the FFN the
  streams are collapsed with weights ``pre`` (``y = sum_k pre_k x_k``); behind, the block output is spread back with ``post`` and the
  old streams are mixed with a ``hc x hc`` matrix ``comb``: ``x_k = post_k f + sum_j comb[j, k] old_j``.  ``pre, post, comb`` come
  from one small fp32 projection of the flattened streams (scaled by their RMS), sigmoids, and a Sinkhorn normalisation of ``comb``
  (softmax over rows, then ``hc_iters`` rounds of column / row normalisation).  The head collapses the streams with sigmoid
  weights (no Sinkhorn);
* **attention** is multi-query over ONE latent row per position that serves as key and value (``kv_lora == q_head_dim``): queries
  ``wq_b norm(wq_a x)`` are RMS-normalised per head without a weight, the last ``qk_rope_dim`` features of queries and of the latent
  are rotated (interleaved pairs); a token attends the last ``window_size`` positions plus a learned per-head **sink** logit that only
  enters the softmax denominator; the rope features of the output are rotated back by the query position;
* the output projection is block-diagonal: the heads are cut into ``o_groups`` groups, group g goes through its own
  ``[o_lora, heads * head_dim / o_groups]`` slice of ``wo_a``, then ``wo_b`` maps ``o_groups * o_lora`` to hidden;
* router: ``score = sqrt(softplus(logit))``, experts picked by ``score + bias``, weights ``score / sum * routed_scale``; SwiGLU with
  the gate clamped from above and the up branch clamped on both sides by ``swiglu_limit``; shared expert always added;
* layers with a non-zero compression ratio use the YaRN-scaled RoPE table with ``compress_rope_theta``, the others the plain one.

Not built: the KV compressor / lightning indexer of those layers (the reference's ``DS4F_TIERB2`` path; here every layer attends its
sliding window, which is what the reference's exact mode does without that switch), token-id ("hash") routing of the first layers,
the MTP head.  The reference's implementation is written against Arm SVE intrinsics without a scalar fallback and does not compile
on this machine, so unlike the other engines this one is tested against its own properties only (tests/test_ds4f_cpu.py).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from . import m3


@dataclass
class DS4FConfig:
    n_layers: int = 43
    hidden: int = 4096
    vocab: int = 129280
    n_heads: int = 64
    q_head_dim: int = 512
    qk_rope_dim: int = 64
    q_lora: int = 1024
    kv_lora: int = 512
    o_groups: int = 8
    o_lora: int = 1024
    n_experts: int = 256
    n_active: int = 6
    moe_inter: int = 2048
    shared_inter: int = 2048
    routed_scale: float = 1.5
    hc_mult: int = 4
    hc_iters: int = 20
    hc_eps: float = 1e-6
    norm_eps: float = 1e-6
    window_size: int = 128
    swiglu_limit: float = 10.0
    rope_theta: float = 1e4
    compress_rope_theta: float = 1.6e5
    rope_factor: int = 16
    beta_fast: int = 32
    beta_slow: int = 1
    original_seq_len: int = 65536
    compress_ratios: List[int] = field(default_factory=list)      # per layer; non-zero selects the YaRN table
    max_pos: int = 4096

    def __post_init__(self):
        if self.kv_lora != self.q_head_dim:
            raise ValueError("the latent row is key and value of every head: kv_lora must equal q_head_dim")
        if not self.compress_ratios:
            self.compress_ratios = [0, 0] + [4 if i % 2 == 0 else 128 for i in range(max(self.n_layers - 2, 0))]

    @property
    def o_inter(self) -> int:
        return self.o_groups * self.o_lora

    # names the shared cache code of the M3 base reads
    def is_moe(self, li: int) -> bool:
        return False

    @property
    def rotary_dim(self) -> int:
        return self.qk_rope_dim


def rope_freqs(dim: int, base: float, factor: int = 1, beta_fast: int = 32, beta_slow: int = 1, original_seq_len: int = 0) -> torch.Tensor:
    """Rotation frequencies ``base^(-2k / dim)``; with ``original_seq_len > 0`` the YaRN ramp: frequencies below the ``beta_slow``
    correction dimension are divided by ``factor``, those above ``beta_fast`` stay, linear in between."""
    k = torch.arange(dim // 2, dtype=torch.float64)
    freq = 1.0 / base ** (2.0 * k / dim)
    if original_seq_len > 0:
        lo = dim * math.log(original_seq_len / (beta_fast * 2.0 * math.pi)) / (2.0 * math.log(base))
        hi = dim * math.log(original_seq_len / (beta_slow * 2.0 * math.pi)) / (2.0 * math.log(base))
        low, high = max(math.floor(lo), 0), min(math.ceil(hi), dim - 1)
        if low == high:
            high += 0.001
        smooth = 1.0 - ((k - low) / (high - low)).clamp(0.0, 1.0)
        freq = freq / factor * (1.0 - smooth) + freq * smooth
    return freq


def sinkhorn(mixes: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, hc: int, iters: int, eps: float):
    """``mixes`` [..., (2 + hc) * hc] -> ``pre`` [..., hc], ``post`` [..., hc], ``comb`` [..., hc, hc]."""
    pre = torch.sigmoid(mixes[..., :hc] * scale[0] + base[:hc]) + eps
    post = 2.0 * torch.sigmoid(mixes[..., hc: 2 * hc] * scale[1] + base[hc: 2 * hc])
    comb = (mixes[..., 2 * hc:] * scale[2] + base[2 * hc:]).reshape(*mixes.shape[:-1], hc, hc)
    comb = torch.softmax(comb, dim=-1) + eps
    comb = comb / (comb.sum(-2, keepdim=True) + eps)
    for _ in range(iters - 1):
        comb = comb / (comb.sum(-1, keepdim=True) + eps)
        comb = comb / (comb.sum(-2, keepdim=True) + eps)
    return pre, post, comb


def random_tensors(cfg: DS4FConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    u = lambda amp, *s: ((torch.rand(*s, generator=g) * 2 - 1) * amp)
    bf = lambda amp, *s: u(amp, *s).to(torch.bfloat16)
    nw = lambda n: (1.0 + u(0.1, n)).to(torch.bfloat16)
    c, nh, hd, hc = cfg.hidden, cfg.n_heads, cfg.q_head_dim, cfg.hc_mult
    mix, gin = (2 + hc) * hc, nh * hd // cfg.o_groups
    t = {"embed": bf(0.5, cfg.vocab, c), "head": bf(0.05, cfg.vocab, c), "out_norm": nw(c), "hc_head_fn": u(0.05, hc, hc * c),
         "hc_head_base": u(0.5, hc), "hc_head_scale": 1.0 + u(0.2, 1)}
    for li in range(cfg.n_layers):
        p = f"l{li}."
        t.update({p + "attn_norm": nw(c), p + "ffn_norm": nw(c), p + "q_norm": nw(cfg.q_lora), p + "kv_norm": nw(cfg.kv_lora),
                  p + "wq_a": bf(0.08, cfg.q_lora, c), p + "wq_b": bf(0.08, nh * hd, cfg.q_lora), p + "wkv": bf(0.08, cfg.kv_lora, c),
                  p + "wo_a": bf(0.08, cfg.o_inter, gin), p + "wo_b": bf(0.08, c, cfg.o_inter), p + "attn_sink": u(1.0, nh) - 2.0,
                  p + "gate": bf(0.1, cfg.n_experts, c), p + "gate_bias": u(0.1, cfg.n_experts), p + "sh_w1": bf(0.08, cfg.shared_inter, c),
                  p + "sh_w3": bf(0.08, cfg.shared_inter, c), p + "sh_w2": bf(0.08, c, cfg.shared_inter),
                  p + "ex_w1": bf(0.08, cfg.n_experts, cfg.moe_inter, c), p + "ex_w3": bf(0.08, cfg.n_experts, cfg.moe_inter, c),
                  p + "ex_w2": bf(0.08, cfg.n_experts, c, cfg.moe_inter)})
        for blk in ("attn", "ffn"):
            t.update({p + f"hc_{blk}_fn": u(0.05, mix, hc * c), p + f"hc_{blk}_base": u(0.5, mix), p + f"hc_{blk}_scale": 1.0 + u(0.2, 3)})
    return t


class DS4FModel(m3.M3Model):
    def __init__(self, cfg: DS4FConfig, tensors: Dict[str, torch.Tensor], device="cpu", dtype=torch.float32, ep_rank: int = 0, ep_size: int = 1,
                 group=None):
        super().__init__(cfg, tensors, device, dtype, ep_rank, ep_size, group, int4_kv=False, msa=False)
        for k, v in tensors.items():                                    # the hyper-connection parameters and sinks stay fp32
            if ".hc_" in k or k.startswith("hc_") or k.endswith("attn_sink"):
                self.t[k] = v.to(self.device, torch.float32)
        rd = cfg.qk_rope_dim
        self.freq_dense = rope_freqs(rd, cfg.rope_theta).to(self.device)
        self.freq_comp = rope_freqs(rd, cfg.compress_rope_theta, cfg.rope_factor, cfg.beta_fast, cfg.beta_slow, cfg.original_seq_len).to(self.device)

    def reset(self, batch: int = 1, max_pos: Optional[int] = None) -> None:
        cfg = self.cfg
        n = max_pos or cfg.max_pos
        self.pos, self.batch = 0, batch
        self.cache = [{"kv": torch.zeros(batch, n, 1, cfg.kv_lora, dtype=torch.bfloat16, device=self.device)} for _ in range(cfg.n_layers)]

    # ------------------------------------------------------------------------------------------ pieces
    def _norm(self, x: torch.Tensor, w: Optional[torch.Tensor]) -> torch.Tensor:
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.norm_eps)
        return (y * w.float() if w is not None else y).to(x.dtype)

    def _rot(self, x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, inverse: bool = False) -> torch.Tensor:
        """Rotate the last ``qk_rope_dim`` features of ``x`` [B, T, H, D] (interleaved pairs) by the positions; ``inverse`` turns back."""
        rd = self.cfg.qk_rope_dim
        ang = positions.double()[:, None] * freq[None, :]
        cos, sin = ang.cos().float()[None, :, None, :], ang.sin().float()[None, :, None, :]
        if inverse:
            sin = -sin
        tail = x[..., -rd:].float()
        a, b = tail[..., 0::2], tail[..., 1::2]
        rot = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)
        return torch.cat([x[..., :-rd].float(), rot], dim=-1).to(x.dtype)

    def _hc_pre(self, x4: torch.Tensor, prefix: str):
        cfg, tt = self.cfg, self.t
        flat = x4.reshape(*x4.shape[:2], -1).float()
        rsq = torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + cfg.norm_eps)
        mixes = (flat @ tt[prefix + "_fn"].t()) * rsq
        pre, post, comb = sinkhorn(mixes, tt[prefix + "_scale"], tt[prefix + "_base"], cfg.hc_mult, cfg.hc_iters, cfg.hc_eps)
        return (pre[..., None] * x4).sum(2), post, comb

    @staticmethod
    def _hc_post(resid: torch.Tensor, f: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
        """``x_k = post_k f + sum_j comb[j, k] resid_j``."""
        return post[..., None] * f[:, :, None, :] + torch.einsum("btjk,btjd->btkd", comb, resid)

    def _swiglu(self, g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
        lim = self.cfg.swiglu_limit
        gf = g.float().clamp(max=lim)
        return (gf * torch.sigmoid(gf) * u.float().clamp(-lim, lim)).to(g.dtype)

    def _moe(self, li: int, h2: torch.Tensor) -> torch.Tensor:
        cfg, tt, p = self.cfg, self.t, f"l{li}."
        b, t, h = h2.shape
        x = h2.reshape(b * t, h)
        score = torch.sqrt(torch.nn.functional.softplus(x.float() @ tt[p + "gate"].t()))          # the router runs in fp32
        key = score + tt[p + "gate_bias"][None, :] if (p + "gate_bias") in tt else score
        pick = torch.topk(key, cfg.n_active, dim=-1).indices
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
            route.index_add_(0, rows, (act @ tt[p + "ex_w2"][slot].t()).float() * (w * hit)[rows].sum(-1, keepdim=True))
        if self.ep_size > 1 and self.group is not None:
            import torch.distributed as dist
            dist.all_reduce(route, group=self.group)
        sh = self._swiglu(x @ tt[p + "sh_w1"].t(), x @ tt[p + "sh_w3"].t()) @ tt[p + "sh_w2"].t()
        return (route + sh.float()).reshape(b, t, h)

    # ------------------------------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, ids: torch.Tensor, all_logits: bool = False) -> torch.Tensor:
        cfg, tt = self.cfg, self.t
        ids = ids.to(self.device).long()
        b, t = ids.shape
        if not self.cache or b != self.batch:
            self.reset(b)
        p0 = self.pos
        n = p0 + t
        positions = torch.arange(p0, n, device=self.device)
        kpos = torch.arange(n, device=self.device)
        mask = (kpos[None, :] <= positions[:, None]) & (kpos[None, :] > positions[:, None] - cfg.window_size)      # [T, n]
        nh, hd, og = cfg.n_heads, cfg.q_head_dim, cfg.o_groups
        x4 = tt["embed"][ids].float()[:, :, None, :].expand(b, t, cfg.hc_mult, cfg.hidden).contiguous()
        for li in range(cfg.n_layers):
            p, c = f"l{li}.", self.cache[li]
            freq = self.freq_comp if cfg.compress_ratios[li] else self.freq_dense
            y, post, comb = self._hc_pre(x4, p + "hc_attn")
            hn = self._norm(y, tt[p + "attn_norm"]).to(self.dtype)
            q_lat = self._norm(hn @ tt[p + "wq_a"].t(), tt[p + "q_norm"])
            q = self._rot(self._norm((q_lat @ tt[p + "wq_b"].t()).reshape(b, t, nh, hd), None), positions, freq)
            lat = self._rot(self._norm(hn @ tt[p + "wkv"].t(), tt[p + "kv_norm"]).reshape(b, t, 1, hd), positions, freq)
            self._store(c, "kv", lat, p0)
            rows = self._load(c, "kv", n)[:, :, 0]                                              # [B, n, D]: key and value of every head
            sc = torch.einsum("bqhd,bnd->bhqn", q.float(), rows) / math.sqrt(hd)
            sc = sc.masked_fill(~mask[None, None], float("-inf"))
            sink = tt[p + "attn_sink"][None, :, None, None].expand(b, nh, t, 1)
            w = torch.softmax(torch.cat([sc, sink], dim=-1), dim=-1)[..., :-1]                  # the sink takes its share and gives nothing
            a = self._rot(torch.einsum("bhqn,bnd->bqhd", w, rows), positions, freq, inverse=True)
            a = a.reshape(b, t, og, nh * hd // og).to(self.dtype)
            o1 = torch.einsum("btgi,goi->btgo", a, tt[p + "wo_a"].reshape(og, cfg.o_lora, -1)).reshape(b, t, cfg.o_inter)
            x4 = self._hc_post(x4, (o1 @ tt[p + "wo_b"].t()).float(), post, comb)
            y, post, comb = self._hc_pre(x4, p + "hc_ffn")
            h2 = self._norm(y, tt[p + "ffn_norm"]).to(self.dtype)
            x4 = self._hc_post(x4, self._moe(li, h2), post, comb)
        self.pos = n
        xs = x4 if all_logits else x4[:, -1:]
        flat = xs.reshape(*xs.shape[:2], -1)
        rsq = torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + cfg.norm_eps)
        pre = torch.sigmoid((flat @ tt["hc_head_fn"].t()) * rsq * tt["hc_head_scale"][0] + tt["hc_head_base"]) + cfg.hc_eps
        y = (pre[..., None] * xs).sum(2)
        logits = (self._norm(y, tt["out_norm"]).to(self.dtype) @ tt["head"].t()).float()
        return logits if all_logits else logits[:, 0]
