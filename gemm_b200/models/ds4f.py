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

* ``tierb2`` (the reference's ``DS4F_TIERB2`` switch, common/ds4f_impl.h:3613-3670): layers with a non-zero ratio also attend
  **compressed latents** in the same softmax.  A ``Compressor`` pools every ``ratio`` positions of the layer input into one latent
  (gated, a softmax per feature; ratio 4 overlaps two windows); layers with ratio 4 pick the ``index_topk`` best latents per query with
  the **lightning indexer** (its own compressor for the keys, Hadamard-rotated FP4-rounded queries and keys,
  ``sum_h relu(q_h . k) w_h``), the others attend all finished latents;
* with ``tid2eid`` tables the first ``n_hash_layers`` layers take a token's experts from its id; ``mtp``: the next-token block
  (``mtp_predict``) and self-speculative greedy decoding with it (``generate(..., use_mtp=True)``).

The reference's implementation is written against Arm SVE intrinsics and its matrix kernels live outside its common/ tree, so the
engine as a whole does not run on this machine.  Its scalar building blocks do compile (with a stand-in SVE header): the
compressor, the indexer step, top-k, the gathered attention with sinks, the Hadamard rotation and the FP4 rounding are checked
against them (tests/test_ds4f_tierb2_cpu.py); the rest is checked against a scalar restatement of the reference's formulas and
against its own properties (tests/test_ds4f_cpu.py).  Not built: the int8 / int4 forms of the caches.
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
    tierb2: bool = False              # layers with a non-zero ratio also attend compressed latents (compressor + indexer)
    index_n_heads: int = 64
    index_head_dim: int = 128
    index_topk: int = 512
    n_hash_layers: int = 0            # the first layers pick their experts from a token-id table when the checkpoint has one
    mtp: bool = False                 # tensors of the next-token (MTP) block are present

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


def hadamard(x: torch.Tensor) -> torch.Tensor:
    """Sylvester Walsh-Hadamard transform of the last axis (a power of two) times ``n^-0.5``, butterflies in the order of the
    reference's loop (common/ds4f_impl.h:991-998) so that fp32 results agree bit for bit."""
    n = x.shape[-1]
    if n & (n - 1):
        raise ValueError("the Hadamard rotation needs a power-of-two width")
    y, h = x.float(), 1
    while h < n:
        y = y.reshape(*x.shape[:-1], n // (2 * h), 2, h)
        y = torch.stack([y[..., 0, :] + y[..., 1, :], y[..., 0, :] - y[..., 1, :]], dim=-2).reshape(*x.shape)
        h *= 2
    return y * (1.0 / math.sqrt(n))


_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def fp4_act_quant(x: torch.Tensor, block: int = 32) -> torch.Tensor:
    """Quantise-dequantise to FP4 (e2m1) in blocks of ``block`` along the last axis with a power-of-two scale
    ``2^ceil(log2(amax / 6))``, round-to-nearest with ties to the even code, result rounded to bf16
    (common/ds4f_impl.h:947-989)."""
    shp = x.shape
    xb = x.float().reshape(*shp[:-1], shp[-1] // block, block)
    amax = xb.abs().amax(-1, keepdim=True).clamp_min(6.0 * 1.1754944e-38)
    m, e = torch.frexp(amax * torch.tensor(1.0 / 6.0, dtype=torch.float32, device=x.device))     # t = m * 2^e, m in [0.5, 1)
    scale = torch.ldexp(torch.ones_like(m), torch.where(m == 0.5, e - 1, e))
    a = (xb / scale).clamp(-6.0, 6.0)
    grid = torch.tensor(_E2M1, dtype=torch.float32, device=x.device)
    dist = (a.abs()[..., None] - grid).abs()
    even = torch.tensor([1, 0, 1, 0, 1, 0, 1, 0], dtype=torch.bool, device=x.device)
    best = dist.amin(-1, keepdim=True)
    key = torch.where(dist == best, torch.where(even, 0, 1), 2)                                   # among the nearest: the even code
    snapped = grid[key.argmin(-1)] * torch.where(a < 0, -1.0, 1.0)
    return (snapped * scale).to(torch.bfloat16).float().reshape(shp)


def index_scores(q: torch.Tensor, kv: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """Lightning-indexer score of compressed slot t for a query: ``sum_h relu(q_h . kv_t) * weights_h``
    (common/ds4f_impl.h:1366-1386).  ``q`` [..., H, D], ``kv`` [..., T, D], ``weights`` [..., H] -> [..., T]."""
    return torch.einsum("...ht,...h->...t", torch.relu(torch.einsum("...hd,...td->...ht", q.float(), kv.float())), weights.float())


def index_topk(score: torch.Tensor, valid: torch.Tensor, k: int) -> torch.Tensor:
    """Boolean selection of the ``min(k, valid.sum())`` best slots among ``valid`` per row, ties to the lower slot
    (common/ds4f_impl.h:1396-1464)."""
    masked = score.masked_fill(~valid, float("-inf"))
    order = torch.sort(masked, dim=-1, descending=True, stable=True).indices
    rank = torch.empty_like(order)
    rank.scatter_(-1, order, torch.arange(score.shape[-1], device=score.device).expand_as(order))
    return valid & (rank < k)


class Compressor:
    """Stateful gated pooling of ``ratio`` consecutive positions into one latent of width ``d`` (common/ds4f_impl.h:1081-1138 for
    a whole prompt, :1484-1554 one token at a time; both give the same latents).  Two projections of the layer input give, per
    position, values and gate scores of width ``W``; the score gets a bias per position-in-window (``ape``).  ``ratio == 4``
    overlaps: ``W = 2 d``, latent w pools the first halves of window w - 1 and the second halves of window w (8 rows; for w = 0 the
    missing rows weigh nothing); otherwise ``W = d`` and latent w pools its own ``ratio`` rows.  The weights are a softmax over
    the pooled rows PER FEATURE.  Then RMSNorm, rotation of the last ``rd`` features by the window's first position, and for the
    indexer's compressor (``rotate``) a Hadamard rotation and FP4 rounding.  Rows of the unfinished window (and of the one before
    it when overlapping) are kept between calls."""

    def __init__(self, wkv, wgate, ape, norm_w, d: int, ratio: int, rd: int, eps: float, rotate: bool):
        self.wkv, self.wgate, self.ape, self.norm_w = wkv, wgate, ape.float(), norm_w
        self.d, self.ratio, self.rd, self.eps, self.rotate = d, ratio, rd, eps, rotate
        self.overlap = ratio == 4
        self.reset(1)

    def reset(self, batch: int) -> None:
        w = (2 if self.overlap else 1) * self.d
        dev = self.wkv.device
        self.rows_kv = torch.zeros(batch, 0, w, device=dev)
        self.rows_sc = torch.zeros(batch, 0, w, device=dev)
        self.first = 0                                   # absolute position of row 0 of the kept rows
        self.out = torch.zeros(batch, 0, self.d, device=dev)

    def snapshot(self):
        return (self.rows_kv.clone(), self.rows_sc.clone(), self.first, self.out.shape[1])

    def restore(self, snap) -> None:
        self.rows_kv, self.rows_sc, self.first, n = snap[0].clone(), snap[1].clone(), snap[2], snap[3]
        self.out = self.out[:, :n]

    def step(self, hn: torch.Tensor, p0: int, rot) -> int:
        """Feed positions ``p0 .. p0 + T - 1`` (``hn`` [B, T, hidden]); ``rot(x [B, n, 1, d], positions)`` rotates the rope features.
        Returns the number of latents so far."""
        b, t, _ = hn.shape
        ratio, d = self.ratio, self.d
        x = hn.float()
        pos = torch.arange(p0, p0 + t, device=x.device)
        self.rows_kv = torch.cat([self.rows_kv, x @ self.wkv.float().t()], 1)
        self.rows_sc = torch.cat([self.rows_sc, x @ self.wgate.float().t() + self.ape[pos % ratio][None]], 1)
        done, total = self.out.shape[1], (p0 + t) // ratio
        if total > done:
            wins = torch.arange(done, total, device=x.device)
            cur = (wins * ratio - self.first)[:, None] + torch.arange(ratio, device=x.device)[None]           # [nw, ratio] row numbers
            if self.overlap:
                prev = cur - ratio
                ok = (wins > 0)[None, :, None, None]
                pk = self.rows_kv[:, prev.clamp_min(0), :d] * ok
                ps = self.rows_sc[:, prev.clamp_min(0), :d].masked_fill(~ok, float("-inf"))
                kk = torch.cat([pk, self.rows_kv[:, cur, d:]], 2)                                             # [B, nw, 2 ratio, d]
                ss = torch.cat([ps, self.rows_sc[:, cur, d:]], 2)
            else:
                kk, ss = self.rows_kv[:, cur], self.rows_sc[:, cur]
            lat = (kk * torch.softmax(ss, dim=2)).sum(2)                                                      # [B, nw, d]
            lat = lat * torch.rsqrt(lat.double().pow(2).mean(-1, keepdim=True).float() + self.eps) * self.norm_w.float()
            lat = rot(lat[:, :, None, :], wins * ratio)[:, :, 0]
            if self.rotate:
                lat = fp4_act_quant(hadamard(lat))
            self.out = torch.cat([self.out, lat], 1)
        keep = max(self.first, (total - (1 if self.overlap else 0)) * ratio, 0)
        if keep > self.first:
            self.rows_kv, self.rows_sc = self.rows_kv[:, keep - self.first:], self.rows_sc[:, keep - self.first:]
            self.first = keep
        return total


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
        ratio = cfg.compress_ratios[li]
        if cfg.tierb2 and ratio:
            coff = 2 if ratio == 4 else 1
            t.update({p + "cmp_wkv": bf(0.08, coff * cfg.kv_lora, c), p + "cmp_wgate": bf(0.08, coff * cfg.kv_lora, c),
                      p + "cmp_ape": u(1.0, ratio, coff * cfg.kv_lora), p + "cmp_norm": nw(cfg.kv_lora)})
            if ratio == 4:
                hi, ihd = cfg.index_n_heads, cfg.index_head_dim
                t.update({p + "idx_wq_b": bf(0.08, hi * ihd, cfg.q_lora), p + "idx_wproj": bf(0.08, hi, c),
                          p + "idx_cmp_wkv": bf(0.08, 2 * ihd, c), p + "idx_cmp_wgate": bf(0.08, 2 * ihd, c),
                          p + "idx_cmp_ape": u(1.0, 4, 2 * ihd), p + "idx_cmp_norm": nw(ihd)})
        if li < cfg.n_hash_layers:
            t[p + "tid2eid"] = torch.stack([torch.randperm(cfg.n_experts, generator=g)[: cfg.n_active] for _ in range(cfg.vocab)])
            del t[p + "gate_bias"]
    if cfg.mtp:                                                   # one more block (no shared expert) + the fusion and its own head
        p = "mtp."
        t.update({p + "attn_norm": nw(c), p + "ffn_norm": nw(c), p + "q_norm": nw(cfg.q_lora), p + "kv_norm": nw(cfg.kv_lora),
                  p + "wq_a": bf(0.08, cfg.q_lora, c), p + "wq_b": bf(0.08, nh * hd, cfg.q_lora), p + "wkv": bf(0.08, cfg.kv_lora, c),
                  p + "wo_a": bf(0.08, cfg.o_inter, gin), p + "wo_b": bf(0.08, c, cfg.o_inter), p + "attn_sink": u(1.0, nh) - 2.0,
                  p + "gate": bf(0.1, cfg.n_experts, c), p + "gate_bias": u(0.1, cfg.n_experts),
                  p + "ex_w1": bf(0.08, cfg.n_experts, cfg.moe_inter, c), p + "ex_w3": bf(0.08, cfg.n_experts, cfg.moe_inter, c),
                  p + "ex_w2": bf(0.08, cfg.n_experts, c, cfg.moe_inter),
                  p + "enorm": nw(c), p + "hnorm": nw(c), p + "norm": nw(c), p + "e_proj": bf(0.08, c, c), p + "h_proj": bf(0.08, c, c),
                  p + "hc_head_fn": u(0.05, hc, hc * c), p + "hc_head_base": u(0.5, hc), p + "hc_head_scale": 1.0 + u(0.2, 1)})
        for blk in ("attn", "ffn"):
            t.update({p + f"hc_{blk}_fn": u(0.05, mix, hc * c), p + f"hc_{blk}_base": u(0.5, mix), p + f"hc_{blk}_scale": 1.0 + u(0.2, 3)})
    return t


class DS4FModel(m3.M3Model):
    def __init__(self, cfg: DS4FConfig, tensors: Dict[str, torch.Tensor], device="cpu", dtype=torch.float32, ep_rank: int = 0, ep_size: int = 1,
                 group=None):
        super().__init__(cfg, tensors, device, dtype, ep_rank, ep_size, group, int4_kv=False, msa=False)
        for k, v in tensors.items():                                    # the hyper-connection parameters, sinks and score biases stay fp32
            if ".hc_" in k or k.startswith("hc_") or k.endswith("attn_sink") or k.endswith("_ape"):
                self.t[k] = v.to(self.device, torch.float32)
            elif k.endswith("tid2eid"):
                self.t[k] = v.to(self.device, torch.long)
        self.trace: Optional[Dict[str, torch.Tensor]] = None            # set to {} to record a layer's attention inputs (tests)
        self.last_hc: Optional[torch.Tensor] = None                     # streams behind the last block, [B, T, hc, hidden]
        rd = cfg.qk_rope_dim
        self.freq_dense = rope_freqs(rd, cfg.rope_theta).to(self.device)
        self.freq_comp = rope_freqs(rd, cfg.compress_rope_theta, cfg.rope_factor, cfg.beta_fast, cfg.beta_slow, cfg.original_seq_len).to(self.device)

    def reset(self, batch: int = 1, max_pos: Optional[int] = None) -> None:
        cfg = self.cfg
        n = max_pos or cfg.max_pos
        self.pos, self.batch = 0, batch
        self.cache = [{"kv": torch.zeros(batch, n, 1, cfg.kv_lora, dtype=torch.bfloat16, device=self.device)} for _ in range(cfg.n_layers)]
        self.mtp_cache = {"kv": torch.zeros(batch, n, 1, cfg.kv_lora, dtype=torch.bfloat16, device=self.device)} if cfg.mtp else None
        self.comp: Dict[int, Compressor] = {}                           # layer -> compressor of its latents / of the indexer's keys
        self.icomp: Dict[int, Compressor] = {}
        if cfg.tierb2:
            tt = self.t
            for li, ratio in enumerate(cfg.compress_ratios[: cfg.n_layers]):
                p = f"l{li}."
                if not ratio or (p + "cmp_wkv") not in tt:
                    continue
                self.comp[li] = Compressor(tt[p + "cmp_wkv"], tt[p + "cmp_wgate"], tt[p + "cmp_ape"], tt[p + "cmp_norm"], cfg.kv_lora, ratio,
                                           cfg.qk_rope_dim, cfg.norm_eps, rotate=False)
                self.comp[li].reset(batch)
                if ratio == 4:
                    self.icomp[li] = Compressor(tt[p + "idx_cmp_wkv"], tt[p + "idx_cmp_wgate"], tt[p + "idx_cmp_ape"], tt[p + "idx_cmp_norm"],
                                                cfg.index_head_dim, ratio, cfg.qk_rope_dim, cfg.norm_eps, rotate=True)
                    self.icomp[li].reset(batch)

    def snapshot(self):
        """State that a rejected draft position must put back: the position and the compressors' pending rows (the window cache
        heals itself: rows past the position are overwritten before they are read; common/ds4f_impl.h:4676-4705)."""
        return (self.pos, {li: c.snapshot() for li, c in self.comp.items()}, {li: c.snapshot() for li, c in self.icomp.items()})

    def restore(self, snap) -> None:
        self.pos = snap[0]
        for li, sn in snap[1].items():
            self.comp[li].restore(sn)
        for li, sn in snap[2].items():
            self.icomp[li].restore(sn)

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

    def _moe(self, p: str, h2: torch.Tensor, ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Routed experts + shared expert of the block with tensor prefix ``p``.  With a ``tid2eid`` table (the first
        ``n_hash_layers`` layers of the released model) the experts of a token are the table's row for its id and only the
        weights come from the router; the reference leaves that table unread and routes those layers without a bias
        (common/ds4f_impl.h:2285, :3712-3718)."""
        cfg, tt = self.cfg, self.t
        b, t, h = h2.shape
        x = h2.reshape(b * t, h)
        score = torch.sqrt(torch.nn.functional.softplus(x.float() @ tt[p + "gate"].float().t()))  # the router runs in fp32
        if (p + "tid2eid") in tt and ids is not None:
            pick = tt[p + "tid2eid"][ids.reshape(-1)]
        else:
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
        pending = None
        if self.ep_size > 1 and self.group is not None:          # the reduce over the ranks overlaps the shared expert
            import torch.distributed as dist
            pending = dist.all_reduce(route, group=self.group, async_op=True)
        sh = (self._swiglu(x @ tt[p + "sh_w1"].t(), x @ tt[p + "sh_w3"].t()) @ tt[p + "sh_w2"].t()).float() if (p + "sh_w1") in tt else None
        if pending is not None:
            pending.wait()
        if sh is not None:
            route = route + sh
        return route.reshape(b, t, h)

    # ------------------------------------------------------------------------------------------ forward
    def _compressed_term(self, li: int, hn: torch.Tensor, q_lat: torch.Tensor, positions: torch.Tensor, p0: int, freq: torch.Tensor):
        """Latents of the layer's compressor so far ``[B, S, D]`` and which of them each query of this call attends ``[B, T, S]``
        (common/ds4f_impl.h:3613-3670).  A query at position s may see slot t once its window is complete, ``t < (s + 1) // ratio``;
        layers with ratio 4 keep the ``index_topk`` best of those by the indexer's score (its own compressor makes the keys, its
        queries come from the query latent, both Hadamard-rotated and rounded to FP4), the other layers keep all of them."""
        cfg, tt, p = self.cfg, self.t, f"l{li}."
        ratio = cfg.compress_ratios[li]
        rot = lambda x, pos: self._rot(x, pos, freq)
        comp = self.comp[li]
        comp.step(hn, p0, rot)
        lat = comp.out
        slots = torch.arange(lat.shape[1], device=self.device)
        allowed = (slots[None, :] < ((positions + 1) // ratio)[:, None])[None].expand(hn.shape[0], -1, -1)        # [B, T, S]
        if li not in self.icomp:
            return lat, allowed
        b, t, _ = hn.shape
        hi, ihd = cfg.index_n_heads, cfg.index_head_dim
        self.icomp[li].step(hn, p0, rot)
        keys = self.icomp[li].out                                                                                # [B, S, ihd]
        qi = (q_lat.float() @ tt[p + "idx_wq_b"].float().t()).reshape(b, t, hi, ihd)
        qi = fp4_act_quant(hadamard(self._rot(qi, positions, freq)))
        wts = (hn.float() @ tt[p + "idx_wproj"].float().t()) * (ihd ** -0.5 * hi ** -0.5)                        # [B, T, Hi]
        score = index_scores(qi, keys[:, None], wts)                                                             # [B, T, S]
        if self.trace is not None and self.trace.get("layer") == li:
            self.trace.update(idx_score=score.clone(), idx_keys=keys.clone())
        return lat, index_topk(score, allowed, cfg.index_topk)

    def _block(self, p: str, li: Optional[int], x4: torch.Tensor, cache, positions: torch.Tensor, p0: int, freq: torch.Tensor,
               ids: Optional[torch.Tensor]) -> torch.Tensor:
        """One block on the streams ``x4`` [B, T, hc, hidden]: attention and expert FFN, each between a collapse and a spread of the
        streams.  ``li`` None: the MTP block (no compressed term)."""
        cfg, tt = self.cfg, self.t
        b, t = x4.shape[:2]
        n = p0 + t
        nh, hd, og = cfg.n_heads, cfg.q_head_dim, cfg.o_groups
        kpos = torch.arange(n, device=self.device)
        mask = (kpos[None, :] <= positions[:, None]) & (kpos[None, :] > positions[:, None] - cfg.window_size)      # [T, n]
        y, post, comb = self._hc_pre(x4, p + "hc_attn")
        hn = self._norm(y, tt[p + "attn_norm"]).to(self.dtype)
        q_lat = self._norm(hn @ tt[p + "wq_a"].t(), tt[p + "q_norm"])
        q = self._rot(self._norm((q_lat @ tt[p + "wq_b"].t()).reshape(b, t, nh, hd), None), positions, freq)
        lat = self._rot(self._norm(hn @ tt[p + "wkv"].t(), tt[p + "kv_norm"]).reshape(b, t, 1, hd), positions, freq)
        self._store(cache, "kv", lat, p0)
        rows = self._load(cache, "kv", n)[:, :, 0]                                              # [B, n, D]: key and value of every head
        sc = torch.einsum("bqhd,bnd->bhqn", q.float(), rows) / math.sqrt(hd)
        sc = sc.masked_fill(~mask[None, None], float("-inf"))
        parts, values = [sc], [rows]
        if li is not None and li in self.comp:
            clat, pick = self._compressed_term(li, hn, q_lat, positions, p0, freq)
            csc = torch.einsum("bqhd,bsd->bhqs", q.float(), clat) / math.sqrt(hd)
            parts.append(csc.masked_fill(~pick[:, None], float("-inf")))
            values.append(clat)
            if self.trace is not None and self.trace.get("layer") == li:
                self.trace.update(hn=hn.float().clone(), q_lat=q_lat.float().clone(), q=q.float().clone(), rows=rows.float().clone(),
                                  cmp=clat.clone(), pick=pick.clone())
        parts.append(tt[p + "attn_sink"][None, :, None, None].expand(b, nh, t, 1))
        w = torch.softmax(torch.cat(parts, dim=-1), dim=-1)[..., :-1]                           # the sink takes its share and gives nothing
        a = torch.einsum("bhqn,bnd->bqhd", w, torch.cat(values, dim=1))
        if self.trace is not None and self.trace.get("layer") == li:
            self.trace["attn"] = a.clone()
        a = self._rot(a, positions, freq, inverse=True)
        a = a.reshape(b, t, og, nh * hd // og).to(self.dtype)
        o1 = torch.einsum("btgi,goi->btgo", a, tt[p + "wo_a"].reshape(og, cfg.o_lora, -1)).reshape(b, t, cfg.o_inter)
        x4 = self._hc_post(x4, (o1 @ tt[p + "wo_b"].t()).float(), post, comb)
        y, post, comb = self._hc_pre(x4, p + "hc_ffn")
        h2 = self._norm(y, tt[p + "ffn_norm"]).to(self.dtype)
        return self._hc_post(x4, self._moe(p, h2, ids), post, comb)

    def _head(self, xs: torch.Tensor, prefix: str, norm: str) -> torch.Tensor:
        """Collapse the streams with sigmoid weights, normalise, project onto the vocabulary (the MTP block has its own collapse and
        norm and shares the projection)."""
        cfg, tt = self.cfg, self.t
        flat = xs.reshape(*xs.shape[:2], -1)
        rsq = torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + cfg.norm_eps)
        pre = torch.sigmoid((flat @ tt[prefix + "hc_head_fn"].t()) * rsq * tt[prefix + "hc_head_scale"][0] + tt[prefix + "hc_head_base"]) + cfg.hc_eps
        y = (pre[..., None] * xs).sum(2)
        return (self._norm(y, tt[norm]).to(self.dtype) @ tt["head"].t()).float()

    @torch.no_grad()
    def forward(self, ids: torch.Tensor, all_logits: bool = False) -> torch.Tensor:
        cfg, tt = self.cfg, self.t
        ids = ids.to(self.device).long()
        b, t = ids.shape
        if not self.cache or b != self.batch:
            self.reset(b)
        p0 = self.pos
        positions = torch.arange(p0, p0 + t, device=self.device)
        x4 = tt["embed"][ids].float()[:, :, None, :].expand(b, t, cfg.hc_mult, cfg.hidden).contiguous()
        for li in range(cfg.n_layers):
            freq = self.freq_comp if cfg.compress_ratios[li] else self.freq_dense
            x4 = self._block(f"l{li}.", li, x4, self.cache[li], positions, p0, freq, ids)
        self.pos = p0 + t
        self.last_hc = x4
        logits = self._head(x4 if all_logits else x4[:, -1:], "", "out_norm")
        return logits if all_logits else logits[:, 0]

    @torch.no_grad()
    def mtp_predict(self, next_ids: torch.Tensor, hc_state: torch.Tensor, p0: int) -> torch.Tensor:
        """Logits of the token AFTER ``next_ids`` [B, T] from the main model's streams ``hc_state`` [B, T, hc, hidden] at positions
        ``p0 ..`` (common/ds4f_impl.h:4707-4784): every stream becomes ``e_proj(norm(embed(next))) + h_proj(norm(stream))``, one
        block (plain RoPE table, window attention only, no shared expert, its own cache), then the MTP block's own stream
        collapse and norm in front of the shared vocabulary projection."""
        cfg, tt = self.cfg, self.t
        if not cfg.mtp:
            raise ValueError("this checkpoint has no MTP block")
        next_ids = next_ids.to(self.device).long()
        t = next_ids.shape[1]
        e = self._norm(tt["embed"][next_ids].float(), tt["mtp.enorm"]).to(self.dtype) @ tt["mtp.e_proj"].t()      # [B, T, hidden]
        h = self._norm(hc_state.float(), tt["mtp.hnorm"]).to(self.dtype) @ tt["mtp.h_proj"].t()                   # [B, T, hc, hidden]
        x4 = (e[:, :, None, :] + h).float()
        positions = torch.arange(p0, p0 + t, device=self.device)
        x4 = self._block("mtp.", None, x4, self.mtp_cache, positions, p0, self.freq_dense, None)
        return self._head(x4, "mtp.", "mtp.norm")

    @torch.no_grad()
    def generate(self, prompt, max_new_tokens: int = 16, use_mtp: bool = False):
        """Greedy continuation of one prompt.  ``use_mtp``: self-speculative decoding with the MTP block as the draft: after the main
        model picks token a, the MTP block proposes the token b after it; the next main step runs a and b together, keeps b when the
        main model agrees and otherwise takes the state back to just after a.  Returns the same tokens either way; with
        ``use_mtp`` also the number of main-model steps as the second element of a pair."""
        ids = torch.tensor([list(prompt)], device=self.device)
        self.reset(1, len(prompt) + max_new_tokens + 2)
        logits = self.forward(ids)
        out: List[int] = []
        if not use_mtp:
            for _ in range(max_new_tokens):
                out.append(int(logits[0].argmax()))
                logits = self.forward(torch.tensor([[out[-1]]], device=self.device))
            return out
        steps = 1
        if len(prompt) > 1:                                              # the MTP cache over the prompt: position i holds (stream i, token i + 1)
            self.mtp_predict(ids[:, 1:], self.last_hc[:, :-1], 0)
        hc_last = self.last_hc[:, -1:]
        while len(out) < max_new_tokens:
            a = int(logits[0].argmax())
            out.append(a)
            if len(out) >= max_new_tokens:
                break
            pa = self.pos                                                # position a will take
            draft = int(self.mtp_predict(torch.tensor([[a]], device=self.device), hc_last, pa - 1)[0, -1].argmax())
            before = self.snapshot()
            both = self.forward(torch.tensor([[a, draft]], device=self.device), all_logits=True)
            steps += 1
            if int(both[0, 0].argmax()) == draft:                        # accepted: two tokens from one step
                out.append(draft)
                self.mtp_predict(torch.tensor([[draft]], device=self.device), self.last_hc[:, :1], pa)
                logits, hc_last = both[:, 1], self.last_hc[:, 1:]
            else:                                                        # rejected: back to just after a
                hc_a, la = self.last_hc[:, :1], both[:, 0]
                self.restore(before)
                self.forward(torch.tensor([[a]], device=self.device))   # rebuilds the compressors' rows for a
                steps += 1
                logits, hc_last = la, hc_a
        return out[:max_new_tokens], steps
