"""GLM-5 style engine as a PyTorch-op forward pass (CPU or CUDA): multi-head latent attention (MLA) over a compressed KV cache, the
block-sparse indexer, and the sigmoid-router MoE it shares with the M3 engine (``models.m3``).

Reference: common/glm5.h:60-114 (configuration), common/glm5_impl.h:1016-1200 (one token through the stack), :941-1008 (block
selection), :917-927 (latent cache codec).  Attention of a layer:

* queries go through a low-rank pair: ``q_lat = norm(wq_a x)``, ``q = wq_b q_lat`` -> per head ``[qk_nope | qk_rope]``; the rope
  part is rotated on interleaved pairs ``(2k, 2k + 1)``;
* keys / values are ONE latent row per position: ``wkv_a x`` -> ``[kv_lora | qk_rope]``, the first part normalised, the second
  rotated; that row (bf16, or int4 with one scale) is all the cache holds: ``kv_lora + qk_rope`` values per position and layer
  instead of ``2 * heads * head_dim``;
* per head, ``wkv_b`` expands a latent row into ``k_nope`` (``qk_nope`` values) and ``v`` (``v_head_dim``); the score is
  ``(q_nope . k_nope + q_rope . k_rope) / sqrt(qk_head_dim)``.  Here the expansion is one batched product over the cached rows;
  the reference's "absorbed" form (``wkv_b`` folded into the query and applied to the context once) is the same arithmetic in
  another order (common/glm5_impl.h:1066-1100);
* the indexer (off by default, as in the reference's bring-up: ``GLM5_MSA=0``) selects blocks the way the M3 engine does; layers
  without an indexer of their own reuse the selection of the last layer that has one (common/glm5.h:121-131).

Norms multiply by ``w`` (not ``1 + w``) and the FFN activation is plain SiLU(gate) * up.  Weights are bf16, products are library
tensor ops.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from . import m3


@dataclass
class GLM5Config:
    n_layers: int = 78
    n_dense_layers: int = 3
    hidden: int = 6144
    vocab: int = 154880
    norm_eps: float = 1e-5
    n_heads: int = 64
    qk_nope_dim: int = 192
    qk_rope_dim: int = 64
    v_head_dim: int = 256
    q_lora: int = 2048
    kv_lora: int = 512
    rope_theta: float = 8e6
    index_dim: int = 128
    index_n_heads: int = 32
    index_topk_freq: int = 4
    msa_block_size: int = 128
    msa_topk_blocks: int = 16
    msa_init_block: int = 0
    msa_local_block: int = 1
    n_experts: int = 256
    n_active: int = 8
    moe_inter: int = 2048
    dense_inter: int = 12288
    routed_scale: float = 2.5
    max_pos: int = 2048

    # the names the shared MoE / indexer code reads
    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_dim + self.qk_rope_dim

    @property
    def rotary_dim(self) -> int:
        return self.qk_rope_dim

    @property
    def msa_index_dim(self) -> int:
        return self.index_dim

    @property
    def msa_n_index_heads(self) -> int:
        return self.index_n_heads

    @property
    def kv_cache_dim(self) -> int:
        return self.kv_lora + self.qk_rope_dim

    def is_moe(self, li: int) -> bool:
        return li >= self.n_dense_layers

    def has_full_indexer(self, li: int) -> bool:
        if li < self.n_dense_layers:
            return True
        first = self.n_dense_layers + self.index_topk_freq - 1
        return li >= first and (li - first) % self.index_topk_freq == 0


def random_tensors(cfg: GLM5Config, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    u = lambda amp, *s: ((torch.rand(*s, generator=g) * 2 - 1) * amp)
    bf = lambda amp, *s: u(amp, *s).to(torch.bfloat16)
    h, nh = cfg.hidden, cfg.n_heads
    t = {"embed": bf(0.05, cfg.vocab, h), "head": bf(0.05, cfg.vocab, h), "out_norm": 1.0 + bf(0.1, h).float()}
    t["out_norm"] = t["out_norm"].to(torch.bfloat16)
    for li in range(cfg.n_layers):
        p = f"l{li}."
        nw = lambda n: (1.0 + u(0.1, n)).to(torch.bfloat16)
        t.update({p + "input_norm": nw(h), p + "post_norm": nw(h), p + "wq_a": bf(0.03, cfg.q_lora, h), p + "wq_b": bf(0.03, nh * cfg.qk_head_dim, cfg.q_lora),
                  p + "wkv_a": bf(0.03, cfg.kv_cache_dim, h), p + "wkv_b": bf(0.03, nh * (cfg.qk_nope_dim + cfg.v_head_dim), cfg.kv_lora),
                  p + "wo": bf(0.03, h, nh * cfg.v_head_dim), p + "q_a_norm": nw(cfg.q_lora), p + "kv_a_norm": nw(cfg.kv_lora)})
        if cfg.is_moe(li):
            e, it = cfg.n_experts, cfg.moe_inter
            t.update({p + "idx_wq": bf(0.03, cfg.index_n_heads * cfg.index_dim, h), p + "idx_wk": bf(0.03, cfg.index_dim, h),
                      p + "idx_q_norm": nw(cfg.index_dim), p + "idx_k_norm": nw(cfg.index_dim), p + "gate": bf(0.03, e, h), p + "gate_bias": u(0.1, e),
                      p + "sh_w1": bf(0.03, it, h), p + "sh_w3": bf(0.03, it, h), p + "sh_w2": bf(0.03, h, it), p + "ex_w1": bf(0.03, e, it, h),
                      p + "ex_w3": bf(0.03, e, it, h), p + "ex_w2": bf(0.03, e, h, it)})
        else:
            t.update({p + "ff_gate": bf(0.03, cfg.dense_inter, h), p + "ff_up": bf(0.03, cfg.dense_inter, h), p + "ff_down": bf(0.03, h, cfg.dense_inter)})
    return t


class GLM5Model(m3.M3Model):
    def __init__(self, cfg: GLM5Config, tensors: Dict[str, torch.Tensor], device="cpu", dtype=torch.float32, ep_rank: int = 0, ep_size: int = 1,
                 group=None, int4_kv: bool = False, msa: bool = False):
        super().__init__(cfg, tensors, device, dtype, ep_rank, ep_size, group, int4_kv, msa)

    def reset(self, batch: int = 1, max_pos: Optional[int] = None) -> None:
        cfg = self.cfg
        n = max_pos or cfg.max_pos
        self.pos, self.batch, self.cache = 0, batch, []
        for li in range(cfg.n_layers):
            c: Dict[str, torch.Tensor] = {}
            for nm, width in [("kv", cfg.kv_cache_dim)] + ([("ik", cfg.index_dim)] if cfg.is_moe(li) else []):
                shp = (batch, n, 1, width)
                if self.int4_kv:
                    c[nm + "_q"] = torch.zeros(shp, dtype=torch.int8, device=self.device)
                    c[nm + "_s"] = torch.zeros(shp[:-1] + (1,), dtype=torch.bfloat16, device=self.device)
                else:
                    c[nm] = torch.zeros(shp, dtype=torch.bfloat16, device=self.device)
            self.cache.append(c)

    def _norm(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.norm_eps) * w.float()).to(x.dtype)

    def _swiglu(self, g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
        gf = g.float()
        return (gf * torch.sigmoid(gf) * u.float()).to(g.dtype)

    def _rope_interleaved(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """``x`` [B, T, H, qk_rope]: rotates the pairs (2k, 2k + 1)."""
        ang = positions.double()[:, None] * self.inv_freq[None, :]
        cos, sin = ang.cos().float()[None, :, None, :], ang.sin().float()[None, :, None, :]
        a, b = x[..., 0::2].float(), x[..., 1::2].float()
        return torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2).to(x.dtype)

    @torch.no_grad()
    def forward(self, ids: torch.Tensor, all_logits: bool = False) -> torch.Tensor:
        cfg, tt = self.cfg, self.t
        ids = ids.to(self.device).long()
        b, t = ids.shape
        if not self.cache or b != self.batch:
            self.reset(b)
        p0 = self.pos
        positions = torch.arange(p0, p0 + t, device=self.device)
        nh, nope, rope, vd, lora = cfg.n_heads, cfg.qk_nope_dim, cfg.qk_rope_dim, cfg.v_head_dim, cfg.kv_lora
        n = p0 + t
        causal = (torch.arange(n, device=self.device)[None, :] <= positions[:, None])[None].expand(b, t, n)
        x = tt["embed"][ids].float()
        last_sel = None
        for li in range(cfg.n_layers):
            p, c = f"l{li}.", self.cache[li]
            hn = self._norm(x, tt[p + "input_norm"]).to(self.dtype)
            q_lat = self._norm(hn @ tt[p + "wq_a"].t(), tt[p + "q_a_norm"])
            q = (q_lat @ tt[p + "wq_b"].t()).reshape(b, t, nh, nope + rope)
            q_nope, q_rope = q[..., :nope].float(), self._rope_interleaved(q[..., nope:], positions).float()
            kv = hn @ tt[p + "wkv_a"].t()
            lat = self._norm(kv[..., :lora], tt[p + "kv_a_norm"])
            kr = self._rope_interleaved(kv[..., lora:].reshape(b, t, 1, rope), positions)
            self._store(c, "kv", torch.cat([lat.reshape(b, t, 1, lora).float(), kr.float()], dim=-1), p0)
            if cfg.is_moe(li) and self.msa and cfg.has_full_indexer(li):
                mask = last_sel = self._msa_mask(li, hn, positions, p0, q_lat)
            elif cfg.is_moe(li) and self.msa and last_sel is not None:
                mask = last_sel                                                 # a layer without an indexer reuses the last selection
            else:
                mask = causal
            rows = self._load(c, "kv", n)[:, :, 0]                              # [B, n, kv_lora + rope]
            wkv_b = tt[p + "wkv_b"].reshape(nh, nope + vd, lora).float()
            k_nope = torch.einsum("bnl,hdl->bnhd", rows[..., :lora], wkv_b[:, :nope])
            v = torch.einsum("bnl,hdl->bnhd", rows[..., :lora], wkv_b[:, nope:])
            sc = (torch.einsum("bqhd,bnhd->bhqn", q_nope, k_nope) + torch.einsum("bqhd,bnd->bhqn", q_rope, rows[..., lora:])) / math.sqrt(nope + rope)
            sc = sc.masked_fill(~mask[:, None], float("-inf"))
            a = torch.einsum("bhqn,bnhd->bqhd", torch.softmax(sc, dim=-1), v).reshape(b, t, nh * vd).to(self.dtype)
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


# ---------------------------------------------------------------------------------------------------- checkpoints
# tensor names of the GLM-5 checkpoints as the reference's loader reads them (common/glm5_impl.h:773-1010): per layer under
# "model.layers.<l>.", experts under ".mlp.experts.<e>."; FP8 weights carry "<name>_scale_inv" (fp32 per 128 x 128 block)
_HF_LAYER = {"input_norm": "input_layernorm.weight", "post_norm": "post_attention_layernorm.weight", "wq_a": "self_attn.q_a_proj.weight",
             "q_a_norm": "self_attn.q_a_layernorm.weight", "wq_b": "self_attn.q_b_proj.weight", "wkv_a": "self_attn.kv_a_proj_with_mqa.weight",
             "kv_a_norm": "self_attn.kv_a_layernorm.weight", "wkv_b": "self_attn.kv_b_proj.weight", "wo": "self_attn.o_proj.weight",
             "idx_wq_b": "self_attn.indexer.wq_b.weight", "idx_wk": "self_attn.indexer.wk.weight", "idx_k_norm": "self_attn.indexer.k_norm.weight",
             "gate": "mlp.gate.weight", "gate_bias": "mlp.gate.e_score_correction_bias", "sh_w1": "mlp.shared_experts.gate_proj.weight",
             "sh_w3": "mlp.shared_experts.up_proj.weight", "sh_w2": "mlp.shared_experts.down_proj.weight", "ff_gate": "mlp.gate_proj.weight",
             "ff_up": "mlp.up_proj.weight", "ff_down": "mlp.down_proj.weight"}
_HF_EXPERT = {"ex_w1": "gate_proj.weight", "ex_w3": "up_proj.weight", "ex_w2": "down_proj.weight"}
_HF_GLOBAL = {"embed": "model.embed_tokens.weight", "head": "lm_head.weight", "out_norm": "model.norm.weight"}
_HF_PREFIX, _HF_EXPERTS = "model.layers.{l}.", "mlp.experts.{e}."


def checkpoint_shapes(cfg: GLM5Config) -> Dict[str, torch.Tensor]:
    """Names, shapes and dtypes (meta tensors) of a checkpoint of ``cfg``: the indexer reads the query latent (``idx_wq_b``) and
    exists on the MoE layers that have one of their own."""
    with torch.device("meta"):
        h, nh = cfg.hidden, cfg.n_heads
        bf = lambda *s: torch.empty(*s, dtype=torch.bfloat16)
        t = {"embed": bf(cfg.vocab, h), "head": bf(cfg.vocab, h), "out_norm": bf(h)}
        for li in range(cfg.n_layers):
            p = f"l{li}."
            t.update({p + "input_norm": bf(h), p + "post_norm": bf(h), p + "wq_a": bf(cfg.q_lora, h), p + "wq_b": bf(nh * cfg.qk_head_dim, cfg.q_lora),
                      p + "wkv_a": bf(cfg.kv_cache_dim, h), p + "wkv_b": bf(nh * (cfg.qk_nope_dim + cfg.v_head_dim), cfg.kv_lora),
                      p + "wo": bf(h, nh * cfg.v_head_dim), p + "q_a_norm": bf(cfg.q_lora), p + "kv_a_norm": bf(cfg.kv_lora)})
            if cfg.is_moe(li):
                e, it = cfg.n_experts, cfg.moe_inter
                if cfg.has_full_indexer(li):
                    t.update({p + "idx_wq_b": bf(cfg.index_n_heads * cfg.index_dim, cfg.q_lora), p + "idx_wk": bf(cfg.index_dim, h),
                              p + "idx_k_norm": bf(cfg.index_dim)})
                t.update({p + "gate": bf(e, h), p + "gate_bias": torch.empty(e, dtype=torch.float32), p + "sh_w1": bf(it, h), p + "sh_w3": bf(it, h),
                          p + "sh_w2": bf(h, it), p + "ex_w1": bf(e, it, h), p + "ex_w3": bf(e, it, h), p + "ex_w2": bf(e, h, it)})
            else:
                t.update({p + "ff_gate": bf(cfg.dense_inter, h), p + "ff_up": bf(cfg.dense_inter, h), p + "ff_down": bf(h, cfg.dense_inter)})
    return t


def save_checkpoint(cfg: GLM5Config, tensors: Dict[str, torch.Tensor], path: str, fp8: bool = False) -> None:
    """An HF-layout directory; ``fp8`` stores the projection matrices as F8_E4M3 with fp32 ``_scale_inv`` per 128 x 128 block (the
    dense format of the GLM-5 checkpoints)."""
    import dataclasses
    import json
    import os
    from .loader import save_safetensors
    os.makedirs(path, exist_ok=True)
    named = m3.checkpoint_names(tensors, _HF_LAYER, _HF_EXPERT, _HF_GLOBAL, _HF_PREFIX, _HF_EXPERTS)
    out: Dict[str, torch.Tensor] = {}
    for name, v in named.items():
        quant = fp8 and v.dim() == 2 and "norm" not in name and "embed" not in name and "lm_head" not in name and "gate.weight" not in name
        if quant:
            rows, cols = v.shape
            pr, pc = (rows + 127) // 128 * 128, (cols + 127) // 128 * 128
            w = torch.zeros(pr, pc)
            w[:rows, :cols] = v.float()
            sc = (w.reshape(pr // 128, 128, pc // 128, 128).abs().amax(dim=(1, 3)) / 448.0).clamp_min(1e-12)
            q = (w / sc.repeat_interleave(128, 0).repeat_interleave(128, 1))[:rows, :cols].to(torch.float8_e4m3fn)
            out[name], out[name + "_scale_inv"] = q, sc.float()
        else:
            out[name] = v
    save_safetensors(out, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump({"model_type": "glm5", "gemm_b200": dataclasses.asdict(cfg)}, fh)


def load_checkpoint(path: str, device="cpu", dtype=torch.float32, cfg: Optional[GLM5Config] = None, **kw) -> "GLM5Model":
    import json
    import os
    if cfg is None:
        with open(os.path.join(path, "config.json")) as fh:
            cfg = GLM5Config(**json.load(fh)["gemm_b200"])
    t = m3.read_checkpoint(path, checkpoint_shapes(cfg), _HF_LAYER, _HF_EXPERT, _HF_GLOBAL, _HF_PREFIX, _HF_EXPERTS)
    return GLM5Model(cfg, t, device, dtype, **kw)
