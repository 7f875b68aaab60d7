"""Gemma4 text model: GGUF loader / writer and a forward pass written with PyTorch tensor ops (CPU or CUDA).

What sets the architecture apart from the Qwen stacks of ``models.transformer`` (reference: common/transformer.h:1712-1758 for the
hyper-parameters, :1848-1914 for the tensors, :3510-3515 / :3563-3612 / :3624-3851 for the forward pass, :3529-3532 for the head):

* two kinds of layers: sliding-window layers (head size ``head_dim_swa``, RoPE base ``rope_base_swa``, a circular cache of
  ``window`` positions) and full-attention layers (head size ``head_dim_full``, RoPE base ``rope_base``, optionally divided per
  frequency by ``rope_freqs``); the number of KV heads is a property of the layer (rows of ``attn_k`` / head size);
* the last ``shared_kv_layers`` layers project no K / V: a sliding-window one reads the cache of layer
  ``n_kv_from_start - 2``, a full one that of ``n_kv_from_start - 1``;
* Q and K are RMS-normalised per head with a weight, V without one (or with ``attn_v_norm``); a layer without ``attn_v`` uses
  the normalised K as V; the attention scale is 1;
* the outputs of attention and FFN are normalised (``post_attention_norm``, ``post_ffw_norm``) before the residual add; the FFN is
  GELU(gate) * up (erf form);
* per-layer embeddings: a second embedding table ``per_layer_token_embd`` ([vocab, layers * ple_dim], scaled by sqrt(ple_dim)) plus a
  projection of the scaled token embedding (``per_layer_model_proj`` / sqrt(hidden), RMS-normalised per layer slice), averaged with
  1 / sqrt(2); after the FFN every layer gates its slice with GELU(``inp_gate`` x), projects it back (``proj``), normalises
  (``post_norm``) and adds it; then the stream is scaled by ``layer_output_scale``;
* token embeddings are scaled by sqrt(hidden); the logits are soft-capped: cap * tanh(logits / cap).

The projections are plain matrix products of the chosen dtype: no fused kernel of this repository serves head sizes 256 / 512, so
this family runs on library tensor ops on either device.  Parity with the reference's CPU engine on a GGUF file written by
``save_gguf`` is the test (tests/test_gemma4_cpu.py).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..utils import gguf as G


@dataclass
class Gemma4Config:
    n_layers: int
    hidden: int
    n_heads: int
    n_kv_heads: int
    ffn: int
    vocab: int
    head_dim_full: int = 512
    head_dim_swa: int = 256
    window: int = 512
    ple_dim: int = 256
    shared_kv_layers: int = 0
    softcap: float = 30.0
    rope_base: float = 1e6
    rope_base_swa: float = 1e4
    rms_eps: float = 1e-6
    swa_pattern: List[bool] = field(default_factory=list)      # True = sliding-window layer
    max_seq_len: int = 4096

    def __post_init__(self):
        if not self.swa_pattern:
            self.swa_pattern = [((i + 1) % 6) != 0 for i in range(self.n_layers)]     # the reference's default: every sixth layer is full

    @property
    def n_kv_from_start(self) -> int:
        return self.n_layers - self.shared_kv_layers

    def kv_source(self, li: int) -> int:
        """The layer whose cache layer ``li`` reads (itself unless it is one of the trailing shared-KV layers)."""
        if li < self.n_kv_from_start:
            return li
        return max(0, self.n_kv_from_start - (2 if self.swa_pattern[li] else 1))

    def head_dim(self, li: int) -> int:
        return self.head_dim_swa if self.swa_pattern[li] else self.head_dim_full


def config_from_gguf(f: G.GGUFFile) -> Gemma4Config:
    m = f.metadata
    if m.get("general.architecture") != "gemma4":
        raise ValueError("not a gemma4 GGUF file")
    k = lambda name, d=None: m.get("gemma4." + name, d)
    n_layers = int(k("block_count"))
    pat = k("attention.sliding_window_pattern")
    vocab = k("vocab_size")
    return Gemma4Config(
        n_layers=n_layers, hidden=int(k("embedding_length")), n_heads=int(k("attention.head_count")),
        n_kv_heads=int(k("attention.head_count_kv", k("attention.head_count"))), ffn=int(k("feed_forward_length")),
        vocab=int(vocab) if vocab is not None else f.tensors["token_embd.weight"].shape[0],
        head_dim_full=int(k("attention.key_length", 512)), head_dim_swa=int(k("attention.key_length_swa", 256)),
        window=int(k("attention.sliding_window", 512)), ple_dim=int(k("embedding_length_per_layer_input", 256)),
        shared_kv_layers=int(k("attention.shared_kv_layers", 0)), softcap=float(k("final_logit_softcapping", 30.0)),
        rope_base=float(k("rope.freq_base", 5e6)), rope_base_swa=float(k("rope.freq_base_swa", 1e4)),
        rms_eps=float(k("attention.layer_norm_rms_epsilon", 1e-6)),
        swa_pattern=[bool(x) for x in pat[:n_layers]] if pat is not None else [], max_seq_len=int(k("context_length", 4096)))


# tensors of a layer: (suffix, required)
_LAYER_TENSORS = ("attn_norm", "attn_q", "attn_q_norm", "attn_output", "attn_k", "attn_v", "attn_k_norm", "attn_v_norm", "post_attention_norm",
                  "ffn_norm", "ffn_gate", "ffn_up", "ffn_down", "post_ffw_norm", "layer_output_scale", "inp_gate", "proj", "post_norm")
_GLOBAL_TENSORS = ("token_embd", "output_norm", "output", "per_layer_token_embd", "per_layer_model_proj", "per_layer_proj_norm", "rope_freqs")


def load_gguf(path: str, device="cpu", dtype=torch.float32) -> "Gemma4Model":
    """Every tensor is dequantised once (any ggml type the decoders know) into ``dtype`` on ``device``."""
    with G.GGUFFile(path) as f:
        cfg = config_from_gguf(f)
        t: Dict[str, torch.Tensor] = {}
        for name, gt in f.tensors.items():
            x = gt.to_float()
            keep32 = x.dim() == 1                          # norm weights, scales, frequency factors stay fp32
            t[name] = x.to(device=device, dtype=torch.float32 if keep32 else dtype)
    return Gemma4Model(cfg, t, device, dtype)


def random_tensors(cfg: Gemma4Config, seed: int = 0, ple: bool = True, v_proj_on_swa: bool = True, kv_heads_full: Optional[int] = None,
                   rope_freqs: bool = True) -> Dict[str, torch.Tensor]:
    """A random-init checkpoint of the architecture (fp32): N(0, 0.05) matrices, norm weights around 1."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g) * 0.05
    nw = lambda n: 1.0 + 0.1 * torch.randn(n, generator=g)
    h, L = cfg.hidden, cfg.n_layers
    t = {"token_embd.weight": rn(cfg.vocab, h), "output_norm.weight": nw(h), "output.weight": rn(cfg.vocab, h)}
    if ple:
        t["per_layer_token_embd.weight"] = rn(cfg.vocab, L * cfg.ple_dim)
        t["per_layer_model_proj.weight"] = rn(L * cfg.ple_dim, h)
        t["per_layer_proj_norm.weight"] = nw(cfg.ple_dim)
    if rope_freqs:
        t["rope_freqs.weight"] = 1.0 + torch.rand(cfg.head_dim_full // 2, generator=g) * 3.0
    for li in range(L):
        p, hd, swa = f"blk.{li}.", cfg.head_dim(li), cfg.swa_pattern[li]
        kvh = cfg.n_kv_heads if (swa or kv_heads_full is None) else kv_heads_full
        t[p + "attn_norm.weight"] = nw(h)
        t[p + "attn_q.weight"] = rn(cfg.n_heads * hd, h)
        t[p + "attn_q_norm.weight"] = nw(hd)
        t[p + "attn_output.weight"] = rn(h, cfg.n_heads * hd)
        if li < cfg.n_kv_from_start:
            t[p + "attn_k.weight"] = rn(kvh * hd, h)
            t[p + "attn_k_norm.weight"] = nw(hd)
            if v_proj_on_swa or not swa:
                t[p + "attn_v.weight"] = rn(kvh * hd, h)
        for nm in ("post_attention_norm", "ffn_norm", "post_ffw_norm"):
            t[p + nm + ".weight"] = nw(h)
        t[p + "ffn_gate.weight"] = rn(cfg.ffn, h)
        t[p + "ffn_up.weight"] = rn(cfg.ffn, h)
        t[p + "ffn_down.weight"] = rn(h, cfg.ffn)
        t[p + "layer_output_scale.weight"] = 0.8 + 0.4 * torch.rand(1, generator=g)
        if ple:
            t[p + "inp_gate.weight"] = rn(cfg.ple_dim, h)
            t[p + "proj.weight"] = rn(h, cfg.ple_dim)
            t[p + "post_norm.weight"] = nw(h)
    return t


def save_gguf(cfg: Gemma4Config, tensors: Dict[str, torch.Tensor], path: str, wtype: str = "F16") -> None:
    """Write a gemma4 GGUF file: matrices as ``wtype``, vectors as F32, the hyper-parameters under the keys the reference reads."""
    w = G.GGUFWriter()
    w.add_string("general.architecture", "gemma4")
    for key, v in (("block_count", cfg.n_layers), ("embedding_length", cfg.hidden), ("attention.head_count", cfg.n_heads),
                   ("attention.head_count_kv", cfg.n_kv_heads), ("feed_forward_length", cfg.ffn), ("vocab_size", cfg.vocab),
                   ("context_length", cfg.max_seq_len), ("attention.key_length", cfg.head_dim_full), ("attention.key_length_swa", cfg.head_dim_swa),
                   ("attention.sliding_window", cfg.window), ("embedding_length_per_layer_input", cfg.ple_dim),
                   ("attention.shared_kv_layers", cfg.shared_kv_layers)):
        w.add_u32("gemma4." + key, v)
    for key, v in (("attention.layer_norm_rms_epsilon", cfg.rms_eps), ("rope.freq_base", cfg.rope_base), ("rope.freq_base_swa", cfg.rope_base_swa),
                   ("final_logit_softcapping", cfg.softcap)):
        w.add_f32("gemma4." + key, v)
    w.add_array("gemma4.attention.sliding_window_pattern", [bool(x) for x in cfg.swa_pattern], G.KV_BOOL)
    for name, x in tensors.items():
        w.add_tensor(name, x.float(), "F32" if x.dim() == 1 else wtype)
    w.write(path)


def _rms(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float() if w is not None else y).to(x.dtype)


def _gelu(x: torch.Tensor) -> torch.Tensor:
    xf = x.float()
    return (xf * 0.5 * (1.0 + torch.erf(xf * 0.7071067811865476))).to(x.dtype)


class Gemma4Model:
    """One batch of ``batch`` sequences that advance together (the reference engine's unit is one sequence, token by token; here
    a call takes ``[batch, T]`` tokens at the same positions: a prefill chunk or a decode step)."""

    def __init__(self, cfg: Gemma4Config, tensors: Dict[str, torch.Tensor], device="cpu", dtype=torch.float32):
        self.cfg, self.t, self.device, self.dtype = cfg, tensors, torch.device(device), dtype
        self.has_ple = "per_layer_token_embd.weight" in tensors and "per_layer_model_proj.weight" in tensors
        self.kv_heads: List[int] = []
        for li in range(cfg.n_layers):
            src = cfg.kv_source(li)
            if src == li:
                k = tensors.get(f"blk.{li}.attn_k.weight")
                self.kv_heads.append(k.shape[0] // cfg.head_dim(li) if k is not None else cfg.n_kv_heads)
            else:
                self.kv_heads.append(self.kv_heads[src])
        # RoPE frequencies of the two layer kinds (pairs (j, j + half), common/transformer.h:3672-3701)
        hs, hf = cfg.head_dim_swa // 2, cfg.head_dim_full // 2
        self.inv_freq_swa = (1.0 / cfg.rope_base_swa ** (torch.arange(hs, dtype=torch.float32) * 2 / cfg.head_dim_swa)).to(self.device)
        inv = 1.0 / cfg.rope_base ** (torch.arange(hf, dtype=torch.float32) * 2 / cfg.head_dim_full)
        ff = tensors.get("rope_freqs.weight")
        if ff is not None:
            n = min(hf, ff.numel())
            inv[:n] = inv[:n] / ff.float().cpu()[:n]
        self.inv_freq_full = inv.to(self.device)
        self.k_cache: Dict[int, torch.Tensor] = {}
        self.v_cache: Dict[int, torch.Tensor] = {}
        self.pos = 0
        self.batch = 0

    # ------------------------------------------------------------------------------------------ state
    def reset(self, batch: int = 1, max_seq_len: Optional[int] = None) -> None:
        """Allocate the caches: ``window`` positions (circular) for sliding-window layers, ``max_seq_len`` for full layers; none
        for the layers that read another layer's cache."""
        cfg = self.cfg
        n = max_seq_len or cfg.max_seq_len
        self.k_cache, self.v_cache, self.pos, self.batch = {}, {}, 0, batch
        for li in range(cfg.n_layers):
            if cfg.kv_source(li) != li:
                continue
            ln = cfg.window if cfg.swa_pattern[li] else n
            shape = (batch, ln, self.kv_heads[li], cfg.head_dim(li))
            self.k_cache[li] = torch.zeros(shape, dtype=self.dtype, device=self.device)
            self.v_cache[li] = torch.zeros(shape, dtype=self.dtype, device=self.device)

    def kv_bytes(self) -> int:
        return sum(x.numel() * x.element_size() for x in self.k_cache.values()) * 2

    # ------------------------------------------------------------------------------------------ pieces
    def _lin(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return x @ self.t[name].t()

    def _rope(self, x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
        """``x`` [B, T, H, D]; rotates the pairs (j, j + D/2)."""
        ang = positions.float()[:, None] * inv_freq[None, :]                 # [T, D/2]
        cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
        half = x.shape[-1] // 2
        a, b = x[..., :half].float(), x[..., half:].float()
        return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1).to(x.dtype)

    def _keys(self, li: int, k_new: torch.Tensor, v_new: torch.Tensor, p0: int):
        """Write this step's K / V rows ``[B, T, Hkv, D]`` of layer ``li`` into its cache and return what the step's queries can see:
        ``(k, v, key positions)``.  A sliding-window layer returns the cached window in front of the chunk followed by the chunk's
        own rows (its circular cache afterwards holds only the last ``window`` positions, too few for the chunk's first queries)."""
        cfg = self.cfg
        t = k_new.shape[1]
        kc, vc = self.k_cache[li], self.v_cache[li]
        qpos = torch.arange(p0, p0 + t, device=self.device)
        if cfg.swa_pattern[li]:
            win = cfg.window
            hist = torch.arange(max(0, p0 - win + 1), p0, device=self.device)
            k_all = torch.cat([kc[:, hist % win], k_new], dim=1)
            v_all = torch.cat([vc[:, hist % win], v_new], dim=1)
            keep = qpos[-win:]
            kc[:, keep % win] = k_new[:, -keep.numel():]
            vc[:, keep % win] = v_new[:, -keep.numel():]
            return k_all, v_all, torch.cat([hist, qpos])
        kc[:, p0: p0 + t] = k_new
        vc[:, p0: p0 + t] = v_new
        return kc[:, : p0 + t], vc[:, : p0 + t], torch.arange(0, p0 + t, device=self.device)

    def _attention(self, li: int, q: torch.Tensor, keys, p0: int) -> torch.Tensor:
        """``q`` [B, T, H, D] at positions ``p0 .. p0 + T - 1`` against ``keys`` = ``_keys(...)`` of the layer whose cache this
        layer reads (itself, or the shared-KV source, which ran earlier in the same step)."""
        cfg = self.cfg
        b, t, h, d = q.shape
        k_all, v_all, kpos = keys
        qpos = torch.arange(p0, p0 + t, device=self.device)
        mask = kpos[None, :] <= qpos[:, None]
        if cfg.swa_pattern[li]:
            mask = mask & (kpos[None, :] > qpos[:, None] - cfg.window)
        g = h // k_all.shape[2]
        kf = k_all.float().repeat_interleave(g, dim=2)
        vf = v_all.float().repeat_interleave(g, dim=2)
        sc = torch.einsum("bqhd,bkhd->bhqk", q.float(), kf)                   # scale 1: the head norms carry it
        sc = sc.masked_fill(~mask[None, None], float("-inf"))
        out = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, dim=-1), vf)
        return out.to(q.dtype)

    # ------------------------------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, ids: torch.Tensor, all_logits: bool = False, embeds: Optional[torch.Tensor] = None,
                embeds_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``ids`` int [B, T]: the next T tokens of every sequence.  Returns f32 logits [B, V] of the last token (``all_logits``:
        [B, T, V]) and advances the position.  Where ``embeds_mask`` [B, T] is set, row ``embeds[b, t]`` ([B, T, hidden], soft tokens
        of the vision or audio encoder) enters the stack unscaled in place of the token's embedding, and the per-layer embedding
        is the one of token 0 (common/transformer.h:4317-4332)."""
        cfg, tt = self.cfg, self.t
        ids = ids.to(self.device).long()
        b, t = ids.shape
        if not self.k_cache or b != self.batch:
            self.reset(b)
        p0 = self.pos
        positions = torch.arange(p0, p0 + t, device=self.device)
        eps, h, L = cfg.rms_eps, cfg.hidden, cfg.n_layers
        x = tt["token_embd.weight"][ids].to(self.dtype) * math.sqrt(h)
        if embeds is not None:
            mask = torch.ones(b, t, dtype=torch.bool, device=self.device) if embeds_mask is None else embeds_mask.to(self.device).bool()
            x = torch.where(mask[..., None], embeds.to(self.device, self.dtype), x)
            ids = ids.masked_fill(mask, 0)
        ple = None
        if self.has_ple:
            tok = tt["per_layer_token_embd.weight"][ids].float() * math.sqrt(cfg.ple_dim)               # [B, T, L * ple]
            proj = self._lin(x, "per_layer_model_proj.weight").float() / math.sqrt(h)
            proj = proj.reshape(b, t, L, cfg.ple_dim)
            nw = tt.get("per_layer_proj_norm.weight")
            if nw is not None:
                proj = _rms(proj, nw, eps)
            ple = ((proj + tok.reshape(b, t, L, cfg.ple_dim)) / math.sqrt(2.0)).to(self.dtype)
        step_keys: Dict[int, tuple] = {}
        for li in range(L):
            p = f"blk.{li}."
            hd, swa, own = cfg.head_dim(li), cfg.swa_pattern[li], cfg.kv_source(li) == li
            inv_freq = self.inv_freq_swa if swa else self.inv_freq_full
            hn = _rms(x, tt[p + "attn_norm.weight"], eps)
            q = _rms(self._lin(hn, p + "attn_q.weight").reshape(b, t, cfg.n_heads, hd), tt[p + "attn_q_norm.weight"], eps)
            q = self._rope(q, positions, inv_freq)
            if own:
                kvh = self.kv_heads[li]
                k = _rms(self._lin(hn, p + "attn_k.weight").reshape(b, t, kvh, hd), tt[p + "attn_k_norm.weight"], eps)
                v = self._lin(hn, p + "attn_v.weight").reshape(b, t, kvh, hd) if (p + "attn_v.weight") in tt else k
                v = _rms(v, tt.get(p + "attn_v_norm.weight"), eps)
                step_keys[li] = self._keys(li, self._rope(k, positions, inv_freq), v, p0)
            a = self._attention(li, q, step_keys[cfg.kv_source(li)], p0).reshape(b, t, cfg.n_heads * hd)
            x = x + _rms(self._lin(a, p + "attn_output.weight"), tt[p + "post_attention_norm.weight"], eps)
            hn = _rms(x, tt[p + "ffn_norm.weight"], eps)
            f = _gelu(self._lin(hn, p + "ffn_gate.weight")) * self._lin(hn, p + "ffn_up.weight")
            x = x + _rms(self._lin(f, p + "ffn_down.weight"), tt[p + "post_ffw_norm.weight"], eps)
            if ple is not None and (p + "inp_gate.weight") in tt:
                gte = _gelu(self._lin(x, p + "inp_gate.weight"))
                pj = self._lin(ple[:, :, li] * gte, p + "proj.weight")
                if (p + "post_norm.weight") in tt:
                    pj = _rms(pj, tt[p + "post_norm.weight"], eps)
                x = x + pj
            sc = tt.get(p + "layer_output_scale.weight")
            if sc is not None:
                x = x * sc.float().reshape(()).to(x.dtype)
        self.pos = p0 + t
        xo = _rms(x if all_logits else x[:, -1:], tt["output_norm.weight"], eps)
        head = tt["output.weight"] if "output.weight" in tt else tt["token_embd.weight"]
        logits = (xo @ head.t()).float()
        if cfg.softcap > 0:
            logits = cfg.softcap * torch.tanh(logits / cfg.softcap)
        return logits if all_logits else logits[:, 0]

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, chunk: int = 2048, embeds: Optional[torch.Tensor] = None,
                embeds_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run a prompt ``[B, T]`` in chunks (the score matrix of a chunk is materialised); returns the logits of the last token."""
        out = None
        for i in range(0, ids.shape[1], chunk):
            e = None if embeds is None else embeds[:, i: i + chunk]
            m = None if embeds_mask is None else embeds_mask[:, i: i + chunk]
            out = self.forward(ids[:, i: i + chunk], embeds=e, embeds_mask=m)
        return out

    @torch.no_grad()
    def generate(self, prompt: Sequence[int], max_new_tokens: int = 16, soft: Optional[torch.Tensor] = None, soft_at: int = 0) -> List[int]:
        """Greedy continuation of one prompt.  ``soft`` [n, hidden]: encoder rows spliced in front of prompt token ``soft_at`` (the
        reference's multimodal prompt: text, the image or audio rows, text; cuda/llm/test_gemma4_st.c:150-156)."""
        ids, embeds, mask = list(prompt), None, None
        if soft is not None and soft.shape[0] > 0:
            n = soft.shape[0]
            ids = ids[:soft_at] + [0] * n + ids[soft_at:]
            embeds = torch.zeros(1, len(ids), self.cfg.hidden, dtype=torch.float32)
            embeds[0, soft_at: soft_at + n] = soft.float().cpu()
            mask = torch.zeros(1, len(ids), dtype=torch.bool)
            mask[0, soft_at: soft_at + n] = True
        self.reset(1, len(ids) + max_new_tokens + 1)
        logits = self.prefill(torch.tensor([ids]), embeds=embeds, embeds_mask=mask)
        out = []
        for _ in range(max_new_tokens):
            out.append(int(logits[0].argmax()))
            logits = self.forward(torch.tensor([[out[-1]]]))
        return out
