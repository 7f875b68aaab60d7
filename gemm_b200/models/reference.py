"""Plain PyTorch fp32 oracle of the decoder: no paging, no fusion, no custom kernels.

It mirrors the arithmetic of the reference CPU engine (common/transformer.h:3550-4174: RMSNorm, fused QKV,
per-head QK-norm, NeoX RoPE, causal GQA softmax attention, SwiGLU or softmax-top-k MoE with renormalised
weights, final norm, LM head) on dequantised weights, and is what every GPU engine test compares against.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..ops.elementwise import rope_ref
from .weights import ModelWeights


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()


@torch.no_grad()
def reference_logits(weights: ModelWeights, tokens: torch.Tensor, n_layers: Optional[int] = None,
                     return_hidden: bool = False) -> torch.Tensor:
    """Logits ``[S, V]`` for one sequence of token ids ``[S]`` processed from position 0 (unsharded weights)."""
    cfg = weights.cfg
    assert weights.tp_size == 1 and weights.ep_size == 1
    dev = weights.embed.device
    s = tokens.numel()
    d, hq, hkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
    g = hq // hkv
    x = weights.embed[tokens.long()].float()
    pos = torch.arange(s, device=dev)
    layers = weights.layers if n_layers is None else weights.layers[:n_layers]
    for lw in layers:
        h = _rms(x, lw.attn_norm, cfg.rms_eps)
        qkv = h @ lw.wqkv.dequantized().t()
        if lw.wqkv.bias is not None:
            qkv = qkv + lw.wqkv.bias.float()
        q = qkv[:, : hq * d].reshape(s, hq, d)
        k = qkv[:, hq * d:(hq + hkv) * d].reshape(s, hkv, d)
        v = qkv[:, (hq + hkv) * d:].reshape(s, hkv, d)
        if lw.q_norm is not None:
            q = _rms(q, lw.q_norm, cfg.rms_eps)
            k = _rms(k, lw.k_norm, cfg.rms_eps)
        q = rope_ref(q, pos, cfg.rope_theta, cfg.rope_dim)
        k = rope_ref(k, pos, cfg.rope_theta, cfg.rope_dim)
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
        sc = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(d)
        mask = torch.ones(s, s, dtype=torch.bool, device=dev).tril()
        if cfg.sliding_window > 0:
            mask &= ~torch.ones(s, s, dtype=torch.bool, device=dev).tril(-cfg.sliding_window)
        sc = sc.masked_fill(~mask, float("-inf"))
        a = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), v).reshape(s, hq * d)
        x = x + a @ lw.wo.dequantized().t()
        h = _rms(x, lw.ffn_norm, cfg.rms_eps)
        if lw.w13 is not None:
            e, kk, inter = cfg.n_experts, cfg.n_experts_used, cfg.expert_ffn
            logits = h @ lw.router.float().t()
            if cfg.router == "softmax":
                p = torch.softmax(logits, -1)
                sel = p
            else:
                p = torch.sigmoid(logits)
                sel = p + (lw.router_bias.float() if lw.router_bias is not None else 0.0)
            idx = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, :kk]
            wts = torch.gather(p, 1, idx)
            if cfg.norm_topk:
                wts = wts / wts.sum(-1, keepdim=True)
            wts = wts * cfg.routed_scale
            w13 = lw.w13.dequantized().reshape(e, 2 * inter, cfg.hidden)
            w2 = lw.w2.dequantized().reshape(e, cfg.hidden, inter)
            y = torch.zeros_like(x)
            for ei in range(e):
                tok, slot = (idx == ei).nonzero(as_tuple=True)
                if tok.numel() == 0:
                    continue
                r = h[tok] @ w13[ei].t()
                act = torch.nn.functional.silu(r[:, :inter]) * r[:, inter:]
                y.index_add_(0, tok, (act @ w2[ei].t()) * wts[tok, slot].unsqueeze(-1))
            x = x + y
        else:
            f = lw.w_gate_up.n // 2
            r = h @ lw.w_gate_up.dequantized().t()
            x = x + (torch.nn.functional.silu(r[:, :f]) * r[:, f:]) @ lw.w_down.dequantized().t()
    if return_hidden:
        return x
    hn = _rms(x, weights.final_norm, cfg.rms_eps)
    return hn @ weights.lm_head.dequantized().t()
