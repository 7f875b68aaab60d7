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
        if lw.ssm is not None:
            x = x + _deltanet_layer(cfg, lw.ssm, h)
            x = x + _ffn(cfg, lw, _rms(x, lw.ffn_norm, cfg.rms_eps))
            continue
        qkv = h @ lw.wqkv.dequantized().t()
        if lw.wqkv.bias is not None:
            qkv = qkv + lw.wqkv.bias.float()
        q = qkv[:, : hq * d].reshape(s, hq, d)
        k = qkv[:, hq * d:(hq + hkv) * d].reshape(s, hkv, d)
        v = qkv[:, (hq + hkv) * d:(hq + 2 * hkv) * d].reshape(s, hkv, d)
        gate = qkv[:, (hq + 2 * hkv) * d:] if cfg.attn_output_gate else None
        if lw.q_norm is not None:
            q = _rms(q, lw.q_norm, cfg.rms_eps)
            k = _rms(k, lw.k_norm, cfg.rms_eps)
        rd = 2 * sum(cfg.mrope_sections) if (cfg.mrope_sections and sum(cfg.mrope_sections) > 0) else cfg.rope_dim
        q = rope_ref(q, pos, cfg.rope_theta, rd)
        k = rope_ref(k, pos, cfg.rope_theta, rd)
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
        sc = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(d)
        mask = torch.ones(s, s, dtype=torch.bool, device=dev).tril()
        if cfg.sliding_window > 0:
            mask &= ~torch.ones(s, s, dtype=torch.bool, device=dev).tril(-cfg.sliding_window)
        sc = sc.masked_fill(~mask, float("-inf"))
        a = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), v).reshape(s, hq * d)
        if gate is not None:
            a = a * torch.sigmoid(gate)
        x = x + a @ lw.wo.dequantized().t()
        x = x + _ffn(cfg, lw, _rms(x, lw.ffn_norm, cfg.rms_eps))
    if return_hidden:
        return x
    hn = _rms(x, weights.final_norm, cfg.rms_eps)
    return hn @ weights.lm_head.dequantized().t()


def _deltanet_layer(cfg, ssm, h: torch.Tensor) -> torch.Tensor:
    """One gated Delta-Net layer over a whole sequence from an all-zero state (common/transformer.h:2861-3113)."""
    s = h.shape[0]
    ng, hv, ds, ck = cfg.ssm_n_heads_k, cfg.ssm_n_heads_v, cfg.ssm_head_dim, cfg.ssm_d_conv
    qd = cfg.ssm_qkv_dim
    proj = h @ ssm.w_in.dequantized().t()
    qkv, z = proj[:, :qd], proj[:, qd:]
    ab = h @ ssm.w_ab.float().t()
    sp = torch.nn.functional.softplus(ab[:, :hv] + ssm.dt_bias.float(), threshold=20.0)
    decay = torch.exp(sp * ssm.a.float())                                    # [S, hv]
    beta = torch.sigmoid(ab[:, hv:])
    pad = torch.cat([torch.zeros(ck - 1, qd, device=h.device), qkv], 0)      # causal window, zero history
    conv = sum(pad[f:f + s] * ssm.conv_w.float()[:, f] for f in range(ck))
    conv = conv * torch.sigmoid(conv)
    q = conv[:, : ng * ds].reshape(s, ng, ds)
    k = conv[:, ng * ds: 2 * ng * ds].reshape(s, ng, ds)
    v = conv[:, 2 * ng * ds:].reshape(s, hv, ds)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + cfg.rms_eps) * ds ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + cfg.rms_eps)
    grp = torch.arange(hv, device=h.device) % ng
    state = torch.zeros(hv, ds, ds, device=h.device)
    outs = []
    for t in range(s):
        qt, kt = q[t, grp], k[t, grp]
        state = state * decay[t, :, None, None]
        delta = (v[t] - torch.einsum("hrc,hc->hr", state, kt)) * beta[t, :, None]
        state = state + delta[:, :, None] * kt[:, None, :]
        outs.append(torch.einsum("hrc,hc->hr", state, qt))
    o = torch.stack(outs)                                                    # [S, hv, ds]
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * ssm.norm.float()
    zz = z.reshape(s, hv, ds)
    return (o * zz * torch.sigmoid(zz)).reshape(s, hv * ds) @ ssm.w_out.dequantized().t()


def _ffn(cfg, lw, h: torch.Tensor) -> torch.Tensor:
    """Dense SwiGLU or top-k MoE (+ sigmoid-gated shared expert) output for normalised input ``h``."""
    x = h
    if True:
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
            if lw.sh_gate_up is not None:
                fs = lw.sh_gate_up.n // 2
                r = h @ lw.sh_gate_up.dequantized().t()
                sh = (torch.nn.functional.silu(r[:, :fs]) * r[:, fs:]) @ lw.sh_down.dequantized().t()
                if lw.sh_gate is not None:
                    sh = sh * torch.sigmoid(h @ lw.sh_gate.float().t())
                y = y + sh
            return y
        f = lw.w_gate_up.n // 2
        r = h @ lw.w_gate_up.dequantized().t()
        return (torch.nn.functional.silu(r[:, :f]) * r[:, f:]) @ lw.w_down.dequantized().t()
