"""Greedy comparison against Hugging Face ``transformers`` running the same checkpoint in fp32: the independent reference
implementation of the Qwen2 / Qwen3 / Qwen3-MoE architectures (the reference project does the same with its Python server,
ref/llm/llm_server.py, and reports token agreement and edit distance of the greedy continuations).

``compare(path_or_weights, ...)`` runs the prompt through both, decodes ``steps`` tokens greedily on each side (each side on its
own continuation) and returns per-step logit differences, the token agreement and the Levenshtein distance.  Synthetic models are
written as an HF checkpoint directory first (``models.loader.save_hf_checkpoint``), so both sides read the same bf16 weights.
"""
from __future__ import annotations

import tempfile
from typing import Dict, List, Optional, Sequence

import torch


def edit_distance(a: Sequence[int], b: Sequence[int]) -> int:
    d = list(range(len(b) + 1))
    for i, x in enumerate(a, 1):
        prev, d[0] = d[0], i
        for j, y in enumerate(b, 1):
            prev, d[j] = d[j], min(d[j] + 1, d[j - 1] + 1, prev + (x != y))
    return d[-1]


def hf_greedy(path: str, prompt: Sequence[int], steps: int):
    """(tokens, logits per step) of the HF model at ``path`` (fp32, eager attention, KV cache off: every step re-runs the
    sequence, which keeps this arm independent of any cache implementation)."""
    import transformers
    model = transformers.AutoModelForCausalLM.from_pretrained(path, dtype=torch.float32, attn_implementation="eager")
    model.eval()
    toks, rows = list(prompt), []
    with torch.no_grad():
        for _ in range(steps):
            logits = model(torch.tensor([toks]), use_cache=False).logits[0, -1].float()
            rows.append(logits)
            toks.append(int(logits.argmax()))
    return toks[len(prompt):], rows


def ours_greedy(weights, prompt: Sequence[int], steps: int, device: str = "cpu"):
    from ..models.transformer import ForwardBatch, KvCache, Transformer
    cfg = weights.cfg
    page = 16 if device == "cpu" else 128
    n_pages = (len(prompt) + steps + page) // page + 1
    bt = torch.arange(n_pages, dtype=torch.int32).unsqueeze(0)
    m = Transformer(weights, KvCache.allocate(cfg, n_pages, page, device))
    toks, rows = list(prompt), []
    fb = ForwardBatch.build([len(toks)], [0], torch.tensor(toks), bt, page, cfg.n_heads, cfg.n_kv_heads, device)
    logits = m.forward(fb).float().cpu()[0]
    for _ in range(steps):
        rows.append(logits)
        toks.append(int(logits.argmax()))
        fb = ForwardBatch.build([1], [len(toks) - 1], torch.tensor(toks[-1:]), bt, page, cfg.n_heads, cfg.n_kv_heads, device)
        logits = m.forward(fb).float().cpu()[0]
    return toks[len(prompt):], rows


def compare(model: str, prompt: Sequence[int], steps: int = 8, fmt: str = "bf16", device: str = "cpu", seed: int = 0) -> Dict:
    """``model``: an HF checkpoint directory, or ``synthetic:<config name>`` (random weights, written to a temporary directory)."""
    from ..models import loader
    from ..models.config import get_config
    from ..models.weights import RandomSource
    tmp: Optional[tempfile.TemporaryDirectory] = None
    if model.startswith("synthetic:"):
        cfg = get_config(model.split(":", 1)[1])
        if cfg.arch not in ("qwen2", "qwen3", "qwen3moe"):
            raise ValueError(f"no Hugging Face arm for architecture {cfg.arch}")
        tmp = tempfile.TemporaryDirectory()
        loader.save_hf_checkpoint(cfg, RandomSource(cfg, seed), tmp.name)
        path = tmp.name
    else:
        path = model
    try:
        w = loader.load_safetensors(path, fmt, device)
        ours_t, ours_l = ours_greedy(w, prompt, steps, device)
        hf_t, hf_l = hf_greedy(path, prompt, steps)
    finally:
        if tmp is not None:
            tmp.cleanup()
    n = min(len(ours_t), len(hf_t))
    # the logit comparison stops where the two continuations part (after that the sides see different contexts)
    same = next((i for i in range(n) if ours_t[i] != hf_t[i]), n)
    rel: List[float] = [float((ours_l[i] - hf_l[i]).norm() / (hf_l[i].norm() + 1e-12)) for i in range(min(same + 1, n))]
    return {"prompt_len": len(prompt), "steps": steps, "ours_tokens": ours_t, "hf_tokens": hf_t, "logit_rel_per_step": [round(r, 5) for r in rel],
            "token_agreement": sum(int(a == b) for a, b in zip(ours_t, hf_t)) / max(1, n), "edit_distance": edit_distance(ours_t, hf_t)}


def hf_qwen35_model(cfg, src):
    """A Hugging Face ``Qwen3_5ForCausalLM`` (fp32, eager) holding the weights of ``src`` (a tensor source with GGUF names, e.g.
    ``models.weights.RandomSource``) for a hybrid configuration (gated Delta-Net + gated attention layers; dense FFN or MoE with a
    gated shared expert: ``Qwen3_5MoeForCausalLM``).

    What differs between the two layouts: HF's RMSNorm multiplies by ``1 + w`` (GGUF files carry ``1 + w``); HF's value head ``j`` of
    a Delta-Net layer uses key head ``j // (Hv / Hk)``, the GGUF order is ``j % Hk`` (common/transformer.h:2861-3113), so value
    heads (rows of the V block of ``attn_qkv``, of ``attn_gate``, ``ssm_alpha``, ``ssm_beta``, conv channels, ``ssm_a``, ``ssm_dt.bias``,
    columns of ``ssm_out``) are permuted; ``ssm_a`` is ``-exp(A_log)``."""
    if not cfg.attn_output_gate or cfg.full_attention_interval <= 0:
        raise ValueError("the Hugging Face arm for hybrid models covers the qwen35 / qwen35moe architectures")
    if cfg.is_moe:
        # the MoE variant: softmax router with renormalised top-k, stacked experts ([gate | up] rows), shared expert behind a sigmoid gate
        from transformers.models.qwen3_5_moe import modeling_qwen3_5_moe as M
        from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeTextConfig as Qwen3_5TextConfig
        extra = dict(moe_intermediate_size=cfg.expert_ffn, shared_expert_intermediate_size=cfg.shared_expert_ffn, num_experts=cfg.n_experts,
                     num_experts_per_tok=cfg.n_experts_used)
    else:
        from transformers.models.qwen3_5 import modeling_qwen3_5 as M
        from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig
        extra = dict(intermediate_size=cfg.ffn)
    g_, hv, ds, h = cfg.ssm_n_heads_k, cfg.ssm_n_heads_v, cfg.ssm_head_dim, cfg.hidden
    r_ = hv // g_
    perm = torch.tensor([(j % r_) * g_ + (j // r_) for j in range(hv)])
    hc = Qwen3_5TextConfig(
        hidden_size=h, num_hidden_layers=cfg.n_layers, num_attention_heads=cfg.n_heads, num_key_value_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
        vocab_size=cfg.vocab, rms_norm_eps=cfg.rms_eps, linear_conv_kernel_dim=cfg.ssm_d_conv, linear_key_head_dim=ds, **extra,
        linear_value_head_dim=ds, linear_num_key_heads=g_, linear_num_value_heads=hv,
        layer_types=["linear_attention" if cfg.is_ssm_layer(i) else "full_attention" for i in range(cfg.n_layers)],
        rope_parameters={"rope_type": "default", "rope_theta": cfg.rope_theta, "partial_rotary_factor": (cfg.rope_dim or cfg.head_dim) / cfg.head_dim,
                         "mrope_section": list(cfg.mrope_sections[:3]) if cfg.mrope_sections else [11, 11, 10]},
        tie_word_embeddings=False, attention_bias=False, max_position_embeddings=max(cfg.max_seq_len, 4096), hidden_act="silu")
    hc._attn_implementation = "eager"
    model = (M.Qwen3_5MoeForCausalLM if cfg.is_moe else M.Qwen3_5ForCausalLM)(hc).float().eval()
    f32 = lambda name, shape: src.get(name, shape).float()
    qd, di, kdim = cfg.ssm_qkv_dim, cfg.ssm_d_inner, g_ * ds
    vrows = (perm[:, None] * ds + torch.arange(ds)[None, :]).reshape(-1)
    chan = torch.cat([torch.arange(2 * kdim), 2 * kdim + vrows])
    new = {"model.embed_tokens.weight": f32("token_embd.weight", (cfg.vocab, h)), "lm_head.weight": f32("output.weight", (cfg.vocab, h)),
           "model.norm.weight": f32("output_norm.weight", (h,)) - 1.0}
    for li in range(cfg.n_layers):
        p, q = f"blk.{li}.", f"model.layers.{li}."
        new[q + "input_layernorm.weight"] = f32(p + "attn_norm.weight", (h,)) - 1.0
        new[q + "post_attention_layernorm.weight"] = f32(p + "ffn_norm.weight", (h,)) - 1.0
        if cfg.is_moe:
            e, it, fs = cfg.n_experts, cfg.expert_ffn, cfg.shared_expert_ffn
            new[q + "mlp.gate.weight"] = f32(p + "ffn_gate_inp.weight", (e, h))
            new[q + "mlp.experts.gate_up_proj"] = torch.stack([torch.cat([src.get_expert(p + "ffn_gate_exps.weight", x, (it, h)).float(),
                                                                             src.get_expert(p + "ffn_up_exps.weight", x, (it, h)).float()]) for x in range(e)])
            new[q + "mlp.experts.down_proj"] = torch.stack([src.get_expert(p + "ffn_down_exps.weight", x, (h, it)).float() for x in range(e)])
            for a, b_, shp in (("ffn_gate_shexp", "gate_proj", (fs, h)), ("ffn_up_shexp", "up_proj", (fs, h)), ("ffn_down_shexp", "down_proj", (h, fs))):
                new[q + f"mlp.shared_expert.{b_}.weight"] = f32(p + a + ".weight", shp)
            new[q + "mlp.shared_expert_gate.weight"] = f32(p + "ffn_gate_inp_shexp.weight", (h,)).reshape(1, h)
        else:
            for a, b_, shp in (("ffn_gate", "gate_proj", (cfg.ffn, h)), ("ffn_up", "up_proj", (cfg.ffn, h)), ("ffn_down", "down_proj", (h, cfg.ffn))):
                new[q + f"mlp.{b_}.weight"] = f32(p + a + ".weight", shp)
        if cfg.is_ssm_layer(li):
            la = q + "linear_attn."
            new[la + "in_proj_qkv.weight"] = f32(p + "attn_qkv.weight", (qd, h))[chan]
            new[la + "in_proj_z.weight"] = f32(p + "attn_gate.weight", (di, h))[vrows]
            new[la + "in_proj_a.weight"] = f32(p + "ssm_alpha.weight", (hv, h))[perm]
            new[la + "in_proj_b.weight"] = f32(p + "ssm_beta.weight", (hv, h))[perm]
            new[la + "conv1d.weight"] = f32(p + "ssm_conv1d.weight", (qd, cfg.ssm_d_conv))[chan].unsqueeze(1)
            new[la + "A_log"] = torch.log(-f32(p + "ssm_a", (hv,)))[perm]
            new[la + "dt_bias"] = f32(p + "ssm_dt.bias", (hv,))[perm]
            new[la + "norm.weight"] = f32(p + "ssm_norm.weight", (ds,))
            new[la + "out_proj.weight"] = f32(p + "ssm_out.weight", (h, di))[:, vrows]
        else:
            sa = q + "self_attn."
            new[sa + "q_proj.weight"] = f32(p + "attn_q.weight", (2 * cfg.q_dim, h))          # [q_h | gate_h] per head in both layouts
            new[sa + "k_proj.weight"] = f32(p + "attn_k.weight", (cfg.kv_dim, h))
            new[sa + "v_proj.weight"] = f32(p + "attn_v.weight", (cfg.kv_dim, h))
            new[sa + "o_proj.weight"] = f32(p + "attn_output.weight", (h, cfg.q_dim))
            new[sa + "q_norm.weight"] = f32(p + "attn_q_norm.weight", (cfg.head_dim,)) - 1.0
            new[sa + "k_norm.weight"] = f32(p + "attn_k_norm.weight", (cfg.head_dim,)) - 1.0
    model.load_state_dict(new)
    return model


def hf_qwen3vl_text_model(cfg, src):
    """``(Qwen3VLTextModel in fp32, LM head matrix)`` holding the weights of ``src`` (GGUF names) for a dense Qwen3 configuration with
    M-RoPE sections: the text side of Qwen3-VL, which takes embedding rows, (t, h, w) positions and DeepStack features."""
    from transformers.models.qwen3_vl import modeling_qwen3_vl as M
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLTextConfig
    h = cfg.hidden
    hc = Qwen3VLTextConfig(hidden_size=h, num_hidden_layers=cfg.n_layers, num_attention_heads=cfg.n_heads, num_key_value_heads=cfg.n_kv_heads,
                           head_dim=cfg.head_dim, intermediate_size=cfg.ffn, vocab_size=cfg.vocab, rms_norm_eps=cfg.rms_eps,
                           rope_parameters={"rope_type": "default", "rope_theta": cfg.rope_theta, "mrope_section": list(cfg.mrope_sections[:3])},
                           tie_word_embeddings=False, attention_bias=False, max_position_embeddings=max(cfg.max_seq_len, 4096))
    hc._attn_implementation = "eager"
    model = M.Qwen3VLTextModel(hc).float().eval()
    sd = model.state_dict()
    f32 = lambda name, shape: src.get(name, shape).float()
    new = {"embed_tokens.weight": f32("token_embd.weight", (cfg.vocab, h)), "norm.weight": f32("output_norm.weight", (h,))}
    names = {"attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm", "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj",
             "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj", "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm",
             "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj"}
    for li in range(cfg.n_layers):
        for a, b in names.items():
            k = f"layers.{li}.{b}.weight"
            new[k] = f32(f"blk.{li}.{a}.weight", tuple(sd[k].shape))
    model.load_state_dict(new)
    return model, f32("output.weight", (cfg.vocab, h))
