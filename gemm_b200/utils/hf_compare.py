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
