"""Weight stager: cut a checkpoint into per-rank files in the run-time format, plus a manifest.

Counterpart of the reference's ``*_stage.c`` tools (common/m3_stage.c:59-69,121-123, common/glm5_stage.c,
a64fx/llm/ds4f_stage.c): experts are kept by the rank that owns them, dense tensors are TP-sliced, and every rank later
loads only its own blob.  Here a blob is a safetensors file holding exactly what the kernels consume (bf16 matrices, or
e4m3 bytes + E8M0 scale atoms for MXFP8), so start-up is a plain read without re-quantising.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch

from ..models import loader
from ..models.config import ModelConfig
from ..models.weights import LayerWeights, LinearWeight, ModelWeights, build_weights
from ..ops.mxfp8 import MxTensor


def _put_linear(out: Dict[str, torch.Tensor], key: str, lw: Optional[LinearWeight]) -> None:
    if lw is None:
        return
    if lw.fmt == "bf16":
        out[key + ".w"] = lw.untiled_data()
    else:
        out[key + ".q"] = lw.untiled_data()
        out[key + ".sf"] = lw.mx.sf
    if lw.bias is not None:
        out[key + ".bias"] = lw.bias
    out[key + ".meta"] = torch.tensor([lw.n, lw.k, lw.groups, lw.rows_per_group, lw.mx.rows if lw.mx is not None else 0], dtype=torch.int64)


def _get_linear(st, key: str, fmt_hint: str) -> Optional[LinearWeight]:
    if key + ".meta" not in st.info:
        return None
    n, k, groups, rpg, rows = [int(v) for v in st.get(key + ".meta")]
    bias = st.get(key + ".bias").clone() if key + ".bias" in st.info else None
    if key + ".w" in st.info:
        return LinearWeight("bf16", n, k, w=st.get(key + ".w").clone(), bias=bias, groups=groups, rows_per_group=rpg)
    return LinearWeight("mxfp8", n, k, mx=MxTensor(st.get(key + ".q").clone(), st.get(key + ".sf").clone(), rows, k), bias=bias, groups=groups,
                        rows_per_group=rpg)


def stage(cfg: ModelConfig, src, out_dir: str, fmt: str, tp_size: int = 1, ep_size: int = 1, shard_vocab: bool = False) -> None:
    """Write ``rankNN.safetensors`` for every rank of a (tp_size x ep_size) layout and ``manifest.json``."""
    os.makedirs(out_dir, exist_ok=True)
    world = max(tp_size, ep_size)
    for r in range(world):
        w = build_weights(cfg, src, fmt, "cpu", tp_rank=r if tp_size > 1 else 0, tp_size=tp_size, ep_rank=r if ep_size > 1 else 0,
                          ep_size=ep_size, shard_vocab=shard_vocab)
        out: Dict[str, torch.Tensor] = {"embed": w.embed, "final_norm": w.final_norm}
        _put_linear(out, "lm_head", w.lm_head)
        for li, l in enumerate(w.layers):
            p = f"l{li}."
            out[p + "attn_norm"], out[p + "ffn_norm"] = l.attn_norm, l.ffn_norm
            for nm in ("q_norm", "k_norm", "router", "router_bias"):
                t = getattr(l, nm)
                if t is not None:
                    out[p + nm] = t
            for nm in ("wqkv", "wo", "w_gate_up", "w_down", "w13", "w2"):
                _put_linear(out, p + nm, getattr(l, nm))
        loader.save_safetensors(out, os.path.join(out_dir, f"rank{r:02d}.safetensors"))
    with open(os.path.join(out_dir, "manifest.json"), "w") as fh:
        json.dump({"config": cfg.to_dict(), "fmt": fmt, "tp_size": tp_size, "ep_size": ep_size, "shard_vocab": shard_vocab,
                   "files": [f"rank{r:02d}.safetensors" for r in range(world)]}, fh)


def load_staged(out_dir: str, rank: int, device="cuda") -> ModelWeights:
    """Load the blob of ``rank`` written by ``stage``."""
    with open(os.path.join(out_dir, "manifest.json")) as fh:
        man = json.load(fh)
    cfg = ModelConfig(**man["config"])
    st = loader.SafetensorsFile(os.path.join(out_dir, man["files"][rank]))
    fmt = man["fmt"]
    layers = []
    for li in range(cfg.n_layers):
        p = f"l{li}."
        g = lambda nm: st.get(p + nm).clone() if (p + nm) in st.info else None
        layers.append(LayerWeights(attn_norm=g("attn_norm"), wqkv=_get_linear(st, p + "wqkv", fmt), wo=_get_linear(st, p + "wo", fmt),
                                   ffn_norm=g("ffn_norm"), q_norm=g("q_norm"), k_norm=g("k_norm"), w_gate_up=_get_linear(st, p + "w_gate_up", fmt),
                                   w_down=_get_linear(st, p + "w_down", fmt), router=g("router"), router_bias=g("router_bias"),
                                   w13=_get_linear(st, p + "w13", fmt), w2=_get_linear(st, p + "w2", fmt)))
    tp, ep = man["tp_size"], man["ep_size"]
    w = ModelWeights(cfg=cfg, embed=st.get("embed").clone(), layers=layers, final_norm=st.get("final_norm").clone(),
                     lm_head=_get_linear(st, "lm_head", "bf16"), fmt=fmt, tp_rank=rank if tp > 1 else 0, tp_size=tp, ep_rank=rank if ep > 1 else 0,
                     ep_size=ep)
    if man.get("shard_vocab") and tp > 1:
        from ..models.weights import shard_range
        w.vocab_start = shard_range(cfg.vocab, tp, rank)[0]
    return w.to(device)
