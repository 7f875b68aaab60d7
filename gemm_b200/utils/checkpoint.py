"""Inference-state checkpoints: save the KV cache of the live sequences (plus positions and pending tokens) and resume
later — e.g. to skip a long prefill when sweeping decode settings.

Counterpart of the reference's 'TPCP' files (a64fx/llm/tp_runner.c:155-563: magic + version, model and TP geometry,
cache position, next token, then per-layer K / V buffers; every header field is validated on load,
tp_cache_matches_model :356-387).  Our file: magic ``GBKV1\\n``, a JSON header line (geometry, sequences), then for every layer
the K and V rows of the used cache slots in sequence order: bf16, or with ``kv_format="q8"`` int8 rows followed by one f32 scale per
(slot, KV head) (``ops.kvquant``: about half the size, the reference's INT8 KV rule).  Layers of the hybrid models that keep a recurrent state
instead of K/V (gated Delta-Net) write, per live sequence, the f32 conv history and the f32 recurrent matrix of its state slot
(the reference stores conv state and recurrent state per layer as well, tp_runner.c:155-563).  A truncated or mismatching file
is rejected.
"""
from __future__ import annotations

import json
import struct
from typing import Dict, List

import torch

MAGIC = b"GBKV1\n"


def _geometry(engine) -> Dict:
    cfg = engine.cfg
    return {"arch": cfg.arch, "n_layers": len(engine.w.layers), "hidden": cfg.hidden, "n_kv_heads_local": _kv_rows(engine)[0],
            "head_dim": cfg.head_dim, "vocab": cfg.vocab, "tp_size": engine.w.tp_size, "tp_rank": engine.w.tp_rank,
            "ep_size": engine.w.ep_size, "ep_rank": engine.w.ep_rank, "fmt": engine.w.fmt,
            "ssm_layers": [i for i in range(len(engine.kv.k)) if engine.kv.k[i].shape[0] == 0]}


def _kv_rows(engine):
    """(kv heads, head dim) of the attention layers' cache rows (the recurrent layers hold 0-row tensors)."""
    for t in engine.kv.k:
        if t.shape[0] > 0:
            return t.shape[1], t.shape[2]
    return engine.kv.k[0].shape[1], engine.kv.k[0].shape[2]


def save_state(engine, path: str, next_tokens=None, kv_format: str = "bf16") -> None:
    """Write the cached K/V of all sequences of ``engine`` (a ``serve.engine.Engine``); ``kv_format`` "bf16" or "q8"."""
    if kv_format not in ("bf16", "q8"):
        raise ValueError(f"unknown KV format {kv_format!r}")
    from ..ops import kvquant
    ps = engine.page_size
    header = {"geometry": _geometry(engine), "seq_len": list(engine.seq_len), "page_size": ps, "kv_format": kv_format,
              "next_tokens": [int(t) for t in (next_tokens.tolist() if next_tokens is not None else [])]}
    slots = []
    for s, n in enumerate(engine.seq_len):
        pages = engine.seq_pages[s]
        for p in range(n):
            slots.append(pages[p // ps] * ps + p % ps)
    idx = torch.tensor(slots, dtype=torch.long, device=engine.device)
    with open(path, "wb") as f:
        f.write(MAGIC)
        hb = json.dumps(header).encode()
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        n_seq = len(engine.seq_len)
        for li in range(len(engine.kv.k)):
            if engine.kv.k[li].shape[0] == 0:
                # recurrent layer: the state slots of the live sequences (slot s belongs to sequence s in a static-batch engine)
                for t in (engine.kv.conv[li], engine.kv.rec[li]):
                    f.write(t[:n_seq].contiguous().cpu().numpy().tobytes())
                continue
            for t in (engine.kv.k[li], engine.kv.v[li]):
                rows = t[idx].contiguous()
                if kv_format == "q8":
                    q, sc = kvquant.quantize_q8(rows)
                    f.write(q.cpu().view(torch.uint8).numpy().tobytes())
                    f.write(sc.cpu().numpy().tobytes())
                else:
                    f.write(rows.cpu().view(torch.uint8).numpy().tobytes())


def load_state(engine, path: str) -> torch.Tensor:
    """Restore sequences into an empty ``engine``; returns the saved pending tokens (int32).  Raises on any mismatch."""
    with open(path, "rb") as f:
        if f.read(len(MAGIC)) != MAGIC:
            raise ValueError("not a KV state file (bad magic)")
        raw = f.read(8)
        if len(raw) != 8:
            raise ValueError("truncated KV state file")
        (hl,) = struct.unpack("<Q", raw)
        if hl > (1 << 26):
            raise ValueError("implausible header length")
        header = json.loads(f.read(hl))
        geo, mine = header["geometry"], _geometry(engine)
        for k, v in mine.items():
            if geo.get(k) != v:
                raise ValueError(f"KV state file does not match the model: {k} is {geo.get(k)!r} in the file, {v!r} here")
        if header["page_size"] <= 0:
            raise ValueError("bad page size")
        kv_format = header.get("kv_format", "bf16")
        if kv_format not in ("bf16", "q8"):
            raise ValueError(f"unknown KV format {kv_format!r} in the file")
        from ..ops import kvquant
        engine.reset()
        ps = engine.page_size
        slots = []
        for n in header["seq_len"]:
            engine.seq_pages.append([])
            engine.seq_len.append(0)
            s = len(engine.seq_pages) - 1
            engine._ensure_pages(s, n)
            engine.seq_len[s] = n
            pages = engine.seq_pages[s]
            slots.extend(pages[p // ps] * ps + p % ps for p in range(n))
        idx = torch.tensor(slots, dtype=torch.long, device=engine.device)
        hk, hd = _kv_rows(engine)
        row = hk * hd * 2
        n_seq = len(header["seq_len"])
        for li in range(len(engine.kv.k)):
            if engine.kv.k[li].shape[0] == 0:
                for t in (engine.kv.conv[li], engine.kv.rec[li]):
                    nb = n_seq * t[0].numel() * 4
                    buf = f.read(nb)
                    if len(buf) != nb:
                        raise ValueError("truncated KV state file")
                    t[:n_seq] = torch.frombuffer(bytearray(buf), dtype=torch.float32).reshape(n_seq, *t.shape[1:]).to(engine.device)
                continue
            for t in (engine.kv.k[li], engine.kv.v[li]):
                if kv_format == "q8":
                    nq, ns = len(slots) * (row // 2), len(slots) * t.shape[1] * 4
                    buf, sbuf = f.read(nq), f.read(ns)
                    if len(buf) != nq or len(sbuf) != ns:
                        raise ValueError("truncated KV state file")
                    q = torch.frombuffer(bytearray(buf), dtype=torch.int8).reshape(len(slots), t.shape[1], t.shape[2])
                    sc = torch.frombuffer(bytearray(sbuf), dtype=torch.float32).reshape(len(slots), t.shape[1])
                    t[idx] = kvquant.dequantize_q8(q.to(engine.device), sc.to(engine.device))
                    continue
                buf = f.read(len(slots) * row)
                if len(buf) != len(slots) * row:
                    raise ValueError("truncated KV state file")
                vals = torch.frombuffer(bytearray(buf), dtype=torch.uint8).view(torch.bfloat16).reshape(len(slots), t.shape[1], t.shape[2])
                t[idx] = vals.to(engine.device)
    return torch.tensor(header["next_tokens"], dtype=torch.int32)
