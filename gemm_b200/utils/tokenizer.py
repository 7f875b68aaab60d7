"""Tokenizer: Python face of csrc/host/tokenizer.cc (byte-level BPE with Qwen2 / Qwen3.5 pre-tokenisation).

API parity with the reference (common/bpe_tokenizer.h:28-50): load from the GGUF vocabulary arrays, encode,
token -> string, byte-decode, EOS / EOT ids.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence

import numpy as np

from .. import _native


def _lib():
    lib = _native.host()
    if not getattr(lib, "_tok_ready", False):
        lib.gbh_tok_create.restype = ctypes.c_void_p
        lib.gbh_tok_encode.restype = ctypes.c_long
        lib.gbh_tok_decode.restype = ctypes.c_long
        lib.gbh_tok_vocab_size.restype = ctypes.c_long
        lib._tok_ready = True
    return lib


class Tokenizer:
    def __init__(self, tokens: Sequence[bytes], merges: Sequence[bytes], token_types: Optional[Sequence[int]] = None, pre: str = "qwen2",
                 special_ids: Optional[Dict[str, int]] = None):
        toks = [t.encode() if isinstance(t, str) else bytes(t) for t in tokens]
        mrg = [m.encode() if isinstance(m, str) else bytes(m) for m in merges]
        tl = (ctypes.c_uint64 * max(1, len(toks)))(*[len(t) for t in toks])
        ml = (ctypes.c_uint64 * max(1, len(mrg)))(*[len(m) for m in mrg])
        types = None
        if token_types is not None:
            types = (ctypes.c_int * len(toks))(*[int(x) for x in token_types])
        self._h = _lib().gbh_tok_create(b"".join(toks), tl, ctypes.c_long(len(toks)), b"".join(mrg), ml, ctypes.c_long(len(mrg)), types,
                                        pre.encode())
        self.pre = pre
        self.special_ids = dict(special_ids or {})
        self.n_vocab = len(toks)
        self._tokens = toks

    @classmethod
    def from_gguf(cls, f) -> "Tokenizer":
        """Build from an open ``GGUFFile`` (keys ``tokenizer.ggml.tokens`` [required], ``.merges``, ``.token_type``, ``.pre``, ``.model``,
        ``.{eos,bos,eot,padding,unknown}_token_id``)."""
        m = f.metadata
        if "tokenizer.ggml.tokens" not in m:
            raise KeyError("the GGUF file has no tokenizer.ggml.tokens array")
        pre = m.get("tokenizer.ggml.pre", "qwen2")
        if m.get("tokenizer.ggml.model") == "gemma4":
            pre = "gemma4"
        ids = {}
        for name in ("eos", "bos", "eot", "padding", "unknown"):
            key = f"tokenizer.ggml.{name}_token_id"
            if key in m:
                ids[name] = int(m[key])
        types = m.get("tokenizer.ggml.token_type")
        return cls(m["tokenizer.ggml.tokens"], m.get("tokenizer.ggml.merges", []), None if types is None else list(types), pre, ids)

    def encode(self, text: str, parse_special: bool = True) -> List[int]:
        b = text.encode("utf-8")
        cap = max(16, len(b) + 8)
        buf = (ctypes.c_int * cap)()
        n = _lib().gbh_tok_encode(ctypes.c_void_p(self._h), b, ctypes.c_long(len(b)), 1 if parse_special else 0, buf, ctypes.c_long(cap))
        if n > cap:
            buf = (ctypes.c_int * n)()
            n = _lib().gbh_tok_encode(ctypes.c_void_p(self._h), b, ctypes.c_long(len(b)), 1 if parse_special else 0, buf, ctypes.c_long(n))
        return list(buf[:n])

    def decode_bytes(self, ids: Sequence[int]) -> bytes:
        arr = (ctypes.c_int * max(1, len(ids)))(*[int(i) for i in ids])
        cap = 16 * max(1, len(ids)) + 64
        out = ctypes.create_string_buffer(cap)
        n = _lib().gbh_tok_decode(ctypes.c_void_p(self._h), arr, ctypes.c_long(len(ids)), out, ctypes.c_long(cap))
        if n > cap:
            out = ctypes.create_string_buffer(n)
            n = _lib().gbh_tok_decode(ctypes.c_void_p(self._h), arr, ctypes.c_long(len(ids)), out, ctypes.c_long(n))
        return out.raw[:n]

    def decode(self, ids: Sequence[int]) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")

    def token_to_str(self, i: int) -> bytes:
        return self._tokens[i]

    @property
    def eos_id(self) -> int:
        return self.special_ids.get("eos", -1)

    @property
    def eot_id(self) -> int:
        return self.special_ids.get("eot", -1)

    def __del__(self):
        try:
            if self._h:
                _lib().gbh_tok_free(ctypes.c_void_p(self._h))
                self._h = None
        except Exception:
            pass


def byte_alphabet() -> List[str]:
    """The 256 printable stand-ins of the GPT-2 byte-level alphabet (index = byte value)."""
    out, n = [], 0
    for b in range(256):
        keep = (33 <= b <= 126) or (161 <= b <= 172) or (174 <= b <= 255)
        out.append(chr(b) if keep else chr(256 + n))
        if not keep:
            n += 1
    return out


def toy_vocab(corpus: str, n_merges: int = 200):
    """A small trained byte-level BPE vocabulary (tokens, merges) for tests and synthetic checkpoints."""
    alpha = byte_alphabet()
    words: Dict[tuple, int] = {}
    for w in corpus.split(" "):
        sym = tuple(alpha[b] for b in (" " + w).encode("utf-8"))
        if sym:
            words[sym] = words.get(sym, 0) + 1
    tokens = list(alpha)
    merges: List[str] = []
    for _ in range(n_merges):
        pairs: Dict[tuple, int] = {}
        for sym, c in words.items():
            for a, b in zip(sym, sym[1:]):
                pairs[(a, b)] = pairs.get((a, b), 0) + c
        if not pairs:
            break
        (a, b), cnt = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))
        if cnt < 2:
            break
        merges.append(f"{a} {b}")
        tokens.append(a + b)
        new_words = {}
        for sym, c in words.items():
            out, i = [], 0
            while i < len(sym):
                if i + 1 < len(sym) and sym[i] == a and sym[i + 1] == b:
                    out.append(a + b); i += 2
                else:
                    out.append(sym[i]); i += 1
            new_words[tuple(out)] = new_words.get(tuple(out), 0) + c
        words = new_words
    return tokens, merges
