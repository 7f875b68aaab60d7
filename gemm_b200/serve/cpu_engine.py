"""``CpuEngine``: the native CPU engine (csrc/host/cpu_engine.cc) behind a small Python class.

Dense Qwen2 / Qwen3 GGUF checkpoints run from their memory-mapped ggml blocks on a pool of threads: batched prefill, single-token
decode steps, greedy sampling.  Counterpart of the reference's ``transformer_load -> forward -> argmax`` loop
(cpu/llm/test_transformer.c:209-345 over common/transformer.h)."""
from __future__ import annotations

import ctypes
from typing import List, Sequence, Tuple

import numpy as np

from .. import _native


def _lib():
    lib = _native.host()
    if not getattr(lib, "_cpu_engine_ready", False):
        lib.gbh_cpu_engine_load.restype = ctypes.c_void_p
        lib.gbh_cpu_engine_load.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
        lib.gbh_cpu_engine_free.argtypes = [ctypes.c_void_p]
        lib.gbh_cpu_engine_vocab.argtypes = [ctypes.c_void_p]
        lib.gbh_cpu_engine_threads.argtypes = [ctypes.c_void_p]
        lib.gbh_cpu_engine_profile.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        lib.gbh_cpu_engine_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        lib.gbh_cpu_engine_generate.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                                ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]
        lib._cpu_engine_ready = True
    return lib


class CpuEngine:
    def __init__(self, gguf_path: str, max_seq_len: int = 4096, threads: int = 0):
        self._h = _lib().gbh_cpu_engine_load(gguf_path.encode(), max_seq_len, threads)
        if not self._h:
            raise RuntimeError(_lib().gbh_last_error().decode(errors="replace"))
        self.vocab = _lib().gbh_cpu_engine_vocab(self._h)
        self.threads = _lib().gbh_cpu_engine_threads(self._h)

    def forward(self, tokens: Sequence[int], pos0: int = 0) -> np.ndarray:
        """Batched pass over ``tokens`` at positions ``pos0 ...`` (the KV cache is filled); fp32 logits of the last token."""
        ids = np.asarray(tokens, dtype=np.int32)
        out = np.empty(self.vocab, dtype=np.float32)
        if _lib().gbh_cpu_engine_forward(self._h, ids.ctypes.data, len(ids), pos0, out.ctypes.data) != 0:
            raise RuntimeError(_lib().gbh_last_error().decode(errors="replace"))
        return out

    PHASES = ("qkv", "rope_cache", "attention", "o_proj", "norm_residual", "gate_up_silu", "down", "head")

    def profile(self, reset: bool = True) -> dict:
        """Seconds per phase since the engine was loaded or since the last reset (the reference prints such tables from
        common/profiler.h)."""
        buf = (ctypes.c_double * 9)()
        _lib().gbh_cpu_engine_profile(self._h, buf, 1 if reset else 0)
        return {k: float(buf[i]) for i, k in enumerate(self.PHASES)}

    def generate(self, prompt: Sequence[int], max_new_tokens: int) -> Tuple[List[int], float, float]:
        """Greedy generation.  Returns ``(tokens, prefill seconds, decode seconds)``."""
        ids = np.asarray(prompt, dtype=np.int32)
        out = np.empty(max_new_tokens, dtype=np.int32)
        tp, td = ctypes.c_double(), ctypes.c_double()
        if _lib().gbh_cpu_engine_generate(self._h, ids.ctypes.data, len(ids), max_new_tokens, out.ctypes.data, ctypes.byref(tp), ctypes.byref(td)) != 0:
            raise RuntimeError(_lib().gbh_last_error().decode(errors="replace"))
        return out.tolist(), tp.value, td.value

    def close(self) -> None:
        if self._h:
            _lib().gbh_cpu_engine_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CpuEngineModel:
    """The native engine behind the interface ``serve.sequential.SequentialLLM`` drives (``reset`` / ``forward`` on ``[1, T]`` ids,
    logits of the last token), so that ``generate`` and the HTTP server run a GGUF checkpoint on a machine without a GPU, which is
    what the reference's server does with its CPU engine (server/server_llm.c over common/transformer.h)."""

    def __init__(self, gguf_path: str, max_seq_len: int = 4096, threads: int = 0):
        import torch
        self._torch = torch
        self.engine = CpuEngine(gguf_path, max_seq_len=max_seq_len, threads=threads)
        self.max_seq_len, self.pos = max_seq_len, 0

    def reset(self, batch: int = 1, max_pos: int = 0) -> None:
        if batch != 1:
            raise ValueError("the CPU engine runs one sequence at a time")
        if max_pos > self.max_seq_len:
            raise ValueError(f"the request needs {max_pos} positions, the cache holds {self.max_seq_len}")
        self.pos = 0                                             # the cache is overwritten from position 0 on

    def forward(self, ids):
        row = [int(v) for v in ids.reshape(-1).tolist()]
        logits = self.engine.forward(row, self.pos)
        self.pos += len(row)
        return self._torch.from_numpy(logits)[None]
