"""Sampling ops (csrc/kernels/sampler.cu): greedy arg-max and temperature / top-k / top-p sampling.

Reference: transformer_sample_topk (common/transformer.h:5415-5467) and sample_token
(server/server_llm.c:220-284).  Ties resolve to the lower token id.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from .. import _native

_c, _i, _f, _l, _u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_long, ctypes.c_ulonglong


def _p(t):
    return _c(t.data_ptr()) if t is not None else _c(0)


def argmax(logits: torch.Tensor, idx_offset: int = 0, want_value: bool = False):
    """Row-wise arg-max of ``logits [B, V]`` (f32 or bf16) -> int32 [B] (+ f32 values)."""
    b, v = logits.shape
    if not logits.is_cuda:
        lf = torch.nan_to_num(logits.float(), nan=-3.4e38)
        val, idx = lf.max(dim=-1)
        # torch.max returns the first maximal index on CPU
        idx = (idx + idx_offset).to(torch.int32)
        return (idx, val) if want_value else idx
    out = torch.empty(b, dtype=torch.int32, device=logits.device)
    val = torch.empty(b, dtype=torch.float32, device=logits.device) if want_value else None
    dt = 0 if logits.dtype == torch.float32 else 1
    stream = _c(torch.cuda.current_stream().cuda_stream)
    if v >= 16384:
        chunks = max(1, min(64, 1184 // max(1, b)))
        pv = torch.empty(chunks * b, dtype=torch.float32, device=logits.device)
        pi = torch.empty(chunks * b, dtype=torch.int32, device=logits.device)
        rc = _native.cuda().gb_argmax2(_p(logits), _p(out), _p(val), _p(pv), _p(pi), _i(b), _i(v), _l(logits.stride(0)), _i(dt),
                                       _i(idx_offset), _i(chunks), stream)
        _native.check(rc, "gb_argmax2", n=2)
    else:
        rc = _native.cuda().gb_argmax(_p(logits), _p(out), _p(val), _i(b), _i(v), _l(logits.stride(0)), _i(dt), _i(idx_offset), stream)
        _native.check(rc, "gb_argmax")
    return (out, val) if want_value else out


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0,
           step: int = 0, step_ctr: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Draw one token per row.  ``temperature <= 0`` means greedy.  At most 1024 candidates are kept.  The random numbers are a
    function of ``(seed, step + step_ctr[0], row)``; ``step_ctr`` (int64 [1], on the logits' device) is read by the kernel, so a
    launch captured in a CUDA graph draws from a new step at every replay."""
    if temperature <= 0.0:
        return argmax(logits)
    b, v = logits.shape
    if not logits.is_cuda:
        return sample_ref(logits, temperature, top_k, top_p, seed, step + (int(step_ctr[0]) if step_ctr is not None else 0))
    out = torch.empty(b, dtype=torch.int32, device=logits.device)
    dt = 0 if logits.dtype == torch.float32 else 1
    rc = _native.cuda().gb_sample(_p(logits), _p(out), _i(b), _i(v), _l(logits.stride(0)), _i(dt), _f(temperature), _i(top_k),
                                  _f(top_p), _u64(seed), _u64(step), _p(step_ctr), _c(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "gb_sample")
    return out


def candidate_set_ref(logits_row: torch.Tensor, temperature: float, top_k: int, top_p: float):
    """Token ids that may be drawn and their probabilities (descending), for tests."""
    v = logits_row.numel()
    kk = min(1024, v) if top_k <= 0 or top_k > 1024 else min(top_k, v)
    vals, idx = torch.sort(logits_row.float(), descending=True, stable=True)
    vals, idx = vals[:kk], idx[:kk]
    p = torch.softmax(vals / max(temperature, 1e-6), dim=-1)
    if top_p < 1.0:
        cum = torch.cumsum(p, 0)
        keep = int((cum >= top_p).nonzero()[0]) + 1 if bool((cum >= top_p).any()) else kk
        p, idx = p[:keep], idx[:keep]
        p = p / p.sum()
    return idx, p


def sample_ref(logits, temperature, top_k, top_p, seed, step):
    g = torch.Generator().manual_seed(seed * 1000003 + step)
    out = []
    for r in range(logits.shape[0]):
        idx, p = candidate_set_ref(logits[r], temperature, top_k, top_p)
        out.append(int(idx[torch.multinomial(p, 1, generator=g)]))
    return torch.tensor(out, dtype=torch.int32)
