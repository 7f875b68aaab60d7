"""INT8 codec for KV rows: ``[rows, head_dim]`` bf16 <-> int8 + one f32 scale per row (a row = one cache slot of one KV head).

``scale = amax / 127``, ``q = round(x / scale)`` clamped to [-127, 127]: the rule of the reference's ``kv_cache_store_q8``
(cuda/llm/cuda_llm_runner.c:220-241) with the maximum taken over the whole head.  Used by ``utils.checkpoint`` to write KV state
files at half the size; the attention kernels read bf16 pages.
"""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from .. import _native

_c, _i, _l = ctypes.c_void_p, ctypes.c_int, ctypes.c_long


def quantize_q8_ref(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    xf = x.float()
    amax = xf.abs().amax(-1)
    inv = torch.where(amax > 0, 127.0 / amax, torch.zeros_like(amax))
    q = torch.round(xf * inv.unsqueeze(-1)).clamp_(-127, 127).to(torch.int8)
    return q, amax / 127.0


def quantize_q8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``[..., D]`` -> (int8 same shape, f32 scales ``[...]``)."""
    d = x.shape[-1]
    if not x.is_cuda or d % 32 or d > 256:
        return quantize_q8_ref(x)
    xc = x.contiguous()
    rows = xc.numel() // d
    q = torch.empty(xc.shape, dtype=torch.int8, device=x.device)
    sc = torch.empty(xc.shape[:-1], dtype=torch.float32, device=x.device)
    rc = _native.cuda().gb_kv_quant_q8(_c(xc.data_ptr()), _c(q.data_ptr()), _c(sc.data_ptr()), _l(rows), _i(d),
                                       _c(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "gb_kv_quant_q8")
    return q, sc


def dequantize_q8(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Inverse of ``quantize_q8``: bf16 of ``q``'s shape."""
    d = q.shape[-1]
    if not q.is_cuda:
        return (q.float() * scale.float().unsqueeze(-1)).to(torch.bfloat16)
    qc, sc = q.contiguous(), scale.contiguous()
    out = torch.empty(qc.shape, dtype=torch.bfloat16, device=q.device)
    rc = _native.cuda().gb_kv_dequant_q8(_c(qc.data_ptr()), _c(sc.data_ptr()), _c(out.data_ptr()), _l(qc.numel() // d), _i(d),
                                         _c(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "gb_kv_dequant_q8")
    return out
