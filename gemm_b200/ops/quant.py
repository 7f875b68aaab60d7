"""ggml-quantised weights on the GPU: raw GGUF blocks stay in HBM; small batches run the fused dequant-GEMV, large ones
dequantise to bf16 once per call (or once at load) and use the tensor-core GEMM.  Kernels: csrc/kernels/dequant.cu.

Reference: launch_matvec_auto / launch_batch_matvec (cuda/llm/cuda_llm_runner.c:13363-13506,16241-16475) pick per-type kernels
in the same two regimes; the host decoders used as oracle are csrc/host/dequant.cc (bit-exact vs common/ggml_dequant.h)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import _native
from ..utils import gguf as G

_c, _i, _l = ctypes.c_void_p, ctypes.c_int, ctypes.c_long
_codebooks_ready = set()


def _ensure_codebooks(device) -> None:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key in _codebooks_ready:
        return
    lib = _native.cuda()
    for which in range(7):
        arr = G.codebook(which)
        raw = arr.tobytes()
        _native.check(lib.gb_set_codebook(_i(which), raw, _l(len(raw))), "gb_set_codebook", n=0)
    _codebooks_ready.add(key)


@dataclass
class QuantWeight:
    """A ``[rows, k]`` matrix stored as raw ggml blocks (uint8 tensor of ``rows * row_bytes`` bytes)."""
    raw: torch.Tensor
    ggml_type: int
    rows: int
    k: int

    @staticmethod
    def from_float(w: torch.Tensor, t, device=None) -> "QuantWeight":
        raw = G.quantize(w, t)
        return QuantWeight(raw.to(device) if device is not None else raw, G.type_id(t), w.shape[0], w.shape[1])

    def to(self, device) -> "QuantWeight":
        return QuantWeight(self.raw.to(device), self.ggml_type, self.rows, self.k)

    def dequantize(self) -> torch.Tensor:
        """bf16 ``[rows, k]`` (GPU kernel on CUDA tensors, host decoder otherwise)."""
        n = self.rows * self.k
        if not self.raw.is_cuda:
            return G.dequantize(self.raw, self.ggml_type, n).reshape(self.rows, self.k).to(torch.bfloat16)
        _ensure_codebooks(self.raw.device)
        out = torch.empty(self.rows, self.k, dtype=torch.bfloat16, device=self.raw.device)
        rc = _native.cuda().gb_dequant_bf16(_c(self.raw.data_ptr()), _c(out.data_ptr()), _l(n), _i(self.ggml_type),
                                            _c(torch.cuda.current_stream().cuda_stream))
        _native.check(rc, "gb_dequant_bf16")
        return out


def linear_quant(x: torch.Tensor, w: QuantWeight, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``x [M, K] (bf16) @ W^T`` with W in ggml blocks."""
    m = x.shape[0]
    if not x.is_cuda:
        return (x.float() @ w.dequantize().float().t()).to(out_dtype)
    if m <= 8:
        _ensure_codebooks(x.device)
        y = torch.empty(m, w.rows, dtype=torch.float32, device=x.device)
        rc = _native.cuda().gb_gemv_quant(_c(w.raw.data_ptr()), _c(x.data_ptr()), _c(y.data_ptr()), _i(w.rows), _i(w.k), _i(m), _i(w.ggml_type),
                                          _i(x.stride(0)), _i(w.rows), _c(torch.cuda.current_stream().cuda_stream))
        _native.check(rc, "gb_gemv_quant")
        return y if out_dtype == torch.float32 else y.to(out_dtype)
    from . import gemm
    return gemm.linear(x, w.dequantize(), out_dtype=out_dtype)
