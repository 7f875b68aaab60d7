"""Linear layers whose weights stay in ggml blocks (Q4_K, Q8_0) in HBM.

* one to four tokens: the fused dequant-GEMV (csrc/kernels/qgemv.cu: int8 activations, dp4a, scales per 32-wide sub-block);
* five tokens and more: the fused dequant-GEMM (csrc/kernels/qgemm.cu: the blocks are unpacked in registers into the swizzled
  bf16 operand tiles of ``tcgen05.mma``).

Both read the tiled layout of ``ops.ggml_torch``; the bytes are the file's blocks, only their order differs.  On CPU tensors the
same calls run an fp32 reference (the blocks are decoded, then multiplied), which is what the layer logic is tested with.

Reference: launch_matvec_auto and launch_batch_matvec (cuda/llm/cuda_llm_runner.c:13363-13506, 16241-16475) choose between
per-type GEMV kernels and tensor-core GEMMs in the same two regimes; CPU oracle tf_qmatvec_worker (common/transformer.h:648-738).
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native
from . import ggml_torch as gt
from .gemm import PendingPartials

_c, _i, _l = ctypes.c_void_p, ctypes.c_int, ctypes.c_long

GGML_OF_FMT = {"q4_k": gt.Q4_K, "q8_0": gt.Q8_0}
GEMV_MAX_TOKENS = 4


@dataclass
class QTensor:
    """A ``[rows, k]`` matrix as tiled ggml blocks: ``data`` uint8 ``[ceil(rows / 128), k / 256, tile_bytes]``; rows past ``rows``
    (padding up to the tile) are zero blocks."""
    data: torch.Tensor
    ggml_type: int
    rows: int
    k: int

    @staticmethod
    def from_float(w: torch.Tensor, ggml_type: int) -> "QTensor":
        """Quantise a float matrix (on its device) and tile it."""
        rows, k = w.shape
        return QTensor.from_blocks(gt.quantize(w, ggml_type), ggml_type, rows, k)

    @staticmethod
    def from_blocks(raw: torch.Tensor, ggml_type: int, rows: int, k: int) -> "QTensor":
        """``raw``: row-major blocks as they sit in a GGUF file (uint8, ``rows * row_bytes`` bytes)."""
        blk, nb = gt.BLOCK[ggml_type]
        raw = raw.reshape(rows, (k // blk) * nb)
        rp = (rows + 127) // 128 * 128
        if rp != rows:
            raw = torch.cat([raw, torch.zeros(rp - rows, raw.shape[1], dtype=torch.uint8, device=raw.device)])
        return QTensor(gt.tile(raw, ggml_type, rp, k), ggml_type, rows, k)

    def to(self, device) -> "QTensor":
        return QTensor(self.data.to(device), self.ggml_type, self.rows, self.k)

    def blocks(self) -> torch.Tensor:
        """Row-major blocks (file order) of the valid rows."""
        rp = self.data.shape[0] * 128
        return gt.untile(self.data, self.ggml_type, rp, self.k)[: self.rows]

    def dequantize(self) -> torch.Tensor:
        """fp32 ``[rows, k]``."""
        return gt.dequantize(self.blocks(), self.ggml_type, self.rows, self.k)

    def nbytes(self) -> int:
        return self.data.numel()


class QGemvPeer(ctypes.Structure):
    """Tensor-parallel tail of ``gb_qgemv`` (mirrors ``struct QGemvPeer`` in csrc/kernels/qgemv.cu)."""
    _fields_ = [("peer_out", ctypes.c_void_p * 8), ("signal_flags", ctypes.c_void_p * 8), ("peer_bcast", ctypes.c_int),
                ("signal_n", ctypes.c_int), ("done_ctr", ctypes.c_void_p), ("epoch_ptr", ctypes.c_void_p),
                ("epoch_self_tick", ctypes.c_int), ("pad", ctypes.c_int)]


def _stream():
    return _c(torch.cuda.current_stream().cuda_stream)


def pick_splits(rows: int, k: int, m: int, ggml_type: int = gt.Q4_K, sms: int = 148) -> int:
    """K splits of a decode-sized GEMV.  The kernel is persistent (two CTAs per SM walk the (row tile, split) items in a fixed
    stride), so the split count is the one that spreads the items most evenly over the CTAs, with at least two K tiles per item
    and a K range whose quantised activations fit shared memory; ties go to fewer splits (fewer partial slabs)."""
    tiles = (rows + 127) // 128
    num_kb = k // 256
    ctas = 2 * sms
    best, best_eff = 1, -1.0
    for sp in range(1, max(1, num_kb // 2) + 1):
        per = -(-num_kb // sp)
        if -(-num_kb // per) != sp:
            continue
        items = tiles * sp
        g = min(items, ctas)
        eff = items / (g * -(-items // g)) * min(1.0, items / ctas)
        if eff > best_eff + 0.02:
            best, best_eff = sp, eff
    sp = _native.cuda().gb_qgemv_splits(_i(ggml_type), _i(k), _i(m), _i(best))
    return max(1, sp)


def gemv_partials(x: torch.Tensor, w: QTensor, splits: Optional[int] = None, bias: Optional[torch.Tensor] = None,
                  peer: Optional[QGemvPeer] = None, out: Optional[torch.Tensor] = None) -> PendingPartials:
    """``x [m <= 4, k]`` (bf16) times ``w^T``: fp32 partial sums ``[splits, m, rows]``, one slab per K split, for the consumer to add
    (``ops.elementwise.rmsnorm``, ``qk_norm_rope``, ``silu_mul_partials``).  GPU only."""
    m, k = x.shape
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.stride(1) == 1 and k == w.k and 1 <= m <= GEMV_MAX_TOKENS
    sp = splits if splits is not None else pick_splits(w.rows, k, m, w.ggml_type)
    if out is None:
        out = torch.empty(sp, m, w.rows, dtype=torch.float32, device=x.device)
    rc = _native.cuda().gb_qgemv(_c(w.data.data_ptr()), _i(w.ggml_type), _c(x.data_ptr()), _i(x.stride(0)), _c(out.data_ptr()), _i(w.rows),
                                 _l(m * w.rows), _c(bias.data_ptr()) if bias is not None else _c(0), _i(w.rows), _i(k), _i(m), _i(sp),
                                 ctypes.byref(peer) if peer is not None else _c(0), _c(_native.status_ptr()), _stream())
    _native.check(rc, "gb_qgemv")
    return PendingPartials(out)


# token-tile widths of the dequant-GEMM
def _pick_tn(m: int) -> int:
    for tn in (16, 32, 64, 128):
        if m <= tn:
            return tn
    return 128


def gemm(x: torch.Tensor, w: QTensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
         out_dtype=torch.bfloat16) -> torch.Tensor:
    """``x [m, k]`` (bf16) times ``w^T`` on the tensor cores with the blocks unpacked on the fly.  GPU only."""
    m, k = x.shape
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.stride(1) == 1 and k == w.k
    if out is None:
        out = torch.empty(m, w.rows, dtype=out_dtype, device=x.device)
    rc = _native.cuda().gb_qgemm(_c(w.data.data_ptr()), _i(w.ggml_type), _c(x.data_ptr()), _i(x.stride(0)), _c(out.data_ptr()),
                                 _i(out.stride(0)), _i(1 if out.dtype == torch.float32 else 0), _c(bias.data_ptr()) if bias is not None else _c(0),
                                 _i(w.rows), _i(k), _i(m), _i(_pick_tn(m)), _i(0), _c(_native.status_ptr()), _stream())
    _native.check(rc, "gb_qgemm")
    return out


def pick_gemm_splits(rows: int, k: int, m: int, sms: int = 148) -> int:
    """K splits of the dequant-GEMM for a decode-sized projection with few row tiles (Qwen3-32B down projection: 40 tiles over
    100 K blocks): the split count (at most 8, at least 8 K blocks per split, none empty) that fills the last round of CTAs best."""
    if m > 64:
        return 1
    tiles, num_kb = (rows + 127) // 128, k // 256
    best, best_eff = 1, 0.0
    for sp in range(1, 9):
        if sp > 1 and num_kb // sp < 8:
            break
        per = -(-num_kb // sp)
        if -(-num_kb // per) != sp:
            continue
        units = tiles * sp
        eff = units / (-(-units // sms) * sms)
        if eff > best_eff * 1.05:
            best, best_eff = sp, eff
    return best


def gemm_partials(x: torch.Tensor, w: QTensor, splits: int, bias: Optional[torch.Tensor] = None) -> PendingPartials:
    """The dequant-GEMM cut along K: fp32 partial sums ``[splits, m, rows]`` for the consumer to add (as ``gemv_partials``)."""
    m, k = x.shape
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.stride(1) == 1 and k == w.k and splits >= 1
    out = torch.empty(splits, m, w.rows, dtype=torch.float32, device=x.device)
    rc = _native.cuda().gb_qgemm(_c(w.data.data_ptr()), _i(w.ggml_type), _c(x.data_ptr()), _i(x.stride(0)), _c(out.data_ptr()), _i(w.rows),
                                 _i(1), _c(bias.data_ptr()) if bias is not None else _c(0), _i(w.rows), _i(k), _i(m), _i(_pick_tn(m)),
                                 _i(splits), _c(_native.status_ptr()), _stream())
    _native.check(rc, "gb_qgemm")
    return PendingPartials(out)


def linear(x: torch.Tensor, w: QTensor, bias: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``x @ w^T (+ bias)``: GEMV up to four tokens, tensor-core GEMM above; fp32 reference on CPU tensors."""
    if not x.is_cuda:
        y = x.float() @ w.dequantize().t()
        if bias is not None:
            y = y + bias.float()
        return y.to(out_dtype)
    if x.shape[0] <= GEMV_MAX_TOKENS:
        return gemv_partials(x, w, bias=bias).buf.sum(0).to(out_dtype)
    sp = pick_gemm_splits(w.rows, w.k, x.shape[0])
    if sp > 1:
        return gemm_partials(x, w, sp, bias=bias).buf.sum(0).to(out_dtype)
    return gemm(x, w, bias=bias, out_dtype=out_dtype)


def linear_swiglu(x: torch.Tensor, w_gate_up: QTensor) -> torch.Tensor:
    """``silu(x Wg^T) * (x Wu^T)`` with ``w_gate_up = [Wg ; Wu]`` stacked along rows; bf16 ``[m, rows / 2]``."""
    inter = w_gate_up.rows // 2
    if not x.is_cuda:
        y = x.float() @ w_gate_up.dequantize().t()
        return (torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]).to(torch.bfloat16)
    if x.shape[0] <= GEMV_MAX_TOKENS:
        from . import elementwise as ew
        return ew.silu_mul_partials(gemv_partials(x, w_gate_up))
    from . import elementwise as ew
    return ew.silu_mul(gemm(x, w_gate_up))
