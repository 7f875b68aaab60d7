"""Linear layers on the tcgen05 GEMM kernel (csrc/kernels/gemm_tc.cu) and their PyTorch references.

``linear`` / ``linear_mx`` / ``grouped_*`` run the CUDA kernel when the tensors live on a GPU and the
fp32 PyTorch reference on CPU tensors (the CPU path exists for tests and for the CPU engine; there is
no silent fallback on a GPU: a missing library raises).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .. import _native
from . import mxfp8
from .mxfp8 import MxTensor

GEMM_MX, GEMM_DUAL, GEMM_QUANT_OUT, GEMM_OUT_F32, GEMM_W_TILED, GEMM_DUAL_RAW = 1, 2, 4, 8, 16, 32


class GemmExtras(ctypes.Structure):
    """Expert-parallel arguments of ``gb_gemm`` (mirrors ``struct GemmExtras`` in csrc/kernels/gemm_tc.cu)."""
    _fields_ = [("w_group_mod", ctypes.c_int), ("wait_n", ctypes.c_int), ("wait_flags", ctypes.c_void_p),
                ("epoch_ptr", ctypes.c_void_p), ("peer_out", ctypes.c_void_p * 8), ("peer_region_rows", ctypes.c_int),
                ("peer_rank", ctypes.c_int), ("signal_flags", ctypes.c_void_p * 8), ("signal_n", ctypes.c_int),
                ("pad", ctypes.c_int), ("done_ctr", ctypes.c_void_p), ("splits", ctypes.c_int), ("pad2", ctypes.c_int),
                ("sk_ws", ctypes.c_void_p), ("sk_ctr", ctypes.c_void_p), ("amax_val", ctypes.c_void_p), ("amax_idx", ctypes.c_void_p),
                ("sk_ws_bytes", ctypes.c_long), ("sk_ctr_count", ctypes.c_long), ("peer_bcast", ctypes.c_int), ("epoch_self_tick", ctypes.c_int),
                ("sfa_bytes", ctypes.c_size_t), ("sfb_bytes", ctypes.c_size_t), ("out_bytes", ctypes.c_size_t), ("out_sf_bytes", ctypes.c_size_t),
                ("partial_stride", ctypes.c_long)]


_SK_WS_BYTES = 64 << 20
_SK_CTR = 1 << 16
_sk_state = {}


SPLIT_K = os.environ.get("GB_SPLITK", "0") == "1"
# MXFP8 GEMMs over 256 or more tokens use 256-token tiles: one block-scaled tcgen05.mma costs the issuing thread about 160
# cycles whether it is 128 or 256 columns wide, so the wide tile nearly doubles the tensor throughput of the prefill GEMMs.
WIDE_TILE = os.environ.get("GB_WIDE_TILE", "1") != "0"


def _splitk_extras(n_out: int, m_tok: int, k: int, tn: int, mx: bool, device, force: bool = False) -> Optional["GemmExtras"]:
    """Extras that turn on split-K when the plain tiling would leave most SMs idle (decode-sized GEMMs).

    Off unless asked for (``force`` / ``GB_SPLITK=1``): on B200 the decode projections measured faster without it
    (one CTA streams a 128-row weight panel in a few microseconds; the partial-sum round trip costs more)."""
    if not (force or SPLIT_K):
        return None
    tiles = ((n_out + 127) // 128) * ((m_tok + tn - 1) // tn)
    sms = 148
    if tiles * 4 > sms:
        return None
    num_kb = (k + (127 if mx else 63)) // (128 if mx else 64)
    splits = min(sms // tiles, num_kb // 4, 8)
    if splits < 2:
        return None
    key = (device.index if device.index is not None else torch.cuda.current_device())
    if key not in _sk_state:
        _sk_state[key] = (torch.empty(_SK_WS_BYTES, dtype=torch.uint8, device=device), torch.zeros(_SK_CTR, dtype=torch.int32, device=device))
    ws, ctr = _sk_state[key]
    ex = GemmExtras()
    ex.splits = splits
    ex.sk_ws, ex.sk_ctr = ws.data_ptr(), ctr.data_ptr()
    ex.sk_ws_bytes, ex.sk_ctr_count = _SK_WS_BYTES, _SK_CTR
    return ex

_c = ctypes.c_void_p
_i = ctypes.c_int


def _p(t: Optional[torch.Tensor]):
    return _c(t.data_ptr()) if t is not None else _c(0)


def _stream():
    return _c(torch.cuda.current_stream().cuda_stream)


def pick_tn(m_tok: int, mx: bool = False, dual: bool = False) -> int:
    """Token-tile width: the smallest supported tile that covers the batch, capped by TMEM capacity.
    MXFP8 operands come in two scale layouts, so their tile is 32 (sf_layout 32) or 128 (sf_layout 128)."""
    if mx:
        return 32 if m_tok <= 32 else 128
    lo = 32 if mx else 16
    hi = 128 if (mx or dual) else 256
    tn = lo
    while tn < hi and tn < m_tok:
        tn *= 2
    return tn


_next_wait = None


def wait_before_next_launch(flags_ptr: int, n: int, epoch_ptr: int) -> None:
    """The NEXT GEMM launched through this module waits (bounded, on the device) until ``flags[i] >= *epoch_ptr`` for ``i < n`` before
    it reads its token rows: the consumer side of an all-gather whose rows the peers store into this GPU's memory (the kernel
    that produced them raised the flags)."""
    global _next_wait
    _next_wait = (flags_ptr, n, epoch_ptr)


def _launch(w, x, out, n_out, k, m_tok, ldw, ldx, ldo, flags, tn, num_groups=0, w_rows_per_group=0, up_row_offset=0,
            seg_start=None, seg_count=None, x_rows=None, sfa=None, sfb=None, out_sf=None, bias=None, row_map=None,
            row_scale=None, extras=None):
    global _next_wait
    lib = _native.cuda()
    if extras is None:
        extras = GemmExtras()
    restore = None
    if _next_wait is not None:
        if extras.signal_n or extras.wait_n:
            raise RuntimeError("gemm: a pending all-gather wait met a launch that has its own flag protocol")
        restore = (extras.wait_flags, extras.wait_n, extras.epoch_ptr)
        extras.wait_flags, extras.wait_n, extras.epoch_ptr = _next_wait
        _next_wait = None
    # extents of the caller's buffers: the kernel checks its scale-atom loads and its stores against them
    nb = lambda t: t.numel() * t.element_size() if t is not None else 0
    extras.sfa_bytes, extras.sfb_bytes, extras.out_bytes, extras.out_sf_bytes = nb(sfa), nb(sfb), nb(out), nb(out_sf)
    rc = lib.gb_gemm(_p(w), _p(x), _p(out), _i(n_out), _i(k), _i(m_tok), _i(ldw), _i(ldx), _i(ldo), _i(flags), _i(tn),
                     _i(num_groups), _i(w_rows_per_group), _i(up_row_offset), _p(seg_start), _p(seg_count),
                     _i(x_rows if x_rows is not None else m_tok), _p(sfa), _p(sfb), _p(out_sf), _p(bias), _p(row_map),
                     _p(row_scale), ctypes.byref(extras) if extras is not None else _c(0), _c(_native.status_ptr()), _stream())
    if restore is not None:
        extras.wait_flags, extras.wait_n, extras.epoch_ptr = restore
    _native.check(rc, "gb_gemm")


# --------------------------------------------------------------------------------------------- bf16
def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
           out_dtype=torch.bfloat16, tn: Optional[int] = None, split_k: bool = False, w_tiled: bool = False) -> torch.Tensor:
    """``x [M, K] @ w[N, K]^T`` (bf16 operands, fp32 accumulate).  ``w_tiled``: ``w`` is in ``mxfp8.tile_weight`` layout."""
    m, k = x.shape
    n = w.shape[0]
    if not x.is_cuda:
        y = x.float() @ (mxfp8.untile_weight(w) if w_tiled else w).float().t()
        if bias is not None:
            y = y + bias.float()
        return y.to(out_dtype)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=x.device)
    flags = (GEMM_OUT_F32 if out.dtype == torch.float32 else 0) | (GEMM_W_TILED if w_tiled else 0)
    tn = tn or pick_tn(m)
    _launch(w, x, out, n, k, m, w.stride(0), x.stride(0), out.stride(0), flags, tn, bias=bias,
            extras=_splitk_extras(n, m, k, tn, False, x.device, split_k))
    return out


def linear_argmax(x: torch.Tensor, w: torch.Tensor, idx_offset: int = 0, want_value: bool = False, w_tiled: bool = False):
    """Greedy sampling fused into the LM head: ``argmax_n (x W^T)[t, n]`` without ever writing the logits.  Returns int32 ``[M]``
    (+ the winning values).  Ties resolve to the lower index."""
    m, k = x.shape
    n = w.shape[0]
    if not x.is_cuda:
        y = torch.nan_to_num(x.float() @ (mxfp8.untile_weight(w) if w_tiled else w).float().t(), nan=-3.4e38)
        val, idx = y.max(dim=-1)
        idx = (idx + idx_offset).to(torch.int32)
        return (idx, val) if want_value else idx
    parts = ((n + 127) // 128) * 4
    pv = torch.empty(parts, m, dtype=torch.float32, device=x.device)
    pi = torch.empty(parts, m, dtype=torch.int32, device=x.device)
    ex = GemmExtras()
    ex.amax_val, ex.amax_idx = pv.data_ptr(), pi.data_ptr()
    _launch(w, x, None, n, k, m, w.stride(0), x.stride(0), n, GEMM_OUT_F32 | (GEMM_W_TILED if w_tiled else 0), pick_tn(m), extras=ex)
    out = torch.empty(m, dtype=torch.int32, device=x.device)
    val = torch.empty(m, dtype=torch.float32, device=x.device) if want_value else None
    rc = _native.cuda().gb_argmax_pairs(_p(pv), _p(pi), _p(out), _p(val), _i(parts), _i(m), _i(idx_offset), _stream())
    _native.check(rc, "gb_argmax_pairs")
    return (out, val) if want_value else out


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: Optional[torch.Tensor] = None,
                  tn: Optional[int] = None, w_tiled: bool = False) -> torch.Tensor:
    """``silu(x @ Wg^T) * (x @ Wu^T)`` with ``w_gate_up = [Wg; Wu]`` stacked along rows ([2I, K])."""
    m, k = x.shape
    inter = w_gate_up.shape[0] // 2
    if not x.is_cuda:
        y = x.float() @ (mxfp8.untile_weight(w_gate_up) if w_tiled else w_gate_up).float().t()
        return (torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]).to(torch.bfloat16)
    if out is None:
        out = torch.empty(m, inter, dtype=torch.bfloat16, device=x.device)
    _launch(w_gate_up, x, out, inter, k, m, w_gate_up.stride(0), x.stride(0), out.stride(0), GEMM_DUAL | (GEMM_W_TILED if w_tiled else 0),
            tn or pick_tn(m, dual=True), up_row_offset=inter)
    return out


# --------------------------------------------------------------------------------------------- mxfp8
def linear_mx(x: MxTensor, w: MxTensor, out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16,
              tn: Optional[int] = None, bias: Optional[torch.Tensor] = None, split_k: bool = False) -> torch.Tensor:
    """Block-scaled fp8 linear: both operands MXFP8, bf16 (or f32) result [x.rows, w.rows]."""
    if not x.data.is_cuda:
        y = mxfp8.dequantize(x) @ mxfp8.dequantize(w).t()
        if bias is not None:
            y = y + bias.float()
        return y.to(out_dtype)
    m, n, k = x.rows, w.rows, w.k
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=x.data.device)
    flags = GEMM_MX | (GEMM_OUT_F32 if out.dtype == torch.float32 else 0) | (GEMM_W_TILED if w.tiled else 0)
    assert w.sf_layout == 128
    if tn is None:
        tn = 64 if (x.sf_layout == 128 and m <= 64) else x.sf_layout      # a single token block may use the 64-wide tile
        if WIDE_TILE and tn == 128 and m >= 256 and out.dtype == torch.bfloat16 and not split_k:
            tn = 256
    _launch(w.data, x.data, out, n, k, m, k, k, out.stride(0), flags, tn, x_rows=x.data.shape[0],
            sfa=w.sf, sfb=x.sf, bias=bias, extras=_splitk_extras(n, m, k, tn, True, x.data.device, split_k))
    return out


class PendingPartials:
    """K-split partial sums of a projection, ``buf`` f32 ``[n, rows, hidden]``: the consumer (the next residual add + RMSNorm,
    ``ops.elementwise.rmsnorm``) sums them in split order, so a decode-sized GEMM can spread over the whole GPU without a
    reduction pass of its own."""

    def __init__(self, buf: torch.Tensor):
        self.buf = buf
        self.n, self.rows, self.hidden = buf.shape

    def materialize(self) -> torch.Tensor:
        return self.buf.sum(0).to(torch.bfloat16)


def pick_partials(n_out: int, m_tok: int, k: int, mx: bool, sms: int = 148) -> int:
    """Number of K splits for a decode-sized projection: the split count (at most 8, at least 4 k-steps per split, no empty split)
    that fills the last wave of CTAs best; ties go to fewer splits.  96 tiles -> 3 splits (288 CTAs = 1.95 waves), 16 tiles -> 8."""
    if m_tok > 64:
        return 1
    tiles = (n_out + 127) // 128
    num_kb = k // (128 if mx else 64)
    best, best_eff = 1, 0.0
    for sp in range(1, 9):
        if sp > 1 and num_kb // sp < 4:
            break
        kb_per = -(-num_kb // sp)
        if -(-num_kb // kb_per) != sp:
            continue
        units = tiles * sp
        eff = units / (-(-units // sms) * sms)
        if eff > best_eff * 1.05:
            best, best_eff = sp, eff
    return best


def linear_partials(x: torch.Tensor, w: torch.Tensor, splits: int, bias: Optional[torch.Tensor] = None, w_tiled: bool = False) -> PendingPartials:
    """bf16 ``linear`` with the K range cut into ``splits`` CTAs per output tile, one fp32 partial slab per split (GPU only)."""
    m, k = x.shape
    n = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    out = torch.empty(splits, m, n, dtype=torch.float32, device=x.device)
    ex = GemmExtras()
    ex.splits, ex.partial_stride = splits, m * n
    _launch(w, x, out, n, k, m, w.stride(0), x.stride(0), n, GEMM_OUT_F32 | (GEMM_W_TILED if w_tiled else 0), pick_tn(m), bias=bias, extras=ex)
    return PendingPartials(out)


def pick_partials_dual(inter: int, m_tok: int, k: int, mx: bool) -> int:
    """K splits for a decode-sized gate/up projection (a tile = 128 gate rows + 128 up rows)."""
    return pick_partials(inter, m_tok, k, mx)


def swiglu_partials(x, w_gate_up, splits: int, w_tiled: bool = False) -> PendingPartials:
    """Gate/up projection cut along K: raw fp32 partial sums ``[splits, M, 2I]`` (gate columns first); ``ops.elementwise.silu_mul_partials``
    adds the slabs and applies SiLU(gate) * up.  ``x`` / ``w_gate_up`` are bf16 tensors or ``MxTensor`` operands.  GPU only."""
    mx = isinstance(x, MxTensor)
    if mx:
        m, k, two_i = x.rows, x.k, w_gate_up.rows
        xd, wd, dev = x.data, w_gate_up.data, x.data.device
        tn = 64 if (x.sf_layout == 128 and m <= 64) else x.sf_layout
        flags = GEMM_MX | GEMM_DUAL | GEMM_OUT_F32 | (GEMM_W_TILED if w_gate_up.tiled else 0)
        kw = dict(x_rows=xd.shape[0], sfa=w_gate_up.sf, sfb=x.sf)
        ldw = ldx = k
    else:
        m, k = x.shape
        two_i = w_gate_up.shape[0]
        xd, wd, dev = x, w_gate_up, x.device
        tn = pick_tn(m, dual=True)
        flags = GEMM_DUAL | GEMM_OUT_F32 | (GEMM_W_TILED if w_tiled else 0)
        kw = {}
        ldw, ldx = w_gate_up.stride(0), x.stride(0)
    inter = two_i // 2
    out = torch.empty(splits, m, two_i, dtype=torch.float32, device=dev)
    ex = GemmExtras()
    ex.splits, ex.partial_stride = splits, m * two_i
    _launch(wd, xd, out, inter, k, m, ldw, ldx, two_i, flags, tn, up_row_offset=inter, extras=ex, **kw)
    return PendingPartials(out)


def linear_mx_partials(x: MxTensor, w: MxTensor, splits: int, bias: Optional[torch.Tensor] = None) -> PendingPartials:
    """``linear_mx`` with the K range cut into ``splits`` CTAs per output tile; every split stores its fp32 partial (the bias
    goes into split 0).  GPU only."""
    m, n, k = x.rows, w.rows, w.k
    out = torch.empty(splits, m, n, dtype=torch.float32, device=x.data.device)
    tn = 64 if (x.sf_layout == 128 and m <= 64) else x.sf_layout
    ex = GemmExtras()
    ex.splits, ex.partial_stride = splits, m * n
    _launch(w.data, x.data, out, n, k, m, k, k, n, GEMM_MX | GEMM_OUT_F32 | (GEMM_W_TILED if w.tiled else 0), tn, x_rows=x.data.shape[0],
            sfa=w.sf, sfb=x.sf, bias=bias, extras=ex)
    return PendingPartials(out)


def linear_mx_swiglu_quant(x: MxTensor, w_gate_up: MxTensor, tn: Optional[int] = None) -> MxTensor:
    """MXFP8 gate/up projection with SiLU(gate)*up and re-quantisation to MXFP8 in the epilogue."""
    inter = w_gate_up.rows // 2
    if not x.data.is_cuda:
        y = mxfp8.dequantize(x) @ mxfp8.dequantize(w_gate_up).t()
        h = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
        return mxfp8.quantize(h, sf_layout=x.sf_layout)
    rows_p = x.data.shape[0]
    out = torch.empty(rows_p, inter, dtype=torch.uint8, device=x.data.device)
    out_sf = torch.empty((rows_p // x.sf_layout, inter // 128, 512), dtype=torch.uint8, device=x.data.device)
    _launch(w_gate_up.data, x.data, out, inter, x.k, x.rows, x.k, x.k, inter,
            GEMM_MX | GEMM_DUAL | GEMM_QUANT_OUT | (GEMM_W_TILED if w_gate_up.tiled else 0),
            tn or x.sf_layout, up_row_offset=inter, x_rows=rows_p, sfa=w_gate_up.sf, sfb=x.sf, out_sf=out_sf)
    return MxTensor(out, out_sf, x.rows, inter, x.sf_layout)


# --------------------------------------------------------------------------------------------- grouped
def grouped_linear(x: torch.Tensor, w: torch.Tensor, seg_start: torch.Tensor, seg_count: torch.Tensor, tn: int,
                   out: Optional[torch.Tensor] = None, dual: bool = False, row_map: Optional[torch.Tensor] = None,
                   row_scale: Optional[torch.Tensor] = None, sfa=None, sfb=None, quant_out: bool = False,
                   out_sf: Optional[torch.Tensor] = None, extras=None, w_groups: Optional[int] = None,
                   w_tiled: bool = False, pair_rows: bool = False) -> torch.Tensor:
    """One GEMM per group over row segments of ``x``.

    ``w`` is ``[G, R, K]`` (R = 2I stacked gate/up rows when ``dual``); group g multiplies the rows
    ``seg_start[g] : seg_start[g] + seg_count[g]`` of ``x``.  ``seg_start`` entries must be multiples of
    ``min(tn, 128)``.  With ``sfa``/``sfb`` the operands are e4m3 bytes with scale atoms (MXFP8); that mode
    needs ``tn`` 32 or 128, segments aligned to ``tn`` and activation scales in the matching atom layout.
    """
    g, r, k = w.shape
    if w_groups is not None:
        g = w_groups                      # more row groups than weight groups (expert parallel: group = (source, expert))
    # ``pair_rows``: a tile takes row blocks n and R/2 + n of the SAME projection (two accumulators, plain stores): half the tiles
    # and token-tile loads for projections with a short K, such as the expert down projection of a decode step
    pair = bool(pair_rows and not dual and not quant_out and row_map is None and row_scale is None and x.is_cuda and r % 256 == 0)
    n_out = r // 2 if (dual or pair) else r
    mx = sfa is not None
    if not x.is_cuda:
        if w_tiled:
            w = mxfp8.untile_weight(w.reshape(-1, k)).reshape(w.shape)
        return _grouped_reference(x, w, seg_start, seg_count, dual, row_map, row_scale, sfa, sfb, quant_out, out, out_sf)
    flags = (GEMM_MX if mx else 0) | (GEMM_DUAL if dual else 0) | (GEMM_QUANT_OUT if quant_out else 0) | (GEMM_W_TILED if w_tiled else 0)
    if pair:
        flags |= GEMM_DUAL | GEMM_DUAL_RAW
    if out is None:
        if quant_out:
            out = torch.empty(x.shape[0], n_out, dtype=torch.uint8, device=x.device)
        else:
            out = torch.empty(x.shape[0], r if pair else n_out, dtype=torch.bfloat16, device=x.device)
    if out.dtype == torch.float32:
        flags |= GEMM_OUT_F32
    if (WIDE_TILE and mx and tn == 128 and not dual and not pair and not quant_out and row_map is None and row_scale is None
            and out.dtype == torch.bfloat16 and x.shape[0] >= 256 * g):
        tn = 256                          # prefill-sized segments (the scale atoms keep the 128-row layout)
    _launch(w, x, out, n_out, k, x.shape[0], k, x.stride(0), out.stride(0), flags, tn, num_groups=g, w_rows_per_group=r,
            up_row_offset=n_out if (dual or pair) else 0, seg_start=seg_start, seg_count=seg_count, x_rows=x.shape[0], sfa=sfa,
            sfb=sfb, out_sf=out_sf, row_map=row_map, row_scale=row_scale, extras=extras)
    return out


def _grouped_reference(x, w, seg_start, seg_count, dual, row_map, row_scale, sfa, sfb, quant_out, out, out_sf=None):
    g, r, k = w.shape
    n_out = r // 2 if dual else r
    if sfa is not None:
        lay = 32 if sfb.shape[0] * 32 == x.shape[0] else 128
        wf = mxfp8.dequantize_rowmajor(w.reshape(g * r, k), mxfp8.unpack_sf_atoms(sfa, g * r, k // 32)).reshape(g, r, k)
        xf = mxfp8.dequantize_rowmajor(x, mxfp8.unpack_sf_atoms(sfb, x.shape[0], k // 32, lay))
    else:
        wf, xf = w.float(), x.float()
    res = torch.zeros(x.shape[0], n_out, dtype=torch.float32)
    for gi in range(g):
        s, c = int(seg_start[gi]), int(seg_count[gi])
        if c == 0:
            continue
        y = xf[s:s + c] @ wf[gi].t()
        if dual:
            y = torch.nn.functional.silu(y[:, :n_out]) * y[:, n_out:]
        res[s:s + c] = y
    if quant_out:
        q = mxfp8.quantize(res, sf_layout=(32 if (out_sf is not None and out_sf.shape[0] * 32 == res.shape[0]) else 128))
        if out is not None:
            out.copy_(q.data[: out.shape[0]])
            out_sf.copy_(q.sf)
            return out
        return q.data
    if row_scale is not None:
        res = res * row_scale.float().unsqueeze(-1)
    if row_map is not None:
        assert out is not None
        keep = row_map >= 0
        out[row_map[keep].long()] = res[keep].to(out.dtype)
        return out
    return res.to(torch.bfloat16)
