"""Token-wise ops: embedding gather, RMSNorm (+residual add, +MXFP8 output), QK-norm + RoPE + paged KV
write, SiLU-gate, MXFP8 activation quantiser.  CUDA kernels live in csrc/kernels/elementwise.cu; each
function falls back to the fp32 PyTorch reference only for CPU tensors.

Reference behaviour: common/transformer.h:593-637 (RMSNorm), :1281-1315 (per-head QK-norm),
:1183-1219 (NeoX RoPE, pairs (j, j + d/2), inv_freq = theta^(-2j/d)).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch

from .. import _native
from . import mxfp8
from .mxfp8 import MxTensor

_c, _i, _f, _l = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_long


def _p(t):
    return _c(t.data_ptr()) if t is not None else _c(0)


def _s():
    return _c(torch.cuda.current_stream().cuda_stream)


# ------------------------------------------------------------------------------------------ embed
def embed(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Rows of a bf16 embedding table; ids int32 [T]."""
    if not table.is_cuda:
        return table[ids.long()].to(torch.bfloat16)
    out = torch.empty(ids.numel(), table.shape[1], dtype=torch.bfloat16, device=table.device)
    _native.check(_native.cuda().gb_embed(_p(ids), _p(table), _p(out), _i(ids.numel()), _i(table.shape[1]),
                                          _i(table.shape[0]), _s()), "gb_embed")
    return out


# ------------------------------------------------------------------------------------------ rmsnorm
def rmsnorm_ref(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(torch.bfloat16)


def sf_alloc(rows_padded: int, k: int, device, layout: int = 128, init: bool = True) -> torch.Tensor:
    """Scale-atom buffer for ``rows_padded`` rows (a multiple of 128).  ``init`` fills it with scale 1; the hot paths
    skip the fill: rows that no kernel writes only ever feed accumulator columns that the GEMM epilogue drops
    (every token is its own MMA column, so their contents cannot reach a valid row)."""
    shape = (rows_padded // layout, k // 128, 512)
    if not init:
        return torch.empty(shape, dtype=torch.uint8, device=device)
    return torch.full(shape, 127, dtype=torch.uint8, device=device)


class RmsBcast(ctypes.Structure):
    """All-gather in the RMSNorm's epilogue (mirrors ``RmsBcast`` in csrc/kernels/elementwise.cu): where the bf16 rows go on every
    GPU, the flags raised afterwards, the epoch and arrival counters."""
    _fields_ = [("out", ctypes.c_void_p * 8), ("flag", ctypes.c_void_p * 8), ("world", ctypes.c_int), ("partials_bf16", ctypes.c_int),
                ("epoch_ctr", ctypes.c_void_p), ("done_ctr", ctypes.c_void_p)]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None,
            quantize: bool = False, want_bf16: bool = True, sf_layout: int = 128, out_buf: Optional[torch.Tensor] = None,
            bcast: Optional[RmsBcast] = None):
    """RMSNorm of ``x`` (or of ``residual += x`` when ``residual`` is given; the sum is written back).

    Returns the bf16 result, or ``(bf16 | None, MxTensor)`` when ``quantize`` asks for an MXFP8 copy that
    feeds a block-scaled GEMM.  ``bcast`` (only with K-split partial sums as ``x``): the kernel also stores the bf16 rows on
    every GPU and raises the arrival flags; ``out_buf`` must then be the local destination among ``bcast.out``.
    """
    pend = None
    if hasattr(x, "buf") and hasattr(x, "materialize"):          # ops.gemm.PendingPartials: K-split partial sums, summed by this kernel
        if residual is None or not x.buf.is_cuda or residual.stride(0) != x.hidden:
            x = x.materialize()
        else:
            rows, hidden = x.rows, x.hidden
            out = (out_buf[:rows] if out_buf is not None else torch.empty(rows, hidden, dtype=torch.bfloat16, device=residual.device)) if want_bf16 else None
            q = sf = None
            if quantize:
                rp = (rows + 127) // 128 * 128
                q = torch.empty(rp, hidden, dtype=torch.uint8, device=residual.device)
                sf = sf_alloc(rp, hidden, residual.device, sf_layout, init=False)
            if bcast is not None:
                # the local copy is one of the kernel's gather destinations: no separate bf16 store
                rc = _native.cuda().gb_rmsnorm_reduce_bcast(_p(residual), _p(x.buf), _i(x.n), _l(rows * hidden), _p(w), _c(0), _p(q), _p(sf),
                                                            _i(rows), _i(hidden), _f(eps), _i(1 if sf_layout == 32 else 0), _c(0), _i(0), _c(0),
                                                            _c(_native.status_ptr()), ctypes.byref(bcast), _s())
                _native.check(rc, "gb_rmsnorm_reduce_bcast")
                out = out_buf[:rows]
                return (out, MxTensor(q, sf, rows, hidden, sf_layout)) if quantize else out
            rc = _native.cuda().gb_rmsnorm_reduce(_p(residual), _p(x.buf), _i(x.n), _l(rows * hidden), _p(w), _p(out), _p(q), _p(sf), _i(rows),
                                                  _i(hidden), _f(eps), _i(1 if sf_layout == 32 else 0), _c(0), _i(0), _c(0),
                                                  _c(_native.status_ptr()), _s())
            _native.check(rc, "gb_rmsnorm_reduce")
            return (out, MxTensor(q, sf, rows, hidden, sf_layout)) if quantize else out
    if hasattr(x, "materialize"):                    # ops.moe.PendingCombine: the MoE combine is done by this kernel
        if residual is None or not x.y.is_cuda:
            x = x.materialize()
        else:
            pend = x
            x = pend.y
    rows, hidden = (pend.n_tok, pend.y.shape[1]) if pend is not None else x.shape
    if not x.is_cuda:
        if residual is not None:
            residual.copy_((residual.float() + x.float()).to(torch.bfloat16))
            src = residual
        else:
            src = x
        y = rmsnorm_ref(src, w, eps)
        if quantize:
            return (y if want_bf16 else None), mxfp8.quantize(y.float(), sf_layout=sf_layout)
        return y
    # ``out_buf``: a caller-owned bf16 buffer (at least ``rows`` contiguous rows) that receives the result instead of a fresh tensor
    out = (out_buf[:rows] if out_buf is not None else torch.empty(rows, hidden, dtype=torch.bfloat16, device=x.device)) if want_bf16 else None
    q = sf = None
    if quantize:
        rp = (rows + 127) // 128 * 128
        q = torch.empty(rp, hidden, dtype=torch.uint8, device=x.device)
        sf = sf_alloc(rp, hidden, x.device, sf_layout, init=False)
    if pend is not None:
        assert residual.stride(0) == hidden
        rc = _native.cuda().gb_rmsnorm_combine(_p(residual), _p(pend.y), _p(pend.pair_row), _p(pend.weights), _i(pend.k), _i(pend.y.stride(0)),
                                               _p(w), _p(out), _p(q), _p(sf), _i(rows), _i(hidden), _f(eps), _i(1 if sf_layout == 32 else 0),
                                               _c(pend.wait_flags), _i(pend.wait_n), _c(pend.epoch_ptr), _c(_native.status_ptr()), _s())
    elif residual is not None and bcast is not None:
        assert x.stride(0) == residual.stride(0)
        rc = _native.cuda().gb_rmsnorm_bcast(_p(residual), _p(x), _p(w), _p(q), _p(sf), _i(rows), _i(hidden), _f(eps), _i(residual.stride(0)),
                                             _i(1 if sf_layout == 32 else 0), ctypes.byref(bcast), _s())
        out = out_buf[:rows]
    elif residual is not None:
        rc = _native.cuda().gb_rmsnorm(_p(residual), _p(x), _c(0), _p(w), _p(out), _p(q), _p(sf), _i(rows), _i(hidden),
                                       _f(eps), _i(residual.stride(0)), _i(hidden), _i(1 if sf_layout == 32 else 0), _s())
    else:
        rc = _native.cuda().gb_rmsnorm(_c(0), _c(0), _p(x), _p(w), _p(out), _p(q), _p(sf), _i(rows), _i(hidden), _f(eps),
                                       _i(x.stride(0)), _i(hidden), _i(1 if sf_layout == 32 else 0), _s())
    _native.check(rc, "gb_rmsnorm")
    if quantize:
        return out, MxTensor(q, sf, rows, hidden, sf_layout)
    return out


# ------------------------------------------------------------------------------------------ qk norm + rope + kv write
def rope_ref(x: torch.Tensor, positions: torch.Tensor, theta: float, rope_dim: Optional[int] = None) -> torch.Tensor:
    """NeoX rotation of ``x [T, H, D]`` (fp32 math)."""
    t, h, d = x.shape
    rd = rope_dim or d
    half = rd // 2
    j = torch.arange(half, dtype=torch.float32, device=x.device)
    inv = theta ** (-2.0 * j / rd)
    ang = positions.to(torch.float32).unsqueeze(-1) * inv            # [T, half]
    cos, sin = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
    xf = x.float().clone()
    a, b = xf[..., :half].clone(), xf[..., half:rd].clone()
    xf[..., :half] = a * cos - b * sin
    xf[..., half:rd] = a * sin + b * cos
    return xf


def rope_table(max_pos: int, rope_dim: int, theta: float, device) -> torch.Tensor:
    """(cos, sin) of every (position, rotary pair): f32 ``[max_pos, rope_dim / 2, 2]``, computed in float64."""
    j = torch.arange(rope_dim // 2, dtype=torch.float64)
    inv = theta ** (-2.0 * j / rope_dim)
    ang = torch.arange(max_pos, dtype=torch.float64).unsqueeze(-1) * inv
    return torch.stack([ang.cos(), ang.sin()], -1).to(torch.float32).to(device).contiguous()


def mrope_positions(positions3: torch.Tensor, sections, pairs: int) -> torch.Tensor:
    """Position used by every rotary pair under M-RoPE: ``[T, pairs]`` from ``positions3 [3, T]`` (t, h, w) and the
    section sizes: pair j belongs to section j % 3 while j < 3 * size of that section, otherwise to the temporal one."""
    j = torch.arange(pairs, device=positions3.device)
    which = torch.zeros(pairs, dtype=torch.long, device=positions3.device)
    which[(j % 3 == 1) & (j < 3 * sections[1])] = 1
    which[(j % 3 == 2) & (j < 3 * sections[2])] = 2
    return positions3.long().t()[:, which]                     # [T, pairs]


def _rope_pairs_ref(x: torch.Tensor, pos_pairs: torch.Tensor, theta: float, rope_dim: int) -> torch.Tensor:
    """NeoX rotation with an own position per (token, pair)."""
    half = rope_dim // 2
    j = torch.arange(half, dtype=torch.float32, device=x.device)
    ang = pos_pairs.to(torch.float32) * theta ** (-2.0 * j / rope_dim)
    cos, sin = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
    xf = x.float().clone()
    a, b = xf[..., :half].clone(), xf[..., half:rope_dim].clone()
    xf[..., :half] = a * cos - b * sin
    xf[..., half:rope_dim] = a * sin + b * cos
    return xf


def qk_norm_rope_ref(qkv, positions, q_w, k_w, hq, hkv, d, theta, eps, q_scale, rope_dim=None, positions3=None, sections=None):
    t = qkv.shape[0]
    q = qkv[:, : hq * d].float().reshape(t, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].float().reshape(t, hkv, d)
    v = qkv[:, (hq + hkv) * d:(hq + 2 * hkv) * d].reshape(t, hkv, d)
    if q_w is not None:
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_w.float()
    if k_w is not None:
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_w.float()
    if positions3 is not None and sections:
        rd = rope_dim or d
        pp = mrope_positions(positions3, sections, rd // 2)
        q = _rope_pairs_ref(q, pp, theta, rd) * q_scale
        k = _rope_pairs_ref(k, pp, theta, rd)
    else:
        q = rope_ref(q, positions, theta, rope_dim) * q_scale
        k = rope_ref(k, positions, theta, rope_dim)
    return q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)


def qk_norm_rope(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, q_w, k_w, k_cache: torch.Tensor,
                 v_cache: torch.Tensor, hq: int, hkv: int, d: int, theta: float, eps: float, q_scale: float,
                 rope_dim: Optional[int] = None, table: Optional[torch.Tensor] = None, positions3: Optional[torch.Tensor] = None,
                 sections=None) -> torch.Tensor:
    """Per-head RMSNorm (optional) + RoPE on the fused QKV rows; K / V go to cache slot ``slots[t]``.

    ``k_cache`` / ``v_cache`` are ``[num_slots, Hkv, D]``.  Returns ``q [T, Hq, D]`` multiplied by ``q_scale``.
    ``table`` (from ``rope_table``) replaces the in-kernel powf / sincosf; ``positions3`` int32 ``[3, T]`` + ``sections`` select
    M-RoPE.
    """
    if hasattr(qkv, "buf"):                  # ops.gemm.PendingPartials: K-split partial sums of the QKV projection
        pend = qkv
        pairs = (rope_dim or d) // 2
        if pend.buf.is_cuda and d == 128 and pairs == 64 and pend.hidden % 4 == 0:
            t = pend.rows
            q_out = torch.empty(t, hq, d, dtype=torch.bfloat16, device=pend.buf.device)
            rc = _native.cuda().gb_qk_norm_rope_partials(_p(pend.buf), _i(pend.n), _l(pend.rows * pend.hidden), _p(positions), _p(slots), _p(q_w),
                                                         _p(k_w), _p(q_out), _p(k_cache), _p(v_cache), _i(t), _i(hq), _i(hkv), _f(theta), _f(eps),
                                                         _i(pend.hidden), _f(q_scale), _p(table), _i(table.shape[0] if table is not None else 0),
                                                         _p(positions3 if (positions3 is not None and sections) else None),
                                                         _i(3 * sections[1] if sections else 0), _i(3 * sections[2] if sections else 0), _s())
            _native.check(rc, "gb_qk_norm_rope_partials")
            return q_out
        qkv = pend.materialize()
    t = qkv.shape[0]
    if not qkv.is_cuda:
        q, k, v = qk_norm_rope_ref(qkv, positions, q_w, k_w, hq, hkv, d, theta, eps, q_scale, rope_dim, positions3, sections)
        ok = slots >= 0
        k_cache[slots[ok].long()] = k[ok]
        v_cache[slots[ok].long()] = v[ok]
        return q
    q_out = torch.empty(t, hq, d, dtype=torch.bfloat16, device=qkv.device)
    pairs = (rope_dim or d) // 2
    rc = _native.cuda().gb_qk_norm_rope(_p(qkv), _p(positions), _p(slots), _p(q_w), _p(k_w), _p(q_out), _p(k_cache),
                                        _p(v_cache), _i(t), _i(hq), _i(hkv), _i(d), _i(pairs), _f(theta), _f(eps),
                                        _i(qkv.stride(0)), _f(q_scale), _p(table), _i(table.shape[0] if table is not None else 0),
                                        _p(positions3 if (positions3 is not None and sections) else None),
                                        _i(3 * sections[1] if sections else 0), _i(3 * sections[2] if sections else 0), _s())
    _native.check(rc, "gb_qk_norm_rope")
    return q_out


# ------------------------------------------------------------------------------------------ misc
def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` over ``[rows, 2I]`` rows laid out as [gate | up]."""
    rows, two_i = gate_up.shape
    inter = two_i // 2
    if not gate_up.is_cuda:
        g = gate_up.float()
        return (torch.nn.functional.silu(g[:, :inter]) * g[:, inter:]).to(torch.bfloat16)
    out = torch.empty(rows, inter, dtype=torch.bfloat16, device=gate_up.device)
    _native.check(_native.cuda().gb_silu_mul(_p(gate_up), _p(out), _l(rows), _i(inter), _i(gate_up.stride(0)), _s()),
                  "gb_silu_mul")
    return out


def silu_mul_partials(pend, quantize: bool = False, sf_layout: int = 128):
    """SiLU(gate) * up from the K-split partial sums of ``ops.gemm.swiglu_partials`` (``pend.buf`` f32 ``[S, M, 2I]``): bf16 ``[M, I]``, or
    an ``MxTensor`` when ``quantize``."""
    s_, m, two_i = pend.buf.shape
    inter = two_i // 2
    if not pend.buf.is_cuda:
        y = pend.buf.sum(0)
        h = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
        return mxfp8.quantize(h, sf_layout=sf_layout) if quantize else h.to(torch.bfloat16)
    dev = pend.buf.device
    out = q = sf = None
    if quantize:
        rp = (m + 127) // 128 * 128
        q = torch.empty(rp, inter, dtype=torch.uint8, device=dev)
        sf = sf_alloc(rp, inter, dev, sf_layout, init=False)
    else:
        out = torch.empty(m, inter, dtype=torch.bfloat16, device=dev)
    rc = _native.cuda().gb_silu_mul_partials(_p(pend.buf), _i(s_), _l(m * two_i), _p(out), _p(q), _p(sf), _l(m), _i(inter),
                                             _i(1 if sf_layout == 32 else 0), _s())
    _native.check(rc, "gb_silu_mul_partials")
    return MxTensor(q, sf, m, inter, sf_layout) if quantize else out


def silu_mul_quant(gate_up: torch.Tensor, out_q: torch.Tensor, out_sf: torch.Tensor, row_valid: Optional[torch.Tensor] = None,
                   sf_layout: int = 128) -> None:
    """``SiLU(gate) * up`` of ``gate_up [rows, 2I]`` (bf16) quantised to MXFP8 into ``out_q [rows, I]`` / ``out_sf`` (scale atoms of
    layout ``sf_layout``).  Rows with ``row_valid < 0`` are left untouched."""
    rows, two_i = gate_up.shape
    inter = two_i // 2
    if not gate_up.is_cuda:
        g = gate_up.float()
        h = torch.nn.functional.silu(g[:, :inter]) * g[:, inter:]
        t = mxfp8.quantize(h, sf_layout=sf_layout)
        out_q[:rows].copy_(t.data[:rows])
        out_sf.copy_(t.sf[: out_sf.shape[0]])
        return
    _native.check(_native.cuda().gb_silu_mul_quant(_p(gate_up), _p(row_valid), _p(out_q), _p(out_sf), _l(rows), _i(inter),
                                                   _i(gate_up.stride(0)), _i(1 if sf_layout == 32 else 0), _s()), "gb_silu_mul_quant")


def mx_quantize(x: torch.Tensor, src_rows: Optional[torch.Tensor] = None, out_rows: Optional[int] = None,
                sf_layout: int = 128) -> MxTensor:
    """bf16 ``[rows, K]`` -> MXFP8.  With ``src_rows`` (int32) output row r is input row ``src_rows[r]``
    (negative = padding row, left unwritten on the GPU and zero on the CPU): the gather of MoE dispatch fused with the
    quantiser."""
    k = x.shape[1]
    n = out_rows if out_rows is not None else (src_rows.numel() if src_rows is not None else x.shape[0])
    if not x.is_cuda:
        if src_rows is not None:
            g = torch.zeros(n, k, dtype=torch.float32)
            ok = src_rows[:n] >= 0
            g[ok] = x.float()[src_rows[:n][ok].long()]
        else:
            g = x.float()
        t = mxfp8.quantize(g, sf_layout=sf_layout)
        return t
    rp = (n + 127) // 128 * 128
    q = torch.empty(rp, k, dtype=torch.uint8, device=x.device)
    sf = sf_alloc(rp, k, x.device, sf_layout, init=False)
    _native.check(_native.cuda().gb_mx_quant(_p(x), _p(src_rows), _p(q), _p(sf), _l(n), _i(k), _i(x.stride(0)),
                                             _i(1 if sf_layout == 32 else 0), _s()), "gb_mx_quant")
    return MxTensor(q, sf, n, k, sf_layout)


def mx_gather_rows(x: MxTensor, src_rows: torch.Tensor, sf_layout: int = 128) -> MxTensor:
    """Rows of an MXFP8 tensor in the order of ``src_rows`` (int32; negative = padding row, left unwritten on the GPU and zero
    on the CPU), scales re-laid for ``sf_layout``: the MoE gather when the tokens are already quantised."""
    n, k = src_rows.numel(), x.k
    if not x.data.is_cuda:
        g = torch.zeros(n, k, dtype=torch.float32)
        ok = src_rows >= 0
        g[ok] = mxfp8.dequantize(x)[src_rows[ok].long()]
        return mxfp8.quantize(g, sf_layout=sf_layout)
    rp = (n + 127) // 128 * 128
    q = torch.empty(rp, k, dtype=torch.uint8, device=x.data.device)
    sf = sf_alloc(rp, k, x.data.device, sf_layout, init=False)
    _native.check(_native.cuda().gb_mx_gather_rows(_p(x.data), _p(x.sf), _p(src_rows), _p(q), _p(sf), _l(n), _i(k),
                                                   _i(1 if x.sf_layout == 32 else 0), _i(1 if sf_layout == 32 else 0), _s()), "gb_mx_gather_rows")
    return MxTensor(q, sf, n, k, sf_layout)


def softmax_scale_log2(d: int) -> float:
    """``q_scale`` that the attention kernel expects folded into Q: 1/sqrt(d) * log2(e)."""
    return (1.0 / math.sqrt(d)) * math.log2(math.e)


def decode_advance(positions: torch.Tensor, kv_len: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, page_size: int,
                   live: Optional[torch.Tensor] = None, step_ctr: Optional[torch.Tensor] = None, cp_world: int = 1, cp_rank: int = 0) -> None:
    """In place: position += 1, kv_len = position + 1, slot from the block table (per decode sequence).  ``step_ctr`` (int64 [1]):
    the step counter of the sampler, advanced by one (``ops.sampling.sample`` reads it on the device).  ``cp_world > 1`` (context
    parallelism, page g of a sequence on rank g % world): positions stay global, ``kv_len`` counts the positions this rank stores,
    ``block_table`` holds this rank's pages and the slot is -1 where another rank stores the new position."""
    n = positions.numel()
    if cp_world > 1:
        assert live is None
        if not positions.is_cuda:
            if step_ctr is not None:
                step_ctr += 1
            positions += 1
            rnd = page_size * cp_world
            rem = ((positions + 1) % rnd - cp_rank * page_size).clamp(0, page_size)
            kv_len.copy_((positions + 1) // rnd * page_size + rem)
            g = positions // page_size
            pages = block_table[torch.arange(n), (g // cp_world).long().clamp_max(block_table.shape[1] - 1)]
            slots.copy_(torch.where(g % cp_world == cp_rank, pages * page_size + positions % page_size, torch.full_like(slots, -1)))
            return
        _native.check(_native.cuda().gb_decode_advance_cp(_p(positions), _p(kv_len), _p(slots), _p(block_table), _i(block_table.shape[1]),
                                                          _i(page_size), _i(n), _i(cp_world), _i(cp_rank), _p(step_ctr), _s()),
                      "gb_decode_advance_cp")
        return
    if not positions.is_cuda:
        if step_ctr is not None:
            step_ctr += 1
        sel = torch.ones(n, dtype=torch.bool) if live is None else live.bool()
        positions[sel] += 1
        kv_len[sel] = positions[sel] + 1
        idx = torch.arange(n)[sel]
        pages = block_table[idx, (positions[sel] // page_size).long().clamp_max(block_table.shape[1] - 1)]
        slots[sel] = pages * page_size + positions[sel] % page_size
        return
    _native.check(_native.cuda().gb_decode_advance(_p(positions), _p(kv_len), _p(slots), _p(block_table), _p(live),
                                                   _i(block_table.shape[1]), _i(page_size), _i(n), _p(step_ctr), _s()), "gb_decode_advance")
