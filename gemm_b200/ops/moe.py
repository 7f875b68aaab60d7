"""Mixture-of-experts routing ops (csrc/kernels/moe.cu) and their PyTorch references.

``route``    router logits -> top-k ids and weights (softmax + renormalise, or sigmoid + bias)
``plan``     expert-sorted row layout for the grouped GEMM, computed on the device
``combine``  router-weighted sum of the k expert outputs of every token

Reference semantics: common/transformer.h:4050-4130 (softmax over all experts, top-k, renormalise, weighted
sum) and common/m3_impl.h:692-714 (sigmoid router with selection bias and routed scale).
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import _native

_c, _i, _f, _l = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_long


def _p(t):
    return _c(t.data_ptr()) if t is not None else _c(0)


def _s():
    return _c(torch.cuda.current_stream().cuda_stream)


def router_logits(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Router logits ``f32 [T, E] = h [T, H] @ w [E, H]^T`` (bf16 operands).  Up to 256 tokens run on a CUDA-core kernel that spreads
    the small matrix over many CTAs; larger batches use the tensor-core GEMM."""
    from . import gemm
    t, k = h.shape
    if h.is_cuda and t <= 256 and k % 256 == 0 and k <= 8192 and h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        out = torch.empty(t, w.shape[0], dtype=torch.float32, device=h.device)
        rc = _native.cuda().gb_small_linear(_p(h), _p(w), _p(out), _i(t), _i(w.shape[0]), _i(k), _i(h.stride(0)), _i(w.stride(0)),
                                            _i(out.stride(0)), _s())
        _native.check(rc, "gb_small_linear")
        return out
    return gemm.linear(h, w, out_dtype=torch.float32)


def route_ref(logits: torch.Tensor, k: int, mode: str = "softmax", bias: Optional[torch.Tensor] = None,
              renorm: bool = True, routed_scale: float = 1.0):
    lf = torch.nan_to_num(logits.float(), nan=-3.4e38)
    if mode == "softmax":
        p = torch.softmax(lf, dim=-1)
        sel = p
    else:
        p = torch.sigmoid(lf)
        sel = p + (bias.float() if bias is not None else 0.0)
    # ties -> lower index: stable descending sort
    order = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, :k]
    w = torch.gather(p, 1, order)
    if renorm:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return order.to(torch.int32), (w * routed_scale).float()


def route(logits: torch.Tensor, k: int, mode: str = "softmax", bias: Optional[torch.Tensor] = None, renorm: bool = True,
          routed_scale: float = 1.0, local_range: Optional[Tuple[int, int]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``logits`` f32 [T, E] -> (ids int32 [T, k], weights f32 [T, k]).  ``local_range = (first, count)`` turns the ids into
    indices of this rank's experts (``id - first``) and marks the picks that belong to other ranks with -1; the weights are
    still those of the full top-k."""
    if not logits.is_cuda:
        ids, w = route_ref(logits, k, mode, bias, renorm, routed_scale)
        if local_range is not None:
            lid = ids - local_range[0]
            ids = torch.where((lid >= 0) & (lid < local_range[1]), lid, torch.full_like(lid, -1))
        return ids, w
    t, e = logits.shape
    ids = torch.empty(t, k, dtype=torch.int32, device=logits.device)
    w = torch.empty(t, k, dtype=torch.float32, device=logits.device)
    rc = _native.cuda().gb_moe_route(_p(logits), _p(bias), _p(ids), _p(w), _i(t), _i(e), _i(k), _i(0 if mode == "softmax" else 1),
                                     _i(1 if renorm else 0), _f(routed_scale), _i(logits.stride(0)),
                                     _i(local_range[0] if local_range else 0), _i(local_range[1] if local_range else 0), _s())
    _native.check(rc, "gb_moe_route")
    return ids, w


# Off by default: on the 48-layer benchmark model (64 tokens x top-8 of 128 experts per step) the cluster kernel measured 13.55 ms per
# decode step against 13.45 ms for the projection kernel followed by the routing kernel (8 co-scheduled CTAs and a cluster
# barrier cost more than the launch they save).  GB_FUSED_ROUTER=1 switches it on.
FUSED_ROUTER = os.environ.get("GB_FUSED_ROUTER", "0") == "1"


def can_route_hidden(h: torch.Tensor, w: torch.Tensor, k: int) -> bool:
    """Shapes the fused router projection + routing kernel takes: decode-sized batches, at most 128 experts."""
    e, hid = w.shape
    return bool(FUSED_ROUTER and h.is_cuda and h.shape[0] <= 64 and e <= 128 and e % 16 == 0 and hid % 256 == 0 and hid <= 8192 and k <= 16
                and h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and h.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)


def route_hidden(h: torch.Tensor, w: torch.Tensor, k: int, mode: str = "softmax", bias: Optional[torch.Tensor] = None, renorm: bool = True,
                 routed_scale: float = 1.0, local_range: Optional[Tuple[int, int]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``route(router_logits(h, w), ...)`` in one launch (a thread-block cluster per 8 tokens keeps the logits in shared memory).
    Falls back to the two ops for shapes ``can_route_hidden`` refuses."""
    if not can_route_hidden(h, w, k):
        return route(router_logits(h, w), k, mode, bias, renorm, routed_scale, local_range)
    t, e = h.shape[0], w.shape[0]
    ids = torch.empty(t, k, dtype=torch.int32, device=h.device)
    wt = torch.empty(t, k, dtype=torch.float32, device=h.device)
    rc = _native.cuda().gb_router_route(_p(h), _p(w), _i(t), _i(e), _i(h.shape[1]), _i(h.stride(0)), _i(w.stride(0)), _p(bias), _p(ids), _p(wt),
                                        _i(k), _i(0 if mode == "softmax" else 1), _i(1 if renorm else 0), _f(routed_scale),
                                        _i(local_range[0] if local_range else 0), _i(local_range[1] if local_range else 0), _s())
    _native.check(rc, "gb_router_route")
    return ids, wt


def route_plan_hidden(h: torch.Tensor, w: torch.Tensor, k: int, n_exp: int, align: int, mode: str = "softmax",
                      bias: Optional[torch.Tensor] = None, renorm: bool = True, routed_scale: float = 1.0,
                      local_range: Optional[Tuple[int, int]] = None, regions: int = 1, epoch_ctr: int = 0, region_rows: Optional[int] = None):
    """Router projection, routing and plan from the hidden rows: ``(ids, weights, MoePlan)`` (see ``route_plan``)."""
    if can_route_hidden(h, w, k) and h.shape[0] * k > FUSED_ROUTE_PAIRS:
        ids, wt = route_hidden(h, w, k, mode, bias, renorm, routed_scale, local_range)
        return ids, wt, plan(ids, n_exp, align, regions, epoch_ctr=epoch_ctr, region_rows=region_rows)
    return route_plan(router_logits(h, w), k, n_exp, align, mode, bias, renorm, routed_scale, local_range, regions, epoch_ctr, region_rows)


# One-launch router + routing + plan + gather for decode-sized batches (csrc/kernels/moe_prep.cu); GB_MOE_PREP=0 keeps the
# separate kernels.
MOE_PREP = os.environ.get("GB_MOE_PREP", "1") != "0"


def can_prep(h: torch.Tensor, w: torch.Tensor, k: int) -> bool:
    """Shapes ``prep_hidden`` takes: up to 64 tokens, up to 128 experts, hidden a multiple of 256 (256 .. 4096 in powers of two)."""
    if not (MOE_PREP and h.is_cuda and h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and h.stride(1) == 1 and w.stride(1) == 1):
        return False
    if h.stride(0) % 8 or w.stride(0) % 8 or h.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    return bool(_native.cuda().gb_moe_prep_supported(_i(h.shape[0]), _i(h.shape[1]), _i(w.shape[0]), _i(k)))


def prep_hidden(h: torch.Tensor, w: torch.Tensor, k: int, n_exp: int, align: int, mode: str = "softmax", bias: Optional[torch.Tensor] = None,
                renorm: bool = True, routed_scale: float = 1.0, local_range: Optional[Tuple[int, int]] = None, quantize: bool = True,
                wait_flags: int = 0, wait_n: int = 0, epoch_ptr: int = 0):
    """Router projection, routing, plan AND the gather of the token rows into expert order in one launch.

    Returns ``(ids, weights, MoePlan, rows)``; ``rows`` is an ``MxTensor`` (MXFP8 with scale atoms in the ``align``-row layout,
    ``align`` 32 or 128) when ``quantize`` else a bf16 tensor ``[capacity, hidden]``.  Rows of the buffer that no (token, expert)
    pair maps to are left unwritten: the grouped GEMM computes them and drops them.  ``n_exp`` is the number of experts the plan
    covers (the local count with ``local_range``).  ``wait_*``: flags of peer GPUs to wait for before the tokens are read."""
    from . import elementwise as ew
    from .mxfp8 import MxTensor
    t, hid = h.shape
    dev = h.device
    n_pairs = t * k
    _, capacity = plan_capacity(n_pairs, n_exp, align, 1, k)
    ids = torch.empty(t, k, dtype=torch.int32, device=dev)
    wt = torch.empty(t, k, dtype=torch.float32, device=dev)
    seg_start = torch.empty(n_exp, dtype=torch.int32, device=dev)
    seg_count = torch.empty(n_exp, dtype=torch.int32, device=dev)
    pair_row = torch.empty(n_pairs, dtype=torch.int32, device=dev)
    row_token = torch.empty(capacity, dtype=torch.int32, device=dev)
    xq = xsf = xs = None
    if quantize:
        assert align in (32, 128) and hid % 128 == 0
        xq = torch.empty(capacity, hid, dtype=torch.uint8, device=dev)
        xsf = ew.sf_alloc(capacity, hid, dev, align, init=False)
    else:
        xs = torch.empty(capacity, hid, dtype=torch.bfloat16, device=dev)
    rc = _native.cuda().gb_moe_prep(_p(h), _i(h.stride(0)), _i(t), _i(hid), _p(w), _i(w.stride(0)), _i(w.shape[0]), _p(bias), _i(k),
                                    _i(0 if mode == "softmax" else 1), _i(1 if renorm else 0), _f(routed_scale),
                                    _i(local_range[0] if local_range else 0), _i(local_range[1] if local_range else 0), _i(align),
                                    _i(capacity), _p(ids), _p(wt), _p(seg_start), _p(seg_count), _p(pair_row), _p(row_token), _p(xq), _p(xsf),
                                    _i(1 if align == 32 else 0), _p(xs), _c(wait_flags), _i(wait_n), _c(epoch_ptr),
                                    _c(_native.status_ptr()), _s())
    _native.check(rc, "gb_moe_prep")
    pl = MoePlan(seg_start, seg_count, pair_row, row_token, torch.empty(0, dtype=torch.int32, device=dev), capacity, capacity)
    rows = MxTensor(xq, xsf, capacity, hid, align) if quantize else xs
    return ids, wt, pl, rows


# gate/up + activation + down of a decode-sized batch as one persistent launch (GB_MOE_FFN_FUSED=0: two grouped GEMMs)
MOE_FFN_FUSED = os.environ.get("GB_MOE_FFN_FUSED", "1") != "0"
_ffn_ctr = {}


def can_fuse_ffn(xq, w13, w2, n_groups: int, capacity: int) -> bool:
    """Shapes ``expert_ffn_fused`` takes: MXFP8 rows with one scale atom per 32 rows, tiled MXFP8 expert weights."""
    if not (MOE_FFN_FUSED and xq.data.is_cuda and xq.sf_layout == 32 and w13.mx is not None and w2.mx is not None and w13.mx.tiled and w2.mx.tiled):
        return False
    return bool(_native.cuda().gb_moe_ffn_supported(_i(w13.k), _i(w2.k), _i(n_groups), _i(capacity)))


def expert_ffn_fused(xq, w13, w2, n_groups: int, pl: "MoePlan", scatter: Optional[dict] = None) -> torch.Tensor:
    """``y [capacity, hidden]`` bf16: rows of ``xq`` (an ``MxTensor`` in expert order, 32-row scale atoms) through
    ``down(SiLU(gate(x)) * up(x))`` of their expert.  Rows beyond a segment's count are not written.

    ``scatter`` (expert parallelism, every rank holds all tokens): ``dict(weights, n_tok, k, tokens_per_rank, slots, flags, world,
    epoch)``; the launch then also forms every token's router-weighted sum of its local rows and stores it (fp32) into this
    rank's slot on the token's home GPU, and raises the flags (what ``gb_moe_combine_scatter`` does as a launch of its own)."""
    from . import elementwise as ew
    lib = _native.cuda()
    dev = xq.data.device
    hid, inter, cap = w13.k, w2.k, pl.capacity
    key = (dev.index, torch.cuda.current_stream().cuda_stream)
    ctr = _ffn_ctr.get(key)
    if ctr is None:
        # one counter block per stream: launches on one stream run one after the other, the kernel leaves the block zeroed
        ctr = _ffn_ctr[key] = torch.zeros(int(lib.gb_moe_ffn_ctr_count()), dtype=torch.int32, device=dev)
    hq = torch.empty(cap, inter, dtype=torch.uint8, device=dev)
    hsf = ew.sf_alloc(cap, inter, dev, 32, init=False)
    y = torch.empty(cap, hid, dtype=torch.bfloat16, device=dev)
    nb = lambda t: _l(t.numel() * t.element_size())
    rc = lib.gb_moe_ffn(_p(w13.mx.data), _p(w13.mx.sf), nb(w13.mx.sf), _p(w2.mx.data), _p(w2.mx.sf), nb(w2.mx.sf),
                        _p(xq.data), _i(xq.data.stride(0)), _p(xq.sf), nb(xq.sf), _p(hq), _i(hq.stride(0)), _p(hsf), nb(hsf),
                        _p(y), _i(y.stride(0)), nb(y), _i(hid), _i(inter), _i(n_groups), _p(pl.seg_start), _p(pl.seg_count), _i(cap),
                        _p(ctr), _i(ctr.numel()),
                        _p(pl.pair_row) if scatter else _c(0), _p(scatter["weights"]) if scatter else _c(0),
                        _i(scatter["n_tok"] if scatter else 0), _i(scatter["k"] if scatter else 0),
                        _i(scatter["tokens_per_rank"] if scatter else 0), scatter["slots"] if scatter else _c(0),
                        scatter["flags"] if scatter else _c(0), _i(scatter["world"] if scatter else 0),
                        _c(scatter["epoch"]) if scatter else _c(0), _c(_native.status_ptr()), _s())
    _native.check(rc, "gb_moe_ffn")
    return y


@dataclass
class MoePlan:
    seg_start: torch.Tensor      # int32 [E]   first row of each expert's segment
    seg_count: torch.Tensor      # int32 [E]   valid rows per expert
    pair_row: torch.Tensor       # int32 [T*k] row of every (token, k) pair (-1 = dropped)
    row_token: torch.Tensor      # int32 [capacity] source token of every row (-1 = padding)
    region_used: torch.Tensor    # int32 [regions] rows used (padded) in each region
    capacity: int
    region_rows: int


def plan_capacity(n_pairs: int, n_exp: int, align: int, regions: int = 1, k: int = 8) -> Tuple[int, int]:
    """(rows per region, total rows) that can never overflow, whatever the routing."""
    epr = n_exp // regions
    tokens = (n_pairs + k - 1) // k
    per_region = tokens * min(k, epr) + epr * (align - 1)
    per_region = (per_region + 127) // 128 * 128
    return per_region, per_region * regions


def plan_ref(ids: torch.Tensor, n_exp: int, k: int, align: int, regions: int = 1) -> MoePlan:
    """CPU reference of the device plan.  Ids outside ``[0, n_exp)`` are dropped (their ``pair_row`` is -1)."""
    flat = ids.reshape(-1).long()
    n_pairs = flat.numel()
    region_rows, capacity = plan_capacity(n_pairs, n_exp, align, regions, k)
    epr = n_exp // regions
    ok = (flat >= 0) & (flat < n_exp)
    counts = torch.bincount(flat[ok], minlength=n_exp)[:n_exp]
    seg_start = torch.zeros(n_exp, dtype=torch.int64)
    region_used = torch.zeros(regions, dtype=torch.int64)
    for r in range(regions):
        pos = 0
        for i in range(epr):
            e = r * epr + i
            seg_start[e] = r * region_rows + pos
            pos += (int(counts[e]) + align - 1) // align * align
        region_used[r] = pos
    key = torch.where(ok, flat, torch.full_like(flat, n_exp))
    order = torch.sort(key, stable=True).indices              # by expert, then (token, k)
    sorted_e = key[order]
    first = torch.zeros(n_exp + 2, dtype=torch.int64)
    first[1:n_exp + 1] = torch.cumsum(counts, 0)
    first[n_exp + 1] = n_pairs
    rank = torch.zeros(n_pairs, dtype=torch.int64)
    rank[order] = torch.arange(n_pairs) - first[sorted_e]
    pair_row = torch.where(ok, seg_start[flat.clamp(0, n_exp - 1)] + rank, torch.full_like(flat, -1))
    row_token = torch.full((capacity,), -1, dtype=torch.int32)
    row_token[pair_row[ok]] = (torch.arange(n_pairs)[ok] // k).to(torch.int32)
    return MoePlan(seg_start.to(torch.int32), counts.to(torch.int32), pair_row.to(torch.int32), row_token,
                   region_used.to(torch.int32), capacity, region_rows)


def plan(ids: torch.Tensor, n_exp: int, align: int, regions: int = 1, workspace=None, epoch_ctr: int = 0,
         region_rows: Optional[int] = None) -> MoePlan:
    """Device-side plan from ``ids int32 [T, k]``; no host synchronisation.  ``region_rows`` fixes the rows per
    region (expert parallel: the same value on every rank); it must be at least ``plan_capacity``'s."""
    t, k = ids.shape
    if not ids.is_cuda:
        return plan_ref(ids, n_exp, k, align, regions)
    n_pairs = t * k
    need_rows, capacity = plan_capacity(n_pairs, n_exp, align, regions, k)
    if region_rows is None:
        region_rows = need_rows
    else:
        assert region_rows >= need_rows and region_rows % 128 == 0
        capacity = region_rows * regions
    dev = ids.device
    nb = (n_pairs + 255) // 256
    ws = torch.empty(max(1, nb * n_exp), dtype=torch.int32, device=dev)
    seg_start = torch.empty(n_exp, dtype=torch.int32, device=dev)
    seg_count = torch.empty(n_exp, dtype=torch.int32, device=dev)
    region_used = torch.empty(regions, dtype=torch.int32, device=dev)
    pair_row = torch.empty(n_pairs, dtype=torch.int32, device=dev)
    row_token = torch.empty(capacity, dtype=torch.int32, device=dev)
    rc = _native.cuda().gb_moe_plan(_p(ids), _p(ws), _p(seg_start), _p(seg_count), _p(region_used), _p(pair_row), _p(row_token),
                                    _l(n_pairs), _i(n_exp), _i(k), _i(n_exp // regions), _i(region_rows), _i(align),
                                    _l(capacity), _c(epoch_ctr), _s())
    _native.check(rc, "gb_moe_plan", n=1 if n_pairs <= 2048 else 4)
    return MoePlan(seg_start, seg_count, pair_row, row_token, region_used, capacity, region_rows)


# Up to this many (token, expert) pairs routing and planning run as one single-CTA kernel.  Above it the routing alone keeps
# one SM busy for longer than the separate kernels take: measured on the 48-layer benchmark model, 64 tokens x top-8 per
# step, 14.25 ms per decode step fused against 13.79 ms with the routing in its own multi-CTA kernel.
FUSED_ROUTE_PAIRS = int(os.environ.get("GB_FUSED_ROUTE_PAIRS", "256"))


def route_plan(logits: torch.Tensor, k: int, n_exp: int, align: int, mode: str = "softmax", bias: Optional[torch.Tensor] = None,
               renorm: bool = True, routed_scale: float = 1.0, local_range: Optional[Tuple[int, int]] = None, regions: int = 1,
               epoch_ctr: int = 0, region_rows: Optional[int] = None):
    """``route`` followed by ``plan``; decode-sized batches (T * k <= ``FUSED_ROUTE_PAIRS``) do both in ONE kernel.  ``n_exp`` is the number of
    experts the plan is built over (the local count when ``local_range`` is given).  Returns ``(ids, weights, MoePlan)``."""
    t, e_all = logits.shape
    if not logits.is_cuda or t * k > FUSED_ROUTE_PAIRS:
        ids, w = route(logits, k, mode, bias, renorm, routed_scale, local_range)
        return ids, w, plan(ids, n_exp, align, regions, epoch_ctr=epoch_ctr, region_rows=region_rows)
    dev = logits.device
    n_pairs = t * k
    need_rows, capacity = plan_capacity(n_pairs, n_exp, align, regions, k)
    if region_rows is None:
        region_rows = need_rows
    else:
        assert region_rows >= need_rows and region_rows % 128 == 0
        capacity = region_rows * regions
    ids = torch.empty(t, k, dtype=torch.int32, device=dev)
    w = torch.empty(t, k, dtype=torch.float32, device=dev)
    seg_start = torch.empty(n_exp, dtype=torch.int32, device=dev)
    seg_count = torch.empty(n_exp, dtype=torch.int32, device=dev)
    region_used = torch.empty(regions, dtype=torch.int32, device=dev)
    pair_row = torch.empty(n_pairs, dtype=torch.int32, device=dev)
    row_token = torch.empty(capacity, dtype=torch.int32, device=dev)
    rc = _native.cuda().gb_moe_route_plan(_p(logits), _p(bias), _p(ids), _p(w), _i(t), _i(e_all), _i(k), _i(0 if mode == "softmax" else 1),
                                          _i(1 if renorm else 0), _f(routed_scale), _i(logits.stride(0)),
                                          _i(local_range[0] if local_range else 0), _i(local_range[1] if local_range else 0),
                                          _p(seg_start), _p(seg_count), _p(region_used), _p(pair_row), _p(row_token), _i(n_exp),
                                          _i(n_exp // regions), _i(region_rows), _i(align), _l(capacity), _c(epoch_ctr), _s())
    _native.check(rc, "gb_moe_route_plan")
    return ids, w, MoePlan(seg_start, seg_count, pair_row, row_token, region_used, capacity, region_rows)


def combine(y: torch.Tensor, pair_row: torch.Tensor, weights: Optional[torch.Tensor], n_tok: int, k: int,
            wait_flags: int = 0, wait_n: int = 0, epoch_ptr: int = 0) -> torch.Tensor:
    """``out[t] = sum_j weights[t, j] * y[pair_row[t*k + j]]`` (bf16, fp32 accumulation in fixed order)."""
    hidden = y.shape[1]
    if not y.is_cuda:
        rows = pair_row.reshape(n_tok, k).long()
        g = y.float()[rows.clamp_min(0)] * (rows >= 0).unsqueeze(-1)
        w = weights.float().unsqueeze(-1) if weights is not None else 1.0
        return (g * w).sum(1).to(torch.bfloat16)
    out = torch.empty(n_tok, hidden, dtype=torch.bfloat16, device=y.device)
    rc = _native.cuda().gb_moe_combine(_p(y), _p(pair_row), _p(weights), _p(out), _i(n_tok), _i(hidden), _i(k), _i(y.stride(0)),
                                       _c(wait_flags), _i(wait_n), _c(epoch_ptr), _c(_native.status_ptr()), _s())
    _native.check(rc, "gb_moe_combine")
    return out


@dataclass
class PendingCombine:
    """Expert outputs whose router-weighted sum has not been formed yet.  ``ops.elementwise.rmsnorm`` accepts it as the
    residual update and does the combine inside the normalisation kernel (one launch and one round trip through memory
    less per MoE layer); ``materialize`` forms the plain tensor."""
    y: torch.Tensor
    pair_row: torch.Tensor
    weights: Optional[torch.Tensor]
    n_tok: int
    k: int
    wait_flags: int = 0
    wait_n: int = 0
    epoch_ptr: int = 0

    @property
    def shape(self):
        return (self.n_tok, self.y.shape[1])

    def materialize(self) -> torch.Tensor:
        return combine(self.y, self.pair_row, self.weights, self.n_tok, self.k, self.wait_flags, self.wait_n, self.epoch_ptr)


def gather_rows(x: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """``out[r] = x[src[r]]`` (zeros where src < 0), bf16."""
    if not x.is_cuda:
        out = torch.zeros(src.numel(), x.shape[1], dtype=x.dtype)
        ok = src >= 0
        out[ok] = x[src[ok].long()]
        return out
    out = torch.empty(src.numel(), x.shape[1], dtype=torch.bfloat16, device=x.device)
    rc = _native.cuda().gb_gather_rows(_p(x), _p(src), _p(out), _l(src.numel()), _i(x.shape[1]), _i(x.stride(0)), _s())
    _native.check(rc, "gb_gather_rows")
    return out
