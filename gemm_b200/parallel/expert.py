"""Expert parallelism over the NVLink fabric: data-parallel attention + expert-parallel MoE.

Rank ``r`` owns the experts ``[r * E/N, (r+1) * E/N)`` and attends to its own sequences.  A MoE layer is

  route + plan (local)  ->  dispatch kernel: gather, MXFP8-quantise and STORE every (token, expert) row into the
  owning GPU's expert buffer over NVLink, then raise a flag there  ->  grouped gate/up GEMM on the owner (waits
  for the flags of all sources, groups = (source rank, local expert))  ->  grouped down GEMM whose epilogue STORES
  the result rows straight back into the source GPU's combine buffer and raises its flag  ->  combine kernel on
  the source (waits for the owners' flags, router-weighted sum in fixed order).

Decode-sized batches (at most ``gather_max`` tokens per rank) take a second route, because there the step is bound by
the expert weights every GPU has to stream, and per-source row groups would make each GPU stream its experts once per
source: the ranks all-gather their few token rows (peer stores), every rank routes ALL tokens and runs its own experts
over one merged token tile per expert, and the combine kernel sums this rank's experts per token in fp32 and stores the
row into its slot on the token's home GPU, where the next RMSNorm kernel adds the ranks' slots to the residual.

No NCCL call and no host synchronisation is involved; the exchange is the prologue / epilogue of the compute
kernels.  ``fused=False`` selects the baseline that only calls NCCL: all-gather the tokens, run the owned experts on
all of them, reduce-scatter the partial sums — the reference's own expert-parallel formulation
("replicate tokens, compute owned experts, all-reduce", common/m3_impl.h:699-714,924-950).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

from .. import _native
from ..ops import elementwise as ew
from ..ops import gemm, moe
from .fabric import Fabric

_c, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t


# token all-gather of the decode route as the epilogue of the RMSNorm in front of the MoE block (GB_FOLD_GATHER=0: exchange kernel)
FOLD_GATHER = os.environ.get("GB_FOLD_GATHER", "1") != "0"
# router-weighted sums + scatter of the decode route as the last phase of the fused expert kernel (GB_FOLD_COMBINE=0: own launch)
FOLD_COMBINE = os.environ.get("GB_FOLD_COMBINE", "1") != "0"


class PendingSlots:
    """fp32 partial sums of a MoE layer sitting in the per-rank slots of this GPU; finished by the next RMSNorm."""

    def __init__(self, g: dict, rows: int):
        self.g, self.rows = g, rows


# GB_EP_DISPATCH_MX=0: the dispatch quantises the bf16 rows itself instead of copying the rows the RMSNorm already quantised
DISPATCH_MX = os.environ.get("GB_EP_DISPATCH_MX", "1") != "0"


class ExpertParallel:
    use_gather = True        # False forces the dispatch route for every batch size (tests)
    tp_size = 1
    tp_rank = 0

    gather_max = 64          # tokens per rank up to which the all-gather route is taken

    def __init__(self, group, device: torch.device, fused: bool = True):
        self.group = group
        self.device = device
        self.ep_size = dist.get_world_size(group)
        self.ep_rank = dist.get_rank(group)
        self.fused = fused
        self.fab: Optional[Fabric] = None
        self._buckets: Dict[int, dict] = {}

    # ------------------------------------------------------------------------------------------ setup
    def attach(self, engine, cfg, max_tokens: int) -> None:
        """Size the symmetric buffers for at most ``max_tokens`` tokens per rank and forward pass."""
        self.cfg = cfg
        self.max_tokens = max_tokens
        self.mx = getattr(getattr(engine, "w", None), "fmt", "bf16") == "mxfp8"
        if not self.fused:
            return
        w, k, e, hid = self.ep_size, cfg.n_experts_used, cfg.n_experts, cfg.hidden
        self.e_local = e // w
        rows_big, _ = moe.plan_capacity(max_tokens * k, e, 128, w, k)
        total_rows = rows_big * w
        mx = engine.w.fmt == "mxfp8"
        x_bytes = total_rows * hid * (1 if mx else 2)
        sf_bytes = (total_rows // 32) * (hid // 128) * 512 if mx else 0
        y_bytes = total_rows * hid * 2
        g_caps = sorted({min(c, max_tokens) for c in (8, 16, 32, self.gather_max)})
        heap = x_bytes + sf_bytes + y_bytes + (4 << 20) + sum(w * c * hid * (2 + 4) + 4096 for c in g_caps)
        self.fab = Fabric(self.group, self.device, heap)
        f = self.fab
        self.x_off = f.alloc(x_bytes)
        self.sf_off = f.alloc(max(sf_bytes, 16))
        self.y_off = f.alloc(y_bytes)
        self.meta_off = f.alloc(2 * w * self.e_local * 4)
        self.flags_d = f.alloc(8 * 4)
        self.flags_c = f.alloc(8 * 4)
        self.epoch = f.ctl_word()
        self.done_d, self.done_g = f.ctl_word(), f.ctl_word()
        self.mx = mx
        self.total_rows_max = total_rows
        self.meta = f.view(self.meta_off, (2, w * self.e_local), torch.int32)
        # all-gather route: per capacity a gather buffer, the fp32 partial slots and one flag per source rank
        self._gather = {}
        for cap in g_caps:
            g = {"cap": cap, "ag": f.make_exchange(cap * hid * 2, chunks=max(1, min(8, cap // 8)), handshake=False)}   # the combine exchange of every layer orders the ranks between two gathers
            g["stage"] = torch.zeros(cap, hid, dtype=torch.bfloat16, device=self.device)
            g["slots_off"] = f.alloc(w * cap * hid * 4)
            g["flags_off"] = f.alloc(32)
            g["epoch"], g["done"] = f.ctl_word(), f.ctl_word()
            g["slot_ptrs"] = (ctypes.c_void_p * 8)(*[f.peer_ptr(p, g["slots_off"]) + self.ep_rank * cap * hid * 4 for p in range(w)])
            g["flag_ptrs"] = (ctypes.c_void_p * 8)(*[f.peer_ptr(p, g["flags_off"]) + 4 * self.ep_rank for p in range(w)])
            # The token all-gather as the epilogue of the RMSNorm in front of the MoE block: the norm stores its rows into this rank's
            # region of every GPU's gather buffer and raises flags the MoE front-end kernel waits on (no exchange launch).  Only
            # where that front-end kernel takes the gathered batch; reuse of the buffer is ordered by the layer's combine round.
            g["fold"] = bool(FOLD_GATHER and moe.MOE_PREP and _native.cuda().gb_moe_prep_supported(_i(w * cap), _i(hid), _i(e), _i(k)))
            if g["fold"]:
                ag = g["ag"]
                g["gflags_off"] = f.alloc(32)
                g["gepoch"], g["gdone"] = f.ctl_word(), f.ctl_word()
                g["recv_local"] = f.view(ag.out_off + self.ep_rank * ag.bytes_per_dst, (cap, hid), torch.bfloat16)
                bc = ew.RmsBcast()
                for p in range(w):
                    bc.out[p] = f.peer_ptr(p, ag.out_off) + self.ep_rank * ag.bytes_per_dst
                    bc.flag[p] = f.peer_ptr(p, g["gflags_off"]) + 4 * self.ep_rank
                bc.world, bc.epoch_ctr, bc.done_ctr = w, g["gepoch"], g["gdone"]
                g["bc"] = bc
                ag.out_view.zero_()          # rows of a region beyond a rank's token count are read (and dropped) by the front end: keep them finite
            self._gather[cap] = g
        self._bcast_done = None
        self.stats = {"fold_gather": 0, "fold_combine": 0}      # how often the folded forms ran (tests assert on them)

    def _bucket(self, t: int) -> dict:
        """Buffer geometry for a forward pass of ``t`` tokens (rounded up so that all ranks agree)."""
        for cap in sorted({min(c, self.max_tokens) for c in (8, 64, 1024, self.max_tokens)}):
            if t <= cap:
                break
        else:
            raise ValueError(f"{t} tokens exceed the expert-parallel buffers ({self.max_tokens})")
        if cap in self._buckets:
            return self._buckets[cap]
        cfg, w = self.cfg, self.ep_size
        k, e, hid, inter = cfg.n_experts_used, cfg.n_experts, cfg.hidden, cfg.expert_ffn
        tn = 32 if (cap * k) // e <= 24 else 128        # rows per (source, expert) group
        rows, _ = moe.plan_capacity(cap * k, e, tn, w, k)
        total = rows * w
        f = self.fab
        b = {"tn": tn, "region_rows": rows, "total": total}
        b["x"] = f.view(self.x_off, (total, hid), torch.uint8 if self.mx else torch.bfloat16)
        b["sf"] = f.view(self.sf_off, (total // tn, hid // 128, 512), torch.uint8) if self.mx else None
        b["y"] = f.view(self.y_off, (total, hid), torch.bfloat16)
        if self.mx:
            b["hq"] = torch.zeros(total, inter, dtype=torch.uint8, device=self.device)
            b["hsf"] = ew.sf_alloc(total, inter, self.device, tn)
        else:
            b["act"] = torch.zeros(total, inter, dtype=torch.bfloat16, device=self.device)
        n_groups = w * self.e_local
        ex1 = gemm.GemmExtras()
        ex1.w_group_mod = self.e_local
        ex1.wait_n = w
        ex1.wait_flags = f.local_base + self.flags_d
        ex1.epoch_ptr = self.epoch
        ex2 = gemm.GemmExtras()
        ex2.w_group_mod = self.e_local
        ex2.epoch_ptr = self.epoch
        for p in range(w):
            ex2.peer_out[p] = f.peer_ptr(p, self.y_off)
            ex2.signal_flags[p] = f.peer_ptr(p, self.flags_c) + 4 * self.ep_rank
        ex2.peer_region_rows = rows
        ex2.peer_rank = self.ep_rank
        ex2.signal_n = w
        ex2.done_ctr = self.done_g
        b["ex1"], b["ex2"], b["groups"] = ex1, ex2, n_groups
        self._buckets[cap] = b
        return b

    # ------------------------------------------------------------------------------------------ model hooks
    def tp_all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def row_linear(self, lw, x, x_mx=None):
        from ..models.transformer import apply_linear_split
        return apply_linear_split(lw, x, x_mx)

    def ffn_in_buffer(self, rows: int, lw):
        """Where the RMSNorm in front of an MoE block should leave its bf16 rows: the staging buffer of the decode all-gather, so that
        no copy kernel runs between the norm and the exchange (None = no preference)."""
        if not (self.fused and self.use_gather and lw.w13 is not None and getattr(self, "_gather", None)) or rows > self.gather_max:
            return None
        caps = [c for c in self._gather if rows <= c]
        if not caps:
            return None
        g = self._gather[min(caps)]
        return g["recv_local"] if g["fold"] else g["stage"]

    def add_norm(self, delta, weight, eps, residual, quantize=False, want_bf16=True, sf_layout=128, out_buf=None):
        if not isinstance(delta, PendingSlots):
            kw = dict(quantize=quantize, want_bf16=want_bf16, sf_layout=sf_layout) if quantize else {}
            if out_buf is not None:
                kw["out_buf"] = out_buf
                g = next((x for x in self._gather.values() if x["fold"] and x["recv_local"].data_ptr() == out_buf.data_ptr()), None) \
                    if getattr(self, "_gather", None) else None
                partial_sums = hasattr(delta, "buf") and delta.buf.is_cuda and residual is not None and residual.stride(0) == self.cfg.hidden
                plain = torch.is_tensor(delta) and delta.is_cuda and residual is not None and delta.stride(0) == residual.stride(0)
                if g is not None and (partial_sums or plain):
                    # o_proj's result (K-split partial sums, or plain rows): added, normalised and all-gathered by one kernel
                    kw["bcast"] = g["bc"]
                    self._bcast_done = g
                    self.stats["fold_gather"] += 1
            return ew.rmsnorm(delta, weight, eps, residual=residual, **kw)
        f, g = self.fab, delta.g
        rows, hidden, cap = delta.rows, self.cfg.hidden, g["cap"]
        out = (out_buf[:rows] if out_buf is not None else torch.empty(rows, hidden, dtype=torch.bfloat16, device=self.device)) \
            if want_bf16 or not quantize else None
        q = sf = None
        if quantize:
            rp = (rows + 127) // 128 * 128
            q = torch.empty(rp, hidden, dtype=torch.uint8, device=self.device)
            sf = ew.sf_alloc(rp, hidden, self.device, sf_layout, init=False)
        p = lambda t: _c(t.data_ptr()) if t is not None else _c(0)
        rc = f.lib.gb_rmsnorm_reduce(p(residual), _c(f.local_base + g["slots_off"]), _i(self.ep_size), ctypes.c_long(cap * hidden), p(weight),
                                     p(out), p(q), p(sf), _i(rows), _i(hidden), ctypes.c_float(eps), _i(1 if sf_layout == 32 else 0),
                                     _c(f.local_base + g["flags_off"]), _i(self.ep_size), _c(g["epoch"]), _c(_native.status_ptr()),
                                     _c(torch.cuda.current_stream().cuda_stream))
        _native.check(rc, "gb_rmsnorm_reduce")
        if quantize:
            from ..ops.mxfp8 import MxTensor
            return out, MxTensor(q, sf, rows, hidden, sf_layout)
        return out

    def materialize(self, delta):
        if isinstance(delta, PendingSlots):
            f, g = self.fab, delta.g
            slots = f.view(g["slots_off"], (self.ep_size, g["cap"], self.cfg.hidden), torch.float32)
            f.barrier()          # every rank's combine kernel (and its stores) precede its arrival at the barrier
            return slots[:, : delta.rows].sum(0).to(torch.bfloat16)
        return delta.materialize() if hasattr(delta, "materialize") else delta

    def _moe_gather(self, model, lw, h: torch.Tensor):
        """Decode-sized batches: all-gather the token rows, run the local experts over all of them, scatter fp32 partial sums."""
        cfg, w, f = self.cfg, self.ep_size, self.fab
        t = h.shape[0]
        k, inter, hid = cfg.n_experts_used, cfg.expert_ffn, cfg.hidden
        g = self._gather[min(c for c in self._gather if t <= c)]
        cap = g["cap"]
        folded = self._bcast_done is g and h.data_ptr() == g["recv_local"].data_ptr()
        self._bcast_done = None
        rt = dict(mode=cfg.router, bias=lw.router_bias, renorm=cfg.norm_topk, routed_scale=cfg.routed_scale,
                  local_range=(self.ep_rank * self.e_local, self.e_local))
        if folded:
            # the norm in front of this block has already stored the rows on every GPU: the front-end kernel waits for the flags
            allh = g["ag"].out_view.view(torch.bfloat16).view(w * cap, hid)
            if not moe.can_prep(allh, lw.router, k):
                raise RuntimeError("expert parallel: the gathered batch does not fit the MoE front-end kernel the folded all-gather relies on "
                                   "(set GB_FOLD_GATHER=0)")
            rt.update(wait_flags=f.local_base + g["gflags_off"], wait_n=w, epoch_ptr=g["gepoch"])
        else:
            if h.data_ptr() != g["stage"].data_ptr():      # a norm that could not gather wrote somewhere else: stage, then exchange
                g["stage"][:t].copy_(h)
            allh = g["ag"].all_gather(g["stage"]).view(torch.bfloat16).view(w * cap, hid)
        if self.mx:
            from ..models.transformer import expert_gate_up_mx
            tn = 32
            if moe.can_prep(allh, lw.router, k):
                ids, wts, pl, xq = moe.prep_hidden(allh, lw.router, k, self.e_local, tn, **rt)
            else:
                ids, wts, pl = moe.route_plan_hidden(allh, lw.router, k, self.e_local, tn, **rt)
                xq = ew.mx_quantize(allh, pl.row_token, sf_layout=tn)
            if moe.can_fuse_ffn(xq, lw.w13, lw.w2, self.e_local, pl.capacity):
                # gate/up, down, the router-weighted sums and their scatter to the tokens' home GPUs: one launch, one flag round
                sc = dict(weights=wts, n_tok=w * cap, k=k, tokens_per_rank=cap, slots=g["slot_ptrs"], flags=g["flag_ptrs"], world=w,
                          epoch=g["epoch"]) if FOLD_COMBINE else None
                y = moe.expert_ffn_fused(xq, lw.w13, lw.w2, self.e_local, pl, scatter=sc)
                if sc is not None:
                    self.stats["fold_combine"] += 1
                    return PendingSlots(g, t)
            else:
                hq = torch.empty(pl.capacity, inter, dtype=torch.uint8, device=h.device)
                hsf = ew.sf_alloc(pl.capacity, inter, h.device, tn, init=False)
                expert_gate_up_mx(xq.data, xq.sf, lw.w13, self.e_local, pl.seg_start, pl.seg_count, tn, hq, hsf, pl.row_token)
                from ..models.transformer import PAIR_DOWN
                y = gemm.grouped_linear(hq, lw.w2.mx.data.view(self.e_local, hid, inter), pl.seg_start, pl.seg_count, tn, sfa=lw.w2.mx.sf,
                                        sfb=hsf, w_tiled=lw.w2.mx.tiled, pair_rows=PAIR_DOWN)
        else:
            tn = gemm.pick_tn(max(1, (w * cap * k + cfg.n_experts - 1) // cfg.n_experts), dual=True)
            if moe.can_prep(allh, lw.router, k):
                ids, wts, pl, xs = moe.prep_hidden(allh, lw.router, k, self.e_local, tn, quantize=False, **rt)
            else:
                ids, wts, pl = moe.route_plan_hidden(allh, lw.router, k, self.e_local, tn, **rt)
                xs = moe.gather_rows(allh, pl.row_token)
            act = gemm.grouped_linear(xs, lw.w13.w.view(self.e_local, 2 * inter, hid), pl.seg_start, pl.seg_count, tn, dual=True, w_tiled=lw.w13.tiled)
            y = gemm.grouped_linear(act, lw.w2.w.view(self.e_local, hid, inter), pl.seg_start, pl.seg_count, tn, w_tiled=lw.w2.tiled)
        rc = f.lib.gb_moe_combine_scatter(_c(y.data_ptr()), _c(pl.pair_row.data_ptr()), _c(wts.data_ptr()), _i(w * cap), _i(hid), _i(k),
                                          _i(y.stride(0)), _i(cap), g["slot_ptrs"], g["flag_ptrs"], _i(w), _c(g["epoch"]), _c(g["done"]),
                                          _c(torch.cuda.current_stream().cuda_stream))
        _native.check(rc, "gb_moe_combine_scatter")
        return PendingSlots(g, t)

    def moe_ffn(self, model, lw, h: torch.Tensor, h_mx=None) -> torch.Tensor:
        if not self.fused:
            return self._moe_nccl(model, lw, h)
        if h.shape[0] <= min(self.gather_max, self.max_tokens) and self.use_gather:
            return self._moe_gather(model, lw, h)
        cfg, w, f = self.cfg, self.ep_size, self.fab
        t = h.shape[0]
        e, k, inter, hid = cfg.n_experts, cfg.n_experts_used, cfg.expert_ffn, cfg.hidden
        b = self._bucket(t)
        tn, rows = b["tn"], b["region_rows"]
        logits = moe.router_logits(h, lw.router)
        ids, wts = moe.route(logits, k, cfg.router, lw.router_bias, cfg.norm_topk, cfg.routed_scale)
        pl = moe.plan(ids, e, tn, regions=w, epoch_ctr=self.epoch, region_rows=rows)
        stream = _c(torch.cuda.current_stream().cuda_stream)
        if self.mx and h_mx is not None and h_mx.data.is_cuda and DISPATCH_MX:
            # the tokens are already MXFP8 (quantised by the RMSNorm in front of this block): the dispatch copies bytes and scales
            rc = f.lib.gb_ep_dispatch_mx(f.bases_arr, _i(w), _i(self.ep_rank), _c(h_mx.data.data_ptr()), _c(h_mx.sf.data_ptr()),
                                         _i(1 if h_mx.sf_layout == 32 else 0), _i(hid), _c(pl.row_token.data_ptr()), _c(pl.seg_start.data_ptr()),
                                         _c(pl.seg_count.data_ptr()), _i(rows), _i(self.e_local), _sz(self.x_off), _sz(self.sf_off),
                                         _sz(self.meta_off), _sz(self.flags_d), _i(1 if tn == 32 else 0), _c(self.epoch), _c(self.done_d),
                                         _c(_native.status_ptr()), stream)
            _native.check(rc, "gb_ep_dispatch_mx")
        else:
            rc = f.lib.gb_ep_dispatch(f.bases_arr, _i(w), _i(self.ep_rank), _c(h.data_ptr()), _i(h.stride(0)), _i(hid), _c(pl.row_token.data_ptr()),
                                      _c(pl.seg_start.data_ptr()), _c(pl.seg_count.data_ptr()), _i(rows), _i(self.e_local), _sz(self.x_off),
                                      _sz(self.sf_off), _sz(self.meta_off), _sz(self.flags_d), _i(1 if self.mx else 0), _i(1 if tn == 32 else 0),
                                      _c(self.epoch), _c(self.done_d), _c(_native.status_ptr()), stream)
            _native.check(rc, "gb_ep_dispatch")
        seg_start, seg_count = self.meta[0], self.meta[1]
        if self.mx:
            from ..models.transformer import expert_gate_up_mx
            if tn != 32 and "gu" not in b:
                b["gu"] = torch.empty(b["total"], 2 * inter, dtype=torch.bfloat16, device=self.device)
            expert_gate_up_mx(b["x"], b["sf"], lw.w13, self.e_local, seg_start, seg_count, tn, b["hq"], b["hsf"], None, extras=b["ex1"],
                              w_groups=b["groups"], scratch=b.get("gu"))
            gemm.grouped_linear(b["hq"], lw.w2.mx.data.view(self.e_local, hid, inter), seg_start, seg_count, tn, out=b["y"],
                                sfa=lw.w2.mx.sf, sfb=b["hsf"], extras=b["ex2"], w_groups=b["groups"], w_tiled=lw.w2.mx.tiled)
        else:
            gemm.grouped_linear(b["x"], lw.w13.w.view(self.e_local, 2 * inter, hid), seg_start, seg_count, tn, out=b["act"], dual=True,
                                extras=b["ex1"], w_groups=b["groups"], w_tiled=lw.w13.tiled)
            gemm.grouped_linear(b["act"], lw.w2.w.view(self.e_local, hid, inter), seg_start, seg_count, tn, out=b["y"], extras=b["ex2"],
                                w_groups=b["groups"], w_tiled=lw.w2.tiled)
        return moe.PendingCombine(b["y"], pl.pair_row, wts, t, k, wait_flags=f.local_base + self.flags_c, wait_n=w, epoch_ptr=self.epoch)

    # ------------------------------------------------------------------------------------------ NCCL-only baseline
    def _moe_nccl(self, model, lw, h: torch.Tensor) -> torch.Tensor:
        cfg, w = self.cfg, self.ep_size
        t, hid = h.shape
        k, e = cfg.n_experts_used, cfg.n_experts
        e_local = e // w
        allh = torch.empty(w * t, hid, dtype=h.dtype, device=h.device)
        if h.is_cuda:
            dist.all_gather_into_tensor(allh, h.contiguous(), group=self.group)
        else:                                   # gloo (CPU ranks in the tests) has no tensor all-gather / reduce-scatter
            parts = [torch.empty_like(h) for _ in range(w)]
            dist.all_gather(parts, h.contiguous(), group=self.group)
            allh = torch.cat(parts)
        logits = moe.router_logits(allh, lw.router)
        ids, wts = moe.route(logits, k, cfg.router, lw.router_bias, cfg.norm_topk, cfg.routed_scale)
        local = ids - self.ep_rank * e_local
        local = torch.where((local >= 0) & (local < e_local), local, torch.full_like(local, -1))
        inter = cfg.expert_ffn
        tn = 32 if (w * t * k) // e <= 24 else 128
        pl = moe.plan(local, e_local, tn)
        if model.mx:
            xq = ew.mx_quantize(allh, pl.row_token, sf_layout=tn)
            hq = torch.empty(pl.capacity, inter, dtype=torch.uint8, device=h.device)
            hsf = ew.sf_alloc(pl.capacity, inter, h.device, tn, init=False)
            from ..models.transformer import expert_gate_up_mx
            expert_gate_up_mx(xq.data, xq.sf, lw.w13, e_local, pl.seg_start, pl.seg_count, tn, hq, hsf, pl.row_token)
            y = gemm.grouped_linear(hq, lw.w2.mx.data.view(e_local, hid, inter), pl.seg_start, pl.seg_count, tn, sfa=lw.w2.mx.sf, sfb=hsf,
                                    w_tiled=lw.w2.mx.tiled)
        else:
            xs = moe.gather_rows(allh, pl.row_token)
            act = gemm.grouped_linear(xs, lw.w13.w.view(e_local, 2 * inter, hid), pl.seg_start, pl.seg_count, tn, dual=True, w_tiled=lw.w13.tiled)
            y = gemm.grouped_linear(act, lw.w2.w.view(e_local, hid, inter), pl.seg_start, pl.seg_count, tn, w_tiled=lw.w2.tiled)
        part = moe.combine(y, pl.pair_row, wts, w * t, k).float()
        if not h.is_cuda:
            dist.all_reduce(part, group=self.group)
            return part[self.ep_rank * t:(self.ep_rank + 1) * t].to(torch.bfloat16)
        out = torch.empty(t, hid, dtype=torch.float32, device=h.device)
        dist.reduce_scatter_tensor(out, part, group=self.group)
        return out.to(torch.bfloat16)

    def close(self) -> None:
        if self.fab is not None:
            self.fab.close()
