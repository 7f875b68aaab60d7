"""Tensor parallelism (Megatron style) with the reduction fused into the kernels around it.

Weights are cut at load time: q/k/v/gate/up by rows (column parallel), o_proj/down_proj by columns (row parallel); KV heads
are sharded, or replicated when there are fewer KV heads than ranks.  The reference does this between CPU ranks with an
all-reduce of ``n_embd`` floats after o_proj and after ffn_down (common/transformer.h:4178-4283,
cpu/llm/test_transformer_parallel.c:431-525).  Here, for decode-sized batches, there is no all-reduce kernel at all:

  row-parallel GEMM epilogue  --stores fp32 partial rows into this rank's slot on EVERY GPU, then raises a flag-->
  next RMSNorm kernel         --waits for all ranks' flags, sums the slots in rank order, adds the residual, normalises
                                (and quantises to MXFP8 for the next GEMM)

so the collective costs one NVLink store per output element and no extra launch; sums are bit-identical on all ranks,
which keeps greedy decoding in lock step without broadcasting tokens.  Large (prefill) batches use the two-shot
reduce-scatter + all-gather kernel of the fabric.  ``fused=False`` is the NCCL baseline.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native
from ..ops import elementwise as ew
from ..ops import gemm
from ..ops.mxfp8 import MxTensor
from .fabric import Fabric

_c, _i, _f, _l = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_long


TP_DIRECT = os.environ.get("GB_TP_DIRECT", "1") != "0"
# prefill-sized row-parallel projections: GEMM -> reduce-scatter in the epilogue, all-gather -> GEMM in the consumer's prologue.
# GB_TP_SEQ_PAR = 1 / 0 forces it on / off; by default it is on up to 4 ranks: measured on Qwen3-8B bf16, 32 x 1024 prefill tokens/s
# against the two-shot all-reduce kernel: 2 GPUs 97.4k vs 91.8k, 4 GPUs 137.5k vs 128.7k, 8 GPUs 142.6k vs 155.8k (with 8 ranks a
# rank's GEMM is short and 7/8 of its result leaves through 64-byte epilogue stores, which then bound it).
_SEQ_PAR_ENV = os.environ.get("GB_TP_SEQ_PAR", "auto")


def _seq_par_on(world: int) -> bool:
    return _SEQ_PAR_ENV == "1" or (_SEQ_PAR_ENV != "0" and world <= 4)


@dataclass
class PendingReduce:
    """Partial sums of a row-parallel projection sitting in the slots of channel ``chan``; finished by ``add_norm``."""
    chan: int
    rows: int
    hidden: int
    splits: int = 1          # K-split slabs per rank inside its slot


@dataclass
class PendingScatter:
    """Partial sums of a prefill-sized row-parallel projection, reduce-scattered by the GEMM's epilogue: rows ``[p * region, (p + 1) *
    region)`` of every rank's partial result sit in GPU p's slots of channel ``chan``; finished by ``add_norm`` on the owner."""
    chan: int
    rows: int
    hidden: int
    region: int


class TensorParallel:
    """``ep_experts=True`` is the hybrid layout of the large MoE models (the reference runs the same N ranks as a tensor-parallel
    group for attention and as an expert-parallel group for the experts: common/glm5.h:178-202, common/m3_impl.h:653-660,
    716-722): attention and the dense projections are cut as above and every rank sees every token, each rank holds
    ``E / N`` whole experts, evaluates them on the rows routed to them, and the ranks' router-weighted sums are added by the
    same slot reduction that finishes a row-parallel projection.  No token exchange is needed in front of the experts.
    Build the weights with ``tp_rank / tp_size`` AND ``ep_rank = tp_rank, ep_size = tp_size``."""
    ep_size = 1
    ep_rank = 0

    def __init__(self, group, device: torch.device, fused: bool = True, max_fused_rows: int = 256, ep_experts: bool = False):
        self.group, self.device, self.fused = group, device, fused
        self.tp_size = dist.get_world_size(group)
        self.tp_rank = dist.get_rank(group)
        self.ep_experts = ep_experts
        if ep_experts:
            self.ep_size, self.ep_rank = self.tp_size, self.tp_rank
        self.max_fused_rows = max_fused_rows
        self.fab: Optional[Fabric] = None
        self._chan = 0
        self._sp_chan = 0
        self._x_sharded, self._x_region = False, 0
        self.sp = None
        self.sp_launches = 0        # row-parallel GEMMs that took the fused reduce-scatter path (tests assert on it)
        self._sp_ok = True          # cleared by the model for forward passes that read the whole residual stream between layers

    def attach(self, engine, cfg, max_tokens: int) -> None:
        self.cfg = cfg
        if not self.fused:
            return
        w, h = self.tp_size, cfg.hidden
        slot = self.max_fused_rows * h * 4
        big = max_tokens * h
        heap = 2 * w * slot + 2 * big * 2 + (8 << 20)
        if _seq_par_on(w) and w > 1 and max_tokens >= w * 256:
            heap += self.seq_par_heap_bytes(w, h, max_tokens)
        self.fab = f = Fabric(self.group, self.device, heap)
        self.slot_elems = self.max_fused_rows * h
        self.slots_off = [f.alloc(w * slot), f.alloc(w * slot)]
        self.flags_off = [f.alloc(32), f.alloc(32)]
        self.epoch = [f.ctl_word(), f.ctl_word()]
        self.done = [f.ctl_word(), f.ctl_word()]
        self.big = f.make_allreduce_large(big, torch.bfloat16)
        self.argmax = f.make_argmax(4096)
        self._attach_seq_par(f, cfg, max_tokens)
        self._extras = []
        for ch in range(2):
            ex = gemm.GemmExtras()
            ex.epoch_ptr = self.epoch[ch]
            ex.epoch_self_tick = 1
            ex.peer_bcast = w
            for p in range(w):
                ex.peer_out[p] = f.peer_ptr(p, self.slots_off[ch]) + self.tp_rank * slot
                ex.signal_flags[p] = f.peer_ptr(p, self.flags_off[ch]) + 4 * self.tp_rank
            ex.signal_n = w
            ex.done_ctr = self.done[ch]
            self._extras.append(ex)

    # ------------------------------------------------------------------------------------------ prefill: GEMM -> reduce-scatter, all-gather -> GEMM
    def _attach_seq_par(self, f: Fabric, cfg, max_tokens: int) -> None:
        """Buffers of the fused prefill path.  A row-parallel GEMM (o_proj, down_proj) stores the rows of region p of its partial
        result (as bf16) straight into slot [this rank] on GPU p (its epilogue is the reduce-scatter, tile by tile under the math) and raises a
        flag there; GPU p's residual-add + RMSNorm kernel waits for all flags, sums the slots in rank order, updates ITS rows of
        the residual stream, and stores the normalised bf16 rows into the gather buffer of every GPU (its epilogue is the
        all-gather); the next column-parallel GEMM (QKV, gate/up) waits for all ranks' gather flags before it loads its token
        tiles.  Between the two GEMMs the residual stream is sharded by rows (sequence parallelism): per layer two exchanges of
        rows / W rows instead of two all-reduces of all rows, no all-reduce launch, and the norm is computed once, not W times."""
        self.sp = None
        w, h = self.tp_size, cfg.hidden
        if not (_seq_par_on(w) and w > 1 and max_tokens >= w * 256):
            return
        region_max = -(-max_tokens // (w * 256)) * 256
        sp = {"region_max": region_max}
        sp["slots_off"] = [f.alloc(w * region_max * h * 2) for _ in range(2)]
        sp["gather_off"] = [f.alloc(w * region_max * h * 2) for _ in range(2)]
        sp["rs_flags"] = [f.alloc(32) for _ in range(2)]
        sp["ag_flags"] = [f.alloc(32) for _ in range(2)]
        sp["rs_epoch"], sp["rs_done"] = [f.ctl_word(), f.ctl_word()], [f.ctl_word(), f.ctl_word()]
        sp["ag_epoch"], sp["ag_done"] = [f.ctl_word(), f.ctl_word()], [f.ctl_word(), f.ctl_word()]
        self.sp = sp

    @staticmethod
    def seq_par_heap_bytes(world: int, hidden: int, max_tokens: int) -> int:
        region_max = -(-max_tokens // (world * 256)) * 256
        return 2 * world * region_max * hidden * (2 + 2) + (1 << 20)

    def _scatter_linear(self, lw, x: torch.Tensor, rows: int):
        """Row-parallel bf16 projection whose epilogue reduce-scatters (see ``_attach_seq_par``)."""
        sp, f, w = self.sp, self.fab, self.tp_size
        ch = self._sp_chan
        self._sp_chan ^= 1
        self.sp_launches += 1
        n = lw.n
        region = -(-rows // (w * 256)) * 256
        ex = gemm.GemmExtras()
        for p in range(w):
            ex.peer_out[p] = f.peer_ptr(p, sp["slots_off"][ch])
            ex.signal_flags[p] = f.peer_ptr(p, sp["rs_flags"][ch]) + 4 * self.tp_rank
        ex.peer_region_rows, ex.peer_rank, ex.signal_n = region, self.tp_rank, w
        ex.done_ctr, ex.epoch_ptr, ex.epoch_self_tick = sp["rs_done"][ch], sp["rs_epoch"][ch], 1
        tn = gemm.pick_tn(rows)
        # the partial rows travel as bf16 (the precision of the all-reduce they replace, half the link bytes of fp32)
        gemm._launch(lw.w, x, None, n, lw.k, rows, lw.w.stride(0), x.stride(0), n, gemm.GEMM_W_TILED if lw.tiled else 0, tn,
                     bias=lw.bias if self.tp_rank == 0 else None, extras=ex)
        return PendingScatter(ch, rows, n, region)

    def _scatter_norm(self, ps: PendingScatter, weight, eps, residual: torch.Tensor):
        """Owner side of the reduce-scatter + the all-gather of the normalised rows; returns the gathered rows (a view of the heap).
        The consumer GEMM that follows waits for the gather flags (``gemm.wait_before_next_launch``)."""
        sp, f, w, ch = self.sp, self.fab, self.tp_size, ps.chan
        h, region = ps.hidden, ps.region
        r0 = self.tp_rank * region
        mine = max(0, min(ps.rows, r0 + region) - r0)
        bc = ew.RmsBcast()
        for p in range(w):
            bc.out[p] = f.peer_ptr(p, sp["gather_off"][ch]) + r0 * h * 2
            bc.flag[p] = f.peer_ptr(p, sp["ag_flags"][ch]) + 4 * self.tp_rank
        bc.world, bc.epoch_ctr, bc.done_ctr, bc.partials_bf16 = w, sp["ag_epoch"][ch], sp["ag_done"][ch], 1
        stream = _c(torch.cuda.current_stream().cuda_stream)
        if mine > 0:
            res = residual[r0: r0 + mine]
            assert res.is_contiguous() and residual.stride(0) == h
            rc = f.lib.gb_rmsnorm_reduce_bcast(_c(res.data_ptr()), _c(f.local_base + sp["slots_off"][ch]), _i(w), _l(region * h), _c(weight.data_ptr()),
                                               _c(0), _c(0), _c(0), _i(mine), _i(h), _f(eps), _i(0), _c(f.local_base + sp["rs_flags"][ch]), _i(w),
                                               _c(sp["rs_epoch"][ch]), _c(_native.status_ptr()), ctypes.byref(bc), stream)
            _native.check(rc, "gb_rmsnorm_reduce_bcast")
        else:
            _native.check(f.lib.gb_bcast_signal(ctypes.byref(bc), stream), "gb_bcast_signal")
        gemm.wait_before_next_launch(f.local_base + sp["ag_flags"][ch], w, sp["ag_epoch"][ch])
        return f.view(sp["gather_off"][ch], (ps.rows, h), torch.bfloat16)

    def finish_residual(self, x: torch.Tensor, delta) -> None:
        """Before the residual stream is read as a whole (final norm, snapshots): while the fused prefill path is in use every rank
        keeps only its own rows of ``x`` current; gather the others (once per forward pass, NCCL)."""
        if not isinstance(delta, PendingScatter) and not self._x_sharded:
            return
        region = self._x_region
        w, rows = self.tp_size, x.shape[0]
        pad = torch.zeros(w * region, x.shape[1], dtype=x.dtype, device=x.device)
        r0 = self.tp_rank * region
        mine = max(0, min(rows, r0 + region) - r0)
        part = torch.zeros(region, x.shape[1], dtype=x.dtype, device=x.device)
        part[:mine] = x[r0: r0 + mine]
        dist.all_gather_into_tensor(pad, part, group=self.group)
        x.copy_(pad[:rows])
        self._x_sharded = False

    # ------------------------------------------------------------------------------------------ model hooks
    def tp_all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_size == 1:
            return x
        if not self.fused:
            dist.all_reduce(x, group=self.group)
            return x
        return self.big(x.contiguous())

    def row_linear(self, lw, x, x_mx: Optional[MxTensor] = None):
        from ..models.transformer import apply_linear
        rows = x.shape[0] if x is not None else x_mx.rows
        if lw.is_quant:
            return self._row_linear_quant(lw, x, rows)
        if not self.fused or self.tp_size == 1 or rows > self.max_fused_rows:
            if (self.fused and self.tp_size > 1 and self.sp is not None and lw.fmt == "bf16" and x is not None and x.is_cuda and lw.n == self.cfg.hidden
                    and rows >= self.tp_size * 256 and -(-rows // (self.tp_size * 256)) * 256 <= self.sp["region_max"] and self._sp_ok):
                return self._scatter_linear(lw, x, rows)
            if TP_DIRECT and self.fused and self.tp_size > 1 and rows * lw.n <= self.big.n and (x if x is not None else x_mx.data).is_cuda:
                # prefill-sized: the GEMM writes its partial result straight into the all-reduce's input buffer in the fabric heap
                out = self.big.input_view[: rows * lw.n].view(rows, lw.n)
                if lw.fmt == "bf16":
                    gemm.linear(x, lw.w, bias=lw.bias, out=out, w_tiled=lw.tiled)
                else:
                    xm = x_mx if x_mx is not None else ew.mx_quantize(x, sf_layout=32 if rows <= 32 else 128)
                    gemm.linear_mx(xm, lw.mx, out=out, bias=lw.bias)
                return self.big(out)
            return self.tp_all_reduce(apply_linear(lw, x, x_mx))
        ch = self._chan
        self._chan ^= 1
        n, k = lw.n, lw.k
        ex = self._extras[ch]
        # decode-sized batches: the shard's K range is cut further, every split stores its own slab inside this rank's slot
        sp = gemm.pick_partials(n, rows, k, lw.fmt != "bf16") if n % 128 == 0 else 1
        # every slab goes to every GPU (fp32): keep what one rank sends per projection near 4 MB, or the K splits cost more link
        # time than they save in the GEMM (8 GPUs, 32 rows x 4096: 0.5 MB per peer and slab)
        while sp > 1 and (sp * rows * n > self.slot_elems or sp * rows * n * 4 * (self.tp_size - 1) > (4 << 20)):
            sp -= 1
        kb = k // (64 if lw.fmt == "bf16" else 128)
        if sp > 1 and -(-kb // -(-kb // sp)) != sp:
            sp = 1
        ex.splits, ex.partial_stride = (sp, rows * n) if sp > 1 else (0, 0)
        if lw.fmt == "bf16":
            tn = gemm.pick_tn(rows)
            gemm._launch(lw.w, x, None, n, k, rows, lw.w.stride(0), x.stride(0), n, gemm.GEMM_OUT_F32 | (gemm.GEMM_W_TILED if lw.tiled else 0), tn, bias=None,
                         extras=ex)
        else:
            xm = x_mx if x_mx is not None else ew.mx_quantize(x, sf_layout=32 if rows <= 32 else 128)
            gemm._launch(lw.mx.data, xm.data, None, n, k, rows, k, k, n, gemm.GEMM_MX | gemm.GEMM_OUT_F32 | (gemm.GEMM_W_TILED if lw.mx.tiled else 0), xm.sf_layout,
                         x_rows=xm.data.shape[0], sfa=lw.mx.sf, sfb=xm.sf, extras=ex)
        return PendingReduce(ch, rows, n, max(sp, 1))

    def _row_linear_quant(self, lw, x: torch.Tensor, rows: int):
        """Row-parallel projection over ggml blocks.  Up to four tokens: the fused dequant-GEMV stores its fp32 partial sums
        straight into this rank's slot on every GPU and raises the arrival flags (the one-shot all-reduce is the GEMV's tail,
        the sum happens in the RMSNorm that follows).  Larger batches: dequant-GEMM, then the stand-alone all-reduce."""
        from ..ops import qlinear
        if not self.fused or self.tp_size == 1 or rows > qlinear.GEMV_MAX_TOKENS or not x.is_cuda:
            return self.tp_all_reduce(qlinear.linear(x, lw.q, bias=lw.bias if self.tp_rank == 0 else None))
        ch = self._chan
        self._chan ^= 1
        ex = self._extras[ch]
        n, k = lw.n, lw.k
        sp = qlinear.pick_splits(n, k, rows, lw.q.ggml_type)
        while sp > 1 and sp * rows * n > self.slot_elems:
            sp -= 1
        sp = max(1, _native.cuda().gb_qgemv_splits(_i(lw.q.ggml_type), _i(k), _i(rows), _i(sp)))
        if sp * rows * n > self.slot_elems:
            return self.tp_all_reduce(qlinear.linear(x, lw.q, bias=lw.bias if self.tp_rank == 0 else None))
        peer = qlinear.QGemvPeer()
        for p in range(self.tp_size):
            peer.peer_out[p] = ex.peer_out[p]
            peer.signal_flags[p] = ex.signal_flags[p]
        peer.peer_bcast, peer.signal_n = self.tp_size, self.tp_size
        peer.done_ctr, peer.epoch_ptr, peer.epoch_self_tick = ex.done_ctr, ex.epoch_ptr, 1
        qlinear.gemv_partials(x, lw.q, splits=sp, bias=lw.bias if self.tp_rank == 0 else None, peer=peer,
                              out=torch.empty(sp, 0, 0, dtype=torch.float32, device=x.device))
        return PendingReduce(ch, rows, n, sp)

    def _reduce_norm(self, pr: PendingReduce, weight, eps, residual, quantize=False, want_bf16=True, sf_layout=128):
        f = self.fab
        rows, hidden = pr.rows, pr.hidden
        out = torch.empty(rows, hidden, dtype=torch.bfloat16, device=self.device) if want_bf16 else None
        q = sf = None
        if quantize:
            rp = (rows + 127) // 128 * 128
            q = torch.empty(rp, hidden, dtype=torch.uint8, device=self.device)
            sf = ew.sf_alloc(rp, hidden, self.device, sf_layout, init=False)
        p = lambda t: _c(t.data_ptr()) if t is not None else _c(0)
        rc = f.lib.gb_rmsnorm_reduce2(p(residual), _c(f.local_base + self.slots_off[pr.chan]), _i(self.tp_size), _l(self.slot_elems),
                                      _i(pr.splits), _l(rows * hidden), p(weight),
                                      p(out), p(q), p(sf), _i(rows), _i(hidden), _f(eps), _i(1 if sf_layout == 32 else 0),
                                      _c(f.local_base + self.flags_off[pr.chan]), _i(self.tp_size), _c(self.epoch[pr.chan]),
                                      _c(_native.status_ptr()), _c(torch.cuda.current_stream().cuda_stream))
        _native.check(rc, "gb_rmsnorm_reduce2")
        if quantize:
            return out, MxTensor(q, sf, rows, hidden, sf_layout)
        return out

    def add_norm(self, delta, weight, eps, residual, **kw):
        if isinstance(delta, PendingReduce):
            return self._reduce_norm(delta, weight, eps, residual, **kw)
        if isinstance(delta, PendingScatter):
            if kw.get("quantize") or residual is None:
                raise RuntimeError("the fused prefill path serves bf16 models with a residual stream")
            self._x_sharded, self._x_region = True, delta.region
            return self._scatter_norm(delta, weight, eps, residual)
        return ew.rmsnorm(delta, weight, eps, residual=residual, **kw)

    def materialize(self, delta):
        """Finish a pending reduction into a plain tensor (sum of the ranks' partials, bf16)."""
        if isinstance(delta, PendingScatter):
            # every rank sums its own region of the slots, the regions are gathered (end of a forward pass: once, NCCL)
            f, sp, w, h = self.fab, self.sp, self.tp_size, delta.hidden
            f.barrier()          # every rank's GEMM (and its stores) precede its arrival at the barrier
            slots = f.view(sp["slots_off"][delta.chan], (w, delta.region * h), torch.bfloat16)
            part = slots.float().sum(0).to(torch.bfloat16).view(delta.region, h)
            full = torch.empty(w * delta.region, h, dtype=torch.bfloat16, device=self.device)
            dist.all_gather_into_tensor(full, part.contiguous(), group=self.group)
            return full[: delta.rows]
        if not isinstance(delta, PendingReduce):
            return delta.materialize() if hasattr(delta, "materialize") else delta
        f = self.fab
        slots = f.view(self.slots_off[delta.chan], (self.tp_size, self.slot_elems), torch.float32)
        # order the read after the peers' stores: a fabric barrier (device side) covers the flags of this channel
        f.barrier()
        n = delta.rows * delta.hidden
        return slots[:, : delta.splits * n].reshape(self.tp_size * delta.splits, n).sum(0).reshape(delta.rows, delta.hidden).to(torch.bfloat16)

    def moe_ffn(self, model, lw, h, h_mx=None):
        if not self.ep_experts or self.tp_size == 1:
            return None                  # experts replicated: the model evaluates all of them locally
        e_l = self.cfg.n_experts // self.ep_size
        pc = model.moe_local(lw, h, h_mx, local_range=(self.ep_rank * e_l, e_l))
        rows, hid = h.shape[0], self.cfg.hidden
        if not (self.fused and h.is_cuda and rows <= self.max_fused_rows):
            return self.tp_all_reduce(pc.materialize())
        # decode-sized: this rank's router-weighted partial sums go into its slot on every GPU; the next RMSNorm adds the slots
        ch = self._chan
        self._chan ^= 1
        ex, w = self._extras[ch], self.tp_size
        slots = (ctypes.c_void_p * w)(*[ex.peer_out[p] for p in range(w)])
        flags = (ctypes.c_void_p * w)(*[ex.signal_flags[p] for p in range(w)])
        rc = self.fab.lib.gb_moe_combine_scatter(_c(pc.y.data_ptr()), _c(pc.pair_row.data_ptr()), _c(pc.weights.data_ptr()), _i(rows), _i(hid),
                                                 _i(pc.k), _i(pc.y.stride(0)), _i(0), slots, flags, _i(w), _c(self.epoch[ch]), _c(self.done[ch]),
                                                 _c(torch.cuda.current_stream().cuda_stream))
        _native.check(rc, "gb_moe_combine_scatter")
        return PendingReduce(ch, rows, hid, 1)

    def merge_sampled(self, tok: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        """Greedy merge for a vocabulary-sharded LM head: arg-max all-reduce of this shard's (value, index)."""
        if self.tp_size == 1 or logits.shape[1] == self.cfg.vocab:
            return tok
        val = logits.gather(1, (tok.long() - self._vocab_start).clamp_min(0).unsqueeze(1)).squeeze(1).contiguous()
        if self.fused:
            idx, _ = self.argmax(val, tok.contiguous())
            return idx
        vals = [torch.empty_like(val) for _ in range(self.tp_size)]
        toks = [torch.empty_like(tok) for _ in range(self.tp_size)]
        dist.all_gather(vals, val, group=self.group)
        dist.all_gather(toks, tok, group=self.group)
        v, t = torch.stack(vals), torch.stack(toks)
        best = v.max(0).values
        cand = torch.where(v == best, t, torch.full_like(t, 2 ** 31 - 1))
        return cand.min(0).values

    _vocab_start = 0

    def close(self) -> None:
        if self.fab is not None:
            self.fab.close()
