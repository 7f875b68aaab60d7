"""Decoder-only transformer (Qwen2 / Qwen3 dense and Qwen3-MoE) over a paged KV cache.

One ``forward`` serves prefill chunks, decode steps and mixed batches: tokens of all sequences are packed
into ``[T, hidden]`` rows, attention works from per-sequence metadata (``ForwardBatch``).  Every op is a
hand-written sm_100a kernel from ``gemm_b200.ops`` when the tensors are on a GPU; on CPU tensors the same
call sequence runs the PyTorch references, which is how the layer logic is tested without a GPU.

Layer recipe (reference: common/transformer.h:3550-4174):
  h = RMSNorm(x); qkv = h Wqkv^T (+bias); per-head QK-RMSNorm; NeoX RoPE; K/V -> paged cache;
  a = causal GQA attention; x += a Wo^T  [tensor-parallel: all-reduce]
  h = RMSNorm(x); dense: x += (SiLU(h Wg^T) * h Wu^T) Wd^T  [TP all-reduce]
                  MoE  : softmax router -> top-k -> renormalise; x += sum_k w_k FFN_k(h)  [EP dispatch / combine]
  logits = RMSNorm(x) Whead^T on the last token of every sequence.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .. import _native
from ..ops import attention as att
from ..ops import elementwise as ew
from ..ops import deltanet as dn
from ..ops import gemm, moe, qlinear, sampling
from ..ops.mxfp8 import MxTensor
from .config import ModelConfig
from .weights import LinearWeight, ModelWeights
from ..utils import profiler


@dataclass
class KvCache:
    """Paged KV storage: per layer ``k`` and ``v`` of shape ``[num_pages * page_size, Hkv_local, D]`` (bf16)."""
    k: List[torch.Tensor]
    v: List[torch.Tensor]
    page_size: int
    num_pages: int
    # Delta-Net layers of the hybrid models keep a fixed-size state per sequence slot instead of K/V pages:
    # conv[l] f32 [slots, conv_k - 1, qkv_dim], rec[l] f32 [slots, heads_v, d, d] (None for attention layers)
    conv: Optional[List[Optional[torch.Tensor]]] = None
    rec: Optional[List[Optional[torch.Tensor]]] = None
    # INT8 mode (``kv_dtype="int8"``): the pages live in ``kq`` / ``vq`` (int8 ``[slots, Hkv, D]``) with one f32 scale per slot and
    # head in ``ks`` / ``vs`` (the format of ops.attention.kv_store_q8), read directly by the INT8 decode attention kernel.  ``k`` /
    # ``v`` then name ONE bf16 staging buffer shared by all layers: the QK-norm + RoPE kernel writes a step's new rows there, the
    # prefill attention of a layer reads them there, and the store kernel quantises them into the layer's pages.
    kq: Optional[List[torch.Tensor]] = None
    vq: Optional[List[torch.Tensor]] = None
    ks: Optional[List[torch.Tensor]] = None
    vs: Optional[List[torch.Tensor]] = None

    @property
    def quantized(self) -> bool:
        return self.kq is not None

    @staticmethod
    def allocate(cfg: ModelConfig, num_pages: int, page_size: int, device, hkv_local: Optional[int] = None,
                 n_layers: Optional[int] = None, n_seq_slots: int = 64, first_layer: int = 0, kv_dtype: str = "bf16",
                 stage_pages: int = 0) -> "KvCache":
        """``kv_dtype="int8"`` keeps the pages as int8 + scales; ``stage_pages`` pages of bf16 staging (enough for the tokens of one
        forward pass, every sequence starting on a page boundary) are shared by all layers."""
        hkv = hkv_local if hkv_local is not None else cfg.n_kv_heads
        nl = n_layers if n_layers is not None else cfg.n_layers
        shape = (num_pages * page_size, hkv, cfg.head_dim)
        ssm = [cfg.is_ssm_layer(first_layer + i) for i in range(nl)]
        none = (0, hkv, cfg.head_dim)
        if kv_dtype == "int8":
            if any(ssm) or cfg.head_dim != 128:
                raise ValueError("the INT8 KV cache is built for attention-only models with head_dim 128")
            stage = (max(stage_pages, 1) * page_size, hkv, cfg.head_dim)
            sk = torch.zeros(stage, dtype=torch.bfloat16, device=device)
            sv = torch.zeros(stage, dtype=torch.bfloat16, device=device)
            kv = KvCache([sk] * nl, [sv] * nl, page_size, num_pages)
            kv.kq = [torch.zeros(shape, dtype=torch.int8, device=device) for _ in range(nl)]
            kv.vq = [torch.zeros(shape, dtype=torch.int8, device=device) for _ in range(nl)]
            kv.ks = [torch.zeros(shape[:2], dtype=torch.float32, device=device) for _ in range(nl)]
            kv.vs = [torch.zeros(shape[:2], dtype=torch.float32, device=device) for _ in range(nl)]
            return kv
        if kv_dtype != "bf16":
            raise ValueError(f"unknown kv_dtype {kv_dtype!r}")
        kv = KvCache([torch.zeros(none if ssm[i] else shape, dtype=torch.bfloat16, device=device) for i in range(nl)],
                     [torch.zeros(none if ssm[i] else shape, dtype=torch.bfloat16, device=device) for i in range(nl)], page_size, num_pages)
        if any(ssm):
            kv.conv = [torch.zeros(n_seq_slots, cfg.ssm_d_conv - 1, cfg.ssm_qkv_dim, dtype=torch.float32, device=device) if ssm[i] else None
                       for i in range(nl)]
            kv.rec = [torch.zeros(n_seq_slots, cfg.ssm_n_heads_v, cfg.ssm_head_dim, cfg.ssm_head_dim, dtype=torch.float32, device=device)
                      if ssm[i] else None for i in range(nl)]
        return kv

    def reset_slots(self, slots) -> None:
        """Zero the recurrent state of the given sequence slots (a new sequence starts from an empty state)."""
        if self.conv is None:
            return
        idx = torch.as_tensor(list(slots), dtype=torch.long, device=self.k[0].device)
        for c, r in zip(self.conv, self.rec):
            if c is not None:
                c[idx] = 0
                r[idx] = 0

    def copy_pages(self, pairs) -> None:
        """``page dst <- page src`` for every ``(src, dst)`` of ``pairs`` in every layer's K and V: the copy-on-write step of a
        forked sequence (``serve.scheduler.KvBlockManager.fork`` names the tail page to copy)."""
        pairs = [p for p in pairs if p is not None]
        if not pairs:
            return
        dev = self.k[0].device
        src = torch.tensor([p[0] for p in pairs], dtype=torch.int32, device=dev)
        dst = torch.tensor([p[1] for p in pairs], dtype=torch.int32, device=dev)
        if self.quantized:
            for t in list(self.kq) + list(self.vq) + list(self.ks) + list(self.vs):
                pg = t.view(self.num_pages, self.page_size, *t.shape[1:])
                pg[dst.long()] = pg[src.long()]
            return
        for t in list(self.k) + list(self.v):
            if t.shape[0] == 0:
                continue
            if not t.is_cuda:
                pg = t.view(self.num_pages, self.page_size, *t.shape[1:])
                pg[dst.long()] = pg[src.long()]
                continue
            page_bytes = self.page_size * t.shape[1] * t.shape[2] * t.element_size()
            rc = _native.cuda().gb_kv_copy_pages(ctypes.c_void_p(t.data_ptr()), ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(dst.data_ptr()),
                                                 ctypes.c_int(len(pairs)), ctypes.c_int(self.num_pages), ctypes.c_long(page_bytes),
                                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            _native.check(rc, "gb_kv_copy_pages")

    def nbytes(self) -> int:
        if self.quantized:
            return sum(t.numel() * t.element_size() for t in list(self.kq) + list(self.vq) + list(self.ks) + list(self.vs)) + \
                2 * self.k[0].numel() * 2
        tot = sum(t.numel() * 2 for t in self.k) * 2
        if self.conv is not None:
            tot += sum(c.numel() * 4 + r.numel() * 4 for c, r in zip(self.conv, self.rec) if c is not None)
        return tot


@dataclass
class ForwardBatch:
    ids: torch.Tensor              # int32 [T]
    positions: torch.Tensor        # int32 [T]
    slots: torch.Tensor            # int32 [T] cache slot of every token (-1 = do not store)
    cu_q: torch.Tensor             # int32 [B+1]
    kv_len: torch.Tensor           # int32 [B] length including this step's tokens
    block_table: torch.Tensor      # int32 [B, max_pages]
    work: torch.Tensor             # int32 [n_work, 4] attention work list
    logit_rows: torch.Tensor       # int32/int64 [B'] rows of T whose logits are wanted
    num_splits: int = 1
    embeds: Optional[torch.Tensor] = None   # bf16 [T, H]: injected embeddings instead of ids (vision tokens)
    n_tokens: int = 0
    seq_slots: Optional[torch.Tensor] = None   # int32 [B] state slot of every sequence (Delta-Net layers); default 0..B-1
    positions3: Optional[torch.Tensor] = None  # int32 [3, T] (t, h, w) positions for M-RoPE; default: all three = positions
    is_decode: bool = False                    # every sequence contributes exactly one token (selects the decode attention kernel)
    deepstack: Optional[torch.Tensor] = None   # bf16 [n_deepstack, T, H] added to the stream after the first layers (Qwen3-VL)
    # INT8 KV cache: where a step's new K / V rows sit in the bf16 staging buffer, and (prefill) the block table of the staged sequences
    stage_slots: Optional[torch.Tensor] = None # int32 [T]
    stage_bt: Optional[torch.Tensor] = None    # int32 [B, pages]
    # context-parallel prefill: the cache slots whose K / V rows this rank contributes to the per-layer all-gather (staging order)
    cp_send_slots: Optional[torch.Tensor] = None   # int64 [p_local * page_size]

    @staticmethod
    def build(q_lens: Sequence[int], ctx_lens: Sequence[int], ids, block_table: torch.Tensor, page_size: int, hq: int, hkv: int,
              device, num_splits: int = 1, all_logits: bool = False, seq_slots: Optional[Sequence[int]] = None,
              stage: bool = False) -> "ForwardBatch":
        """Host-side assembly from per-sequence chunk lengths and the lengths already cached.  ``stage`` (INT8 KV cache) also lays the
        step's tokens out in the staging buffer: a decode step row by row, a prefill step with every sequence on a page boundary."""
        b = len(q_lens)
        pos, slots, cu = [], [], [0]
        bt = block_table.cpu()
        for s in range(b):
            for i in range(q_lens[s]):
                p = ctx_lens[s] + i
                pos.append(p)
                slots.append(int(bt[s, p // page_size]) * page_size + p % page_size)
            cu.append(cu[-1] + q_lens[s])
        t = cu[-1]
        rows = list(range(t)) if all_logits else [cu[s + 1] - 1 for s in range(b) if q_lens[s] > 0]
        i32 = dict(dtype=torch.int32, device=device)
        ids_t = ids.to(device=device, dtype=torch.int32) if torch.is_tensor(ids) else torch.tensor(ids, **i32)
        st_slots = st_bt = None
        if stage:
            if all(q == 1 for q in q_lens):
                st_slots = torch.arange(t, **i32)
            else:
                if any(c != 0 for c in ctx_lens):
                    raise NotImplementedError("INT8 KV cache: a prefill chunk must start its sequence (the attention of a later chunk "
                                              "would have to read the quantised history; raise max_prefill_tokens or use the bf16 cache)")
                pages = [(q + page_size - 1) // page_size for q in q_lens]
                first, ss = [0], []
                for s in range(b):
                    ss.extend(first[s] * page_size + i for i in range(q_lens[s]))
                    first.append(first[s] + pages[s])
                st_slots = torch.tensor(ss, **i32)
                st_bt = torch.zeros(b, max(max(pages), 1), dtype=torch.int32)
                for s in range(b):
                    st_bt[s, : pages[s]] = torch.arange(first[s], first[s] + pages[s], dtype=torch.int32)
                st_bt = st_bt.to(device)
        return ForwardBatch(stage_slots=st_slots, stage_bt=st_bt,
                            ids=ids_t, positions=torch.tensor(pos, **i32), slots=torch.tensor(slots, **i32),
                            cu_q=torch.tensor(cu, **i32), kv_len=torch.tensor([c + q for c, q in zip(ctx_lens, q_lens)], **i32),
                            block_table=block_table.to(device=device, dtype=torch.int32),
                            work=att.build_work(q_lens, hq, hkv, num_splits).to(device),
                            logit_rows=torch.tensor(rows, dtype=torch.int64, device=device), num_splits=num_splits, n_tokens=t,
                            seq_slots=torch.tensor(list(seq_slots) if seq_slots is not None else list(range(b)), **i32),
                            is_decode=(b > 0 and all(q == 1 for q in q_lens)))


# K-split partial sums for decode-sized row projections (GB_SPLIT_PROJ=0 switches them off)
SPLIT_PROJ = os.environ.get("GB_SPLIT_PROJ", "1") != "0"


FUSE_ATTN_QUANT = os.environ.get("GB_FUSE_ATTN_QUANT", "1") != "0"


PAIR_DOWN = os.environ.get("GB_PAIR_DOWN", "1") != "0"


class SingleProcess:
    """Parallel context of an unsharded model: every collective is the identity."""
    tp_size = 1
    tp_rank = 0
    ep_size = 1
    ep_rank = 0

    def tp_all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def row_linear(self, lw: "LinearWeight", x: torch.Tensor, x_mx=None):
        """Row-parallel projection (o_proj / down_proj).  Returns the residual update: a tensor, or an object that
        ``add_norm`` / ``materialize`` know how to finish (a reduction still in flight)."""
        return apply_linear_split(lw, x, x_mx)

    def add_norm(self, delta, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor], **kw):
        """``residual += delta`` (if a residual is given) followed by RMSNorm; see ``ops.elementwise.rmsnorm``."""
        return ew.rmsnorm(delta, weight, eps, residual=residual, **kw)

    def materialize(self, delta) -> torch.Tensor:
        return delta.materialize() if hasattr(delta, "materialize") else delta

    def moe_ffn(self, model: "Transformer", lw, h: torch.Tensor, h_mx=None) -> Optional[torch.Tensor]:
        return None            # None -> the model runs its local MoE path


def apply_linear(lw: LinearWeight, x: torch.Tensor, x_mx: Optional[MxTensor] = None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``x W^T (+ bias)`` in the weight's format; ``x_mx`` is an already-quantised copy of ``x`` if the caller has one."""
    if lw.is_quant:                       # ggml blocks in HBM: fused dequant-GEMV (<= 4 tokens) or dequant-GEMM
        return qlinear.linear(x, lw.q, bias=lw.bias, out_dtype=out_dtype)
    if lw.fmt == "bf16":
        return gemm.linear(x, lw.w, bias=lw.bias, out_dtype=out_dtype, w_tiled=lw.tiled)
    xm = x_mx if x_mx is not None else ew.mx_quantize(x, sf_layout=32 if x.shape[0] <= 32 else 128)
    y = gemm.linear_mx(xm, lw.mx, out_dtype=out_dtype, bias=lw.bias)
    return y


def apply_linear_split(lw: LinearWeight, x: torch.Tensor, x_mx: Optional[MxTensor] = None):
    """``apply_linear`` for a projection whose result goes into the residual stream: a decode-sized MXFP8 projection with few
    output tiles (o_proj: 16 tiles of 128 rows, 32 k-steps each) is cut along K so that it fills the GPU, and the partial sums
    are left for the residual add + RMSNorm kernel that follows."""
    if lw.is_quant:
        if x.is_cuda and x.shape[0] <= qlinear.GEMV_MAX_TOKENS:
            return qlinear.gemv_partials(x, lw.q, bias=lw.bias)      # K-split partial sums, added by the consumer
        if x.is_cuda:
            sp = qlinear.pick_gemm_splits(lw.q.rows, lw.q.k, x.shape[0])
            if sp > 1:
                return qlinear.gemm_partials(x, lw.q, sp, bias=lw.bias)
        return apply_linear(lw, x, x_mx)
    if lw.fmt == "bf16" and SPLIT_PROJ and x is not None and x.is_cuda and lw.n % 128 == 0:
        sp = gemm.pick_partials(lw.n, x.shape[0], lw.k, False)
        if sp > 1:
            return gemm.linear_partials(x, lw.w, sp, bias=lw.bias, w_tiled=lw.tiled)
        return apply_linear(lw, x, x_mx)
    if lw.fmt != "bf16" and SPLIT_PROJ:
        xm = x_mx if x_mx is not None else (ew.mx_quantize(x, sf_layout=32 if x.shape[0] <= 32 else 128) if x.is_cuda else None)
        if xm is not None and xm.data.is_cuda:
            sp = gemm.pick_partials(lw.mx.rows, xm.rows, lw.mx.k, True)
            if sp > 1:
                return gemm.linear_mx_partials(xm, lw.mx, sp, bias=lw.bias)
            return gemm.linear_mx(xm, lw.mx, bias=lw.bias)
    return apply_linear(lw, x, x_mx)


def expert_gate_up_mx(x_q: torch.Tensor, x_sf: torch.Tensor, w13: LinearWeight, n_w_groups: int, seg_start: torch.Tensor,
                      seg_count: torch.Tensor, tn: int, hq: torch.Tensor, hsf: torch.Tensor, row_valid: Optional[torch.Tensor] = None,
                      extras=None, w_groups: Optional[int] = None, scratch: Optional[torch.Tensor] = None) -> None:
    """MXFP8 expert gate/up projection + SiLU(gate) * up + re-quantisation into ``hq`` / ``hsf`` (the down projection's input).

    Decode-sized batches (token tile 32) run the two-accumulator GEMM with the activation and the quantiser in its epilogue.
    Prefill-sized batches (token tile 128) run one plain GEMM over the stacked [gate; up] rows and a fused SiLU*up+quantise
    kernel: two 128-token accumulators cannot be double-buffered in TMEM, so the fused epilogue would serialise with the
    tensor-core work there (measured 2.1 ms against 0.8 ms for 16384 tokens x top-8)."""
    two_i, hid = w13.rows_per_group, w13.k
    wv = w13.mx.data.view(n_w_groups, two_i, hid)
    if tn == 32 or not x_q.is_cuda:
        gemm.grouped_linear(x_q, wv, seg_start, seg_count, tn, out=hq, dual=True, sfa=w13.mx.sf, sfb=x_sf, quant_out=True, out_sf=hsf,
                            extras=extras, w_groups=w_groups, w_tiled=w13.mx.tiled)
        return
    gu = scratch if scratch is not None else torch.empty(x_q.shape[0], two_i, dtype=torch.bfloat16, device=x_q.device)
    gemm.grouped_linear(x_q, wv, seg_start, seg_count, tn, out=gu, sfa=w13.mx.sf, sfb=x_sf, extras=extras, w_groups=w_groups,
                        w_tiled=w13.mx.tiled)
    ew.silu_mul_quant(gu, hq, hsf, row_valid, sf_layout=tn)


class Transformer:
    def __init__(self, weights: ModelWeights, kv: KvCache, par=None):
        self.w = weights
        self.cfg = weights.cfg
        self.kv = kv
        self.par = par if par is not None else SingleProcess()
        cfg = self.cfg
        self.hq_local = cfg.n_heads // weights.tp_size
        self.hkv_local = max(1, cfg.n_kv_heads // weights.tp_size)
        self.q_scale = ew.softmax_scale_log2(cfg.head_dim)
        self.mx = weights.fmt == "mxfp8"
        rd = cfg.rope_dim or cfg.head_dim
        if cfg.mrope_sections and sum(cfg.mrope_sections) > 0:
            rd = 2 * sum(cfg.mrope_sections)           # the rotary width under M-RoPE (common/transformer.h:1229-1232)
        self.rope_dim = rd
        self.rope_table = ew.rope_table(min(max(cfg.max_seq_len, 4096), 65536), rd, cfg.rope_theta, weights.embed.device) \
            if weights.embed.is_cuda else None
        self.snapshots = {}            # layer -> hidden rows captured after that layer (debug / DeepStack)
        self.snapshot_layers: Sequence[int] = ()

    # ------------------------------------------------------------------------------------------------
    def attention_block(self, li: int, lw, h: torch.Tensor, h_mx: Optional[MxTensor], fb: ForwardBatch) -> torch.Tensor:
        cfg = self.cfg
        # decode-sized batches: the projection is cut along K and the rope kernel sums the partials (not with an output gate,
        # whose columns are read again below)
        qkv = apply_linear(lw.wqkv, h, h_mx) if cfg.attn_output_gate else apply_linear_split(lw.wqkv, h, h_mx)
        if self.kv.quantized:
            return self._attention_q8(li, lw, qkv, fb)
        if getattr(self.par, "cp_world", 1) > 1:
            return self._attention_cp(li, lw, qkv, fb)
        q = ew.qk_norm_rope(qkv, fb.positions, fb.slots, lw.q_norm, lw.k_norm, self.kv.k[li], self.kv.v[li], self.hq_local,
                            self.hkv_local, cfg.head_dim, cfg.rope_theta, cfg.rms_eps, self.q_scale, self.rope_dim, table=self.rope_table,
                            positions3=fb.positions3, sections=cfg.mrope_sections)
        if (self.mx and lw.wo.fmt != "bf16" and not cfg.attn_output_gate and FUSE_ATTN_QUANT
                and att.can_decode_mx(q, self.hkv_local, fb.num_splits, fb.is_decode)):
            # decode: the attention kernel emits the MXFP8 operand of the output projection itself
            a_mx = att.attention_decode_mx(q, self.kv.k[li], self.kv.v[li], fb.cu_q, fb.kv_len, fb.block_table, self.kv.page_size, fb.work,
                                           window=cfg.sliding_window, sf_layout=32 if q.shape[0] <= 32 else 128, num_splits=fb.num_splits)
            return self.par.row_linear(lw.wo, None, a_mx)
        if self.mx and lw.wo.fmt != "bf16" and not cfg.attn_output_gate and FUSE_ATTN_QUANT and att.can_attention_mx(q, fb.num_splits):
            a_mx = att.attention_mx(q, self.kv.k[li], self.kv.v[li], fb.cu_q, fb.kv_len, fb.block_table, self.kv.page_size, fb.work,
                                    causal=True, window=cfg.sliding_window, sf_layout=32 if q.shape[0] <= 32 else 128)
            return self.par.row_linear(lw.wo, None, a_mx)
        a = att.attention(q, self.kv.k[li], self.kv.v[li], fb.cu_q, fb.kv_len, fb.block_table, self.kv.page_size, fb.work,
                          num_splits=fb.num_splits, causal=True, window=cfg.sliding_window, decode=fb.is_decode)
        a2 = a.reshape(a.shape[0], self.hq_local * cfg.head_dim)
        if cfg.attn_output_gate:
            g0 = (self.hq_local + 2 * self.hkv_local) * cfg.head_dim
            dn.gate_mul(a2, qkv[:, g0: g0 + self.hq_local * cfg.head_dim])
        return self.par.row_linear(lw.wo, a2)

    def _attention_cp(self, li: int, lw, qkv, fb: ForwardBatch) -> torch.Tensor:
        """Attention under context parallelism (``parallel.context.ContextParallel`` as the parallel context).  The cache holds
        this rank's pages only; ``fb.slots`` is -1 for a token another rank stores.  Decode: flash partials over the local shard,
        merged across the ranks.  Prefill: the rank's own tokens attend over the all-gathered K / V rows of the prompt."""
        cfg, kv = self.cfg, self.kv
        q = ew.qk_norm_rope(qkv, fb.positions, fb.slots, lw.q_norm, lw.k_norm, kv.k[li], kv.v[li], self.hq_local, self.hkv_local,
                            cfg.head_dim, cfg.rope_theta, cfg.rms_eps, self.q_scale, self.rope_dim, table=self.rope_table,
                            positions3=fb.positions3, sections=cfg.mrope_sections)
        if fb.is_decode:
            a = self.par.attention(q, kv.k[li], kv.v[li], fb.cu_q, fb.kv_len, fb.block_table, kv.page_size, fb.work,
                                   num_splits=fb.num_splits, decode=True)
        else:
            if fb.cp_send_slots is None:
                raise ValueError("a context-parallel prefill needs the forward batch of ContextParallel.build_prefill")
            kg, vg = self.par.gather_kv(kv.k[li], kv.v[li], fb.cp_send_slots)
            a = att.attention(q, kg, vg, fb.cu_q, fb.kv_len, fb.block_table, kv.page_size, fb.work, num_splits=1, causal=True)
        a2 = a.reshape(a.shape[0], self.hq_local * cfg.head_dim)
        if cfg.attn_output_gate:
            g0 = (self.hq_local + 2 * self.hkv_local) * cfg.head_dim
            dn.gate_mul(a2, qkv[:, g0: g0 + self.hq_local * cfg.head_dim])
        return self.par.row_linear(lw.wo, a2)

    def _attention_q8(self, li: int, lw, qkv, fb: ForwardBatch) -> torch.Tensor:
        """Attention with the INT8 KV cache: the new K / V rows go through the bf16 staging buffer (QK-norm + RoPE write them
        there), are quantised into the layer's pages, and a decode step reads the INT8 pages directly; a prefill step attends over
        the staged bf16 rows of its own tokens."""
        cfg, kv = self.cfg, self.kv
        if fb.stage_slots is None:
            raise ValueError("the INT8 KV cache needs a ForwardBatch built with stage=True")
        if fb.stage_slots.numel() > kv.k[li].shape[0] or (fb.stage_bt is not None and int(fb.stage_bt.shape[1]) * kv.page_size > kv.k[li].shape[0]):
            raise ValueError("the forward pass has more tokens than the KV staging buffer holds")
        q = ew.qk_norm_rope(qkv, fb.positions, fb.stage_slots, lw.q_norm, lw.k_norm, kv.k[li], kv.v[li], self.hq_local, self.hkv_local,
                            cfg.head_dim, cfg.rope_theta, cfg.rms_eps, self.q_scale, self.rope_dim, table=self.rope_table,
                            positions3=fb.positions3, sections=cfg.mrope_sections)
        att.kv_store_q8(kv.k[li], kv.v[li], fb.stage_slots, fb.slots, kv.kq[li], kv.vq[li], kv.ks[li], kv.vs[li])
        if fb.is_decode:
            a = att.attention_decode_q8(q, kv.kq[li], kv.vq[li], kv.ks[li], kv.vs[li], fb.kv_len, fb.block_table, kv.page_size,
                                        num_splits=fb.num_splits, window=cfg.sliding_window)
        else:
            if fb.stage_bt is None:
                raise NotImplementedError("INT8 KV cache: steps of several tokens per sequence on top of cached history (speculative "
                                          "verification, later prefill chunks) are not built")
            a = att.attention(q, kv.k[li], kv.v[li], fb.cu_q, fb.kv_len, fb.stage_bt, kv.page_size, fb.work, num_splits=1, causal=True,
                              window=cfg.sliding_window)
        a2 = a.reshape(a.shape[0], self.hq_local * cfg.head_dim)
        if cfg.attn_output_gate:
            g0 = (self.hq_local + 2 * self.hkv_local) * cfg.head_dim
            dn.gate_mul(a2, qkv[:, g0: g0 + self.hq_local * cfg.head_dim])
        return self.par.row_linear(lw.wo, a2)

    def ssm_block(self, li: int, lw, h: torch.Tensor, h_mx: Optional[MxTensor], fb: ForwardBatch) -> torch.Tensor:
        """Gated Delta-Net layer: projections -> causal conv + SiLU -> recurrence + gated norm -> output projection."""
        cfg, ssm = self.cfg, lw.ssm
        qd = cfg.ssm_qkv_dim
        proj = apply_linear(ssm.w_in, h, h_mx)                        # [T, qkv_dim + d_inner]
        ab = moe.router_logits(h, ssm.w_ab)                           # f32 [T, 2 * heads_v]
        slots = fb.seq_slots if fb.seq_slots is not None else torch.arange(fb.cu_q.numel() - 1, dtype=torch.int32, device=h.device)
        conv = dn.conv_silu(proj[:, :qd], ssm.conv_w, self.kv.conv[li], fb.cu_q, slots)
        out = dn.deltanet(conv, proj[:, qd:], ab, ssm.a, ssm.dt_bias, ssm.norm, self.kv.rec[li], fb.cu_q, slots, cfg.ssm_n_heads_k,
                          cfg.ssm_n_heads_v, cfg.ssm_head_dim, cfg.rms_eps)
        return self.par.row_linear(ssm.w_out, out)

    def shared_expert(self, lw, h: torch.Tensor) -> torch.Tensor:
        """Always-on expert of the qwen35moe layers, scaled by sigmoid(h . g) (cuda/llm/cuda_llm_runner.c:11879-11897)."""
        if lw.sh_gate_up.fmt == "bf16":
            act = gemm.linear_swiglu(h, lw.sh_gate_up.w, w_tiled=lw.sh_gate_up.tiled)
            y = apply_linear(lw.sh_down, act)
        else:
            xm = ew.mx_quantize(h, sf_layout=32 if h.shape[0] <= 32 else 128)
            y = apply_linear(lw.sh_down, None, gemm.linear_mx_swiglu_quant(xm, lw.sh_gate_up.mx))
        if lw.sh_gate is not None:
            g = torch.sigmoid(moe.router_logits(h, lw.sh_gate) if h.is_cuda and h.shape[1] % 256 == 0 else h.float() @ lw.sh_gate.float().t())
            y = (y.float() * g).to(torch.bfloat16)
        return y

    def dense_ffn(self, lw, h: torch.Tensor, h_mx: Optional[MxTensor]) -> torch.Tensor:
        gu = lw.w_gate_up
        inter = gu.n // 2
        if gu.is_quant:
            return self.par.row_linear(lw.w_down, qlinear.linear_swiglu(h, gu.q))
        if gu.fmt == "bf16":
            sp = gemm.pick_partials_dual(inter, h.shape[0], gu.k, False) if (SPLIT_PROJ and h.is_cuda and inter % 128 == 0) else 1
            if sp > 1:      # decode-sized batch: the projection is cut along K to fill the GPU, the activation kernel adds the partials
                act = ew.silu_mul_partials(gemm.swiglu_partials(h, gu.w, sp, w_tiled=gu.tiled))
            else:
                act = gemm.linear_swiglu(h, gu.w, w_tiled=gu.tiled)
            return self.par.row_linear(lw.w_down, act)
        xm = h_mx if h_mx is not None else ew.mx_quantize(h, sf_layout=32 if h.shape[0] <= 32 else 128)
        sp = gemm.pick_partials_dual(inter, xm.rows, gu.k, True) if (SPLIT_PROJ and xm.data.is_cuda and inter % 128 == 0) else 1
        if sp > 1:
            act = ew.silu_mul_partials(gemm.swiglu_partials(xm, gu.mx, sp), quantize=True, sf_layout=xm.sf_layout)
        else:
            act = gemm.linear_mx_swiglu_quant(xm, gu.mx)
        return self.par.row_linear(lw.w_down, None, act)

    def moe_local(self, lw, h: torch.Tensor, h_mx: Optional[MxTensor] = None, local_range=None) -> torch.Tensor:
        """The experts held by this GPU over the rows ``h``: route -> plan -> (gather + quantise) -> gate/up -> down -> combine.
        ``local_range = (first expert, count)``: the weights are that slice of the experts; (token, expert) pairs routed
        elsewhere are dropped from the plan and contribute nothing to the pending sum (the caller adds the ranks' sums)."""
        cfg = self.cfg
        t = h.shape[0]
        e, k, inter, hid = (local_range[1] if local_range else cfg.n_experts), cfg.n_experts_used, cfg.expert_ffn, cfg.hidden
        rt = dict(mode=cfg.router, bias=lw.router_bias, renorm=cfg.norm_topk, routed_scale=cfg.routed_scale, local_range=local_range)
        if self.mx:
            # token tile (= scale-atom layout) by the expected rows per expert: 32 for decode-sized batches
            tn = 32 if (t * k) // cfg.n_experts <= 24 else 128
            if tn == 32 and moe.can_prep(h, lw.router, k):
                # decode-sized batch: router projection, routing, plan and the quantised gather are one launch
                ids, wts, pl, xq = moe.prep_hidden(h, lw.router, k, e, tn, **rt)
            else:
                ids, wts, pl = moe.route_plan_hidden(h, lw.router, k, e, tn, **rt)
                # the RMSNorm before this block already quantised the tokens: gather bytes and scales (every token is quantised
                # once, not once per selected expert)
                xq = ew.mx_gather_rows(h_mx, pl.row_token, sf_layout=tn) if h_mx is not None else ew.mx_quantize(h, pl.row_token, sf_layout=tn)
            dev = h.device
            if tn == 32 and moe.can_fuse_ffn(xq, lw.w13, lw.w2, e, pl.capacity):
                y = moe.expert_ffn_fused(xq, lw.w13, lw.w2, e, pl)          # gate/up, activation and down as one persistent launch
            else:
                hq = torch.empty(pl.capacity, inter, dtype=torch.uint8, device=dev)
                hsf = ew.sf_alloc(pl.capacity, inter, dev, tn, init=False)
                expert_gate_up_mx(xq.data, xq.sf, lw.w13, e, pl.seg_start, pl.seg_count, tn, hq, hsf, pl.row_token)
                y = gemm.grouped_linear(hq, lw.w2.mx.data.view(e, hid, inter), pl.seg_start, pl.seg_count, tn, sfa=lw.w2.mx.sf, sfb=hsf,
                                        w_tiled=lw.w2.mx.tiled, pair_rows=(tn == 32 and PAIR_DOWN))
        else:
            tn = gemm.pick_tn(max(1, (t * k + cfg.n_experts - 1) // cfg.n_experts), dual=True)
            if moe.can_prep(h, lw.router, k):
                ids, wts, pl, xs = moe.prep_hidden(h, lw.router, k, e, tn, quantize=False, **rt)
            else:
                ids, wts, pl = moe.route_plan_hidden(h, lw.router, k, e, tn, **rt)
                xs = moe.gather_rows(h, pl.row_token)
            act = gemm.grouped_linear(xs, lw.w13.w.view(e, 2 * inter, hid), pl.seg_start, pl.seg_count, tn, dual=True, w_tiled=lw.w13.tiled)
            y = gemm.grouped_linear(act, lw.w2.w.view(e, hid, inter), pl.seg_start, pl.seg_count, tn, w_tiled=lw.w2.tiled)
        return moe.PendingCombine(y, pl.pair_row, wts, t, k)

    # ------------------------------------------------------------------------------------------------
    def forward_hidden(self, fb: ForwardBatch, first_layer: int = 0, last_layer: Optional[int] = None,
                       x: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Residual stream after layers ``[first_layer, last_layer)`` (pipeline stages pass ``x`` in)."""
        cfg, w = self.cfg, self.w
        last_layer = len(w.layers) if last_layer is None else last_layer
        if x is None:
            x = fb.embeds if fb.embeds is not None else ew.embed(fb.ids, w.embed)
        delta = None
        if hasattr(self.par, "_sp_ok"):
            # the fused tensor-parallel prefill path keeps the residual stream sharded by rows between the layers' GEMMs: only for
            # plain dense stacks (nothing reads the whole stream or the normalised rows outside a GEMM in between)
            self.par._sp_ok = not (cfg.is_moe or cfg.attn_output_gate or fb.deepstack is not None or self.snapshot_layers or
                                   any(l.ssm is not None for l in w.layers[first_layer:last_layer]))
        for li in range(first_layer, last_layer):
            lw = w.layers[li]
            lay = 32 if x.shape[0] <= 32 else 128
            par = self.par
            is_ssm = lw.ssm is not None
            if self.mx:
                h, h_mx = par.add_norm(delta if delta is not None else x, lw.attn_norm, cfg.rms_eps, x if delta is not None else None,
                                       quantize=True, want_bf16=is_ssm, sf_layout=lay)
            else:
                h, h_mx = par.add_norm(delta if delta is not None else x, lw.attn_norm, cfg.rms_eps, x if delta is not None else None), None
            with profiler.region("ssm" if is_ssm else "attention", "block", "attention", li):
                delta = self.ssm_block(li, lw, h, h_mx, fb) if is_ssm else self.attention_block(li, lw, h, h_mx, fb)
            need_bf16 = (not self.mx) or cfg.is_moe
            # a parallel context may name the buffer the normalised rows should land in (the staging buffer of its exchange)
            ob = par.ffn_in_buffer(x.shape[0], lw) if (hasattr(par, "ffn_in_buffer") and x.is_cuda) else None
            okw = {"out_buf": ob} if ob is not None else {}
            if self.mx:
                h, h_mx = par.add_norm(delta, lw.ffn_norm, cfg.rms_eps, x, quantize=True, want_bf16=need_bf16, sf_layout=lay, **okw)
            else:
                h, h_mx = par.add_norm(delta, lw.ffn_norm, cfg.rms_eps, x, **okw), None
            with profiler.region("moe" if lw.w13 is not None else "ffn", "block", "ffn", li):
                if lw.w13 is not None:
                    delta = self.par.moe_ffn(self, lw, h, h_mx)
                    if delta is None:
                        delta = self.moe_local(lw, h, h_mx)
                    if lw.sh_gate_up is not None:
                        delta = (self.par.materialize(delta).float() + self.shared_expert(lw, h).float()).to(torch.bfloat16)
                else:
                    delta = self.dense_ffn(lw, h, h_mx)
            if fb.deepstack is not None and li < fb.deepstack.shape[0]:
                # DeepStack (Qwen3-VL): vision features of deeper encoder layers join the stream after the first decoder layers
                delta = (self.par.materialize(delta).float() + fb.deepstack[li].float()).to(torch.bfloat16)
            if li in self.snapshot_layers:
                self.snapshots[li] = (x.float() + self.par.materialize(delta).float())
        # the last delta stays pending: the head (or the next pipeline stage) folds it into the stream
        if hasattr(self.par, "finish_residual"):
            self.par.finish_residual(x, delta)
        self._last_delta = self.par.materialize(delta) if delta is not None else None
        return x

    def forward(self, fb: ForwardBatch) -> torch.Tensor:
        """Logits ``f32 [len(logit_rows), V_local]``."""
        x = self.forward_hidden(fb)
        return self.head(x, fb)

    def _head_input(self, x: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        delta = self._last_delta
        rows = fb.logit_rows
        xr = x[rows]
        if delta is not None:
            xr = (xr.float() + delta[rows].float()).to(torch.bfloat16)
        return ew.rmsnorm(xr.contiguous(), w.final_norm, cfg.rms_eps)

    def head(self, x: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        if self.w.lm_head.is_quant:
            return qlinear.linear(self._head_input(x, fb), self.w.lm_head.q, out_dtype=torch.float32)
        return gemm.linear(self._head_input(x, fb), self.w.lm_head.w, out_dtype=torch.float32, w_tiled=self.w.lm_head.tiled)

    def forward_greedy(self, fb: ForwardBatch, want_value: bool = False):
        """Greedy next tokens ``int32 [len(logit_rows)]``: the arg-max runs in the LM-head GEMM's epilogue, no logits are stored."""
        x = self.forward_hidden(fb)
        if self.w.lm_head.is_quant:
            logits = qlinear.linear(self._head_input(x, fb), self.w.lm_head.q, out_dtype=torch.float32)
            return sampling.argmax(logits, idx_offset=self.w.vocab_start, want_value=want_value)
        return gemm.linear_argmax(self._head_input(x, fb), self.w.lm_head.w, idx_offset=self.w.vocab_start, want_value=want_value,
                                  w_tiled=self.w.lm_head.tiled)

    def final_hidden(self, x: torch.Tensor) -> torch.Tensor:
        """Residual stream with the pending delta folded in (what a pipeline stage hands to the next)."""
        if self._last_delta is None:
            return x
        return (x.float() + self._last_delta.float()).to(torch.bfloat16)


def greedy_tokens(logits: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    return sampling.argmax(logits, idx_offset=vocab_start)
