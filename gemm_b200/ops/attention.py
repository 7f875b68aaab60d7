"""Attention over the paged KV cache: wrapper of csrc/kernels/flash_attn.cu (prefill and decode share one
tcgen05 kernel; small decode batches split the KV range and merge partials) and the PyTorch reference.

Conventions: ``q [T, Hq, D]`` is already multiplied by ``softmax_scale * log2(e)`` (see
``elementwise.softmax_scale_log2``); ``k_cache`` / ``v_cache`` are ``[num_slots, Hkv, D]`` with
``slot = page * page_size + offset``; ``cu_q [B+1]`` gives each sequence's span of query tokens,
``kv_len [B]`` the sequence length including those tokens; ``block_table [B, max_pages]`` lists pages.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import List, Optional, Sequence

import torch

from .. import _native

_c, _i, _l = ctypes.c_void_p, ctypes.c_int, ctypes.c_long


def _p(t):
    return _c(t.data_ptr()) if t is not None else _c(0)


USE_DECODE_KERNEL = os.environ.get("GB_DECODE_ATTN", "1") != "0"      # 0: decode steps use the general kernel (A/B measurements)


def build_work(q_lens: Sequence[int], hq: int, hkv: int, num_splits: int = 1) -> torch.Tensor:
    """Host-side work list ``[n, 4] = {seq, kv_head, q_tok0, split}``: longest tiles first within a sequence,
    the heads of one tile adjacent (their K/V blocks hit in L2)."""
    g = hq // hkv
    tpt = 128 // g
    items: List[List[int]] = []
    for s, ql in enumerate(q_lens):
        n_tiles = (ql + tpt - 1) // tpt
        for ti in reversed(range(n_tiles)):
            for sp in range(num_splits):
                for h in range(hkv):
                    items.append([s, h, ti * tpt, sp])
    return torch.tensor(items, dtype=torch.int32).reshape(-1, 4)


def pick_splits(n_seqs: int, hkv: int, max_kv: int, sm_count: int = 148, ctas_per_sm: int = 2) -> int:
    """Number of KV splits for decode: enough CTAs to fill the GPU (the decode kernel runs two CTAs per SM, and one CTA streams
    its KV range at a fraction of an SM's share of the memory bandwidth), at least 2 KV blocks per split."""
    base = max(1, n_seqs * hkv)
    blocks = max(1, (max_kv + 127) // 128)
    splits = max(1, min((sm_count * ctas_per_sm) // base, blocks // 2 if blocks >= 2 else 1, 16))
    return splits


def attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
              block_table: torch.Tensor, page_size: int, work: torch.Tensor, num_splits: int = 1, causal: bool = True,
              window: int = 0, out: Optional[torch.Tensor] = None, scratch=None, decode: bool = False) -> torch.Tensor:
    """Attention output ``[T, Hq, D]`` (bf16).  ``work`` comes from ``build_work`` (moved to the device).  ``decode`` (every
    sequence has exactly one query token, at most 16 query heads per KV head) selects the decode-specialised kernel."""
    t, hq, d = q.shape
    hkv = k_cache.shape[1]
    if not q.is_cuda:
        return attention_ref(q, k_cache, v_cache, cu_q, kv_len, block_table, page_size, causal, window)
    if out is None:
        out = torch.empty(t, hq, d, dtype=torch.bfloat16, device=q.device)
    lib = _native.cuda()
    part_o = part_lse = None
    if num_splits > 1:
        if scratch is not None:
            part_o, part_lse = scratch
        else:
            part_o = torch.empty(num_splits, t, hq, d, dtype=torch.float32, device=q.device)
            part_lse = torch.empty(num_splits, t, hq, dtype=torch.float32, device=q.device)
    stream = _c(torch.cuda.current_stream().cuda_stream)
    if decode and USE_DECODE_KERNEL and hq // hkv <= 16:
        rc = lib.gb_flash_decode(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(part_o), _p(part_lse), _p(work), _i(work.shape[0]),
                                 _p(cu_q), _p(kv_len), _p(block_table), _i(block_table.shape[1]), _i(page_size),
                                 _l(k_cache.shape[0]), _i(t), _i(hq), _i(hkv), _i(d), _i(num_splits), _i(window),
                                 _c(_native.status_ptr()), stream)
        _native.check(rc, "gb_flash_decode")
    else:
        rc = lib.gb_flash_attn(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(part_o), _p(part_lse), _p(work), _i(work.shape[0]),
                               _p(cu_q), _p(kv_len), _p(block_table), _i(block_table.shape[1]), _i(page_size),
                               _l(k_cache.shape[0]), _i(t), _i(hq), _i(hkv), _i(d), _i(num_splits), _i(1 if causal else 0),
                               _i(window), _c(_native.status_ptr()), stream)
        _native.check(rc, "gb_flash_attn")
    if num_splits > 1:
        rc = lib.gb_fa_combine(_p(part_o), _p(part_lse), _p(out), _c(0), _i(num_splits), _l(t * hq), stream)
        _native.check(rc, "gb_fa_combine")
    return out


def kv_store_q8(k_src: torch.Tensor, v_src: torch.Tensor, src_slots: Optional[torch.Tensor], dst_slots: torch.Tensor, kq: torch.Tensor,
                vq: torch.Tensor, ks: torch.Tensor, vs: torch.Tensor) -> None:
    """Quantise the bf16 K / V rows ``k_src[src_slots[t]]`` (``[rows, Hkv, 128]``; row ``t`` when ``src_slots`` is None) of the
    new tokens into the INT8 cache at ``dst_slots[t]`` (negative: skipped): int8 ``kq`` / ``vq`` ``[slots, Hkv, 128]`` and one f32
    scale per slot and head in ``ks`` / ``vs`` ``[slots, Hkv]`` (``x = scale * q``, ``scale = amax / 127``)."""
    from .kvquant import quantize_q8_ref
    n = dst_slots.numel()
    if not k_src.is_cuda:
        src = src_slots.long() if src_slots is not None else torch.arange(n)
        ok = dst_slots >= 0
        for cache, sc, rows in ((kq, ks, k_src), (vq, vs, v_src)):
            q, scale = quantize_q8_ref(rows[src[ok]])
            cache[dst_slots[ok].long()] = q
            sc[dst_slots[ok].long()] = scale
        return
    rc = _native.cuda().gb_kv_store_q8(_p(k_src), _p(v_src), _p(src_slots), _p(dst_slots), _p(kq), _p(vq), _p(ks), _p(vs), _i(n),
                                       _i(kq.shape[1]), _i(kq.shape[2]), _l(k_src.shape[0]), _l(kq.shape[0]),
                                       _c(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "gb_kv_store_q8")


def attention_decode_q8(q: torch.Tensor, kq: torch.Tensor, vq: torch.Tensor, ks: torch.Tensor, vs: torch.Tensor, kv_len: torch.Tensor,
                        block_table: torch.Tensor, page_size: int, num_splits: int = 1, window: int = 0) -> torch.Tensor:
    """Decode attention (one query token per sequence) over the INT8 cache of ``kv_store_q8``; ``q`` as for ``attention``.
    Returns bf16 ``[B, Hq, 128]``.  (Reference: attn_decode_q8, cuda/llm/cuda_llm_runner.c:244-330.)"""
    b, hq, d = q.shape
    hkv = kq.shape[1]
    if not q.is_cuda:
        k = (kq.float() * ks.unsqueeze(-1)).to(torch.bfloat16)
        v = (vq.float() * vs.unsqueeze(-1)).to(torch.bfloat16)
        cu = torch.arange(b + 1, dtype=torch.int32)
        return attention_ref(q, k, v, cu, kv_len, block_table, page_size, True, window)
    out = torch.empty(b, hq, d, dtype=torch.bfloat16, device=q.device)
    part_o = part_lse = None
    if num_splits > 1:
        part_o = torch.empty(num_splits, b, hq, d, dtype=torch.float32, device=q.device)
        part_lse = torch.empty(num_splits, b, hq, dtype=torch.float32, device=q.device)
    lib = _native.cuda()
    stream = _c(torch.cuda.current_stream().cuda_stream)
    rc = lib.gb_attn_decode_q8(_p(q), _p(kq), _p(vq), _p(ks), _p(vs), _p(out), _p(part_o), _p(part_lse), _p(kv_len), _p(block_table),
                               _i(block_table.shape[1]), _i(page_size), _l(kq.shape[0]), _i(b), _i(hq), _i(hkv), _i(d), _i(num_splits),
                               _i(window), _c(_native.status_ptr()), stream)
    _native.check(rc, "gb_attn_decode_q8")
    if num_splits > 1:
        rc = lib.gb_fa_combine(_p(part_o), _p(part_lse), _p(out), _c(0), _i(num_splits), _l(b * hq), stream)
        _native.check(rc, "gb_fa_combine")
    return out


def attention_decode_mx(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                        block_table: torch.Tensor, page_size: int, work: torch.Tensor, window: int = 0, sf_layout: int = 128,
                        num_splits: int = 1):
    """Decode attention (one token per sequence, one KV split) whose output leaves the kernel as the MXFP8 operand of the output
    projection: ``MxTensor`` of ``[T, Hq * D]``.  GPU only; the caller checks ``can_decode_mx``."""
    from . import elementwise as ew
    from .mxfp8 import MxTensor
    t, hq, d = q.shape
    hkv = k_cache.shape[1]
    rp = (t + 127) // 128 * 128
    oq = torch.empty(rp, hq * d, dtype=torch.uint8, device=q.device)
    sf = ew.sf_alloc(rp, hq * d, q.device, sf_layout, init=False)
    if num_splits > 1:
        # split KV ranges: fp32 partials from the decode kernel, merged (and quantised) by the combine kernel
        lib, stream = _native.cuda(), _c(torch.cuda.current_stream().cuda_stream)
        part_o = torch.empty(num_splits, t, hq, d, dtype=torch.float32, device=q.device)
        part_lse = torch.empty(num_splits, t, hq, dtype=torch.float32, device=q.device)
        rc = lib.gb_flash_decode(_p(q), _p(k_cache), _p(v_cache), _c(0), _p(part_o), _p(part_lse), _p(work), _i(work.shape[0]),
                                 _p(cu_q), _p(kv_len), _p(block_table), _i(block_table.shape[1]), _i(page_size),
                                 _l(k_cache.shape[0]), _i(t), _i(hq), _i(hkv), _i(d), _i(num_splits), _i(window),
                                 _c(_native.status_ptr()), stream)
        _native.check(rc, "gb_flash_decode")
        rc = lib.gb_fa_combine_mx(_p(part_o), _p(part_lse), _p(oq), _p(sf), _i(1 if sf_layout == 32 else 0), _i(hq), _i(num_splits), _l(t * hq), stream)
        _native.check(rc, "gb_fa_combine_mx")
        return MxTensor(oq, sf, t, hq * d, sf_layout)
    rc = _native.cuda().gb_flash_decode_mx(_p(q), _p(k_cache), _p(v_cache), _p(oq), _p(sf), _i(1 if sf_layout == 32 else 0), _p(work),
                                           _i(work.shape[0]), _p(cu_q), _p(kv_len), _p(block_table), _i(block_table.shape[1]), _i(page_size),
                                           _l(k_cache.shape[0]), _i(t), _i(hq), _i(hkv), _i(d), _i(window), _c(_native.status_ptr()),
                                           _c(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "gb_flash_decode_mx")
    return MxTensor(oq, sf, t, hq * d, sf_layout)


def attention_mx(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                 block_table: torch.Tensor, page_size: int, work: torch.Tensor, causal: bool = True, window: int = 0, sf_layout: int = 128):
    """The general (prefill / mixed batch) kernel with the output leaving as the MXFP8 operand of the output projection
    (``MxTensor`` of ``[T, Hq * D]``): a softmax thread owns a whole (token, head) row, so its scale blocks are thread-local."""
    from . import elementwise as ew
    from .mxfp8 import MxTensor
    t, hq, d = q.shape
    hkv = k_cache.shape[1]
    rp = (t + 127) // 128 * 128
    oq = torch.empty(rp, hq * d, dtype=torch.uint8, device=q.device)
    sf = ew.sf_alloc(rp, hq * d, q.device, sf_layout, init=False)
    rc = _native.cuda().gb_flash_attn_mx(_p(q), _p(k_cache), _p(v_cache), _p(oq), _p(sf), _i(1 if sf_layout == 32 else 0), _p(work),
                                         _i(work.shape[0]), _p(cu_q), _p(kv_len), _p(block_table), _i(block_table.shape[1]), _i(page_size),
                                         _l(k_cache.shape[0]), _i(t), _i(hq), _i(hkv), _i(d), _i(1 if causal else 0), _i(window),
                                         _c(_native.status_ptr()), _c(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "gb_flash_attn_mx")
    return MxTensor(oq, sf, t, hq * d, sf_layout)


def can_attention_mx(q: torch.Tensor, num_splits: int) -> bool:
    return bool(q.is_cuda and num_splits == 1 and q.shape[2] == 128)


def can_decode_mx(q: torch.Tensor, hkv: int, num_splits: int, decode: bool) -> bool:
    return bool(decode and USE_DECODE_KERNEL and q.is_cuda and num_splits >= 1 and q.shape[2] == 128 and q.shape[1] // hkv <= 16)


def attention_partial(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                      block_table: torch.Tensor, page_size: int, work: torch.Tensor, num_splits: int = 1, causal: bool = False,
                      window: int = 0, decode: bool = False):
    """Flash partials of the attention over THIS cache only: ``(part_o f32 [S, T, Hq, D]`` normalised by its own sum,
    ``part_lse f32 [S, T, Hq]`` base 2; -inf where a row saw no key).  The caller merges them with partials of other KV
    shards (``combine_partials``): the building block of context parallelism.  ``decode`` (one query per sequence, which sees
    every cached key) selects the decode-specialised kernel, whose ``num_splits`` KV ranges are partials of their own."""
    t, hq, d = q.shape
    if not q.is_cuda:
        o, l = _attention_partial_ref(q, k_cache, v_cache, cu_q, kv_len, block_table, page_size, causal, window)
        if num_splits > 1:         # the reference computes one partial; the other splits saw no key
            o = torch.cat([o, torch.zeros(num_splits - 1, *o.shape[1:])])
            l = torch.cat([l, torch.full((num_splits - 1, *l.shape[1:]), float("-inf"))])
        return o, l
    part_o = torch.empty(num_splits, t, hq, d, dtype=torch.float32, device=q.device)
    part_lse = torch.empty(num_splits, t, hq, dtype=torch.float32, device=q.device)
    if decode and USE_DECODE_KERNEL and hq // k_cache.shape[1] <= 16:
        rc = _native.cuda().gb_flash_decode(_p(q), _p(k_cache), _p(v_cache), _c(0), _p(part_o), _p(part_lse), _p(work), _i(work.shape[0]),
                                            _p(cu_q), _p(kv_len), _p(block_table), _i(block_table.shape[1]), _i(page_size),
                                            _l(k_cache.shape[0]), _i(t), _i(hq), _i(k_cache.shape[1]), _i(d), _i(num_splits), _i(window),
                                            _c(_native.status_ptr()), _c(torch.cuda.current_stream().cuda_stream))
        _native.check(rc, "gb_flash_decode")
        return part_o, part_lse
    rc = _native.cuda().gb_flash_attn(_p(q), _p(k_cache), _p(v_cache), _c(0), _p(part_o), _p(part_lse), _p(work), _i(work.shape[0]),
                                      _p(cu_q), _p(kv_len), _p(block_table), _i(block_table.shape[1]), _i(page_size),
                                      _l(k_cache.shape[0]), _i(t), _i(hq), _i(k_cache.shape[1]), _i(d), _i(num_splits), _i(1 if causal else 0),
                                      _i(window), _c(_native.status_ptr()), _c(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "gb_flash_attn")
    return part_o, part_lse


def _attention_partial_ref(q, k_cache, v_cache, cu_q, kv_len, block_table, page_size, causal, window):
    """CPU reference of ``attention_partial`` (one split).  ``q`` carries softmax_scale * log2(e), scores are base 2."""
    t, hq, d = q.shape
    hkv = k_cache.shape[1]
    g = hq // hkv
    out = torch.zeros(1, t, hq, d, dtype=torch.float32)
    lse = torch.full((1, t, hq), float("-inf"), dtype=torch.float32)
    cu = cu_q.tolist()
    for s in range(len(cu) - 1):
        q0, q1 = cu[s], cu[s + 1]
        ql, kl = q1 - q0, int(kv_len[s])
        if ql == 0 or kl == 0:
            continue
        n_pages = (kl + page_size - 1) // page_size
        idx = (block_table[s, :n_pages].long().unsqueeze(1) * page_size + torch.arange(page_size)).reshape(-1)[:kl]
        k = k_cache[idx].float().repeat_interleave(g, dim=1)
        v = v_cache[idx].float().repeat_interleave(g, dim=1)
        sc = torch.einsum("qhd,khd->hqk", q[q0:q1].float(), k)
        if causal:
            qpos = torch.arange(kl - ql, kl).unsqueeze(1)
            sc = sc.masked_fill(~(torch.arange(kl).unsqueeze(0) <= qpos), float("-inf"))
        l2 = torch.logsumexp(sc * math.log(2.0), dim=-1) / math.log(2.0)
        p = torch.exp2(sc - l2.unsqueeze(-1))
        out[0, q0:q1] = torch.einsum("hqk,khd->qhd", p, v)
        lse[0, q0:q1] = l2.t()
    return out, lse


def combine_partials(part_o: torch.Tensor, part_lse: torch.Tensor):
    """Merge flash partials ``part_o [S, R, D]`` (each normalised by its own sum) and base-2 ``part_lse [S, R]``.
    Returns ``(out bf16 [R, D], lse f32 [R])``.  Also the rule for context parallelism (KV sharded over GPUs)."""
    s, r, d = part_o.shape
    if not part_o.is_cuda:
        mx = part_lse.max(dim=0).values
        w = torch.exp2(part_lse - mx)
        w = torch.where(torch.isinf(part_lse) & (part_lse < 0), torch.zeros_like(w), w)
        den = w.sum(0)
        out = (w.unsqueeze(-1) * part_o).sum(0) / den.clamp_min(1e-30).unsqueeze(-1)
        return out.to(torch.bfloat16), mx + torch.log2(den)
    out = torch.empty(r, d, dtype=torch.bfloat16, device=part_o.device)
    lse = torch.empty(r, dtype=torch.float32, device=part_o.device)
    rc = _native.cuda().gb_fa_combine(_p(part_o), _p(part_lse), _p(out), _p(lse), _i(s), _l(r),
                                      _c(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "gb_fa_combine")
    return out, lse


def attention_ref(q, k_cache, v_cache, cu_q, kv_len, block_table, page_size, causal=True, window=0) -> torch.Tensor:
    """fp32 reference: gathers each sequence's K/V through the block table and applies masked softmax."""
    t, hq, d = q.shape
    hkv = k_cache.shape[1]
    g = hq // hkv
    out = torch.zeros(t, hq, d, dtype=torch.float32, device=q.device)
    cu = cu_q.tolist()
    for s in range(len(cu) - 1):
        q0, q1 = cu[s], cu[s + 1]
        ql, kl = q1 - q0, int(kv_len[s])
        if ql == 0:
            continue
        n_pages = (kl + page_size - 1) // page_size
        slots = (block_table[s, :n_pages].long().unsqueeze(1) * page_size + torch.arange(page_size, device=q.device)).reshape(-1)[:kl]
        k = k_cache[slots].float()          # [kl, hkv, d]
        v = v_cache[slots].float()
        qs = q[q0:q1].float()               # [ql, hq, d]  (already scaled, log2 domain)
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
        sc = torch.einsum("qhd,khd->hqk", qs, k) * math.log(2.0)
        qpos = torch.arange(kl - ql, kl, device=q.device).unsqueeze(1)
        kpos = torch.arange(kl, device=q.device).unsqueeze(0)
        mask = torch.ones(ql, kl, dtype=torch.bool, device=q.device)
        if causal:
            mask &= kpos <= qpos
        if window > 0:
            mask &= kpos > qpos - window
        sc = sc.masked_fill(~mask.unsqueeze(0), float("-inf"))
        p = torch.softmax(sc, dim=-1)
        out[q0:q1] = torch.einsum("hqk,khd->qhd", p, v)
    return out.to(torch.bfloat16)
