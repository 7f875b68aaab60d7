"""Gated Delta-Net ops of the Qwen3.5 hybrid models (csrc/kernels/deltanet.cu) and their PyTorch references.

``conv_silu``   causal depthwise conv1d with per-sequence history + SiLU over packed tokens
``deltanet``    the recurrence S <- S * exp(alpha) + ((v - S k) * beta) k^T, o = S q, followed by the gated RMSNorm
``gate_mul``    x *= sigmoid(gate) (output gate of the full-attention layers)

State tensors: ``conv_state`` f32 ``[slots, conv_k - 1, channels]`` (oldest row first) and ``rec_state`` f32
``[slots, dt_rank, d_state, d_state]`` (row = value index, column = key index); both are updated in place.
Reference semantics: common/transformer.h:2861-3113 and :3857-3935.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _native

_c, _i, _f, _l = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_long


def _p(t):
    return _c(t.data_ptr()) if t is not None else _c(0)


def _s():
    return _c(torch.cuda.current_stream().cuda_stream)


def conv_silu_ref(x, w, state, cu_q, seq_slots):
    t, ch = x.shape
    conv_k = w.shape[1]
    out = torch.empty(t, ch, dtype=torch.float32)
    cu = cu_q.tolist()
    xf = x.float()
    for s in range(len(cu) - 1):
        slot = int(seq_slots[s])
        win = state[slot].clone().float()                    # [conv_k - 1, ch]
        for ti in range(cu[s], cu[s + 1]):
            full = torch.cat([win, xf[ti:ti + 1]], 0)         # [conv_k, ch]
            acc = (full * w.float().t()).sum(0)
            out[ti] = acc * torch.sigmoid(acc)
            win = full[1:]
        if cu[s + 1] > cu[s]:
            state[slot].copy_(win)
    return out.to(torch.bfloat16)


def conv_silu(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor, seq_slots: torch.Tensor) -> torch.Tensor:
    """``x`` bf16 [T, C] (may be a column slice), ``w`` f32 [C, conv_k] -> bf16 [T, C]; ``state`` is advanced."""
    t, ch = x.shape
    if not x.is_cuda:
        return conv_silu_ref(x, w, state, cu_q, seq_slots)
    out = torch.empty(t, ch, dtype=torch.bfloat16, device=x.device)
    rc = _native.cuda().gb_ssm_conv_silu(_p(x), _i(x.stride(0)), _p(w), _p(state), _p(cu_q), _p(seq_slots), _p(out), _i(ch), _i(ch),
                                         _i(w.shape[1]), _i(cu_q.numel() - 1), _s())
    _native.check(rc, "gb_ssm_conv_silu")
    return out


# The chunked prefill scan (GB_DELTANET_CHUNKED=0 keeps the per-token kernel): taken when the launch averages at least this many
# tokens per sequence (a decode step, one token per sequence, always takes the per-token kernel)
CHUNKED = os.environ.get("GB_DELTANET_CHUNKED", "1") != "0"
CHUNKED_MIN_TOKENS = 48
_ws_cache = {}


def _chunk_workspace(device, nbytes: int) -> torch.Tensor:
    """Scratch of the chunked scan, kept per device and grown on demand (every layer of a forward pass reuses it: the launches
    are ordered on the stream)."""
    cur = _ws_cache.get(device)
    if cur is None or cur.numel() < nbytes:
        cur = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _ws_cache[device] = cur
    return cur


def deltanet_ref(qkv, z, ab, a, dt_bias, norm_w, state, cu_q, seq_slots, n_group, dt_rank, d_state, eps):
    t = qkv.shape[0]
    ds = d_state
    out = torch.empty(t, dt_rank * ds, dtype=torch.float32)
    cu = cu_q.tolist()
    qf, zf = qkv.float(), z.float()
    scale = ds ** -0.5
    for s in range(len(cu) - 1):
        slot = int(seq_slots[s])
        S = state[slot].clone().float()                      # [dt_rank, ds, ds]
        for ti in range(cu[s], cu[s + 1]):
            q = qf[ti, : n_group * ds].reshape(n_group, ds)
            k = qf[ti, n_group * ds: 2 * n_group * ds].reshape(n_group, ds)
            v = qf[ti, 2 * n_group * ds:].reshape(dt_rank, ds)
            q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + eps) * scale
            k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + eps)
            idx = torch.arange(dt_rank) % n_group
            qh, kh = q[idx], k[idx]                           # [dt_rank, ds]
            ar = ab[ti, :dt_rank].float() + dt_bias.float()
            sp = torch.where(ar > 20, ar, torch.log1p(torch.exp(ar)))
            decay = torch.exp(sp * a.float())
            beta = torch.sigmoid(ab[ti, dt_rank:].float())
            S = S * decay[:, None, None]
            sk = torch.einsum("hrc,hc->hr", S, kh)
            delta = (v - sk) * beta[:, None]
            S = S + delta[:, :, None] * kh[:, None, :]
            o = torch.einsum("hrc,hc->hr", S, qh)
            o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * norm_w.float()[None, :]
            zz = zf[ti].reshape(dt_rank, ds)
            out[ti] = (o * zz * torch.sigmoid(zz)).reshape(-1)
        if cu[s + 1] > cu[s]:
            state[slot].copy_(S)
    return out.to(torch.bfloat16)


def deltanet(qkv: torch.Tensor, z: torch.Tensor, ab: torch.Tensor, a: torch.Tensor, dt_bias: torch.Tensor, norm_w: torch.Tensor,
             state: torch.Tensor, cu_q: torch.Tensor, seq_slots: torch.Tensor, n_group: int, dt_rank: int, d_state: int,
             eps: float) -> torch.Tensor:
    """``qkv`` bf16 [T, (2 n_group + dt_rank) d_state] (after conv + SiLU), ``z`` bf16 [T, dt_rank d_state] (column slices allowed),
    ``ab`` f32 [T, 2 dt_rank] -> bf16 [T, dt_rank d_state]; ``state`` is advanced."""
    t = qkv.shape[0]
    if not qkv.is_cuda:
        return deltanet_ref(qkv, z, ab, a, dt_bias, norm_w, state, cu_q, seq_slots, n_group, dt_rank, d_state, eps)
    out = torch.empty(t, dt_rank * d_state, dtype=torch.bfloat16, device=qkv.device)
    assert ab.is_contiguous() and ab.dtype == torch.float32 and state.dtype == torch.float32
    n_seqs = cu_q.numel() - 1
    if CHUNKED and d_state == 128 and t >= CHUNKED_MIN_TOKENS * n_seqs:
        # prefill: the chunked scan (64 tokens per step of the serial chain, the chunk-local part parallel over all chunks)
        lib = _native.cuda()
        lib.gb_deltanet_chunk_workspace.restype = ctypes.c_long
        need = int(lib.gb_deltanet_chunk_workspace(_l(t), _i(n_seqs), _i(dt_rank)))
        ws = _chunk_workspace(qkv.device, need)
        rc = lib.gb_deltanet_chunked(_p(qkv), _i(qkv.stride(0)), _p(z), _i(z.stride(0)), _p(ab), _p(a), _p(dt_bias), _p(norm_w), _p(state),
                                     _p(cu_q), _p(seq_slots), _p(out), _i(n_group), _i(dt_rank), _i(d_state), _f(eps), _i(n_seqs), _l(t),
                                     _p(ws), _l(ws.numel()), _s())
        _native.check(rc, "gb_deltanet_chunked")
        return out
    rc = _native.cuda().gb_deltanet(_p(qkv), _i(qkv.stride(0)), _p(z), _i(z.stride(0)), _p(ab), _p(a), _p(dt_bias), _p(norm_w), _p(state),
                                    _p(cu_q), _p(seq_slots), _p(out), _i(n_group), _i(dt_rank), _i(d_state), _f(eps), _i(cu_q.numel() - 1), _s())
    _native.check(rc, "gb_deltanet")
    return out


def gate_mul(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """In place ``x *= sigmoid(gate)`` (bf16 [T, C]; ``gate`` may be a column slice of a wider tensor)."""
    if not x.is_cuda:
        x.copy_((x.float() * torch.sigmoid(gate.float())).to(x.dtype))
        return x
    rows, cols = x.shape
    rc = _native.cuda().gb_sigmoid_gate_mul(_p(x), _i(x.stride(0)), _p(gate), _i(gate.stride(0)), _l(rows), _i(cols), _s())
    _native.check(rc, "gb_sigmoid_gate_mul")
    return x
