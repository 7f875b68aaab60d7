"""ggml block formats handled with torch ops on any device: encoders for Q8_0 and Q4_K that run on the GPU (a synthetic
30 B-parameter checkpoint is quantised where it is generated, not on the host), decoders for the same two formats, and the
tile re-packing the quantised GEMV / GEMM kernels read (csrc/kernels/qgemv.cu, qgemm.cu).

Formats (common/ggml_dequant.h:30-34,1479-1489 and :1582-1618 in the reference; the decoders of csrc/host/dequant.cc are the oracle):

* Q8_0   block of 32: ``{f16 d; int8 q[32]}``, ``w = d * q``.
* Q4_K   super-block of 256: ``{f16 d; f16 dmin; u8 scales[12]; u8 qs[128]}``; eight sub-blocks of 32 with 6-bit ``(sc, m)``;
         ``w = d * sc * q - dmin * m``; of every 64 values the first 32 sit in the low nibbles, the next 32 in the high nibbles.

The encoders produce valid blocks of these formats; they do not search for the error-minimising scales the way ggml's
``make_qkx2_quants`` does (the reference has no quantiser at all), they take min / max per sub-block.

Tiled layout.  A quantised matrix ``[rows, k]`` (rows a multiple of 128, k a multiple of 256) is stored as
``[rows / 128][k / 256]`` tiles; a tile holds 128 rows x 256 columns and is one contiguous piece of memory, so a CTA that owns a
row tile streams whole tiles:

* Q4_K tile: 128 super-blocks of 144 bytes, row after row (18 432 bytes).
* Q8_0 tile: 128 rows of 272 bytes, a row being its 256 int8 values followed by its eight f16 scales: the same 34 bytes per
  block as in the file, with the values 16-byte aligned (and a row stride that spreads the rows over the shared-memory banks).
"""
from __future__ import annotations

from typing import Tuple

import torch

Q8_0, Q4_K = 8, 12
BLOCK = {Q8_0: (32, 34), Q4_K: (256, 144)}
TILE_ROWS, TILE_K = 128, 256


def tile_bytes(t: int) -> int:
    blk, nb = BLOCK[t]
    return TILE_ROWS * (TILE_K // blk) * nb


# ------------------------------------------------------------------------------------------------ Q8_0
def quantize_q8_0(w: torch.Tensor) -> torch.Tensor:
    """``w [rows, k]`` (k % 32 == 0) -> uint8 ``[rows, k / 32 * 34]`` of row-major Q8_0 blocks."""
    rows, k = w.shape
    x = w.float().reshape(rows, k // 32, 32)
    d = (x.abs().amax(-1) / 127.0).to(torch.float16)
    inv = torch.where(d.float() > 0, 1.0 / d.float(), torch.zeros_like(d, dtype=torch.float32))
    q = torch.clamp(torch.round(x * inv.unsqueeze(-1)), -127, 127).to(torch.int8)
    out = torch.empty(rows, k // 32, 34, dtype=torch.uint8, device=w.device)
    out[..., :2] = d.view(torch.uint8).reshape(rows, k // 32, 2)
    out[..., 2:] = q.view(torch.uint8)
    return out.reshape(rows, -1)


def dequantize_q8_0(raw: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    b = raw.reshape(rows, k // 32, 34)
    d = b[..., :2].contiguous().view(torch.float16).float()
    q = b[..., 2:].contiguous().view(torch.int8).float()
    return (d * q).reshape(rows, k)


# ------------------------------------------------------------------------------------------------ Q4_K
def _pack_scales_k4(sc: torch.Tensor, mn: torch.Tensor) -> torch.Tensor:
    """6-bit ``sc`` / ``mn`` ``[..., 8]`` (uint8) -> the 12 packed bytes of a K-quant super-block (the inverse of get_scale_min_k4)."""
    sc, mn = sc.to(torch.int32), mn.to(torch.int32)
    out = torch.empty(sc.shape[:-1] + (12,), dtype=torch.int32, device=sc.device)
    out[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 15) | ((mn[..., 4:8] & 15) << 4)
    return out.to(torch.uint8)


def _unpack_scales_k4(s: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    s = s.to(torch.int32)
    sc = torch.empty(s.shape[:-1] + (8,), dtype=torch.int32, device=s.device)
    mn = torch.empty_like(sc)
    sc[..., 0:4] = s[..., 0:4] & 63
    mn[..., 0:4] = s[..., 4:8] & 63
    sc[..., 4:8] = (s[..., 8:12] & 15) | ((s[..., 0:4] >> 6) << 4)
    mn[..., 4:8] = (s[..., 8:12] >> 4) | ((s[..., 4:8] >> 6) << 4)
    return sc, mn


def quantize_q4_k(w: torch.Tensor) -> torch.Tensor:
    """``w [rows, k]`` (k % 256 == 0) -> uint8 ``[rows, k / 256 * 144]`` of row-major Q4_K super-blocks."""
    rows, k = w.shape
    nb = k // 256
    x = w.float().reshape(rows, nb, 8, 32)
    lo = torch.clamp(x.amin(-1), max=0.0)                        # w = d*sc*q - dmin*m with m >= 0: the offset is -min (>= 0)
    hi = x.amax(-1)
    scale = (hi - lo) / 15.0                                     # per sub-block step
    mins = -lo
    d = (scale.amax(-1) / 63.0).to(torch.float16)                # super-block scale of the 6-bit steps
    dmin = (mins.amax(-1) / 63.0).to(torch.float16)
    df, dmf = d.float().unsqueeze(-1), dmin.float().unsqueeze(-1)
    sc = torch.where(df > 0, torch.round(scale / torch.where(df > 0, df, torch.ones_like(df))), torch.zeros_like(scale)).clamp(0, 63)
    mn = torch.where(dmf > 0, torch.round(mins / torch.where(dmf > 0, dmf, torch.ones_like(dmf))), torch.zeros_like(mins)).clamp(0, 63)
    step = (df * sc).unsqueeze(-1)
    off = (dmf * mn).unsqueeze(-1)
    q = torch.where(step > 0, torch.round((x + off) / torch.where(step > 0, step, torch.ones_like(step))), torch.zeros_like(x)).clamp(0, 15)
    q = q.to(torch.uint8).reshape(rows, nb, 4, 2, 32)            # [.., pair of sub-blocks, low / high, 32]
    qs = (q[..., 0, :] | (q[..., 1, :] << 4)).reshape(rows, nb, 128)
    out = torch.empty(rows, nb, 144, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = d.view(torch.uint8).reshape(rows, nb, 2)
    out[..., 2:4] = dmin.view(torch.uint8).reshape(rows, nb, 2)
    out[..., 4:16] = _pack_scales_k4(sc.to(torch.uint8), mn.to(torch.uint8))
    out[..., 16:] = qs
    return out.reshape(rows, -1)


def dequantize_q4_k(raw: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    nb = k // 256
    b = raw.reshape(rows, nb, 144)
    d = b[..., 0:2].contiguous().view(torch.float16).float()     # [rows, nb, 1]
    dmin = b[..., 2:4].contiguous().view(torch.float16).float()
    sc, mn = _unpack_scales_k4(b[..., 4:16])
    qs = b[..., 16:].reshape(rows, nb, 4, 32)
    q = torch.stack([qs & 15, qs >> 4], dim=3).reshape(rows, nb, 8, 32).float()
    w = (d * sc.float()).unsqueeze(-1) * q - (dmin * mn.float()).unsqueeze(-1)
    return w.reshape(rows, k)


def quantize(w: torch.Tensor, t: int) -> torch.Tensor:
    return quantize_q8_0(w) if t == Q8_0 else quantize_q4_k(w)


def dequantize(raw: torch.Tensor, t: int, rows: int, k: int) -> torch.Tensor:
    return dequantize_q8_0(raw, rows, k) if t == Q8_0 else dequantize_q4_k(raw, rows, k)


# ------------------------------------------------------------------------------------------------ tiles
def tile(raw: torch.Tensor, t: int, rows: int, k: int) -> torch.Tensor:
    """Row-major blocks ``[rows, row_bytes]`` -> the tiled layout (uint8 ``[rows / 128, k / 256, tile_bytes]``)."""
    if rows % TILE_ROWS or k % TILE_K:
        raise ValueError(f"tiled ggml weights need rows % 128 == 0 and k % 256 == 0 (got {rows} x {k})")
    rt, kt = rows // TILE_ROWS, k // TILE_K
    if t == Q4_K:
        return raw.reshape(rt, TILE_ROWS, kt, 144).permute(0, 2, 1, 3).reshape(rt, kt, TILE_ROWS * 144).contiguous()
    b = raw.reshape(rt, TILE_ROWS, kt, 8, 34).permute(0, 2, 1, 3, 4)                     # [rt, kt, 128, 8, 34]
    out = torch.empty(rt, kt, TILE_ROWS, 272, dtype=torch.uint8, device=raw.device)
    out[..., :256] = b[..., 2:].reshape(rt, kt, TILE_ROWS, 256)
    out[..., 256:] = b[..., :2].reshape(rt, kt, TILE_ROWS, 16)
    return out.reshape(rt, kt, tile_bytes(Q8_0))


def untile(tiled: torch.Tensor, t: int, rows: int, k: int) -> torch.Tensor:
    """Inverse of ``tile``: row-major blocks ``[rows, row_bytes]``."""
    rt, kt = rows // TILE_ROWS, k // TILE_K
    if t == Q4_K:
        return tiled.reshape(rt, kt, TILE_ROWS, 144).permute(0, 2, 1, 3).reshape(rows, kt * 144).contiguous()
    t4 = tiled.reshape(rt, kt, TILE_ROWS, 272)
    q = t4[..., :256].reshape(rt, kt, TILE_ROWS, 8, 32)
    d = t4[..., 256:].reshape(rt, kt, TILE_ROWS, 8, 2)
    return torch.cat([d, q], dim=-1).permute(0, 2, 1, 3, 4).reshape(rows, kt * 8 * 34).contiguous()
