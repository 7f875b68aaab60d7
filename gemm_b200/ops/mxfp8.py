"""MXFP8 (OCP microscaling) tensors: e4m3 payload + one E8M0 scale per 1x32 block along K.

Semantics follow the reference's MXFP8 readers (common/glm5_mxfp8.h:24-35, common/m3_mxfp8.h):
``w = e4m3(W) * 2^(s - 127)`` with the "fn" flavour of e4m3.  The reference has no quantiser; ours
picks the smallest power-of-two scale that keeps the block inside +-448 so that nothing saturates.

Two scale layouts exist:

* ``rowmajor``  uint8 [rows, K/32] — what checkpoints store (``weight_scale_inv``).
* ``atoms``     uint8 [ceil(rows/128), K/128, 512] — what the tcgen05 block-scaled MMA consumes after a
  ``tcgen05.cp.32x128b.warpx4``: inside one 512-byte atom the scale of (row r, 32-block b) sits at
  ``(r % 32) * 16 + ((r // 32) % 4) * 4 + (b % 4)``.

The functions here are the plain PyTorch reference (CPU or GPU); the fused CUDA quantisers must match
them bit for bit.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

E4M3_MAX = 448.0
_INV448 = torch.tensor(1.0 / 448.0, dtype=torch.float32)


@dataclass
class MxTensor:
    """Row-major e4m3 bytes plus scales in atom layout.  ``rows`` counts valid rows (storage may be padded)."""
    data: torch.Tensor      # uint8 [rows_padded, k]
    sf: torch.Tensor        # uint8 [ceil(rows_padded/128), k/128, 512]  (or [rows_padded/32, k/128, 512] when sf_layout == 32)
    rows: int
    k: int
    sf_layout: int = 128    # rows per scale atom: 128 (default) or 32 (token tiles of 32 rows)
    tiled: bool = False     # ``data`` holds the tiled weight layout (see ``tile_weight``); same shape, permuted memory

    def to(self, device):
        return MxTensor(self.data.to(device), self.sf.to(device), self.rows, self.k, self.sf_layout, self.tiled)


def tile_weight(w: torch.Tensor) -> torch.Tensor:
    """Row-major ``[rows, K]`` -> the tiled weight layout of the GEMM kernel, returned with the same shape.

    Memory order becomes ``[rows/128][K/box][128 rows][box]`` with ``box`` = 128 bytes of elements (128 fp8 / 64 bf16):
    every 16 KB operand tile that the kernel's TMA fetches is one contiguous block, so a decode step streams the weights
    as long DRAM bursts instead of 128-byte lines that are a row pitch apart."""
    rows, k = w.shape
    box = 128 // w.element_size()
    assert rows % 128 == 0 and k % box == 0, "tiled weights need rows % 128 == 0 and K a multiple of 128 bytes"
    return w.reshape(rows // 128, 128, k // box, box).permute(0, 2, 1, 3).contiguous().view(rows, k)


def untile_weight(t: torch.Tensor) -> torch.Tensor:
    rows, k = t.shape
    box = 128 // t.element_size()
    return t.reshape(rows // 128, k // box, 128, box).permute(0, 2, 1, 3).contiguous().view(rows, k)


def can_tile(w: torch.Tensor) -> bool:
    return w.dim() == 2 and w.shape[0] % 128 == 0 and (w.shape[1] * w.element_size()) % 128 == 0


def e8m0_from_amax(amax: torch.Tensor) -> torch.Tensor:
    """Biased exponent (int32 in [1, 254]) of the smallest power of two s with amax / s <= 448."""
    s = (amax.to(torch.float32) * _INV448.to(amax.device)).contiguous()
    bits = s.view(torch.int32)
    e = (bits >> 23) & 0xFF
    e = e + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    e = e.clamp(1, 254)
    return torch.where(amax == 0, torch.full_like(e, 127), e)     # an all-zero block gets scale 1


def quantize_rowmajor(x: torch.Tensor):
    """x [rows, K] (K % 32 == 0) -> (uint8 e4m3 bytes [rows, K], uint8 E8M0 [rows, K/32])."""
    rows, k = x.shape
    assert k % 32 == 0
    xf = x.to(torch.float32).reshape(rows, k // 32, 32)
    amax = xf.abs().amax(dim=-1)
    e = e8m0_from_amax(amax)
    inv = ((254 - e) << 23).to(torch.int32).view(torch.float32)      # 2^(127 - e)
    q = (xf * inv.unsqueeze(-1)).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).reshape(rows, k), e.to(torch.uint8)


def dequantize_rowmajor(q: torch.Tensor, e: torch.Tensor) -> torch.Tensor:
    """Inverse of quantize_rowmajor -> float32 [rows, K]."""
    rows, k = q.shape
    v = q.view(torch.float8_e4m3fn).to(torch.float32).reshape(rows, k // 32, 32)
    scale = (e.to(torch.int32) << 23).view(torch.float32)           # 2^(e - 127)
    return (v * scale.unsqueeze(-1)).reshape(rows, k)


def pack_sf_atoms(e: torch.Tensor, layout: int = 128) -> torch.Tensor:
    """uint8 [rows, K/32] -> uint8 [ceil(rows/128), ceil(K/128), 512] (padding scales = 127 i.e. 1.0).

    ``layout=32`` gives one atom per 32 rows, ``[ceil(rows/32), ceil(K/128), 512]``: the four scales of
    (row, k-atom) sit in bytes 0..3 of the row's 16-byte lane slot, the other 12 bytes are unused."""
    rows, nb = e.shape
    rp, kp = (rows + 127) // 128 * 128, (nb + 3) // 4 * 4
    pad = torch.full((rp, kp), 127, dtype=torch.uint8, device=e.device)
    pad[:rows, :nb] = e
    if layout == 32:
        t = torch.full((rp // 32, kp // 4, 32, 16), 127, dtype=torch.uint8, device=e.device)
        t[..., :4] = pad.reshape(rp // 32, 32, kp // 4, 4).permute(0, 2, 1, 3)
        return t.reshape(rp // 32, kp // 4, 512)
    # [R/128, 4(row group), 32(lane), K/128, 4(sub-block)] -> [R/128, K/128, 32, 4, 4]
    t = pad.reshape(rp // 128, 4, 32, kp // 4, 4).permute(0, 3, 2, 1, 4).contiguous()
    return t.reshape(rp // 128, kp // 4, 512)


def unpack_sf_atoms(sf: torch.Tensor, rows: int, nb: int, layout: int = 128) -> torch.Tensor:
    """Inverse of pack_sf_atoms."""
    rb, kb, _ = sf.shape
    if layout == 32:
        t = sf.reshape(rb, kb, 32, 16)[..., :4].permute(0, 2, 1, 3).contiguous().reshape(rb * 32, kb * 4)
        return t[:rows, :nb].contiguous()
    t = sf.reshape(rb, kb, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().reshape(rb * 128, kb * 4)
    return t[:rows, :nb].contiguous()


def quantize(x: torch.Tensor, pad_rows_to: int = 128, sf_layout: int = 128) -> MxTensor:
    """Quantise [rows, K] (K % 128 == 0) into an MxTensor whose storage rows are padded with zeros."""
    rows, k = x.shape
    assert k % 128 == 0, "MXFP8 GEMM operands need K % 128 == 0"
    q, e = quantize_rowmajor(x)
    rp = (rows + pad_rows_to - 1) // pad_rows_to * pad_rows_to
    if rp != rows:
        q = torch.cat([q, torch.zeros(rp - rows, k, dtype=torch.uint8, device=q.device)])
        e = torch.cat([e, torch.full((rp - rows, k // 32), 127, dtype=torch.uint8, device=e.device)])
    return MxTensor(q.contiguous(), pack_sf_atoms(e, sf_layout), rows, k, sf_layout)


def dequantize(t: MxTensor) -> torch.Tensor:
    e = unpack_sf_atoms(t.sf, t.data.shape[0], t.k // 32, t.sf_layout)
    return dequantize_rowmajor(untile_weight(t.data) if t.tiled else t.data, e)[: t.rows]
