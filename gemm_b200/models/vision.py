"""Qwen3-VL vision encoder (the "mmproj" GGUF file): image -> embeddings for the text model, as a PyTorch-op forward pass.

Pipeline (reference: common/vision_encoder.h:421-531 for the tensors, :554-1008 for the forward pass):

1. patches of ``patch_size`` x ``patch_size`` pixels in raster order, each a linear map of its CHW pixels (two kernels added: the
   temporal pair of the video model applied to one image) plus bias;
2. learned position embeddings taken from the top-left ``gh x gw`` sub-grid of the trained grid;
3. ``n_blocks`` pre-LayerNorm ViT blocks: fused QKV with bias, 2-D rotary embedding (the first half of a head's rotation pairs
   turns with the patch row, the second half with the column; frequencies ``10000^(-2 i / (head_dim / 2))`` restarting in each
   half; pairs are ``(i, i + head_dim / 2)``), full attention over all patches, output projection, GELU (tanh form) MLP;
4. after the blocks flagged in ``deepstack_layers``: 2 x 2 spatial merge -> LayerNorm -> fc1 -> GELU -> fc2 (the DeepStack
   features the text model adds to its stream after its first layers);
5. post-LayerNorm, 2 x 2 spatial merge, ``mm.0`` -> GELU -> ``mm.2``.

``encode`` returns ``[n_merged, proj_dim * (1 + n_deepstack)]`` (main embedding, then the DeepStack slices, per token) like the
reference; ``forward_inputs`` splits it into what ``ForwardBatch`` takes (``embeds`` and ``deepstack``).  The matrix products are
library tensor ops (head size 64 is outside the flash kernels of this repository).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from ..utils import gguf as G


@dataclass
class VisionConfig:
    n_blocks: int = 24
    dim: int = 1024
    n_heads: int = 16
    ffn: int = 4096
    patch_size: int = 16
    image_size: int = 768
    proj_dim: int = 2048
    spatial_merge: int = 2
    ln_eps: float = 1e-6
    image_mean: Tuple[float, float, float] = (0.5, 0.5, 0.5)
    image_std: Tuple[float, float, float] = (0.5, 0.5, 0.5)
    deepstack_layers: List[int] = field(default_factory=list)      # block indices whose output feeds a DeepStack head

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @property
    def grid(self) -> int:
        return self.image_size // self.patch_size


def config_from_gguf(f: G.GGUFFile) -> VisionConfig:
    m = f.metadata
    k = lambda name, d: m.get("clip.vision." + name, d)
    flags = m.get("clip.vision.is_deepstack_layers")
    return VisionConfig(
        n_blocks=int(k("block_count", 24)), dim=int(k("embedding_length", 1024)), n_heads=int(k("attention.head_count", 16)),
        ffn=int(k("feed_forward_length", 4096)), patch_size=int(k("patch_size", 16)), image_size=int(k("image_size", 768)),
        proj_dim=int(k("projection_dim", 2048)), spatial_merge=int(k("spatial_merge_size", 2)),
        ln_eps=float(k("attention.layer_norm_epsilon", 1e-6)),
        image_mean=tuple(float(x) for x in k("image_mean", (0.5, 0.5, 0.5))), image_std=tuple(float(x) for x in k("image_std", (0.5, 0.5, 0.5))),
        deepstack_layers=[i for i, x in enumerate(flags) if x] if flags is not None else [])


def load_gguf(path: str, device="cpu", dtype=torch.float32) -> "VisionEncoder":
    with G.GGUFFile(path) as f:
        cfg = config_from_gguf(f)
        t = {}
        for name, gt in f.tensors.items():
            x = gt.to_float()
            t[name] = x.to(device=device, dtype=torch.float32 if x.dim() == 1 else dtype)
    return VisionEncoder(cfg, t, device, dtype)


def random_tensors(cfg: VisionConfig, seed: int = 0, dual_patch: bool = True) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g) * 0.05
    vec = lambda n, c=0.0: c + 0.1 * torch.randn(n, generator=g)
    d, ps, md = cfg.dim, cfg.patch_size, cfg.dim * cfg.spatial_merge ** 2
    t = {"v.patch_embd.weight": rn(d, 3, ps, ps), "v.patch_embd.bias": vec(d), "v.position_embd.weight": rn(cfg.grid ** 2, d),
         "v.post_ln.weight": vec(d, 1.0), "v.post_ln.bias": vec(d), "mm.0.weight": rn(md, md), "mm.0.bias": vec(md),
         "mm.2.weight": rn(cfg.proj_dim, md), "mm.2.bias": vec(cfg.proj_dim)}
    if dual_patch:
        t["v.patch_embd.weight.1"] = rn(d, 3, ps, ps)
    for l in range(cfg.n_blocks):
        p = f"v.blk.{l}."
        t.update({p + "attn_qkv.weight": rn(3 * d, d), p + "attn_qkv.bias": vec(3 * d), p + "attn_out.weight": rn(d, d), p + "attn_out.bias": vec(d),
                  p + "ffn_up.weight": rn(cfg.ffn, d), p + "ffn_up.bias": vec(cfg.ffn), p + "ffn_down.weight": rn(d, cfg.ffn),
                  p + "ffn_down.bias": vec(d), p + "ln1.weight": vec(d, 1.0), p + "ln1.bias": vec(d), p + "ln2.weight": vec(d, 1.0),
                  p + "ln2.bias": vec(d)})
    for l in cfg.deepstack_layers:
        p = f"v.deepstack.{l}."
        t.update({p + "fc1.weight": rn(md, md), p + "fc1.bias": vec(md), p + "fc2.weight": rn(cfg.proj_dim, md), p + "fc2.bias": vec(cfg.proj_dim),
                  p + "norm.weight": vec(md, 1.0), p + "norm.bias": vec(md)})
    return t


def save_gguf(cfg: VisionConfig, tensors: Dict[str, torch.Tensor], path: str, wtype: str = "F16") -> None:
    w = G.GGUFWriter()
    w.add_string("general.architecture", "clip")
    for key, v in (("block_count", cfg.n_blocks), ("embedding_length", cfg.dim), ("attention.head_count", cfg.n_heads),
                   ("feed_forward_length", cfg.ffn), ("patch_size", cfg.patch_size), ("image_size", cfg.image_size),
                   ("projection_dim", cfg.proj_dim), ("spatial_merge_size", cfg.spatial_merge)):
        w.add_u32("clip.vision." + key, v)
    w.add_f32("clip.vision.attention.layer_norm_epsilon", cfg.ln_eps)
    w.add_array("clip.vision.image_mean", list(cfg.image_mean), G.KV_F32)
    w.add_array("clip.vision.image_std", list(cfg.image_std), G.KV_F32)
    if cfg.deepstack_layers:
        w.add_array("clip.vision.is_deepstack_layers", [i in cfg.deepstack_layers for i in range(cfg.n_blocks)], G.KV_BOOL)
    for name, x in tensors.items():
        w.add_tensor(name, x.float(), "F32" if x.dim() == 1 else wtype)
    w.write(path)


def _gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    xf = x.float()
    return (0.5 * xf * (1.0 + torch.tanh(0.7978845608 * (xf + 0.044715 * xf ** 3)))).to(x.dtype)


class VisionEncoder:
    def __init__(self, cfg: VisionConfig, tensors: Dict[str, torch.Tensor], device="cpu", dtype=torch.float32):
        self.cfg, self.t, self.device, self.dtype = cfg, tensors, torch.device(device), dtype

    def normalize_image(self, rgb: torch.Tensor) -> torch.Tensor:
        """uint8 ``[H, W, 3]`` -> f32 ``[H, W, 3]``: (x / 255 - mean) / std per channel."""
        mean = torch.tensor(self.cfg.image_mean, dtype=torch.float32, device=rgb.device)
        std = torch.tensor(self.cfg.image_std, dtype=torch.float32, device=rgb.device)
        return (rgb.float() / 255.0 - mean) / std

    def _lin(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return x @ self.t[name + ".weight"].t() + self.t[name + ".bias"].to(x.dtype)

    def _ln(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), self.t[name + ".weight"].float(), self.t[name + ".bias"].float(),
                                              self.cfg.ln_eps).to(x.dtype)

    def _merge(self, x: torch.Tensor, gh: int, gw: int) -> torch.Tensor:
        """``[gh * gw, dim]`` raster order -> ``[gh/s * gw/s, s * s * dim]``: the s x s neighbours of a cell, row by row."""
        s, d = self.cfg.spatial_merge, x.shape[-1]
        return x.reshape(gh // s, s, gw // s, s, d).permute(0, 2, 1, 3, 4).reshape((gh // s) * (gw // s), s * s * d)

    def _rope(self, gh: int, gw: int):
        hd = self.cfg.head_dim
        half, sect = hd // 2, hd // 4
        i = torch.arange(half, device=self.device)
        freq = (10000.0 ** (-2.0 / half)) ** (i % sect).float()
        py = torch.arange(gh, device=self.device).repeat_interleave(gw).float()
        px = torch.arange(gw, device=self.device).repeat(gh).float()
        pos = torch.where(i[None, :] < sect, py[:, None], px[:, None])              # [patches, half]
        ang = pos * freq[None, :]
        return ang.cos()[:, None, :], ang.sin()[:, None, :]

    @torch.no_grad()
    def encode(self, rgb_norm: torch.Tensor) -> torch.Tensor:
        """``rgb_norm`` f32 ``[H, W, 3]`` (H, W multiples of patch_size * spatial_merge, at most ``image_size``)."""
        cfg, t = self.cfg, self.t
        ps, d, nh, hd = cfg.patch_size, cfg.dim, cfg.n_heads, cfg.head_dim
        hgt, wid, _ = rgb_norm.shape
        gh, gw = hgt // ps, wid // ps
        if gh * gw > cfg.grid ** 2 or gh % cfg.spatial_merge or gw % cfg.spatial_merge:
            raise ValueError("image larger than the trained grid, or its patch grid is not a multiple of the spatial merge")
        img = rgb_norm.to(self.device, self.dtype)[: gh * ps, : gw * ps]
        patches = img.reshape(gh, ps, gw, ps, 3).permute(0, 2, 4, 1, 3).reshape(gh * gw, 3 * ps * ps)      # CHW inside a patch
        wk = t["v.patch_embd.weight"].reshape(d, -1)
        if "v.patch_embd.weight.1" in t:
            wk = wk + t["v.patch_embd.weight.1"].reshape(d, -1)
        x = patches @ wk.t()
        if "v.patch_embd.bias" in t:
            x = x + t["v.patch_embd.bias"].to(x.dtype)
        pos = t["v.position_embd.weight"].reshape(cfg.grid, cfg.grid, d)[:gh, :gw].reshape(gh * gw, d)
        x = x + pos.to(x.dtype)
        cos, sin = self._rope(gh, gw)
        half = hd // 2
        feats = []
        for l in range(cfg.n_blocks):
            p = f"v.blk.{l}."
            qkv = self._lin(self._ln(x, p + "ln1"), p + "attn_qkv").reshape(gh * gw, 3, nh, hd).float()
            q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
            rot = lambda z: torch.cat([z[..., :half] * cos - z[..., half:] * sin, z[..., :half] * sin + z[..., half:] * cos], dim=-1)
            q, k = rot(q), rot(k)
            sc = torch.einsum("qhd,khd->hqk", q, k) * hd ** -0.5
            a = torch.einsum("hqk,khd->qhd", torch.softmax(sc, dim=-1), v).reshape(gh * gw, d).to(self.dtype)
            x = x + self._lin(a, p + "attn_out")
            x = x + self._lin(_gelu_tanh(self._lin(self._ln(x, p + "ln2"), p + "ffn_up")), p + "ffn_down")
            if l in cfg.deepstack_layers:
                dp = f"v.deepstack.{l}."
                m = self._ln(self._merge(x, gh, gw), dp + "norm")
                feats.append(self._lin(_gelu_tanh(self._lin(m, dp + "fc1")), dp + "fc2"))
        m = self._merge(self._ln(x, "v.post_ln"), gh, gw)
        main = self._lin(_gelu_tanh(self._lin(m, "mm.0")), "mm.2")
        return torch.cat([main] + feats, dim=1).float()

    def forward_inputs(self, features: torch.Tensor):
        """``encode`` output -> ``(embeds bf16 [T, proj_dim], deepstack bf16 [n_deepstack, T, proj_dim] or None)``: the vision
        tokens' rows of ``ForwardBatch.embeds`` and ``ForwardBatch.deepstack``."""
        pd = self.cfg.proj_dim
        n_ds = features.shape[1] // pd - 1
        embeds = features[:, :pd].to(torch.bfloat16)
        ds = features[:, pd:].reshape(-1, n_ds, pd).permute(1, 0, 2).contiguous().to(torch.bfloat16) if n_ds > 0 else None
        return embeds, ds


def _decode_png(data: bytes) -> torch.Tensor:
    """8-bit non-interlaced PNG (grey, grey + alpha, RGB, RGBA, palette) -> uint8 [H, W, 3]; alpha is dropped.  The container and
    the inflate step are handled here, the scanline filters by the host library (csrc/host/image.cc)."""
    import ctypes
    import struct
    import zlib
    from .. import _native
    pos, idat, plte, hdr = 8, [], None, None
    while pos + 8 <= len(data):
        n, kind = struct.unpack(">I4s", data[pos: pos + 8])
        body = data[pos + 8: pos + 8 + n]
        if kind == b"IHDR":
            if len(body) != 13:
                raise ValueError("PNG header of the wrong size")
            hdr = struct.unpack(">IIBBBBB", body)
        elif kind == b"PLTE":
            if len(body) % 3 or not body:
                raise ValueError("PNG palette of the wrong size")
            plte = torch.frombuffer(bytearray(body), dtype=torch.uint8).reshape(-1, 3)
        elif kind == b"IDAT":
            idat.append(body)
        elif kind == b"IEND":
            break
        pos += 12 + n
    if hdr is None or not idat:
        raise ValueError("PNG without header or data")
    wd, ht, depth, ctype, _, _, interlace = hdr
    channels = {0: 1, 2: 3, 3: 1, 4: 2, 6: 4}.get(ctype)
    if depth != 8 or channels is None or interlace != 0:
        raise ValueError("only 8-bit non-interlaced PNG files are read")
    row = wd * channels
    if wd <= 0 or ht <= 0 or wd * ht > (1 << 26):
        raise ValueError(f"PNG of {wd} x {ht} pixels is not read (64 Mpixel at most)")
    try:
        raw = zlib.decompressobj().decompress(b"".join(idat), ht * (row + 1) + 1)      # bounded: the header says how much there is
    except zlib.error as e:
        raise ValueError(f"PNG data: {e}")
    if len(raw) != ht * (row + 1):
        raise ValueError("PNG data does not match its header")
    out = torch.empty(ht, wd, channels, dtype=torch.uint8)
    src = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
    if _native.host().gbh_png_unfilter(ctypes.c_void_p(src.data_ptr()), ctypes.c_long(ht), ctypes.c_long(row), ctypes.c_int(channels),
                                       ctypes.c_void_p(out.data_ptr())) != 0:
        raise ValueError(_native.host().gbh_last_error().decode(errors="replace"))
    if ctype == 3:
        if plte is None:
            raise ValueError("palette PNG without a palette")
        if int(out.max()) >= plte.shape[0]:
            raise ValueError("PNG pixel names a colour outside its palette")
        return plte[out[..., 0].long()].contiguous()
    if ctype in (0, 4):
        return out[..., :1].expand(ht, wd, 3).contiguous()
    return out[..., :3].contiguous()


def _decode_jpeg(data: bytes) -> torch.Tensor:
    """Baseline JPEG -> uint8 [H, W, 3] through the host library's decoder (csrc/host/image.cc)."""
    import ctypes
    from .. import _native
    lib = _native.host()
    buf = torch.frombuffer(bytearray(data), dtype=torch.uint8)
    w, h, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    if lib.gbh_jpeg_info(ctypes.c_void_p(buf.data_ptr()), ctypes.c_long(len(data)), ctypes.byref(w), ctypes.byref(h), ctypes.byref(c)) != 0:
        raise ValueError(lib.gbh_last_error().decode(errors="replace"))
    out = torch.empty(h.value, w.value, 3, dtype=torch.uint8)
    if lib.gbh_jpeg_decode(ctypes.c_void_p(buf.data_ptr()), ctypes.c_long(len(data)), ctypes.c_void_p(out.data_ptr())) != 0:
        raise ValueError(lib.gbh_last_error().decode(errors="replace"))
    return out


def resize_image(rgb: torch.Tensor, height: int, width: int) -> torch.Tensor:
    """uint8 [H, W, 3] -> uint8 [height, width, 3], bilinear with anti-aliasing when shrinking (the reference's server resizes
    with an area filter before it encodes, cuda/llm/test_gemma4_st.c:165-168)."""
    x = rgb.permute(2, 0, 1)[None].float()
    y = torch.nn.functional.interpolate(x, size=(height, width), mode="bilinear", antialias=True, align_corners=False)
    return y[0].permute(1, 2, 0).round().clamp(0, 255).to(torch.uint8).contiguous()


def decode_image(data: bytes) -> torch.Tensor:
    """uint8 ``[H, W, 3]`` from the bytes of a PNG, a baseline JPEG, a binary PPM (P6, maxval 255) or a ``.npy`` file holding such an
    array; no image library is involved."""
    if data[:8] == b"\x89PNG\r\n\x1a\n":
        return _decode_png(data)
    if data[:2] == b"\xff\xd8":
        return _decode_jpeg(data)
    if data[:6] == b"\x93NUMPY":
        import io
        import numpy as np
        arr = np.load(io.BytesIO(data), allow_pickle=False)
        if arr.ndim != 3 or arr.shape[2] != 3 or arr.dtype != np.uint8:
            raise ValueError("the .npy image must be uint8 [H, W, 3]")
        return torch.from_numpy(arr.copy())
    parts, pos = [], 0
    while len(parts) < 4:                                   # magic, width, height, maxval; comments start with '#'
        while data[pos:pos + 1].isspace():
            pos += 1
        if data[pos:pos + 1] == b"#":
            pos = data.index(b"\n", pos) + 1
            continue
        end = pos
        while end < len(data) and not data[end:end + 1].isspace():
            end += 1
        if end == pos:
            raise ValueError("truncated PPM header")
        parts.append(data[pos:end])
        pos = end
    if parts[0] != b"P6" or int(parts[3]) != 255:
        raise ValueError("only PNG, baseline JPEG, binary PPM (P6, maxval 255) and .npy images are read")
    wd, ht = int(parts[1]), int(parts[2])
    body = data[pos + 1: pos + 1 + wd * ht * 3]
    if len(body) != wd * ht * 3:
        raise ValueError("truncated PPM data")
    return torch.frombuffer(bytearray(body), dtype=torch.uint8).reshape(ht, wd, 3)


def prompt_inputs(embed_table: torch.Tensor, ids_before, features: torch.Tensor, ids_after, proj_dim: int):
    """Input rows of a prompt ``text, image, text``: ``(placeholder ids int32 [T], embeds bf16 [T, hidden], deepstack bf16
    [n_deepstack, T, hidden] or None)``.  Text rows are the token embeddings, the image rows the encoder's main embedding; the
    DeepStack slices sit on the image rows and are zero elsewhere.  Positions run on through the image (one per vision token), as in
    the reference's server (server/server_llm.c:526-533 feeds the vision rows at consecutive positions)."""
    ids_before = torch.as_tensor(ids_before, dtype=torch.long)
    ids_after = torch.as_tensor(ids_after, dtype=torch.long)
    n_img = features.shape[0]
    n_ds = features.shape[1] // proj_dim - 1
    tab = embed_table
    rows = [tab[ids_before.to(tab.device)].to(torch.bfloat16), features[:, :proj_dim].to(tab.device, torch.bfloat16),
            tab[ids_after.to(tab.device)].to(torch.bfloat16)]
    embeds = torch.cat(rows)
    t = embeds.shape[0]
    ds = None
    if n_ds > 0:
        ds = torch.zeros(n_ds, t, proj_dim, dtype=torch.bfloat16, device=tab.device)
        ds[:, ids_before.numel(): ids_before.numel() + n_img] = features[:, proj_dim:].reshape(n_img, n_ds, proj_dim).permute(1, 0, 2).to(tab.device, torch.bfloat16)
    ids = torch.cat([ids_before, torch.zeros(n_img, dtype=torch.long), ids_after]).to(torch.int32)
    return ids, embeds, ds


# ---------------------------------------------------------------------------------------------------- Gemma4 vision tower
@dataclass
class Gemma4VisionConfig:
    n_blocks: int = 16
    dim: int = 768
    n_heads: int = 12
    ffn: int = 3072
    patch_size: int = 16
    image_size: int = 224
    proj_dim: int = 2560
    pool: int = 3                     # average-pooling kernel over the patch grid
    ln_eps: float = 1e-6
    n_pos: int = 64                   # rows of each of the two position tables (x and y)
    rope_theta: float = 100.0
    projector: str = ""               # "gemma4uv": the block-free variant, one token per (patch_size * pool)-pixel square

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @property
    def unified(self) -> bool:
        return self.projector == "gemma4uv"


class Gemma4VisionEncoder:
    """The ViT tower of the Gemma4 mmproj files (reference: common/gemma4_vision_encoder.h:676-934 for the pieces, :1168-1290 for the
    pipeline): pixels scaled to [-1, 1]; patch embedding; x and y position tables added; blocks of RMSNorm -> separate q / k / v
    -> per-head RMSNorm of q and k -> 2-D RoPE (first half of a head turns with x, second half with y, pairs ``(j, j + D/4)``
    inside a half, theta 100) -> attention WITHOUT a score scale -> output projection -> post-norm -> residual, then RMSNorm ->
    GELU(gate) * up -> down -> post-norm -> residual; ``pool x pool`` average pooling; times sqrt(dim); ``mm.input_projection``;
    weightless RMSNorm.

    The "gemma4uv" projector of the same files (common/gemma4_vision_encoder.h:936-1166) has no transformer blocks: squares of
    ``patch_size * pool`` pixels -> LayerNorm over the square's values -> patch matrix + bias -> LayerNorm -> x and y position rows
    added -> LayerNorm -> weightless RMSNorm -> ``mm.input_projection``; one token per square."""

    def __init__(self, cfg: Gemma4VisionConfig, tensors: Dict[str, torch.Tensor], device="cpu", dtype=torch.float32):
        self.cfg, self.t, self.device, self.dtype = cfg, tensors, torch.device(device), dtype

    @staticmethod
    def random_tensors(cfg: Gemma4VisionConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
        g = torch.Generator().manual_seed(seed)
        rn = lambda *s: torch.randn(*s, generator=g) * 0.05
        nw = lambda n: 1.0 + 0.1 * torch.randn(n, generator=g)
        d, ps = cfg.dim, cfg.patch_size
        t = {"v.patch_embd.weight": rn(d, 3, ps, ps), "v.position_embd.weight": rn(2, cfg.n_pos, d), "mm.input_projection.weight": rn(cfg.proj_dim, d)}
        if cfg.unified:
            pd = 3 * (ps * cfg.pool) ** 2
            t["v.patch_embd.weight"], t["v.patch_embd.bias"] = rn(d, pd), rn(d)
            for i, n in ((1, pd), (2, d), (3, d)):
                t[f"v.patch_norm.{i}.weight"], t[f"v.patch_norm.{i}.bias"] = nw(n), rn(n)
            return t
        for b in range(cfg.n_blocks):
            p = f"v.blk.{b}."
            t.update({p + "attn_q.weight": rn(d, d), p + "attn_k.weight": rn(d, d), p + "attn_v.weight": rn(d, d), p + "attn_out.weight": rn(d, d),
                      p + "attn_q_norm.weight": nw(cfg.head_dim), p + "attn_k_norm.weight": nw(cfg.head_dim), p + "attn_post_norm.weight": nw(d),
                      p + "ffn_gate.weight": rn(cfg.ffn, d), p + "ffn_up.weight": rn(cfg.ffn, d), p + "ffn_down.weight": rn(d, cfg.ffn),
                      p + "ffn_post_norm.weight": nw(d), p + "ln1.weight": nw(d), p + "ln2.weight": nw(d)})
        return t

    @staticmethod
    def save_gguf(cfg: Gemma4VisionConfig, tensors: Dict[str, torch.Tensor], path: str, wtype: str = "F16") -> None:
        w = G.GGUFWriter()
        w.add_string("general.architecture", "clip")
        for key, v in (("block_count", cfg.n_blocks), ("embedding_length", cfg.dim), ("attention.head_count", cfg.n_heads),
                       ("feed_forward_length", cfg.ffn), ("patch_size", cfg.patch_size), ("image_size", cfg.image_size), ("projection_dim", cfg.proj_dim)):
            w.add_u32("clip.vision." + key, v)
        w.add_f32("clip.vision.attention.layer_norm_epsilon", cfg.ln_eps)
        if cfg.projector:
            w.add_string("clip.vision.projector_type", cfg.projector)
        for name, x in tensors.items():
            w.add_tensor(name, x.float(), "F32" if x.dim() == 1 else wtype)
        w.write(path)

    @staticmethod
    def load_gguf(path: str, device="cpu", dtype=torch.float32) -> "Gemma4VisionEncoder":
        with G.GGUFFile(path) as f:
            m = f.metadata
            k = lambda name, d: m.get("clip.vision." + name, d)
            t = {}
            for name, gt in f.tensors.items():
                x = gt.to_float()
                t[name] = x.to(device=device, dtype=torch.float32 if x.dim() == 1 else dtype)
            cfg = Gemma4VisionConfig(n_blocks=int(k("block_count", 16)), dim=int(k("embedding_length", 768)), n_heads=int(k("attention.head_count", 12)),
                                     ffn=int(k("feed_forward_length", 3072)), patch_size=int(k("patch_size", 16)), image_size=int(k("image_size", 224)),
                                     proj_dim=int(k("projection_dim", 2560)), ln_eps=float(k("attention.layer_norm_epsilon", 1e-6)),
                                     n_pos=int(t["v.position_embd.weight"].shape[1]),
                                     projector="gemma4uv" if k("projector_type", "") == "gemma4uv" else "")
        return Gemma4VisionEncoder(cfg, t, device, dtype)

    def _ln(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return F.layer_norm(x.float(), x.shape[-1:], self.t[name + ".weight"].float(), self.t[name + ".bias"].float(), self.cfg.ln_eps).to(x.dtype)

    def _encode_unified(self, rgb: torch.Tensor) -> torch.Tensor:
        cfg, t = self.cfg, self.t
        ps = cfg.patch_size * cfg.pool
        gh, gw = rgb.shape[0] // ps, rgb.shape[1] // ps
        if max(gh, gw) > cfg.n_pos or gh * gw == 0:
            raise ValueError("image smaller than one square of the projector or larger than its position tables")
        img = (rgb.to(self.device).float() / 255.0 * 2.0 - 1.0)[: gh * ps, : gw * ps]
        sq = img.reshape(gh, ps, gw, ps, 3).permute(0, 2, 4, 1, 3).reshape(gh * gw, 3 * ps * ps)        # channel, row, column inside a square
        x = self._ln(sq, "v.patch_norm.1").to(self.dtype) @ t["v.patch_embd.weight"].reshape(cfg.dim, -1).t()
        if "v.patch_embd.bias" in t:
            x = x + t["v.patch_embd.bias"].to(x.dtype)
        x = self._ln(x, "v.patch_norm.2")
        py = torch.arange(gh, device=self.device).repeat_interleave(gw)
        px = torch.arange(gw, device=self.device).repeat(gh)
        pos = t["v.position_embd.weight"]
        x = self._ln(x + pos[0][px].to(x.dtype) + pos[1][py].to(x.dtype), "v.patch_norm.3")
        return (self._rms(x, None) @ t["mm.input_projection.weight"].t()).float()

    def _rms(self, x: torch.Tensor, w: Optional[torch.Tensor]) -> torch.Tensor:
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.ln_eps)
        return (y * w.float() if w is not None else y).to(x.dtype)

    def _rope2d(self, x: torch.Tensor, px: torch.Tensor, py: torch.Tensor) -> torch.Tensor:
        """``x`` [N, H, D]."""
        d = x.shape[-1]
        half, quarter = d // 2, d // 4
        freq = self.cfg.rope_theta ** (-(2.0 * torch.arange(quarter, device=self.device).float()) / half)
        out = []
        for pos, sl in ((px, x[..., :half]), (py, x[..., half:])):
            ang = pos.float()[:, None, None] * freq[None, None, :]
            a, b = sl[..., :quarter].float(), sl[..., quarter:].float()
            out += [a * ang.cos() - b * ang.sin(), a * ang.sin() + b * ang.cos()]
        return torch.cat(out, dim=-1).to(x.dtype)

    @torch.no_grad()
    def encode(self, rgb: torch.Tensor) -> torch.Tensor:
        """uint8 ``[H, W, 3]`` (H, W multiples of patch_size * pool) -> f32 ``[tokens, proj_dim]``."""
        cfg, t = self.cfg, self.t
        if cfg.unified:
            return self._encode_unified(rgb)
        ps, d, nh, hd = cfg.patch_size, cfg.dim, cfg.n_heads, cfg.head_dim
        hgt, wid, _ = rgb.shape
        gh, gw = hgt // ps, wid // ps
        if max(gh, gw) > cfg.n_pos or gh % cfg.pool or gw % cfg.pool:
            raise ValueError("image larger than the position tables, or its patch grid is not a multiple of the pooling kernel")
        img = (rgb.to(self.device).float() / 255.0 * 2.0 - 1.0).to(self.dtype)[: gh * ps, : gw * ps]
        patches = img.reshape(gh, ps, gw, ps, 3).permute(0, 2, 4, 1, 3).reshape(gh * gw, 3 * ps * ps)
        x = patches @ t["v.patch_embd.weight"].reshape(d, -1).t()
        if "v.patch_embd.bias" in t:
            x = x + t["v.patch_embd.bias"].to(x.dtype)
        py = torch.arange(gh, device=self.device).repeat_interleave(gw)
        px = torch.arange(gw, device=self.device).repeat(gh)
        pos = t["v.position_embd.weight"]
        x = x + pos[0][px].to(x.dtype) + pos[1][py].to(x.dtype)
        for b in range(cfg.n_blocks):
            p = f"v.blk.{b}."
            xn = self._rms(x, t[p + "ln1.weight"])
            q = self._rope2d(self._rms((xn @ t[p + "attn_q.weight"].t()).reshape(-1, nh, hd), t[p + "attn_q_norm.weight"]), px, py)
            k = self._rope2d(self._rms((xn @ t[p + "attn_k.weight"].t()).reshape(-1, nh, hd), t[p + "attn_k_norm.weight"]), px, py)
            v = (xn @ t[p + "attn_v.weight"].t()).reshape(-1, nh, hd)
            sc = torch.einsum("qhd,khd->hqk", q.float(), k.float())                # no 1 / sqrt(d): the head norms carry the scale
            a = torch.einsum("hqk,khd->qhd", torch.softmax(sc, dim=-1), v.float()).reshape(-1, d).to(self.dtype)
            x = x + self._rms(a @ t[p + "attn_out.weight"].t(), t[p + "attn_post_norm.weight"])
            xn = self._rms(x, t[p + "ln2.weight"])
            gate = xn @ t[p + "ffn_gate.weight"].t()
            f = (gate.float() * 0.5 * (1.0 + torch.erf(gate.float() * 0.7071067811865476))).to(self.dtype) * (xn @ t[p + "ffn_up.weight"].t())
            x = x + self._rms(f @ t[p + "ffn_down.weight"].t(), t[p + "ffn_post_norm.weight"])
        k_ = cfg.pool
        pooled = x.float().reshape(gh // k_, k_, gw // k_, k_, d).mean(dim=(1, 3)).reshape(-1, d) * (d ** 0.5)
        proj = pooled.to(self.dtype) @ t["mm.input_projection.weight"].t()
        return self._rms(proj, None).float()
