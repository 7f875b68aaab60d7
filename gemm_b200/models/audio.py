"""Audio front end of the Gemma4 audio path: 16 kHz mono PCM -> log-mel features ``[frames, 128]`` (what the Conformer encoder
consumes).  Reference: common/gemma4_audio_mel.h:60-84 (window, filter bank), :165-185 (framing and the transform): frames of 320
samples every 160, the signal padded in front with 160 zeros, periodic Hann window, 512-point DFT magnitude (257 bins), 128
triangular HTK-mel filters on 0..8000 Hz without area normalisation, ``log(mel + 1e-3)``.

``wav_load`` reads RIFF/WAVE PCM (8 / 16 / 32-bit integer or 32-bit float, any channel count, mixed down to mono).

``Gemma4AudioEncoder`` is the Conformer behind it (common/gemma4_audio_encoder.h): two stride-2 3 x 3 convolutions with a channel
LayerNorm + ReLU each, an input projection, 12 blocks of half-step FFN / local causal attention with relative-position keys and
soft-capped scores / gated depthwise convolution / half-step FFN / RMSNorm, the output projection and the embedder (weightless
RMSNorm + projection into the text model's width).  Log-mel ``[frames, 128]`` in, ``[ceil(ceil(frames / 2) / 2), out]`` soft tokens
out.  ``load_checkpoint`` reads the "qat-mobile" safetensors layout (2-bit and 4-bit packed linears with one scale per output
row, F32 or BF16 norms, convolutions and projections); ``save_checkpoint`` writes it.
"""
from __future__ import annotations

import math
import os
import struct
from dataclasses import dataclass
from typing import Dict, Tuple

import torch
import torch.nn.functional as F

FRAME, HOP, FFT, BINS, N_MEL, FLOOR, RATE, FMIN, FMAX = 320, 160, 512, 257, 128, 1e-3, 16000, 0.0, 8000.0


def _hz_to_mel(f: torch.Tensor) -> torch.Tensor:
    return 2595.0 * torch.log10(1.0 + f / 700.0)


def _mel_to_hz(m: torch.Tensor) -> torch.Tensor:
    return 700.0 * (10.0 ** (m / 2595.0) - 1.0)


def mel_filters() -> torch.Tensor:
    """``[257, 128]`` triangular filters (float32, computed in float64)."""
    mel = torch.linspace(float(_hz_to_mel(torch.tensor(FMIN, dtype=torch.float64))), float(_hz_to_mel(torch.tensor(FMAX, dtype=torch.float64))),
                         N_MEL + 2, dtype=torch.float64)
    ff = _mel_to_hz(mel)
    fft_freq = torch.linspace(0.0, RATE / 2, BINS, dtype=torch.float64)
    down = -(ff[None, :-2] - fft_freq[:, None]) / (ff[1:-1] - ff[:-2])[None, :]
    up = (ff[None, 2:] - fft_freq[:, None]) / (ff[2:] - ff[1:-1])[None, :]
    return torch.minimum(down, up).clamp_min(0.0).float()


def log_mel(pcm: torch.Tensor) -> torch.Tensor:
    """``pcm`` float [n] in [-1, 1] -> float32 ``[frames, 128]``; ``frames = (n + 160 - 321) // 160 + 1``."""
    pcm = pcm.float().flatten()
    dev = pcm.device
    padded = torch.cat([torch.zeros(FRAME // 2, device=dev), pcm])
    nf = (padded.numel() - (FRAME + 1)) // HOP + 1
    if nf <= 0:
        return torch.zeros(0, N_MEL, device=dev)
    idx = torch.arange(nf, device=dev)[:, None] * HOP + torch.arange(FRAME, device=dev)[None, :]
    window = (0.5 - 0.5 * torch.cos(2.0 * math.pi * torch.arange(FRAME, dtype=torch.float64) / FRAME)).float().to(dev)
    frames = (padded[idx] * window).double()
    mag = torch.fft.rfft(frames, n=FFT).abs().float()                              # [frames, 257]
    return torch.log(mag.double() @ mel_filters().to(dev).double() + FLOOR).float()


def wav_load(path: str) -> Tuple[torch.Tensor, int]:
    """(mono float samples in [-1, 1], sample rate)."""
    with open(path, "rb") as fh:
        raw = fh.read()
    if raw[:4] != b"RIFF" or raw[8:12] != b"WAVE":
        raise ValueError("not a RIFF/WAVE file")
    pos, fmt, ch, rate, bits, data = 12, 1, 1, RATE, 16, None
    while pos + 8 <= len(raw):
        cid, size = raw[pos:pos + 4], struct.unpack("<I", raw[pos + 4:pos + 8])[0]
        body = raw[pos + 8: pos + 8 + size]
        if cid == b"fmt ":
            fmt, ch, rate = struct.unpack("<HHI", body[:8])
            bits = struct.unpack("<H", body[14:16])[0]
        elif cid == b"data":
            data = body
        pos += 8 + size + (size & 1)
    if data is None:
        raise ValueError("no data chunk")
    if bits == 16:
        x = torch.frombuffer(bytearray(data), dtype=torch.int16).double() / 32768.0
    elif bits == 32 and fmt == 3:
        x = torch.frombuffer(bytearray(data), dtype=torch.float32).double()
    elif bits == 32:
        x = torch.frombuffer(bytearray(data), dtype=torch.int32).double() / 2147483648.0
    elif bits == 8:
        x = (torch.frombuffer(bytearray(data), dtype=torch.uint8).double() - 128.0) / 128.0
    else:
        raise ValueError(f"unsupported sample format: {bits} bits, format tag {fmt}")
    n = x.numel() // max(ch, 1)
    return x[: n * ch].reshape(n, max(ch, 1)).mean(1).float(), int(rate)


# ---------------------------------------------------------------------------------------------------------------------------
# Conformer encoder
# ---------------------------------------------------------------------------------------------------------------------------

@dataclass
class Gemma4AudioConfig:
    """Dimensions of the audio tower.  The defaults are the ones the reference fixes at compile time
    (common/gemma4_audio_encoder.h:51-67); smaller ones serve tests of the tensor code alone."""
    hidden: int = 1024
    heads: int = 8
    layers: int = 12
    ffn: int = 4096
    conv_kernel: int = 5
    window: int = 12                 # a query sees itself and the window - 1 positions before it
    n_mel: int = N_MEL
    conv_channels: Tuple[int, int] = (128, 32)
    out_dim: int = 1536
    eps: float = 1e-6
    softcap: float = 50.0
    residual: float = 0.5            # weight of a half-step FFN's output

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def conv_features(self) -> int:
        """Width of a frame after both convolutions: channels x remaining mel bins."""
        w = (self.n_mel - 1) // 2 + 1
        w = (w - 1) // 2 + 1
        return w * self.conv_channels[1]


_TOWER = "model.audio_tower."
_EMBED = "model.embed_audio.embedding_projection.weight"
# name within a layer -> bits of its packed form (common/gemma4_audio_encoder.h:183-198)
_QAT_LINEARS = {"feed_forward1.ffw_layer_1.linear": 2, "feed_forward1.ffw_layer_2.linear": 2,
                "feed_forward2.ffw_layer_1.linear": 2, "feed_forward2.ffw_layer_2.linear": 2,
                "self_attn.q_proj.linear": 2, "self_attn.k_proj.linear": 2, "self_attn.v_proj.linear": 2, "self_attn.post.linear": 2,
                "lconv1d.linear_start.linear": 4, "lconv1d.linear_end.linear": 2}


def qat_unpack(packed: torch.Tensor, scale: torch.Tensor, bits: int) -> torch.Tensor:
    """Packed QAT linear -> f32 ``[out, in]``.  ``packed`` uint8 ``[out, in * bits / 8]``: value ``k`` of a byte sits at bits
    ``k * bits`` and up, stored with an offset of ``2^(bits - 1)``; int8 ``[out, in]`` is taken as is.  One scale per row
    (common/gemma4_audio_encoder.h:126-147)."""
    if packed.dtype == torch.int8:
        return packed.float() * scale.float()[:, None]
    per, zp, mask = 8 // bits, 1 << (bits - 1), (1 << bits) - 1
    shifts = torch.arange(per, device=packed.device, dtype=torch.int32) * bits
    vals = ((packed.to(torch.int32)[:, :, None] >> shifts) & mask) - zp
    return vals.reshape(packed.shape[0], -1).float() * scale.float()[:, None]


def qat_pack(w: torch.Tensor, bits: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """f32 ``[out, in]`` -> (packed uint8, f32 scale per row): round-to-nearest onto ``[-2^(bits-1), 2^(bits-1) - 1]`` with the
    smallest scale that clips neither end."""
    per, zp = 8 // bits, 1 << (bits - 1)
    scale = torch.maximum((-w).amax(1) / zp, w.amax(1) / (zp - 1)).clamp_min(1e-12).float()
    q = torch.round(w / scale[:, None]).clamp(-zp, zp - 1).to(torch.int32) + zp
    q = q.reshape(w.shape[0], -1, per)
    shifts = torch.arange(per, dtype=torch.int32) * bits
    return (q << shifts).sum(-1).to(torch.uint8).contiguous(), scale


def audio_tensor_shapes(cfg: Gemma4AudioConfig) -> Dict[str, Tuple[int, ...]]:
    """Logical (unpacked) shape of every tensor of the tower under its checkpoint name (common/gemma4_audio_encoder.h:168-204)."""
    h, f, c0, c1 = cfg.hidden, cfg.ffn, cfg.conv_channels[0], cfg.conv_channels[1]
    t = {_TOWER + "subsample_conv_projection.layer0.conv.weight": (c0, 1, 3, 3),
         _TOWER + "subsample_conv_projection.layer0.norm.weight": (c0,),
         _TOWER + "subsample_conv_projection.layer1.conv.weight": (c1, c0, 3, 3),
         _TOWER + "subsample_conv_projection.layer1.norm.weight": (c1,),
         _TOWER + "subsample_conv_projection.input_proj_linear.weight": (h, cfg.conv_features),
         _TOWER + "output_proj.weight": (cfg.out_dim, h), _TOWER + "output_proj.bias": (cfg.out_dim,),
         _EMBED: (cfg.out_dim, cfg.out_dim)}
    lin = {"feed_forward1.ffw_layer_1.linear": (f, h), "feed_forward1.ffw_layer_2.linear": (h, f),
           "feed_forward2.ffw_layer_1.linear": (f, h), "feed_forward2.ffw_layer_2.linear": (h, f),
           "self_attn.q_proj.linear": (h, h), "self_attn.k_proj.linear": (h, h), "self_attn.v_proj.linear": (h, h),
           "self_attn.post.linear": (h, h), "lconv1d.linear_start.linear": (2 * h, h), "lconv1d.linear_end.linear": (h, h)}
    for li in range(cfg.layers):
        base = f"{_TOWER}layers.{li}."
        for k, shp in lin.items():
            t[base + k + ".weight"] = shp
        for k in ("feed_forward1.pre_layer_norm", "feed_forward1.post_layer_norm", "feed_forward2.pre_layer_norm",
                  "feed_forward2.post_layer_norm", "lconv1d.pre_layer_norm", "lconv1d.conv_norm", "norm_pre_attn", "norm_post_attn",
                  "norm_out"):
            t[base + k + ".weight"] = (h,)
        t[base + "self_attn.relative_k_proj.weight"] = (h, h)
        t[base + "self_attn.per_dim_scale"] = (cfg.head_dim,)
        t[base + "lconv1d.depthwise_conv1d.weight"] = (h, cfg.conv_kernel)
    return t


def _is_qat(name: str) -> int:
    """Bits of the packed form of tensor ``name`` (0: stored unpacked)."""
    if name.startswith(_TOWER + "layers.") and name.endswith(".weight"):
        return _QAT_LINEARS.get(name.split(".", 4)[4][: -len(".weight")], 0)
    return 0


def random_audio_tensors(cfg: Gemma4AudioConfig, seed: int = 0, quantised: bool = True) -> Dict[str, torch.Tensor]:
    """Random-init f32 tensors under the checkpoint names.  With ``quantised`` the packed linears hold values their packed form
    represents exactly, so that a checkpoint written from them reads back unchanged."""
    g = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for name, shp in audio_tensor_shapes(cfg).items():
        if len(shp) == 1 and not name.endswith("bias") and not name.endswith("per_dim_scale"):
            w = 1.0 + 0.1 * torch.randn(shp, generator=g)
        elif len(shp) == 1:
            w = 0.5 * torch.randn(shp, generator=g)
        else:
            fan_in = 1
            for d in shp[1:]:
                fan_in *= d
            w = torch.randn(shp, generator=g) / math.sqrt(fan_in)
        bits = _is_qat(name)
        if bits and quantised:                                  # integer codes (both end codes in every row) times a power of two
            zp = 1 << (bits - 1)
            codes = torch.randint(-zp, zp, shp, generator=g)
            codes[:, 0], codes[:, 1] = -zp, zp - 1
            step = 2.0 ** round(math.log2(1.0 / (math.sqrt(shp[1]) * codes.float().std().item())))
            w = codes.float() * step
        out[name] = w
    return out


def save_audio_checkpoint(cfg: Gemma4AudioConfig, tensors: Dict[str, torch.Tensor], path: str) -> None:
    """Write ``path/model.safetensors`` in the layout ``load_audio_checkpoint`` and the reference's loader read."""
    from . import loader
    os.makedirs(path, exist_ok=True)
    st: Dict[str, torch.Tensor] = {}
    for name, w in tensors.items():
        bits = _is_qat(name)
        if bits:
            st[name], st[name + "_scale"] = qat_pack(w.float(), bits)
        elif name.endswith("depthwise_conv1d.weight"):
            st[name] = w.float().reshape(w.shape[0], 1, -1).contiguous()
        else:
            st[name] = w.float().contiguous()
    loader.save_safetensors(st, os.path.join(path, "model.safetensors"))


def load_audio_checkpoint(path: str, cfg: Gemma4AudioConfig = None) -> Dict[str, torch.Tensor]:
    """f32 tensors of the audio tower from a checkpoint directory (``model.safetensors`` or shards) or a single file; the other
    tensors of a multimodal checkpoint are skipped."""
    from . import loader
    cfg = cfg or Gemma4AudioConfig()
    files = [path]
    if os.path.isdir(path):
        files = sorted(os.path.join(path, f) for f in os.listdir(path) if f.endswith(".safetensors"))
    raw: Dict[str, torch.Tensor] = {}
    for f in files:
        sf = loader.SafetensorsFile(f)
        try:
            for name in sf.keys():
                if name.startswith(_TOWER) or name == _EMBED:
                    raw[name] = sf.get(name).clone()            # a copy: the views die with the mapping
        finally:
            sf.close()
    out: Dict[str, torch.Tensor] = {}
    for name, shp in audio_tensor_shapes(cfg).items():
        if name not in raw:
            raise KeyError(f"audio checkpoint: missing {name}")
        bits = _is_qat(name)
        if bits:
            if name + "_scale" not in raw:
                raise KeyError(f"audio checkpoint: missing {name}_scale")
            w = qat_unpack(raw[name], raw[name + "_scale"], bits)
        else:
            w = raw[name].float()
        if w.numel() != math.prod(shp):
            raise ValueError(f"audio checkpoint: {name} has {tuple(w.shape)}, expected {shp}")
        out[name] = w.reshape(shp)
    return out


def _rms(x: torch.Tensor, w, eps: float) -> torch.Tensor:
    y = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps)
    return (y if w is None else y * w.float()).to(x.dtype)


class Gemma4AudioEncoder:
    """The audio tower as tensor ops on any device (see the module text for its structure)."""

    def __init__(self, cfg: Gemma4AudioConfig, tensors: Dict[str, torch.Tensor], device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        keep32 = ("norm.weight", "per_dim_scale", "bias")
        self.w = {k: v.to(self.device, torch.float32 if (v.dim() == 1 or k.endswith(keep32)) else dtype) for k, v in tensors.items()}
        # sinusoid rows for distances 0 .. window: sin | cos halves over hidden / 2 timescales (common/gemma4_audio_encoder.h:307-319)
        nts = cfg.hidden // 2
        inv = torch.exp(-torch.arange(nts, dtype=torch.float64) * (math.log(10000.0) / (nts - 1))).float()
        ang = torch.arange(cfg.window + 1, dtype=torch.float32)[:, None] * inv[None, :]
        self.pos_rows = torch.cat([ang.sin(), ang.cos()], 1).to(self.device, dtype)              # [window + 1, hidden], row d = distance d

    @classmethod
    def from_checkpoint(cls, path: str, cfg: Gemma4AudioConfig = None, device="cpu", dtype=torch.float32) -> "Gemma4AudioEncoder":
        cfg = cfg or Gemma4AudioConfig()
        return cls(cfg, load_audio_checkpoint(path, cfg), device, dtype)

    # -- pieces -------------------------------------------------------------------------------------------------------
    def _lin(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return x @ self.w[name].t()

    def subsample(self, mel: torch.Tensor) -> torch.Tensor:
        """``[frames, n_mel]`` -> ``[T, hidden]`` (common/gemma4_audio_encoder.h:244-304)."""
        c, p = self.cfg, _TOWER + "subsample_conv_projection."
        x = mel.to(self.device, self.dtype)[None, None]                                          # [1, 1, frames, mel]
        for i in (0, 1):
            x = F.conv2d(x, self.w[p + f"layer{i}.conv.weight"], stride=2, padding=1)
            xc = x.float().permute(0, 2, 3, 1)                                                   # channels last
            xc = (xc - xc.mean(-1, keepdim=True)) * torch.rsqrt(xc.var(-1, unbiased=False, keepdim=True) + c.eps)
            x = torch.relu(xc * self.w[p + f"layer{i}.norm.weight"]).permute(0, 3, 1, 2).to(self.dtype)
        t = x.shape[2]
        rows = x[0].permute(1, 2, 0).reshape(t, -1)                                              # [T, mel bin x channel]
        return self._lin(rows, p + "input_proj_linear.weight")

    def _ffn(self, x: torch.Tensor, base: str) -> torch.Tensor:
        c = self.cfg
        h = self._lin(_rms(x, self.w[base + "pre_layer_norm.weight"], c.eps), base + "ffw_layer_1.linear.weight")
        h = self._lin(F.silu(h.float()).to(x.dtype), base + "ffw_layer_2.linear.weight")
        return x + c.residual * _rms(h, self.w[base + "post_layer_norm.weight"], c.eps)

    def _attention(self, x: torch.Tensor, base: str) -> torch.Tensor:
        """Causal attention over the last ``window`` positions.  A score is ``q . k`` plus ``q .`` (the projected sinusoid row of
        the distance), soft-capped by ``cap * tanh(s / cap)``.  The reference computes it per chunk of 12 queries over a context
        of 24 keys with a shift of the position term (common/gemma4_audio_encoder.h:346-391); every unmasked entry of that form
        is the one written here, since query i of a chunk and context slot i + 12 - d index row i, column 12 - d of the
        position term, the row of distance d."""
        c = self.cfg
        t, h, hd, wdw = x.shape[0], c.heads, c.head_dim, c.window
        q = self._lin(x, base + "q_proj.linear.weight").float().view(t, h, hd)
        k = self._lin(x, base + "k_proj.linear.weight").float().view(t, h, hd)
        v = self._lin(x, base + "v_proj.linear.weight").float().view(t, h, hd)
        q = q * (hd ** -0.5 / math.log(2.0)) * F.softplus(self.w[base + "per_dim_scale"])
        k = k * (math.log(1.0 + math.e) / math.log(2.0))
        rel = self._lin(self.pos_rows[:wdw], base + "relative_k_proj.weight").float().view(wdw, h, hd)    # [d, h, hd]
        idx = torch.arange(t, device=x.device)[:, None] - torch.arange(wdw, device=x.device)[None, :]   # key of query g at distance d
        ok = idx >= 0
        idx = idx.clamp_min(0)
        s = torch.einsum("thd,twhd->thw", q, k[idx]) + torch.einsum("thd,whd->thw", q, rel)
        s = torch.tanh(s / c.softcap) * c.softcap
        s = s.masked_fill(~ok[:, None, :], float("-inf"))
        o = torch.einsum("thw,twhd->thd", torch.softmax(s, -1), v[idx]).reshape(t, h * hd)
        return self._lin(o.to(x.dtype), base + "post.linear.weight")

    def _lconv(self, x: torch.Tensor, base: str) -> torch.Tensor:
        """Gated linear unit, causal depthwise convolution over time, RMSNorm, SiLU, projection; added to ``x``
        (common/gemma4_audio_encoder.h:405-432)."""
        c = self.cfg
        st = self._lin(_rms(x, self.w[base + "pre_layer_norm.weight"], c.eps), base + "linear_start.linear.weight").float()
        glu = st[:, : c.hidden] * torch.sigmoid(st[:, c.hidden:])
        dw = self.w[base + "depthwise_conv1d.weight"].float().reshape(c.hidden, 1, c.conv_kernel)
        cv = F.conv1d(F.pad(glu.t()[None], (c.conv_kernel - 1, 0)), dw, groups=c.hidden)[0].t()
        cv = F.silu(_rms(cv, self.w[base + "conv_norm.weight"], c.eps))
        return x + self._lin(cv.to(x.dtype), base + "linear_end.linear.weight")

    # -- whole tower --------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def tower(self, mel: torch.Tensor) -> torch.Tensor:
        """``[frames, n_mel]`` -> ``[T, out_dim]`` before the embedder."""
        c = self.cfg
        x = self.subsample(mel)
        for li in range(c.layers):
            b = f"{_TOWER}layers.{li}."
            x = self._ffn(x, b + "feed_forward1.")
            a = self._attention(_rms(x, self.w[b + "norm_pre_attn.weight"], c.eps), b + "self_attn.")
            x = x + _rms(a, self.w[b + "norm_post_attn.weight"], c.eps)
            x = self._lconv(x, b + "lconv1d.")
            x = self._ffn(x, b + "feed_forward2.")
            x = _rms(x, self.w[b + "norm_out.weight"], c.eps)
        return self._lin(x, _TOWER + "output_proj.weight") + self.w[_TOWER + "output_proj.bias"].to(x.dtype)

    @torch.no_grad()
    def encode(self, mel: torch.Tensor) -> torch.Tensor:
        """Soft tokens ``[T, out_dim]`` for the text model (common/gemma4_audio_encoder.h:434-479)."""
        return self._lin(_rms(self.tower(mel), None, self.cfg.eps), _EMBED)

    def encode_pcm(self, pcm: torch.Tensor) -> torch.Tensor:
        return self.encode(log_mel(pcm))
