"""Audio front end of the Gemma4 audio path: 16 kHz mono PCM -> log-mel features ``[frames, 128]`` (what the Conformer encoder
consumes).  Reference: common/gemma4_audio_mel.h:60-84 (window, filter bank), :165-185 (framing and the transform): frames of 320
samples every 160, the signal padded in front with 160 zeros, periodic Hann window, 512-point DFT magnitude (257 bins), 128
triangular HTK-mel filters on 0..8000 Hz without area normalisation, ``log(mel + 1e-3)``.

``wav_load`` reads RIFF/WAVE PCM (8 / 16 / 32-bit integer or 32-bit float, any channel count, mixed down to mono).  The Conformer
encoder itself (common/gemma4_audio_encoder.h: fixed 12 x 1024 dimensions, 2-bit QAT safetensors) is not built.
"""
from __future__ import annotations

import math
import struct
from typing import Tuple

import torch

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
