"""Log-mel audio front end (models/audio.py) against the reference's (common/gemma4_audio_mel.h)."""
import ctypes
import struct

import numpy as np
import pytest
import torch

from tests import reference_oracle as oracle
from gemm_b200.models import audio


def _wav(path, x, ch=1):
    pcm = (x.clamp(-1, 1) * 32767).to(torch.int16)
    body = pcm.numpy().tobytes()
    with open(path, "wb") as fh:
        fh.write(b"RIFF" + struct.pack("<I", 36 + len(body)) + b"WAVE" + b"fmt " + struct.pack("<IHHIIHH", 16, 1, ch, 16000, 16000 * 2 * ch, 2 * ch, 16)
                 + b"data" + struct.pack("<I", len(body)) + body)


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not present")
def test_log_mel_and_wav_match_reference(tmp_path):
    g = torch.Generator().manual_seed(0)
    t = torch.arange(16000 * 2) / 16000.0
    x = 0.3 * torch.sin(2 * torch.pi * 440 * t) + 0.1 * torch.sin(2 * torch.pi * 3000 * t) + 0.02 * torch.randn(t.numel(), generator=g)
    got = audio.log_mel(x)
    ref = oracle.audio_mel_lib()
    fe = ref.g4a_mel_init()
    buf = np.ascontiguousarray(x.numpy(), dtype=np.float32)
    nf = ctypes.c_int()
    p = ref.g4a_mel_extract(fe, buf.ctypes.data, buf.size, ctypes.byref(nf))
    want = torch.from_numpy(np.ctypeslib.as_array(p, shape=(nf.value, 128)).copy())
    assert got.shape == want.shape == ((x.numel() + 160 - 321) // 160 + 1, 128)
    assert (got - want).abs().max() < 2e-3, (got - want).abs().max()
    # the same samples through a two-channel 16-bit WAV file
    path = str(tmp_path / "a.wav")
    stereo = torch.stack([x, x * 0.5], dim=1).reshape(-1)
    _wav(path, stereo, ch=2)
    mine, rate = audio.wav_load(path)
    n = ctypes.c_int()
    q = ref.g4a_wav_load(path.encode(), ctypes.byref(n))
    theirs = torch.from_numpy(np.ctypeslib.as_array(q, shape=(n.value,)).copy())
    assert rate == 16000 and mine.shape == theirs.shape and (mine - theirs).abs().max() < 1e-6


def test_short_input_gives_no_frames():
    assert audio.log_mel(torch.zeros(100)).shape == (0, 128)
    assert audio.log_mel(torch.zeros(161)).shape == (1, 128)
