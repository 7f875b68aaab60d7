"""The Gemma4 audio Conformer (models/audio.py) against the reference's encoder on the same checkpoint, and its pieces."""
import ctypes
import math

import numpy as np
import pytest
import torch

from gemm_b200.models import audio
from tests import reference_oracle as oracle


def _rel(a, b):
    return ((a.double() - b.double()).norm() / (b.double().norm() + 1e-30)).item()


SMALL = audio.Gemma4AudioConfig(hidden=64, heads=4, layers=2, ffn=128, out_dim=48, conv_channels=(16, 8), n_mel=32)
SMALL128 = audio.Gemma4AudioConfig(hidden=64, heads=4, layers=2, ffn=128, out_dim=48, conv_channels=(8, 2))      # 128 mel bins, as log_mel makes


@pytest.mark.parametrize("bits", [2, 4])
def test_qat_pack_round_trip(bits):
    g = torch.Generator().manual_seed(bits)
    w = torch.randn(24, 64, generator=g)
    packed, scale = audio.qat_pack(w, bits)
    assert packed.dtype == torch.uint8 and packed.shape == (24, 64 * bits // 8)
    back = audio.qat_unpack(packed, scale, bits)
    assert ((back - w).abs() <= 0.5 * scale[:, None] * 1.0001).all()
    again = audio.qat_unpack(*audio.qat_pack(back, bits), bits)
    assert torch.equal(again, back)                                                                      # representable values survive
    # value k of a byte sits at bits k * bits and up, offset 2^(bits - 1)
    per, zp = 8 // bits, 1 << (bits - 1)
    b0 = int(packed[0, 0])
    want = [((b0 >> (k * bits)) & ((1 << bits) - 1)) - zp for k in range(per)]
    assert torch.allclose(back[0, :per], torch.tensor(want, dtype=torch.float32) * scale[0])
    i8 = torch.randint(-128, 128, (4, 16), dtype=torch.int8)
    assert torch.equal(audio.qat_unpack(i8, torch.full((4,), 0.5), 8), i8.float() * 0.5)


def test_checkpoint_round_trip(tmp_path):
    t = audio.random_audio_tensors(SMALL, seed=1)
    audio.save_audio_checkpoint(SMALL, t, str(tmp_path))
    back = audio.load_audio_checkpoint(str(tmp_path), SMALL)
    assert set(back) == set(t)
    for k in t:
        assert torch.equal(back[k].reshape(t[k].shape), t[k]), k
    mel = torch.randn(40, SMALL.n_mel, generator=torch.Generator().manual_seed(2))
    a = audio.Gemma4AudioEncoder(SMALL, t).encode(mel)
    b = audio.Gemma4AudioEncoder.from_checkpoint(str(tmp_path), SMALL).encode(mel)
    assert torch.equal(a, b) and a.shape == (10, SMALL.out_dim)
    with pytest.raises(KeyError):
        audio.load_audio_checkpoint(str(tmp_path), audio.Gemma4AudioConfig(hidden=64, heads=4, layers=3, ffn=128, out_dim=48, conv_channels=(16, 8), n_mel=32))


def test_attention_is_causal_and_local():
    """Soft token t depends on mel frames up to its own receptive field only, and not on anything further back than the windows
    of the layers reach."""
    t = audio.random_audio_tensors(SMALL, seed=3)
    enc = audio.Gemma4AudioEncoder(SMALL, t)
    mel = torch.randn(120, SMALL.n_mel, generator=torch.Generator().manual_seed(4))
    base = enc.encode(mel)
    late = mel.clone()
    late[80:] += 1.0                                            # frames >= 80 feed soft tokens >= 19 only (two stride-2 3-tap convs)
    out = enc.encode(late)
    assert torch.equal(out[:19], base[:19]) and not torch.allclose(out[22:], base[22:])
    early = mel.clone()
    early[:4] += 1.0                                            # reach per layer: 11 positions of attention + 4 of the convolution
    out = enc.encode(early)
    reach = 2 + SMALL.layers * (SMALL.window - 1 + SMALL.conv_kernel - 1)
    assert torch.allclose(out[reach + 1:], base[reach + 1:], atol=1e-6) and not torch.allclose(out[:2], base[:2])


def _chunked_attention(enc, x, base):
    """The reference's formulation (common/gemma4_audio_encoder.h:346-391): chunks of 12 queries, a context of 24 keys, the position
    term read through the shift ``idx = i * 24 + c -> (idx // 25, idx % 25)``."""
    c = enc.cfg
    t, h, hd = x.shape[0], c.heads, c.head_dim
    w = enc.w
    q = (x @ w[base + "q_proj.linear.weight"].t()).view(t, h, hd) * (hd ** -0.5 / math.log(2.0)) * torch.nn.functional.softplus(w[base + "per_dim_scale"])
    k = (x @ w[base + "k_proj.linear.weight"].t()).view(t, h, hd) * (math.log(1.0 + math.e) / math.log(2.0))
    v = (x @ w[base + "v_proj.linear.weight"].t()).view(t, h, hd)
    pos = torch.arange(12, -1, -1, dtype=torch.float32)
    nts = c.hidden // 2
    inv = torch.exp(-torch.arange(nts, dtype=torch.float64) * (math.log(10000.0) / (nts - 1))).float()
    pe = torch.cat([(pos[:, None] * inv).sin(), (pos[:, None] * inv).cos()], 1)
    relk = (pe @ w[base + "relative_k_proj.weight"].t()).view(13, h, hd)
    out = torch.zeros(t, h, hd)
    for b in range((t + 11) // 12):
        for hh in range(h):
            bd = torch.zeros(12, 13)
            for i in range(12):
                if b * 12 + i < t:
                    bd[i] = relk[:, hh] @ q[b * 12 + i, hh]
            for i in range(12):
                g = b * 12 + i
                if g >= t:
                    continue
                logits = torch.full((24,), float("-inf"))
                for cc in range(24):
                    gk = b * 12 + cc - 12
                    if not (0 <= gk < t and i < cc <= i + 12):
                        continue
                    idx = i * 24 + cc
                    r, col = idx // 25, idx % 25
                    term = bd[r, col] if (col < 13 and r < 12) else 0.0
                    s = q[g, hh] @ k[gk, hh] + term
                    logits[cc] = torch.tanh(s / c.softcap) * c.softcap
                p = torch.softmax(logits, 0)
                for cc in range(24):
                    gk = b * 12 + cc - 12
                    if p[cc] > 0 and 0 <= gk < t:
                        out[g, hh] += p[cc] * v[gk, hh]
    return out.reshape(t, h * hd) @ w[base + "post.linear.weight"].t()


def test_windowed_attention_equals_the_chunked_form():
    t = audio.random_audio_tensors(SMALL, seed=5)
    enc = audio.Gemma4AudioEncoder(SMALL, t)
    x = torch.randn(29, SMALL.hidden, generator=torch.Generator().manual_seed(6))
    base = "model.audio_tower.layers.1.self_attn."
    assert _rel(enc._attention(x, base), _chunked_attention(enc, x, base)) < 1e-5


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not available")
def test_encoder_matches_the_reference(tmp_path):
    """Full-size tower (the reference fixes its dimensions) on a random 2-bit / 4-bit checkpoint: 62 mel frames -> 16 soft tokens,
    which spans two of the reference's attention chunks."""
    cfg = audio.Gemma4AudioConfig()
    t = audio.random_audio_tensors(cfg, seed=7)
    audio.save_audio_checkpoint(cfg, t, str(tmp_path))
    mel = (torch.randn(62, cfg.n_mel, generator=torch.Generator().manual_seed(8)) * 2.0 - 3.0).contiguous()
    lib = oracle.audio_encoder_lib()
    m = lib.g4a_load_safetensors(str(tmp_path).encode())
    assert m
    nt, dim = ctypes.c_int(), ctypes.c_int()
    p = lib.g4a_encode(m, mel.data_ptr(), mel.shape[0], ctypes.byref(nt), ctypes.byref(dim))
    want = torch.from_numpy(np.ctypeslib.as_array(p, shape=(nt.value, dim.value)).copy())
    lib.ref_free(p)
    lib.g4a_free(m)
    got = audio.Gemma4AudioEncoder.from_checkpoint(str(tmp_path), cfg).encode(mel)
    assert got.shape == want.shape == (16, 1536)
    assert _rel(got, want) < 2e-4


def test_encode_audio_command(tmp_path, capsys, monkeypatch):
    """``encode-audio`` on a WAV file: mel frames and token count follow from the clip length; the checkpoint is the small one, read
    through a patched default configuration."""
    import json
    import struct
    from gemm_b200 import __main__ as cli
    audio.save_audio_checkpoint(SMALL128, audio.random_audio_tensors(SMALL128, seed=9), str(tmp_path / "ckpt"))
    n = 16000
    pcm = (torch.sin(torch.arange(n) * 2 * math.pi * 440 / 16000) * 12000).to(torch.int16)
    wav = tmp_path / "a.wav"
    with open(wav, "wb") as fh:
        fh.write(b"RIFF" + struct.pack("<I", 36 + 2 * n) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, 1, 16000, 32000, 2, 16))
        fh.write(b"data" + struct.pack("<I", 2 * n) + pcm.numpy().tobytes())
    monkeypatch.setattr(audio, "Gemma4AudioConfig", lambda: SMALL128)
    out = tmp_path / "soft.npy"
    assert cli.main(["encode-audio", "--model", str(tmp_path / "ckpt"), "--wav", str(wav), "--out", str(out), "--max-seconds", "0.5"]) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    frames = (8000 + 160 - 321) // 160 + 1
    assert line["mel_frames"] == frames and line["tokens"] == ((frames - 1) // 2) // 2 + 1 and line["features_per_token"] == 48
    assert np.load(out).shape == (line["tokens"], 48)


def test_generate_with_an_audio_clip(tmp_path, capsys, monkeypatch):
    """``generate --audio``: WAV -> mel -> soft tokens -> spliced into the Gemma4 prompt at ``<audio>``; equals the same steps by hand."""
    import json
    import struct
    from gemm_b200 import __main__ as cli
    from gemm_b200.models import gemma4
    acfg = audio.Gemma4AudioConfig(hidden=64, heads=4, layers=2, ffn=128, out_dim=64, conv_channels=(8, 2))
    audio.save_audio_checkpoint(acfg, audio.random_audio_tensors(acfg, seed=2), str(tmp_path / "aud"))
    gcfg = gemma4.Gemma4Config(n_layers=4, hidden=64, n_heads=2, n_kv_heads=1, ffn=128, vocab=96, head_dim_full=32, head_dim_swa=32, window=8, ple_dim=8,
                               shared_kv_layers=0, swa_pattern=[True, True, True, False], max_seq_len=128)
    gguf = str(tmp_path / "g4.gguf")
    gemma4.save_gguf(gcfg, gemma4.random_tensors(gcfg, seed=3), gguf, "F16")
    n = 6400
    pcm = (torch.sin(torch.arange(n) * 2 * math.pi * 330 / 16000) * 9000).to(torch.int16)
    wav = tmp_path / "a.wav"
    with open(wav, "wb") as fh:
        fh.write(b"RIFF" + struct.pack("<I", 36 + 2 * n) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, 1, 16000, 32000, 2, 16))
        fh.write(b"data" + struct.pack("<I", 2 * n) + pcm.numpy().tobytes())
    monkeypatch.setattr(audio, "Gemma4AudioConfig", lambda: acfg)
    assert cli.main(["generate", "--model", gguf, "--device", "cpu", "--ids", "--audio", str(wav), "--audio-model", str(tmp_path / "aud"),
                     "--prompt", "5 6 7 <audio> 8 9", "--max-new-tokens", "4"]) is None
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    soft = audio.Gemma4AudioEncoder.from_checkpoint(str(tmp_path / "aud"), acfg).encode_pcm(audio.wav_load(str(wav))[0])
    want = gemma4.load_gguf(gguf, "cpu", torch.float32).generate([5, 6, 7, 8, 9], 4, soft=soft, soft_at=3)
    assert line["token_ids"] == want and line["audio_tokens"] == soft.shape[0] > 5
