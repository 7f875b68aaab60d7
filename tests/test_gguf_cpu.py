"""GGUF reader / writer, ggml quantisers and decoders (host C++ library)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from gemm_b200.utils import gguf
from tests import reference_oracle as oracle

ALL_BLOCK_TYPES = ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "IQ1_S", "IQ1_M", "IQ2_XXS",
                   "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ4_NL", "IQ4_XS", "TQ1_0", "TQ2_0", "MXFP4", "NVFP4", "Q1_0", "F16", "BF16", "F32"]


def test_block_table_matches_format():
    expect = {"Q4_0": (32, 18), "Q4_1": (32, 20), "Q5_0": (32, 22), "Q5_1": (32, 24), "Q8_0": (32, 34), "Q2_K": (256, 84), "Q3_K": (256, 110),
              "Q4_K": (256, 144), "Q5_K": (256, 176), "Q6_K": (256, 210), "IQ2_XXS": (256, 66), "IQ2_XS": (256, 74), "IQ3_XXS": (256, 98),
              "IQ1_S": (256, 50), "IQ4_NL": (32, 18), "IQ3_S": (256, 110), "IQ2_S": (256, 82), "IQ4_XS": (256, 136), "IQ1_M": (256, 56),
              "TQ1_0": (256, 54), "TQ2_0": (256, 66), "MXFP4": (32, 17), "NVFP4": (64, 36), "Q1_0": (128, 18), "F32": (1, 4), "F16": (1, 2), "BF16": (1, 2)}
    for t, v in expect.items():
        assert gguf.block_info(t) == v
    assert len(gguf.QUANT_TYPES_24) == 24


@pytest.mark.parametrize("t,tol", [("Q8_0", 0.01), ("Q4_0", 0.12), ("Q4_1", 0.1), ("Q5_0", 0.06), ("Q5_1", 0.05), ("Q4_K", 0.09), ("Q5_K", 0.05),
                                   ("Q6_K", 0.025), ("Q2_K", 0.4), ("Q3_K", 0.2), ("IQ4_NL", 0.1), ("F16", 1e-3), ("BF16", 5e-3), ("F32", 0.0)])
def test_quantize_roundtrip(t, tol):
    torch.manual_seed(0)
    x = torch.randn(8, 512) * 0.02
    raw = gguf.quantize(x, t)
    assert raw.numel() == gguf.row_bytes(t, x.numel())
    y = gguf.dequantize(raw, t, x.numel()).reshape(x.shape)
    rel = ((x - y).norm() / x.norm()).item()
    assert rel <= tol, rel


def test_tq2_roundtrip_exact_on_ternary():
    x = torch.randint(-1, 2, (2, 256)).float() * 0.5
    y = gguf.dequantize(gguf.quantize(x, "TQ2_0"), "TQ2_0", x.numel()).reshape(x.shape)
    assert torch.equal(x, y)


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not present")
@pytest.mark.parametrize("t", ALL_BLOCK_TYPES)
def test_decoders_bit_exact_vs_reference(t):
    """Random block bytes (with sane fp16 scale fields) through our decoder and the reference's: identical floats."""
    ref = oracle.dequant_lib()
    rng = np.random.default_rng(1234)
    blk, nbytes = gguf.block_info(t)
    n_blocks = 64
    raw = rng.integers(0, 256, size=n_blocks * nbytes, dtype=np.uint8)
    if t == "F32":
        raw = rng.standard_normal(n_blocks).astype(np.float32).view(np.uint8)
    # keep half-precision scale fields finite: clear the top exponent bit of every 16-bit word that is an fp16 field
    fp16_fields = {"Q4_0": [0], "Q4_1": [0, 2], "Q5_0": [0], "Q5_1": [0, 2], "Q8_0": [0], "Q2_K": [80, 82], "Q3_K": [108], "Q4_K": [0, 2],
                   "Q5_K": [0, 2], "Q6_K": [208], "IQ2_XXS": [0], "IQ2_XS": [0], "IQ2_S": [0], "IQ3_XXS": [0], "IQ3_S": [0], "IQ4_NL": [0],
                   "IQ4_XS": [0], "IQ1_S": [0], "TQ1_0": [52], "TQ2_0": [64], "Q1_0": [0]}
    if t in fp16_fields:
        r2 = raw.reshape(n_blocks, nbytes)
        for off in fp16_fields[t]:
            r2[:, off + 1] &= 0x3F
    if t == "F16":
        raw.reshape(-1, 2)[:, 1] &= 0xBF
    if t == "IQ1_M":                       # its fp16 scale is scattered over the top nibbles of the four scale words
        r2 = raw.reshape(n_blocks, nbytes)
        r2[:, 55] &= 0x3F
    n = n_blocks * blk
    ours = gguf.dequantize(raw, t, n).numpy()
    theirs = np.empty(n, dtype=np.float32)
    rc = ref.dequant_row(gguf.type_id(t), raw.ctypes.data, theirs.ctypes.data, n)
    assert rc == 0 or rc == n or rc is not None
    assert np.array_equal(ours.view(np.uint32), theirs.view(np.uint32)), f"{t}: decoder differs from the reference"


def test_gguf_write_then_read(tmp_path):
    torch.manual_seed(1)
    w = gguf.GGUFWriter()
    w.add_string("general.architecture", "qwen3")
    w.add_u32("qwen3.block_count", 2)
    w.add_f32("qwen3.rope.freq_base", 1e6)
    w.add_bool("some.flag", True)
    w.add_u64("big", 2 ** 40)
    w.add_string_array("tokenizer.ggml.tokens", ["a", "b", b"\xff\xfe", "hello world"])
    w.add_array("tokenizer.ggml.token_type", [1, 1, 3, 1])
    a = torch.randn(4, 64)
    b = torch.randn(2, 3, 256)
    w.add_tensor("token_embd.weight", a, "F32")
    w.add_tensor("blk.0.ffn_gate_exps.weight", b, "Q4_K")
    w.add_tensor("blk.0.attn_q.weight", a, "Q8_0")
    path = str(tmp_path / "t.gguf")
    w.write(path)
    with gguf.GGUFFile(path) as f:
        assert f.version == 3 and f.alignment == 32
        m = f.metadata
        assert m["general.architecture"] == "qwen3" and m["qwen3.block_count"] == 2 and m["some.flag"] is True and m["big"] == 2 ** 40
        assert abs(m["qwen3.rope.freq_base"] - 1e6) < 1
        assert m["tokenizer.ggml.tokens"] == [b"a", b"b", b"\xff\xfe", b"hello world"]
        assert m["tokenizer.ggml.token_type"].tolist() == [1, 1, 3, 1]
        t = f.tensors["token_embd.weight"]
        assert t.shape == (4, 64) and t.type_name == "F32" and torch.equal(t.to_float(), a)
        t = f.tensors["blk.0.ffn_gate_exps.weight"]
        assert t.shape == (2, 3, 256) and t.type_name == "Q4_K"
        assert ((t.to_float() - b).norm() / b.norm()).item() < 0.1
        q = f.tensors["blk.0.attn_q.weight"]
        assert q.nbytes == 4 * 2 * 34 and ((q.to_float() - a).norm() / a.norm()).item() < 0.01
        # tensor data is aligned
        for t in f.tensors.values():
            assert t._ptr % 32 == 0


def test_gguf_rejects_garbage(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGUF" + b"\x03\x00\x00\x00" + b"\xff" * 40)
    with pytest.raises(IOError):
        gguf.GGUFFile(str(p))
    p.write_bytes(b"NOPE" + b"\x00" * 64)
    with pytest.raises(IOError):
        gguf.GGUFFile(str(p))
