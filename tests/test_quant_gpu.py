"""GPU decoders for every ggml type and the fused dequant-GEMV vs the host decoders (which are bit-exact vs the reference)."""
import numpy as np
import pytest
import torch

from gemm_b200.ops import quant
from gemm_b200.utils import gguf

pytestmark = pytest.mark.gpu
TYPES = ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "IQ1_S", "IQ1_M", "IQ2_XXS", "IQ2_XS", "IQ2_S",
         "IQ3_XXS", "IQ3_S", "IQ4_NL", "IQ4_XS", "TQ1_0", "TQ2_0", "MXFP4", "NVFP4", "Q1_0", "F16", "BF16", "F32"]
FP16_FIELDS = {"Q4_0": [0], "Q4_1": [0, 2], "Q5_0": [0], "Q5_1": [0, 2], "Q8_0": [0], "Q2_K": [80, 82], "Q3_K": [108], "Q4_K": [0, 2], "Q5_K": [0, 2],
               "Q6_K": [208], "IQ2_XXS": [0], "IQ2_XS": [0], "IQ2_S": [0], "IQ3_XXS": [0], "IQ3_S": [0], "IQ4_NL": [0], "IQ4_XS": [0], "IQ1_S": [0],
               "TQ1_0": [52], "TQ2_0": [64], "Q1_0": [0]}


def _random_blocks(t, rows, k):
    rng = np.random.default_rng(7)
    blk, nbytes = gguf.block_info(t)
    n_blocks = rows * k // blk
    if t == "F32":
        return torch.from_numpy(rng.standard_normal(n_blocks).astype(np.float32).view(np.uint8).copy())
    raw = rng.integers(0, 256, size=n_blocks * nbytes, dtype=np.uint8)
    r2 = raw.reshape(n_blocks, nbytes)
    for off in FP16_FIELDS.get(t, []):
        r2[:, off + 1] = (r2[:, off + 1] & 0x83) | 0x28          # exponent around 2^-5 .. 2^-2: finite, moderate magnitudes
    if t == "F16":
        r2[:, 1] &= 0xBF
    if t == "BF16":
        r2[:, 1] = (r2[:, 1] & 0x80) | 0x3C
    if t == "IQ1_M":
        r2[:, 55] = (r2[:, 55] & 0x8F) | 0x20
    if t == "MXFP4":
        r2[:, 0] = 120 + (r2[:, 0] & 7)
    return torch.from_numpy(raw)


@pytest.mark.parametrize("t", TYPES)
def test_dequant_kernel_matches_host_decoder(t):
    rows, k = 4, 512
    raw = _random_blocks(t, rows, k)
    ref = gguf.dequantize(raw, t, rows * k).reshape(rows, k)
    w = quant.QuantWeight(raw.cuda(), gguf.type_id(t), rows, k)
    got = w.dequantize().float().cpu()
    assert torch.equal(got, ref.to(torch.bfloat16).float()), t


@pytest.mark.parametrize("t", ["Q8_0", "Q4_K", "Q6_K", "IQ2_XXS", "IQ4_XS", "TQ1_0", "Q5_0", "F16"])
@pytest.mark.parametrize("m", [1, 5, 8, 20])
def test_linear_quant(t, m):
    torch.manual_seed(0)
    rows, k = 96, 1024
    raw = _random_blocks(t, rows, k)
    w = quant.QuantWeight(raw.cuda(), gguf.type_id(t), rows, k)
    x = (torch.randn(m, k, device="cuda") * 0.3).bfloat16()
    y = quant.linear_quant(x, w, out_dtype=torch.float32)
    wf = gguf.dequantize(raw, t, rows * k).reshape(rows, k).cuda()
    ref = x.float() @ wf.t()
    tol = 2e-3 if m <= 8 else 1.5e-2          # the large-batch path rounds the weights to bf16 first
    assert ((y - ref).norm() / (ref.norm() + 1e-9)).item() < tol
