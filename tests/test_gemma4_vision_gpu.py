"""Gemma4 and the Qwen3-VL vision encoder on the GPU (bf16 tensor ops) against their fp32 CPU runs."""
import pytest
import torch

from gemm_b200.models import gemma4, vision

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float().cpu() - b.float().cpu()).norm() / (b.float().cpu().norm() + 1e-12)).item()


def test_gemma4_cuda_matches_cpu():
    cfg = gemma4.Gemma4Config(n_layers=6, hidden=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=640, head_dim_full=128, head_dim_swa=64, window=16,
                              ple_dim=32, shared_kv_layers=2, swa_pattern=[True, True, True, False, True, False], max_seq_len=128)
    t = gemma4.random_tensors(cfg, seed=2, v_proj_on_swa=False, kv_heads_full=1)
    ids = torch.randint(0, cfg.vocab, (2, 40), generator=torch.Generator().manual_seed(0))
    cpu = gemma4.Gemma4Model(cfg, t)
    cpu.reset(2, 64)
    want = torch.cat([cpu.forward(ids[:, :33], all_logits=True), cpu.forward(ids[:, 33:], all_logits=True)], dim=1)
    # fp32 on the device: the same arithmetic; bf16: weights and activations rounded through 6 layers of 4 norms each
    for dtype, tol, agree in ((torch.float32, 2e-3, 0.95), (torch.bfloat16, 0.2, 0.6)):
        tg = {k: v.to("cuda", torch.float32 if v.dim() == 1 else dtype) for k, v in t.items()}
        gpu = gemma4.Gemma4Model(cfg, tg, "cuda", dtype)
        gpu.reset(2, 64)
        got = torch.cat([gpu.forward(ids[:, :33], all_logits=True), gpu.forward(ids[:, 33:], all_logits=True)], dim=1)
        assert _rel(got, want) < tol, (dtype, _rel(got, want))
        assert (got.argmax(-1).cpu() == want.argmax(-1)).float().mean() > agree
    assert len(gpu.generate(ids[0, :10].tolist(), 4)) == 4


def test_vision_encoder_cuda_matches_cpu():
    cfg = vision.VisionConfig(n_blocks=3, dim=128, n_heads=4, ffn=256, patch_size=8, image_size=64, proj_dim=96, deepstack_layers=[0, 2])
    t = vision.random_tensors(cfg, seed=3)
    img = torch.randn(48, 64, 3, generator=torch.Generator().manual_seed(1))
    want = vision.VisionEncoder(cfg, t).encode(img)
    for dtype, tol in ((torch.float32, 2e-3), (torch.bfloat16, 0.1)):
        tg = {k: v.to("cuda", torch.float32 if v.dim() == 1 else dtype) for k, v in t.items()}
        enc = vision.VisionEncoder(cfg, tg, "cuda", dtype)
        got = enc.encode(img)
        assert got.shape == want.shape == (12, 96 * 3)
        assert _rel(got, want) < tol, (dtype, _rel(got, want))
    embeds, ds = enc.forward_inputs(got)
    assert embeds.is_cuda and ds.shape == (2, 12, 96)
