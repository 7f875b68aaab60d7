"""The tensor-op engines with bf16 weights and activations (the GPU configuration) on CPU tensors: every product sees matching
dtypes, the result stays near the fp32 run."""
import pytest
import torch

from gemm_b200.models import gemma4, vision
from tests.test_engines_gpu import _cases, _rel


@pytest.mark.parametrize("name,make,vocab", list(_cases()), ids=[c[0] for c in _cases()])
def test_bf16_path(name, make, vocab):
    ids = torch.randint(0, vocab, (2, 40), generator=torch.Generator().manual_seed(5))
    ref = make("cpu", torch.float32)
    ref.reset(2, 64)
    want = ref.forward(ids, all_logits=True)
    half = make("cpu", torch.bfloat16)
    half.reset(2, 64)
    got = torch.cat([half.forward(ids[:, :29], all_logits=True), half.forward(ids[:, 29:], all_logits=True)], dim=1)
    assert torch.isfinite(got).all() and _rel(got[:, :8], want[:, :8]) < 0.25


def test_bf16_gemma4_and_vision():
    cfg = gemma4.Gemma4Config(n_layers=4, hidden=64, n_heads=2, n_kv_heads=1, ffn=128, vocab=200, head_dim_full=32, head_dim_swa=16, window=8,
                              ple_dim=8, shared_kv_layers=2, swa_pattern=[True, False, True, False], max_seq_len=64)
    t = gemma4.random_tensors(cfg, 1)
    tb = {k: v.to(torch.float32 if v.dim() == 1 else torch.bfloat16) for k, v in t.items()}
    m = gemma4.Gemma4Model(cfg, tb, "cpu", torch.bfloat16)
    m.reset(1, 32)
    assert torch.isfinite(m.forward(torch.randint(0, 200, (1, 12)))).all()
    vc = vision.VisionConfig(n_blocks=2, dim=64, n_heads=4, ffn=128, patch_size=4, image_size=16, proj_dim=32, deepstack_layers=[0])
    vt = {k: v.to(torch.float32 if v.dim() == 1 else torch.bfloat16) for k, v in vision.random_tensors(vc, 1).items()}
    assert torch.isfinite(vision.VisionEncoder(vc, vt, "cpu", torch.bfloat16).encode(torch.randn(16, 16, 3))).all()
    gc = vision.Gemma4VisionConfig(n_blocks=2, dim=64, n_heads=4, ffn=96, patch_size=4, image_size=24, proj_dim=40, n_pos=12)
    gt = {k: v.to(torch.float32 if v.dim() == 1 else torch.bfloat16) for k, v in vision.Gemma4VisionEncoder.random_tensors(gc, 1).items()}
    out = vision.Gemma4VisionEncoder(gc, gt, "cpu", torch.bfloat16).encode(torch.randint(0, 256, (24, 24, 3), dtype=torch.uint8))
    assert torch.isfinite(out).all()


def test_audio_and_unified_vision_encoders_in_bf16():
    """The encoders' bf16 mode (what a GPU runs) stays close to fp32 and mixes no dtypes in a product."""
    from gemm_b200.models import audio, vision
    cfg = audio.Gemma4AudioConfig(hidden=64, heads=4, layers=2, ffn=128, out_dim=48, conv_channels=(16, 8), n_mel=32)
    t = audio.random_audio_tensors(cfg, 0)
    mel = torch.randn(50, 32, generator=torch.Generator().manual_seed(1))
    a = audio.Gemma4AudioEncoder(cfg, t).encode(mel)
    b = audio.Gemma4AudioEncoder(cfg, t, dtype=torch.bfloat16).encode(mel)
    assert b.dtype == torch.bfloat16 and ((a - b.float()).norm() / a.norm()).item() < 3e-2
    c = vision.Gemma4VisionConfig(n_blocks=0, dim=64, n_heads=4, ffn=96, patch_size=4, image_size=24, proj_dim=40, n_pos=12, projector="gemma4uv")
    tt = vision.Gemma4VisionEncoder.random_tensors(c, 1)
    rgb = torch.randint(0, 256, (24, 24, 3), generator=torch.Generator().manual_seed(2), dtype=torch.uint8)
    x = vision.Gemma4VisionEncoder(c, tt).encode(rgb)
    y = vision.Gemma4VisionEncoder(c, {k: (v if v.dim() == 1 else v.bfloat16()) for k, v in tt.items()}, dtype=torch.bfloat16).encode(rgb)
    assert ((x - y).norm() / x.norm()).item() < 3e-2


def test_ds4f_compressed_attention_and_mtp_in_bf16():
    from gemm_b200.models import ds4f
    cfg = ds4f.DS4FConfig(n_layers=3, hidden=64, vocab=96, n_heads=4, q_head_dim=32, qk_rope_dim=8, q_lora=32, kv_lora=32, o_groups=2, o_lora=16,
                          n_experts=8, n_active=2, moe_inter=32, shared_inter=32, window_size=6, max_pos=96, original_seq_len=16, hc_iters=5,
                          compress_ratios=[0, 4, 8], tierb2=True, index_n_heads=4, index_head_dim=32, index_topk=3, n_hash_layers=1, mtp=True)
    t = ds4f.random_tensors(cfg, 1)
    ids = torch.randint(0, cfg.vocab, (1, 30), generator=torch.Generator().manual_seed(0))
    a = ds4f.DS4FModel(cfg, t)
    a.reset(1, 64)
    b = ds4f.DS4FModel(cfg, t, dtype=torch.bfloat16)
    b.reset(1, 64)
    la, lb = a.forward(ids), b.forward(ids)
    assert ((la - lb).norm() / la.norm()).item() < 5e-2
    assert b.mtp_predict(ids[:, 1:], b.last_hc[:, :-1], 0).shape == (1, 29, cfg.vocab)
