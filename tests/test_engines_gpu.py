"""The tensor-op engines (M3, GLM-5, DS4F styles) on the GPU: fp32 on the device equals the CPU run, bf16 stays close and finite."""
import pytest
import torch

from gemm_b200.models import ds4f, glm5, m3

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float().cpu() - b.float().cpu()).norm() / (b.float().cpu().norm() + 1e-12)).item()


def _cases():
    c3 = m3.M3Config(n_layers=3, n_dense_layers=1, hidden=128, vocab=160, n_heads=4, n_kv_heads=2, head_dim=64, rotary_dim=32, msa_index_dim=32,
                     msa_n_index_heads=2, msa_block_size=8, msa_topk_blocks=2, msa_init_block=1, msa_local_block=1, n_experts=8, n_active=2,
                     moe_inter=64, dense_inter=192, max_pos=128)
    yield "m3", lambda dev, dt, **kw: m3.M3Model(c3, m3.random_tensors(c3, 1), dev, dt, **kw), c3.vocab
    yield "m3-int4", lambda dev, dt: m3.M3Model(c3, m3.random_tensors(c3, 1), dev, dt, int4_kv=True), c3.vocab
    c5 = glm5.GLM5Config(n_layers=4, n_dense_layers=1, hidden=128, vocab=160, n_heads=4, qk_nope_dim=48, qk_rope_dim=16, v_head_dim=64, q_lora=64,
                         kv_lora=32, index_dim=32, index_n_heads=2, index_topk_freq=2, msa_block_size=8, msa_topk_blocks=2, msa_init_block=1,
                         msa_local_block=1, n_experts=8, n_active=2, moe_inter=64, dense_inter=192, max_pos=128)
    yield "glm5", lambda dev, dt: glm5.GLM5Model(c5, glm5.random_tensors(c5, 2), dev, dt, msa=True), c5.vocab
    c4 = ds4f.DS4FConfig(n_layers=3, hidden=128, vocab=160, n_heads=4, q_head_dim=64, qk_rope_dim=16, q_lora=64, kv_lora=64, o_groups=2, o_lora=32,
                         n_experts=8, n_active=2, moe_inter=64, shared_inter=64, window_size=16, max_pos=128, original_seq_len=32, hc_iters=6)
    yield "ds4f", lambda dev, dt: ds4f.DS4FModel(c4, ds4f.random_tensors(c4, 3), dev, dt), c4.vocab


@pytest.mark.parametrize("name,make,vocab", list(_cases()), ids=[c[0] for c in _cases()])
def test_device_run_matches_cpu(name, make, vocab):
    ids = torch.randint(0, vocab, (2, 60), generator=torch.Generator().manual_seed(5))
    cpu = make("cpu", torch.float32)
    cpu.reset(2, 96)
    want = torch.cat([cpu.forward(ids[:, :41], all_logits=True), cpu.forward(ids[:, 41:], all_logits=True)], dim=1)
    dev = make("cuda", torch.float32)
    dev.reset(2, 96)
    got = torch.cat([dev.forward(ids[:, :41], all_logits=True), dev.forward(ids[:, 41:], all_logits=True)], dim=1)
    # near-ties in block / expert selection may flip between devices: most positions must agree closely, all must be finite
    per_pos = torch.tensor([_rel(got[:, i], want[:, i]) for i in range(60)])
    assert torch.isfinite(got).all() and (per_pos < 2e-3).float().mean() > 0.85, per_pos
    half = make("cuda", torch.bfloat16)
    half.reset(2, 96)
    out = half.forward(ids[:, :41], all_logits=True)
    assert torch.isfinite(out).all() and _rel(out[:, :8], want[:, :8]) < 0.25
