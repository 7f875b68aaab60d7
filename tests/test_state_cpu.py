"""Inference-state checkpoints and the weight stager (CPU)."""
import json

import pytest
import torch

from gemm_b200.models.config import get_config
from gemm_b200.models.weights import RandomSource, build_weights, synthetic_weights
from gemm_b200.serve.engine import Engine, SamplingParams
from gemm_b200.utils import checkpoint, stage


def test_kv_state_roundtrip_and_validation(tmp_path):
    torch.manual_seed(0)
    cfg = get_config("tiny-dense")
    w = synthetic_weights(cfg, "bf16", device="cpu", seed=1)
    prompts = [torch.randint(0, cfg.vocab, (n,), dtype=torch.int32) for n in (19, 7)]
    a = Engine(w, max_batch=2, max_seq_len=64, page_size=16)
    first = a._sample(a.prefill(prompts, reserve=8), SamplingParams(), 0)
    path = str(tmp_path / "state.gbkv")
    checkpoint.save_state(a, path, first)
    a.begin_decode(first, SamplingParams(), 6, use_graph=False)
    ref = [a.decode_step().clone() for _ in range(4)]
    b = Engine(w, max_batch=2, max_seq_len=64, page_size=16, num_pages=20)      # different page pool -> different page ids
    b.pages.alloc(3)
    nxt = checkpoint.load_state(b, path)
    assert torch.equal(nxt, first.cpu().to(torch.int32)) and b.seq_len == [19, 7]
    b.begin_decode(nxt, SamplingParams(), 6, use_graph=False)
    got = [b.decode_step().clone() for _ in range(4)]
    assert all(torch.equal(x, y) for x, y in zip(ref, got))
    # mismatching model and truncated file are rejected
    other = Engine(synthetic_weights(get_config("tiny-moe"), "bf16", device="cpu"), max_batch=2, max_seq_len=64, page_size=16)
    with pytest.raises(ValueError):
        checkpoint.load_state(other, path)
    data = open(path, "rb").read()
    open(path, "wb").write(data[: len(data) // 2])
    with pytest.raises(ValueError):
        checkpoint.load_state(b, path)


def test_kv_state_q8_is_half_the_size_and_close(tmp_path):
    import os
    from gemm_b200.ops import kvquant
    torch.manual_seed(1)
    x = (torch.randn(50, 2, 128) * torch.rand(50, 2, 1) * 3).bfloat16()
    q, sc = kvquant.quantize_q8(x)
    back = kvquant.dequantize_q8(q, sc)
    assert q.dtype == torch.int8 and sc.shape == (50, 2)
    assert ((back.float() - x.float()).abs() <= x.float().abs().amax(-1, keepdim=True) / 127 * 0.51 + 1e-2 * x.float().abs()).all()
    cfg = get_config("tiny-dense")
    w = synthetic_weights(cfg, "bf16", device="cpu", seed=1)
    prompts = [torch.randint(0, cfg.vocab, (n,), dtype=torch.int32) for n in (23, 9)]
    a = Engine(w, max_batch=2, max_seq_len=64, page_size=16)
    first = a._sample(a.prefill(prompts, reserve=8), SamplingParams(), 0)
    p16, p8 = str(tmp_path / "s16.gbkv"), str(tmp_path / "s8.gbkv")
    checkpoint.save_state(a, p16, first)
    checkpoint.save_state(a, p8, first, kv_format="q8")
    assert os.path.getsize(p8) < 0.56 * os.path.getsize(p16)
    b = Engine(w, max_batch=2, max_seq_len=64, page_size=16)
    nxt = checkpoint.load_state(b, p8)
    assert torch.equal(nxt, first.cpu().to(torch.int32)) and b.seq_len == [23, 9]
    # the restored cache is the int8 rounding of the original
    for li in range(len(a.kv.k)):
        for ta, tb, sa, sb in ((a.kv.k[li], b.kv.k[li], a.seq_pages, b.seq_pages),):
            ra = torch.cat([ta[sa[s][p // 16] * 16 + p % 16].unsqueeze(0) for s, n in enumerate(a.seq_len) for p in range(n)])
            rb = torch.cat([tb[sb[s][p // 16] * 16 + p % 16].unsqueeze(0) for s, n in enumerate(b.seq_len) for p in range(n)])
            rel = (ra.float() - rb.float()).norm() / ra.float().norm()
            assert rel < 2e-2
    with pytest.raises(ValueError):
        checkpoint.save_state(a, p8, first, kv_format="q4")


@pytest.mark.parametrize("fmt", ["bf16", "mxfp8"])
def test_stage_per_rank_blobs(tmp_path, fmt):
    cfg = get_config("tiny-moe")
    src = RandomSource(cfg, seed=2)
    d = str(tmp_path / "staged")
    stage.stage(cfg, src, d, fmt, ep_size=2)
    man = json.load(open(d + "/manifest.json"))
    assert man["files"] == ["rank00.safetensors", "rank01.safetensors"]
    for r in range(2):
        w = stage.load_staged(d, r, device="cpu")
        ref = build_weights(cfg, src, fmt, "cpu", ep_rank=r, ep_size=2)
        assert w.ep_rank == r and w.layers[0].w13.groups == cfg.n_experts // 2
        assert torch.equal(w.layers[1].w13.dequantized(), ref.layers[1].w13.dequantized())
        assert torch.equal(w.layers[0].wqkv.dequantized(), ref.layers[0].wqkv.dequantized())
        assert torch.equal(w.embed, ref.embed)


def test_kv_state_of_a_hybrid_model_carries_the_recurrent_state(tmp_path):
    """Delta-Net layers have no K/V rows; their conv history and recurrent matrix per sequence go into the file instead."""
    torch.manual_seed(0)
    cfg = get_config("tiny-qwen35")
    w = synthetic_weights(cfg, "bf16", device="cpu", seed=5)
    prompts = [torch.randint(0, cfg.vocab, (n,), dtype=torch.int32) for n in (13, 6)]
    a = Engine(w, max_batch=2, max_seq_len=64, page_size=16)
    first = a._sample(a.prefill(prompts, reserve=8), SamplingParams(), 0)
    path = str(tmp_path / "hybrid.gbkv")
    checkpoint.save_state(a, path, first)
    a.begin_decode(first, SamplingParams(), 6, use_graph=False)
    ref = [a.decode_step().clone() for _ in range(4)]
    b = Engine(w, max_batch=2, max_seq_len=64, page_size=16)
    nxt = checkpoint.load_state(b, path)
    b.begin_decode(nxt, SamplingParams(), 6, use_graph=False)
    got = [b.decode_step().clone() for _ in range(4)]
    assert all(torch.equal(x, y) for x, y in zip(ref, got))
