"""The engine's call sequence (paged cache, packed batches, chunked prefill + decode) on CPU tensors,
where every op runs its PyTorch reference, against the plain fp32 oracle."""
import pytest
import torch

from gemm_b200.models import reference
from gemm_b200.models.config import get_config
from gemm_b200.models.transformer import ForwardBatch, KvCache, Transformer
from gemm_b200.models.weights import synthetic_weights


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("name,fmt", [("tiny-dense", "bf16"), ("tiny-moe", "bf16"), ("tiny-qwen2", "bf16"), ("tiny-moe", "mxfp8"),
                                      ("tiny-dense", "mxfp8"), ("tiny-qwen35", "bf16"), ("tiny-qwen35moe", "bf16"), ("tiny-qwen35", "mxfp8")])
def test_prefill_then_decode_matches_oracle(name, fmt):
    torch.manual_seed(0)
    cfg = get_config(name)
    w = synthetic_weights(cfg, fmt, device="cpu", seed=1)
    page = 16
    kv = KvCache.allocate(cfg, 32, page, "cpu")
    model = Transformer(w, kv)
    lens = [23, 40]
    toks = [torch.randint(0, cfg.vocab, (n + 3,)) for n in lens]
    bt = torch.tensor([[5, 1, 7, 9], [2, 0, 11, 3]], dtype=torch.int32)
    # chunked prefill: first 10 tokens of each, then the rest
    ctx = [0, 0]
    outs = None
    for chunk in ([10, 10], [lens[0] - 10, lens[1] - 10]):
        ids = torch.cat([toks[s][ctx[s]:ctx[s] + chunk[s]] for s in range(2)])
        fb = ForwardBatch.build(chunk, ctx, ids, bt, page, cfg.n_heads, cfg.n_kv_heads, "cpu")
        outs = model.forward(fb)
        ctx = [c + q for c, q in zip(ctx, chunk)]
    tol = 3e-2 if fmt == "bf16" else 0.2      # e4m3 activations: ~4% noise per GEMM operand
    if "qwen35" in name and fmt == "bf16":
        # four layers; in the MoE variant a bf16-sized perturbation can flip a near-tied expert choice (random router weights),
        # which moves single logits rows by ~10 %: every component alone agrees with the oracle to 0.3 %
        tol = 0.15 if "moe" in name else 6e-2
    for s in range(2):
        ref = reference.reference_logits(w, toks[s][: lens[s]])[-1]
        assert _rel(outs[s], ref) < tol
    # three decode steps with the true next tokens
    for step in range(3):
        ids = torch.stack([toks[s][lens[s] + step] for s in range(2)])
        fb = ForwardBatch.build([1, 1], ctx, ids, bt, page, cfg.n_heads, cfg.n_kv_heads, "cpu")
        outs = model.forward(fb)
        ctx = [c + 1 for c in ctx]
        for s in range(2):
            ref = reference.reference_logits(w, toks[s][: lens[s] + step + 1])[-1]
            assert _rel(outs[s], ref) < tol
