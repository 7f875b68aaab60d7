"""Speculative decoding on the GPU kernels: verification runs through the chunked-prefill attention path with cached context;
every produced token must be a legitimate greedy choice of the fp32 oracle (within the kernels' rounding)."""
import pytest
import torch

from gemm_b200 import _native
from gemm_b200.models import reference
from gemm_b200.models.config import get_config
from gemm_b200.models.transformer import KvCache, Transformer
from gemm_b200.models.weights import synthetic_weights
from gemm_b200.serve.speculative import CallableDrafter, SpeculativeDecoder

pytestmark = pytest.mark.gpu


def _check_greedy(w_cpu, prompt, out):
    seq = torch.tensor(list(prompt) + list(out))
    logits = reference.reference_logits(w_cpu, seq[:-1]).float()
    for j, tok in enumerate(out):
        row = logits[len(prompt) - 1 + j]
        assert row[tok] >= row.max() - 0.3 * row.std(), (j, tok, float(row[tok]), float(row.max()), float(row.std()))


@pytest.mark.parametrize("name", ["tiny-dense", "tiny-moe"])
def test_speculative_decode_on_gpu(name):
    torch.manual_seed(4)
    cfg = get_config(name)
    w_cpu = synthetic_weights(cfg, "bf16", device="cpu", seed=3)
    w = w_cpu.to("cuda")
    page, n_pages, n_new = 16, 64, 12
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (33, 70)]

    def decoder(drafter):
        kv = KvCache.allocate(cfg, n_pages, page, "cuda")
        return SpeculativeDecoder(Transformer(w, kv), kv, page, n_pages, drafter)

    plain = decoder(None)
    ref = plain.generate(prompts, n_new)
    full = [p + o for p, o in zip(prompts, ref)]

    def oracle(tokens):
        for f in full:
            if list(tokens) == f[: len(tokens)]:
                return f[len(tokens): len(tokens) + 4]
        return [1, 2]                                       # off the plain path (a near-tie went the other way): junk drafts
    dec = decoder(CallableDrafter(oracle, gamma=4))
    out = dec.generate(prompts, n_new)
    _native.assert_status_ok()
    assert all(len(o) == n_new for o in out)
    for p, o, r in zip(prompts, out, ref):
        _check_greedy(w_cpu, p, r)
        _check_greedy(w_cpu, p, o)
    assert dec.stats.verify_steps < plain.stats.verify_steps
    assert dec.stats.tokens_per_step > 2.0                  # two sequences, more than one token each per verify step
    assert any("libgb_cuda" in p for p in _native.loaded_libraries())
