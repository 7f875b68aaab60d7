"""Gemma4 text model (PyTorch-op forward of models/gemma4.py) against the reference project's CPU engine on a GGUF file our
writer produced: sliding-window + full layers with different head sizes and KV head counts, shared-KV tail layers, V = normalised
K on layers without attn_v, per-layer embeddings, layer output scales, proportional RoPE, soft-capped logits."""
import numpy as np
import pytest
import torch

from tests import reference_oracle as oracle
from gemm_b200.models import gemma4


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _cfg(**kw):
    base = dict(n_layers=6, hidden=128, n_heads=4, n_kv_heads=2, ffn=256, vocab=320, head_dim_full=64, head_dim_swa=32, window=8, ple_dim=16,
                shared_kv_layers=2, softcap=30.0, rope_base=1e6, rope_base_swa=1e4, swa_pattern=[True, True, True, False, True, False],
                max_seq_len=64)
    base.update(kw)
    return gemma4.Gemma4Config(**base)


def test_chunked_prefill_equals_token_by_token():
    cfg = _cfg()
    t = gemma4.random_tensors(cfg, seed=3, v_proj_on_swa=False, kv_heads_full=1)
    ids = torch.randint(0, cfg.vocab, (2, 21), generator=torch.Generator().manual_seed(0))
    a = gemma4.Gemma4Model(cfg, t)
    a.reset(2, 32)
    one = torch.stack([a.forward(ids[:, i: i + 1]) for i in range(21)], dim=1)
    b = gemma4.Gemma4Model(cfg, t)
    b.reset(2, 32)
    chunks = torch.cat([b.forward(ids[:, :11], all_logits=True), b.forward(ids[:, 11:13], all_logits=True), b.forward(ids[:, 13:], all_logits=True)], dim=1)
    assert _rel(chunks, one) < 1e-5
    assert b.k_cache[0].shape[1] == cfg.window and b.k_cache[3].shape[1] == 32 and 4 not in b.k_cache     # circular / full / shared


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not present")
@pytest.mark.parametrize("variant", ["ple", "no_ple_mqa"])
def test_matches_reference_cpu_engine(tmp_path, variant):
    if variant == "ple":
        cfg = _cfg()
        t = gemma4.random_tensors(cfg, seed=5, v_proj_on_swa=False)
    else:
        cfg = _cfg(shared_kv_layers=0)
        t = gemma4.random_tensors(cfg, seed=6, ple=False, kv_heads_full=1, rope_freqs=False)
    path = str(tmp_path / "g4.gguf")
    gemma4.save_gguf(cfg, t, path, "F16")
    ref = oracle.engine_lib()
    g = ref.gguf_open(path.encode(), 1)
    assert g
    m = ref.transformer_load(g, 64)
    assert m, "the reference engine refused our gemma4 GGUF file"
    ref.transformer_set_f64_accum(m, 1)
    assert ref.ref_n_vocab(m) == cfg.vocab
    toks = torch.randint(0, cfg.vocab, (20,), generator=torch.Generator().manual_seed(1))
    want = []
    for pos, tk in enumerate(toks.tolist()):
        p = ref.transformer_forward_logits(m, tk, pos)
        want.append(torch.from_numpy(np.ctypeslib.as_array(p, shape=(cfg.vocab,)).copy()))
    want = torch.stack(want)
    model = gemma4.load_gguf(path, "cpu", torch.float32)
    model.reset(1, 64)
    got = torch.cat([model.forward(toks[None, :13], all_logits=True), model.forward(toks[None, 13:], all_logits=True)], dim=1)[0]   # 13 > window
    for pos in (0, 7, 8, 13, 19):
        assert _rel(got[pos], want[pos]) < 2e-3, (pos, _rel(got[pos], want[pos]))
    assert (got.argmax(-1) == want.argmax(-1)).float().mean() > 0.9
    # greedy generation through the public call
    out = model.generate(toks[:10].tolist(), 4)
    assert len(out) == 4


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not present")
def test_soft_token_rows_match_the_reference(tmp_path):
    """Encoder rows spliced into a prompt (text, 5 soft tokens, text) against the reference's embedding entry point."""
    cfg = _cfg()
    t = gemma4.random_tensors(cfg, seed=8, v_proj_on_swa=False)
    path = str(tmp_path / "g4.gguf")
    gemma4.save_gguf(cfg, t, path, "F16")
    ref = oracle.engine_lib()
    m = ref.transformer_load(ref.gguf_open(path.encode(), 1), 64)
    assert m
    ref.transformer_set_f64_accum(m, 1)
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(1, cfg.vocab, (12,), generator=g)
    soft = torch.randn(5, cfg.hidden, generator=g).contiguous()
    want, pos = [], 0
    for tk in toks[:4].tolist():
        p = ref.transformer_forward_logits(m, tk, pos); pos += 1
    for r in range(5):
        p = ref.transformer_forward_embd_logits(m, soft[r].data_ptr(), pos); pos += 1
        want.append(torch.from_numpy(np.ctypeslib.as_array(p, shape=(cfg.vocab,)).copy()))
    for tk in toks[4:].tolist():
        p = ref.transformer_forward_logits(m, tk, pos); pos += 1
        want.append(torch.from_numpy(np.ctypeslib.as_array(p, shape=(cfg.vocab,)).copy()))
    want = torch.stack(want)
    model = gemma4.load_gguf(path, "cpu", torch.float32)
    model.reset(1, 64)
    ids = torch.cat([toks[:4], torch.zeros(5, dtype=toks.dtype), toks[4:]])[None]
    embeds = torch.zeros(1, 17, cfg.hidden)
    embeds[0, 4:9] = soft
    mask = torch.zeros(1, 17, dtype=torch.bool)
    mask[0, 4:9] = True
    got = model.forward(ids, all_logits=True, embeds=embeds, embeds_mask=mask)[0, 4:]
    for i in (0, 4, 5, 12):
        assert _rel(got[i], want[i]) < 2e-3, (i, _rel(got[i], want[i]))
    # the public call gives the continuation of the same prompt
    first = model.generate(toks.tolist(), 3, soft=soft, soft_at=4)
    assert first[0] == int(want[-1].argmax())
