"""Speculative greedy decoding: the output equals plain greedy decoding whatever the drafts are (engine on CPU tensors)."""
import torch

from gemm_b200.models.config import get_config
from gemm_b200.models.transformer import KvCache, Transformer
from gemm_b200.models.weights import synthetic_weights
from gemm_b200.serve.speculative import CallableDrafter, NgramDrafter, SpeculativeDecoder, accept_greedy


def test_accept_rule():
    assert accept_greedy([], [7]) == (0, 7)
    assert accept_greedy([1, 2, 3], [1, 2, 3, 4]) == (3, 4)
    assert accept_greedy([1, 9, 3], [1, 2, 3, 4]) == (1, 2)
    assert accept_greedy([9, 2, 3], [1, 2, 3, 4]) == (0, 1)


def test_ngram_drafter():
    d = NgramDrafter(gamma=3, max_ngram=2)
    assert d.propose([5, 6, 7, 8, 9, 5, 6]) == [7, 8, 9]
    assert d.propose([1, 2, 3]) == []
    assert d.propose([4, 4, 4, 4]) == [4]                     # latest earlier occurrence of (4, 4) is followed by one token
    assert NgramDrafter(gamma=2, max_ngram=3).propose([1, 2, 3, 9, 1, 2, 3]) == [9, 1]


def _decoder(name, drafter, page=16, n_pages=64):
    cfg = get_config(name)
    w = synthetic_weights(cfg, "bf16", device="cpu", seed=3)
    kv = KvCache.allocate(cfg, n_pages, page, "cpu")
    return cfg, SpeculativeDecoder(Transformer(w, kv), kv, page, n_pages, drafter)


def test_speculative_equals_plain_greedy_for_any_draft():
    torch.manual_seed(1)
    cfg, plain = _decoder("tiny-dense", None)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (21, 9, 40)]
    n_new = 14
    ref = plain.generate(prompts, n_new)
    assert all(len(o) == n_new for o in ref)
    assert plain.stats.verify_steps == n_new - 1 and plain.stats.drafted == 0

    # an oracle that knows the continuation: every draft is accepted, gamma + 1 tokens per step
    full = [p + o for p, o in zip(prompts, ref)]

    def oracle(tokens):
        for f in full:
            if list(tokens) == f[: len(tokens)]:
                return f[len(tokens): len(tokens) + 4]
        return []
    _, dec = _decoder("tiny-dense", CallableDrafter(oracle, gamma=4))
    assert dec.generate(prompts, n_new) == ref
    assert dec.stats.acceptance == 1.0 and dec.stats.verify_steps == 3          # 1 + 5 + 5 + 3 tokens
    assert dec.stats.produced == 3 * (n_new - 1)

    # drafts that are right for two tokens and then wrong: the wrong tail is dropped, its K/V overwritten later
    def half_right(tokens):
        good = oracle(tokens)[:2]
        return good + [(good[-1] + 1) % cfg.vocab if good else 0, 1]
    _, dec = _decoder("tiny-dense", CallableDrafter(half_right, gamma=4))
    assert dec.generate(prompts, n_new) == ref
    assert 0.0 < dec.stats.acceptance < 1.0

    # always wrong: one token per step, like plain decoding
    _, dec = _decoder("tiny-dense", CallableDrafter(lambda t: [(t[-1] + 1) % 7, 3, 3], gamma=3))
    out = dec.generate(prompts, n_new)
    assert out == ref

    # prompt lookup (whatever it finds) and a stop token
    _, dec = _decoder("tiny-dense", NgramDrafter(gamma=3))
    assert dec.generate(prompts, n_new) == ref
    stop = ref[0][5]
    _, dec = _decoder("tiny-dense", CallableDrafter(oracle, gamma=4))
    got = dec.generate(prompts, n_new, stop_token_ids=[stop])
    for g, r in zip(got, ref):
        cut = r.index(stop) + 1 if stop in r else len(r)
        assert g == r[:cut]


def test_moe_model_and_hybrid_refusal():
    torch.manual_seed(2)
    cfg, plain = _decoder("tiny-moe", None)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (12, 30)]
    ref = plain.generate(prompts, 8)
    full = [p + o for p, o in zip(prompts, ref)]

    def oracle(tokens):
        for f in full:
            if list(tokens) == f[: len(tokens)]:
                return f[len(tokens): len(tokens) + 3]
        return []
    _, dec = _decoder("tiny-moe", CallableDrafter(oracle, gamma=3))
    assert dec.generate(prompts, 8) == ref
    import pytest
    with pytest.raises(ValueError):
        _decoder("tiny-qwen35", None)


def test_draft_model():
    """A draft model equal to the target gets every draft accepted; a different one changes the step count, never the tokens."""
    from gemm_b200.serve.speculative import ModelDrafter
    torch.manual_seed(6)
    cfg, plain = _decoder("tiny-dense", None)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (18, 35, 7)]
    n_new = 13
    ref = plain.generate(prompts, n_new)

    def drafter(seed, gamma=3):
        w = synthetic_weights(cfg, "bf16", device="cpu", seed=seed)
        kv = KvCache.allocate(cfg, 64, 16, "cpu")
        return ModelDrafter(Transformer(w, kv), kv, 16, 64, gamma=gamma)

    same = drafter(3)                                       # the weights of the target
    _, dec = _decoder("tiny-dense", same)
    assert dec.generate(prompts, n_new) == ref
    assert dec.stats.acceptance == 1.0 and dec.stats.verify_steps == 3          # 1 + 4 + 4 + 4 tokens
    assert same.blocks.num_free == 64                       # the draft cache is returned
    other = drafter(11)
    _, dec = _decoder("tiny-dense", other)
    assert dec.generate(prompts, n_new) == ref
    assert dec.stats.acceptance < 1.0 and dec.stats.drafted > 0
    # a second group on the same drafter starts from clean sequences
    assert dec.generate(prompts[:2], 6) == [r[:6] for r in ref[:2]]


def test_drafts_inside_continuous_batching():
    """``LLM.set_drafter``: decode items carry draft tokens through the scheduler (reserved look-ahead positions, several
    tokens committed per step); outputs equal those of the plain engine, with fewer steps when the drafts hit."""
    from gemm_b200.serve.engine import SamplingParams
    from gemm_b200.serve.llm import LLM
    torch.manual_seed(8)
    cfg = get_config("tiny-dense")
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (19, 5, 33, 12, 27)]
    sp = SamplingParams(max_new_tokens=11)

    def make():
        return LLM.from_synthetic("tiny-dense", device="cpu", seed=3, max_running=3, max_batch_tokens=48, num_pages=32, page_size=16)
    plain = make()
    ref = plain.generate(prompts, sp)
    full = [p + o for p, o in zip(prompts, ref)]

    def oracle(tokens):
        for f in full:
            if list(tokens) == f[: len(tokens)]:
                return f[len(tokens): len(tokens) + 3]
        return []
    llm = make()
    llm.set_drafter(CallableDrafter(oracle, gamma=3))
    assert llm.generate(prompts, sp) == ref
    assert llm.spec_accepted == llm.spec_drafted > 0 and llm.steps < plain.steps
    assert llm.blocks.num_free == 32

    wrong = make()
    wrong.set_drafter(CallableDrafter(lambda t: [(t[-1] + 1) % 5, 2, 2], gamma=3))
    assert wrong.generate(prompts, sp) == ref
    assert wrong.spec_accepted < wrong.spec_drafted

    # sampled requests take no drafts; greedy ones beside them still do; streaming yields every accepted token
    mixed = make()
    mixed.set_drafter(CallableDrafter(oracle, gamma=3))
    a = mixed.add_request(prompts[0], sp)
    b = mixed.add_request(prompts[1], SamplingParams(max_new_tokens=6, temperature=0.8, top_k=20, seed=1))
    while mixed.has_work():
        mixed.step()
    assert mixed._reqs[a].out == ref[0] and len(mixed._reqs[b].out) == 6
    st = make()
    st.set_drafter(CallableDrafter(oracle, gamma=3))
    assert list(st.stream(prompts[2], sp)) == ref[2]
    st.set_drafter(None)
    assert st.generate([prompts[3]], sp) == [ref[3]]

    # a draft model (here: the target's own weights, so every draft is right), batched over the step's decode items
    from gemm_b200.serve.speculative import ModelDrafter
    wd = synthetic_weights(cfg, "bf16", device="cpu", seed=3)
    kvd = KvCache.allocate(cfg, 48, 16, "cpu")
    md = ModelDrafter(Transformer(wd, kvd), kvd, 16, 48, gamma=3)
    dm = make()
    dm.set_drafter(md)
    assert dm.generate(prompts, sp) == ref
    assert dm.spec_accepted == dm.spec_drafted > 0 and dm.steps < plain.steps
    assert md.blocks.num_free == 48                         # finished requests return their draft cache
