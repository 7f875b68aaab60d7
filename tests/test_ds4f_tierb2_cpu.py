"""The compressed-attention pieces of the DeepSeek-V4-Flash engine (models/ds4f.py: Hadamard rotation, FP4 rounding, the stateful
compressor, indexer scoring and top-k) against the scalar building blocks of the reference (common/ds4f_impl.h), and the model
with them switched on against itself (whole prompt, chunks, token by token) and against a token-at-a-time restatement that drives
the reference's own compressor / indexer steps."""
import ctypes
import math

import numpy as np
import pytest
import torch

from gemm_b200.models import ds4f
from tests import reference_oracle as oracle

needs_ref = pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not present")


def _p(t):
    return t.data_ptr()


def _rope_tables(freq, n):
    ang = torch.arange(n, dtype=torch.float64)[:, None] * freq[None, :]
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


def _rot(freq):
    """The model's rotation of the last ``2 * len(freq)`` features, as the Compressor expects it."""
    def rot(x, positions):
        rd = 2 * freq.numel()
        ang = positions.double()[:, None] * freq[None, :]
        cos, sin = ang.cos().float()[None, :, None, :], ang.sin().float()[None, :, None, :]
        tail = x[..., -rd:]
        a, b = tail[..., 0::2], tail[..., 1::2]
        return torch.cat([x[..., :-rd], torch.stack([a * cos - b * sin, a * sin + b * cos], -1).flatten(-2)], -1)
    return rot


@needs_ref
def test_hadamard_and_fp4_rounding_match_the_reference():
    lib = oracle.ds4f_lib()
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 128, generator=g) * torch.tensor([1e-3, 0.1, 1.0, 30.0, 1e4])[:, None]
    want = x.clone()
    for r in range(5):
        lib.ref_rotate(_p(want[r]), 128)
    assert torch.equal(ds4f.hadamard(x), want)
    # values on and around the rounding boundaries of every code, in blocks whose largest value fixes the scale
    edge = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 0.2499, 0.7501, 2.4999, 5.0001, -0.25, -2.5, -5.0, 0.0] * 2)
    y = torch.cat([x.reshape(-1, 32), edge[None], edge[None] * 0.37, torch.zeros(1, 32)])
    want = y.clone().contiguous()
    for r in range(want.shape[0]):
        lib.ref_fp4(_p(want[r]), 32, 32)
    assert torch.equal(ds4f.fp4_act_quant(y), want)


@needs_ref
@pytest.mark.parametrize("ratio,rotate", [(4, False), (4, True), (8, False)])
def test_compressor_matches_the_reference_whole_prompt_and_stepwise(ratio, rotate):
    lib = oracle.ds4f_lib()
    g = torch.Generator().manual_seed(ratio + rotate)
    dim, d, rd, n = 48, 32, 8, 37
    coff = 2 if ratio == 4 else 1
    wkv, wgate = torch.randn(coff * d, dim, generator=g) * 0.2, torch.randn(coff * d, dim, generator=g) * 0.2
    ape = torch.randn(ratio, coff * d, generator=g)
    norm_w = (1.0 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16)
    x = torch.randn(n, dim, generator=g)
    freq = ds4f.rope_freqs(rd, 1e4).float()
    rcos, rsin = _rope_tables(freq.double(), n)
    nwin = n // ratio
    want = torch.zeros(nwin, d)
    lib.ref_compress_prefill(_p(x), n, dim, d, rd, ratio, _p(wkv), _p(wgate), _p(ape), _p(norm_w), _p(rcos), _p(rsin), 1e-6, int(rotate), _p(want))
    # the reference token by token gives the same latents as its whole-prompt form
    rows = coff * ratio
    kvs, scs, out, step = torch.zeros(rows, coff * d), torch.zeros(rows, coff * d), torch.zeros(d), []
    lib.ref_compress_reset(_p(kvs), _p(scs), ratio, d)
    for pos in range(n):
        if lib.ref_compress_step(_p(x[pos]), dim, d, rd, ratio, pos, _p(wkv), _p(wgate), _p(ape), _p(norm_w), _p(rcos), _p(rsin), 1e-6, int(rotate),
                                 _p(kvs), _p(scs), _p(out)):
            step.append(out.clone())
    step = torch.stack(step)
    assert (step - want).abs().max() <= 1e-5 or rotate
    for chunks in ([n], [5, 1, 1, 9, 21], [1] * n):
        c = ds4f.Compressor(wkv, wgate, ape, norm_w, d, ratio, rd, 1e-6, rotate)
        p0 = 0
        for t in chunks:
            c.step(x[None, p0: p0 + t], p0, _rot(freq.double()))
            p0 += t
        got = c.out[0]
        assert got.shape == want.shape
        if rotate:                                  # FP4 codes: equal except where a value sits on a rounding boundary
            assert ((got - want).abs() > 1e-6).float().mean() < 0.01
        else:
            assert (got - want).abs().max() < 2e-5, (chunks, (got - want).abs().max())
    # snapshot / restore puts the state back (a rejected draft position)
    c = ds4f.Compressor(wkv, wgate, ape, norm_w, d, ratio, rd, 1e-6, rotate)
    c.step(x[None, :10], 0, _rot(freq.double()))
    snap = c.snapshot()
    c.step(x[None, 10:13].flip(1), 10, _rot(freq.double()))
    c.restore(snap)
    c.step(x[None, 10:], 10, _rot(freq.double()))
    assert ((c.out[0] - got).abs() > 1e-5).float().mean() < (0.01 if rotate else 1e-9)


@needs_ref
def test_index_scores_and_topk_match_the_reference():
    lib = oracle.ds4f_lib()
    g = torch.Generator().manual_seed(3)
    H, hd, T, k = 6, 32, 40, 7
    q, kv, w = torch.randn(H, hd, generator=g), torch.randn(T, hd, generator=g), torch.randn(H, generator=g)
    want = torch.zeros(T)
    lib.ref_index_score(_p(q), _p(kv), _p(w), H, hd, T, _p(want))
    got = ds4f.index_scores(q, kv, w)
    assert (got - want).abs().max() < 1e-4
    score = torch.randn(T, generator=g).round(decimals=1)            # rounded: plenty of ties
    for thr in (0, 3, 7, 8, 25, 40):
        sel = torch.full((k,), -2, dtype=torch.int32)
        lib.ref_index_topk(_p(score), T, thr, k, 0, _p(sel))
        valid = torch.arange(T) < thr
        mask = ds4f.index_topk(score[None], valid[None], k)[0]
        assert sorted(mask.nonzero().flatten().tolist()) == [int(v) for v in sel.tolist() if v >= 0], thr


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


CFG = ds4f.DS4FConfig(n_layers=4, hidden=64, vocab=96, n_heads=4, q_head_dim=32, qk_rope_dim=8, q_lora=32, kv_lora=32, o_groups=2, o_lora=16,
                      n_experts=8, n_active=2, moe_inter=32, shared_inter=32, window_size=6, max_pos=96, original_seq_len=16, hc_iters=5,
                      compress_ratios=[0, 4, 8, 4], tierb2=True, index_n_heads=4, index_head_dim=32, index_topk=3)


def test_model_whole_prompt_chunks_and_token_by_token_agree():
    t = ds4f.random_tensors(CFG, seed=11)
    assert "l1.idx_wq_b" in t and "l2.cmp_wkv" in t and "l2.idx_wq_b" not in t and "l0.cmp_wkv" not in t
    ids = torch.randint(0, CFG.vocab, (2, 45), generator=torch.Generator().manual_seed(1))
    a = ds4f.DS4FModel(CFG, t)
    a.reset(2, 64)
    whole = a.forward(ids, all_logits=True)
    b = ds4f.DS4FModel(CFG, t)
    b.reset(2, 64)
    chunks = torch.cat([b.forward(ids[:, :7], all_logits=True), b.forward(ids[:, 7:8], all_logits=True), b.forward(ids[:, 8:30], all_logits=True),
                        b.forward(ids[:, 30:], all_logits=True)], 1)
    c = ds4f.DS4FModel(CFG, t)
    c.reset(2, 64)
    single = torch.stack([c.forward(ids[:, i: i + 1]) for i in range(45)], 1)
    assert _rel(chunks, whole) < 1e-4 and _rel(single, whole) < 1e-4
    assert a.comp[1].out.shape[1] == 11 and a.comp[2].out.shape[1] == 5 and a.icomp[1].out.shape[1] == 11 and 2 not in a.icomp
    # the compressed term matters: without it the logits past the window differ
    off = ds4f.DS4FModel(ds4f.DS4FConfig(**{**CFG.__dict__, "tierb2": False}), t)
    off.reset(2, 64)
    plain = off.forward(ids, all_logits=True)
    assert _rel(plain[:, :3], whole[:, :3]) < 1e-5 and _rel(plain[:, 20:], whole[:, 20:]) > 1e-3


@needs_ref
@pytest.mark.parametrize("layer", [1, 2])
def test_compressed_attention_of_a_layer_against_the_reference_steps(layer):
    """One layer's attention, token at a time, from the reference's own steps: its compressor (and, at ratio 4, its indexer step
    with selection) on the inputs our layer saw, then its gathered attention over window rows + selected latents."""
    lib = oracle.ds4f_lib()
    cfg = CFG
    t = ds4f.random_tensors(cfg, seed=12)
    n = 41
    ids = torch.randint(0, cfg.vocab, (1, n), generator=torch.Generator().manual_seed(2))
    m = ds4f.DS4FModel(cfg, t)
    m.reset(1, 64)
    m.trace = {"layer": layer}
    m.forward(ids)
    tr = m.trace
    ratio, d, rd, hid = cfg.compress_ratios[layer], cfg.kv_lora, cfg.qk_rope_dim, cfg.hidden
    coff = 2 if ratio == 4 else 1
    p = f"l{layer}."
    f32 = lambda k: t[p + k].float().contiguous()
    rcos, rsin = _rope_tables(m.freq_comp.double().cpu(), 64)
    hn, q_lat, q, rows = tr["hn"][0].contiguous(), tr["q_lat"][0].contiguous(), tr["q"][0].contiguous(), tr["rows"][0].contiguous()
    wkv, wgate, ape, cnorm = f32("cmp_wkv"), f32("cmp_wgate"), f32("cmp_ape"), t[p + "cmp_norm"].contiguous()
    kvs, scs = torch.zeros(coff * ratio, coff * d), torch.zeros(coff * ratio, coff * d)
    lib.ref_compress_reset(_p(kvs), _p(scs), ratio, d)
    nslot = n // ratio
    cmp = torch.zeros(max(nslot, 1), d)
    out = torch.zeros(d)
    if ratio == 4:
        hi, ihd, k = cfg.index_n_heads, cfg.index_head_dim, cfg.index_topk
        iwq, iwp, icw, icg, ica, icn = f32("idx_wq_b"), f32("idx_wproj"), f32("idx_cmp_wkv"), f32("idx_cmp_wgate"), f32("idx_cmp_ape"), t[p + "idx_cmp_norm"].contiguous()
        ikvs, iscs = torch.zeros(2 * ratio, 2 * ihd), torch.zeros(2 * ratio, 2 * ihd)
        lib.ref_compress_reset(_p(ikvs), _p(iscs), ratio, ihd)
        idx_kv, q_scr, score_scr = torch.zeros(max(nslot, 1), ihd), torch.zeros(hi * ihd), torch.zeros(max(nslot, 1))
        sel = torch.zeros(k, dtype=torch.int32)
    sink = t[p + "attn_sink"].float().contiguous()
    worst, flips = 0.0, 0
    for pos in range(n):
        if lib.ref_compress_step(_p(hn[pos]), hid, d, rd, ratio, pos, _p(wkv), _p(wgate), _p(ape), _p(cnorm), _p(rcos), _p(rsin), cfg.norm_eps, 0,
                                 _p(kvs), _p(scs), _p(out)):
            cmp[pos // ratio] = out
        T = (pos + 1) // ratio
        if ratio == 4:
            if pos == 0:
                seed = torch.zeros(ihd)
                lib.ref_compress_step(_p(hn[0]), hid, ihd, rd, ratio, 0, _p(icw), _p(icg), _p(ica), _p(icn), _p(rcos), _p(rsin), cfg.norm_eps, 1,
                                      _p(ikvs), _p(iscs), _p(seed))
                chosen = []
            else:
                lib.ref_index_step(_p(hn[pos]), hid, _p(q_lat[pos]), cfg.q_lora, hi, ihd, rd, ratio, pos, 0, k, _p(iwq), _p(iwp), _p(icw), _p(icg), _p(ica),
                                   _p(icn), _p(rcos), _p(rsin), cfg.norm_eps, _p(ikvs), _p(iscs), _p(idx_kv), _p(q_scr), _p(score_scr), _p(sel))
                chosen = [int(v) for v in sel.tolist() if v >= 0]
        else:
            chosen = list(range(T))
        ours = tr["pick"][0, pos].nonzero().flatten().tolist()
        if sorted(ours) != sorted(chosen):                       # FP4-rounded scores can tie differently at the k-th place
            flips += 1
            continue
        lo = max(0, pos - cfg.window_size + 1)
        idxs = list(range(lo, pos + 1)) + [n + c for c in chosen]
        row = torch.tensor(idxs, dtype=torch.int32)
        kvall = torch.cat([rows, cmp]).contiguous()
        o = torch.zeros(cfg.n_heads * d)
        lib.ref_sparse_attn(_p(q[pos]), _p(kvall), _p(sink), _p(row), 1, cfg.n_heads, d, len(idxs), 1.0 / math.sqrt(d), _p(o))
        worst = max(worst, _rel(tr["attn"][0, pos].reshape(-1), o))
    assert (tr["cmp"][0] - cmp[:nslot]).abs().max() < 1e-4
    assert flips <= 2 and worst < 1e-4, (flips, worst)


def test_token_table_routing_and_mtp_generation():
    cfg = ds4f.DS4FConfig(**{**CFG.__dict__, "n_hash_layers": 2, "mtp": True})
    t = ds4f.random_tensors(cfg, seed=13)
    assert t["l0.tid2eid"].shape == (cfg.vocab, cfg.n_active) and "l0.gate_bias" not in t and "l2.gate_bias" in t and "mtp.e_proj" in t
    m = ds4f.DS4FModel(cfg, t)
    ids = torch.randint(0, cfg.vocab, (1, 9), generator=torch.Generator().manual_seed(3))
    m.reset(1, 64)
    base = m.forward(ids)
    t2 = dict(t)
    t2["l0.tid2eid"] = (t["l0.tid2eid"] + 1) % cfg.n_experts      # other experts for every token: the output moves
    m2 = ds4f.DS4FModel(cfg, t2)
    m2.reset(1, 64)
    assert _rel(m2.forward(ids), base) > 1e-4
    # MTP logits: shape, and dependence on both inputs of the fusion
    hc = m.last_hc
    a = m.mtp_predict(ids[:, 1:], hc[:, :-1], 0)
    assert a.shape == (1, 8, cfg.vocab) and torch.isfinite(a).all()
    m.reset(1, 64); m.forward(ids)
    b = m.mtp_predict((ids[:, 1:] + 1) % cfg.vocab, hc[:, :-1], 0)
    assert _rel(a, b) > 1e-4
    # self-speculative decoding returns the tokens of plain greedy decoding
    prompt = ids[0].tolist()
    want = ds4f.DS4FModel(cfg, t).generate(prompt, 12)
    got, steps = ds4f.DS4FModel(cfg, t).generate(prompt, 12, use_mtp=True)
    assert got == want and steps >= 7
    # a draft that always agrees halves the main-model steps: here the MTP call is replaced by the main model's own next token
    class AgreeingDraft(ds4f.DS4FModel):
        def mtp_predict(self, next_ids, hc_state, p0):
            if next_ids.shape[1] != 1:
                return ds4f.DS4FModel.mtp_predict(self, next_ids, hc_state, p0)
            probe = ds4f.DS4FModel(cfg, t)
            probe.reset(1, 64)
            seq = prompt + want[: p0 + 2 - len(prompt)]                  # tokens up to and including the one at position p0 + 1
            return probe.forward(torch.tensor([seq]))[:, None]
    got2, steps2 = AgreeingDraft(cfg, t).generate(prompt, 12, use_mtp=True)
    assert got2 == want and steps2 <= 7
