"""DeepSeek-V4-Flash style engine (models/ds4f.py).  The reference's implementation needs Arm SVE and cannot run here, so the checks
are: a token-at-a-time scalar restatement of the reference's formulas (loops over heads, streams, groups, positions, written from
common/ds4f_impl.h) against the batched tensor code; the properties of the pieces (Sinkhorn, sink, window, rotation round trip, YaRN
table); chunked against token-by-token; expert parallelism on the model level."""
import math

import torch

from gemm_b200.models import ds4f


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


CFG = ds4f.DS4FConfig(n_layers=3, hidden=64, vocab=96, n_heads=4, q_head_dim=32, qk_rope_dim=8, q_lora=32, kv_lora=32, o_groups=2, o_lora=16,
                      n_experts=8, n_active=2, moe_inter=32, shared_inter=32, window_size=6, max_pos=64, original_seq_len=16, hc_iters=5,
                      compress_ratios=[0, 4, 128])


def _scalar_forward(cfg, t, toks):
    """One sequence, one token at a time, loops instead of tensor ops; fp32 weights widened from the same bf16 tensors."""
    f = {k: v.float() for k, v in t.items()}
    C, nh, HD, rd, hc, og = cfg.hidden, cfg.n_heads, cfg.q_head_dim, cfg.qk_rope_dim, cfg.hc_mult, cfg.o_groups
    half, nope = rd // 2, HD - rd
    fd = ds4f.rope_freqs(rd, cfg.rope_theta)
    fc = ds4f.rope_freqs(rd, cfg.compress_rope_theta, cfg.rope_factor, cfg.beta_fast, cfg.beta_slow, cfg.original_seq_len)

    def rms(x, w=None):
        y = x * (1.0 / math.sqrt(float((x.double() ** 2).mean()) + cfg.norm_eps))
        return y * w if w is not None else y

    def rope(v, pos, freq, inverse=False):
        v = v.clone()
        for k in range(half):
            a, b = float(v[2 * k]), float(v[2 * k + 1])
            c, s = math.cos(pos * float(freq[k])), math.sin(pos * float(freq[k]))
            if inverse:
                v[2 * k], v[2 * k + 1] = a * c + b * s, -a * s + b * c
            else:
                v[2 * k], v[2 * k + 1] = a * c - b * s, a * s + b * c
        return v

    def hc_pre(x4, fn, scale, base):
        flat = x4.reshape(-1)
        rsq = 1.0 / math.sqrt(float((flat.double() ** 2).mean()) + cfg.norm_eps)
        mixes = (fn @ flat) * rsq
        pre = torch.sigmoid(mixes[:hc] * scale[0] + base[:hc]) + cfg.hc_eps
        post = 2.0 * torch.sigmoid(mixes[hc:2 * hc] * scale[1] + base[hc:2 * hc])
        comb = torch.empty(hc, hc)
        for j in range(hc):
            for k in range(hc):
                comb[j, k] = mixes[j * hc + k + 2 * hc] * scale[2] + base[j * hc + k + 2 * hc]
        for j in range(hc):
            comb[j] = torch.softmax(comb[j], 0) + cfg.hc_eps
        for k in range(hc):
            comb[:, k] = comb[:, k] / (comb[:, k].sum() + cfg.hc_eps)
        for _ in range(cfg.hc_iters - 1):
            for j in range(hc):
                comb[j] = comb[j] / (comb[j].sum() + cfg.hc_eps)
            for k in range(hc):
                comb[:, k] = comb[:, k] / (comb[:, k].sum() + cfg.hc_eps)
        y = sum(pre[k] * x4[k] for k in range(hc))
        return y, post, comb

    def hc_post(resid, fo, post, comb):
        out = torch.empty_like(resid)
        for k in range(hc):
            out[k] = post[k] * fo
            for j in range(hc):
                out[k] = out[k] + comb[j, k] * resid[j]
        return out

    def swiglu(g, u):
        g = g.clamp(max=cfg.swiglu_limit)
        return g * torch.sigmoid(g) * u.clamp(-cfg.swiglu_limit, cfg.swiglu_limit)

    caches = [[] for _ in range(cfg.n_layers)]
    logits = []
    for pos, tok in enumerate(toks):
        x4 = f["embed"][tok][None, :].repeat(hc, 1)
        for L in range(cfg.n_layers):
            p = f"l{L}."
            freq = fc if cfg.compress_ratios[L] else fd
            y, post, comb = hc_pre(x4, f[p + "hc_attn_fn"], f[p + "hc_attn_scale"], f[p + "hc_attn_base"])
            resid = x4.clone()
            hn = rms(y, f[p + "attn_norm"])
            q = (f[p + "wq_b"] @ rms(f[p + "wq_a"] @ hn, f[p + "q_norm"])).reshape(nh, HD)
            lat = rms(f[p + "wkv"] @ hn, f[p + "kv_norm"])
            lat[nope:] = rope(lat[nope:], pos, freq)
            caches[L].append(lat.to(torch.bfloat16).float())
            lo = max(0, pos - cfg.window_size + 1)
            attn = torch.zeros(nh, HD)
            for h in range(nh):
                qh = rms(q[h])
                qh[nope:] = rope(qh[nope:], pos, freq)
                s = torch.tensor([float(qh @ caches[L][j]) / math.sqrt(HD) for j in range(lo, pos + 1)])
                mx = float(s.max())
                e = torch.exp(s - mx)
                denom = math.exp(float(f[p + "attn_sink"][h]) - mx) + float(e.sum())
                out = sum((e[i] / denom) * caches[L][lo + i] for i in range(len(e)))
                out[nope:] = rope(out[nope:], pos, freq, inverse=True)
                attn[h] = out
            gin = nh * HD // og
            flat = attn.reshape(-1)
            o1 = torch.cat([f[p + "wo_a"][g * cfg.o_lora:(g + 1) * cfg.o_lora] @ flat[g * gin:(g + 1) * gin] for g in range(og)])
            x4 = hc_post(resid, f[p + "wo_b"] @ o1, post, comb)
            y, post, comb = hc_pre(x4, f[p + "hc_ffn_fn"], f[p + "hc_ffn_scale"], f[p + "hc_ffn_base"])
            resid = x4.clone()
            h2 = rms(y, f[p + "ffn_norm"])
            moe = f[p + "sh_w2"] @ swiglu(f[p + "sh_w1"] @ h2, f[p + "sh_w3"] @ h2)
            score = torch.sqrt(torch.nn.functional.softplus(f[p + "gate"] @ h2))
            pick = torch.topk(score + f[p + "gate_bias"], cfg.n_active).indices.tolist()
            tot = sum(float(score[e]) for e in pick)
            for e in pick:
                moe = moe + (float(score[e]) / tot * cfg.routed_scale) * (f[p + "ex_w2"][e] @ swiglu(f[p + "ex_w1"][e] @ h2, f[p + "ex_w3"][e] @ h2))
            x4 = hc_post(resid, moe, post, comb)
        flat = x4.reshape(-1)
        rsq = 1.0 / math.sqrt(float((flat.double() ** 2).mean()) + cfg.norm_eps)
        pre = torch.sigmoid((f["hc_head_fn"] @ flat) * rsq * f["hc_head_scale"][0] + f["hc_head_base"]) + cfg.hc_eps
        y = sum(pre[k] * x4[k] for k in range(hc))
        logits.append(f["head"] @ rms(y, f["out_norm"]))
    return torch.stack(logits)


def test_tensor_code_equals_scalar_restatement_and_chunks_equal_tokens():
    t = ds4f.random_tensors(CFG, 4)
    toks = torch.randint(0, CFG.vocab, (14,), generator=torch.Generator().manual_seed(2))
    want = _scalar_forward(CFG, t, toks.tolist())
    model = ds4f.DS4FModel(CFG, t)
    model.reset(1, 32)
    got = torch.cat([model.forward(toks[None, :9], all_logits=True), model.forward(toks[None, 9:], all_logits=True)], dim=1)[0]
    assert _rel(got, want) < 2e-4, _rel(got, want)
    assert (got.argmax(-1) == want.argmax(-1)).all()
    one = ds4f.DS4FModel(CFG, t)
    one.reset(1, 32)
    step = torch.cat([one.forward(toks[None, i: i + 1], all_logits=True) for i in range(14)], dim=1)[0]
    assert _rel(step, got) < 1e-4


def test_pieces():
    # Sinkhorn: comb ends close to doubly stochastic, pre in (0, 1), post in (0, 2)
    g = torch.Generator().manual_seed(0)
    hc = 4
    mixes = torch.randn(3, 5, (2 + hc) * hc, generator=g)
    pre, post, comb = ds4f.sinkhorn(mixes, torch.tensor([1.0, 0.7, 1.3]), torch.randn((2 + hc) * hc, generator=g) * 0.3, hc, 20, 1e-6)
    assert comb.shape == (3, 5, hc, hc) and (comb > 0).all()
    assert (comb.sum(-1) - 1).abs().max() < 1e-3 and (comb.sum(-2) - 1).abs().max() < 1e-3
    assert (pre > 0).all() and (pre < 1.001).all() and (post > 0).all() and (post < 2).all()
    # YaRN: off -> plain frequencies; on -> high frequencies kept, low ones divided by the factor
    plain = ds4f.rope_freqs(64, 1e4)
    assert torch.allclose(plain, 1.0 / 1e4 ** (torch.arange(32, dtype=torch.float64) * 2 / 64))
    yarn = ds4f.rope_freqs(64, 1.6e5, 16, 32, 1, 65536)
    base = ds4f.rope_freqs(64, 1.6e5)
    assert torch.allclose(yarn[0], base[0]) and torch.allclose(yarn[-1], base[-1] / 16) and (yarn <= base + 1e-18).all()
    # rotation and its inverse; only the last qk_rope_dim features move
    m = ds4f.DS4FModel(CFG, ds4f.random_tensors(CFG, 1))
    x = torch.randn(2, 3, 4, CFG.q_head_dim, generator=g)
    pos = torch.tensor([5, 6, 7])
    r = m._rot(x, pos, m.freq_comp)
    assert torch.equal(r[..., :-CFG.qk_rope_dim], x[..., :-CFG.qk_rope_dim]) and _rel(r, x) > 1e-2
    assert _rel(m._rot(r, pos, m.freq_comp, inverse=True), x) < 1e-6


def test_window_and_sink():
    t = ds4f.random_tensors(CFG, 6)
    toks = torch.randint(0, CFG.vocab, (1, 16), generator=torch.Generator().manual_seed(3))
    a = ds4f.DS4FModel(CFG, t)
    a.reset(1, 32)
    base = a.forward(toks, all_logits=True)
    # a token outside every window of the last position cannot change its logits ... through attention of ONE layer; with three
    # layers of window 6 the reach is 3 * 5 = 15 positions back: position 0 is out of reach of position 15 + 1 only, so test with
    # a single layer
    cfg1 = ds4f.DS4FConfig(**{**CFG.__dict__, "n_layers": 1, "compress_ratios": [0]})
    t1 = ds4f.random_tensors(cfg1, 6)
    m1 = ds4f.DS4FModel(cfg1, t1)
    m1.reset(1, 32)
    x = m1.forward(toks, all_logits=True)
    toks2 = toks.clone()
    toks2[0, 2] = (toks2[0, 2] + 1) % cfg1.vocab
    m2 = ds4f.DS4FModel(cfg1, t1)
    m2.reset(1, 32)
    y = m2.forward(toks2, all_logits=True)
    assert _rel(y[:, 2 + cfg1.window_size:], x[:, 2 + cfg1.window_size:]) < 1e-6 and _rel(y[:, 2], x[:, 2]) > 1e-3
    # a very negative sink is plain softmax; a large one drains the attention output
    tl = dict(t1)
    tl["l0.attn_sink"] = torch.full((cfg1.n_heads,), -60.0)
    th = dict(t1)
    th["l0.attn_sink"] = torch.full((cfg1.n_heads,), 60.0)
    lo = ds4f.DS4FModel(cfg1, tl)
    lo.reset(1, 32)
    hi = ds4f.DS4FModel(cfg1, th)
    hi.reset(1, 32)
    assert _rel(lo.forward(toks, all_logits=True), x) > 1e-4 and torch.isfinite(hi.forward(toks, all_logits=True)).all()
    assert torch.isfinite(base).all()


def test_expert_shards_sum_to_the_whole():
    """Two ranks' routed partial sums add up to the unsharded routed output (the all-reduce of the engine)."""
    t = ds4f.random_tensors(CFG, 8)
    full = ds4f.DS4FModel(CFG, t)
    h2 = torch.randn(1, 5, CFG.hidden, generator=torch.Generator().manual_seed(4))
    whole = full._moe("l1.", h2)
    parts = [ds4f.DS4FModel(CFG, t, ep_rank=r, ep_size=2)._moe("l1.", h2) for r in range(2)]
    # each part carries the shared expert once
    x = h2.reshape(5, -1)
    sh = (full._swiglu(x @ full.t["l1.sh_w1"].t(), x @ full.t["l1.sh_w3"].t()) @ full.t["l1.sh_w2"].t()).reshape(1, 5, -1)
    assert _rel(parts[0] + parts[1] - sh, whole) < 1e-5
