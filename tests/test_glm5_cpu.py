"""GLM-5 style engine (models/glm5.py: MLA over a latent KV cache, block indexer with shared selections, sigmoid MoE) against the
reference's engine (common/glm5.h, synthetic weights read out of the reference model)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from tests import reference_oracle as oracle
from gemm_b200.models import glm5


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


CFG = glm5.GLM5Config(n_layers=5, n_dense_layers=1, hidden=64, vocab=96, n_heads=4, qk_nope_dim=24, qk_rope_dim=8, v_head_dim=32, q_lora=32,
                      kv_lora=16, index_dim=16, index_n_heads=2, index_topk_freq=2, msa_block_size=4, msa_topk_blocks=2, msa_init_block=1,
                      msa_local_block=1, n_experts=8, n_active=2, moe_inter=32, dense_inter=96, max_pos=64)
_WHICH = {"input_norm": 10, "post_norm": 11, "wq_a": 12, "wq_b": 13, "wkv_a": 14, "wkv_b": 15, "wo": 16, "q_a_norm": 17, "kv_a_norm": 18,
          "idx_wq": 19, "idx_wk": 20, "idx_q_norm": 21, "idx_k_norm": 22, "gate": 23, "gate_bias": 24, "sh_w1": 25, "sh_w3": 26, "sh_w2": 27,
          "ex_w1": 28, "ex_w3": 29, "ex_w2": 30, "ff_gate": 31, "ff_up": 32, "ff_down": 33}


def _reference_model(cfg):
    ref = oracle.glm5_lib()
    v = (ctypes.c_int * 22)(cfg.n_layers, cfg.n_dense_layers, cfg.hidden, cfg.vocab, cfg.n_heads, cfg.qk_nope_dim, cfg.qk_rope_dim, cfg.v_head_dim,
                            cfg.q_lora, cfg.kv_lora, cfg.index_dim, cfg.index_n_heads, cfg.index_topk_freq, cfg.msa_block_size,
                            cfg.msa_topk_blocks, cfg.msa_init_block, cfg.msa_local_block, cfg.n_experts, cfg.n_active, cfg.moe_inter,
                            cfg.dense_inter, cfg.max_pos)
    m = ref.ref_glm5_new(v)
    assert m
    shapes = glm5.random_tensors(cfg, 0)

    def read(l, which, e, like):
        p = ref.ref_glm5_tensor(m, l, which, e)
        n = like.numel()
        if like.dtype == torch.bfloat16:
            a = np.ctypeslib.as_array(ctypes.cast(p, ctypes.POINTER(ctypes.c_uint16)), shape=(n,)).copy()
            return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16).reshape(like.shape)
        a = np.ctypeslib.as_array(ctypes.cast(p, ctypes.POINTER(ctypes.c_float)), shape=(n,)).copy()
        return torch.from_numpy(a).reshape(like.shape)

    t = {"embed": read(0, 0, 0, shapes["embed"]), "head": read(0, 1, 0, shapes["head"]), "out_norm": read(0, 2, 0, shapes["out_norm"])}
    for name, like in shapes.items():
        if not name.startswith("l"):
            continue
        li, key = int(name[1:name.index(".")]), name[name.index(".") + 1:]
        if key.startswith("ex_w"):
            t[name] = torch.stack([read(li, _WHICH[key], e, like[e]) for e in range(cfg.n_experts)])
        else:
            t[name] = read(li, _WHICH[key], 0, like)
    return ref, m, t


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not present")
@pytest.mark.parametrize("mode", ["dense", "indexer", "int4"])
def test_matches_reference_engine(mode):
    env = {"GLM5_MSA": "1" if mode == "indexer" else "0", "GLM5_INT4_KV": "1" if mode == "int4" else "0"}
    os.environ.update(env)
    try:
        ref, m, t = _reference_model(CFG)
        n_tok = 44                                          # 11 blocks of 4; 44 >= 32 cached rows also takes the reference's absorbed form
        toks = torch.randint(0, CFG.vocab, (n_tok,), generator=torch.Generator().manual_seed(1))
        want = torch.empty(n_tok, CFG.vocab)
        for pos, tk in enumerate(toks.tolist()):
            buf = np.empty(CFG.vocab, dtype=np.float32)
            ref.ref_glm5_forward(m, tk, pos, buf.ctypes.data)
            want[pos] = torch.from_numpy(buf)
    finally:
        for k in env:
            os.environ.pop(k, None)
    model = glm5.GLM5Model(CFG, t, int4_kv=(mode == "int4"), msa=(mode == "indexer"))
    model.reset(1, 64)
    got = torch.cat([model.forward(toks[None, :17], all_logits=True), model.forward(toks[None, 17:18], all_logits=True),
                     model.forward(toks[None, 18:], all_logits=True)], dim=1)[0]
    worst = max(_rel(got[p], want[p]) for p in range(n_tok))
    assert worst < (5e-2 if mode == "int4" else 5e-3), worst
    assert (got.argmax(-1) == want.argmax(-1)).float().mean() > (0.9 if mode == "int4" else 0.97)


def test_latent_cache_is_small_and_indexer_changes_late_tokens():
    t = glm5.random_tensors(CFG, 2)
    toks = torch.randint(0, CFG.vocab, (1, 44), generator=torch.Generator().manual_seed(3))
    dense = glm5.GLM5Model(CFG, t)
    dense.reset(1, 64)
    a = dense.forward(toks, all_logits=True)
    sparse = glm5.GLM5Model(CFG, t, msa=True)
    sparse.reset(1, 64)
    b = sparse.forward(toks, all_logits=True)
    keep = (CFG.msa_topk_blocks + CFG.msa_local_block + CFG.msa_init_block) * CFG.msa_block_size
    assert _rel(b[:, :keep], a[:, :keep]) < 1e-6 and _rel(b[:, -1], a[:, -1]) > 1e-4
    # the cache holds kv_lora + rope values per position and layer (plus the index keys of the MoE layers)
    per_pos = sum(v.shape[-1] for c in dense.cache for v in c.values())
    assert per_pos == CFG.n_layers * CFG.kv_cache_dim + (CFG.n_layers - CFG.n_dense_layers) * CFG.index_dim
    assert CFG.kv_cache_dim < 2 * CFG.n_heads * CFG.v_head_dim / 8


def test_checkpoint_round_trip_bf16_and_fp8(tmp_path):
    """HF-layout checkpoints under the reference loader's tensor names: bf16 reads back exactly; FP8 with 128 x 128 block scales reads
    back as the values it encodes (the model then runs on the dequantised weights); the indexer takes the query latent."""
    from gemm_b200.models import m3
    cfg = glm5.GLM5Config(**{**CFG.__dict__, "hidden": 128, "q_lora": 128, "moe_inter": 128, "dense_inter": 128})
    shapes = glm5.checkpoint_shapes(cfg)
    g = torch.Generator().manual_seed(3)
    t = {k: (((torch.rand(v.shape, generator=g) * 2 - 1) * 0.05) + (1.0 if k.endswith("norm") else 0.0)).to(v.dtype) for k, v in shapes.items()}
    assert "l2.idx_wq_b" in t and "l1.idx_wq_b" not in t and "l0.idx_wk" not in t          # layer 2 is the first MoE layer with an indexer
    toks = torch.randint(0, cfg.vocab, (1, 40), generator=g)
    base = glm5.GLM5Model(cfg, t, msa=True)
    want = base.forward(toks, all_logits=True)
    d = str(tmp_path / "bf16")
    glm5.save_checkpoint(cfg, t, d)
    m = glm5.load_checkpoint(d, msa=True)
    assert m.cfg == cfg and torch.equal(m.forward(toks, all_logits=True), want)
    d8 = str(tmp_path / "fp8")
    glm5.save_checkpoint(cfg, t, d8, fp8=True)
    from gemm_b200.models.loader import SafetensorsSource
    src = SafetensorsSource(d8)
    assert "model.layers.1.self_attn.q_a_proj.weight_scale_inv" in src.where and "model.layers.1.mlp.experts.3.down_proj.weight_scale_inv" in src.where
    del src
    m8 = glm5.load_checkpoint(d8, msa=True)
    got = m8.forward(toks, all_logits=True)
    assert _rel(m8.t["l1.wq_a"], base.t["l1.wq_a"]) < 0.05 and _rel(got[:, :8], want[:, :8]) < 0.5 and torch.isfinite(got).all()       # e4m3 keeps 3 mantissa bits
    # M3 checkpoints the same way
    c3 = m3.M3Config(n_layers=2, n_dense_layers=1, hidden=64, vocab=96, n_heads=4, n_kv_heads=2, head_dim=32, rotary_dim=16, msa_index_dim=16,
                     msa_n_index_heads=2, msa_block_size=4, msa_topk_blocks=2, n_experts=4, n_active=2, moe_inter=32, dense_inter=96, max_pos=64)
    t3 = m3.random_tensors(c3, 1)
    d3 = str(tmp_path / "m3")
    m3.save_checkpoint(c3, t3, d3)
    x = torch.randint(0, 96, (1, 20), generator=g)
    assert torch.equal(m3.load_checkpoint(d3).forward(x, all_logits=True), m3.M3Model(c3, t3).forward(x, all_logits=True))


def test_runtime_clones_share_weights_and_keep_their_own_state():
    import torch
    from gemm_b200.models import ds4f, glm5, m3
    cfg = glm5.GLM5Config(n_layers=2, n_dense_layers=1, hidden=32, vocab=120, n_heads=2, qk_nope_dim=8, qk_rope_dim=8, v_head_dim=16, q_lora=16,
                          kv_lora=8, index_dim=8, index_n_heads=2, n_experts=4, n_active=2, moe_inter=16, dense_inter=32, max_pos=64)
    a = glm5.GLM5Model(cfg, glm5.random_tensors(cfg, 3))
    b = a.clone_runtime()
    assert all(b.t[k].data_ptr() == a.t[k].data_ptr() for k in a.t)
    g = torch.Generator().manual_seed(0)
    s1, s2 = torch.randint(0, cfg.vocab, (1, 12), generator=g), torch.randint(0, cfg.vocab, (1, 9), generator=g)
    a.reset(1, 32); b.reset(1, 32)
    # interleaved steps of two different sequences on the two runtimes equal each sequence run alone
    la = [a.forward(s1[:, :5])]; lb = [b.forward(s2[:, :4])]; la.append(a.forward(s1[:, 5:])); lb.append(b.forward(s2[:, 4:]))
    alone = glm5.GLM5Model(cfg, glm5.random_tensors(cfg, 3))
    alone.reset(1, 32); wa = alone.forward(s1)
    alone.reset(1, 32); wb = alone.forward(s2)
    assert torch.allclose(la[-1], wa, atol=1e-5) and torch.allclose(lb[-1], wb, atol=1e-5) and a.pos == 12 and b.pos == 9
    # the DS4F engine's clone drops the compressor state as well
    dcfg = ds4f.DS4FConfig(n_layers=2, hidden=64, vocab=96, n_heads=4, q_head_dim=32, qk_rope_dim=8, q_lora=32, kv_lora=32, o_groups=2, o_lora=16,
                           n_experts=8, n_active=2, moe_inter=32, shared_inter=32, window_size=6, max_pos=64, original_seq_len=16, hc_iters=5,
                           compress_ratios=[0, 4], tierb2=True, index_n_heads=4, index_head_dim=32, index_topk=3)
    d = ds4f.DS4FModel(dcfg, ds4f.random_tensors(dcfg, 1))
    ids = torch.randint(0, dcfg.vocab, (1, 20), generator=g)
    d.reset(1, 32); want = d.forward(ids)
    e = d.clone_runtime()
    assert e.comp == {} and e.cache == []
    e.reset(1, 32)
    assert torch.allclose(e.forward(ids), want, atol=1e-5) and e.comp[1] is not d.comp[1]
