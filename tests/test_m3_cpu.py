"""MiniMax-M3 style engine (models/m3.py) against the reference's engine (common/m3.h, synthetic weights read out of the reference
model): dense + MSA/MoE layers, block selection beyond the dense regime, int4 KV cache; and expert parallelism on gloo ranks."""
import ctypes
import os

import numpy as np
import pytest
import torch

from tests import reference_oracle as oracle
from gemm_b200.models import m3


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


CFG = m3.M3Config(n_layers=3, n_dense_layers=1, hidden=64, vocab=96, n_heads=4, n_kv_heads=2, head_dim=32, rotary_dim=16, msa_index_dim=16,
                  msa_n_index_heads=2, msa_block_size=4, msa_topk_blocks=2, msa_init_block=1, msa_local_block=1, n_experts=8, n_active=2,
                  moe_inter=32, dense_inter=96, max_pos=64)
_WHICH = {"input_norm": 10, "post_norm": 11, "wq": 12, "wk": 13, "wv": 14, "wo": 15, "q_norm": 16, "k_norm": 17, "idx_wq": 18, "idx_wk": 19,
          "idx_q_norm": 20, "idx_k_norm": 21, "gate": 22, "gate_bias": 23, "sh_w1": 24, "sh_w3": 25, "sh_w2": 26, "ex_w1": 27, "ex_w3": 28,
          "ex_w2": 29, "ff_gate": 30, "ff_up": 31, "ff_down": 32}


def _reference_model(cfg):
    ref = oracle.m3_lib()
    v = (ctypes.c_int * 19)(cfg.n_layers, cfg.n_dense_layers, cfg.hidden, cfg.vocab, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.rotary_dim,
                            cfg.msa_index_dim, cfg.msa_n_index_heads, cfg.msa_block_size, cfg.msa_topk_blocks, cfg.msa_init_block,
                            cfg.msa_local_block, cfg.n_experts, cfg.n_active, cfg.moe_inter, cfg.dense_inter, cfg.max_pos)
    m = ref.ref_m3_new(v)
    assert m
    shapes = m3.random_tensors(cfg, 0)                      # only for the names, shapes and dtypes

    def read(l, which, e, like):
        p = ref.ref_m3_tensor(m, l, which, e)
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
@pytest.mark.parametrize("int4", [False, True])
def test_matches_reference_engine(int4):
    os.environ["M3_INT4_KV"] = "1" if int4 else "0"
    try:
        ref, m, t = _reference_model(CFG)
    finally:
        os.environ.pop("M3_INT4_KV", None)
    n_tok = 40                                              # 10 blocks of 4: well beyond init + local + top-2 = 4 blocks
    toks = torch.randint(0, CFG.vocab, (n_tok,), generator=torch.Generator().manual_seed(1))
    want = torch.empty(n_tok, CFG.vocab)
    for pos, tk in enumerate(toks.tolist()):
        buf = np.empty(CFG.vocab, dtype=np.float32)
        ref.ref_m3_forward(m, tk, pos, buf.ctypes.data)
        want[pos] = torch.from_numpy(buf)
    model = m3.M3Model(CFG, t, int4_kv=int4)
    model.reset(1, 64)
    got = torch.cat([model.forward(toks[None, :13], all_logits=True), model.forward(toks[None, 13:14], all_logits=True),
                     model.forward(toks[None, 14:], all_logits=True)], dim=1)[0]
    worst = max(_rel(got[p], want[p]) for p in range(n_tok))
    assert worst < (5e-2 if int4 else 5e-3), worst                  # int4: a near-tie in the block ranking may pick another block
    assert (got.argmax(-1) == want.argmax(-1)).float().mean() > (0.9 if int4 else 0.97)
    if int4:
        full = m3.M3Model(CFG, t)
        full.reset(1, 64)
        assert model.kv_bytes() * 3 < full.kv_bytes()


def test_msa_selects_blocks_and_dense_regime():
    t = m3.random_tensors(CFG, 3)
    toks = torch.randint(0, CFG.vocab, (1, 40), generator=torch.Generator().manual_seed(2))
    a = m3.M3Model(CFG, t)
    a.reset(1, 64)
    sparse = a.forward(toks, all_logits=True)
    b = m3.M3Model(CFG, t, msa=False)
    b.reset(1, 64)
    dense = b.forward(toks, all_logits=True)
    keep_tokens = (CFG.msa_topk_blocks + CFG.msa_local_block + CFG.msa_init_block) * CFG.msa_block_size
    assert _rel(sparse[:, :keep_tokens], dense[:, :keep_tokens]) < 1e-6          # while every block is kept the two agree
    assert _rel(sparse[:, -1], dense[:, -1]) > 1e-4                                # later tokens attend a subset
    one = m3.M3Model(CFG, t)
    one.reset(1, 64)
    step = torch.cat([one.forward(toks[:, i: i + 1], all_logits=True) for i in range(40)], dim=1)
    assert _rel(step, sparse) < 1e-4                                               # chunked == token by token
