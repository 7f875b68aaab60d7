"""Checkpoint round trips (GGUF in several ggml types, HF safetensors incl. MXFP8) and parity of our engine with the
reference CPU engine on a GGUF file written by our writer."""
import numpy as np
import pytest
import torch

from gemm_b200.models import loader, reference
from gemm_b200.models.config import get_config
from gemm_b200.models.transformer import ForwardBatch, KvCache, Transformer
from gemm_b200.models.weights import RandomSource, build_weights
from tests import reference_oracle as oracle


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("name,wtype,tol", [("tiny-dense", "F16", 2e-3), ("tiny-moe", "Q8_0", 2e-2), ("tiny-qwen2", "Q4_K", 0.2), ("tiny-dense", "BF16", 1e-6)])
def test_gguf_checkpoint_roundtrip(tmp_path, name, wtype, tol):
    cfg = get_config(name)
    src = RandomSource(cfg, seed=3)
    path = str(tmp_path / "m.gguf")
    loader.save_gguf(cfg, src, path, wtype)
    w = loader.load_gguf(path, "bf16", device="cpu")
    w0 = build_weights(cfg, src, "bf16", device="cpu")
    assert w.cfg.n_layers == cfg.n_layers and w.cfg.hidden == cfg.hidden and w.cfg.n_experts == cfg.n_experts and w.cfg.qk_norm == cfg.qk_norm
    assert w.cfg.qkv_bias == cfg.qkv_bias and w.cfg.tie_embeddings == cfg.tie_embeddings
    for a, b in zip(w.layers, w0.layers):
        assert _rel(a.wqkv.w, b.wqkv.w) <= tol
        if cfg.is_moe:
            assert _rel(a.w13.w, b.w13.w) <= tol and _rel(a.w2.w, b.w2.w) <= tol and torch.equal(a.router, b.router)
        else:
            assert _rel(a.w_down.w, b.w_down.w) <= tol
    toks = torch.randint(0, cfg.vocab, (12,))
    assert _rel(reference.reference_logits(w, toks), reference.reference_logits(w0, toks)) <= max(10 * tol, 1e-5)


@pytest.mark.parametrize("mx", [False, True])
def test_hf_safetensors_roundtrip(tmp_path, mx):
    cfg = get_config("tiny-moe")
    src = RandomSource(cfg, seed=4)
    d = str(tmp_path / "hf")
    loader.save_hf_checkpoint(cfg, src, d, mxfp8=mx)
    cfg2 = loader.config_from_hf(d)
    assert cfg2.n_experts == cfg.n_experts and cfg2.arch == "qwen3moe" and cfg2.head_dim == cfg.head_dim
    w = loader.load_safetensors(d, "bf16", device="cpu")
    w0 = build_weights(cfg, src, "bf16", device="cpu")
    tol = 0.05 if mx else 1e-6
    assert _rel(w.layers[0].wqkv.w, w0.layers[0].wqkv.w) <= tol and _rel(w.layers[1].w13.w, w0.layers[1].w13.w) <= tol
    assert torch.equal(w.embed, w0.embed)
    if mx:
        # an MXFP8 checkpoint loaded straight into the MXFP8 run-time format reproduces the stored values exactly
        wm = loader.load_safetensors(d, "mxfp8", device="cpu")
        assert _rel(wm.layers[0].wo.dequantized(), w.layers[0].wo.w.float()) < 1e-6


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not present")
@pytest.mark.parametrize("name,wtype", [("tiny-dense", "Q8_0"), ("tiny-moe", "F16"), ("tiny-qwen2", "Q4_K"), ("tiny-qwen35:ssm", "F16"),
                                        ("tiny-qwen35:attn", "F16"), ("tiny-qwen35:mixed", "F16"), ("tiny-moe:vl", "F16"), ("tiny-qwen2:vl", "F16")])
def test_engine_matches_reference_cpu_engine(tmp_path, name, wtype):
    """The reference's own transformer.h loads the GGUF our writer produced and runs it token by token; our engine
    (loading the same file) must give the same logits up to bf16 rounding of activations."""
    if ":" in name:
        # Qwen3.5 hybrid: a stack of Delta-Net layers, a stack of gated-attention (M-RoPE) layers, and the released interleaving of
        # the two (block 0 is then a Delta-Net layer without QK-norm tensors: what a loader finds in block 0 says nothing about
        # the attention layers)
        name, kind = name.split(":")
        cfg = get_config(name)
        if kind == "vl":                                         # the vision-language variants of the text stacks: M-RoPE sections (+ DeepStack)
            cfg = cfg.with_(arch="qwen3vlmoe", mrope_sections=[24, 20, 20, 0], n_deepstack_layers=2) if cfg.is_moe else \
                cfg.with_(arch="qwen2vl", mrope_sections=[16, 24, 24, 0])
        elif kind != "mixed":
            cfg = cfg.with_(full_attention_interval=5 if kind == "ssm" else 1)
    else:
        cfg = get_config(name)
    path = str(tmp_path / "m.gguf")
    loader.save_gguf(cfg, RandomSource(cfg, seed=5), path, wtype)
    ref = oracle.engine_lib()
    g = ref.gguf_open(path.encode(), 1)
    assert g
    m = ref.transformer_load(g, 256)
    assert m, "the reference engine refused our GGUF file"
    ref.transformer_set_f64_accum(m, 1)
    assert ref.ref_n_vocab(m) == cfg.vocab
    torch.manual_seed(0)
    toks = torch.randint(0, cfg.vocab, (20,))
    ref_logits = []
    for pos, t in enumerate(toks.tolist()):
        p = ref.transformer_forward_logits(m, t, pos)
        ref_logits.append(torch.from_numpy(np.ctypeslib.as_array(p, shape=(cfg.vocab,)).copy()))
    w = loader.load_gguf(path, "bf16", device="cpu")
    if any(not cfg.is_ssm_layer(i) for i in range(cfg.n_layers)):                 # read off the attention layers, wherever they sit
        assert w.cfg.qk_norm == cfg.qk_norm and w.cfg.qkv_bias == cfg.qkv_bias
    # fp32 oracle on the loaded weights == the reference arithmetic
    ours32 = reference.reference_logits(w, toks)
    assert _rel(ours32[-1], ref_logits[-1]) < 5e-3 and _rel(ours32[5], ref_logits[5]) < 5e-3
    # the paged engine (bf16 activations)
    model = Transformer(w, KvCache.allocate(cfg, 8, 16, "cpu"))
    bt = torch.tensor([[3, 1, 0, 2]], dtype=torch.int32)
    fb = ForwardBatch.build([20], [0], toks, bt, 16, cfg.n_heads, cfg.n_kv_heads, "cpu", all_logits=True)
    ours = model.forward(fb)
    assert _rel(ours[-1], ref_logits[-1]) < 3e-2
    assert int(ours[-1].argmax()) == int(ref_logits[-1].argmax()) or _rel(ours[-1], ref_logits[-1]) < 1e-2


def test_fp8_block_scaled_and_mxfp4_checkpoints(tmp_path):
    """Dense FP8 weights with 128 x 128 f32 block scales (GLM-5 / DeepSeek-V4-Flash layout) and MXFP4 weights are read back as
    the values they encode."""
    torch.manual_seed(9)
    w = torch.randn(256, 384) * 0.05
    sc = w.reshape(2, 128, 3, 128).abs().amax(dim=(1, 3)) / 448.0
    q = (w / sc.repeat_interleave(128, 0).repeat_interleave(128, 1)).to(torch.float8_e4m3fn)
    w4 = torch.randn(64, 128) * 0.3
    p4, s4 = loader.mxfp4_quant(w4)
    path = str(tmp_path / "q.safetensors")
    loader.save_safetensors({"model.embed_tokens.weight": q, "model.embed_tokens.weight_scale_inv": sc.float(),
                             "model.norm.weight": p4, "model.norm.weight_scale": s4}, path)
    src = loader.SafetensorsSource(path)
    got = src.get("token_embd.weight", (256, 384))
    assert torch.equal(got, q.float() * sc.repeat_interleave(128, 0).repeat_interleave(128, 1))
    assert _rel(got, w) < 0.05
    got4 = src._raw("model.norm.weight")
    assert got4.shape == (64, 128) and _rel(got4, w4) < 0.15
    again = loader.mxfp4_dequant(*loader.mxfp4_quant(got4))      # representable values survive another encode / decode
    assert torch.equal(again, got4)


@pytest.mark.parametrize("wtype", ["Q4_K", "Q8_0"])
def test_gguf_blocks_are_kept_without_conversion(tmp_path, wtype):
    """``load_gguf(fmt="ggml")``: Q4_K / Q8_0 matrices stay the file's blocks (only re-ordered into tiles), tensor-parallel shards
    are cut on block boundaries, and the engine over the kept blocks equals the engine over the decoded matrices."""
    from gemm_b200.utils import gguf as G
    cfg = get_config("tiny-dense")
    src = RandomSource(cfg, seed=4)
    path = str(tmp_path / "q.gguf")
    loader.save_gguf(cfg, src, path, wtype)
    w = loader.load_gguf(path, "ggml", device="cpu")
    with G.GGUFFile(path) as f:
        for li, lw in enumerate(w.layers):
            assert lw.wqkv.is_quant and lw.wo.is_quant and lw.w_gate_up.is_quant and lw.w_down.is_quant
            file_rows = np.concatenate([np.array(f.tensors[f"blk.{li}.attn_{n}.weight"].raw()) for n in "qkv"])
            assert np.array_equal(lw.wqkv.q.blocks().reshape(-1).numpy(), file_rows)              # bit for bit the file's blocks
            down = f.tensors[f"blk.{li}.ffn_down.weight"]
            assert np.array_equal(lw.w_down.q.blocks().reshape(-1).numpy(), np.array(down.raw()))
    wf = loader.load_gguf(path, "bf16", device="cpu")
    toks = torch.randint(0, cfg.vocab, (10,))
    assert _rel(reference.reference_logits(w, toks), reference.reference_logits(wf, toks)) < 2e-2
    # two tensor-parallel shards: K ranges of the row-parallel projections fall on 256-column boundaries and add up to the matrix
    parts = [loader.load_gguf(path, "ggml", device="cpu", tp_rank=r, tp_size=2) for r in range(2)]
    for li in range(cfg.n_layers):
        full = w.layers[li].w_down.dequantized()
        got = torch.cat([p.layers[li].w_down.dequantized() for p in parts], dim=1)
        assert all(p.layers[li].w_down.k % 256 == 0 for p in parts) and torch.equal(got, full)


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not present")
def test_mrope_positions_and_deepstack_match_reference_cpu_engine(tmp_path):
    """A Qwen3-VL style text model from our GGUF file: text tokens, then image rows fed as embeddings with separate t / h / w positions
    and DeepStack slices, then text again, through the reference's embedding entry point and through ours."""
    cfg = get_config("tiny-dense").with_(arch="qwen3vl", mrope_sections=[24, 20, 20, 0], n_deepstack_layers=2)
    path = str(tmp_path / "vl.gguf")
    src = RandomSource(cfg, seed=6)
    loader.save_gguf(cfg, src, path, "F16")
    ref = oracle.engine_lib()
    m = ref.transformer_load(ref.gguf_open(path.encode(), 1), 64)
    assert m and ref.ref_n_deepstack(m) == 2
    ref.transformer_set_f64_accum(m, 1)
    h, t = cfg.hidden, 18
    ref.ref_set_ds_stride(m, 3 * h)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab, (t,), generator=g)
    vis = torch.zeros(t, dtype=torch.bool)
    vis[4:10] = True                                                # an image of 2 x 3 merged patches at t = 4
    pos3 = torch.arange(t).repeat(3, 1)
    pos3[0, 4:10] = 4
    pos3[1, 4:10] = 4 + torch.arange(6) // 3
    pos3[2, 4:10] = 4 + torch.arange(6) % 3
    pos3[:, 10:] = torch.arange(10, t) - 10 + 4 + 3
    rows = torch.randn(6, 3 * h, generator=g) * 0.05                 # main embedding | DeepStack slice 0 | slice 1
    w = loader.load_gguf(path, "bf16", device="cpu")
    want = []
    for i in range(t):
        if vis[i]:
            r = rows[i - 4].contiguous()
            p = ref.transformer_forward_embd_logits_pos(m, r.data_ptr(), i, int(pos3[0, i]), int(pos3[1, i]), int(pos3[2, i]))
        elif i < 4:
            p = ref.transformer_forward_logits(m, int(ids[i]), i)
        else:                                                        # text behind the image: its position is not its cache slot
            e = w.embed[int(ids[i])].float().contiguous()
            buf = torch.cat([e, torch.zeros(2 * h)]).contiguous()      # kept alive across the call
            p = ref.transformer_forward_embd_logits_pos(m, buf.data_ptr(), i, int(pos3[0, i]), int(pos3[1, i]), int(pos3[2, i]))
        want.append(torch.from_numpy(np.ctypeslib.as_array(p, shape=(cfg.vocab,)).copy()))
    want = torch.stack(want)
    assert w.cfg.n_deepstack_layers == 2 and list(w.cfg.mrope_sections) == [24, 20, 20, 0]
    model = Transformer(w, KvCache.allocate(w.cfg, 4, 16, "cpu"))
    fb = ForwardBatch.build([t], [0], ids, torch.tensor([[0, 1]], dtype=torch.int32), 16, cfg.n_heads, cfg.n_kv_heads, "cpu", all_logits=True)
    emb = w.embed[ids.long()].float().clone()
    emb[vis] = rows[:, :h]
    ds = torch.zeros(2, t, h)
    ds[0, vis], ds[1, vis] = rows[:, h: 2 * h], rows[:, 2 * h:]
    fb.embeds, fb.positions3, fb.deepstack = emb.to(torch.bfloat16), pos3.to(torch.int32), ds.to(torch.bfloat16)
    got = model.forward(fb).float()
    for i in (0, 3, 4, 9, 10, 17):
        assert _rel(got[i], want[i]) < 3e-2, (i, _rel(got[i], want[i]))
