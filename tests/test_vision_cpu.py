"""Qwen3-VL vision encoder (models/vision.py) against the reference project's encoder on a GGUF file our writer produced, and its
hand-over to the text model (embeddings + DeepStack features)."""
import numpy as np
import pytest
import torch

from tests import reference_oracle as oracle
from gemm_b200.models import vision


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _cfg():
    return vision.VisionConfig(n_blocks=4, dim=64, n_heads=4, ffn=128, patch_size=4, image_size=32, proj_dim=48, spatial_merge=2,
                               deepstack_layers=[1, 2], image_mean=(0.48, 0.46, 0.41), image_std=(0.27, 0.26, 0.28))


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not present")
@pytest.mark.parametrize("hw", [(32, 32), (16, 24)])
def test_matches_reference_encoder(tmp_path, hw):
    cfg = _cfg()
    path = str(tmp_path / "mmproj.gguf")
    vision.save_gguf(cfg, vision.random_tensors(cfg, seed=2), path, "F16")
    enc = vision.load_gguf(path)
    h, w = hw
    rgb = torch.randint(0, 256, (h, w, 3), generator=torch.Generator().manual_seed(4), dtype=torch.uint8)
    x = enc.normalize_image(rgb)
    got = enc.encode(x)
    n_merged = (h // 4) * (w // 4) // 4
    assert got.shape == (n_merged, 48 * 3)
    ref = oracle.vision_lib()
    g = ref.gguf_open(path.encode(), 1)
    vm = ref.vision_load(g)
    assert vm, "the reference encoder refused our mmproj file"
    xin = np.ascontiguousarray(x.numpy(), dtype=np.float32)
    p = ref.vision_encode(vm, xin.ctypes.data, w, h, 1)
    assert p
    want = torch.from_numpy(np.ctypeslib.as_array(p, shape=(n_merged, 48 * 3)).copy())
    assert _rel(got, want) < 2e-3, _rel(got, want)
    for s in range(3):                                  # the main embedding and each DeepStack slice on its own
        assert _rel(got[:, 48 * s: 48 * (s + 1)], want[:, 48 * s: 48 * (s + 1)]) < 2e-3


def test_features_feed_the_text_model():
    """Vision tokens enter the text model as embedding rows with (t, h, w) positions; DeepStack slices join after the first layers."""
    from gemm_b200.models.config import get_config
    from gemm_b200.models.transformer import ForwardBatch, KvCache, Transformer
    from gemm_b200.models.weights import synthetic_weights
    cfg_t = get_config("tiny-dense").with_(n_deepstack_layers=2)
    cfg_v = vision.VisionConfig(n_blocks=3, dim=64, n_heads=4, ffn=128, patch_size=4, image_size=16, proj_dim=cfg_t.hidden, deepstack_layers=[0, 1])
    enc = vision.VisionEncoder(cfg_v, vision.random_tensors(cfg_v, 1))
    feats = enc.encode(torch.randn(16, 16, 3))
    embeds, ds = enc.forward_inputs(feats)
    assert embeds.shape == (4, cfg_t.hidden) and ds.shape == (2, 4, cfg_t.hidden)
    w = synthetic_weights(cfg_t, "bf16", "cpu", 3)
    model = Transformer(w, KvCache.allocate(cfg_t, 2, 16, "cpu"))
    bt = torch.tensor([[0, 1]], dtype=torch.int32)
    fb = ForwardBatch.build([4], [0], torch.zeros(4, dtype=torch.int32), bt, 16, cfg_t.n_heads, cfg_t.n_kv_heads, "cpu")
    fb.embeds, fb.deepstack = embeds, ds
    with_ds = model.forward(fb).float()
    model2 = Transformer(w, KvCache.allocate(cfg_t, 2, 16, "cpu"))
    fb2 = ForwardBatch.build([4], [0], torch.zeros(4, dtype=torch.int32), bt, 16, cfg_t.n_heads, cfg_t.n_kv_heads, "cpu")
    fb2.embeds = embeds
    without = model2.forward(fb2).float()
    assert torch.isfinite(with_ds).all() and _rel(with_ds, without) > 1e-3       # the DeepStack features reach the logits


def test_engine_prefill_with_image_rows():
    """A multimodal prompt through ``Engine.prefill`` (chunked) equals the same rows through one forward pass, and the image
    changes the continuation."""
    from gemm_b200.models.config import get_config
    from gemm_b200.models.transformer import ForwardBatch, KvCache, Transformer
    from gemm_b200.models.weights import synthetic_weights
    from gemm_b200.serve.engine import Engine
    cfg_t = get_config("tiny-dense").with_(n_deepstack_layers=2)
    cfg_v = vision.VisionConfig(n_blocks=2, dim=64, n_heads=4, ffn=128, patch_size=4, image_size=16, proj_dim=cfg_t.hidden, deepstack_layers=[0, 1])
    enc = vision.VisionEncoder(cfg_v, vision.random_tensors(cfg_v, 1))
    feats = enc.encode(torch.randn(16, 16, 3, generator=torch.Generator().manual_seed(2)))
    w = synthetic_weights(cfg_t, "bf16", "cpu", 3)
    ids, embeds, ds = vision.prompt_inputs(w.embed, [5, 6, 7], feats, [8, 9], cfg_t.hidden)
    assert ids.numel() == 3 + 4 + 2 and embeds.shape == (9, cfg_t.hidden) and ds.shape == (2, 9, cfg_t.hidden)
    assert float(ds[:, :3].abs().max()) == 0 and float(ds[:, 3:7].abs().max()) > 0
    eng = Engine(w, max_batch=2, max_seq_len=32, page_size=16, max_prefill_tokens=4)          # forces three chunks
    logits = eng.prefill([ids], reserve=4, embeds=[embeds], deepstack=[ds])
    model = Transformer(w, KvCache.allocate(cfg_t, 2, 16, "cpu"))
    fb = ForwardBatch.build([9], [0], ids, torch.tensor([[0, 1]], dtype=torch.int32), 16, cfg_t.n_heads, cfg_t.n_kv_heads, "cpu")
    fb.embeds, fb.deepstack = embeds, ds
    want = model.forward(fb).float()
    assert _rel(logits, want) < 2e-2
    eng2 = Engine(w, max_batch=2, max_seq_len=32, page_size=16)
    text_only = eng2.prefill([torch.tensor([5, 6, 7, 8, 9], dtype=torch.int32)], reserve=4)
    assert _rel(logits, text_only) > 1e-2


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not present")
@pytest.mark.parametrize("hw", [(24, 24), (12, 36)])
def test_gemma4_vision_tower_matches_reference(tmp_path, hw):
    cfg = vision.Gemma4VisionConfig(n_blocks=3, dim=64, n_heads=4, ffn=96, patch_size=4, image_size=24, proj_dim=40, n_pos=12)
    path = str(tmp_path / "g4v.gguf")
    vision.Gemma4VisionEncoder.save_gguf(cfg, vision.Gemma4VisionEncoder.random_tensors(cfg, 5), path, "F16")
    enc = vision.Gemma4VisionEncoder.load_gguf(path)
    assert enc.cfg.n_pos == 12 and enc.cfg.n_blocks == 3
    h, w = hw
    rgb = torch.randint(0, 256, (h, w, 3), generator=torch.Generator().manual_seed(6), dtype=torch.uint8)
    got = enc.encode(rgb)
    n_tok = (h // 4 // 3) * (w // 4 // 3)
    assert got.shape == (n_tok, 40)
    ref = oracle.gemma4_vision_lib()
    g = ref.gguf_open(path.encode(), 1)
    vm = ref.g4v_load(g)
    assert vm, "the reference tower refused our mmproj file"
    buf = np.ascontiguousarray(rgb.numpy())
    p = ref.g4v_encode(vm, buf.ctypes.data, w, h)
    assert p
    want = torch.from_numpy(np.ctypeslib.as_array(p, shape=(n_tok, 40)).copy())
    assert _rel(got, want) < 2e-3, _rel(got, want)
