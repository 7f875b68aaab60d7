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


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not present")
@pytest.mark.parametrize("hw", [(24, 24), (12, 36)])
def test_gemma4_unified_projector_matches_reference(tmp_path, hw):
    """The block-free "gemma4uv" projector: one token per 12-pixel square (patch 4 x merge 3)."""
    cfg = vision.Gemma4VisionConfig(n_blocks=0, dim=64, n_heads=4, ffn=96, patch_size=4, image_size=24, proj_dim=40, n_pos=12, projector="gemma4uv")
    path = str(tmp_path / "g4uv.gguf")
    vision.Gemma4VisionEncoder.save_gguf(cfg, vision.Gemma4VisionEncoder.random_tensors(cfg, 7), path, "F16")
    enc = vision.Gemma4VisionEncoder.load_gguf(path)
    assert enc.cfg.unified and enc.cfg.n_blocks == 0
    h, w = hw
    rgb = torch.randint(0, 256, (h, w, 3), generator=torch.Generator().manual_seed(8), dtype=torch.uint8)
    got = enc.encode(rgb)
    n_tok = (h // 12) * (w // 12)
    assert got.shape == (n_tok, 40)
    ref = oracle.gemma4_vision_lib()
    vm = ref.g4v_load(ref.gguf_open(path.encode(), 1))
    assert vm, "the reference tower refused our mmproj file"
    buf = np.ascontiguousarray(rgb.numpy())
    p = ref.g4v_encode(vm, buf.ctypes.data, w, h)
    assert p
    want = torch.from_numpy(np.ctypeslib.as_array(p, shape=(n_tok, 40)).copy())
    assert _rel(got, want) < 2e-3, _rel(got, want)


def test_multimodal_requests_through_llm_and_server():
    """An image + text prompt through the continuous-batching loop (chunked prefill, a text-only request in the same batch) equals the
    engine's one-shot prefill + decode, and the HTTP endpoint takes the image as base64."""
    import base64
    import io
    import json
    import urllib.request
    import numpy as np
    from gemm_b200.models.config import get_config
    from gemm_b200.models.weights import synthetic_weights
    from gemm_b200.serve.engine import Engine, SamplingParams
    from gemm_b200.serve.llm import LLM
    from gemm_b200.serve.server import serve
    from gemm_b200.utils.tokenizer import Tokenizer, toy_vocab
    cfg_t = get_config("tiny-dense").with_(n_deepstack_layers=2)
    cfg_v = vision.VisionConfig(n_blocks=2, dim=64, n_heads=4, ffn=128, patch_size=4, image_size=16, proj_dim=cfg_t.hidden, deepstack_layers=[0, 1])
    enc = vision.VisionEncoder(cfg_v, vision.random_tensors(cfg_v, 1))
    rgb = torch.randint(0, 256, (16, 16, 3), generator=torch.Generator().manual_seed(3), dtype=torch.uint8)
    feats = enc.encode(enc.normalize_image(rgb))
    w = synthetic_weights(cfg_t, "bf16", "cpu", 3)
    tokens, merges = toy_vocab("describe the picture of a quick brown fox " * 3, 60)
    tokens = (tokens + ["<|im_end|>"] + [f"<x{i}>" for i in range(cfg_t.vocab)])[: cfg_t.vocab]
    tok = Tokenizer(tokens, merges, [1] * len(tokens), "qwen2", {"eos": tokens.index("<|im_end|>")})
    before, after = tok.encode("describe "), tok.encode(" the picture")
    ids, embeds, ds = vision.prompt_inputs(w.embed, before, feats, after, cfg_t.hidden)
    # reference: the static engine, whole prompt at once
    eng = Engine(w, max_batch=1, max_seq_len=64, page_size=16)
    logits = eng.prefill([ids], reserve=8, embeds=[embeds], deepstack=[ds])
    first = logits.argmax(-1).to(torch.int32)
    eng.begin_decode(first, SamplingParams(), 8, use_graph=False)
    want = [int(first[0])] + [int(eng.decode_step()[0]) for _ in range(4)]
    # continuous batching with a token budget that cuts the prompt into chunks, next to a text-only request
    llm = LLM(w, tok, max_running=4, max_batch_tokens=6, num_pages=32, page_size=16)
    sp = SamplingParams(max_new_tokens=5)
    r_img = llm.add_request(ids.tolist(), sp, embeds=embeds, deepstack=ds)
    r_txt = llm.add_request(tok.encode("a quick brown fox"), sp)
    outs = {r_img: [], r_txt: []}
    while llm.has_work():
        llm.step()
        for rid, toks in llm.produced_all.items():
            outs[rid].extend(toks)
    assert outs[r_img] == want and len(outs[r_txt]) == 5
    # the HTTP endpoint: the same image as base64 .npy and as PPM
    httpd, engine = serve(llm, port=0, block=False, vision=enc)
    port = httpd.server_address[1]
    try:
        buf = io.BytesIO()
        np.save(buf, rgb.numpy())
        ppm = b"P6\n16 16\n255\n" + rgb.numpy().tobytes()
        got = []
        for raw in (buf.getvalue(), ppm):
            body = {"prompt": "describe <image> the picture", "image": base64.b64encode(raw).decode(), "max_tokens": 5}
            req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions", data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
            got.append(json.loads(urllib.request.urlopen(req, timeout=60).read()))
        assert got[0]["token_ids"] == got[1]["token_ids"] == want[: len(got[0]["token_ids"])]
        assert got[0]["usage"]["prompt_tokens"] == len(before) + 4 + len(after)
        bad = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions", data=json.dumps({"prompt": "x", "image": "AAAA"}).encode(),
                                     headers={"Content-Type": "application/json"})
        try:
            urllib.request.urlopen(bad, timeout=60)
            assert False, "a broken image must be refused"
        except urllib.error.HTTPError as e:
            assert e.code == 400
    finally:
        engine.stop_flag = True
        httpd.shutdown()


def test_png_and_jpeg_decoding_and_resize():
    """PNG (all 8-bit colour types) bit-exact and baseline JPEG (4:4:4, 4:2:2, 4:2:0, grey, restart markers, optimised tables) within
    rounding of a reference decoder; progressive files are refused with a message; resizing keeps flat colours."""
    import io
    Image = pytest.importorskip("PIL.Image")
    g = np.random.default_rng(0)
    yy, xx = np.mgrid[0:75, 0:101]
    img = np.stack([(127 + 100 * np.sin(xx / 9.0) * np.cos(yy / 7.0)), (xx * 2.3) % 256, (yy * 3.1 + xx) % 256], -1).astype(np.uint8)
    img[20:40, 30:60] = g.integers(0, 256, (20, 30, 3))
    for mode in ("RGB", "RGBA", "L", "LA", "P"):
        im = Image.fromarray(img).convert(mode)
        buf = io.BytesIO()
        im.save(buf, "PNG")
        assert torch.equal(vision.decode_image(buf.getvalue()), torch.from_numpy(np.array(im.convert("RGB")))), mode
    cases = [("RGB", dict(quality=90, subsampling=0), 2.5, 0.1), ("RGB", dict(quality=85, subsampling=2), 6.0, 0.8), ("RGB", dict(quality=75, subsampling=1), 6.0, 0.8),
             ("RGB", dict(quality=95, subsampling=0, optimize=True), 2.5, 0.1), ("RGB", dict(quality=80, subsampling=2, restart_marker_blocks=5), 6.0, 0.8),
             ("L", dict(quality=90), 2.5, 0.2)]
    for mode, kw, worst, mean in cases:
        buf = io.BytesIO()
        Image.fromarray(img).convert(mode).save(buf, "JPEG", **kw)
        got = vision.decode_image(buf.getvalue()).float()
        want = torch.from_numpy(np.array(Image.open(io.BytesIO(buf.getvalue())).convert("RGB"))).float()
        d = (got - want).abs()
        assert got.shape == (75, 101, 3) and d.max() <= worst and d.mean() <= mean, (kw, d.max().item(), d.mean().item())
    buf = io.BytesIO()
    Image.fromarray(img).save(buf, "JPEG", progressive=True)
    with pytest.raises(ValueError, match="progressive"):
        vision.decode_image(buf.getvalue())
    with pytest.raises(ValueError):
        vision.decode_image(b"\x89PNG\r\n\x1a\n" + b"\0" * 20)
    flat = torch.full((60, 90, 3), 77, dtype=torch.uint8)
    small = vision.resize_image(flat, 20, 32)
    assert small.shape == (20, 32, 3) and (small == 77).all()
    ramp = torch.arange(64, dtype=torch.uint8)[None, :, None].expand(8, 64, 3).contiguous()
    half = vision.resize_image(ramp, 8, 32)[0, :, 0].float()
    assert (half[1:] >= half[:-1]).all() and abs(float(half.mean()) - 31.5) < 1.0
