"""The text side of Qwen3-VL (embedding rows in, M-RoPE with separate t / h / w positions on the image rows, DeepStack features added
after the first layers) against Hugging Face's Qwen3VLTextModel in fp32 on the same weights."""
import pytest
import torch

pytest.importorskip("transformers.models.qwen3_vl")

from gemm_b200.models.config import get_config  # noqa: E402
from gemm_b200.models.transformer import ForwardBatch, KvCache, Transformer  # noqa: E402
from gemm_b200.models.weights import RandomSource, build_weights  # noqa: E402
from gemm_b200.utils import hf_compare  # noqa: E402


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_mrope_and_deepstack_match_transformers():
    cfg = get_config("tiny-dense").with_(mrope_sections=[24, 20, 20, 0], n_deepstack_layers=2)
    src = RandomSource(cfg, 5)
    hf, head = hf_compare.hf_qwen3vl_text_model(cfg, src)
    w = build_weights(cfg, src, "bf16", "cpu")
    h, t = cfg.hidden, 20
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg.vocab, (t,), generator=g)
    # rows 5 .. 12 are an image of 2 x 4 merged patches at t = 5; the text resumes after the larger grid side
    vis = torch.zeros(t, dtype=torch.bool)
    vis[5:13] = True
    pos3 = torch.arange(t).repeat(3, 1)
    pos3[0, 5:13] = 5
    pos3[1, 5:13] = 5 + torch.arange(8) // 4
    pos3[2, 5:13] = 5 + torch.arange(8) % 4
    pos3[:, 13:] = torch.arange(13, t) - 13 + 5 + 4
    emb = src.get("token_embd.weight", (cfg.vocab, h)).float()[ids].clone()
    emb[vis] = torch.randn(8, h, generator=g) * 0.02
    ds = torch.randn(2, 8, h, generator=g) * 0.02
    with torch.no_grad():
        out = hf(inputs_embeds=emb[None], position_ids=pos3[:, None, :], visual_pos_masks=vis[None], deepstack_visual_embeds=[ds[0], ds[1]],
                 use_cache=False).last_hidden_state[0]
        want = out @ head.t()
        plain = hf(inputs_embeds=emb[None], position_ids=torch.arange(t).repeat(3, 1)[:, None, :], use_cache=False).last_hidden_state[0] @ head.t()
    m = Transformer(w, KvCache.allocate(cfg, 2, 16, "cpu"))
    fb = ForwardBatch.build([t], [0], ids, torch.tensor([[0, 1]], dtype=torch.int32), 16, cfg.n_heads, cfg.n_kv_heads, "cpu", all_logits=True)
    fb.embeds, fb.positions3 = emb.to(torch.bfloat16), pos3.to(torch.int32)
    dsf = torch.zeros(2, t, h)
    dsf[:, vis] = ds
    fb.deepstack = dsf.to(torch.bfloat16)
    got = m.forward(fb).float()
    assert _rel(got, want) < 2e-2 and _rel(got[5:13], want[5:13]) < 2e-2 and _rel(got[13:], want[13:]) < 2e-2
    assert _rel(plain[13:], want[13:]) > 5e-2            # the image positions and features do change the rows behind them


def test_vision_language_checkpoint_written_by_transformers_loads_and_agrees(tmp_path):
    """The text side of a Qwen3-VL checkpoint saved by transformers (weights under ``model.language_model.``, ``text_config`` nesting,
    M-RoPE sections, DeepStack indexes in the vision configuration) through ``loader.load_safetensors``: text-only logits equal."""
    from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration
    from gemm_b200.models import loader, reference
    tc = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
              max_position_embeddings=128, rope_parameters={"rope_type": "default", "rope_theta": 50000.0, "mrope_section": [6, 5, 5]}, tie_word_embeddings=False)
    vc = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4, spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=64,
              num_position_embeddings=16, deepstack_visual_indexes=[0, 1], in_channels=3)
    torch.manual_seed(0)
    hf = Qwen3VLForConditionalGeneration(Qwen3VLConfig(text_config=tc, vision_config=vc, image_token_id=290, video_token_id=291, vision_start_token_id=292,
                                                       vision_end_token_id=293)).float().eval()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    cfg = loader.config_from_hf(str(tmp_path))
    assert cfg.arch == "qwen3vl" and list(cfg.mrope_sections) == [6, 5, 5, 0] and cfg.n_deepstack_layers == 2 and cfg.rope_theta == 50000.0 and cfg.qk_norm
    w = loader.load_safetensors(str(tmp_path), "bf16", device="cpu")
    ids = torch.randint(0, 280, (15,), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        want = hf(input_ids=ids[None]).logits[0]
    got = reference.reference_logits(w, ids)
    assert _rel(got, want) < 2e-2
