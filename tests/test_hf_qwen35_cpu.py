"""The hybrid stack (gated Delta-Net layers mixed with gated attention layers, partial rotary, output gates) against Hugging Face's
Qwen3.5 text model in fp32 on the same random weights: a third implementation that shares nothing with this framework or with the
reference's CPU engine (which pins the same stack from a GGUF file in tests/test_loader_cpu.py)."""
import pytest
import torch

pytest.importorskip("transformers.models.qwen3_5")

from gemm_b200.models import reference  # noqa: E402
from gemm_b200.models.config import get_config  # noqa: E402
from gemm_b200.models.transformer import ForwardBatch, KvCache, Transformer  # noqa: E402
from gemm_b200.models.weights import RandomSource, build_weights  # noqa: E402
from gemm_b200.utils import hf_compare  # noqa: E402


class _Source(RandomSource):
    """Random weights with norm weights away from one, so that the ``1 + w`` convention is exercised."""

    def get(self, name, shape):
        if name.endswith("norm.weight"):
            return (1.0 + self._randn(name, shape).float() * 5).to(torch.bfloat16)
        return super().get(name, shape)


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("name", ["tiny-qwen35", "tiny-qwen35moe"])
def test_mixed_stack_matches_transformers(name):
    cfg = get_config(name)
    src = _Source(cfg, 5)
    hf = hf_compare.hf_qwen35_model(cfg, src)
    w = build_weights(cfg, src, "bf16", "cpu")
    ids = torch.randint(0, cfg.vocab, (1, 70), generator=torch.Generator().manual_seed(1))         # more than one 64-token chunk of HF's scan
    with torch.no_grad():
        want = hf(ids, use_cache=False).logits[0].float()
    # the fp32 restatement of our model code: the same arithmetic as theirs
    o32 = reference.reference_logits(w, ids[0])
    assert _rel(o32, want) < 1e-4 and (o32.argmax(-1) == want.argmax(-1)).float().mean() > 0.97
    assert _rel(o32[1], want[1]) < 1e-4                                            # the second position included
    # the engine path (bf16 activations), prefill in two chunks then one decode-sized step
    page, bt = 16, torch.arange(6, dtype=torch.int32).unsqueeze(0)
    m = Transformer(w, KvCache.allocate(cfg, 6, page, "cpu"))
    outs = []
    for lo, hi in ((0, 37), (37, 69), (69, 70)):
        fb = ForwardBatch.build([hi - lo], [lo], ids[0, lo:hi], bt, page, cfg.n_heads, cfg.n_kv_heads, "cpu", all_logits=True)
        outs.append(m.forward(fb).float())
    got = torch.cat(outs)
    tol = 8e-2 if cfg.is_moe else 4e-2              # bf16 activations flip a near-tie of the router here and there
    assert _rel(got, want) < tol and (got.argmax(-1) == want.argmax(-1)).float().mean() > 0.85


@pytest.mark.parametrize("name", ["tiny-qwen35", "tiny-qwen35moe"])
def test_checkpoints_written_by_transformers_load_and_agree(tmp_path, name):
    """The import direction: a hybrid model saved by transformers (``save_pretrained``: its tensor names under ``model.language_model.``,
    its configuration keys) read by ``loader.load_safetensors`` gives transformers' logits."""
    from gemm_b200.models import loader
    from gemm_b200.utils import hf_compare
    cfg = get_config(name)
    hf = hf_compare.hf_qwen35_model(cfg, RandomSource(cfg, 9))
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    got_cfg = loader.config_from_hf(str(tmp_path))
    for field in ("arch", "n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "rope_dim", "full_attention_interval", "ssm_n_heads_k", "ssm_n_heads_v",
                  "ssm_head_dim", "ssm_d_conv", "n_experts", "n_experts_used", "expert_ffn", "shared_expert_ffn", "attn_output_gate", "qk_norm"):
        assert getattr(got_cfg, field) == getattr(cfg, field), field
    assert list(got_cfg.mrope_sections) == list(cfg.mrope_sections)
    w = loader.load_safetensors(str(tmp_path), "bf16", device="cpu")
    ids = torch.randint(0, cfg.vocab, (17,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids[None]).logits[0]
    got = reference.reference_logits(w, ids)
    assert ((got - want).norm() / want.norm()).item() < 3e-2                  # our copy of the weights is bf16
