"""The model code against Hugging Face transformers (fp32) on the same random-init checkpoints: an implementation of the
architectures that shares nothing with this repository or with the reference project."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from gemm_b200.utils import hf_compare  # noqa: E402


@pytest.mark.parametrize("name", ["tiny-dense", "tiny-moe", "tiny-qwen2"])
def test_greedy_matches_transformers(name):
    prompt = torch.randint(0, 512, (24,), generator=torch.Generator().manual_seed(1)).tolist()
    r = hf_compare.compare(f"synthetic:{name}", prompt, steps=6, device="cpu", seed=5)
    assert r["logit_rel_per_step"][0] < 3e-2, r                 # bf16 activations on our side, fp32 on theirs
    assert r["token_agreement"] >= 5 / 6 and r["edit_distance"] <= 2, r


def test_edit_distance():
    assert hf_compare.edit_distance([1, 2, 3], [1, 2, 3]) == 0
    assert hf_compare.edit_distance([1, 2, 3], [1, 3]) == 1
    assert hf_compare.edit_distance([], [4, 5]) == 2


@pytest.mark.parametrize("family", ["qwen3", "qwen2", "qwen3moe"])
def test_checkpoints_written_by_transformers_load_and_agree(tmp_path, family):
    """The other direction of the comparison: a random model built AND saved by transformers (``save_pretrained``: its config keys,
    its tensor names) is read by our safetensors importer and gives transformers' logits."""
    import transformers as T
    from gemm_b200.models import loader, reference
    torch.manual_seed(0)
    common = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                  max_position_embeddings=128, rope_theta=50000.0)
    if family == "qwen3":
        model = T.Qwen3ForCausalLM(T.Qwen3Config(head_dim=32, tie_word_embeddings=False, **common))
    elif family == "qwen2":
        model = T.Qwen2ForCausalLM(T.Qwen2Config(tie_word_embeddings=True, **common))
    else:
        model = T.Qwen3MoeForCausalLM(T.Qwen3MoeConfig(head_dim=32, moe_intermediate_size=32, num_experts=8, num_experts_per_tok=2, norm_topk_prob=True,
                                                       decoder_sparse_step=1, mlp_only_layers=[], **common))
    model = model.float().eval()
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    cfg = loader.config_from_hf(str(tmp_path))
    assert cfg.rope_theta == 50000.0 and cfg.n_experts == (8 if family == "qwen3moe" else 0) and cfg.tie_embeddings == (family == "qwen2")
    w = loader.load_safetensors(str(tmp_path), "bf16", device="cpu")
    ids = torch.randint(0, 300, (14,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = model(ids[None]).logits[0]
    got = reference.reference_logits(w, ids)
    assert ((got - want).norm() / want.norm()).item() < 2e-2              # our copy of the weights is bf16
    assert (got.argmax(-1) == want.argmax(-1)).float().mean() > 0.8
