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
