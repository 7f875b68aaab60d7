"""Native CPU engine (csrc/host/cpu_engine.cc): logits against the fp32 PyTorch oracle and, when the reference tree is present,
greedy tokens against the reference CPU engine on the same GGUF file."""
import numpy as np
import pytest
import torch

from gemm_b200.models import loader, reference
from gemm_b200.models.config import get_config
from gemm_b200.models.weights import RandomSource
from gemm_b200.serve.cpu_engine import CpuEngine
from gemm_b200.utils import cpubench
from tests import reference_oracle as oracle


def _rel(a, b):
    a, b = torch.as_tensor(a).float(), torch.as_tensor(b).float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("name,wtype", [("tiny-dense", "Q8_0"), ("tiny-qwen2", "Q8_0"), ("tiny-dense", "Q4_K"), ("tiny-dense", "F16"),
                                        ("tiny-moe", "Q8_0"), ("tiny-moe", "F16")])
def test_logits_match_the_fp32_oracle(tmp_path, name, wtype):
    cfg = get_config(name)
    path = str(tmp_path / "m.gguf")
    loader.save_gguf(cfg, RandomSource(cfg, seed=7), path, wtype)
    w = loader.load_gguf(path, "bf16", device="cpu")          # the file's (quantised) weights, decoded: what the engine multiplies with
    toks = torch.randint(0, cfg.vocab, (21,), generator=torch.Generator().manual_seed(1)).tolist()
    want = reference.reference_logits(w, torch.tensor(toks))
    eng = CpuEngine(path, max_seq_len=64, threads=3)
    got_batched = eng.forward(toks, 0)                          # one batched pass
    assert _rel(got_batched, want[-1]) < 2e-2                   # the oracle holds bf16 copies of the decoded weights
    eng2 = CpuEngine(path, max_seq_len=64, threads=1)
    for i, t in enumerate(toks):                                # token by token on one thread: same cache, same logits
        got_seq = eng2.forward([t], i)
    assert np.abs(got_seq - got_batched).max() < (2e-2 if cfg.is_moe else 1e-3) * max(1.0, np.abs(got_batched).max())   # MoE: a near-tie may route differently
    out, _, _ = eng.generate(toks, 5)
    out1, _, _ = eng2.generate(toks, 5)
    assert out == out1 and len(out) == 5


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not available")
def test_greedy_tokens_equal_the_reference_engine(tmp_path):
    cfg = get_config("tiny-dense")
    path = str(tmp_path / "m.gguf")
    loader.save_gguf(cfg, RandomSource(cfg, seed=9), path, "Q8_0")
    prompt = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(2)).tolist()
    ref = cpubench.run_reference(oracle.REF_ROOT, path, prompt, 12, threads=1)
    ours = cpubench.run_ours(path, prompt, 12, threads=4)
    assert ref is not None and ours[0] == ref[0]


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not available")
def test_moe_greedy_tokens_equal_the_reference_engine(tmp_path):
    cfg = get_config("tiny-moe")
    path = str(tmp_path / "moe.gguf")
    loader.save_gguf(cfg, RandomSource(cfg, seed=4), path, "Q8_0")
    prompt = torch.randint(0, cfg.vocab, (20,), generator=torch.Generator().manual_seed(5)).tolist()
    ref = cpubench.run_reference(oracle.REF_ROOT, path, prompt, 10, threads=1)
    ours = cpubench.run_ours(path, prompt, 10, threads=4)
    assert ref is not None and ours[0] == ref[0]


def test_load_errors_are_reported(tmp_path):
    from gemm_b200.models import gemma4
    gcfg = gemma4.Gemma4Config(n_layers=2, hidden=64, n_heads=2, n_kv_heads=1, ffn=128, vocab=64, head_dim_full=32, head_dim_swa=32, window=8, ple_dim=8,
                               shared_kv_layers=0, swa_pattern=[True, False], max_seq_len=32)
    path = str(tmp_path / "g4.gguf")
    gemma4.save_gguf(gcfg, gemma4.random_tensors(gcfg, seed=1), path, "F16")
    with pytest.raises(RuntimeError, match="architecture"):
        CpuEngine(path)
    eng_path = str(tmp_path / "d.gguf")
    cfg2 = get_config("tiny-dense")
    loader.save_gguf(cfg2, RandomSource(cfg2, seed=1), eng_path, "Q8_0")
    eng = CpuEngine(eng_path, max_seq_len=8)
    with pytest.raises(RuntimeError, match="cache"):
        eng.forward(list(range(9)), 0)


def test_profile_covers_the_forward_pass(tmp_path):
    cfg = get_config("tiny-dense")
    path = str(tmp_path / "m.gguf")
    loader.save_gguf(cfg, RandomSource(cfg, seed=3), path, "Q8_0")
    eng = CpuEngine(path, max_seq_len=64, threads=2)
    eng.profile()                                               # reset
    eng.forward(list(range(1, 17)), 0)
    prof = eng.profile()
    assert set(prof) == set(CpuEngine.PHASES) and all(v >= 0.0 for v in prof.values())
    assert prof["qkv"] > 0.0 and prof["down"] > 0.0 and prof["head"] > 0.0
    assert sum(eng.profile().values()) == 0.0                  # the call above reset the counters


def test_portable_paths_give_the_same_logits(tmp_path):
    """The AVX2 tiles on pageable weights (both switches off) against whatever this CPU selects by default."""
    import os
    import subprocess
    import sys
    cfg = get_config("tiny-dense")
    path = str(tmp_path / "m.gguf")
    loader.save_gguf(cfg, RandomSource(cfg, seed=5), path, "Q8_0")
    toks = list(range(3, 22))
    here = CpuEngine(path, max_seq_len=64, threads=2).forward(toks, 0)
    out = str(tmp_path / "logits.npy")
    code = ("import numpy as np; from gemm_b200.serve.cpu_engine import CpuEngine; "
            f"np.save({out!r}, CpuEngine({path!r}, max_seq_len=64, threads=2).forward({toks!r}, 0))")
    env = dict(os.environ, GB_CPU_AVX512="0", GB_CPU_HUGEPAGES="0")
    subprocess.run([sys.executable, "-c", code], check=True, env=env, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    there = np.load(out)
    assert np.abs(here - there).max() < 1e-3 * max(1.0, np.abs(here).max())


def test_generate_and_server_on_the_native_engine(tmp_path, capsys):
    """``generate --cpu-engine`` and the HTTP server over the native engine give the engine's own greedy tokens."""
    import json
    import urllib.request
    from gemm_b200.__main__ import main
    from gemm_b200.serve.cpu_engine import CpuEngineModel
    from gemm_b200.serve.sequential import SequentialLLM
    from gemm_b200.serve.server import serve
    cfg = get_config("tiny-moe")
    path = str(tmp_path / "m.gguf")
    loader.save_gguf(cfg, RandomSource(cfg, seed=6), path, "Q8_0")
    prompt = [5, 9, 200, 31, 7]
    want, _, _ = CpuEngine(path, max_seq_len=64, threads=2).generate(prompt, 6)
    main(["generate", "--model", path, "--cpu-engine", "--threads", "2", "--ids", "--prompt", " ".join(map(str, prompt)), "--max-new-tokens", "6",
          "--pages", "4", "--page-size", "16"])
    out = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert out[0]["token_ids"] == want
    llm = SequentialLLM(CpuEngineModel(path, max_seq_len=64, threads=2), None, max_seq_len=64)
    httpd, eng = serve(llm, port=0, block=False)
    try:
        req = urllib.request.Request(f"http://127.0.0.1:{httpd.server_address[1]}/v1/completions", data=json.dumps({"prompt": prompt, "max_tokens": 6}).encode(),
                                     headers={"Content-Type": "application/json"})
        got = json.loads(urllib.request.urlopen(req, timeout=60).read())
        assert got["token_ids"] == want
    finally:
        eng.stop_flag = True
        httpd.shutdown()
    with pytest.raises(SystemExit):
        from gemm_b200.models import gemma4
        gcfg = gemma4.Gemma4Config(n_layers=2, hidden=64, n_heads=2, n_kv_heads=1, ffn=128, vocab=64, head_dim_full=32, head_dim_swa=32, window=8, ple_dim=8,
                                   shared_kv_layers=0, swa_pattern=[True, False], max_seq_len=32)
        other = str(tmp_path / "g4.gguf")
        gemma4.save_gguf(gcfg, gemma4.random_tensors(gcfg, seed=1), other, "F16")
        main(["generate", "--model", other, "--cpu-engine", "--ids", "--prompt", "1 2 3", "--max-new-tokens", "2"])


@pytest.mark.parametrize("name,wtype", [("tiny-qwen35", "F16"), ("tiny-qwen35", "Q8_0"), ("tiny-qwen35moe", "F16")])
def test_hybrid_models_on_the_native_engine(tmp_path, name, wtype):
    """Delta-Net layers interleaved with gated attention (and, in the mixture variant, a gated shared expert): logits against the fp32
    oracle, whole prompt against chunks against token by token (the recurrent state carries over), and the rule that a recurrent
    state cannot be rewound."""
    cfg = get_config(name)
    path = str(tmp_path / "m.gguf")
    loader.save_gguf(cfg, RandomSource(cfg, seed=8), path, wtype)
    w = loader.load_gguf(path, "bf16", device="cpu")
    toks = torch.randint(0, cfg.vocab, (23,), generator=torch.Generator().manual_seed(2)).tolist()
    want = reference.reference_logits(w, torch.tensor(toks))
    eng = CpuEngine(path, max_seq_len=64, threads=3)
    whole = eng.forward(toks, 0)
    assert _rel(whole, want[-1]) < (2e-2 if wtype == "Q8_0" else 1e-4)
    eng.forward(toks[:9], 0)
    eng.forward(toks[9:10], 9)
    chunks = eng.forward(toks[10:], 10)
    one = CpuEngine(path, max_seq_len=64, threads=1)
    for i, t in enumerate(toks):
        single = one.forward([t], i)
    tol = 2e-2 if cfg.is_moe else 1e-4
    assert np.abs(chunks - whole).max() < tol * max(1.0, np.abs(whole).max()) and np.abs(single - whole).max() < tol * max(1.0, np.abs(whole).max())
    with pytest.raises(RuntimeError, match="recurrent state"):
        eng.forward(toks[:2], 5)
    assert np.abs(eng.forward(toks, 0) - whole).max() < 1e-5 * max(1.0, np.abs(whole).max())      # position 0 starts a new sequence
    out, _, _ = eng.generate(toks, 5)
    out1, _, _ = one.generate(toks, 5)
    assert out == out1


@pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not available")
def test_hybrid_greedy_tokens_equal_the_reference_engine(tmp_path):
    cfg = get_config("tiny-qwen35")
    path = str(tmp_path / "h.gguf")
    loader.save_gguf(cfg, RandomSource(cfg, seed=3), path, "Q8_0")
    prompt = torch.randint(0, cfg.vocab, (18,), generator=torch.Generator().manual_seed(4)).tolist()
    ref = cpubench.run_reference(oracle.REF_ROOT, path, prompt, 10, threads=1)
    ours = cpubench.run_ours(path, prompt, 10, threads=4)
    assert ref is not None and ours[0] == ref[0]
