"""GPU engine (hand-written kernels) vs the same engine on CPU tensors (PyTorch reference ops) and the fp32 oracle."""
import pytest
import torch

from gemm_b200 import _native
from gemm_b200.models import reference
from gemm_b200.models.config import get_config
from gemm_b200.models.transformer import ForwardBatch, KvCache, Transformer
from gemm_b200.models.weights import synthetic_weights

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float().cpu() - b.float().cpu()).norm() / (b.float().cpu().norm() + 1e-12)).item()


def _run(model, cfg, toks, lens, bt, page, device, chunks, decode_steps):
    ctx = [0] * len(lens)
    outs = []
    for chunk in chunks:
        ids = torch.cat([toks[s][ctx[s]:ctx[s] + chunk[s]] for s in range(len(lens))])
        fb = ForwardBatch.build(chunk, ctx, ids, bt, page, cfg.n_heads, cfg.n_kv_heads, device)
        outs.append(model.forward(fb).float().cpu())
        ctx = [c + q for c, q in zip(ctx, chunk)]
    for step in range(decode_steps):
        ids = torch.stack([toks[s][lens[s] + step] for s in range(len(lens))])
        fb = ForwardBatch.build([1] * len(lens), ctx, ids, bt, page, cfg.n_heads, cfg.n_kv_heads, device, num_splits=2 if step == 1 else 1)
        outs.append(model.forward(fb).float().cpu())
        ctx = [c + 1 for c in ctx]
    return outs


@pytest.mark.parametrize("name,fmt", [("tiny-dense", "bf16"), ("tiny-moe", "bf16"), ("tiny-qwen2", "bf16"), ("tiny-dense", "mxfp8"),
                                      ("tiny-moe", "mxfp8"), ("tiny-qwen35", "bf16"), ("tiny-qwen35moe", "bf16"), ("tiny-qwen35", "mxfp8"),
                                      ("tiny-dense", "q8_0"), ("tiny-dense", "q4_k"), ("tiny-qwen2", "q4_k")])
def test_gpu_engine_matches_cpu_engine_and_oracle(name, fmt):
    torch.manual_seed(0)
    cfg = get_config(name)
    w_cpu = synthetic_weights(cfg, fmt, device="cpu", seed=1)
    w_gpu = w_cpu.to("cuda")
    page = 16
    lens = [150, 40, 300]
    toks = [torch.randint(0, cfg.vocab, (n + 3,)) for n in lens]
    pages_per = [(n + 3 + page - 1) // page for n in lens]
    perm = torch.randperm(sum(pages_per) + 2)
    bt = torch.zeros(3, max(pages_per), dtype=torch.int32)
    p0 = 0
    for s in range(3):
        bt[s, : pages_per[s]] = perm[p0:p0 + pages_per[s]]
        p0 += pages_per[s]
    n_pages = sum(pages_per) + 2
    chunks = [[100, 40, 128], [50, 0, 172]]
    m_cpu = Transformer(w_cpu, KvCache.allocate(cfg, n_pages, page, "cpu"))
    m_gpu = Transformer(w_gpu, KvCache.allocate(cfg, n_pages, page, "cuda"))
    o_cpu = _run(m_cpu, cfg, toks, lens, bt, page, "cpu", chunks, 3)
    o_gpu = _run(m_gpu, cfg, toks, lens, bt, page, "cuda", chunks, 3)
    _native.assert_status_ok()
    tol = 2e-2 if fmt == "bf16" else 6e-2
    if "qwen35" in name:
        tol = 0.15 if "moe" in name else (4e-2 if fmt == "bf16" else 0.1)     # 4 layers; near-tied expert choices can flip (CPU test)
    for a, b in zip(o_gpu, o_cpu):
        assert _rel(a, b) < tol
    # oracle on the last prefill chunk (logits of the last token of sequences 0 and 2)
    for row, s in ((0, 0), (1, 2)):
        ref = reference.reference_logits(w_cpu, toks[s][: lens[s]])[-1]
        lim = 3e-2 if fmt == "bf16" else 0.2
        if "qwen35" in name:
            lim = 0.15 if fmt == "bf16" else 0.3          # twice the layers of the other test models
        assert _rel(o_gpu[1][row], ref) < lim
    assert any("libgb_cuda" in p for p in _native.loaded_libraries())


def test_forked_sequence_continues_like_its_parent():
    """KV fork: full pages are shared, the tail page is copied on the device; the fork then decodes exactly like the parent."""
    from gemm_b200.serve.scheduler import KvBlockManager
    torch.manual_seed(5)
    cfg = get_config("tiny-dense")
    w = synthetic_weights(cfg, "bf16", device="cuda", seed=2)
    page, n_pages, n_prompt = 16, 32, 40
    kv = KvCache.allocate(cfg, n_pages, page, "cuda")
    model = Transformer(w, kv)
    blocks = KvBlockManager(n_pages, page)
    a = blocks.new_sequence()
    blocks.reserve(a, n_prompt + 1)
    toks = torch.randint(0, cfg.vocab, (n_prompt + 1,))

    def table(seq):
        pg = blocks.pages(seq)
        return torch.tensor([pg], dtype=torch.int32)

    fb = ForwardBatch.build([n_prompt], [0], toks[:n_prompt], table(a), page, cfg.n_heads, cfg.n_kv_heads, "cuda")
    model.forward(fb)
    b, copy = blocks.fork(a, n_prompt)                      # 2 shared pages + an 8-token tail page to copy
    assert copy is not None
    kv.copy_pages([copy])
    blocks.reserve(b, n_prompt + 1)
    outs = []
    for seq in (a, b):
        fbd = ForwardBatch.build([1], [n_prompt], toks[n_prompt:], table(seq), page, cfg.n_heads, cfg.n_kv_heads, "cuda")
        outs.append(model.forward(fbd).float().cpu())
    _native.assert_status_ok()
    assert torch.equal(outs[0], outs[1])


def test_sampling_under_cuda_graph_equals_eager_sampling():
    """Temperature sampling: the replayed decode graph reads its step number from device memory, so it draws the same tokens
    as step-by-step eager execution with the same seed, and the draws differ from step to step."""
    from gemm_b200.serve.engine import Engine, SamplingParams
    torch.manual_seed(0)
    cfg = get_config("tiny-dense")
    w = synthetic_weights(cfg, "bf16", device=torch.device("cuda", 0), seed=4)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (33, 20, 7)]
    sp = SamplingParams(max_new_tokens=12, temperature=1.5, top_k=50, seed=11)
    outs = []
    for use_graph in (True, False):
        eng = Engine(w, max_batch=4, max_seq_len=256, page_size=128)
        outs.append(eng.generate(prompts, sp, use_graph=use_graph))
    assert outs[0] == outs[1]
    assert any(len(set(o)) > 2 for o in outs[0]), "sampled tokens should vary across steps"
    _native.assert_status_ok()


@pytest.mark.parametrize("fmt", ["bf16", "mxfp8"])
def test_int8_kv_cache_engine_decodes_like_the_bf16_cache(fmt):
    """Engine with the KV pages kept as int8 + scales (decode attention reads them directly, CUDA-graph decode) against the same
    engine with bf16 pages: the logits of the prefill agree closely (same kernels over staged bf16 rows), the greedy tokens
    agree except where a near-tie flips."""
    from gemm_b200.serve.engine import Engine, SamplingParams
    torch.manual_seed(2)
    cfg = get_config("tiny-dense")
    w = synthetic_weights(cfg, fmt, device="cuda", seed=6)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (150, 37, 260, 5)]
    ref_eng = Engine(w, max_batch=4, max_seq_len=512, page_size=16, max_prefill_tokens=512)
    ref = ref_eng.generate(prompts, SamplingParams(max_new_tokens=12))
    eng = Engine(w, max_batch=4, max_seq_len=512, page_size=16, max_prefill_tokens=512, kv_dtype="int8")
    out = eng.generate(prompts, SamplingParams(max_new_tokens=12))
    torch.cuda.synchronize()
    _native.assert_status_ok()
    agree = sum(int(a == b) for o, r in zip(out, ref) for a, b in zip(o, r))
    # of 48; once a near-tie flips, the rest of that sequence differs too (the two engines then decode different texts)
    assert agree >= 30, (agree, out, ref)
    assert sum(int(o[0] == r[0]) for o, r in zip(out, ref)) >= 3      # the token that follows the prefill
    assert eng.kv.kq[0].dtype == torch.int8 and eng._graph is not None
    # eager decode gives the same tokens as the captured graph
    out2 = eng.generate(prompts, SamplingParams(max_new_tokens=12), use_graph=False)
    assert out2 == out
