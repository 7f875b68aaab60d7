"""Engine.generate (paged cache, chunked prefill, decode loop) on CPU against greedy decoding with the fp32 oracle."""
import torch

from gemm_b200.models import reference
from gemm_b200.models.config import get_config
from gemm_b200.models.weights import synthetic_weights
from gemm_b200.serve.engine import Engine, SamplingParams


def _oracle_greedy(w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        logits = reference.reference_logits(w, torch.tensor(toks))[-1]
        toks.append(int(logits.argmax()))
    return toks[len(prompt):]


def test_generate_greedy_matches_oracle():
    torch.manual_seed(0)
    cfg = get_config("tiny-moe")
    w = synthetic_weights(cfg, "bf16", device="cpu", seed=3)
    eng = Engine(w, max_batch=3, max_seq_len=128, page_size=16, max_prefill_tokens=24)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (9, 30, 17)]
    out = eng.generate(prompts, SamplingParams(max_new_tokens=5))
    agree = 0
    for p, o in zip(prompts, out):
        ref = _oracle_greedy(w, p, 5)
        agree += sum(int(a == b) for a, b in zip(o, ref))
    # bf16 rounding in the engine can flip a near-tie; require near-total agreement
    assert agree >= 13
    eng.reset()
    assert len(eng.pages.free) == eng.pages.num_pages


def test_int8_kv_cache_generates_like_the_bf16_cache():
    """The same engine with its KV pages kept as int8 + scales (prefill through the bf16 staging buffer, decode over the quantised
    pages): on CPU tensors this checks the staging layout and the slot bookkeeping; the decoded tokens stay those of the bf16 cache
    except where a near-tie flips."""
    torch.manual_seed(1)
    cfg = get_config("tiny-dense")
    w = synthetic_weights(cfg, "bf16", device="cpu", seed=4)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (11, 40, 23)]
    ref = Engine(w, max_batch=3, max_seq_len=128, page_size=16, max_prefill_tokens=128).generate(prompts, SamplingParams(max_new_tokens=6))
    eng = Engine(w, max_batch=3, max_seq_len=128, page_size=16, max_prefill_tokens=128, kv_dtype="int8")
    assert eng.kv.quantized and eng.kv.kq[0].dtype == torch.int8
    out = eng.generate(prompts, SamplingParams(max_new_tokens=6))
    agree = sum(int(a == b) for o, r in zip(out, ref) for a, b in zip(o, r))
    assert agree >= 15, (out, ref)
    assert eng.kv.nbytes() < 0.62 * Engine(w, max_batch=3, max_seq_len=128, page_size=16, max_prefill_tokens=128).kv.nbytes() + 2 * eng.kv.k[0].numel() * 2
