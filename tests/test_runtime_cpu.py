"""C++ runtime: KV block manager, continuous-batching scheduler, profiler; and the LLM front end on CPU."""
import torch

from gemm_b200.models.config import get_config
from gemm_b200.models.weights import synthetic_weights
from gemm_b200.serve.engine import Engine, SamplingParams
from gemm_b200.serve.llm import LLM
from gemm_b200.serve.scheduler import KvBlockManager, Scheduler
from gemm_b200.utils import profiler


def test_block_manager_alloc_fork_release():
    kv = KvBlockManager(10, 16)
    a = kv.new_sequence()
    kv.reserve(a, 40)                         # 3 pages
    assert len(kv.pages(a)) == 3 and kv.num_free == 7
    b, copy = kv.fork(a, 40)                  # 2 full pages shared, the 8-token tail page copied
    pa, pb = kv.pages(a), kv.pages(b)
    assert pb[:2] == pa[:2] and pb[2] != pa[2] and copy == (pa[2], pb[2])
    assert kv.refcount(pa[0]) == 2 and kv.num_free == 6
    c, copy2 = kv.fork(a, 32)                 # page-aligned fork copies nothing
    assert copy2 is None and kv.pages(c) == pa[:2] and kv.refcount(pa[0]) == 3
    kv.release(a)
    assert kv.refcount(pa[0]) == 2 and kv.num_free == 7
    kv.release(b); kv.release(c)
    assert kv.num_free == 10
    d = kv.new_sequence()
    try:
        kv.reserve(d, 16 * 11)
        assert False, "over-allocation must fail"
    except MemoryError:
        pass
    assert kv.num_free == 10                  # all-or-nothing


def test_scheduler_chunked_prefill_and_decode_first():
    kv = KvBlockManager(64, 16)
    s = Scheduler(kv, max_running=4, max_batch_tokens=32)
    s.add(0, 50, 3)
    s.add(1, 10, 2)
    p = s.plan()                              # budget 32: first chunk of request 0 only
    assert [(i.req_id, i.q_len, i.ctx_len, i.is_prefill, i.emits_token) for i in p] == [(0, 32, 0, True, False)]
    s.commit([False])
    p = s.plan()                              # rest of request 0 (18) + request 1 admitted (10)
    assert [(i.req_id, i.q_len, i.ctx_len, i.emits_token) for i in p] == [(0, 18, 32, True), (1, 10, 0, True)]
    s.commit([False, False])
    p = s.plan()                              # both decode
    assert [(i.req_id, i.q_len, i.ctx_len, i.is_prefill) for i in p] == [(0, 1, 50, False), (1, 1, 10, False)]
    s.commit([False, False])                  # request 1 reached max_new = 2 -> leaves
    assert s.num_running == 1
    p = s.plan()
    assert [(i.req_id, i.ctx_len) for i in p] == [(0, 51)]
    s.commit([False])
    assert s.num_running == 0 and kv.num_free == 64


def test_scheduler_lookahead_and_multi_token_commit():
    """Speculative decoding: decode items reserve and are budgeted for the look-ahead positions; a commit may advance a
    request by several tokens."""
    kv = KvBlockManager(8, 16)
    s = Scheduler(kv, max_running=4, max_batch_tokens=16)
    s.set_lookahead(3)
    s.add(0, 14, 12)
    s.add(1, 6, 9)
    p = s.plan()
    assert [(i.req_id, i.q_len) for i in p] == [(0, 14), (1, 2)]
    s.commit([False, False])
    p = s.plan()                              # request 0 decodes (budget 1 + 3), the rest of request 1's prompt follows
    assert [(i.req_id, i.q_len, i.ctx_len, i.is_prefill) for i in p] == [(0, 1, 14, False), (1, 4, 2, True)]
    assert len(kv.pages(p[0].seq)) == 2       # 14 + 1 generated + 1 new + 3 look-ahead = 19 positions -> two pages
    s.commit([False, False], [4, 1])          # three drafts accepted + the model's own token; request 1 emitted its first token
    p = s.plan()
    assert [(i.req_id, i.ctx_len) for i in p] == [(0, 18), (1, 6)]
    s.commit([False, False], [4, 2])
    p = s.plan()
    assert [(i.req_id, i.ctx_len) for i in p] == [(0, 22), (1, 8)]
    s.commit([True, True], [1, 1])            # both hit a stop token
    assert s.num_running == 0 and kv.num_free == 8


def test_scheduler_preempts_youngest_when_out_of_pages():
    kv = KvBlockManager(5, 16)
    s = Scheduler(kv, max_running=4, max_batch_tokens=64)
    s.add(0, 30, 20)
    s.add(1, 30, 20)
    s.commit([])  # no-op
    steps = 0
    while (s.num_running or s.num_waiting) and steps < 400:
        p = s.plan()
        assert p, "scheduler stalled"
        s.commit([False] * len(p))
        steps += 1
    assert s.num_preempted >= 1 and kv.num_free == 5


def test_llm_continuous_batching_equals_static_batch():
    torch.manual_seed(0)
    cfg = get_config("tiny-dense")
    w = synthetic_weights(cfg, "bf16", device="cpu", seed=2)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (5, 37, 18, 9, 26)]
    sp = SamplingParams(max_new_tokens=4)
    llm = LLM(w, max_running=3, max_batch_tokens=24, num_pages=64, page_size=16)
    out = llm.generate(prompts, sp)
    eng = Engine(w, max_batch=5, max_seq_len=64, page_size=16)
    ref = eng.generate(prompts, sp)
    assert out == ref
    assert llm.blocks.num_free == 64
    # streaming yields the same tokens one by one
    assert list(llm.stream(prompts[1], sp)) == ref[1]


def test_profiler_tables():
    profiler.reset()
    profiler.enable(True)
    with profiler.region("qkv", "gemm", "attention", layer=0, flops=1e9):
        sum(range(1000))
    with profiler.region("norm", "elementwise", "attention", layer=0, nbytes=1e6):
        pass
    text = profiler.summary()
    profiler.enable(False)
    assert "per op" in text and "qkv" in text and "per component" in text and "attention" in text


def _drive(s, kv, n_req, max_steps=400):
    """Run a scheduler to completion, checking after every plan that its items name live, distinct sequences."""
    steps = 0
    while (s.num_running or s.num_waiting) and steps < max_steps:
        p = s.plan()
        s.take_aborted()
        seqs = [i.seq for i in p]
        assert len(set(seqs)) == len(seqs), f"a sequence appears twice in one plan: {p}"
        for i in p:
            pages = kv.pages(i.seq)                          # raises KeyError for a released sequence
            assert len(pages) * kv.page_size >= i.ctx_len + i.q_len, (i, pages)
        if not p:
            break
        s.commit([False] * len(p))
        steps += 1
    return steps


def test_scheduler_never_preempts_a_planned_request():
    """4 pages of 4 tokens, prompts of 6 and 8 tokens: the younger request runs out of pages while the older one already
    has a decode item in the plan; the victim must be the younger one itself."""
    kv = KvBlockManager(4, 4)
    s = Scheduler(kv, max_running=4, max_batch_tokens=64)
    s.add(0, 6, 6)
    s.add(1, 8, 4)
    steps = _drive(s, kv, 2)
    assert steps < 400 and s.num_running == 0 and s.num_waiting == 0
    assert kv.num_free == 4 and s.num_preempted >= 1


def test_scheduler_rejects_and_aborts_what_can_never_fit():
    kv = KvBlockManager(4, 4)
    s = Scheduler(kv, max_running=4, max_batch_tokens=64)
    try:
        s.add(0, 20, 4)                                      # prompt alone exceeds the 16-position cache
        assert False, "must be refused"
    except ValueError:
        pass
    assert s.num_waiting == 0
    # with look-ahead switched on later, a queued request may stop fitting: the plan drops it and reports it
    s.add(1, 10, 5)
    s.set_lookahead(4)
    p = s.plan()
    assert p == [] and s.take_aborted() == [1] and s.num_waiting == 0 and s.num_running == 0 and kv.num_free == 4


def test_llm_reports_requests_that_cannot_fit():
    cfg = get_config("tiny-dense")
    w = synthetic_weights(cfg, "bf16", device="cpu", seed=2)
    llm = LLM(w, max_running=2, max_batch_tokens=32, num_pages=4, page_size=4)
    try:
        llm.generate([list(range(1, 30))], SamplingParams(max_new_tokens=4))
        assert False
    except ValueError:
        pass
    assert not llm.has_work()
    out = llm.generate([[1, 2, 3]], SamplingParams(max_new_tokens=3))
    assert len(out[0]) == 3 and llm.blocks.num_free == 4


def test_hybrid_preemption_restarts_from_an_empty_state():
    """A preempted request of a Delta-Net model re-prefills from position 0: its recurrent slot must be cleared, or the state of
    the first pass leaks into the second.  Tokens with a cache tight enough to preempt equal those of a roomy cache."""
    torch.manual_seed(0)
    cfg = get_config("tiny-qwen35")
    w = synthetic_weights(cfg, "bf16", device="cpu", seed=3)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (9, 11)]
    sp = SamplingParams(max_new_tokens=8)
    roomy = LLM(w, max_running=2, max_batch_tokens=32, num_pages=32, page_size=4)
    ref = roomy.generate(prompts, sp)
    tight = LLM(w, max_running=2, max_batch_tokens=32, num_pages=8, page_size=4)
    out = tight.generate(prompts, sp)
    assert tight.sched.num_preempted >= 1, "the cache was meant to be too small for both requests"
    assert out == ref
