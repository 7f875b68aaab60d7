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
