"""The tensor-op model families behind the serving interface: a Gemma4 model and a GLM-5 style model answer OpenAI-style requests
through ``serve.sequential.SequentialLLM`` (one request at a time, in arrival order)."""
import json
import threading
import urllib.request

import torch

from gemm_b200.models import gemma4, glm5
from gemm_b200.serve.engine import SamplingParams
from gemm_b200.serve.sequential import SequentialLLM
from gemm_b200.serve.server import serve


def _post(port, path, body):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=60) as r:
        return r.read()


def _gemma():
    cfg = gemma4.Gemma4Config(n_layers=4, hidden=64, n_heads=2, n_kv_heads=1, ffn=128, vocab=200, head_dim_full=32, head_dim_swa=16, window=8,
                              ple_dim=8, shared_kv_layers=2, swa_pattern=[True, False, True, False], max_seq_len=64)
    return gemma4.Gemma4Model(cfg, gemma4.random_tensors(cfg, 1))


def test_generate_matches_the_model_and_sampling_is_reproducible():
    model = _gemma()
    want = model.generate([3, 4, 5, 6], 6)
    llm = SequentialLLM(_gemma(), max_seq_len=64, prefill_chunk=3)
    got = llm.generate([[3, 4, 5, 6], [9, 8]], SamplingParams(max_new_tokens=6))
    assert got[0] == want and len(got[1]) == 6
    sp = SamplingParams(max_new_tokens=5, temperature=0.8, top_k=20, top_p=0.9, seed=7)
    a = SequentialLLM(_gemma(), max_seq_len=64).generate([[1, 2, 3]], sp)
    b = SequentialLLM(_gemma(), max_seq_len=64).generate([[1, 2, 3]], sp)
    assert a == b


def test_server_with_tensor_op_models():
    cfg = glm5.GLM5Config(n_layers=2, n_dense_layers=1, hidden=32, vocab=120, n_heads=2, qk_nope_dim=8, qk_rope_dim=8, v_head_dim=16, q_lora=16,
                          kv_lora=8, index_dim=8, index_n_heads=2, n_experts=4, n_active=2, moe_inter=16, dense_inter=32, max_pos=64)
    for model in (_gemma(), glm5.GLM5Model(cfg, glm5.random_tensors(cfg, 2))):
        llm = SequentialLLM(model, max_seq_len=48)
        httpd, eng = serve(llm, port=0, block=False)
        port = httpd.server_address[1]
        try:
            out = json.loads(_post(port, "/v1/completions", {"prompt": [5, 6, 7], "max_tokens": 4}))
            assert len(out["token_ids"]) == 4 and out["usage"]["prompt_tokens"] == 3
            results = [None] * 3

            def worker(i):
                results[i] = json.loads(_post(port, "/v1/completions", {"prompt": [5, 6, 7], "max_tokens": 4}))["token_ids"]
            th = [threading.Thread(target=worker, args=(i,)) for i in range(3)]
            [t.start() for t in th]; [t.join() for t in th]
            assert all(r == out["token_ids"] for r in results)
            raw = _post(port, "/v1/completions", {"prompt": [5, 6, 7], "max_tokens": 3, "stream": True}).decode()
            assert [l for l in raw.splitlines() if l.startswith("data: ")][-1] == "data: [DONE]"
            too_long = json.loads(_post(port, "/v1/completions", {"prompt": list(range(60)), "max_tokens": 4}))
            assert too_long["token_ids"] == []
            prog = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/v1/progress", timeout=10).read())
            assert prog["tokens_generated"] >= 19 and prog["running"] == 0 and prog["waiting"] == 0
        finally:
            eng.stop_flag = True
            httpd.shutdown()
