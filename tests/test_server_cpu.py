"""HTTP front end on CPU: completions, chat, streaming, concurrent requests sharing the engine."""
import json

import pytest
import threading
import urllib.request

import torch

from gemm_b200.models.config import get_config
from gemm_b200.models.weights import synthetic_weights
from gemm_b200.serve.llm import LLM
from gemm_b200.serve.server import build_chat_prompt, serve
from gemm_b200.utils.tokenizer import Tokenizer, toy_vocab


def _post(port, path, body):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=60) as r:
        return r.read()


def test_server_endpoints():
    cfg = get_config("tiny-dense")
    tokens, merges = toy_vocab("the quick brown fox jumps over the lazy dog " * 3, 60)
    specials = ["<|im_start|>", "<|im_end|>"]
    tokens = (tokens + specials + [f"<x{i}>" for i in range(cfg.vocab)])[: cfg.vocab]
    types = [3 if t in specials else 1 for t in tokens]
    tok = Tokenizer(tokens, merges, types, "qwen2", {"eos": tokens.index("<|im_end|>")})
    llm = LLM(synthetic_weights(cfg, "bf16", device="cpu", seed=1), tok, max_running=4, max_batch_tokens=64, num_pages=64, page_size=16)
    httpd, eng = serve(llm, port=0, block=False)
    port = httpd.server_address[1]
    try:
        assert json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=10).read())["status"] == "ok"
        sim = json.loads(_post(port, "/v1/similarity", {"ref": "the quick brown fox", "hyp": "the quick brown dog"}))
        assert sim["ok"] and sim["method"] == "token-agreement" and sim["metrics"]["char_edit_distance"] == 2
        assert 0 < sim["metrics"]["common_prefix_tokens"] <= sim["metrics"]["len_ref"] and sim["metrics"]["char_similarity"] == pytest.approx(1 - 2 / 19)
        same = json.loads(_post(port, "/v1/similarity", {"ref": "abc", "hyp": "abc"}))["metrics"]
        assert same["token_match_rate"] == 1.0 and same["char_edit_distance"] == 0 and same["first_divergence_pos"] == same["len_ref"]
        page = urllib.request.urlopen(f"http://127.0.0.1:{port}/", timeout=10)
        assert page.headers["Content-Type"].startswith("text/html") and b"/v1/chat/completions" in page.read()      # the built-in chat page
        out = json.loads(_post(port, "/v1/completions", {"prompt": "the quick brown", "max_tokens": 5}))
        assert out["object"] == "text_completion" and len(out["token_ids"]) <= 5 and out["usage"]["prompt_tokens"] > 0
        # the same prompt as token ids gives the same tokens (greedy)
        ids = tok.encode("the quick brown")
        out2 = json.loads(_post(port, "/v1/completions", {"prompt": ids, "max_tokens": 5}))
        assert out2["token_ids"] == out["token_ids"]
        chat = json.loads(_post(port, "/v1/chat/completions", {"messages": [{"role": "user", "content": "the dog"}], "max_tokens": 4}))
        assert chat["choices"][0]["message"]["role"] == "assistant"
        # streaming: server-sent events ending with [DONE]
        raw = _post(port, "/v1/completions", {"prompt": "the lazy dog", "max_tokens": 4, "stream": True}).decode()
        events = [l[6:] for l in raw.splitlines() if l.startswith("data: ")]
        assert events[-1] == "[DONE]" and len(events) >= 2 and json.loads(events[0])["object"].endswith(".chunk")
        # concurrent requests are batched by the one engine thread
        results = [None] * 4
        def worker(i):
            results[i] = json.loads(_post(port, "/v1/completions", {"prompt": "the quick brown", "max_tokens": 5}))["token_ids"]
        th = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
        [t.start() for t in th]; [t.join() for t in th]
        assert all(r == out["token_ids"] for r in results)
        prog = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/v1/progress", timeout=10).read())
        assert prog["tokens_generated"] > 0 and prog["running"] == 0
        # speculative decoding behind the same endpoints: same tokens, every accepted token is delivered
        from gemm_b200.serve.speculative import NgramDrafter
        long_plain = json.loads(_post(port, "/v1/completions", {"prompt": "the quick brown fox the quick", "max_tokens": 12}))["token_ids"]
        llm.set_drafter(NgramDrafter(gamma=3))
        long_spec = json.loads(_post(port, "/v1/completions", {"prompt": "the quick brown fox the quick", "max_tokens": 12}))["token_ids"]
        assert long_spec == long_plain
        raw = _post(port, "/v1/completions", {"prompt": "the quick brown fox the quick", "max_tokens": 12, "stream": True}).decode()
        assert len([l for l in raw.splitlines() if l.startswith("data: ") and l != "data: [DONE]"]) >= len(long_plain)
    finally:
        httpd.shutdown()
        eng.stop_flag = True
    assert build_chat_prompt([{"role": "system", "content": "s"}, {"role": "user", "content": "u"}]).endswith("<|im_start|>assistant\n")
