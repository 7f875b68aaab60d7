"""OpenAI-compatible HTTP front end over ``LLM`` (continuous batching).

Endpoints (the set the reference serves in server/server.c:2094-2270 for its LLM):
  POST /v1/chat/completions   messages -> ChatML prompt -> completion (``stream: true`` gives server-sent events)
  POST /v1/similarity         {ref, hyp} -> token agreement and character edit distance of two texts
  POST /v1/completions        raw prompt completion
  GET  /v1/models             the loaded model
  GET  /v1/progress           queue / running counts and tokens produced so far (server.c:1632)
  GET  /health

Unlike the reference (one global model, one request at a time, token-by-token prefill: server/server_llm.c:422-632),
requests from all connections are queued into one engine thread that steps the scheduler, so concurrent
requests share every forward pass.  Standard library only.
"""
from __future__ import annotations

import json
import os
import queue
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict, List, Optional

from .engine import SamplingParams
from .llm import LLM


def build_chat_prompt(messages: List[dict]) -> str:
    """OpenAI ``messages`` -> ChatML text (the template Qwen models are trained with; server_llm.c:298)."""
    parts = []
    for m in messages:
        content = m.get("content", "")
        if isinstance(content, list):                       # multimodal content parts: keep the text parts
            content = "".join(p.get("text", "") for p in content if isinstance(p, dict))
        parts.append(f"<|im_start|>{m.get('role', 'user')}\n{content}<|im_end|>\n")
    parts.append("<|im_start|>assistant\n")
    return "".join(parts)


class EngineThread(threading.Thread):
    """Owns the ``LLM``; HTTP handlers submit requests and read tokens from per-request queues."""

    def __init__(self, llm: LLM):
        super().__init__(daemon=True)
        self.llm = llm
        self.inbox: "queue.Queue" = queue.Queue()
        self.streams: Dict[int, "queue.Queue"] = {}
        self.tokens_total = 0
        self.stop_flag = False
        self.vision = None               # models.vision.VisionEncoder: requests may then carry an image

    def submit(self, ids: List[int], sp: SamplingParams, extra: Optional[dict] = None) -> "queue.Queue":
        """``extra``: keyword arguments for ``add_request`` (``embeds`` / ``deepstack`` of a multimodal prompt)."""
        q: "queue.Queue" = queue.Queue()
        self.inbox.put((ids, sp, q, extra or {}))
        return q

    def run(self):
        while not self.stop_flag:
            try:
                while True:
                    ids, sp, q, extra = self.inbox.get(block=not self.llm.has_work(), timeout=0.05)
                    try:
                        rid = self.llm.add_request(ids, sp, **extra)
                    except (ValueError, TypeError):                   # the cache can never hold this request: end its stream at once
                        q.put(None)
                        continue
                    self.streams[rid] = q
            except queue.Empty:
                pass
            if not self.llm.has_work():
                continue
            try:
                self.llm.step()
            except Exception:
                # a failed step must not leave clients blocked on their queues: end every open stream, drop the requests
                import traceback
                traceback.print_exc()
                for q in self.streams.values():
                    q.put(None)
                self.streams.clear()
                self.stop_flag = True
                break
            for rid, q in list(self.streams.items()):    # requests the scheduler dropped produce no token: close their streams
                r = self.llm._reqs.get(rid)
                if r is not None and r.error:
                    q.put(None)
                    del self.streams[rid]
                    self.llm._reqs.pop(rid, None)
            for rid, toks in self.llm.produced_all.items():
                self.tokens_total += len(toks)
                q = self.streams.get(rid)
                if q is None:
                    continue
                for tok in toks:
                    q.put(tok)
                if self.llm._reqs[rid].done:
                    q.put(None)
                    del self.streams[rid]
                    self.llm._reqs.pop(rid, None)


def make_handler(engine: EngineThread, model_name: str):
    llm = engine.llm

    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, fmt, *args):            # quiet
            pass

        def _json(self, code: int, obj) -> None:
            body = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_GET(self):
            if self.path in ("/", "/index.html", "/chat"):       # the chat page (the reference ships web/llm_chat.html beside its server)
                with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "chat.html"), "rb") as fh:
                    body = fh.read()
                self.send_response(200)
                self.send_header("Content-Type", "text/html; charset=utf-8")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)
                return
            if self.path == "/health":
                return self._json(200, {"status": "ok"})
            if self.path == "/v1/models":
                return self._json(200, {"object": "list", "data": [{"id": model_name, "object": "model"}]})
            if self.path == "/v1/progress":
                return self._json(200, {"waiting": llm.sched.num_waiting, "running": llm.sched.num_running,
                                        "tokens_generated": engine.tokens_total, "steps": llm.steps})
            self._json(404, {"error": "not found"})

        def do_POST(self):
            n = int(self.headers.get("Content-Length", "0"))
            try:
                req = json.loads(self.rfile.read(n) or b"{}")
            except json.JSONDecodeError:
                return self._json(400, {"error": "invalid JSON"})
            if self.path == "/v1/similarity":
                # agreement of two texts, e.g. this server's completion against another implementation's
                # (the reference's comparison server answers the same request, ref/llm/llm_server.py:45-66)
                from ..utils.hf_compare import edit_distance
                ref_t, hyp_t = str(req.get("ref", "")), str(req.get("hyp", ""))
                ced = edit_distance([ord(ch) for ch in ref_t], [ord(ch) for ch in hyp_t])
                metrics = {"char_len_ref": len(ref_t), "char_len_hyp": len(hyp_t), "char_edit_distance": ced,
                           "char_similarity": 1.0 - ced / max(len(ref_t), len(hyp_t), 1)}
                method = "char-levenshtein"
                if llm.tokenizer is not None:
                    a, b = llm.tokenizer.encode(ref_t), llm.tokenizer.encode(hyp_t)
                    n, k = min(len(a), len(b)), 0
                    while k < n and a[k] == b[k]:
                        k += 1
                    same = sum(1 for x, y in zip(a, b) if x == y)
                    metrics.update({"len_ref": len(a), "len_hyp": len(b), "common_prefix_tokens": k, "first_divergence_pos": k,
                                    "token_match_rate": same / max(len(a), len(b), 1), "token_edit_distance": edit_distance(a, b)})
                    method = "token-agreement"
                return self._json(200, {"ok": True, "method": method, "metrics": metrics})
            chat = self.path == "/v1/chat/completions"
            if not chat and self.path != "/v1/completions":
                return self._json(404, {"error": "not found"})
            if chat:
                prompt = build_chat_prompt(req.get("messages", []))
            else:
                prompt = req.get("prompt", "")
            extra = {}
            image_b64 = req.get("image")
            if image_b64 is not None:
                # one image per request: base64 of a PNG, a baseline JPEG, a binary PPM or a .npy (uint8 [H, W, 3]); the text is split at "<image>" (the image
                # comes first when the marker is absent), as the reference's server feeds tokens, vision rows, tokens
                # (server/server_llm.c:503-548)
                if engine.vision is None or llm.tokenizer is None or not hasattr(llm, "w"):
                    return self._json(400, {"error": "no vision encoder loaded (serve --mmproj) or no tokenizer"})
                import base64
                from ..models import vision as V
                try:
                    rgb = V.decode_image(base64.b64decode(image_b64))
                    enc = engine.vision
                    cell = enc.cfg.patch_size * enc.cfg.spatial_merge
                    side = int(req.get("image_max_side", enc.cfg.image_size))
                    if max(rgb.shape[0], rgb.shape[1]) > side:   # larger than the encoder's grid: shrink, keeping the aspect ratio
                        f = side / max(rgb.shape[0], rgb.shape[1])
                        rgb = V.resize_image(rgb, max(cell, int(rgb.shape[0] * f)), max(cell, int(rgb.shape[1] * f)))
                    h, w = rgb.shape[0] // cell * cell, rgb.shape[1] // cell * cell
                    feats = enc.encode(enc.normalize_image(rgb[:h, :w]))
                except Exception as e:                         # a bad image is the client's error, not the server's
                    return self._json(400, {"error": f"image: {e}"})
                text = prompt if isinstance(prompt, str) else ""
                before, _, after = text.partition("<image>") if "<image>" in text else ("", "", text)
                ids_t, embeds, ds = V.prompt_inputs(llm.w.embed, llm.tokenizer.encode(before), feats, llm.tokenizer.encode(after), enc.cfg.proj_dim)
                ids = ids_t.tolist()
                extra = {"embeds": embeds, "deepstack": ds}
            elif isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
                ids = prompt                                   # pre-tokenised prompt
            else:
                if llm.tokenizer is None:
                    return self._json(400, {"error": "no tokenizer loaded: send the prompt as a list of token ids"})
                ids = llm.tokenizer.encode(prompt)
            stops = []
            if llm.tokenizer is not None:
                stops = [i for i in (llm.tokenizer.eos_id, llm.tokenizer.eot_id) if i >= 0]
            sp = SamplingParams(max_new_tokens=int(req.get("max_tokens", 128)), temperature=float(req.get("temperature", 0.0)),
                                top_k=int(req.get("top_k", 0)), top_p=float(req.get("top_p", 1.0)), seed=int(req.get("seed", 0)),
                                stop_token_ids=tuple(stops))
            stop_strings = req.get("stop") or []
            if isinstance(stop_strings, str):
                stop_strings = [stop_strings]
            q = engine.submit(ids, sp, extra)
            rid = "cmpl-" + uuid.uuid4().hex[:24]
            created = int(time.time())
            obj = "chat.completion" if chat else "text_completion"

            def text_of(toks: List[int]) -> str:
                return llm.tokenizer.decode(toks) if llm.tokenizer is not None else " ".join(str(t) for t in toks)

            toks: List[int] = []
            if req.get("stream"):
                self.send_response(200)
                self.send_header("Content-Type", "text/event-stream")
                self.send_header("Cache-Control", "no-cache")
                self.send_header("Transfer-Encoding", "chunked")
                self.end_headers()

                def chunk(payload: dict):
                    data = ("data: " + json.dumps(payload) + "\n\n").encode()
                    self.wfile.write(f"{len(data):X}\r\n".encode() + data + b"\r\n")
                    self.wfile.flush()

                sent = ""
                while True:
                    t = q.get()
                    if t is None:
                        break
                    toks.append(t)
                    full = text_of(toks)
                    delta, sent = full[len(sent):], full
                    piece = {"delta": {"content": delta}} if chat else {"text": delta}
                    chunk({"id": rid, "object": obj + ".chunk", "created": created, "model": model_name,
                           "choices": [dict(index=0, finish_reason=None, **piece)]})
                    if any(s and s in full for s in stop_strings):
                        break
                chunk({"id": rid, "object": obj + ".chunk", "created": created, "model": model_name,
                       "choices": [dict(index=0, finish_reason="stop", **({"delta": {}} if chat else {"text": ""}))]})
                done = b"data: [DONE]\n\n"
                self.wfile.write(f"{len(done):X}\r\n".encode() + done + b"\r\n0\r\n\r\n")
                return
            while True:
                t = q.get()
                if t is None:
                    break
                toks.append(t)
            text = text_of(toks)
            for s in stop_strings:
                if s and s in text:
                    text = text[: text.index(s)]
            finish = "length" if len(toks) >= sp.max_new_tokens else "stop"
            choice = {"index": 0, "finish_reason": finish}
            if chat:
                choice["message"] = {"role": "assistant", "content": text}
            else:
                choice["text"] = text
            self._json(200, {"id": rid, "object": obj, "created": created, "model": model_name, "choices": [choice], "token_ids": toks,
                             "usage": {"prompt_tokens": len(ids), "completion_tokens": len(toks), "total_tokens": len(ids) + len(toks)}})

    return Handler


def serve(llm: LLM, host: str = "127.0.0.1", port: int = 8080, model_name: str = "gemm_b200", block: bool = True, vision=None):
    """Start the engine thread and the HTTP server.  Returns ``(server, engine_thread)``; with ``block`` it serves for ever.
    ``vision``: a ``models.vision.VisionEncoder``; requests may then carry ``"image"`` (base64 PPM or .npy)."""
    engine = EngineThread(llm)
    engine.vision = vision
    engine.start()
    httpd = ThreadingHTTPServer((host, port), make_handler(engine, model_name))
    if block:
        try:
            httpd.serve_forever()
        finally:
            engine.stop_flag = True
    else:
        threading.Thread(target=httpd.serve_forever, daemon=True).start()
    return httpd, engine
