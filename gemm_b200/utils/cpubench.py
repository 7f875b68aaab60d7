"""CPU benchmark of the smallest benchmark configuration: Qwen3-0.6B shape, Q8_0 GGUF, batch 1, a prompt of random token ids,
greedy decode — our native CPU engine against the reference project's CPU engine on the same file and the same ids.

``python -m gemm_b200 cpubench [--prompt-len 128 --new 32 --threads 8 --reference-root DIR]``

The reference arm compiles the reference's own ``common/transformer.h`` with gcc from its source tree (nothing of it lives in
this repository) and drives it through the calls its command-line program makes (cpu/llm/test_transformer.c:284-345:
``transformer_forward`` for every prompt token but the last, ``transformer_forward_logits`` after that, arg-max in between)."""
from __future__ import annotations

import ctypes
import json
import os
import shutil
import subprocess
import tempfile
import time
from typing import List, Optional, Tuple

import torch

_SHIM = r'''
#define GGUF_LOADER_IMPLEMENTATION
#include "gguf_loader.h"
#define GGML_DEQUANT_IMPLEMENTATION
#include "ggml_dequant.h"
#define TRANSFORMER_IMPLEMENTATION
#include "transformer.h"
#include <time.h>
static double now_s(void) { struct timespec t; clock_gettime(CLOCK_MONOTONIC, &t); return t.tv_sec + 1e-9 * t.tv_nsec; }
/* the loop of cpu/llm/test_transformer.c: sequential prefill, then greedy decode */
int ref_generate(const char *path, int max_seq, int n_threads, const int *prompt, int n_prompt, int max_new, int *out, double *prefill_s, double *decode_s) {
    gguf_context *g = gguf_open(path, 1);
    if (!g) return -1;
    transformer_model *m = transformer_load(g, max_seq);
    if (!m) return -2;
    if (n_threads > 1) transformer_set_threads(m, n_threads);
    double t0 = now_s();
    float *logits = NULL;
    for (int i = 0; i < n_prompt; i++) {
        if (i == n_prompt - 1) logits = transformer_forward_logits(m, prompt[i], i);
        else transformer_forward(m, prompt[i], i);
    }
    double t1 = now_s();
    int pos = n_prompt, next = 0;
    for (int s = 0; s < max_new; s++) {
        if (s > 0) { logits = transformer_forward_logits(m, next, pos); pos++; }
        if (!logits) return -3;
        next = 0;
        for (int j = 1; j < m->n_vocab; j++) if (logits[j] > logits[next]) next = j;
        out[s] = next;
    }
    double t2 = now_s();
    *prefill_s = t1 - t0; *decode_s = t2 - t1;
    return 0;
}
'''


def _config(model: str, layers: int = 0, overrides=()):
    """The preset ``model``, cut to ``layers`` layers when > 0, with ``key=value`` overrides of integer fields (a hybrid shape at a
    size that fits: ``--model tiny-qwen35 --set hidden=1024 --set n_layers=8 ...``)."""
    from ..models.config import get_config
    cfg = get_config(model)
    if layers > 0:
        cfg = cfg.with_(n_layers=layers)
    kw = {}
    for item in overrides:
        k, _, v = item.partition("=")
        if not hasattr(cfg, k):
            raise ValueError(f"--set {item}: the configuration has no field {k!r}")
        kw[k] = int(v)
    return cfg.with_(**kw) if kw else cfg


def make_checkpoint(path: str, model: str = "qwen3-0.6b", wtype: str = "Q8_0", seed: int = 0, layers: int = 0, overrides=()) -> None:
    """Write the random-init checkpoint (N(0, 0.02) matrices, unit norms) of ``model`` (cut to ``layers`` layers when > 0) as a GGUF
    file in ggml type ``wtype``."""
    from ..models import loader
    from ..models.weights import RandomSource
    cfg = _config(model, layers, overrides)
    loader.save_gguf(cfg, RandomSource(cfg, seed, "cpu"), path, wtype)


def run_ours(path: str, prompt: List[int], max_new: int, threads: int) -> Tuple[List[int], float, float]:
    from ..serve.cpu_engine import CpuEngine
    eng = CpuEngine(path, max_seq_len=len(prompt) + max_new + 8, threads=threads)
    try:
        return eng.generate(prompt, max_new)
    finally:
        eng.close()


def run_profile(path: str, prompt: List[int], max_new: int, threads: int) -> dict:
    """Milliseconds per phase of the native engine: one batched prefill of the prompt, then ``max_new`` single-token steps (per token)."""
    from ..serve.cpu_engine import CpuEngine
    eng = CpuEngine(path, max_seq_len=len(prompt) + max_new + 8, threads=threads)
    try:
        eng.forward(prompt[: min(8, len(prompt))], 0)                        # warm-up: pages touched, threads started
        eng.profile()
        t0 = time.perf_counter()
        eng.forward(prompt, 0)
        t1 = time.perf_counter()
        pre = eng.profile()
        pos = len(prompt)
        for _ in range(max_new):
            eng.forward([1], pos)
            pos += 1
        t2 = time.perf_counter()
        dec = eng.profile()
    finally:
        eng.close()
    return {"threads": threads, "prefill_ms": round((t1 - t0) * 1e3, 2), "prefill_phases_ms": {k: round(v * 1e3, 2) for k, v in pre.items()},
            "decode_ms_per_token": round((t2 - t1) / max_new * 1e3, 3), "decode_phases_ms_per_token": {k: round(v / max_new * 1e3, 3) for k, v in dec.items()}}


def run_reference(ref_root: str, path: str, prompt: List[int], max_new: int, threads: int) -> Optional[Tuple[List[int], float, float]]:
    """The reference CPU engine on the same file (None when its tree or gcc is missing)."""
    if not os.path.isdir(os.path.join(ref_root, "common")) or shutil.which("gcc") is None:
        return None
    d = tempfile.mkdtemp(prefix="gemm_ref_cpubench_")
    src, so = os.path.join(d, "shim.c"), os.path.join(d, "shim.so")
    with open(src, "w") as f:
        f.write(_SHIM)
    cmd = ["gcc", "-O3", "-march=native", "-mavx2", "-mfma", "-mf16c", "-shared", "-fPIC", "-w", "-I", os.path.join(ref_root, "common"), src, "-o", so,
           "-lm", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building the reference engine failed:\n" + r.stderr[-2000:])
    lib = ctypes.CDLL(so)
    ids = (ctypes.c_int * len(prompt))(*prompt)
    out = (ctypes.c_int * max_new)()
    tp, td = ctypes.c_double(), ctypes.c_double()
    rc = lib.ref_generate(path.encode(), len(prompt) + max_new + 8, threads, ids, len(prompt), max_new, out, ctypes.byref(tp), ctypes.byref(td))
    if rc != 0:
        raise RuntimeError(f"the reference engine failed with code {rc}")
    return list(out), tp.value, td.value


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="CPU benchmark: native CPU engine vs the reference CPU engine (Qwen3-0.6B shape, Q8_0)")
    ap.add_argument("--model", default="qwen3-0.6b")
    ap.add_argument("--wtype", default="Q8_0")
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--new", type=int, default=32)
    ap.add_argument("--layers", type=int, default=0, help="cut the model to this many layers (0: all): a mixture model's shape at a size that fits")
    ap.add_argument("--set", action="append", default=[], metavar="FIELD=INT", help="override an integer field of the preset (repeatable)")
    ap.add_argument("--threads", type=int, default=os.cpu_count() or 1)
    ap.add_argument("--gguf", default="", help="checkpoint to use (default: write the synthetic one to a temporary file)")
    ap.add_argument("--reference-root", default=os.environ.get("GEMM_REFERENCE_ROOT", ""), help="source tree of the reference project (optional)")
    ap.add_argument("--profile", action="store_true", help="print the native engine's time per phase (prefill, and per decoded token) instead of the comparison")
    ap.add_argument("--repeat", type=int, default=3, help="runs per arm, alternating; the fastest prefill and the fastest decode of each arm are "
                    "reported (other jobs on the machine only ever slow a run down)")
    args = ap.parse_args(argv)
    cfg = _config(args.model, args.layers, args.set)
    path = args.gguf
    tmp = None
    if not path:
        tmp = tempfile.mkdtemp(prefix="gemm_b200_cpubench_")
        path = os.path.join(tmp, "model.gguf")
        t0 = time.time()
        make_checkpoint(path, args.model, args.wtype, layers=args.layers, overrides=args.set)
        print(f"[cpubench] wrote {path} ({os.path.getsize(path) / 2**20:.0f} MiB) in {time.time() - t0:.1f}s")
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (args.prompt_len,), generator=g).tolist()
    if args.profile:
        print(json.dumps({"config": {"model": args.model, "layers": args.layers or cfg.n_layers, "wtype": args.wtype, "prompt_len": args.prompt_len,
                                     "new_tokens": args.new, "file_mib": round(os.path.getsize(path) / 2**20, 1)}, **run_profile(path, prompt, args.new, args.threads)}))
        if tmp is not None:
            shutil.rmtree(tmp, ignore_errors=True)
        return 0
    toks, tp, td = run_ours(path, prompt, args.new, args.threads)
    ref = run_reference(args.reference_root, path, prompt, args.new, args.threads) if args.reference_root else None
    for _ in range(max(0, args.repeat - 1)):
        t2, p2, d2 = run_ours(path, prompt, args.new, args.threads)
        assert t2 == toks, "the engine is not deterministic"
        tp, td = min(tp, p2), min(td, d2)
        if ref is not None:
            r2 = run_reference(args.reference_root, path, prompt, args.new, args.threads)
            ref = (ref[0], min(ref[1], r2[1]), min(ref[2], r2[2]))
    n_tok = args.prompt_len + args.new
    line = {"config": {"model": args.model, "layers": cfg.n_layers, "overrides": args.set, "wtype": args.wtype, "prompt_len": args.prompt_len, "new_tokens": args.new, "threads": args.threads},
            "ours": {"prefill_s": round(tp, 4), "decode_s": round(td, 4), "total_s": round(tp + td, 4), "prefill_tok_s": round(args.prompt_len / tp, 2),
                     "decode_tok_s": round((args.new - 1) / td, 2) if td > 0 else None, "tok_s_overall": round(n_tok / (tp + td), 2)}}
    line["config"]["repeat"] = args.repeat
    if args.reference_root:
        if ref is not None:
            rt, rp, rd = ref
            line["reference"] = {"prefill_s": round(rp, 4), "decode_s": round(rd, 4), "total_s": round(rp + rd, 4), "prefill_tok_s": round(args.prompt_len / rp, 2),
                                 "decode_tok_s": round((args.new - 1) / rd, 2) if rd > 0 else None, "tok_s_overall": round(n_tok / (rp + rd), 2)}
            line["tokens_identical"] = rt == toks
            line["speedup_total"] = round((rp + rd) / (tp + td), 2)
            line["speedup_decode"] = round(rd / td, 2) if td > 0 else None
    print(json.dumps(line))
    if tmp is not None:
        shutil.rmtree(tmp, ignore_errors=True)
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
