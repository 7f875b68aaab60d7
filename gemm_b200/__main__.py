"""Command line of the framework: ``python -m gemm_b200 <command> ...``.

  generate   load a checkpoint (GGUF / HF safetensors directory / synthetic preset) and complete one or more prompts
  serve      OpenAI-compatible HTTP server over the continuous-batching engine
  inspect    dump the metadata and tensor table of a GGUF file
  tokenize   print the token ids (and pieces) of a text with the tokenizer stored in a GGUF file
  stage      cut a checkpoint into per-rank blobs in the run-time weight format
  microbench kernel micro-benchmarks (same as ``python -m gemm_b200.utils.microbench``)
  estimate   roofline estimate of decode / prefill throughput for a model preset (tools/decode_estimate.py of the reference)
  compare    run the same prompt through the CPU reference path and the GPU kernels and report the agreement token by token
  dump       run a prompt and write the hidden state after every layer (and the logits) as .npy files for layer-by-layer comparison
  build      compile the native libraries in-tree

The reference spreads these over separate programs: cpu/llm/test_transformer.c (generate: ``<model> [prompt] [max_gen]
[n_threads]``), server/server.c (``--model --host --port``), tests/test_gguf_loader.c, tests/test_bpe_tokenizer.c and
common/m3_stage.c.  Environment variables of the reference (LLM_THREADS, M3_PREFILL, ...) become flags here.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _load_llm(args):
    import os
    from .serve.llm import LLM
    kw = dict(max_running=args.max_running, num_pages=args.pages, page_size=args.page_size)
    if getattr(args, "cpu_engine", False) and os.path.isfile(args.model):
        # a dense or mixture Qwen GGUF on a machine without a GPU: the native CPU engine, one request at a time
        from .serve.cpu_engine import CpuEngineModel
        from .serve.sequential import SequentialLLM
        from .utils import gguf as G
        from .utils.tokenizer import Tokenizer
        with G.GGUFFile(args.model) as f:
            arch = f.metadata.get("general.architecture", "")
            tok = Tokenizer.from_gguf(f) if "tokenizer.ggml.tokens" in f.metadata else None
        if tok is None and args.tokenizer:
            with G.GGUFFile(args.tokenizer) as f:
                tok = Tokenizer.from_gguf(f)
        if arch not in ("qwen2", "qwen3", "qwen3moe", "qwen35", "qwen35moe"):
            sys.exit(f"--cpu-engine: architecture {arch!r} is not one the native CPU engine runs (qwen2, qwen3, qwen3moe, qwen35, qwen35moe)")
        n = args.pages * args.page_size
        return SequentialLLM(CpuEngineModel(args.model, max_seq_len=n, threads=getattr(args, "threads", 0)), tok, max_seq_len=n)
    if _is_gemma4(args.model):
        # Gemma4 runs as a tensor-op model behind the one-request-at-a-time adapter
        import torch
        from .models import gemma4
        from .serve.sequential import SequentialLLM
        from .utils import gguf as G
        from .utils.tokenizer import Tokenizer
        dev = args.device if (args.device != "cuda" or torch.cuda.is_available()) else "cpu"
        model = gemma4.load_gguf(args.model, dev, torch.bfloat16 if dev != "cpu" else torch.float32)
        tok = None
        with G.GGUFFile(args.tokenizer or args.model) as f:
            if "tokenizer.ggml.tokens" in f.metadata:
                tok = Tokenizer.from_gguf(f)
        return SequentialLLM(model, tok, max_seq_len=min(model.cfg.max_seq_len, args.pages * args.page_size))
    if os.path.isfile(os.path.join(args.model, "config.json")):
        # M3 / GLM-5 style checkpoints (models.m3 / models.glm5 save_checkpoint layout) run as tensor-op models
        with open(os.path.join(args.model, "config.json")) as fh:
            mt = json.load(fh).get("model_type", "")
        if mt in ("minimax_m3", "glm5"):
            import torch
            from .models import glm5, m3
            from .serve.sequential import SequentialLLM
            dev = args.device if (args.device != "cuda" or torch.cuda.is_available()) else "cpu"
            mod = m3 if mt == "minimax_m3" else glm5
            model = mod.load_checkpoint(args.model, dev, torch.bfloat16 if dev != "cpu" else torch.float32)
            tok = None
            if args.tokenizer:
                from .utils import gguf as G
                from .utils.tokenizer import Tokenizer
                with G.GGUFFile(args.tokenizer) as f:
                    tok = Tokenizer.from_gguf(f)
            return SequentialLLM(model, tok, max_seq_len=min(model.cfg.max_pos, args.pages * args.page_size))
    if args.model.startswith("synthetic:"):
        return LLM.from_synthetic(args.model.split(":", 1)[1], fmt=args.format, device=args.device, **kw)
    if os.path.isdir(args.model):
        tok = None
        if args.tokenizer:
            from .utils import gguf as G
            from .utils.tokenizer import Tokenizer
            with G.GGUFFile(args.tokenizer) as f:
                tok = Tokenizer.from_gguf(f)
        return LLM.from_safetensors(args.model, fmt=args.format, device=args.device, tokenizer=tok, **kw)
    return LLM.from_gguf(args.model, fmt=args.format, device=args.device, **kw)


def _add_model_args(p):
    p.add_argument("--model", required=True, help="GGUF file, HF safetensors directory, or synthetic:<preset>")
    p.add_argument("--format", default="bf16", choices=["bf16", "mxfp8"], help="run-time weight format")
    p.add_argument("--device", default="cuda")
    p.add_argument("--tokenizer", default="", help="GGUF file to take the tokenizer from (safetensors checkpoints)")
    p.add_argument("--max-running", type=int, default=64)
    p.add_argument("--pages", type=int, default=512, help="KV cache pages")
    p.add_argument("--page-size", type=int, default=128)
    p.add_argument("--cpu-engine", action="store_true", help="run a qwen2 / qwen3 / qwen3moe / qwen35 / qwen35moe GGUF on the native CPU engine (no GPU; one request at a time)")
    p.add_argument("--threads", type=int, default=0, help="worker threads of the native CPU engine (0: all cores)")


def _is_gemma4(path: str) -> bool:
    import os
    if not os.path.isfile(path):
        return False
    from .utils import gguf as G
    try:
        with G.GGUFFile(path) as f:
            return f.metadata.get("general.architecture") == "gemma4"
    except Exception:
        return False


def _generate_with_audio(args):
    """Gemma4 with an audio clip (the reference's driver: cuda/llm/test_gemma4_st.c:83-160): the clip is encoded to soft tokens,
    which are spliced into the prompt where ``<audio>`` stands (in front of it when the marker is absent); greedy decoding."""
    import torch
    from .models import audio, gemma4
    from .utils import gguf as G
    from .utils.tokenizer import Tokenizer
    dev = args.device if (args.device != "cuda" or torch.cuda.is_available()) else "cpu"
    model = gemma4.load_gguf(args.model, dev, torch.bfloat16 if dev != "cpu" else torch.float32)
    pcm, rate = audio.wav_load(args.audio)
    if rate != audio.RATE:
        sys.exit(f"{args.audio}: {rate} Hz; the encoder takes {audio.RATE} Hz mono (resample beforehand)")
    enc = audio.Gemma4AudioEncoder.from_checkpoint(args.audio_model, device=dev, dtype=torch.bfloat16 if dev != "cpu" else torch.float32)
    soft = enc.encode_pcm(pcm[: int(30.0 * audio.RATE)])
    if soft.shape[1] != model.cfg.hidden:
        sys.exit(f"the audio encoder emits rows of {soft.shape[1]}, the text model is {model.cfg.hidden} wide")
    tok = None
    with G.GGUFFile(args.tokenizer or args.model) as f:
        if "tokenizer.ggml.tokens" in f.metadata:
            tok = Tokenizer.from_gguf(f)
    for p in (args.prompt or [""]):
        before, _, after = p.partition("<audio>") if "<audio>" in p else ("", "", p)
        if args.ids:
            a, b = ([int(x) for x in part.replace(",", " ").split()] for part in (before, after))
        elif tok is None:
            sys.exit("this checkpoint carries no tokenizer: pass --ids and prompts as token ids, or --tokenizer <gguf>")
        else:
            a, b = tok.encode(before), tok.encode(after)
        out = model.generate(a + b, args.max_new_tokens, soft=soft, soft_at=len(a))
        text = tok.decode(out) if tok is not None else " ".join(map(str, out))
        print(json.dumps({"prompt": p, "audio_tokens": soft.shape[0], "completion": text, "token_ids": out}))


def cmd_generate(args):
    from .serve.engine import SamplingParams
    if getattr(args, "audio", ""):
        if not (_is_gemma4(args.model) and args.audio_model):
            sys.exit("--audio needs a gemma4 GGUF as --model and --audio-model <checkpoint with the audio tower>")
        return _generate_with_audio(args)
    llm = _load_llm(args)
    prompts = args.prompt or ["Hello"]
    sp = SamplingParams(max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, seed=args.seed)
    enc = []
    for p in prompts:
        if args.ids:
            enc.append([int(x) for x in p.replace(",", " ").split()])
        elif llm.tokenizer is None:
            sys.exit("this checkpoint carries no tokenizer: pass --ids and prompts as token ids, or --tokenizer <gguf>")
        else:
            enc.append(llm.tokenizer.encode(p))
    t0 = time.time()
    stats = None
    if args.speculative > 0 and not hasattr(llm, "generate_speculative"):
        sys.exit("--speculative needs the continuous-batching engine: this model family is served one request at a time")
    if args.speculative > 0:
        if args.temperature != 0.0:
            sys.exit("--speculative verifies drafts against greedy choices: use it with --temperature 0")
        outs, stats = llm.generate_speculative(enc, args.max_new_tokens, gamma=args.speculative)
    else:
        outs = llm.generate(enc, sp)
    dt = time.time() - t0
    n_new = sum(len(o) for o in outs)
    for p, o in zip(prompts, outs):
        text = llm.decode(o) if llm.tokenizer is not None else " ".join(map(str, o))
        print(json.dumps({"prompt": p, "completion": text, "token_ids": o}))
    summary = {"new_tokens": n_new, "seconds": round(dt, 3), "tokens_per_s": round(n_new / max(dt, 1e-9), 1)}
    if stats is not None:
        summary.update(verify_steps=stats.verify_steps, draft_acceptance=round(stats.acceptance, 3), tokens_per_step=round(stats.tokens_per_step, 2))
    print(json.dumps(summary), file=sys.stderr)


def cmd_serve(args):
    from .serve.server import serve
    llm = _load_llm(args)
    if args.speculative > 0 and not hasattr(llm, "set_drafter"):
        sys.exit("--speculative needs the continuous-batching engine: this model family is served one request at a time")
    if args.speculative > 0:
        from .serve.speculative import NgramDrafter
        llm.set_drafter(NgramDrafter(gamma=args.speculative))
    vis = None
    if getattr(args, "mmproj", ""):
        import torch
        from .models import vision
        dev = str(llm.device) if hasattr(llm, "device") else "cpu"
        vis = vision.load_gguf(args.mmproj, dev, torch.bfloat16 if dev.startswith("cuda") else torch.float32)
    print(f"serving {args.model} on http://{args.host}:{args.port}", file=sys.stderr)
    serve(llm, host=args.host, port=args.port, model_name=args.name or args.model, block=True, vision=vis)


def cmd_encode_image(args):
    """Image -> vision tokens (the reference's vision_encode behind its server, server/server_llm.c:503-518): the image is cut to
    whole merge cells (patch_size * spatial_merge pixels); resize it beforehand if it is larger than the encoder's trained grid."""
    import numpy as np
    import torch
    from .models import vision
    with open(args.image, "rb") as fh:
        try:
            rgb = vision.decode_image(fh.read())
        except ValueError as e:
            sys.exit(str(e))
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    enc = vision.load_gguf(args.mmproj, dev, torch.bfloat16 if dev == "cuda" else torch.float32)
    cell = enc.cfg.patch_size * enc.cfg.spatial_merge
    if args.max_side > 0 and max(rgb.shape[0], rgb.shape[1]) > args.max_side:
        f = args.max_side / max(rgb.shape[0], rgb.shape[1])
        rgb = vision.resize_image(rgb, max(cell, int(rgb.shape[0] * f)), max(cell, int(rgb.shape[1] * f)))
    h, w = rgb.shape[0] // cell * cell, rgb.shape[1] // cell * cell
    feats = enc.encode(enc.normalize_image(rgb[:h, :w].to(dev)))
    if args.out:
        np.save(args.out, feats.cpu().numpy())
    print(json.dumps({"image": [h, w], "tokens": feats.shape[0], "features_per_token": feats.shape[1], "deepstack_slices": feats.shape[1] // enc.cfg.proj_dim - 1}))
    return 0


def cmd_encode_audio(args):
    """WAV -> log-mel -> Conformer soft tokens (the audio path of the reference's Gemma4 driver, cuda/llm/test_gemma4_st.c:83-104:
    the clip is cut to ``--max-seconds`` first, 30 s being what the model was trained on)."""
    import numpy as np
    import torch
    from .models import audio
    pcm, rate = audio.wav_load(args.wav)
    if rate != audio.RATE:
        sys.exit(f"{args.wav}: {rate} Hz; the encoder takes {audio.RATE} Hz mono (resample beforehand)")
    if args.max_seconds > 0:
        pcm = pcm[: int(args.max_seconds * audio.RATE)]
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    enc = audio.Gemma4AudioEncoder.from_checkpoint(args.model, device=dev, dtype=torch.bfloat16 if dev == "cuda" else torch.float32)
    mel = audio.log_mel(pcm)
    soft = enc.encode(mel)
    if args.out:
        np.save(args.out, soft.float().cpu().numpy())
    print(json.dumps({"seconds": round(pcm.numel() / audio.RATE, 3), "mel_frames": mel.shape[0], "tokens": soft.shape[0], "features_per_token": soft.shape[1]}))
    return 0


def cmd_mesh(args):
    """Scalar grid (.npy, [nx, ny, nz]) -> welded triangle mesh of its level set (PLY or OBJ), optionally a preview image of it
    (the reference: common/marching_cubes.h mc_write_ply / mc_write_obj, common/preview_render.h)."""
    import numpy as np
    import torch
    from . import geometry as geo
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    grid = torch.from_numpy(np.load(args.grid).astype(np.float32)).to(dev)
    verts, tris = geo.isosurface(grid, args.iso, bounds=args.bounds)
    (geo.write_mesh_obj if args.out.endswith(".obj") else geo.write_mesh_ply)(args.out, verts, tris)
    line = {"vertices": verts.shape[0], "triangles": tris.shape[0], "area": round(geo.mesh_area(verts, tris), 6), "volume": round(geo.mesh_volume(verts, tris), 6)}
    if args.render and tris.shape[0]:
        lo, hi = verts.min(0).values.cpu(), verts.max(0).values.cpu()
        mid, rad = (lo + hi) / 2, float((hi - lo).norm()) / 2
        eye = (float(mid[0]) + 0.8 * rad, float(mid[1]) + 0.9 * rad, float(mid[2]) - 2.6 * rad)
        img = geo.Bvh(verts, tris, device=dev).render(eye, tuple(float(x) for x in mid), args.size, args.size)
        geo.write_ppm(args.render, img["rgb"])
        line["preview"] = args.render
        line["coverage"] = round(float(img["mask"].mean()), 4)
    print(json.dumps(line))
    return 0


def cmd_inspect(args):
    from .utils import gguf as G
    with G.GGUFFile(args.file) as f:
        print(f"version {f.version}  alignment {f.alignment}  tensors {len(f.tensors)}  kv {len(f.metadata)}")
        for k, v in f.metadata.items():
            s = repr(v)
            print(f"  {k} = {s if len(s) < 100 else s[:97] + '...'}")
        if args.tensors:
            for t in f.tensors.values():
                print(f"  {t.name:48s} {str(tuple(t.shape)):28s} {t.type_name:8s} bytes {t.nbytes}")


def cmd_tokenize(args):
    from .utils import gguf as G
    from .utils.tokenizer import Tokenizer
    with G.GGUFFile(args.file) as f:
        tok = Tokenizer.from_gguf(f)
    ids = tok.encode(args.text)
    print(json.dumps({"ids": ids, "pieces": [tok.decode([i]) for i in ids], "roundtrip": tok.decode(ids)}, ensure_ascii=False))


def cmd_stage(args):
    import os
    from .models import loader
    from .utils import gguf as G
    from .utils import stage
    if os.path.isdir(args.model):
        cfg, src = loader.config_from_hf(args.model), loader.SafetensorsSource(args.model)
    else:
        f = G.GGUFFile(args.model)
        cfg, src = loader.config_from_gguf(f), loader.GGUFSource(f)
    stage.stage(cfg, src, args.out, args.format, tp_size=args.tp, ep_size=args.ep)
    print(json.dumps({"ranks": max(args.tp, args.ep), "out": args.out}))


def cmd_compare(args):
    """CPU-vs-GPU comparison token by token (cuda/llm/test_cuda_llm.c prints the same: per-token arg-max of both sides and the
    logit difference), plus the token agreement and edit distance of the two greedy continuations (ref/llm/llm_server.py)."""
    import os
    import torch
    from .models import loader, reference
    from .models.config import get_config
    from .models.transformer import ForwardBatch, KvCache, Transformer
    from .models.weights import synthetic_weights
    if getattr(args, "hf", False):
        from .utils import hf_compare
        vocab = get_config(args.model.split(":", 1)[1]).vocab if args.model.startswith("synthetic:") else loader.config_from_hf(args.model).vocab
        g = torch.Generator().manual_seed(args.seed)
        prompt = [int(x) for x in args.ids.replace(",", " ").split()] if args.ids else torch.randint(0, vocab, (args.prompt_len,), generator=g).tolist()
        print(json.dumps(hf_compare.compare(args.model, prompt, args.steps, args.format, "cuda" if torch.cuda.is_available() else "cpu", args.seed)))
        return 0
    if args.model.startswith("synthetic:"):
        w_cpu = synthetic_weights(get_config(args.model.split(":", 1)[1]), args.format, device="cpu", seed=args.seed)
    elif os.path.isdir(args.model):
        w_cpu = loader.load_safetensors(args.model, args.format, "cpu")
    else:
        w_cpu = loader.load_gguf(args.model, args.format, "cpu")
    cfg = w_cpu.cfg
    g = torch.Generator().manual_seed(args.seed)
    prompt = [int(x) for x in args.ids.replace(",", " ").split()] if args.ids else torch.randint(0, cfg.vocab, (args.prompt_len,), generator=g).tolist()
    page = 16
    n_pages = (len(prompt) + args.steps + page) // page + 1
    bt = torch.arange(n_pages, dtype=torch.int32).unsqueeze(0)
    sides = {"cpu": Transformer(w_cpu, KvCache.allocate(cfg, n_pages, page, "cpu"))}
    if torch.cuda.is_available():
        sides["gpu"] = Transformer(w_cpu.to("cuda"), KvCache.allocate(cfg, n_pages, page, "cuda"))
    outs = {}
    for name, m in sides.items():
        dev = "cpu" if name == "cpu" else "cuda"
        toks, rows = list(prompt), []
        fb = ForwardBatch.build([len(toks)], [0], torch.tensor(toks), bt, page, cfg.n_heads, cfg.n_kv_heads, dev)
        logits = m.forward(fb).float().cpu()[0]
        for _ in range(args.steps):
            rows.append(logits)
            toks.append(int(logits.argmax()))
            fb = ForwardBatch.build([1], [len(toks) - 1], torch.tensor(toks[-1:]), bt, page, cfg.n_heads, cfg.n_kv_heads, dev)
            logits = m.forward(fb).float().cpu()[0]
        outs[name] = (toks[len(prompt):], rows)
    report = {"prompt_len": len(prompt), "steps": args.steps, "cpu_tokens": outs["cpu"][0]}
    if args.oracle:
        ref = reference.reference_logits(w_cpu, torch.tensor(prompt))[-1]
        report["cpu_vs_fp32_oracle_rel"] = float((outs["cpu"][1][0] - ref).norm() / ref.norm())
    if "gpu" in outs:
        a, b = outs["cpu"], outs["gpu"]
        rel = [float((x - y).norm() / (x.norm() + 1e-12)) for x, y in zip(a[1], b[1])]
        agree = sum(int(x == y) for x, y in zip(a[0], b[0]))
        # Levenshtein distance of the two continuations
        d = list(range(len(b[0]) + 1))
        for i, x in enumerate(a[0], 1):
            prev, d[0] = d[0], i
            for j, y in enumerate(b[0], 1):
                prev, d[j] = d[j], min(d[j] + 1, d[j - 1] + 1, prev + (x != y))
        report.update(gpu_tokens=b[0], logit_rel_per_step=[round(r, 5) for r in rel], token_agreement=agree / max(1, args.steps), edit_distance=d[-1])
    print(json.dumps(report))


def cmd_dump(args):
    """Hidden state after every layer + final logits of one prompt as ``.npy`` files (f32): the layer-by-layer debugging aid the
    reference gets from its npy writer (common/npy_io.h) and safetensors_writer.h dumps."""
    import os
    import numpy as np
    import torch
    from .models import loader
    from .models.config import get_config
    from .models.transformer import ForwardBatch, KvCache, Transformer
    from .models.weights import synthetic_weights
    dev = args.device if (args.device != "cuda" or torch.cuda.is_available()) else "cpu"
    if args.model.startswith("synthetic:"):
        w = synthetic_weights(get_config(args.model.split(":", 1)[1]), args.format, device=dev, seed=args.seed)
    elif os.path.isdir(args.model):
        w = loader.load_safetensors(args.model, args.format, dev)
    else:
        w = loader.load_gguf(args.model, args.format, dev)
    cfg = w.cfg
    ids = [int(x) for x in args.ids.replace(",", " ").split()]
    page = 16
    n_pages = len(ids) // page + 2
    m = Transformer(w, KvCache.allocate(cfg, n_pages, page, dev))
    m.snapshot_layers = tuple(range(len(w.layers)))
    bt = torch.arange(n_pages, dtype=torch.int32).unsqueeze(0)
    fb = ForwardBatch.build([len(ids)], [0], torch.tensor(ids), bt, page, cfg.n_heads, cfg.n_kv_heads, dev)
    fb.logit_rows = torch.arange(len(ids), device=fb.ids.device)
    logits = m.forward(fb).float().cpu()
    os.makedirs(args.out, exist_ok=True)
    for li, h in sorted(m.snapshots.items()):
        np.save(os.path.join(args.out, f"layer_{li:03d}.npy"), h.float().cpu().numpy())
    np.save(os.path.join(args.out, "logits.npy"), logits.numpy())
    print(json.dumps({"layers": len(m.snapshots), "tokens": len(ids), "out": args.out, "argmax_last": int(logits[-1].argmax())}))


def cmd_build(args):
    from . import build
    build.build_all(verbose=True)


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] in ("microbench", "estimate"):          # these take their own flags: hand the rest over untouched
        mod = __import__(f"gemm_b200.utils.{argv[0]}", fromlist=["main"])
        return mod.main(argv[1:])
    ap = argparse.ArgumentParser(prog="python -m gemm_b200", description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="complete prompts")
    _add_model_args(g)
    g.add_argument("--prompt", action="append", help="prompt text (repeatable); with --ids, space separated token ids")
    g.add_argument("--ids", action="store_true")
    g.add_argument("--max-new-tokens", type=int, default=64)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--audio", default="", help="16 kHz WAV clip for a gemma4 model; write <audio> in the prompt where it belongs")
    g.add_argument("--audio-model", default="", help="safetensors checkpoint holding the gemma4 audio tower")
    g.add_argument("--speculative", type=int, default=0, metavar="GAMMA",
                   help="greedy speculative decoding with prompt-lookup drafts of up to GAMMA tokens, verified in one batched step")
    g.set_defaults(fn=cmd_generate)
    s = sub.add_parser("serve", help="HTTP server")
    _add_model_args(s)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8080)
    s.add_argument("--speculative", type=int, default=0, metavar="GAMMA",
                   help="greedy requests decode speculatively with prompt-lookup drafts of up to GAMMA tokens")
    s.add_argument("--name", default="")
    s.add_argument("--mmproj", default="", help="GGUF file of the Qwen3-VL vision encoder: requests may then carry \"image\" (base64 PPM / .npy)")
    s.set_defaults(fn=cmd_serve)
    i = sub.add_parser("inspect", help="dump a GGUF file")
    i.add_argument("file")
    i.add_argument("--tensors", action="store_true")
    i.set_defaults(fn=cmd_inspect)
    t = sub.add_parser("tokenize", help="tokenize a text")
    t.add_argument("file")
    t.add_argument("text")
    t.set_defaults(fn=cmd_tokenize)
    st = sub.add_parser("stage", help="per-rank weight blobs")
    st.add_argument("--model", required=True)
    st.add_argument("--out", required=True)
    st.add_argument("--format", default="mxfp8", choices=["bf16", "mxfp8"])
    st.add_argument("--tp", type=int, default=1)
    st.add_argument("--ep", type=int, default=1)
    st.set_defaults(fn=cmd_stage)
    mb = sub.add_parser("microbench", help="kernel micro-benchmarks")
    mb.add_argument("rest", nargs=argparse.REMAINDER)
    mb.set_defaults(fn=lambda a: __import__("gemm_b200.utils.microbench", fromlist=["main"]).main(a.rest))
    es = sub.add_parser("estimate", help="roofline estimate")
    es.add_argument("rest", nargs=argparse.REMAINDER)
    es.set_defaults(fn=lambda a: __import__("gemm_b200.utils.estimate", fromlist=["main"]).main(a.rest))
    cb = sub.add_parser("cpubench", help="native CPU engine against the reference CPU engine (Qwen3-0.6B shape, Q8_0)")
    cb.add_argument("rest", nargs=argparse.REMAINDER)
    cb.set_defaults(fn=lambda a: __import__("gemm_b200.utils.cpubench", fromlist=["main"]).main(a.rest))
    cp = sub.add_parser("compare", help="CPU path against GPU kernels, token by token")
    cp.add_argument("--model", required=True, help="GGUF file, HF safetensors directory, or synthetic:<preset>")
    cp.add_argument("--format", default="bf16", choices=["bf16", "mxfp8"])
    cp.add_argument("--ids", default="", help="prompt as token ids (default: random ids)")
    cp.add_argument("--prompt-len", type=int, default=32)
    cp.add_argument("--steps", type=int, default=8)
    cp.add_argument("--seed", type=int, default=0)
    cp.add_argument("--oracle", action="store_true", help="also compare the CPU path with the fp32 oracle")
    cp.add_argument("--hf", action="store_true", help="compare against Hugging Face transformers (fp32) on the same checkpoint instead: an "
                    "HF directory or synthetic:<preset> of a Qwen2 / Qwen3 / Qwen3-MoE architecture")
    cp.set_defaults(fn=cmd_compare)
    dp = sub.add_parser("dump", help="per-layer hidden states as .npy")
    dp.add_argument("--model", required=True, help="GGUF file, HF safetensors directory, or synthetic:<preset>")
    dp.add_argument("--format", default="bf16", choices=["bf16", "mxfp8"])
    dp.add_argument("--device", default="cuda")
    dp.add_argument("--ids", required=True, help="prompt as token ids")
    dp.add_argument("--out", required=True)
    dp.add_argument("--seed", type=int, default=0)
    dp.set_defaults(fn=cmd_dump)
    ei = sub.add_parser("encode-image", help="run the Qwen3-VL vision encoder (mmproj GGUF) on an image")
    ei.add_argument("--mmproj", required=True, help="GGUF file of the vision encoder")
    ei.add_argument("--image", required=True, help="PNG, baseline JPEG, binary PPM (P6) or .npy (uint8 [H, W, 3])")
    ei.add_argument("--max-side", type=int, default=0, help="shrink the image so that its longer side is at most this many pixels (0: keep)")
    ei.add_argument("--out", default="", help="write the features ([tokens, proj_dim * (1 + deepstack)] f32) as .npy")
    ei.set_defaults(fn=cmd_encode_image)
    ea = sub.add_parser("encode-audio", help="run the Gemma4 audio encoder (safetensors checkpoint) on a 16 kHz WAV file")
    ea.add_argument("--model", required=True, help="checkpoint directory or .safetensors file holding model.audio_tower.*")
    ea.add_argument("--wav", required=True)
    ea.add_argument("--max-seconds", type=float, default=30.0, help="cut the clip (0: keep all of it)")
    ea.add_argument("--out", default="", help="write the soft tokens ([tokens, 1536] f32) as .npy")
    ea.set_defaults(fn=cmd_encode_audio)
    ms = sub.add_parser("mesh", help="level set of a scalar grid (.npy) as a triangle mesh, with an optional preview image")
    ms.add_argument("--grid", required=True, help=".npy file, float [nx, ny, nz]; values below --iso are inside")
    ms.add_argument("--iso", type=float, default=0.0)
    ms.add_argument("--bounds", type=float, nargs=6, default=None, metavar=("XMIN", "YMIN", "ZMIN", "XMAX", "YMAX", "ZMAX"), help="extent of the grid (default: [-1, 1]^3)")
    ms.add_argument("--out", required=True, help="mesh file, .ply (binary) or .obj")
    ms.add_argument("--render", default="", help="also write a preview image (binary PPM)")
    ms.add_argument("--size", type=int, default=256)
    ms.set_defaults(fn=cmd_mesh)
    b = sub.add_parser("build", help="compile the native libraries")
    b.set_defaults(fn=cmd_build)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
