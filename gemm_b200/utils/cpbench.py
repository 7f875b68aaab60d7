"""Long-context benchmark of context parallelism: a dense model's prefill and decode with the KV cache of every sequence dealt to
the ranks page by page (``parallel.context.ContextParallel`` as the engine's parallel context), against the same engine on one GPU:

    python -m gemm_b200.utils.cpbench --layers 8 --batch 4 --ctx 32768
    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 -m gemm_b200.utils.cpbench --layers 8 --batch 4 --ctx 32768

Synthetic token ids, random-init weights of the named shape (``--layers`` of them), CUDA events on the launching stream, maximum
over the ranks.  Prints one JSON line: prefill tokens/s, decode ms per step, KV bytes per rank.

The reference measures this layout on its own hardware as tokens/s of its ring of A64FX nodes (a64fx/m3/m3_ep_runner.c:121-140);
its cost model is tools/decode_estimate.py, ours ``utils.estimate.context_parallel_decode``.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--fmt", default="bf16")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args(argv)
    import torch.distributed as dist
    from ..models.config import get_config
    from ..models.weights import synthetic_weights
    from ..serve.engine import Engine, SamplingParams
    rank, world, lr = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    cfg = get_config(args.model)
    par = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from ..parallel.context import ContextParallel
        par = ContextParallel(dist.group.WORLD, dev, block=128, max_tokens=args.batch, hq=cfg.n_heads, head_dim=cfg.head_dim, max_splits=16)
    w = synthetic_weights(cfg, args.fmt, device=dev, seed=0, n_layers=args.layers)
    new = args.steps + args.warmup + 8
    eng = Engine(w, max_batch=args.batch, max_seq_len=args.ctx + new + 8, page_size=128, par=par, max_prefill_tokens=16384)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (args.ctx,), generator=g, dtype=torch.int32) for _ in range(args.batch)]

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    eng.prefill([p[:512] for p in prompts], reserve=8)        # warm-up: kernels loaded, workspaces allocated
    eng.reset()
    sync()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    logits = eng.prefill(prompts, reserve=new)
    b.record()
    sync()
    t_prefill = a.elapsed_time(b)
    eng.begin_decode(logits.argmax(-1).to(torch.int32), SamplingParams(temperature=0.0), new, True)
    for _ in range(args.warmup):
        eng.decode_step()
    sync()
    a.record()
    for _ in range(args.steps):
        eng.decode_step()
    b.record()
    sync()
    t_step = a.elapsed_time(b) / args.steps
    tok = eng.decode_step().clone()
    t = torch.tensor([t_prefill, t_step], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    from .. import _native
    st = _native.read_status()
    if rank == 0:
        print(json.dumps({"bench": "context_parallel", "model": args.model, "fmt": args.fmt, "layers": args.layers, "batch": args.batch,
                          "ctx": args.ctx, "n_gpus": world, "prefill_ms": round(float(t[0]), 2),
                          "prefill_tokens_per_s": round(args.batch * args.ctx / float(t[0]) * 1000, 1), "decode_ms_per_step": round(float(t[1]), 4),
                          "decode_splits": eng._splits, "kv_gib_per_rank": round(eng.kv.nbytes() / 2**30, 2),
                          "first_tokens": tok[:4].tolist(), "kernel_status": st["what"]}), flush=True)
    if world > 1:
        dist.barrier()
        os._exit(0)


if __name__ == "__main__":
    main()
