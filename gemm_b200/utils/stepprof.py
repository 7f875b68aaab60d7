"""Per-kernel device times of decode steps of the benchmark model, from a CUPTI activity trace (``torch.profiler``):

    GB_PDL=0 python -m gemm_b200.utils.stepprof --layers 8                                    # one GPU
    GB_PDL=0 torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 -m gemm_b200.utils.stepprof --layers 8   # expert parallel

Builds the Qwen3-30B-A3B shape (MXFP8, random weights) with ``--layers`` layers, prefills 64 x 2048 synthetic tokens, replays the
captured decode step and prints, per rank, the kernels by total time: mean duration, launches per step, microseconds per step.
With programmatic dependent launch off (``GB_PDL=0``) a kernel's duration is its own work plus whatever it waits for on other
GPUs; with it on, durations overlap (a dependent kernel starts under its predecessor's tail) and only their shares mean
something.  Numbers taken under the tracer are for reading the step, not for reporting it (``bench.py`` reports).

Counterpart in the reference: the per-op tables of common/profiler.h printed by cpu/llm/test_transformer.c.
"""
from __future__ import annotations

import argparse
import collections
import os

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="qwen3-30b-a3b")
    ap.add_argument("--fmt", default="mxfp8")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--top", type=int, default=16)
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
        from ..parallel.expert import ExpertParallel
        par = ExpertParallel(dist.group.WORLD, dev, fused=True)
    w = synthetic_weights(cfg, args.fmt, device=dev, seed=0, ep_rank=rank, ep_size=world, n_layers=args.layers)
    bl = args.batch // world
    eng = Engine(w, max_batch=bl, max_seq_len=args.prompt_len + 64, page_size=128, par=par, max_prefill_tokens=16384)
    if par is not None:
        par.attach(eng, cfg, max_tokens=16384)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab, (args.batch, args.prompt_len), generator=g, dtype=torch.int32)
    logits = eng.prefill([prompts[rank * bl + i] for i in range(bl)], reserve=48)
    eng.begin_decode(logits.argmax(-1).to(torch.int32), SamplingParams(temperature=0.0), 48, True)
    for _ in range(6):
        eng.decode_step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(20):
        eng.decode_step()
    b.record()
    torch.cuda.synchronize()
    untraced = a.elapsed_time(b) / 20 * 1000
    if world > 1:
        dist.barrier()
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(args.steps):
            eng.decode_step()
        torch.cuda.synchronize()
    by = collections.OrderedDict()
    for e in prof.events():
        if e.device_type is not None and "cuda" in str(e.device_type).lower():
            d = by.setdefault(e.name[:90], [0, 0.0])
            d[0] += 1
            d[1] += e.device_time
    tot = sum(v[1] for v in by.values())
    out = [f"rank {rank} of {world}: {args.layers} layers, step {untraced:.0f} us untraced, {tot / args.steps:.0f} us of kernel time per traced step"]
    for k, (n, t) in sorted(by.items(), key=lambda kv: -kv[1][1])[: args.top]:
        out.append(f"  {t / n:8.1f} us x {n / args.steps:6.1f} / step = {t / args.steps:8.0f} us / step  {k}")
    for r in range(world):
        if world > 1:
            dist.barrier()
        if r == rank:
            print("\n".join(out), flush=True)
    if world > 1:
        dist.barrier()
        os._exit(0)              # captured graphs hold the fabric's kernels: leave without tearing the process group down


if __name__ == "__main__":
    main()
