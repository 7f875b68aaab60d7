"""Cost of ONE context-parallel decode attention step, split into its two parts, with the merge done three ways:

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m gemm_b200.utils.ringbench [--seq 16384 --batch 8]

1. **KV read**: the cache of length ``--seq`` is dealt to the N ranks, every rank runs the decode attention of the batch over its
   ``seq / N`` positions (the decode kernel on a GPU, the tensor-op partial on CPU) and gets partials
   (output, log-sum-exp) per query head;
2. **merge** of the partials, ``Hq * (D + 1)`` floats per token and rank: the all-gather + combine the engine uses
   (``ContextParallel.attention``), a ring (``world - 1`` hops, ``parallel.context.merge_ring``) and recursive doubling
   (``log2(world)`` rounds, ``merge_tree``).

From the measured read time, hop time and round time rank 0 also prints the projection for other rank counts (read ~ 1 / N, ring
~ (N - 1) hops, tree ~ ceil(log2 N) rounds) and the N at which the merge starts to cost more than the read.  This is the
measurement of the reference's a64fx/utofu-tests/ring_attn_bench.c (which models the read from a bandwidth probe and times
the hops on its interconnect) on this framework's own kernels and transports.  On a GPU the times are CUDA-event medians on the
launching stream, the maximum over ranks; on CPU (gloo) they are wall-clock medians and say so.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import time

import torch
import torch.distributed as dist


def _median_ms(fn, iters: int, warm: int, cuda: bool) -> float:
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(iters):
        dist.barrier()
        if cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        else:
            t0 = time.perf_counter()
            fn()
            ts.append((time.perf_counter() - t0) * 1e3)
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], dtype=torch.float64, device="cuda" if cuda else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def projection(read_ms: float, hop_ms: float, round_ms: float, world: int, upto: int = 64):
    """Rows ``{n, read_ms, ring_ms, tree_ms}`` for n = 1, 2, 4, ...: the read of a shard scales with 1 / n from the measured world."""
    rows, n = [], 1
    while n <= upto:
        rows.append({"n": n, "read_ms": round(read_ms * world / n, 4), "ring_ms": round(hop_ms * (n - 1), 4),
                     "tree_ms": round(round_ms * math.ceil(math.log2(n)) if n > 1 else 0.0, 4)})
        n *= 2
    return rows


def crossover(rows, key: str):
    """Smallest n of the projection whose merge costs more than its read (None: not within the table)."""
    for r in rows:
        if r["n"] > 1 and r[key] > r["read_ms"]:
            return r["n"]
    return None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--seq", type=int, default=16384, help="context length of every sequence (dealt to the ranks)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--qh", type=int, default=32)
    ap.add_argument("--kvh", type=int, default=8)
    ap.add_argument("--hd", type=int, default=128)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args(argv)
    from ..ops import attention as att
    from ..ops import elementwise as ew
    from ..parallel import context as cpx
    cuda = torch.cuda.is_available()
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    if cuda:
        torch.cuda.set_device(lr)
        dev = torch.device("cuda", lr)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    page = 128
    local = (args.seq + world - 1) // world                     # positions of a sequence on this rank
    pages = (local + page - 1) // page
    b, hq, hkv, d = args.batch, args.qh, args.kvh, args.hd
    g = torch.Generator().manual_seed(rank)
    k = (torch.randn(b * pages * page, hkv, d, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    v = (torch.randn(b * pages * page, hkv, d, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    q = (torch.randn(b, hq, d, generator=torch.Generator().manual_seed(99)) * 0.5 * ew.softmax_scale_log2(d)).to(torch.bfloat16).to(dev)
    cu = torch.arange(b + 1, dtype=torch.int32, device=dev)
    kv_len = torch.full((b,), local, dtype=torch.int32, device=dev)
    bt = torch.arange(b * pages, dtype=torch.int32, device=dev).reshape(b, pages)
    splits = att.pick_splits(b, hkv, local) if cuda else 1
    work = att.build_work([1] * b, hq, hkv, splits).to(dev)

    def read():
        return att.attention_partial(q, k, v, cu, kv_len, bt, page, work, num_splits=splits, causal=False, decode=True)

    po, pl = read()
    if splits > 1:                                               # one partial per rank for the merges
        o1, l1 = att.combine_partials(po.reshape(splits, b * hq, d), pl.reshape(splits, b * hq))
        o1, l1 = o1.float().reshape(b, hq, d), l1.reshape(b, hq)
    else:
        o1, l1 = po[0], pl[0]

    def gather_merge():
        parts = [torch.empty(b * hq, d + 1, dtype=torch.float32, device=dev) for _ in range(world)]
        dist.all_gather(parts, torch.cat([o1.reshape(b * hq, d), l1.reshape(b * hq, 1)], dim=1).contiguous())
        allp = torch.stack(parts)
        return att.combine_partials(allp[:, :, :d].contiguous(), allp[:, :, d].contiguous())

    read_ms = _median_ms(read, args.iters, args.warmup, cuda)
    out = {"world": world, "device": "cuda" if cuda else "cpu", "timing": "cuda events, median, max over ranks" if cuda else "wall clock, median, max over ranks",
           "config": {"seq": args.seq, "batch": b, "q_heads": hq, "kv_heads": hkv, "head_dim": d, "positions_per_rank": local, "kv_splits": splits},
           "kv_bytes_per_rank": 2 * b * local * hkv * d * 2, "payload_bytes": b * hq * (d + 1) * 4, "read_ms": round(read_ms, 4)}
    out["read_gbs"] = round(out["kv_bytes_per_rank"] / (read_ms * 1e-3) / 1e9, 1)
    if world > 1:
        gather_ms = _median_ms(gather_merge, args.iters, args.warmup, cuda)
        ring_ms = _median_ms(lambda: cpx.merge_ring(o1, l1), args.iters, args.warmup, cuda)
        tree_ms = _median_ms(lambda: cpx.merge_tree(o1, l1), args.iters, args.warmup, cuda)
        want, _ = gather_merge()
        ring_o, _ = cpx.merge_ring(o1, l1)
        tree_o, _ = cpx.merge_tree(o1, l1)
        err = lambda x: ((x.reshape(b * hq, d).float() - want.float()).norm() / want.float().norm()).item()
        hop, rnd = ring_ms / (world - 1), tree_ms / math.ceil(math.log2(world))
        rows = projection(read_ms, hop, rnd, world)
        out.update({"all_gather_merge_ms": round(gather_ms, 4), "ring_merge_ms": round(ring_ms, 4), "tree_merge_ms": round(tree_ms, 4),
                    "hop_ms": round(hop, 4), "round_ms": round(rnd, 4), "ring_rel_err": round(err(ring_o), 6), "tree_rel_err": round(err(tree_o), 6),
                    "projection": rows, "crossover_ring_n": crossover(rows, "ring_ms"), "crossover_tree_n": crossover(rows, "tree_ms")})
    if rank == 0:
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
