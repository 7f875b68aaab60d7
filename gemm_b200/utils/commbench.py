"""Collective micro-benchmarks over the peer-memory fabric, with NCCL as the baseline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m gemm_b200.utils.commbench [--iters 20]

Measures, at the message sizes of the model's call sites (decode: a few rows of the hidden state; prefill: a 16384-token
chunk), the one-shot and two-shot all-reduce, the push all-gather and the push all-to-all of ``parallel/fabric.py`` against
``torch.distributed`` (NCCL).  Times are CUDA-event medians on the launching stream, the maximum over ranks; rank 0 prints one
JSON line per measurement with the latency, the algorithm bandwidth (bytes of one rank's buffer / time) and the bus bandwidth
(x 2(N-1)/N for all-reduce, x (N-1)/N for all-gather and all-to-all, the convention of nccl-tests).

Counterpart in the reference: the collective benchmarks of a64fx/utofu-tests (allreduce / reducescatter_bench.c / allgather_bench.c /
moe_dispatch_bench.c, tabulated in summary.md), which time the same patterns on its interconnect.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time(fn, iters: int, warm: int = 3) -> float:
    """Median milliseconds over ``iters`` timed calls, maximum over ranks."""
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(iters):
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _emit(rank: int, name: str, nbytes: int, ms: float, bus_factor: float, **kw) -> None:
    if rank == 0:
        alg = nbytes / ms / 1e6
        print(json.dumps(dict(case=name, bytes=nbytes, us=round(ms * 1e3, 2), alg_gbs=round(alg, 1), bus_gbs=round(alg * bus_factor, 1), **kw)),
              flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--no-nccl", action="store_true")
    args = ap.parse_args(argv)
    from ..parallel.fabric import Fabric
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    h = args.hidden
    big_rows = 16384
    fab = Fabric(dist.group.WORLD, dev, heap_bytes=(6 * big_rows * h * 2) + (64 << 20))
    ar_f, ag_f = 2.0 * (world - 1) / world, (world - 1) / world

    # ---- all-reduce, decode sizes: fp32 rows of the hidden state (one-shot kernel: push to every peer, sum in rank order)
    for rows in (1, 8, 64):
        n = rows * h
        one = fab.make_allreduce(n, torch.float32)
        x = torch.randn(n, device=dev)
        _emit(rank, "allreduce_oneshot_f32", n * 4, _time(lambda: one(x), args.iters), ar_f, rows=rows, world=world)
        if not args.no_nccl:
            y = x.clone()
            _emit(rank, "nccl_allreduce_f32", n * 4, _time(lambda: dist.all_reduce(y), args.iters), ar_f, rows=rows, world=world)
    # ---- all-reduce, prefill size: bf16 chunk (two-shot kernel: reduce-scatter by peer loads + all-gather by peer stores)
    n = big_rows * h
    two = fab.make_allreduce_large(n, torch.bfloat16)
    xb = torch.randn(n, device=dev).bfloat16()
    _emit(rank, "allreduce_twoshot_bf16", n * 2, _time(lambda: two(xb), args.iters), ar_f, rows=big_rows, world=world)
    if not args.no_nccl:
        yb = xb.clone()
        _emit(rank, "nccl_allreduce_bf16", n * 2, _time(lambda: dist.all_reduce(yb), args.iters), ar_f, rows=big_rows, world=world)
    # ---- all-gather and all-to-all by peer stores (token rows of the expert-parallel routes)
    for rows in (8, 64, 2048):
        per = rows * h * 2
        ex = fab.make_exchange(per)
        src = torch.randn(rows * h, device=dev).bfloat16()
        _emit(rank, "allgather_push_bf16", per * world, _time(lambda: ex.all_gather(src), args.iters), ag_f, rows_per_rank=rows, world=world)
        if not args.no_nccl:
            out = torch.empty(world * rows * h, dtype=torch.bfloat16, device=dev)
            _emit(rank, "nccl_allgather_bf16", per * world, _time(lambda: dist.all_gather_into_tensor(out, src), args.iters), ag_f,
                  rows_per_rank=rows, world=world)
        srcs = torch.randn(world, rows * h, device=dev).bfloat16()
        _emit(rank, "alltoall_push_bf16", per * world, _time(lambda: ex.all_to_all(srcs), args.iters), ag_f, rows_per_pair=rows, world=world)
        if not args.no_nccl:
            out2 = torch.empty_like(srcs)
            _emit(rank, "nccl_alltoall_bf16", per * world, _time(lambda: dist.all_to_all_single(out2, srcs), args.iters), ag_f,
                  rows_per_pair=rows, world=world)
    from .. import _native
    st = _native.read_status()["what"]
    if rank == 0:
        print(json.dumps(dict(kernel_status=st)), flush=True)
    dist.barrier()
    fab.close()


if __name__ == "__main__":
    main()
