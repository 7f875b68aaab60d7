"""Worker of tests/test_multi_gpu.py: one process per GPU, launched by ``torch.distributed.run``.
Checks the fabric collectives against values computed from an NCCL all-gather in fixed rank order, and the
expert-parallel engine (fused peer-memory path and NCCL baseline) against the single-GPU engine."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gemm_b200 import _native  # noqa: E402
from gemm_b200.models.config import get_config  # noqa: E402
from gemm_b200.models.transformer import ForwardBatch, KvCache, Transformer  # noqa: E402
from gemm_b200.models.weights import synthetic_weights  # noqa: E402
from gemm_b200.parallel.expert import ExpertParallel  # noqa: E402
from gemm_b200.parallel.fabric import Fabric  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def check_collectives(fab, rank, world, dev):
    torch.manual_seed(100 + rank)
    for dtype in (torch.float32, torch.bfloat16):
        ar = fab.make_allreduce(4096, dtype, chunks=4)
        for n in (8, 1000 if dtype == torch.float32 else 1000 // 8 * 8, 4096):
            x = torch.randn(n, device=dev).to(dtype)
            gathered = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(gathered, x)
            ref = torch.zeros(n, device=dev)
            for g in gathered:
                ref += g.float()
            for _ in range(3):                       # repeated calls exercise the epoch counters
                y = ar(x)
            assert torch.equal(y, ref.to(dtype)), f"one-shot all-reduce mismatch {dtype} n={n}"
        big = fab.make_allreduce_large(1 << 18, dtype, chunks=16)
        x = torch.randn(200000 // 64 * 64, device=dev).to(dtype)
        gathered = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(gathered, x)
        ref = torch.zeros(x.numel(), device=dev)
        for g in gathered:
            ref += g.float()
        for _ in range(2):
            y = big(x)
        assert torch.equal(y, ref.to(dtype)), f"two-shot all-reduce mismatch {dtype}"
    ex = fab.make_exchange(4096, chunks=2)
    x = torch.full((1024,), float(rank), device=dev)
    ag = ex.all_gather(x).view(torch.float32).view(world, 1024)
    assert all(bool((ag[r] == r).all()) for r in range(world))
    x2 = (torch.arange(world, device=dev, dtype=torch.float32).unsqueeze(1) * 10 + rank).repeat(1, 1024).contiguous()
    a2a = ex.all_to_all(x2).view(torch.float32).view(world, 1024)
    assert all(bool((a2a[r] == rank * 10 + r).all()) for r in range(world))
    am = fab.make_argmax(16)
    val = torch.tensor([1.0, 5.0, float(rank), 7.0], device=dev)
    idx = torch.tensor([rank, 100 - rank, 3, 10 + rank], dtype=torch.int32, device=dev)
    oi, ov = am(val, idx)
    assert oi.tolist() == [0, 100 - (world - 1), 3, 10] and ov.tolist() == [1.0, 5.0, float(world - 1), 7.0], (oi, ov)
    # back-to-back calls with fresh data every time and no host synchronisation in between: a rank may be a whole call ahead of a
    # peer, which the alternating slot sets (one-shot, arg-max) and the entry handshake (exchange) have to absorb
    ar = fab.make_allreduce(2048, torch.float32, chunks=2)
    xs = [torch.randn(2048, device=dev) for _ in range(24)]
    refs = []
    for x in xs:
        gathered = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(gathered, x)
        r = torch.zeros_like(x)
        for gx in gathered:
            r += gx
        refs.append(r)
    torch.cuda.synchronize()
    ys = [ar(x) for x in xs]
    for y, r in zip(ys, refs):
        assert torch.equal(y, r), "back-to-back one-shot all-reduce calls interfered"
    ex2 = fab.make_exchange(2048, chunks=1)
    outs = []
    for i in range(16):
        xi = torch.full((512,), float(rank * 100 + i), device=dev)
        outs.append(ex2.all_gather(xi).view(torch.float32).view(world, 512).clone())
    for i, o in enumerate(outs):
        assert all(bool((o[r] == r * 100 + i).all()) for r in range(world)), "back-to-back exchanges interfered"
    vals = [torch.tensor([float((rank * 7 + i) % world), 1.0], device=dev) for i in range(16)]
    got = [am(v, torch.tensor([rank, 50 + rank], dtype=torch.int32, device=dev)) for v in vals]
    for i, (oi, ov) in enumerate(got):
        win = max(range(world), key=lambda r: ((r * 7 + i) % world, -r))
        assert int(oi[0]) == win and float(ov[0]) == float((win * 7 + i) % world) and int(oi[1]) == 50, (i, oi, ov)
    fab.barrier()
    torch.cuda.synchronize()
    _native.assert_status_ok()


def run_model(model, cfg, toks, page, dev):
    """Prefill (two chunks) + 2 decode steps; returns the list of logits tensors."""
    lens = [t.numel() - 2 for t in toks]
    b = len(toks)
    pages_per = [(t.numel() + page - 1) // page for t in toks]
    bt = torch.zeros(b, max(pages_per), dtype=torch.int32)
    p0 = 0
    for s in range(b):
        bt[s, : pages_per[s]] = torch.arange(p0, p0 + pages_per[s])
        p0 += pages_per[s]
    ctx = [0] * b
    outs = []
    for chunk in ([l // 2 for l in lens], [l - l // 2 for l in lens]):
        ids = torch.cat([toks[s][ctx[s]:ctx[s] + chunk[s]] for s in range(b)])
        fb = ForwardBatch.build(chunk, ctx, ids, bt, page, model.hq_local, model.hkv_local, dev)
        outs.append(model.forward(fb).float())
        ctx = [c + q for c, q in zip(ctx, chunk)]
    for step in range(2):
        ids = torch.stack([toks[s][lens[s] + step] for s in range(b)])
        fb = ForwardBatch.build([1] * b, ctx, ids, bt, page, model.hq_local, model.hkv_local, dev)
        outs.append(model.forward(fb).float())
        ctx = [c + 1 for c in ctx]
    return outs


def check_expert_parallel(rank, world, dev, fmt, fused, gather=True):
    cfg = get_config("tiny-moe")
    page = 16
    # every rank gets sequences of the same lengths (the NCCL baseline gathers equal token counts) with its own content
    g = torch.Generator().manual_seed(7 + rank)
    mine = [torch.randint(0, cfg.vocab, (n,), generator=g) for n in (40, 90)]
    w_full = synthetic_weights(cfg, fmt, device=dev, seed=5)
    w_ep = synthetic_weights(cfg, fmt, device=dev, seed=5, ep_rank=rank, ep_size=world)
    ref_model = Transformer(w_full, KvCache.allocate(cfg, 64, page, dev))
    ref = run_model(ref_model, cfg, mine, page, dev)
    par = ExpertParallel(dist.group.WORLD, dev, fused=fused)
    par.use_gather = gather          # True: small batches all-gather their tokens; False: every batch is dispatched row by row

    class _E:            # the slice of the Engine interface that attach() needs
        w = w_ep
    par.attach(_E, cfg, max_tokens=256)
    model = Transformer(w_ep, KvCache.allocate(cfg, 64, page, dev), par)
    got = run_model(model, cfg, mine, page, dev)
    torch.cuda.synchronize()
    _native.assert_status_ok()
    # the two engines round differently (fp32 partial rows summed over ranks against a bf16 combine), and with random-init routers a
    # near-tied expert choice can flip: the bound is loose enough for one flipped pick, far below what a wrong kernel produces
    tol = 4e-2 if fmt == "bf16" else 6e-2
    rels = [rel(a, b) for a, b in zip(got, ref)]
    if rank == 0:
        print(f"EP({fmt}, fused={fused}, gather={gather}) rel per step: {[round(r, 4) for r in rels]}", flush=True)
    for r in rels:
        assert r < tol, f"EP({fmt}, fused={fused}, gather={gather}) differs from the single-GPU engine: rel {r}"
    if fused and gather:
        # the decode steps took the folded forms: all-gather in the RMSNorm's epilogue, combine + scatter inside the expert kernel
        if rank == 0:
            print(f"EP({fmt}) folded launches: {par.stats}", flush=True)
        assert par.stats["fold_gather"] > 0, par.stats
        if fmt == "mxfp8":
            assert par.stats["fold_combine"] > 0, par.stats
    dist.barrier()
    par.close()


def check_tensor_parallel(rank, world, dev, fmt, fused, name="tiny-dense", ep_experts=False):
    """Every rank runs the same sequences on its weight shard; logits must equal the unsharded engine's, and be
    bit-identical across ranks (lock-step greedy decoding needs that).  ``ep_experts``: an MoE model whose experts are
    spread over the same ranks (tensor-parallel attention in front of expert-parallel experts)."""
    from gemm_b200.parallel.tensor import TensorParallel
    cfg = get_config(name)
    page = 16
    g = torch.Generator().manual_seed(11)
    toks = [torch.randint(0, cfg.vocab, (n,), generator=g) for n in (40, 90)]
    w_full = synthetic_weights(cfg, fmt, device=dev, seed=5)
    w_tp = synthetic_weights(cfg, fmt, device=dev, seed=5, tp_rank=rank, tp_size=world, ep_rank=rank if ep_experts else 0,
                             ep_size=world if ep_experts else 1)
    ref = run_model(Transformer(w_full, KvCache.allocate(cfg, 64, page, dev)), cfg, toks, page, dev)
    par = TensorParallel(dist.group.WORLD, dev, fused=fused, ep_experts=ep_experts)
    par.attach(None, cfg, max_tokens=256)
    hkv_local = max(1, cfg.n_kv_heads // world)
    model = Transformer(w_tp, KvCache.allocate(cfg, 64, page, dev, hkv_local), par)
    got = run_model(model, cfg, toks, page, dev)
    torch.cuda.synchronize()
    _native.assert_status_ok()
    tol = 2e-2 if fmt == "bf16" else 6e-2
    for a, b in zip(got, ref):
        r = rel(a, b)
        assert r < tol, f"TP({fmt}, fused={fused}) differs from the single-GPU engine: rel {r}"
    last = got[-1].contiguous()
    gathered = [torch.empty_like(last) for _ in range(world)]
    dist.all_gather(gathered, last)
    if fused:
        assert all(torch.equal(gathered[0], x) for x in gathered), "ranks disagree bitwise after the fused reduction"
    if fused and fmt in ("q4_k", "q8_0"):
        # decode-sized row-parallel projection over ggml blocks: the GEMV's tail stores the partial sums into every GPU's slot
        from gemm_b200.models.weights import make_linear
        from gemm_b200.ops import elementwise as ew
        hidden, k_shard, rows = cfg.hidden, 2048, 2
        gg = torch.Generator(device="cpu").manual_seed(100 + rank)
        lw = make_linear((torch.randn(hidden, k_shard, generator=gg) * 0.05).to(dev), fmt)
        x_sh = torch.randn(rows, k_shard, generator=gg).to(dev).bfloat16()
        resid = torch.randn(rows, hidden, generator=torch.Generator().manual_seed(3)).to(dev).bfloat16()
        nw = torch.ones(hidden, device=dev, dtype=torch.bfloat16)
        pend = par.row_linear(lw, x_sh)
        assert hasattr(pend, "chan"), "the projection was expected to take the fused GEMV path"
        r1 = resid.clone()
        out = par.add_norm(pend, nw, 1e-6, r1)
        full = x_sh.float() @ lw.dequantized().t()
        dist.all_reduce(full)
        r2 = (resid.float() + full).bfloat16()
        torch.cuda.synchronize()
        _native.assert_status_ok()
        assert rel(r1, r2) < 2e-2 and rel(out, ew.rmsnorm_ref(r2, nw, 1e-6)) < 2e-2, f"quantised row-parallel GEMV: {rel(r1, r2)}"
    if fused and fmt in ("bf16", "mxfp8") and not ep_experts:
        # a decode-sized row-parallel projection whose shard is long enough to be cut along K as well (several slabs per rank in
        # the slot): the fused reduction + RMSNorm against all-reduce + norm in PyTorch
        from gemm_b200.models.weights import make_linear
        from gemm_b200.ops import elementwise as ew
        hidden, k_shard, rows = cfg.hidden, 2048, 24
        gg = torch.Generator(device="cpu").manual_seed(100 + rank)
        w_sh = (torch.randn(hidden, k_shard, generator=gg) * 0.05).to(dev)
        x_sh = torch.randn(rows, k_shard, generator=gg).to(dev).bfloat16()
        lw = make_linear(w_sh, fmt)
        resid = torch.randn(rows, hidden, generator=torch.Generator().manual_seed(3)).to(dev).bfloat16()
        nw = torch.ones(hidden, device=dev, dtype=torch.bfloat16)
        pend = par.row_linear(lw, x_sh)
        assert getattr(pend, "splits", 1) > 1, "the projection was expected to take the K-split path"
        r1 = resid.clone()
        out = par.add_norm(pend, nw, 1e-6, r1)
        full = (x_sh.float() @ lw.dequantized().t()) if fmt == "bf16" else None
        if full is None:
            xq = ew.mx_quantize(x_sh, sf_layout=32)
            from gemm_b200.ops import mxfp8 as _mx
            full = _mx.dequantize(xq) @ lw.dequantized().t()
        dist.all_reduce(full)
        r2 = (resid.float() + full).bfloat16()
        want = ew.rmsnorm_ref(r2, nw, 1e-6)
        torch.cuda.synchronize()
        _native.assert_status_ok()
        assert rel(r1, r2) < 1e-2 and rel(out, want) < 1e-2, f"K-split row-parallel projection: {rel(r1, r2)} {rel(out, want)}"
    dist.barrier()
    par.close()


def check_tp_prefill_fused(rank, world, dev):
    """Prefill-sized tensor parallelism with the GEMM -> reduce-scatter / all-gather -> GEMM path: the row-parallel projections
    scatter their partial rows to the rows' owners from the epilogue, the owners' norm kernels gather the normalised rows to
    every rank, the residual stream is sharded in between.  Logits against the unsharded engine, bitwise agreement of the ranks,
    and a rank that owns no rows (4 ranks)."""
    from gemm_b200.parallel.tensor import TensorParallel
    cfg = get_config("tiny-dense")
    page = 16
    g = torch.Generator().manual_seed(21)
    lens = (1203, 1002) if world >= 4 else (603, 802)      # halves: 1100 rows on 4 ranks -> regions of 512: the last rank owns none
    toks = [torch.randint(0, cfg.vocab, (n,), generator=g) for n in lens]
    n_pages = sum((n + page - 1) // page for n in lens) + 2
    w_full = synthetic_weights(cfg, "bf16", device=dev, seed=5)
    w_tp = synthetic_weights(cfg, "bf16", device=dev, seed=5, tp_rank=rank, tp_size=world)
    ref = run_model(Transformer(w_full, KvCache.allocate(cfg, n_pages, page, dev)), cfg, toks, page, dev)
    par = TensorParallel(dist.group.WORLD, dev, fused=True)
    par.attach(None, cfg, max_tokens=4096)
    assert par.sp is not None
    model = Transformer(w_tp, KvCache.allocate(cfg, n_pages, page, dev, max(1, cfg.n_kv_heads // world)), par)
    got = run_model(model, cfg, toks, page, dev)
    torch.cuda.synchronize()
    _native.assert_status_ok()
    assert par.sp_launches >= 2 * 2 * cfg.n_layers, par.sp_launches        # o_proj and down_proj of both prefill chunks
    for a, b in zip(got, ref):
        r = rel(a, b)
        assert r < 2e-2, f"fused TP prefill differs from the single-GPU engine: rel {r}"
    for t in got[:2]:
        t = t.contiguous()
        gathered = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(gathered, t)
        assert all(torch.equal(gathered[0], x) for x in gathered), "ranks disagree bitwise after the fused prefill path"
    dist.barrier()
    par.close()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    if what in ("all", "collectives"):
        fab = Fabric(dist.group.WORLD, dev, 32 << 20)
        check_collectives(fab, rank, world, dev)
        dist.barrier()
        fab.close()
    if what in ("all", "ep"):
        for fmt, fused, gather in (("bf16", True, True), ("mxfp8", True, True), ("bf16", True, False), ("mxfp8", True, False), ("mxfp8", False, True)):
            check_expert_parallel(rank, world, dev, fmt, fused, gather)
    if what in ("all", "cp"):
        from cp_check import check_context_parallel, check_cp_engine
        for fused in (True, False):
            check_context_parallel(rank, world, dev, fused)
        check_cp_engine(rank, world, dev, True, page=128, prompt_lens=(300, 130, 40, 1800))       # the long one: 3 KV ranges per rank
        check_cp_engine(rank, world, dev, True, name="tiny-moe", fmt="mxfp8", page=128, prompt_lens=(257, 700))
    if what in ("all", "tp"):
        for fmt, fused in (("bf16", True), ("mxfp8", True), ("bf16", False), ("q4_k", True), ("q8_0", True)):
            check_tensor_parallel(rank, world, dev, fmt, fused)
    if what in ("all", "hybrid"):
        for fmt, fused in (("bf16", True), ("mxfp8", True), ("mxfp8", False)):
            check_tensor_parallel(rank, world, dev, fmt, fused, name="tiny-moe", ep_experts=True)
    if what in ("all", "tp", "tp4"):
        check_tp_prefill_fused(rank, world, dev)
    if what == "tp4":
        for fmt, fused in (("bf16", True), ("mxfp8", True)):
            check_tensor_parallel(rank, world, dev, fmt, fused)
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_WORKER_OK", what, "world", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
