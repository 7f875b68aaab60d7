"""Worker of tests/test_dist_cpu.py: CPU ranks over gloo.  Exercises the host-side logic of the parallel runtime —
group layout, tensor parallelism (baseline reduction path), expert parallelism (baseline exchange), pipeline stages,
data-parallel agreement — against the unsharded engine."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gemm_b200.models.config import get_config  # noqa: E402
from gemm_b200.models.transformer import ForwardBatch, KvCache, Transformer  # noqa: E402
from gemm_b200.models.weights import synthetic_weights  # noqa: E402
from gemm_b200.parallel.data import DataParallel  # noqa: E402
from gemm_b200.parallel.expert import ExpertParallel  # noqa: E402
from gemm_b200.parallel.groups import ParallelLayout, init_parallel, pp_layer_range  # noqa: E402
from gemm_b200.parallel.pipeline import PipelineStage  # noqa: E402
from gemm_b200.parallel.tensor import TensorParallel  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def run(model, cfg, toks, page=16, step_fn=None):
    b = len(toks)
    lens = [t.numel() - 2 for t in toks]
    pages_per = [(t.numel() + page - 1) // page for t in toks]
    bt = torch.zeros(b, max(pages_per), dtype=torch.int32)
    p0 = 0
    for s in range(b):
        bt[s, : pages_per[s]] = torch.arange(p0, p0 + pages_per[s])
        p0 += pages_per[s]
    ctx, outs = [0] * b, []
    for chunk in (lens, [1] * b, [1] * b):
        ids = torch.cat([toks[s][ctx[s]:ctx[s] + chunk[s]] for s in range(b)])
        fb = ForwardBatch.build(chunk, ctx, ids, bt, page, model.hq_local * model.w.tp_size, model.hkv_local * 1, "cpu")
        fb.work = __import__("gemm_b200.ops.attention", fromlist=["x"]).build_work(chunk, model.hq_local, model.hkv_local)
        outs.append(step_fn(fb) if step_fn else model.forward(fb).float())
        ctx = [c + q for c, q in zip(ctx, chunk)]
    return outs


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    what = sys.argv[1]
    g = torch.Generator().manual_seed(3)
    if what == "cp":
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from cp_check import check_context_parallel, check_cp_engine
        check_context_parallel(rank, world, "cpu", False)
        check_cp_engine(rank, world, "cpu", False)
        check_cp_engine(rank, world, "cpu", False, name="tiny-moe", prompt_lens=(40, 7))
        check_cp_engine(rank, world, "cpu", False, prompt_lens=(10, 7), new_tokens=12)     # ranks without a page of any prompt
    if what == "m3ep":
        # MiniMax-M3 style engine: experts dealt to the ranks (e % world), partial sums all-reduced, against the unsharded model
        from gemm_b200.models import m3
        cfg = m3.M3Config(n_layers=3, n_dense_layers=1, hidden=64, vocab=96, n_heads=4, n_kv_heads=2, head_dim=32, rotary_dim=16, msa_index_dim=16,
                          msa_n_index_heads=2, msa_block_size=4, msa_topk_blocks=2, msa_init_block=1, msa_local_block=1, n_experts=8, n_active=2,
                          moe_inter=32, dense_inter=96, max_pos=64)
        t = m3.random_tensors(cfg, 7)
        ids = torch.randint(0, cfg.vocab, (2, 30), generator=g)
        full = m3.M3Model(cfg, t)
        full.reset(2, 48)
        want = torch.cat([full.forward(ids[:, :20], all_logits=True), full.forward(ids[:, 20:], all_logits=True)], dim=1)
        mine = m3.M3Model(cfg, t, ep_rank=rank, ep_size=world, group=dist.group.WORLD)
        assert mine.t["l1.ex_w1"].shape[0] == len(range(rank, cfg.n_experts, world))
        mine.reset(2, 48)
        got = torch.cat([mine.forward(ids[:, :20], all_logits=True), mine.forward(ids[:, 20:], all_logits=True)], dim=1)
        assert rel(got, want) < 1e-4, rel(got, want)
    if what == "groups":
        lay = ParallelLayout(tp=2, pp=2, dp=world // 4)
        grp = init_parallel(lay)
        assert (grp.tp_rank, grp.pp_rank, grp.dp_rank) == (rank % 2, (rank // 2) % 2, rank // 4)
        x = torch.tensor([float(rank)])
        dist.all_reduce(x, group=grp.tp_group)
        assert x.item() == sum(lay.tp_group_ranks(rank))
        y = torch.tensor([float(rank)])
        dist.all_reduce(y, group=grp.pp_group)
        assert y.item() == sum(lay.pp_group_ranks(rank))
        assert [pp_layer_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    elif what == "tp":
        cfg = get_config("tiny-dense")
        toks = [torch.randint(0, cfg.vocab, (n,), generator=g) for n in (20, 33)]
        ref = run(Transformer(synthetic_weights(cfg, "bf16", "cpu", 5), KvCache.allocate(cfg, 16, 16, "cpu")), cfg, toks)
        par = TensorParallel(dist.group.WORLD, torch.device("cpu"), fused=False)
        par.attach(None, cfg, 64)
        w = synthetic_weights(cfg, "bf16", "cpu", 5, tp_rank=rank, tp_size=world)
        model = Transformer(w, KvCache.allocate(cfg, 16, 16, "cpu", max(1, cfg.n_kv_heads // world)), par)
        got = run(model, cfg, toks)
        for a, b in zip(got, ref):
            assert rel(a, b) < 2e-2, rel(a, b)
    elif what == "ep":
        cfg = get_config("tiny-moe")
        toks = [torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(7 + rank)) for n in (20, 33)]
        ref = run(Transformer(synthetic_weights(cfg, "bf16", "cpu", 5), KvCache.allocate(cfg, 16, 16, "cpu")), cfg, toks)
        par = ExpertParallel(dist.group.WORLD, torch.device("cpu"), fused=False)
        par.attach(None, cfg, 64)
        w = synthetic_weights(cfg, "bf16", "cpu", 5, ep_rank=rank, ep_size=world)
        got = run(Transformer(w, KvCache.allocate(cfg, 16, 16, "cpu"), par), cfg, toks)
        for a, b in zip(got, ref):
            assert rel(a, b) < 2e-2, rel(a, b)
    elif what == "hybrid":
        # tensor-parallel attention in front of expert-parallel experts on the same ranks: every rank sees every token
        cfg = get_config("tiny-moe")
        toks = [torch.randint(0, cfg.vocab, (n,), generator=g) for n in (20, 33)]
        ref = run(Transformer(synthetic_weights(cfg, "bf16", "cpu", 5), KvCache.allocate(cfg, 16, 16, "cpu")), cfg, toks)
        par = TensorParallel(dist.group.WORLD, torch.device("cpu"), fused=False, ep_experts=True)
        par.attach(None, cfg, 64)
        w = synthetic_weights(cfg, "bf16", "cpu", 5, tp_rank=rank, tp_size=world, ep_rank=rank, ep_size=world)
        assert w.layers[0].w13.groups == cfg.n_experts // world
        model = Transformer(w, KvCache.allocate(cfg, 16, 16, "cpu", max(1, cfg.n_kv_heads // world)), par)
        got = run(model, cfg, toks)
        for a, b in zip(got, ref):
            assert rel(a, b) < 2e-2, rel(a, b)
    elif what == "pp":
        cfg = get_config("tiny-dense").with_(n_layers=5)
        toks = [torch.randint(0, cfg.vocab, (n,), generator=g) for n in (20, 33)]
        full = Transformer(synthetic_weights(cfg, "bf16", "cpu", 5), KvCache.allocate(cfg, 16, 16, "cpu"))
        ref = [o.argmax(-1).to(torch.int32) for o in run(full, cfg, toks)]
        lo, hi = pp_layer_range(cfg.n_layers, world, rank)
        w = synthetic_weights(cfg, "bf16", "cpu", 5, layer_range=(lo, hi))
        stage = PipelineStage(Transformer(w, KvCache.allocate(cfg, 16, 16, "cpu", n_layers=hi - lo)), dist.group.WORLD, cfg.n_layers)
        assert stage.layer_range == (lo, hi)
        got = run(stage.model, cfg, toks, step_fn=stage.step)
        for a, b in zip(got, ref):
            assert torch.equal(a, b), (a, b)
        # micro-batches (one per sequence group) through the overlapped schedule give the tokens of the whole-batch step
        from gemm_b200.ops import attention as att
        seqs = [torch.randint(0, cfg.vocab, (n,), generator=g) for n in (9, 14, 6, 11)]
        page, bt_all, p0 = 16, torch.zeros(4, 1, dtype=torch.int32), 0
        bt_all[:, 0] = torch.arange(4)

        def fb_of(idx):
            fb = ForwardBatch.build([seqs[i].numel() for i in idx], [0] * len(idx), torch.cat([seqs[i] for i in idx]), bt_all[idx], page,
                                    cfg.n_heads, cfg.n_kv_heads, "cpu")
            fb.work = att.build_work([seqs[i].numel() for i in idx], stage.model.hq_local, stage.model.hkv_local)
            return fb
        whole = stage.step(fb_of([0, 1, 2, 3]))
        parts = stage.step_many([fb_of([0, 1]), fb_of([2]), fb_of([3])])
        assert [p.numel() for p in parts] == [2, 1, 1] and torch.equal(torch.cat(parts), whole), (parts, whole)
    elif what == "cpmerge":
        # ring and tree merges of attention partials against the all-gather + combine rule
        from gemm_b200.ops import attention as att
        from gemm_b200.parallel import context as cpx
        gq = torch.Generator().manual_seed(100 + rank)
        o, lse = torch.randn(5, 8, 16, generator=gq), torch.randn(5, 8, generator=gq) * 4
        if rank == 1:
            lse[0] = float("-inf")                                # a rank without keys for that query
        parts_o, parts_l = [torch.empty_like(o) for _ in range(world)], [torch.empty_like(lse) for _ in range(world)]
        dist.all_gather(parts_o, o)
        dist.all_gather(parts_l, lse)
        want, want_l = att.combine_partials(torch.stack(parts_o).reshape(world, 40, 16), torch.stack(parts_l).reshape(world, 40))
        for fn in (cpx.merge_ring, cpx.merge_tree):
            got_o, got_l = fn(o, lse)
            assert rel(got_o.reshape(40, 16), want) < 5e-3, (fn.__name__, rel(got_o.reshape(40, 16), want))
            assert (got_l.reshape(40) - want_l).abs().max() < 1e-4
        got_o, _ = cpx.merge_tree(o, lse)
        same = [torch.empty_like(got_o) for _ in range(world)]
        dist.all_gather(same, got_o)
        assert all(torch.equal(same[0], x) for x in same), "tree merge: ranks disagree"
    elif what == "dp":
        dp = DataParallel(dist.group.WORLD)
        items = list(range(10))
        mine = dp.shard(items)
        assert mine == [i for i in items if i % world == rank]
        out = dp.gather_outputs([[i * 10] for i in mine], len(items))
        assert out == [[i * 10] for i in items]
        assert dp.check_agreement(torch.tensor([1, 2, 3]))
        assert not dp.check_agreement(torch.tensor([1, 2, 3 + rank]))
    dist.barrier()
    if rank == 0:
        print("CPU_DIST_WORKER_OK", what)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
