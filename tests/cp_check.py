"""Context-parallel decode attention against the unsharded attention: used by the CPU (gloo) and the GPU worker."""
import torch
import torch.distributed as dist

from gemm_b200.ops import attention as att
from gemm_b200.ops import elementwise as ew
from gemm_b200.parallel.context import ContextParallel


def check_context_parallel(rank, world, dev, fused):
    torch.manual_seed(17)                                    # every rank builds the same full problem
    hq, hkv, d, page, block = 8, 2, 128, 16, 32
    kv_lens = [70, 33, 129]
    b = len(kv_lens)
    cp = ContextParallel(dist.group.WORLD, torch.device(dev), block=block, fused=fused, max_tokens=8, hq=hq, head_dim=d)
    assert [cp.local_len(100, r) for r in range(world)] == [len(cp.shard_positions(100, r)) for r in range(world)]
    q = (torch.randn(b, hq, d) * 0.5 * ew.softmax_scale_log2(d)).bfloat16()
    cu = torch.arange(b + 1, dtype=torch.int32)
    # full cache, one run of pages per sequence
    pages_full = [(n + page - 1) // page for n in kv_lens]
    kf = torch.zeros(sum(pages_full) * page, hkv, d, dtype=torch.bfloat16)
    vf = torch.zeros_like(kf)
    bt_full = torch.zeros(b, max(pages_full), dtype=torch.int32)
    keys, vals, p0 = [], [], 0
    for s, n in enumerate(kv_lens):
        k, v = (torch.randn(n, hkv, d) * 0.5).bfloat16(), (torch.randn(n, hkv, d) * 0.5).bfloat16()
        keys.append(k); vals.append(v)
        bt_full[s, : pages_full[s]] = torch.arange(p0, p0 + pages_full[s])
        kf[p0 * page: p0 * page + n] = k
        vf[p0 * page: p0 * page + n] = v
        p0 += pages_full[s]
    work = att.build_work([1] * b, hq, hkv)
    to = lambda x: x.to(dev)
    ref = att.attention(to(q), to(kf), to(vf), to(cu), to(torch.tensor(kv_lens, dtype=torch.int32)), to(bt_full), page, to(work), causal=True)
    # this rank's shard: the positions it owns, packed in order into its own pages
    lens_l = [cp.local_len(n) for n in kv_lens]
    pages_l = [max(1, (n + page - 1) // page) for n in lens_l]
    kl = torch.zeros(sum(pages_l) * page, hkv, d, dtype=torch.bfloat16)
    vl = torch.zeros_like(kl)
    bt_l = torch.zeros(b, max(pages_l), dtype=torch.int32)
    p0 = 0
    for s, n in enumerate(kv_lens):
        mine = list(cp.shard_positions(n))
        assert [cp.local_index(p) for p in mine] == list(range(len(mine)))
        bt_l[s, : pages_l[s]] = torch.arange(p0, p0 + pages_l[s])
        kl[p0 * page: p0 * page + len(mine)] = keys[s][mine]
        vl[p0 * page: p0 * page + len(mine)] = vals[s][mine]
        p0 += pages_l[s]
    out = cp.attention(to(q), to(kl), to(vl), to(cu), to(torch.tensor(lens_l, dtype=torch.int32)), to(bt_l), page, to(work))
    r = ((out.float().cpu() - ref.float().cpu()).norm() / ref.float().cpu().norm()).item()
    assert r < 1e-2, f"context-parallel attention (fused={fused}) differs from the unsharded one: rel {r}"
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out.contiguous())
    assert all(torch.equal(gathered[0], g) for g in gathered), "ranks disagree after the context-parallel merge"
    dist.barrier()
    cp.close()


def check_cp_engine(rank, world, dev, fused, name="tiny-dense", fmt="bf16", page=16, prompt_lens=(70, 33, 5, 129), new_tokens=6):
    """Whole-model generation under context parallelism (sequence-parallel prefill, sharded KV cache, merged decode attention)
    against the unsharded engine: prefill logits, decode logits step by step (both engines are fed the reference's tokens)."""
    from gemm_b200.models.config import get_config
    from gemm_b200.models.weights import synthetic_weights
    from gemm_b200.serve.engine import Engine, SamplingParams
    cfg = get_config(name)
    device = torch.device(dev)
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g, dtype=torch.int32) for n in prompt_lens]
    b, max_len = len(prompts), max(prompt_lens) + new_tokens + 2
    w = synthetic_weights(cfg, fmt, device, 5)
    ref = Engine(w, max_batch=b, max_seq_len=max_len, page_size=page)
    cp = ContextParallel(dist.group.WORLD, device, block=page, fused=fused, max_tokens=b, hq=cfg.n_heads, head_dim=cfg.head_dim, max_splits=4)
    eng = Engine(w, max_batch=b, max_seq_len=max_len, page_size=page, par=cp)
    assert eng.kv.k[0].shape[0] < ref.kv.k[0].shape[0] or world == 1, "the context-parallel cache is not smaller than the full one"
    rel = lambda a, c: ((a.float() - c.float()).norm() / (c.float().norm() + 1e-12)).item()
    lr = ref.prefill(prompts, reserve=new_tokens + 1)
    lc = eng.prefill(prompts, reserve=new_tokens + 1)
    per_seq = [round(rel(lc[i], lr[i]), 4) for i in range(b)]
    if rank == 0:
        print(f"cp engine {name} {fmt} world {world}: prefill logits rel per sequence {per_seq}", flush=True)
    tol = 2e-2 if dev == "cpu" else 4e-2              # bf16 kernels with other tile shapes per rank: the tolerance of the EP / TP checks
    assert lc.shape == lr.shape and max(per_seq) < tol, f"context-parallel prefill logits differ: rel per sequence {per_seq}"
    first = lr.argmax(-1).to(torch.int32)
    sp = SamplingParams(temperature=0.0)
    ref.begin_decode(first, sp, new_tokens, use_graph=False)
    eng.begin_decode(first, sp, new_tokens, use_graph=(dev != "cpu"))
    agree = 0
    for _ in range(new_tokens):
        tr = ref.decode_step().clone()
        tc = eng.decode_step().clone()
        agree += int((tr == tc).sum())
        eng.set_next_tokens(tr)                       # keep both engines on the reference's tokens (near ties may flip an arg-max)
    assert agree >= new_tokens * b - 2, f"context-parallel decode: {agree} of {new_tokens * b} tokens agree"
    # the decode steps wrote their K / V rows on the owners only: a last step through the logits path must still agree
    gathered = [torch.empty_like(tc) for _ in range(world)]
    dist.all_gather(gathered, tc.contiguous())
    assert all(torch.equal(gathered[0], x) for x in gathered), "ranks disagree on the decoded tokens"
    dist.barrier()
    cp.close()
