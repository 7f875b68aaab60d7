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
