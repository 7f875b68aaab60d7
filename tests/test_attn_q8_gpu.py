"""INT8 KV cache on the GPU: the store kernel against the reference quantiser (bit for bit), and decode attention reading the int8
pages against fp32 attention over the same pages dequantised (csrc/kernels/attn_q8.cu)."""
import math

import pytest
import torch

from gemm_b200 import _native
from gemm_b200.ops import attention as att
from gemm_b200.ops import elementwise as ew
from gemm_b200.ops.kvquant import quantize_q8_ref

pytestmark = pytest.mark.gpu


def _paged(b, lens, hkv, page, seed):
    g = torch.Generator().manual_seed(seed)
    pages_per = [(n + page - 1) // page for n in lens]
    n_pages = sum(pages_per) + 3
    perm = torch.randperm(n_pages, generator=g)
    bt = torch.zeros(b, max(pages_per), dtype=torch.int32)
    at = 0
    for s in range(b):
        bt[s, : pages_per[s]] = perm[at: at + pages_per[s]].to(torch.int32)
        at += pages_per[s]
    return bt, n_pages


def test_store_matches_reference_quantiser():
    torch.manual_seed(0)
    hkv, slots, t = 4, 512, 37
    k = (torch.randn(t, hkv, 128) * 3).bfloat16().cuda()
    v = torch.randn(t, hkv, 128).bfloat16().cuda()
    v[3] = 0                                                     # an all-zero row has scale 0 and stays zero
    dst = torch.randperm(slots)[:t].to(torch.int32).cuda()
    dst[5] = -1                                                  # not stored
    kq = torch.full((slots, hkv, 128), 7, dtype=torch.int8, device="cuda")
    vq = torch.full_like(kq, 7)
    ks = torch.full((slots, hkv), -1.0, device="cuda")
    vs = torch.full_like(ks, -1.0)
    att.kv_store_q8(k, v, None, dst, kq, vq, ks, vs)
    torch.cuda.synchronize()
    ok = dst >= 0
    for cache, sc, rows in ((kq, ks, k), (vq, vs, v)):
        q_ref, s_ref = quantize_q8_ref(rows[ok].cpu())
        got = cache[dst[ok].long()].cpu()
        # the reference forms 127 / amax as a reciprocal times 127 (two roundings), the kernel divides: a value that lands on a
        # rounding boundary may differ by one step
        diff = (got.int() - q_ref.int()).abs()
        assert int(diff.max()) <= 1 and float((diff == 0).float().mean()) > 0.999
        assert torch.allclose(sc[dst[ok].long()].cpu(), s_ref, rtol=1e-6, atol=0)
    untouched = torch.ones(slots, dtype=torch.bool, device="cuda")
    untouched[dst[ok].long()] = False
    assert bool((kq[untouched] == 7).all()) and bool((ks[untouched] == -1).all())


@pytest.mark.parametrize("hq,hkv,lens,splits,window,page", [
    (32, 4, [2056, 1, 31, 33, 640], 1, 0, 128),       # the benchmark's head layout: 8 query heads per KV head
    (32, 4, [2056, 700, 129], 3, 0, 128),             # KV range split three ways, merged by the combine kernel
    (16, 1, [300, 64], 2, 0, 16),                     # 16 query heads on one KV head, small pages
    (8, 8, [97, 5], 1, 0, 32),                        # no grouping
    (8, 2, [500, 120], 1, 64, 128),                   # sliding window
    (14, 2, [260], 1, 0, 64),                         # 7 heads per KV head
])
def test_decode_attention_over_int8_pages(hq, hkv, lens, splits, window, page):
    b, d = len(lens), 128
    torch.manual_seed(hq + len(lens))
    bt, n_pages = _paged(b, lens, hkv, page, seed=hq)
    slots = n_pages * page
    k = (torch.randn(slots, hkv, d) * 1.5).bfloat16().cuda()
    v = torch.randn(slots, hkv, d).bfloat16().cuda()
    kq = torch.zeros(slots, hkv, d, dtype=torch.int8, device="cuda")
    vq = torch.zeros_like(kq)
    ks = torch.zeros(slots, hkv, device="cuda")
    vs = torch.zeros_like(ks)
    att.kv_store_q8(k, v, None, torch.arange(slots, dtype=torch.int32, device="cuda"), kq, vq, ks, vs)
    q = (torch.randn(b, hq, d) * ew.softmax_scale_log2(d)).bfloat16().cuda()
    kv_len = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = att.attention_decode_q8(q, kq, vq, ks, vs, kv_len, bt.cuda(), page, num_splits=splits, window=window)
    torch.cuda.synchronize()
    _native.assert_status_ok()
    # reference: fp32 attention over the DEQUANTISED pages (the cache's own rounding is not the kernel's error)
    kd = (kq.float() * ks.unsqueeze(-1)).cpu()
    vd = (vq.float() * vs.unsqueeze(-1)).cpu()
    cu = torch.arange(b + 1, dtype=torch.int32)
    ref = att.attention_ref(q.cpu(), kd, vd, cu, kv_len.cpu(), bt, page, True, window).float()
    rel = ((out.float().cpu() - ref).norm() / ref.norm()).item()
    assert rel < 2.5e-2, rel            # the query is rounded to int8 per head and the block sums to half precision
    # and against the unquantised K / V the whole INT8 path stays within a few percent
    ref_full = att.attention_ref(q.cpu(), k.cpu(), v.cpu(), cu, kv_len.cpu(), bt, page, True, window).float()
    assert ((out.float().cpu() - ref_full).norm() / ref_full.norm()).item() < 4e-2
