"""tcgen05 flash attention (prefill, decode, split-KV) vs the fp32 PyTorch reference over the same paged cache."""
import pytest
import torch

from gemm_b200 import _native
from gemm_b200.ops import attention as att
from gemm_b200.ops import elementwise as ew

pytestmark = pytest.mark.gpu


def _setup(q_lens, ctx_lens, hq, hkv, page_size, seed=0):
    torch.manual_seed(seed)
    d = 128
    b = len(q_lens)
    kv_lens = [q + c for q, c in zip(q_lens, ctx_lens)]
    pages_per = [(kl + page_size - 1) // page_size for kl in kv_lens]
    total_pages = sum(pages_per) + 3
    perm = torch.randperm(total_pages)
    bt = torch.zeros(b, max(pages_per), dtype=torch.int32)
    pos = 0
    for s in range(b):
        bt[s, : pages_per[s]] = perm[pos:pos + pages_per[s]]
        pos += pages_per[s]
    k_cache = torch.zeros(total_pages * page_size, hkv, d, dtype=torch.bfloat16, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    for s in range(b):
        kl = kv_lens[s]
        slots = (bt[s, : pages_per[s]].long().unsqueeze(1) * page_size + torch.arange(page_size)).reshape(-1)[:kl].cuda()
        k_cache[slots] = torch.randn(kl, hkv, d, device="cuda").bfloat16()
        v_cache[slots] = torch.randn(kl, hkv, d, device="cuda").bfloat16()
    t = sum(q_lens)
    q = (torch.randn(t, hq, d, device="cuda") * ew.softmax_scale_log2(d)).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    return q, k_cache, v_cache, cu, kvl, bt.cuda()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("q_lens,ctx,hq,hkv,page", [
    ([128], [0], 8, 8, 128),
    ([200, 77], [0, 0], 32, 4, 128),
    ([300], [500], 16, 2, 64),
    ([50, 1, 129], [0, 257, 100], 8, 1, 16),
    ([64], [0], 14, 2, 32),            # group of 7: tile holds 18 tokens x 7 heads
])
def test_prefill(q_lens, ctx, hq, hkv, page):
    q, kc, vc, cu, kvl, bt = _setup(q_lens, ctx, hq, hkv, page)
    work = att.build_work(q_lens, hq, hkv).cuda()
    out = att.attention(q, kc, vc, cu, kvl, bt, page, work)
    ref = att.attention_ref(q, kc, vc, cu, kvl, bt, page)
    _native.assert_status_ok()
    assert _rel(out, ref) < 1.5e-2


@pytest.mark.parametrize("splits", [1, 3, 8])
def test_decode_split(splits):
    b = 6
    q_lens, ctx = [1] * b, [5, 127, 128, 1000, 2047, 300]
    q, kc, vc, cu, kvl, bt = _setup(q_lens, ctx, 32, 4, 128, seed=1)
    work = att.build_work(q_lens, 32, 4, splits).cuda()
    out = att.attention(q, kc, vc, cu, kvl, bt, 128, work, num_splits=splits)
    ref = att.attention_ref(q, kc, vc, cu, kvl, bt, 128)
    _native.assert_status_ok()
    assert _rel(out, ref) < 1.5e-2


def test_sliding_window_and_noncausal():
    q_lens, ctx = [150], [400]
    q, kc, vc, cu, kvl, bt = _setup(q_lens, ctx, 8, 2, 128, seed=2)
    work = att.build_work(q_lens, 8, 2).cuda()
    out = att.attention(q, kc, vc, cu, kvl, bt, 128, work, window=200)
    ref = att.attention_ref(q, kc, vc, cu, kvl, bt, 128, window=200)
    assert _rel(out, ref) < 1.5e-2
    out = att.attention(q, kc, vc, cu, kvl, bt, 128, work, causal=False)
    ref = att.attention_ref(q, kc, vc, cu, kvl, bt, 128, causal=False)
    _native.assert_status_ok()
    assert _rel(out, ref) < 1.5e-2


@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("hq,hkv,page", [(32, 4, 128), (8, 2, 16), (16, 1, 64), (4, 4, 128)])
def test_decode_kernel(hq, hkv, page, splits):
    """The decode-specialised kernel (KV positions on the MMA M axis) against the fp32 reference and the general kernel."""
    b = 7
    q_lens, ctx = [1] * b, [0, 5, 127, 128, 1000, 2047, 300]
    q, kc, vc, cu, kvl, bt = _setup(q_lens, ctx, hq, hkv, page, seed=3)
    work = att.build_work(q_lens, hq, hkv, splits).cuda()
    out = att.attention(q, kc, vc, cu, kvl, bt, page, work, num_splits=splits, decode=True)
    ref = att.attention_ref(q, kc, vc, cu, kvl, bt, page)
    _native.assert_status_ok()
    assert _rel(out, ref) < 1.5e-2
    gen = att.attention(q, kc, vc, cu, kvl, bt, page, work, num_splits=splits)
    assert _rel(out, gen) < 1.5e-2


def test_decode_kernel_sliding_window():
    b = 3
    q_lens, ctx = [1] * b, [700, 90, 300]
    q, kc, vc, cu, kvl, bt = _setup(q_lens, ctx, 8, 2, 128, seed=4)
    work = att.build_work(q_lens, 8, 2).cuda()
    out = att.attention(q, kc, vc, cu, kvl, bt, 128, work, window=200, decode=True)
    ref = att.attention_ref(q, kc, vc, cu, kvl, bt, 128, window=200)
    _native.assert_status_ok()
    assert _rel(out, ref) < 1.5e-2


@pytest.mark.parametrize("b,lay,splits", [(7, 32, 1), (40, 128, 1), (5, 32, 3)])
def test_decode_kernel_mxfp8_output(b, lay, splits):
    """The decode kernel's MXFP8 output (the o_proj operand) equals quantising its bf16 output."""
    from gemm_b200.ops import elementwise as ew
    from gemm_b200.ops import mxfp8
    hq, hkv, page = 32, 4, 128
    q_lens = [1] * b
    ctx = [(37 * i) % 900 for i in range(b)]
    q, kc, vc, cu, kvl, bt = _setup(q_lens, ctx, hq, hkv, page, seed=6)
    work = att.build_work(q_lens, hq, hkv, splits).cuda()
    out = att.attention(q, kc, vc, cu, kvl, bt, page, work, decode=True, num_splits=splits)
    assert att.can_decode_mx(q, hkv, splits, True)
    om = att.attention_decode_mx(q, kc, vc, cu, kvl, bt, page, work, sf_layout=lay, num_splits=splits)
    _native.assert_status_ok()
    want = ew.mx_quantize(out.reshape(b, hq * 128), sf_layout=lay)
    got_f, want_f = mxfp8.dequantize(om), mxfp8.dequantize(want)
    assert _rel(got_f, out.reshape(b, hq * 128)) < 4e-2                 # e4m3 rounding
    # the kernel quantises the fp32 value, the reference path a bf16-rounded one: scales agree, bytes differ by at most one step rarely
    sg = mxfp8.unpack_sf_atoms(om.sf, b, hq * 4, lay).int()
    sw = mxfp8.unpack_sf_atoms(want.sf, b, hq * 4, lay).int()
    assert (sg - sw).abs().max().item() <= 1
    assert _rel(got_f, want_f) < 2e-2


def test_prefill_kernel_mxfp8_output():
    """The general kernel's MXFP8 output equals quantising its bf16 output (mixed batch: prefill chunks and a decode row)."""
    from gemm_b200.ops import elementwise as ew
    from gemm_b200.ops import mxfp8
    hq, hkv, page = 32, 4, 16
    q_lens, ctx = [150, 1, 40], [0, 77, 200]
    q, kc, vc, cu, kvl, bt = _setup(q_lens, ctx, hq, hkv, page, seed=8)
    work = att.build_work(q_lens, hq, hkv, 1).cuda()
    out = att.attention(q, kc, vc, cu, kvl, bt, page, work)
    t = sum(q_lens)
    om = att.attention_mx(q, kc, vc, cu, kvl, bt, page, work, sf_layout=128)
    _native.assert_status_ok()
    want = ew.mx_quantize(out.reshape(t, hq * 128), sf_layout=128)
    sg = mxfp8.unpack_sf_atoms(om.sf, t, hq * 4, 128).int()
    sw = mxfp8.unpack_sf_atoms(want.sf, t, hq * 4, 128).int()
    assert (sg - sw).abs().max().item() <= 1
    assert _rel(mxfp8.dequantize(om), mxfp8.dequantize(want)) < 2e-2
    assert _rel(mxfp8.dequantize(om), out.reshape(t, hq * 128)) < 4e-2

