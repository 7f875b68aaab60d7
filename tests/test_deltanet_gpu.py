"""Delta-Net kernels (conv + SiLU, recurrence + gated norm, sigmoid gate) and M-RoPE against their PyTorch references."""
import pytest
import torch

from gemm_b200 import _native
from gemm_b200.ops import deltanet as dn
from gemm_b200.ops import elementwise as ew

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float().cpu() - b.float().cpu()).norm() / (b.float().cpu().norm() + 1e-12)).item()


def test_conv_silu_with_history():
    torch.manual_seed(1)
    ch, ck, wide = 512, 4, 768
    lens = [5, 1, 37]
    cu = torch.tensor([0, 5, 6, 43], dtype=torch.int32)
    slots = torch.tensor([2, 0, 3], dtype=torch.int32)
    x = torch.randn(43, wide).bfloat16()
    w = torch.randn(ch, ck)
    st = torch.randn(4, ck - 1, ch)
    st_ref, st_gpu = st.clone(), st.clone().cuda()
    ref = dn.conv_silu(x[:, :ch], w, st_ref, cu, slots)
    got = dn.conv_silu(x.cuda()[:, :ch], w.cuda(), st_gpu, cu.cuda(), slots.cuda())
    assert _rel(got, ref) < 1e-2
    assert _rel(st_gpu, st_ref) < 1e-6
    assert torch.equal(st_gpu[1].cpu(), st[1])            # a slot no sequence uses is untouched


@pytest.mark.parametrize("ds,ng,hv", [(64, 2, 4), (128, 2, 6)])
def test_deltanet_recurrence(ds, ng, hv):
    torch.manual_seed(2)
    lens = [9, 1, 20]
    cu = torch.tensor([0, 9, 10, 30], dtype=torch.int32)
    slots = torch.tensor([1, 2, 0], dtype=torch.int32)
    t = 30
    qkv = (torch.randn(t, (2 * ng + hv) * ds) * 0.5).bfloat16()
    z = torch.randn(t, hv * ds + 64).bfloat16()[:, : hv * ds]          # a column slice of a wider tensor
    ab = torch.randn(t, 2 * hv)
    a = -(torch.rand(hv) * 2 + 0.1)
    bias = torch.randn(hv) * 0.5
    nw = torch.rand(ds) + 0.5
    st = torch.randn(3, hv, ds, ds) * 0.1
    st_ref, st_gpu = st.clone(), st.clone().cuda()
    ref = dn.deltanet(qkv, z, ab, a, bias, nw, st_ref, cu, slots, ng, hv, ds, 1e-6)
    got = dn.deltanet(qkv.cuda(), z.cuda(), ab.cuda(), a.cuda(), bias.cuda(), nw.cuda(), st_gpu, cu.cuda(), slots.cuda(), ng, hv, ds, 1e-6)
    _native.assert_status_ok()
    assert _rel(got, ref) < 1e-2
    assert _rel(st_gpu, st_ref) < 1e-4


@pytest.mark.parametrize("lens", [[150, 64, 70, 200], [1000], [63, 65, 128, 129, 48]])
def test_deltanet_chunked_scan(lens):
    """Prefill-sized launches take the chunked scan (64 tokens per serial step, bf16 tiles, fp32 state): against the per-token
    fp32 reference and against the per-token kernel, including partial last chunks and states that are not zero."""
    torch.manual_seed(4)
    ds, ng, hv = 128, 2, 4
    n = len(lens)
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    slots = torch.randperm(n + 1)[:n].to(torch.int32)
    t = sum(lens)
    qkv = torch.randn(t, (2 * ng + hv) * ds).bfloat16()
    z = torch.randn(t, hv * ds + 64).bfloat16()[:, : hv * ds]
    ab = torch.randn(t, 2 * hv)
    a = -(torch.rand(hv) * 2 + 0.1)
    bias = torch.randn(hv) * 0.5
    nw = torch.rand(ds) + 0.5
    st = torch.randn(n + 1, hv, ds, ds) * 0.1
    st_ref, st_gpu, st_tok = st.clone(), st.clone().cuda(), st.clone().cuda()
    assert dn.CHUNKED and t >= dn.CHUNKED_MIN_TOKENS * n
    ref = dn.deltanet(qkv, z, ab, a, bias, nw, st_ref, cu, slots, ng, hv, ds, 1e-6)
    args = (qkv.cuda(), z.cuda(), ab.cuda(), a.cuda(), bias.cuda(), nw.cuda())
    got = dn.deltanet(*args, st_gpu, cu.cuda(), slots.cuda(), ng, hv, ds, 1e-6)
    _native.assert_status_ok()
    dn.CHUNKED = False
    try:
        tok = dn.deltanet(*args, st_tok, cu.cuda(), slots.cuda(), ng, hv, ds, 1e-6)
    finally:
        dn.CHUNKED = True
    assert _rel(tok, ref) < 1e-2
    assert _rel(got, ref) < 2e-2, _rel(got, ref)
    assert _rel(st_gpu, st_ref) < 1e-2, _rel(st_gpu, st_ref)
    unused = [i for i in range(n + 1) if i not in slots.tolist()][0]
    assert torch.equal(st_gpu[unused].cpu(), st[unused])
    # per sequence, so that a wrong chunk of a short sequence cannot hide behind a long one
    for i in range(n):
        assert _rel(got[cu[i]:cu[i + 1]], ref[cu[i]:cu[i + 1]]) < 2e-2, (i, lens[i])


def test_sigmoid_gate_mul():
    torch.manual_seed(3)
    x = torch.randn(19, 512).bfloat16()
    wide = torch.randn(19, 1536).bfloat16()
    ref = (x.float() * torch.sigmoid(wide[:, 1024:].float()))
    got = dn.gate_mul(x.clone().cuda(), wide.cuda()[:, 1024:])
    assert _rel(got, ref) < 1e-2


@pytest.mark.parametrize("d,rope_dim,sections", [(128, 64, [11, 11, 10, 0]), (128, 128, [24, 20, 20, 0]), (64, 64, [16, 8, 8, 0])])
def test_mrope_and_rope_table(d, rope_dim, sections):
    torch.manual_seed(4)
    t, hq, hkv = 21, 4, 2
    qkv = torch.randn(t, (hq + 2 * hkv) * d).bfloat16().cuda()
    pos = torch.randint(0, 3000, (t,), dtype=torch.int32).cuda()
    pos3 = torch.stack([pos, torch.randint(0, 50, (t,), dtype=torch.int32).cuda(), torch.randint(0, 50, (t,), dtype=torch.int32).cuda()]).contiguous()
    slots = torch.arange(t, dtype=torch.int32).cuda()
    qw, kw = (torch.rand(d) + 0.5).bfloat16().cuda(), (torch.rand(d) + 0.5).bfloat16().cuda()
    table = ew.rope_table(4096, rope_dim, 1e6, "cuda")
    for p3, sec in ((None, None), (pos3, sections)):
        kc = torch.zeros(t, hkv, d, dtype=torch.bfloat16, device="cuda")
        vc = torch.zeros_like(kc)
        q = ew.qk_norm_rope(qkv, pos, slots, qw, kw, kc, vc, hq, hkv, d, 1e6, 1e-6, 0.125, rope_dim, table=table, positions3=p3, sections=sec)
        rq, rk, rv = ew.qk_norm_rope_ref(qkv.cpu(), pos.cpu(), qw.cpu(), kw.cpu(), hq, hkv, d, 1e6, 1e-6, 0.125, rope_dim,
                                         p3.cpu() if p3 is not None else None, sec)
        assert _rel(q, rq) < 1e-2 and _rel(kc, rk) < 1e-2 and torch.equal(vc.cpu(), rv)
        # without the table the kernel computes the angles itself: same result
        kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
        q2 = ew.qk_norm_rope(qkv, pos, slots, qw, kw, kc2, vc2, hq, hkv, d, 1e6, 1e-6, 0.125, rope_dim, positions3=p3, sections=sec)
        assert _rel(q2, rq) < 1e-2 and _rel(kc2, rk) < 1e-2
