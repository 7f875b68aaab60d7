"""Token-wise, MoE-routing and sampling kernels vs their PyTorch fp32 references."""
import pytest
import torch

from gemm_b200 import _native
from gemm_b200.ops import elementwise as ew
from gemm_b200.ops import moe, mxfp8, sampling

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_embed():
    table = torch.randn(1000, 256, device="cuda").bfloat16()
    ids = torch.randint(0, 1000, (37,), device="cuda", dtype=torch.int32)
    assert torch.equal(ew.embed(ids, table), table[ids.long()])


@pytest.mark.parametrize("rows,hidden", [(5, 1024), (33, 2048), (7, 4096), (3, 5120), (2, 8192)])
def test_rmsnorm(rows, hidden):
    torch.manual_seed(0)
    x = torch.randn(rows, hidden, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(hidden, device="cuda")).bfloat16()
    y = ew.rmsnorm(x, w, 1e-6)
    assert _rel(y, ew.rmsnorm_ref(x, w, 1e-6)) < 4e-3


def test_rmsnorm_residual_quant():
    torch.manual_seed(1)
    rows, hidden = 70, 2048
    res = torch.randn(rows, hidden, device="cuda").bfloat16()
    delta = torch.randn(rows, hidden, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(hidden, device="cuda")).bfloat16()
    res_ref = (res.float() + delta.float()).bfloat16()
    y_ref = ew.rmsnorm_ref(res_ref, w, 1e-6)
    y, q = ew.rmsnorm(delta, w, 1e-6, residual=res, quantize=True)
    assert torch.equal(res, res_ref)
    assert _rel(y, y_ref) < 4e-3
    # the quantised copy must be exactly what the reference quantiser makes of the kernel's bf16 output
    q_ref = mxfp8.quantize(y.float())
    assert torch.equal(q.data[:rows], q_ref.data[:rows])
    assert torch.equal(mxfp8.unpack_sf_atoms(q.sf, rows, hidden // 32), mxfp8.unpack_sf_atoms(q_ref.sf, rows, hidden // 32))


@pytest.mark.parametrize("d,rope_dim", [(128, None), (64, None), (256, 64)])
def test_qk_norm_rope(d, rope_dim):
    torch.manual_seed(2)
    t, hq, hkv = 19, 8, 2
    qkv = torch.randn(t, (hq + 2 * hkv) * d, device="cuda").bfloat16()
    pos = torch.randint(0, 5000, (t,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(64, device="cuda")[:t].to(torch.int32)
    qw = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    kw = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    kc = torch.zeros(64, hkv, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros(64, hkv, d, device="cuda", dtype=torch.bfloat16)
    q = ew.qk_norm_rope(qkv, pos, slots, qw, kw, kc, vc, hq, hkv, d, 1e6, 1e-6, 0.25, rope_dim)
    qr, kr, vr = ew.qk_norm_rope_ref(qkv, pos, qw, kw, hq, hkv, d, 1e6, 1e-6, 0.25, rope_dim)
    assert _rel(q, qr) < 6e-3
    assert _rel(kc[slots.long()], kr) < 6e-3
    assert torch.equal(vc[slots.long()], vr)


@pytest.mark.parametrize("mrope", [False, True])
def test_qk_norm_rope_head128_table_and_mrope(mrope):
    """The vectorised head_dim-128 kernel with the (cos, sin) table, and with per-section positions."""
    torch.manual_seed(22)
    t, hq, hkv, d = 37, 4, 2, 128
    qkv = torch.randn(t, (hq + 2 * hkv) * d, device="cuda").bfloat16()
    pos = torch.randint(0, 3000, (t,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(64, device="cuda")[:t].to(torch.int32)
    slots[3] = -1
    qw = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    kw = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    kc = torch.zeros(64, hkv, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros(64, hkv, d, device="cuda", dtype=torch.bfloat16)
    tab = ew.rope_table(3000, d, 1e6, "cuda")
    p3 = torch.stack([pos, pos + 5, pos + 9]).contiguous().clamp_max(2999) if mrope else None
    sec = [24, 20, 20] if mrope else None
    q = ew.qk_norm_rope(qkv, pos, slots, qw, kw, kc, vc, hq, hkv, d, 1e6, 1e-6, 0.25, None, table=tab, positions3=p3, sections=sec)
    qr, kr, vr = ew.qk_norm_rope_ref(qkv, pos, qw, kw, hq, hkv, d, 1e6, 1e-6, 0.25, None, p3, sec)
    live = slots >= 0
    assert _rel(q, qr) < 6e-3
    assert _rel(kc[slots[live].long()], kr[live]) < 6e-3
    assert torch.equal(vc[slots[live].long()], vr[live])


def test_qk_norm_rope_from_split_k_partials():
    from gemm_b200.ops import gemm
    torch.manual_seed(24)
    t, hq, hkv, d = 21, 4, 2, 128
    width = (hq + 2 * hkv) * d
    parts = torch.randn(3, t, width, device="cuda") * 0.6
    pend = gemm.PendingPartials(parts)
    qkv = parts.sum(0).bfloat16()
    pos = torch.randint(0, 3000, (t,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(64, device="cuda")[:t].to(torch.int32)
    qw = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    kw = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    kc, vc = (torch.zeros(64, hkv, d, device="cuda", dtype=torch.bfloat16) for _ in range(2))
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    tab = ew.rope_table(3000, d, 1e6, "cuda")
    q = ew.qk_norm_rope(pend, pos, slots, qw, kw, kc, vc, hq, hkv, d, 1e6, 1e-6, 0.25, None, table=tab)
    q2 = ew.qk_norm_rope(qkv, pos, slots, qw, kw, kc2, vc2, hq, hkv, d, 1e6, 1e-6, 0.25, None, table=tab)
    assert _rel(q, q2) < 6e-3 and _rel(kc, kc2) < 6e-3 and _rel(vc, vc2) < 6e-3


@pytest.mark.parametrize("lay_in,lay_out", [(128, 128), (128, 32), (32, 32)])
def test_mx_gather_rows_equals_quantising_gathered_rows(lay_in, lay_out):
    torch.manual_seed(23)
    t, k = 50, 512
    x = (torch.randn(t, k, device="cuda") * torch.rand(t, 1, device="cuda") * 8).bfloat16()
    src = torch.randint(-1, t, (300,), device="cuda", dtype=torch.int32)
    xq = ew.mx_quantize(x, sf_layout=lay_in)
    got = ew.mx_gather_rows(xq, src, sf_layout=lay_out)
    want = ew.mx_quantize(x, src, sf_layout=lay_out)
    ok = (src >= 0).cpu()
    assert torch.equal(got.data[:300].cpu()[ok], want.data[:300].cpu()[ok])
    sg = mxfp8.unpack_sf_atoms(got.sf, 300, k // 32, lay_out).cpu()[ok]
    sw = mxfp8.unpack_sf_atoms(want.sf, 300, k // 32, lay_out).cpu()[ok]
    assert torch.equal(sg, sw)


def test_silu_mul_and_quant_gather():
    torch.manual_seed(3)
    gu = torch.randn(50, 512, device="cuda").bfloat16()
    ref = torch.nn.functional.silu(gu.float()[:, :256]) * gu.float()[:, 256:]
    assert _rel(ew.silu_mul(gu), ref) < 4e-3
    x = torch.randn(40, 256, device="cuda").bfloat16()
    src = torch.tensor([3, -1, 7, 7, 0, 39, -1, 12], device="cuda", dtype=torch.int32)
    q = ew.mx_quantize(x, src)
    g = torch.zeros(8, 256, device="cuda")
    ok = src >= 0
    g[ok] = x.float()[src[ok].long()]
    q_ref = mxfp8.quantize(g)
    # rows without a source are padding of the expert-sorted buffer: they are left unwritten (nothing valid reads them)
    assert torch.equal(q.data[:8][ok], q_ref.data[:8][ok])
    assert torch.equal(mxfp8.unpack_sf_atoms(q.sf, 8, 8)[ok], mxfp8.unpack_sf_atoms(q_ref.sf, 8, 8)[ok])


@pytest.mark.parametrize("mode", ["softmax", "sigmoid"])
def test_moe_route(mode):
    torch.manual_seed(4)
    t, e, k = 300, 128, 8
    logits = torch.randn(t, e, device="cuda")
    logits[5, 7] = float("nan")
    logits[6, :] = 0.0                      # all ties -> ids 0..7
    bias = torch.randn(e, device="cuda") * 0.1 if mode == "sigmoid" else None
    ids, w = moe.route(logits, k, mode, bias, True, 2.5 if mode == "sigmoid" else 1.0)
    ids_r, w_r = moe.route_ref(logits.cpu(), k, mode, bias.cpu() if bias is not None else None, True, 2.5 if mode == "sigmoid" else 1.0)
    assert torch.equal(ids.cpu(), ids_r)
    assert torch.allclose(w.cpu(), w_r, rtol=1e-4, atol=1e-6)
    if mode == "softmax":
        assert ids[6].tolist() == list(range(8))


@pytest.mark.parametrize("t,regions", [(1, 1), (64, 1), (1000, 1), (300, 8), (200, 8), (256, 1)])
def test_moe_plan_and_combine(t, regions):
    torch.manual_seed(5)
    e, k, align, hidden = 128, 8, 128, 256
    logits = torch.randn(t, e, device="cuda")
    ids, w = moe.route(logits, k)
    pl = moe.plan(ids, e, align, regions)
    ref = moe.plan_ref(ids.cpu(), e, k, align, regions)
    assert torch.equal(pl.seg_count.cpu(), ref.seg_count)
    assert torch.equal(pl.seg_start.cpu(), ref.seg_start)
    assert torch.equal(pl.pair_row.cpu(), ref.pair_row)
    assert torch.equal(pl.row_token.cpu(), ref.row_token)
    assert torch.equal(pl.region_used.cpu(), ref.region_used)
    x = torch.randn(t, hidden, device="cuda").bfloat16()
    xs = moe.gather_rows(x, pl.row_token)
    ok = pl.row_token >= 0
    assert torch.equal(xs[ok], x[pl.row_token[ok].long()])
    out = moe.combine(xs, pl.pair_row, w, t, k)
    assert _rel(out, x.float() * w.sum(-1, keepdim=True)) < 5e-3


@pytest.mark.parametrize("quant", [False, True])
def test_rmsnorm_fused_combine(quant):
    """The MoE combine done inside the RMSNorm kernel equals combine -> residual add -> norm done by two kernels, bit for bit."""
    torch.manual_seed(15)
    t, e, k, hidden = 40, 128, 8, 2048
    ids, w = moe.route(torch.randn(t, e, device="cuda"), k)
    pl = moe.plan(ids, e, 32)
    y = torch.randn(pl.capacity, hidden, device="cuda").bfloat16()
    wt = (torch.randn(hidden, device="cuda") * 0.1 + 1).bfloat16()
    r1 = torch.randn(t, hidden, device="cuda").bfloat16()
    r2 = r1.clone()
    kw = dict(quantize=True, want_bf16=True, sf_layout=32) if quant else {}
    a = ew.rmsnorm(moe.combine(y, pl.pair_row, w, t, k), wt, 1e-6, residual=r1, **kw)
    b = ew.rmsnorm(moe.PendingCombine(y, pl.pair_row, w, t, k), wt, 1e-6, residual=r2, **kw)
    assert torch.equal(r1, r2)
    if quant:
        assert torch.equal(a[0], b[0]) and torch.equal(a[1].data[:t], b[1].data[:t])
        assert torch.equal(mxfp8.unpack_sf_atoms(a[1].sf, t, hidden // 32, 32), mxfp8.unpack_sf_atoms(b[1].sf, t, hidden // 32, 32))
    else:
        assert torch.equal(a, b)


def test_argmax_and_sample():
    torch.manual_seed(6)
    b, v = 5, 151936
    logits = torch.randn(b, v, device="cuda")
    logits[2, 100] = logits[2, 50000] = 50.0         # tie -> lower id
    assert sampling.argmax(logits).tolist() == torch.tensor([int(logits[i].argmax()) if i != 2 else 100 for i in range(b)]).tolist()
    assert sampling.argmax(logits.bfloat16(), idx_offset=7)[2].item() == 107
    # sampled tokens must come from the reference candidate set; frequencies roughly follow p
    row = torch.randn(v, device="cuda") * 3
    idx, p = sampling.candidate_set_ref(row.cpu(), 0.8, 20, 0.9)
    draws = torch.stack([sampling.sample(row.unsqueeze(0), 0.8, 20, 0.9, seed=1, step=s) for s in range(400)]).flatten().cpu()
    allowed = set(idx.tolist())
    assert all(int(d) in allowed for d in draws)
    top = int(idx[0])
    freq = (draws == top).float().mean().item()
    assert abs(freq - float(p[0])) < 0.12
    _native.assert_status_ok()


@pytest.mark.parametrize("lay", [32, 128])
def test_silu_mul_quant(lay):
    torch.manual_seed(21)
    rows, inter = 200, 768
    gu = torch.randn(rows, 2 * inter, device="cuda").bfloat16()
    valid = torch.arange(rows, device="cuda", dtype=torch.int32)
    valid[5] = -1
    rp = (rows + 127) // 128 * 128
    q = torch.zeros(rp, inter, dtype=torch.uint8, device="cuda")
    sf = ew.sf_alloc(rp, inter, "cuda", lay)
    ew.silu_mul_quant(gu, q, sf, valid, sf_layout=lay)
    g = gu.float()
    ref = mxfp8.quantize(torch.nn.functional.silu(g[:, :inter]) * g[:, inter:], sf_layout=lay)
    ok = valid >= 0
    # __expf in the kernel against torch's exp: allow one fp8 code of difference on a few elements
    a, b = mxfp8.dequantize(mxfp8.MxTensor(q, sf, rows, inter, lay)), mxfp8.dequantize(ref)
    assert _rel(a[ok], b[ok]) < 2e-2
    assert (q[5] == 0).all()


@pytest.mark.parametrize("t,e,k", [(1, 128, 2048), (64, 128, 2048), (77, 60, 1024), (256, 256, 4096)])
def test_router_logits_small_batch(t, e, k):
    torch.manual_seed(22)
    h = torch.randn(t, k, device="cuda").bfloat16()
    w = (torch.randn(e, k, device="cuda") * 0.05).bfloat16()
    got = moe.router_logits(h, w)
    ref = h.float() @ w.float().t()
    assert got.dtype == torch.float32 and _rel(got, ref) < 1e-5


@pytest.mark.parametrize("t,local", [(1, None), (64, None), (256, None), (64, (32, 16)), (200, (0, 64))])
def test_route_plan_single_kernel(t, local, monkeypatch):
    """Routing + plan in one launch equals the two separate ops."""
    torch.manual_seed(23)
    e, k, align = 128, 8, 32
    logits = torch.randn(t, e, device="cuda")
    n_plan = local[1] if local else e
    monkeypatch.setattr(moe, "FUSED_ROUTE_PAIRS", 2048)      # force the fused kernel also above its default threshold
    ids, w, pl = moe.route_plan(logits, k, n_plan, align, local_range=local)
    ids2, w2 = moe.route(logits, k, local_range=local)
    pl2 = moe.plan(ids2, n_plan, align)
    assert torch.equal(ids, ids2) and torch.equal(w, w2)
    for a, b in ((pl.seg_start, pl2.seg_start), (pl.seg_count, pl2.seg_count), (pl.pair_row, pl2.pair_row), (pl.row_token, pl2.row_token)):
        assert torch.equal(a, b)


@pytest.mark.parametrize("t,e,local,mode", [(64, 128, None, "softmax"), (5, 128, (32, 16), "softmax"), (33, 64, None, "sigmoid"), (8, 16, None, "softmax")])
def test_route_hidden_cluster_kernel(t, e, local, mode, monkeypatch):
    """Router projection + routing in one cluster launch equals the projection kernel followed by the routing kernel."""
    torch.manual_seed(31)
    hid, k = 2048, 8
    h = torch.randn(t, hid, device="cuda").bfloat16()
    w = (torch.randn(e, hid, device="cuda") * 0.05).bfloat16()
    bias = torch.randn(e, device="cuda") * 0.1 if mode == "sigmoid" else None
    monkeypatch.setattr(moe, "FUSED_ROUTER", True)
    assert moe.can_route_hidden(h, w, k)
    ids, wt = moe.route_hidden(h, w, k, mode, bias, True, 1.5, local)
    ids2, wt2 = moe.route(moe.router_logits(h, w), k, mode, bias, True, 1.5, local)
    assert torch.equal(ids, ids2) and torch.equal(wt, wt2)


def test_kv_int8_codec_matches_reference():
    from gemm_b200.ops import kvquant
    torch.manual_seed(41)
    x = (torch.randn(300, 4, 128, device="cuda") * torch.rand(300, 4, 1, device="cuda") * 5).bfloat16()
    x[7, 1] = 0
    q, sc = kvquant.quantize_q8(x)
    q_ref, sc_ref = kvquant.quantize_q8_ref(x.cpu())
    assert torch.equal(sc.cpu(), sc_ref)
    assert (q.cpu().int() - q_ref.int()).abs().max().item() <= 1          # rounding of ties / fma differences
    back = kvquant.dequantize_q8(q, sc)
    assert _rel(back, x) < 1e-2
