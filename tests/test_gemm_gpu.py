"""tcgen05 GEMM kernel vs a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

from gemm_b200 import _native
from gemm_b200.ops import gemm, mxfp8

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("m,n,k", [(8, 256, 512), (16, 128, 64), (37, 384, 1024), (64, 5120, 2048), (130, 200, 264),
                                   (300, 1024, 4096), (1024, 2048, 2048)])
def test_linear_bf16(m, n, k):
    torch.manual_seed(0)
    x = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    y = gemm.linear(x, w)
    ref = x.float() @ w.float().t()
    _native.assert_status_ok()
    assert _rel(y, ref) < 1e-2


def test_linear_bias_f32_out():
    torch.manual_seed(1)
    x = torch.randn(20, 256, device="cuda").bfloat16()
    w = torch.randn(130, 256, device="cuda").bfloat16()
    b = torch.randn(130, device="cuda")
    y = gemm.linear(x, w, bias=b, out_dtype=torch.float32)
    ref = x.float() @ w.float().t() + b
    _native.assert_status_ok()
    assert _rel(y, ref) < 1e-3


@pytest.mark.parametrize("m,inter,k", [(8, 128, 256), (100, 768, 2048), (512, 1536, 1024)])
def test_linear_swiglu(m, inter, k):
    torch.manual_seed(2)
    x = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(2 * inter, k, device="cuda") * 0.05).bfloat16()
    y = gemm.linear_swiglu(x, w)
    r = x.float() @ w.float().t()
    ref = torch.nn.functional.silu(r[:, :inter]) * r[:, inter:]
    _native.assert_status_ok()
    assert _rel(y, ref) < 1e-2


@pytest.mark.parametrize("m,n,k,lay", [(8, 128, 128, 128), (32, 256, 512, 128), (70, 768, 2048, 128), (256, 2048, 768, 128),
                                       (1000, 512, 1024, 128), (8, 256, 512, 32), (32, 5120, 2048, 32)])
def test_linear_mxfp8(m, n, k, lay):
    torch.manual_seed(3)
    x = torch.randn(m, k, device="cuda") * torch.rand(m, 1, device="cuda") * 4
    w = torch.randn(n, k, device="cuda") * 0.05
    xq, wq = mxfp8.quantize(x, sf_layout=lay), mxfp8.quantize(w)
    y = gemm.linear_mx(xq, wq, out_dtype=torch.float32)
    ref = mxfp8.dequantize(xq) @ mxfp8.dequantize(wq).t()
    _native.assert_status_ok()
    assert _rel(y, ref) < 2e-3


@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (300, 384, 768), (700, 512, 2048), (1024, 2048, 4096)])
def test_linear_mxfp8_wide_tile(m, n, k):
    """bf16 results of 256 or more tokens take the 256-token tile (one accumulator buffer, registers staged epilogue); the
    last tile may end in its first or its second half."""
    torch.manual_seed(31)
    x = torch.randn(m, k, device="cuda") * torch.rand(m, 1, device="cuda") * 4
    w = torch.randn(n, k, device="cuda") * 0.05
    bias = torch.randn(n, device="cuda")
    xq, wq = mxfp8.quantize(x, sf_layout=128), mxfp8.quantize(w)
    assert gemm.WIDE_TILE
    y = gemm.linear_mx(xq, wq, bias=bias)
    y128 = gemm.linear_mx(xq, wq, bias=bias, tn=128)
    ref = mxfp8.dequantize(xq) @ mxfp8.dequantize(wq).t() + bias
    _native.assert_status_ok()
    assert y.dtype == torch.bfloat16 and _rel(y, ref) < 4e-3
    assert torch.equal(y, y128)


def test_grouped_mxfp8_wide_tile():
    torch.manual_seed(32)
    g, n, k = 5, 384, 512
    counts = torch.tensor([300, 0, 129, 512, 90], dtype=torch.int32)       # the last segment ends the buffer in a tile's first half
    starts = torch.zeros(g, dtype=torch.int32)
    pos = 0
    for i in range(g):
        starts[i] = pos
        pos += (int(counts[i]) + 127) // 128 * 128
    rows = max(pos, 256 * g)
    x = torch.randn(rows, k, device="cuda")
    w = torch.randn(g, n, k, device="cuda") * 0.05
    xq = mxfp8.quantize(x, sf_layout=128)
    wq = mxfp8.quantize(w.reshape(g * n, k))
    sd, cd = starts.cuda(), counts.cuda()
    y = gemm.grouped_linear(xq.data, wq.data.reshape(g, n, k), sd, cd, 128, sfa=wq.sf, sfb=xq.sf)
    _native.assert_status_ok()
    xf, wf = mxfp8.dequantize(xq), mxfp8.dequantize(wq).reshape(g, n, k)
    for i in range(g):
        s0, c = int(starts[i]), int(counts[i])
        if c:
            assert _rel(y[s0:s0 + c], xf[s0:s0 + c] @ wf[i].t()) < 4e-3, f"group {i}"


@pytest.mark.parametrize("m,inter,k,lay", [(8, 128, 256, 128), (100, 768, 2048, 128), (20, 768, 2048, 32)])
def test_mx_swiglu_quant_epilogue(m, inter, k, lay):
    torch.manual_seed(4)
    x = torch.randn(m, k, device="cuda")
    w = torch.randn(2 * inter, k, device="cuda") * 0.05
    xq, wq = mxfp8.quantize(x, sf_layout=lay), mxfp8.quantize(w)
    hq = gemm.linear_mx_swiglu_quant(xq, wq)
    r = mxfp8.dequantize(xq) @ mxfp8.dequantize(wq).t()
    ref = torch.nn.functional.silu(r[:, :inter]) * r[:, inter:]
    _native.assert_status_ok()
    got = mxfp8.dequantize(hq)
    assert _rel(got, ref) < 5e-2          # e4m3 has 3 mantissa bits
    # scales must be the ones the reference quantiser picks for (nearly) the same values
    ref_q = mxfp8.quantize(ref)
    e_ref = mxfp8.unpack_sf_atoms(ref_q.sf, m, inter // 32).int()
    e_got = mxfp8.unpack_sf_atoms(hq.sf, m, inter // 32, lay).int()
    assert (e_ref - e_got).abs().max().item() <= 1


@pytest.mark.parametrize("mx,tn", [(False, 32), (True, 128), (True, 32)])
def test_grouped(mx, tn):
    torch.manual_seed(5)
    g, inter, k = 6, 256, 512
    counts = torch.tensor([5, 0, 140, 32, 1, 17], dtype=torch.int32)
    starts = torch.zeros(g, dtype=torch.int32)
    pos = 0
    for i in range(g):
        starts[i] = pos
        pos += (int(counts[i]) + tn - 1) // tn * tn
    rows = (pos + 127) // 128 * 128
    x = torch.randn(rows, k, device="cuda")
    w = torch.randn(g, 2 * inter, k, device="cuda") * 0.05
    sd, cd = starts.cuda(), counts.cuda()
    if mx:
        xq = mxfp8.quantize(x, sf_layout=tn)
        wq = mxfp8.quantize(w.reshape(g * 2 * inter, k))
        y = gemm.grouped_linear(xq.data, wq.data.reshape(g, 2 * inter, k), sd, cd, tn, dual=True, sfa=wq.sf, sfb=xq.sf)
        xf, wf = mxfp8.dequantize(xq), mxfp8.dequantize(wq).reshape(g, 2 * inter, k)
    else:
        y = gemm.grouped_linear(x.bfloat16(), w.bfloat16(), sd, cd, tn, dual=True)
        xf, wf = x.bfloat16().float(), w.bfloat16().float()
    _native.assert_status_ok()
    for i in range(g):
        s, c = int(starts[i]), int(counts[i])
        if c == 0:
            continue
        r = xf[s:s + c] @ wf[i].t()
        ref = torch.nn.functional.silu(r[:, :inter]) * r[:, inter:]
        assert _rel(y[s:s + c], ref) < 1e-2, f"group {i}"


@pytest.mark.parametrize("m,n,k,mx", [(8, 2048, 2048, False), (64, 2048, 4096, False), (8, 2048, 2048, True), (64, 2048, 4096, True), (20, 128, 2048, False)])
def test_split_k_small_batches(m, n, k, mx):
    """The optional split-K path (few tiles, long K): same result, and bit-identical from run to run."""
    torch.manual_seed(6)
    x = torch.randn(m, k, device="cuda") * 0.5
    w = torch.randn(n, k, device="cuda") * 0.05
    if mx:
        xq, wq = mxfp8.quantize(x, sf_layout=32 if m <= 32 else 128), mxfp8.quantize(w)
        assert gemm._splitk_extras(n, m, k, xq.sf_layout, True, x.device, True) is not None
        y1 = gemm.linear_mx(xq, wq, out_dtype=torch.float32, tn=xq.sf_layout, split_k=True)
        y2 = gemm.linear_mx(xq, wq, out_dtype=torch.float32, tn=xq.sf_layout, split_k=True)
        ref = mxfp8.dequantize(xq) @ mxfp8.dequantize(wq).t()
    else:
        assert gemm._splitk_extras(n, m, k, gemm.pick_tn(m), False, x.device, True) is not None
        y1 = gemm.linear(x.bfloat16(), w.bfloat16(), out_dtype=torch.float32, split_k=True)
        y2 = gemm.linear(x.bfloat16(), w.bfloat16(), out_dtype=torch.float32, split_k=True)
        ref = x.bfloat16().float() @ w.bfloat16().float().t()
    _native.assert_status_ok()
    assert torch.equal(y1, y2)
    assert _rel(y1, ref) < 2e-3


def test_linear_argmax_matches_logits_argmax():
    torch.manual_seed(7)
    m, n, k = 64, 151936, 256
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = torch.randn(n, k, device="cuda").bfloat16()
    idx, val = gemm.linear_argmax(x, w, idx_offset=5, want_value=True)
    logits = gemm.linear(x, w, out_dtype=torch.float32)
    _native.assert_status_ok()
    ref_val, ref_idx = logits.max(dim=-1)
    assert torch.equal(idx.long() - 5, ref_idx) and torch.equal(val, ref_val)


@pytest.mark.parametrize("m", [8, 64, 300])
def test_tiled_weight_layout_is_bit_identical(m):
    """The tiled weight layout changes where the bytes live, not what is computed."""
    torch.manual_seed(12)
    n, k = 1024, 2048
    x = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    wt = mxfp8.tile_weight(w)
    assert torch.equal(mxfp8.untile_weight(wt), w)
    assert torch.equal(gemm.linear(x, w), gemm.linear(x, wt, w_tiled=True))
    assert torch.equal(gemm.linear_swiglu(x, w), gemm.linear_swiglu(x, wt, w_tiled=True))
    lay = 32 if m <= 32 else 128
    xq, wq = mxfp8.quantize(x.float(), sf_layout=lay), mxfp8.quantize(w.float())
    wqt = mxfp8.MxTensor(mxfp8.tile_weight(wq.data), wq.sf, wq.rows, wq.k, 128, tiled=True)
    assert torch.equal(mxfp8.dequantize(wqt), mxfp8.dequantize(wq))
    assert torch.equal(gemm.linear_mx(xq, wq), gemm.linear_mx(xq, wqt))
    a, b = gemm.linear_mx_swiglu_quant(xq, wq), gemm.linear_mx_swiglu_quant(xq, wqt)
    assert torch.equal(a.data[:m], b.data[:m])
    _native.assert_status_ok()


def test_tiled_grouped_weights():
    torch.manual_seed(13)
    g, inter, k, tn = 8, 256, 512, 32
    counts = torch.tensor([3, 0, 32, 17, 1, 40, 5, 9])
    starts = torch.zeros(g, dtype=torch.int64)
    pos = 0
    for i in range(g):
        starts[i] = pos
        pos += (int(counts[i]) + tn - 1) // tn * tn
    cap = (pos + 127) // 128 * 128
    x = torch.randn(cap, k, device="cuda") * 0.5
    w = torch.randn(g * 2 * inter, k, device="cuda") * 0.05
    sd, cd = starts.to("cuda", torch.int32), counts.to("cuda", torch.int32)
    xq, wq = mxfp8.quantize(x, sf_layout=32), mxfp8.quantize(w)
    y0 = gemm.grouped_linear(xq.data, wq.data.view(g, 2 * inter, k), sd, cd, tn, dual=True, sfa=wq.sf, sfb=xq.sf)
    y1 = gemm.grouped_linear(xq.data, mxfp8.tile_weight(wq.data).view(g, 2 * inter, k), sd, cd, tn, dual=True, sfa=wq.sf, sfb=xq.sf, w_tiled=True)
    for i in range(g):
        s, c = int(starts[i]), int(counts[i])
        assert torch.equal(y0[s:s + c], y1[s:s + c])
    _native.assert_status_ok()


def test_expert_gate_up_prefill_path_matches_fused_epilogue():
    """Token tile 128: plain GEMM + SiLU*up+quantise kernel gives the same activations as the fused two-accumulator epilogue."""
    from gemm_b200.models.transformer import expert_gate_up_mx
    from gemm_b200.models.weights import make_linear
    from gemm_b200.ops import elementwise as ew
    torch.manual_seed(14)
    g, inter, k, tn = 4, 256, 512, 128
    counts = torch.tensor([100, 0, 128, 300])
    starts = torch.tensor([0, 128, 128, 256])
    cap = 640
    x = torch.randn(cap, k, device="cuda") * 0.5
    w13 = make_linear(torch.randn(g * 2 * inter, k, device="cuda") * 0.05, "mxfp8", groups=g)
    sd, cd = starts.to("cuda", torch.int32), counts.to("cuda", torch.int32)
    xq = mxfp8.quantize(x, sf_layout=128)
    hq = torch.zeros(cap, inter, dtype=torch.uint8, device="cuda")
    hsf = ew.sf_alloc(cap, inter, "cuda", 128)
    expert_gate_up_mx(xq.data, xq.sf, w13, g, sd, cd, tn, hq, hsf)
    ref_q = torch.zeros(cap, inter, dtype=torch.uint8, device="cuda")
    ref_sf = ew.sf_alloc(cap, inter, "cuda", 128)
    gemm.grouped_linear(xq.data, w13.mx.data.view(g, 2 * inter, k), sd, cd, tn, out=ref_q, dual=True, sfa=w13.mx.sf, sfb=xq.sf, quant_out=True,
                        out_sf=ref_sf, w_tiled=w13.mx.tiled)
    a = mxfp8.dequantize(mxfp8.MxTensor(hq, hsf, cap, inter, 128))
    b = mxfp8.dequantize(mxfp8.MxTensor(ref_q, ref_sf, cap, inter, 128))
    for i in range(g):
        s, c = int(starts[i]), int(counts[i])
        if c:
            assert _rel(a[s:s + c], b[s:s + c]) < 3e-2, f"group {i}"
    _native.assert_status_ok()


@pytest.mark.parametrize("m,n,k", [(64, 2048, 4096), (8, 2048, 4096), (33, 256, 1024)])
def test_linear_mx_partials_feed_the_norm(m, n, k):
    """K-split partial sums (one fp32 slab per split) summed by the residual add + RMSNorm kernel."""
    from gemm_b200.ops import elementwise as ew
    torch.manual_seed(41)
    x = torch.randn(m, k, device="cuda")
    w = torch.randn(n, k, device="cuda") * 0.05
    bias = torch.randn(n, device="cuda")
    lay = 32 if m <= 32 else 128
    xq, wq = mxfp8.quantize(x, sf_layout=lay), mxfp8.quantize(w)
    sp = gemm.pick_partials(n, m, k, True)
    assert sp > 1
    pend = gemm.linear_mx_partials(xq, wq, sp, bias=bias)
    ref = mxfp8.dequantize(xq) @ mxfp8.dequantize(wq).t() + bias
    _native.assert_status_ok()
    assert _rel(pend.buf.sum(0), ref) < 2e-3
    res = torch.randn(m, n, device="cuda").bfloat16()
    nw = (1 + 0.1 * torch.randn(n, device="cuda")).bfloat16()
    res2 = res.clone()
    got = ew.rmsnorm(pend, nw, 1e-6, residual=res)
    want = ew.rmsnorm(pend.materialize(), nw, 1e-6, residual=res2)
    assert _rel(got, want) < 1e-2 and _rel(res, res2) < 1e-2


@pytest.mark.parametrize("m,n,k", [(32, 4096, 12288), (8, 1024, 4096)])
def test_linear_bf16_partials(m, n, k):
    torch.manual_seed(42)
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    bias = torch.randn(n, device="cuda")
    sp = gemm.pick_partials(n, m, k, False)
    assert sp > 1
    pend = gemm.linear_partials(x, w, sp, bias=bias)
    _native.assert_status_ok()
    ref = x.float() @ w.float().t() + bias
    assert _rel(pend.buf.sum(0), ref) < 2e-3
    assert _rel(pend.materialize(), gemm.linear(x, w, bias=bias)) < 1e-2


@pytest.mark.parametrize("mx", [False, True])
def test_swiglu_from_k_split_partials(mx):
    from gemm_b200.ops import elementwise as ew
    torch.manual_seed(43)
    m, inter, k = 32, 1536, 4096
    x = torch.randn(m, k, device="cuda")
    w = torch.randn(2 * inter, k, device="cuda") * 0.03
    sp = gemm.pick_partials_dual(inter, m, k, mx)
    assert sp > 1
    if mx:
        xq, wq = mxfp8.quantize(x, sf_layout=32), mxfp8.quantize(w)
        got = ew.silu_mul_partials(gemm.swiglu_partials(xq, wq, sp), quantize=True, sf_layout=32)
        want = gemm.linear_mx_swiglu_quant(xq, wq)
        _native.assert_status_ok()
        assert _rel(mxfp8.dequantize(got), mxfp8.dequantize(want)) < 2e-2
    else:
        got = ew.silu_mul_partials(gemm.swiglu_partials(x.bfloat16(), w.bfloat16(), sp))
        want = gemm.linear_swiglu(x.bfloat16(), w.bfloat16())
        _native.assert_status_ok()
        assert _rel(got, want) < 1e-2


@pytest.mark.parametrize("mx", [True, False])
def test_grouped_pair_rows_equals_plain(mx):
    """Two row blocks of one projection per tile (two accumulators, plain stores) give the plain grouped GEMM's result."""
    torch.manual_seed(44)
    g, n, k, tn = 5, 512, 768, 32
    counts = torch.tensor([5, 0, 32, 17, 1], dtype=torch.int32)
    starts = torch.zeros(g, dtype=torch.int32)
    pos = 0
    for i in range(g):
        starts[i] = pos
        pos += (int(counts[i]) + tn - 1) // tn * tn
    rows = (pos + 127) // 128 * 128
    x = torch.randn(rows, k, device="cuda")
    w = torch.randn(g, n, k, device="cuda") * 0.05
    sd, cd = starts.cuda(), counts.cuda()
    if mx:
        xq = mxfp8.quantize(x, sf_layout=tn)
        wq = mxfp8.quantize(w.reshape(g * n, k))
        a = gemm.grouped_linear(xq.data, wq.data.reshape(g, n, k), sd, cd, tn, sfa=wq.sf, sfb=xq.sf, pair_rows=True)
        b = gemm.grouped_linear(xq.data, wq.data.reshape(g, n, k), sd, cd, tn, sfa=wq.sf, sfb=xq.sf)
    else:
        a = gemm.grouped_linear(x.bfloat16(), w.bfloat16(), sd, cd, tn, pair_rows=True)
        b = gemm.grouped_linear(x.bfloat16(), w.bfloat16(), sd, cd, tn)
    _native.assert_status_ok()
    for i in range(g):
        s0, c = int(starts[i]), int(counts[i])
        if c:
            assert torch.equal(a[s0:s0 + c], b[s0:s0 + c]), f"group {i}"
