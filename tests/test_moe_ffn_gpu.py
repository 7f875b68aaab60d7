"""The one-launch expert FFN (gate/up + SiLU * up + MXFP8 re-quantisation + down, csrc/kernels/moe_ffn.cu) against the two grouped
GEMM launches it replaces (bit for bit: same operands, same order of sums) and against an fp32 PyTorch evaluation of the
dequantised operands."""
import pytest
import torch

from gemm_b200 import _native
from gemm_b200.models.transformer import expert_gate_up_mx
from gemm_b200.models.weights import make_linear
from gemm_b200.ops import elementwise as ew, gemm, moe, mxfp8

pytestmark = pytest.mark.gpu


def _setup(t, hidden, inter, e, k, seed):
    torch.manual_seed(seed)
    h = torch.randn(t, hidden, device="cuda").bfloat16()
    router = (torch.randn(e, hidden, device="cuda") * 0.05).bfloat16()
    w13 = make_linear(torch.randn(e * 2 * inter, hidden, device="cuda") * 0.03, "mxfp8", groups=e)
    w2 = make_linear(torch.randn(e * hidden, inter, device="cuda") * 0.03, "mxfp8", groups=e)
    w13.tile_()
    w2.tile_()
    ids, wts, pl, xq = moe.prep_hidden(h, router, k, e, 32)
    return h, w13, w2, ids, wts, pl, xq


def _two_launches(xq, w13, w2, e, pl, hidden, inter):
    hq = torch.empty(pl.capacity, inter, dtype=torch.uint8, device="cuda")
    hsf = ew.sf_alloc(pl.capacity, inter, "cuda", 32, init=False)
    expert_gate_up_mx(xq.data, xq.sf, w13, e, pl.seg_start, pl.seg_count, 32, hq, hsf, pl.row_token)
    return gemm.grouped_linear(hq, w2.mx.data.view(e, hidden, inter), pl.seg_start, pl.seg_count, 32, sfa=w2.mx.sf, sfb=hsf,
                               w_tiled=True, pair_rows=True)


@pytest.mark.parametrize("t,hidden,inter,e,k", [
    (64, 2048, 768, 128, 8),      # the benchmark's decode step: 768 + 1024 tiles on 148 CTAs
    (64, 2048, 768, 16, 8),       # one expert-parallel rank: segments of more than one token block
    (7, 512, 256, 8, 2),          # fewer tiles than CTAs
    (33, 1024, 384, 32, 4),
])
def test_fused_ffn_equals_the_two_grouped_gemms(t, hidden, inter, e, k):
    h, w13, w2, ids, wts, pl, xq = _setup(t, hidden, inter, e, k, seed=t + e)
    assert moe.can_fuse_ffn(xq, w13, w2, e, pl.capacity)
    y = moe.expert_ffn_fused(xq, w13, w2, e, pl)
    y2 = moe.expert_ffn_fused(xq, w13, w2, e, pl)             # the counters were left at zero: a second launch gives the same
    ref = _two_launches(xq, w13, w2, e, pl, hidden, inter)
    torch.cuda.synchronize()
    _native.assert_status_ok()
    rows = (pl.row_token >= 0).nonzero().squeeze(1)
    assert rows.numel() == t * k
    assert torch.equal(y[rows], ref[rows])
    assert torch.equal(y2[rows], y[rows])


def test_fused_ffn_matches_fp32_reference():
    t, hidden, inter, e, k = 48, 1024, 384, 16, 4
    h, w13, w2, ids, wts, pl, xq = _setup(t, hidden, inter, e, k, seed=11)
    y = moe.expert_ffn_fused(xq, w13, w2, e, pl).float().cpu()
    torch.cuda.synchronize()
    _native.assert_status_ok()
    w13f = mxfp8.dequantize_rowmajor(mxfp8.untile_weight(w13.mx.data.cpu()), mxfp8.unpack_sf_atoms(w13.mx.sf.cpu(), e * 2 * inter, hidden // 32))
    w2f = mxfp8.dequantize_rowmajor(mxfp8.untile_weight(w2.mx.data.cpu()), mxfp8.unpack_sf_atoms(w2.mx.sf.cpu(), e * hidden, inter // 32))
    xf = mxfp8.dequantize_rowmajor(xq.data.cpu(), mxfp8.unpack_sf_atoms(xq.sf.cpu(), pl.capacity, hidden // 32, 32))
    seg_start, seg_count = pl.seg_start.cpu(), pl.seg_count.cpu()
    worst = 0.0
    for g in range(e):
        s, c = int(seg_start[g]), int(seg_count[g])
        if c == 0:
            continue
        gu = xf[s:s + c] @ w13f[g * 2 * inter:(g + 1) * 2 * inter].t()
        act = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
        ref = act @ w2f[g * hidden:(g + 1) * hidden].t()
        err = (y[s:s + c] - ref).norm() / (ref.norm() + 1e-12)
        worst = max(worst, float(err))
    assert worst < 0.05, worst        # the activations pass through e4m3 (3 mantissa bits) between the two projections


def test_fused_ffn_reports_bad_segments():
    """Segments that leave a hole in the row space are refused on the device: status word set, nothing written, no hang."""
    t, hidden, inter, e, k = 8, 512, 256, 8, 2
    h, w13, w2, ids, wts, pl, xq = _setup(t, hidden, inter, e, k, seed=5)
    bad = moe.MoePlan(pl.seg_start + 32 * (torch.arange(e, device="cuda", dtype=torch.int32) >= 4).int(), pl.seg_count, pl.pair_row,
                      pl.row_token, pl.region_used, pl.capacity, pl.region_rows)
    if int((pl.seg_count[4:] > 0).sum()) == 0 or int(bad.seg_start.max() + 32) > pl.capacity:
        pytest.skip("routing left no rows behind the hole")
    _native.read_status()
    moe.expert_ffn_fused(xq, w13, w2, e, bad)
    torch.cuda.synchronize()
    st = _native.read_status()
    assert st["code"] == 3 and st["where"] == 631, st
    y = moe.expert_ffn_fused(xq, w13, w2, e, pl)                # the next launch is unaffected
    torch.cuda.synchronize()
    _native.assert_status_ok()
    ref = _two_launches(xq, w13, w2, e, pl, hidden, inter)
    rows = (pl.row_token >= 0).nonzero().squeeze(1)
    assert torch.equal(y[rows], ref[rows])
