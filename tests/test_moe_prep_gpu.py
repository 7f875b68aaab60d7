"""The one-launch MoE front end (router projection + routing + plan + quantised gather, csrc/kernels/moe_prep.cu) against the
fp32 PyTorch references of its four stages."""
import pytest
import torch

from gemm_b200 import _native
from gemm_b200.ops import moe, mxfp8

pytestmark = pytest.mark.gpu


def _reference(h, w, k, n_plan, align, mode, bias, local_range):
    # The kernel multiplies bf16 operands exactly and accumulates in fp32.  The reference does the same in fp64, so the
    # only difference is the order of the fp32 sums; tokens whose k-th and (k+1)-th scores are that close are skipped.
    logits = (h.double().cpu() @ w.double().cpu().t()).float()
    ids, wts = moe.route_ref(logits, k, mode, bias.cpu() if bias is not None else None, True, 1.0)
    sel = torch.softmax(logits, -1) if mode == "softmax" else torch.sigmoid(logits) + (bias.cpu() if bias is not None else 0.0)
    top = torch.sort(sel, dim=-1, descending=True).values
    clear = (top[:, k - 1] - top[:, k]).abs() > 1e-5 * top[:, k - 1].abs() if top.shape[1] > k else torch.ones(len(top), dtype=torch.bool)
    if local_range is not None:
        lid = ids - local_range[0]
        ids = torch.where((lid >= 0) & (lid < local_range[1]), lid, torch.full_like(lid, -1))
    return logits, ids, wts, clear, moe.plan_ref(ids, n_plan, k, align)


@pytest.mark.parametrize("t,hidden,e,k,align,mode,local", [
    (64, 2048, 128, 8, 32, "softmax", None),       # the benchmark's decode step
    (64, 2048, 128, 8, 32, "softmax", (48, 16)),   # one expert-parallel rank of eight
    (37, 2048, 128, 8, 32, "sigmoid", None),
    (5, 256, 8, 2, 32, "softmax", None),           # one CTA, no cluster partner
    (64, 4096, 128, 8, 32, "softmax", None),       # 16-CTA cluster
    (19, 1024, 64, 4, 16, "softmax", None),
])
def test_prep_matches_the_staged_references(t, hidden, e, k, align, mode, local):
    torch.manual_seed(t + hidden + e)
    h = torch.randn(t, hidden, device="cuda").bfloat16()
    w = (torch.randn(e, hidden, device="cuda") * 0.05).bfloat16()
    bias = (torch.randn(e, device="cuda") * 0.1) if mode == "sigmoid" else None
    n_plan = local[1] if local else e
    quant = align in (32, 128)
    assert moe.can_prep(h, w, k)
    ids, wts, pl, rows = moe.prep_hidden(h, w, k, n_plan, align, mode, bias, True, 1.0, local, quantize=quant)
    torch.cuda.synchronize()
    _native.assert_status_ok()
    logits, ids_r, wts_r, clear, pl_r = _reference(h, w, k, n_plan, align, mode, bias, local)
    assert clear.float().mean() > 0.9
    assert torch.equal(ids.cpu()[clear], ids_r[clear])
    assert torch.allclose(wts.cpu()[clear], wts_r[clear], rtol=2e-3, atol=1e-6)
    if not bool(clear.all()):
        return                                   # a near-tie moved a token: the plan differs legitimately
    assert torch.equal(pl.seg_start.cpu(), pl_r.seg_start) and torch.equal(pl.seg_count.cpu(), pl_r.seg_count)
    assert torch.equal(pl.pair_row.cpu(), pl_r.pair_row)
    assert pl.capacity == pl_r.capacity and torch.equal(pl.row_token.cpu(), pl_r.row_token)
    valid = (pl_r.row_token >= 0).nonzero().squeeze(1)
    src = pl_r.row_token[valid].long()
    if quant:
        q_ref = mxfp8.quantize(h.float().cpu(), sf_layout=align)          # every token quantised once, rows then gathered
        assert torch.equal(rows.data.cpu()[valid], q_ref.data[src])
        sf = mxfp8.unpack_sf_atoms(rows.sf.cpu(), pl.capacity, hidden // 32, align)
        sf_ref = mxfp8.unpack_sf_atoms(q_ref.sf, q_ref.data.shape[0], hidden // 32, align)
        assert torch.equal(sf[valid], sf_ref[src])
    else:
        assert torch.equal(rows.cpu()[valid], h.cpu()[src])


def test_prep_equals_the_separate_kernels():
    """Same ids, weights, plan and quantised rows as router projection -> routing -> plan -> quantised gather run as four launches."""
    from gemm_b200.ops import elementwise as ew
    torch.manual_seed(3)
    t, hidden, e, k = 64, 2048, 128, 8
    h = torch.randn(t, hidden, device="cuda").bfloat16()
    w = (torch.randn(e, hidden, device="cuda") * 0.05).bfloat16()
    ids, wts, pl, rows = moe.prep_hidden(h, w, k, e, 32)
    ids2, wts2 = moe.route(moe.router_logits(h, w), k)
    pl2 = moe.plan(ids2, e, 32)
    xq2 = ew.mx_quantize(h, pl2.row_token, sf_layout=32)
    torch.cuda.synchronize()
    same = (ids == ids2).all(dim=1)
    assert same.float().mean() > 0.95                      # the two logit sums add in different orders: near-ties may swap
    assert torch.allclose(wts[same], wts2[same], rtol=1e-3, atol=1e-6)
    if bool(same.all()):
        assert torch.equal(pl.pair_row, pl2.pair_row) and torch.equal(pl.seg_start, pl2.seg_start)
        valid = pl2.row_token >= 0
        assert torch.equal(rows.data[: pl2.capacity][valid], xq2.data[: pl2.capacity][valid])
    _native.assert_status_ok()
