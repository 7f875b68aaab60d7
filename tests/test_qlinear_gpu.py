"""Fused dequant-GEMV / dequant-GEMM over ggml blocks kept in HBM (csrc/kernels/qgemv.cu, qgemm.cu) against a plain fp32
PyTorch product with the decoded weights (decoder = the bit-exact host decoder's torch twin, ops.ggml_torch)."""
import pytest
import torch

from gemm_b200 import _native
from gemm_b200.ops import ggml_torch as gt
from gemm_b200.ops import qlinear

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _case(t, rows, k, m, seed=0):
    torch.manual_seed(seed)
    w = torch.randn(rows, k, device="cuda") * 0.02
    x = torch.randn(m, k, device="cuda").bfloat16()
    qw = qlinear.QTensor.from_float(w, t)
    ref = x.float() @ qw.dequantize().t()
    return qw, x, ref


@pytest.mark.parametrize("t", [gt.Q4_K, gt.Q8_0])
@pytest.mark.parametrize("rows,k,m,splits", [(256, 512, 1, 1), (384, 1024, 3, 2), (5120, 5120, 1, None), (1280, 5120, 4, None),
                                             (200, 768, 2, 3), (5120, 3328, 2, None), (2560, 5120, 3, 1), (1280, 5120, 2, 2),
                                             (51200, 1024, 1, None)])      # the last three: K ranges longer than the tile ring (slots are refilled), many items per CTA
def test_gemv_matches_fp32_reference(t, rows, k, m, splits):
    qw, x, ref = _case(t, rows, k, m, seed=rows + m)
    p = qlinear.gemv_partials(x, qw, splits=splits)
    y = p.buf.sum(0)
    torch.cuda.synchronize()
    _native.assert_status_ok()
    # int8 activations (per-32 scales): the reference engine accepts 0.5 rel-L2 for this arithmetic; we are far below
    assert y.shape == ref.shape and _rel(y, ref) < 1.5e-2


@pytest.mark.parametrize("t", [gt.Q4_K, gt.Q8_0])
@pytest.mark.parametrize("rows,k,m", [(128, 256, 5), (256, 512, 16), (384, 1024, 37), (1280, 5120, 64), (200, 768, 130), (512, 2048, 300)])
def test_gemm_matches_fp32_reference(t, rows, k, m):
    qw, x, ref = _case(t, rows, k, m, seed=rows + m)
    y = qlinear.gemm(x, qw, out_dtype=torch.float32)
    torch.cuda.synchronize()
    _native.assert_status_ok()
    assert y.shape == ref.shape and _rel(y, ref) < 6e-3          # weights reach the tensor core rounded to bf16


@pytest.mark.parametrize("t", [gt.Q4_K, gt.Q8_0])
@pytest.mark.parametrize("rows,k,m,splits", [(256, 4096, 8, 2), (640, 8192, 24, 3), (128, 2048, 64, 8), (384, 2560, 5, 4)])
def test_gemm_k_split_partials_add_up(t, rows, k, m, splits):
    """The K-split form: every split writes its own fp32 slab (bias in the first only); their sum is the plain result."""
    qw, x, ref = _case(t, rows, k, m, seed=rows + m + splits)
    bias = torch.randn(rows, device="cuda")
    pend = qlinear.gemm_partials(x, qw, splits, bias=bias)
    torch.cuda.synchronize()
    _native.assert_status_ok()
    assert pend.buf.shape == (splits, m, rows)
    assert _rel(pend.buf.sum(0), ref + bias) < 6e-3
    # no slab is empty and none holds the whole sum
    norms = pend.buf.float().flatten(1).norm(dim=1)
    assert bool((norms > 0).all()) and float(norms.max()) < float((ref + bias).norm()) * 1.01
    assert qlinear.pick_gemm_splits(5120, 25600, 8) > 1 and qlinear.pick_gemm_splits(51200, 5120, 8) == 1


def test_gemm_bias_bf16_output_and_linear_dispatch():
    qw, x, ref = _case(gt.Q4_K, 640, 1024, 20, seed=5)
    bias = torch.randn(640, device="cuda")
    y = qlinear.linear(x, qw, bias=bias)
    assert y.dtype == torch.bfloat16 and _rel(y, ref + bias) < 1e-2
    y1 = qlinear.linear(x[:2], qw, bias=bias)                    # GEMV route
    assert _rel(y1, (ref + bias)[:2]) < 2e-2
    qgu, x2, ref2 = _case(gt.Q8_0, 512, 512, 3, seed=6)
    act = qlinear.linear_swiglu(x2, qgu)
    want = torch.nn.functional.silu(ref2[:, :256]) * ref2[:, 256:]
    assert _rel(act, want) < 2e-2
    act9 = qlinear.linear_swiglu(torch.cat([x2, x2, x2]), qgu)
    assert _rel(act9[:3], want) < 2e-2
    _native.assert_status_ok()
