"""The geometry kernels (csrc/kernels/geometry.cu) against the host library, which runs the same inline code in loops: splat rows,
iso-surface extraction, BVH ray / closest-point queries and the preview renderer give the same results on the device."""
import pytest
import torch

from gemm_b200 import geometry as geo

pytestmark = pytest.mark.gpu


def _grid(n, fn):
    ax = torch.linspace(-1, 1, n)
    return fn(*torch.meshgrid(ax, ax, ax, indexing="ij"))


def test_geometry_kernels_equal_the_host_path():
    dev = "cuda"
    g = torch.Generator().manual_seed(0)
    n = 1000
    args = [torch.randn(n, 3, generator=g), torch.randn(n, 3, generator=g), torch.randn(n, generator=g), torch.randn(n, 3, generator=g) * 3, torch.randn(n, 4, generator=g)]
    host = geo.gs_rows(*args, opacity_bias=0.1, scaling_bias=0.004)
    devr = geo.gs_rows(*[a.to(dev) for a in args], opacity_bias=0.1, scaling_bias=0.004)
    assert torch.allclose(devr.cpu(), host, atol=1e-5, rtol=1e-5)
    grid = _grid(48, lambda x, y, z: (((x * x + z * z).sqrt() - 0.55) ** 2 + y * y).sqrt() - 0.25 + 0.03 * torch.sin(7 * x))
    v, t = geo.isosurface(grid, 0.0)
    vd, td = geo.isosurface(grid.to(dev), 0.0)
    assert vd.is_cuda and torch.equal(td.cpu(), t) and torch.allclose(vd.cpu(), v, atol=1e-6)
    bh, bd = geo.Bvh(v, t), geo.Bvh(v, t, device=dev)
    o = torch.randn(4000, 3, generator=g) * 1.5
    d = torch.nn.functional.normalize(torch.randn(4000, 3, generator=g) - o, dim=1)
    th, trih, uvh = bh.trace(o, d)
    tdv, trid, uvd = bd.trace(o.to(dev), d.to(dev))
    hit = (trih >= 0) & (trid.cpu() >= 0)
    assert ((trid.cpu() >= 0) != (trih >= 0)).sum() <= 2          # a ray along an edge may fall either way (fused multiply-adds differ)
    assert hit.float().mean() > 0.1 and torch.allclose(tdv.cpu()[hit], th[hit], atol=1e-4, rtol=1e-4)
    assert ((bd.trace(o, d, any_hit=True)[1].cpu() >= 0) != (trih >= 0)).sum() <= 2
    q = torch.randn(4000, 3, generator=g)
    dh, _, ph, _ = bh.closest(q)
    dd, _, pd, wd = bd.closest(q)
    assert torch.allclose(dd.cpu(), dh, atol=1e-5) and torch.allclose(wd.sum(1).cpu(), torch.ones(4000), atol=1e-5)
    ih = bh.render((0, 1.2, -3.0), (0, 0, 0), 160, 120)
    idv = bd.render((0, 1.2, -3.0), (0, 0, 0), 160, 120)
    same = (idv["mask"].cpu() == ih["mask"]).float().mean()
    assert same > 0.999                                           # silhouette pixels may fall either way in the last bit
    agree = (idv["mask"].cpu() == ih["mask"])
    assert (idv["rgb"].cpu() - ih["rgb"]).abs()[agree].mean() < 1e-3 and torch.allclose(idv["depth"].cpu()[agree], ih["depth"][agree], atol=1e-4)
