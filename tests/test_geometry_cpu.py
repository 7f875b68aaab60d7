"""Geometry post-processing (gemm_b200.geometry) on the host path, which runs the inline code of the CUDA kernels in loops: splat
rows and PLY files, iso-surface extraction, BVH ray and closest-point queries, the preview renderer.  Oracles: closed forms, brute
force in torch, and the reference's marching cubes / PLY writer where they apply."""
import ctypes
import math

import numpy as np
import pytest
import torch

from gemm_b200 import geometry as geo
from tests import reference_oracle as oracle

needs_ref = pytest.mark.skipif(not oracle.available(), reason="reference source tree or gcc not present")


def _grid(n, fn, lo=-1.0, hi=1.0):
    ax = torch.linspace(lo, hi, n)
    return fn(*torch.meshgrid(ax, ax, ax, indexing="ij"))


def _edges(tris, n_verts):
    e = torch.cat([tris[:, [0, 1]], tris[:, [1, 2]], tris[:, [2, 0]]]).long()
    return e[:, 0] * n_verts + e[:, 1], e[:, 1] * n_verts + e[:, 0]


def test_splat_rows_and_ply_round_trip(tmp_path):
    g = torch.Generator().manual_seed(0)
    n = 50
    xyz, dc, op, sc, rot = torch.randn(n, 3, generator=g), torch.randn(n, 3, generator=g), torch.randn(n, generator=g), torch.randn(n, 3, generator=g) * 3, torch.randn(n, 4, generator=g)
    rows = geo.gs_rows(xyz, dc, op, sc, rot, opacity_bias=0.1, scaling_bias=0.004)
    shift = math.log(math.expm1(0.004))
    want_scale = torch.log(torch.nn.functional.softplus(sc.double() + shift)).float()
    assert torch.equal(rows[:, :3], xyz) and torch.equal(rows[:, 3:6], torch.zeros(n, 3)) and torch.equal(rows[:, 6:9], dc) and torch.equal(rows[:, 13:], rot)
    assert torch.allclose(rows[:, 9], op + 0.1) and torch.allclose(rows[:, 10:13], want_scale, atol=1e-5, rtol=1e-5)
    path = str(tmp_path / "splats.ply")
    geo.write_gs_ply(path, rows)
    back, names, faces = geo.read_ply(path)
    assert names == list(geo.GS_FIELDS) and faces is None and torch.equal(back, rows)
    if oracle.available():                                       # the reference's writer makes the same bytes from the same fields
        lib = oracle.geometry_lib()
        ref_path = str(tmp_path / "ref.ply")
        cols = [rows[:, :3].contiguous(), None, rows[:, 6:9].contiguous(), rows[:, 9].contiguous(), rows[:, 10:13].contiguous(), rows[:, 13:].contiguous()]
        assert lib.gs_ply_write(ref_path.encode(), n, *[c.data_ptr() if c is not None else None for c in cols]) == 0
        assert open(ref_path, "rb").read() == open(path, "rb").read()


@pytest.mark.parametrize("shape", ["sphere", "torus", "two_spheres"])
def test_isosurface_is_closed_oriented_and_on_the_level_set(shape, tmp_path):
    n = 41
    if shape == "sphere":
        f, euler = lambda x, y, z: (x * x + y * y + z * z).sqrt() - 0.62, 2
        area, vol = 4 * math.pi * 0.62 ** 2, 4 / 3 * math.pi * 0.62 ** 3
    elif shape == "torus":
        f, euler = lambda x, y, z: (((x * x + z * z).sqrt() - 0.55) ** 2 + y * y).sqrt() - 0.22, 0
        area, vol = 4 * math.pi ** 2 * 0.55 * 0.22, 2 * math.pi ** 2 * 0.55 * 0.22 ** 2
    else:
        f = lambda x, y, z: torch.minimum(((x - 0.45) ** 2 + y * y + z * z).sqrt() - 0.3, ((x + 0.45) ** 2 + y * y + z * z).sqrt() - 0.25)
        euler, area, vol = 4, 4 * math.pi * (0.09 + 0.0625), 4 / 3 * math.pi * (0.027 + 0.015625)
    grid = _grid(n, f)
    v, t = geo.isosurface(grid, 0.0)
    assert v.shape[0] > 100 and t.dtype == torch.int32
    fwd, rev = _edges(t, v.shape[0])
    assert fwd.unique().numel() == fwd.numel(), "a directed edge is used twice: orientation flips somewhere"
    assert torch.equal(fwd.sort().values, rev.sort().values), "an edge without its reverse: the surface has a hole"
    assert v.shape[0] - fwd.numel() // 2 + t.shape[0] == euler
    h = 2.0 / (n - 1)
    assert f(v[:, 0], v[:, 1], v[:, 2]).abs().max() < 3 * h * h                # linear interpolation of a smooth field
    assert abs(geo.mesh_area(v, t) / area - 1) < 0.02 and abs(geo.mesh_volume(v, t) / vol - 1) < 0.03
    # bounds move and scale the mesh; the level moves the surface
    v2, t2 = geo.isosurface(grid, 0.0, bounds=(0, 0, 0, 4, 4, 4))
    assert torch.equal(t2, t) and torch.allclose(v2, (v + 1) * 2, atol=1e-5)
    if shape == "sphere":
        v3, t3 = geo.isosurface(grid, 0.1)
        assert abs(geo.mesh_volume(v3, t3) / (4 / 3 * math.pi * 0.72 ** 3) - 1) < 0.03
        assert geo.isosurface(grid, 5.0)[1].shape[0] == 0
        geo.write_mesh_ply(str(tmp_path / "m.ply"), v, t)
        bv, names, bf = geo.read_ply(str(tmp_path / "m.ply"))
        assert names == ["x", "y", "z"] and torch.equal(bv, v) and torch.equal(bf, t)
        geo.write_mesh_obj(str(tmp_path / "m.obj"), v, t)
        lines = open(tmp_path / "m.obj").read().splitlines()
        assert sum(l.startswith("v ") for l in lines) == v.shape[0] and sum(l.startswith("f ") for l in lines) == t.shape[0]


@needs_ref
def test_isosurface_against_the_reference_marching_cubes():
    """Different triangulations of the same level set: area, volume and the distance of every vertex to the other mesh agree."""
    lib = oracle.geometry_lib()
    n = 36
    grid = _grid(n, lambda x, y, z: (x * x + 1.5 * y * y + 0.7 * z * z).sqrt() - 0.6 + 0.08 * torch.sin(5 * x) * torch.cos(4 * z)).contiguous()
    vp, tp, nv, nt = ctypes.POINTER(ctypes.c_float)(), ctypes.POINTER(ctypes.c_int)(), ctypes.c_int(), ctypes.c_int()
    lib.ref_mc(grid.data_ptr(), n, n, n, 0.0, None, ctypes.byref(vp), ctypes.byref(tp), ctypes.byref(nv), ctypes.byref(nt))
    rv = torch.from_numpy(np.ctypeslib.as_array(vp, shape=(nv.value, 3)).copy())
    rt = torch.from_numpy(np.ctypeslib.as_array(tp, shape=(nt.value, 3)).copy())
    v, t = geo.isosurface(grid, 0.0)
    assert abs(geo.mesh_area(v, t) / geo.mesh_area(rv, rt) - 1) < 0.01
    assert abs(abs(geo.mesh_volume(v, t)) / abs(geo.mesh_volume(rv, rt)) - 1) < 0.01
    h = 2.0 / (n - 1)
    d_ours = geo.Bvh(rv, rt).closest(v)[0]
    d_ref = geo.Bvh(v, t).closest(rv)[0]
    assert d_ours.max() < 0.5 * h and d_ref.max() < 0.5 * h


def _brute_trace(verts, tris, o, d):
    a, b, c = (verts[tris[:, i].long()].double() for i in range(3))
    o, d = o.double()[:, None], d.double()[:, None]
    e1, e2 = (b - a)[None], (c - a)[None]
    p = torch.linalg.cross(d.expand(-1, e2.shape[1], -1), e2.expand(d.shape[0], -1, -1))
    det = (e1 * p).sum(-1)
    s = o - a[None]
    u = (s * p).sum(-1) / det
    q = torch.linalg.cross(s, e1.expand(s.shape[0], -1, -1))
    vv = (d * q).sum(-1) / det
    tt = (e2 * q).sum(-1) / det
    ok = (det.abs() > 1e-20) & (u >= 0) & (u <= 1) & (vv >= 0) & (u + vv <= 1) & (tt > 1e-6)
    tt = torch.where(ok, tt, torch.full_like(tt, float("inf")))
    best = tt.min(dim=1)
    return best.values.float(), torch.where(torch.isinf(best.values), torch.full_like(best.indices, -1), best.indices)


def _brute_closest(verts, tris, pts):
    """Distance of points to triangles: to the plane where the foot lies inside, else to the nearest of the three edges."""
    a, b, c = (verts[tris[:, i].long()].double()[None] for i in range(3))
    p = pts.double()[:, None]
    n = torch.linalg.cross(b - a, c - a)
    n = n / n.norm(dim=-1, keepdim=True)
    dist_plane = ((p - a) * n).sum(-1)
    foot = p - dist_plane[..., None] * n
    inside = torch.ones_like(dist_plane, dtype=torch.bool)
    for x, y in ((a, b), (b, c), (c, a)):
        inside &= (torch.linalg.cross((y - x).expand_as(foot), foot - x) * n).sum(-1) >= 0
    best = torch.where(inside, dist_plane.abs(), torch.full_like(dist_plane, float("inf")))
    for x, y in ((a, b), (b, c), (c, a)):
        e = y - x
        s = (((p - x) * e).sum(-1) / (e * e).sum(-1)).clamp(0, 1)
        best = torch.minimum(best, (p - (x + s[..., None] * e)).norm(dim=-1))
    return best.min(dim=1).values.float()


def test_bvh_queries_against_brute_force():
    grid = _grid(25, lambda x, y, z: (((x * x + z * z).sqrt() - 0.55) ** 2 + y * y).sqrt() - 0.25)
    v, t = geo.isosurface(grid, 0.0)
    for leaf in (1, 4, 64):
        bvh = geo.Bvh(v, t, leaf=leaf)
        assert 1 <= bvh.n_nodes <= 2 * t.shape[0]
        g = torch.Generator().manual_seed(leaf)
        o = torch.randn(300, 3, generator=g) * 1.5
        phi = torch.rand(300, generator=g) * 2 * math.pi
        ring = torch.stack([0.55 * phi.cos(), torch.zeros(300), 0.55 * phi.sin()], 1)               # points inside the tube
        d = torch.nn.functional.normalize(ring - o + 0.25 * torch.randn(300, 3, generator=g), dim=1)
        tt, tri, uv = bvh.trace(o, d)
        bt, btri = _brute_trace(v, t, o, d)
        hit = tri >= 0
        assert 0.2 < hit.float().mean() < 1.0 and torch.equal(hit, btri >= 0)
        assert torch.allclose(tt[hit], bt[hit], rtol=1e-4, atol=1e-5)
        # the barycentric coordinates give the hit point
        c0, c1, c2 = (v[t[tri[hit].long(), i].long()] for i in range(3))
        point = (1 - uv[hit].sum(1, keepdim=True)) * c0 + uv[hit][:, :1] * c1 + uv[hit][:, 1:] * c2
        assert torch.allclose(point, o[hit] + tt[hit][:, None] * d[hit], atol=1e-4)
        # an occlusion query agrees on WHETHER something is hit, and range limits are honoured
        assert torch.equal(bvh.trace(o, d, any_hit=True)[1] >= 0, hit)
        assert not (bvh.trace(o, d, tmax=1e-3)[1] >= 0).any()
        q = torch.randn(200, 3, generator=g)
        dist, ctri, pt, w = bvh.closest(q)
        assert torch.allclose(dist, _brute_closest(v, t, q), atol=2e-5, rtol=1e-4)
        c0, c1, c2 = (v[t[ctri.long(), i].long()] for i in range(3))
        assert torch.allclose(w[:, :1] * c0 + w[:, 1:2] * c1 + w[:, 2:] * c2, pt, atol=1e-5) and torch.allclose(w.sum(1), torch.ones(200), atol=1e-5)
        assert torch.allclose((pt - q).norm(dim=1), dist, atol=1e-5) and (w >= -1e-6).all()
    with pytest.raises(ValueError):
        geo.Bvh(v, torch.tensor([[0, 1, v.shape[0]]]))
    empty = geo.Bvh(v, torch.zeros(0, 3, dtype=torch.int32))
    assert empty.trace(torch.zeros(1, 3), torch.tensor([[0.0, 0, 1]]))[1].item() == -1 and empty.closest(torch.zeros(1, 3))[1].item() == -1


def test_preview_render_of_a_sphere_over_a_floor(tmp_path):
    grid = _grid(33, lambda x, y, z: (x * x + y * y + z * z).sqrt() - 0.5)
    v, t = geo.isosurface(grid, 0.0)
    floor_v = torch.tensor([[-3, -0.5, -3], [3, -0.5, -3], [3, -0.5, 3], [-3, -0.5, 3]], dtype=torch.float32)
    floor_t = torch.tensor([[0, 2, 1], [0, 3, 2]], dtype=torch.int32) + v.shape[0]
    bvh = geo.Bvh(torch.cat([v, floor_v]), torch.cat([t, floor_t]))
    w = h = 96
    img = bvh.render(eye=(0, 0.6, -3.0), target=(0, -0.1, 0), width=w, height=h, fov_deg=40, sun_dir=(0.5, 1.0, -0.3))
    assert img["rgb"].shape == (h, w, 3) and torch.isfinite(img["rgb"]).all()
    mask, depth, normal = img["mask"], img["depth"], img["normal"]
    assert mask[0, 0] == 0 and depth[0, 0] == 0 and mask[h // 2, w // 2] == 1               # sky in the corner, the sphere in the middle
    centre = normal[h // 2, w // 2]
    assert centre[2] < -0.8 and abs(normal[h // 2, w // 2].norm() - 1) < 1e-4                # facing the camera
    assert abs(float(depth[h // 2, w // 2]) - (math.sqrt(0.36 + 9.0) - 0.5)) < 0.08
    sky = img["rgb"][0, 0]
    assert sky[2] > sky[0]                                                                    # blue above the horizon
    # the floor: lit far from the sphere, in shadow on the side away from the sun
    rows = normal[..., 1] > 0.99
    lit_floor = img["rgb"][rows & (img["rgb"].sum(-1) > 2.0)]
    dark_floor = img["rgb"][rows & (img["rgb"].sum(-1) < 1.0)]
    assert lit_floor.shape[0] > 50 and dark_floor.shape[0] > 20
    geo.write_ppm(str(tmp_path / "preview.ppm"), img["rgb"])
    raw = open(tmp_path / "preview.ppm", "rb").read()
    assert raw.startswith(b"P6\n96 96\n255\n") and len(raw) == 13 + 96 * 96 * 3


def test_mesh_command(tmp_path, capsys):
    import json
    from gemm_b200.__main__ import main
    np.save(tmp_path / "sdf.npy", _grid(24, lambda x, y, z: (x * x + y * y + z * z).sqrt() - 0.7).numpy())
    assert main(["mesh", "--grid", str(tmp_path / "sdf.npy"), "--out", str(tmp_path / "m.ply"), "--render", str(tmp_path / "p.ppm"), "--size", "48"]) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["triangles"] > 500 and abs(line["volume"] / (4 / 3 * math.pi * 0.343) - 1) < 0.05 and 0.05 < line["coverage"] < 0.9
    v, _, f = geo.read_ply(str(tmp_path / "m.ply"))
    assert v.shape[0] == line["vertices"] and f.shape[0] == line["triangles"]
    assert open(tmp_path / "p.ppm", "rb").read(2) == b"P6"


@needs_ref
def test_dual_grid_mesh_equals_the_reference():
    """A sparse shell of voxels around a sphere with random offsets, crossing flags and split weights: vertices and triangles equal
    the reference's, in its order."""
    lib = oracle.geometry_lib()
    g = torch.Generator().manual_seed(4)
    zz, yy, xx = torch.meshgrid(torch.arange(20), torch.arange(20), torch.arange(20), indexing="ij")
    r = ((zz - 9.5) ** 2 + (yy - 9.5) ** 2 + (xx - 9.5) ** 2).float().sqrt()
    shell = (r > 5.5) & (r < 8.0)
    coords = torch.stack([zz[shell], yy[shell], xx[shell]], 1).to(torch.int32)
    coords = coords[torch.randperm(coords.shape[0], generator=g)].contiguous()                  # no order assumed
    n = coords.shape[0]
    feats = torch.cat([torch.rand(n, 3, generator=g), torch.randn(n, 3, generator=g), torch.rand(n, 1, generator=g)], 1).contiguous()
    aabb = torch.tensor([-0.5, -0.4, -0.3, 0.5, 0.6, 0.7])
    vp, tp, nt = ctypes.POINTER(ctypes.c_float)(), ctypes.POINTER(ctypes.c_int)(), ctypes.c_int()
    nv = lib.ref_fdg(coords.data_ptr(), feats.data_ptr(), n, 0.05, aabb.data_ptr(), ctypes.byref(vp), ctypes.byref(tp), ctypes.byref(nt))
    rv = torch.from_numpy(np.ctypeslib.as_array(vp, shape=(nv, 3)).copy())
    rt = torch.from_numpy(np.ctypeslib.as_array(tp, shape=(nt.value, 3)).copy())
    v, t = geo.dual_grid_mesh(coords, feats, 0.05, aabb.tolist())
    assert nt.value > 1000 and torch.allclose(v, rv, atol=1e-6) and torch.equal(t, rt)
    ev, et = geo.dual_grid_mesh(coords[:0], feats[:0], 0.05, aabb.tolist())
    assert ev.shape == (0, 3) and et.shape == (0, 3)


def test_specular_lobe_adds_a_highlight_where_the_sun_reflects():
    grid = _grid(41, lambda x, y, z: (x * x + y * y + z * z).sqrt() - 0.6)
    v, t = geo.isosurface(grid, 0.0)
    bvh = geo.Bvh(v, t)
    kw = dict(eye=(0, 0, -3.0), target=(0, 0, 0), width=96, height=96, fov_deg=30, sun_dir=(0.0, 0.5, -1.0), albedo=(0.5, 0.5, 0.5))
    matte = bvh.render(**kw)["rgb"]
    shiny = bvh.render(roughness=0.25, **kw)["rgb"]
    diff = (shiny - matte).sum(-1)
    assert diff.min() > -1e-5 and diff.max() > 0.3                       # only adds light
    y, x = divmod(int(diff.argmax()), 96)
    # the highlight sits where the normal halves the directions to the sun and to the eye: above the centre, on the sphere
    assert y < 48 and abs(x - 48) < 6 and bvh.render(**kw)["mask"][y, x] == 1
    rough = bvh.render(roughness=0.8, **kw)["rgb"]
    assert (rough - matte).sum(-1).max() < diff.max()                    # a rougher surface spreads the lobe
