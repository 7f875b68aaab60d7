"""Geometry post-processing around 3-D generative models: what comes after the network.

* ``gs_rows`` / ``write_gs_ply`` / ``read_ply``: Gaussian-splat activations -> the 17 floats per splat of the INRIA PLY layout and
  the binary file (the reference: common/gs_ply_writer.h);
* ``isosurface``: triangle mesh of a level set of a scalar grid, welded (the reference: common/marching_cubes.h; here by
  tetrahedra, see csrc/kernels/geometry.cuh), ``write_mesh_ply`` / ``write_mesh_obj``, ``mesh_volume`` / ``mesh_area``;
* ``dual_grid_mesh``: mesh of a sparse "flexible dual grid" prediction (the reference: common/trellis2_fdg_mesh.h);
* ``Bvh``: bounding-volume hierarchy over a triangle mesh with ``trace`` (closest or any hit of rays), ``closest`` (closest point
  and barycentric weights, the reference: common/closest_point_bvh.h) and ``render`` (preview image with depth / normal / mask,
  the reference: common/preview_render.h), ``write_ppm``.

Tensors on a CUDA device go through the kernels of ``csrc/kernels/geometry.cu``; CPU tensors through the host library, which runs
the same inline code in loops.  The hierarchy is always built on the host.
"""
from __future__ import annotations

import ctypes
import math
import struct
from typing import Optional, Sequence, Tuple

import torch

from .. import _native

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float
GS_FIELDS = ("x", "y", "z", "nx", "ny", "nz", "f_dc_0", "f_dc_1", "f_dc_2", "opacity", "scale_0", "scale_1", "scale_2", "rot_0", "rot_1", "rot_2", "rot_3")


def _p(t: torch.Tensor):
    return _P(t.data_ptr())


def _f3(v: Sequence[float]):
    return (ctypes.c_float * len(v))(*[float(x) for x in v])


def _stream():
    return _P(torch.cuda.current_stream().cuda_stream)


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(torch.float32).contiguous()


# ------------------------------------------------------------------------------------------------------ splats
def gs_rows(xyz: torch.Tensor, f_dc: torch.Tensor, opacity: torch.Tensor, scale: torch.Tensor, rotation: torch.Tensor, opacity_bias: float = 0.0,
            scaling_bias: float = 1.0) -> torch.Tensor:
    """Rows ``[n, 17]`` in the order of ``GS_FIELDS`` from raw network outputs: ``opacity + opacity_bias`` stays a logit, the scale is
    stored as ``log(softplus(raw + softplus^-1(scaling_bias)))``, the rotation un-normalised, normals zero."""
    n = xyz.shape[0]
    xyz, f_dc, opacity, scale, rotation = _f32(xyz).reshape(n, 3), _f32(f_dc).reshape(n, 3), _f32(opacity).reshape(n), _f32(scale).reshape(n, 3), _f32(rotation).reshape(n, 4)
    rows = torch.empty(n, 17, dtype=torch.float32, device=xyz.device)
    if xyz.is_cuda:
        rc = _native.cuda().gb_geo_gs_rows(_L(n), _p(xyz), _p(f_dc), _p(opacity), _p(scale), _p(rotation), _F(opacity_bias), _F(scaling_bias), _p(rows), _stream())
        _native.check(rc, "gb_geo_gs_rows")
    else:
        _native.host().gbh_geo_gs_rows(_L(n), _p(xyz), _p(f_dc), _p(opacity), _p(scale), _p(rotation), _F(opacity_bias), _F(scaling_bias), _p(rows))
    return rows


def write_gs_ply(path: str, rows: torch.Tensor) -> None:
    """Binary little-endian PLY of splat rows ``[n, 17]``."""
    rows = _f32(rows).cpu()
    if rows.dim() != 2 or rows.shape[1] != 17:
        raise ValueError("splat rows are [n, 17]")
    head = "ply\nformat binary_little_endian 1.0\nelement vertex %d\n" % rows.shape[0] + "".join(f"property float {f}\n" for f in GS_FIELDS) + "end_header\n"
    with open(path, "wb") as fh:
        fh.write(head.encode())
        fh.write(rows.numpy().astype("<f4").tobytes())


def read_ply(path: str):
    """Minimal reader of the binary little-endian PLY files written here: ``(vertex properties [n, k] f32, names, faces [m, 3] or None)``."""
    with open(path, "rb") as fh:
        raw = fh.read()
    end = raw.index(b"end_header\n") + len(b"end_header\n")
    names, n_vert, n_face, elem = [], 0, 0, ""
    for line in raw[:end].decode().splitlines():
        tok = line.split()
        if tok[:1] == ["element"]:
            elem = tok[1]
            if elem == "vertex":
                n_vert = int(tok[2])
            elif elem == "face":
                n_face = int(tok[2])
        elif tok[:1] == ["property"] and elem == "vertex":
            if tok[1] != "float":
                raise ValueError("only float vertex properties are read")
            names.append(tok[2])
    k = len(names)
    verts = torch.frombuffer(bytearray(raw[end: end + 4 * k * n_vert]), dtype=torch.float32).reshape(n_vert, k).clone()
    faces, pos = None, end + 4 * k * n_vert
    if n_face:
        out = []
        for _ in range(n_face):
            cnt = raw[pos]
            out.append(struct.unpack_from("<%di" % cnt, raw, pos + 1)[:3])
            pos += 1 + 4 * cnt
        faces = torch.tensor(out, dtype=torch.int32)
    return verts, names, faces


# ------------------------------------------------------------------------------------------------------ iso-surface
def isosurface(grid: torch.Tensor, iso: float = 0.0, bounds: Optional[Sequence[float]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Level set ``grid == iso`` of a grid ``[nx, ny, nz]`` (values below ``iso`` are inside) spanning ``bounds`` = (xmin, ymin, zmin,
    xmax, ymax, zmax), default the cube [-1, 1]^3.  Returns ``(vertices f32 [n, 3], triangles i32 [m, 3])``; triangles face outward,
    vertices on the same grid edge are one vertex, triangles without area are dropped."""
    g = _f32(grid)
    nx, ny, nz = g.shape
    if min(nx, ny, nz) < 2:
        raise ValueError("the grid needs at least 2 samples per axis")
    if (nx * ny * nz) ** 2 >= 2 ** 63:
        raise ValueError("grid too large for 64-bit edge keys")
    b = [float(v) for v in (bounds if bounds is not None else (-1, -1, -1, 1, 1, 1))]
    org, step = _f3(b[:3]), _f3([(b[3 + a] - b[a]) / (n - 1) for a, n in enumerate((nx, ny, nz))])
    cells = (nx - 1) * (ny - 1) * (nz - 1)
    counts = torch.empty(cells, dtype=torch.int32, device=g.device)
    if g.is_cuda:
        _native.check(_native.cuda().gb_geo_iso_count(_p(g), _I(nx), _I(ny), _I(nz), org, step, _F(iso), _p(counts), _stream()), "gb_geo_iso_count")
    else:
        _native.host().gbh_geo_iso_count(_p(g), _I(nx), _I(ny), _I(nz), org, step, _F(iso), _p(counts))
    ends = torch.cumsum(counts.to(torch.int64), 0)
    total = int(ends[-1]) if cells else 0
    if total == 0:
        return torch.zeros(0, 3, device=g.device), torch.zeros(0, 3, dtype=torch.int32, device=g.device)
    offsets = (ends - counts).contiguous()
    pos = torch.empty(total, 3, 3, dtype=torch.float32, device=g.device)
    key = torch.empty(total, 3, dtype=torch.int64, device=g.device)
    if g.is_cuda:
        _native.check(_native.cuda().gb_geo_iso_emit(_p(g), _I(nx), _I(ny), _I(nz), org, step, _F(iso), _p(offsets), _p(counts), _p(pos), _p(key), _stream()),
                      "gb_geo_iso_emit")
    else:
        _native.host().gbh_geo_iso_emit(_p(g), _I(nx), _I(ny), _I(nz), org, step, _F(iso), _p(offsets), _p(counts), _p(pos), _p(key))
    uniq, inv = torch.unique(key.reshape(-1), return_inverse=True)
    verts = torch.empty(uniq.numel(), 3, dtype=torch.float32, device=g.device)
    verts[inv] = pos.reshape(-1, 3)                              # equal keys carry equal positions: any writer wins
    tris = inv.reshape(-1, 3)
    keep = (tris[:, 0] != tris[:, 1]) & (tris[:, 1] != tris[:, 2]) & (tris[:, 0] != tris[:, 2])
    return verts, tris[keep].to(torch.int32).contiguous()


def mesh_area(verts: torch.Tensor, tris: torch.Tensor) -> float:
    a, b, c = (verts[tris[:, i].long()].double() for i in range(3))
    return float(torch.linalg.cross(b - a, c - a).norm(dim=1).sum() * 0.5)


def mesh_volume(verts: torch.Tensor, tris: torch.Tensor) -> float:
    """Signed volume enclosed by a closed mesh (positive when the triangles face outward)."""
    a, b, c = (verts[tris[:, i].long()].double() for i in range(3))
    return float((a * torch.linalg.cross(b, c)).sum() / 6.0)


def write_mesh_ply(path: str, verts: torch.Tensor, tris: torch.Tensor) -> None:
    v, t = _f32(verts).cpu(), tris.to(torch.int32).cpu()
    head = f"ply\nformat binary_little_endian 1.0\nelement vertex {v.shape[0]}\nproperty float x\nproperty float y\nproperty float z\n" \
           f"element face {t.shape[0]}\nproperty list uchar int vertex_indices\nend_header\n"
    import numpy as np
    rec = np.zeros(t.shape[0], dtype=[("n", "u1"), ("i", "<i4", 3)])
    rec["n"], rec["i"] = 3, t.numpy()
    with open(path, "wb") as fh:
        fh.write(head.encode())
        fh.write(v.numpy().astype("<f4").tobytes())
        fh.write(rec.tobytes())


def write_mesh_obj(path: str, verts: torch.Tensor, tris: torch.Tensor) -> None:
    with open(path, "w") as fh:
        for x, y, z in _f32(verts).cpu().tolist():
            fh.write(f"v {x:.7g} {y:.7g} {z:.7g}\n")
        for a, b, c in tris.cpu().tolist():
            fh.write(f"f {a + 1} {b + 1} {c + 1}\n")


# ------------------------------------------------------------------------------------------------------ BVH
class Bvh:
    """Hierarchy over a triangle mesh (``verts`` [n, 3] f32, ``tris`` [m, 3] int): median splits of the triangle centroids along the
    longest axis, leaves of at most ``leaf`` triangles, built on the host; the queries run where ``device`` says."""

    def __init__(self, verts: torch.Tensor, tris: torch.Tensor, leaf: int = 4, device=None):
        v, t = _f32(verts).cpu(), tris.detach().to(torch.int32).cpu().contiguous()
        m = t.shape[0]
        nodes = torch.zeros(max(2 * m, 1), 8, dtype=torch.float32)          # 32 bytes per node
        order = torch.zeros(max(m, 1), dtype=torch.int32)
        n = _native.host().gbh_geo_bvh_build(_p(v), _I(v.shape[0]), _p(t), _I(m), _I(leaf), _p(nodes), _p(order))
        if n < 0:
            raise ValueError(_native.host().gbh_last_error().decode(errors="replace"))
        self.n_nodes = n
        dev = torch.device(device) if device is not None else verts.device
        self.device = dev
        self.verts, self.tris, self.nodes, self.order = v.to(dev), t.to(dev), nodes[: max(n, 1)].contiguous().to(dev), order.to(dev)

    def _mesh(self):
        return _p(self.verts), _p(self.tris), _p(self.nodes), _p(self.order), _I(self.n_nodes)

    def trace(self, origins: torch.Tensor, dirs: torch.Tensor, tmin: float = 1e-6, tmax: float = 1e30, any_hit: bool = False):
        """Rays ``origins + t * dirs``: ``(t f32 [n] (inf on a miss), triangle i32 [n] (-1 on a miss), uv f32 [n, 2])``; the hit point is
        ``(1 - u - v) v0 + u v1 + v v2``.  ``any_hit`` returns the first hit found (occlusion tests)."""
        o, d = _f32(origins).to(self.device).reshape(-1, 3), _f32(dirs).to(self.device).reshape(-1, 3)
        n = o.shape[0]
        t = torch.empty(n, dtype=torch.float32, device=self.device)
        tri = torch.empty(n, dtype=torch.int32, device=self.device)
        uv = torch.empty(n, 2, dtype=torch.float32, device=self.device)
        if self.device.type == "cuda":
            _native.check(_native.cuda().gb_geo_trace(*self._mesh(), _L(n), _p(o), _p(d), _F(tmin), _F(tmax), _I(int(any_hit)), _p(t), _p(tri), _p(uv), _stream()),
                          "gb_geo_trace")
        else:
            _native.host().gbh_geo_trace(*self._mesh(), _L(n), _p(o), _p(d), _F(tmin), _F(tmax), _I(int(any_hit)), _p(t), _p(tri), _p(uv))
        return t, tri, uv

    def closest(self, points: torch.Tensor):
        """Closest point of the mesh to each query: ``(distance [n], triangle [n], point [n, 3], barycentric weights [n, 3])``."""
        q = _f32(points).to(self.device).reshape(-1, 3)
        n = q.shape[0]
        dist = torch.empty(n, dtype=torch.float32, device=self.device)
        tri = torch.empty(n, dtype=torch.int32, device=self.device)
        pt = torch.zeros(n, 3, dtype=torch.float32, device=self.device)
        w = torch.zeros(n, 3, dtype=torch.float32, device=self.device)
        if self.device.type == "cuda":
            _native.check(_native.cuda().gb_geo_closest(*self._mesh(), _L(n), _p(q), _p(dist), _p(tri), _p(pt), _p(w), _stream()), "gb_geo_closest")
        else:
            _native.host().gbh_geo_closest(*self._mesh(), _L(n), _p(q), _p(dist), _p(tri), _p(pt), _p(w))
        return dist, tri, pt, w

    def render(self, eye: Sequence[float], target: Sequence[float], width: int = 256, height: int = 256, fov_deg: float = 40.0,
               up: Sequence[float] = (0.0, 1.0, 0.0), sun_dir: Sequence[float] = (0.3, 0.6, 0.4), albedo: Sequence[float] = (0.8, 0.8, 0.8),
               roughness: float = 0.0, f0: float = 0.04,
               sun_rgb: Sequence[float] = (3.0, 2.9, 2.6), zenith_rgb: Sequence[float] = (0.18, 0.32, 0.62),
               horizon_rgb: Sequence[float] = (0.85, 0.78, 0.70)):
        """Preview image from a pinhole camera: Lambert (and, with ``roughness`` > 0, a GGX lobe of normal reflectance ``f0``) under
        a sun with hard shadows plus half of the sky colour in the direction of the normal as ambient light; a miss shows the sky.  Returns ``dict(rgb [h, w, 3] linear, depth [h, w], normal [h, w, 3], mask [h, w])``."""
        e, tg, u = (torch.tensor([float(x) for x in v], dtype=torch.float64) for v in (eye, target, up))
        fwd = (tg - e) / (tg - e).norm()
        right = torch.linalg.cross(fwd, u)
        right = right / right.norm()
        upv = torch.linalg.cross(right, fwd)
        sun = torch.tensor([float(x) for x in sun_dir], dtype=torch.float64)
        sun = sun / sun.norm()
        cam = _f3(list(e) + list(fwd) + list(right) + list(upv) + [math.tan(math.radians(fov_deg) / 2)])
        light = _f3(list(sun) + list(sun_rgb) + list(zenith_rgb) + list(horizon_rgb))
        alb = _f3(list(albedo) + [roughness, f0])
        dev = self.device
        rgb = torch.empty(height, width, 3, dtype=torch.float32, device=dev)
        depth = torch.empty(height, width, dtype=torch.float32, device=dev)
        normal = torch.empty(height, width, 3, dtype=torch.float32, device=dev)
        mask = torch.empty(height, width, dtype=torch.float32, device=dev)
        if dev.type == "cuda":
            _native.check(_native.cuda().gb_geo_render(*self._mesh(), cam, _I(width), _I(height), light, alb, _p(rgb), _p(depth), _p(normal), _p(mask), _stream()),
                          "gb_geo_render")
        else:
            _native.host().gbh_geo_render(*self._mesh(), cam, _I(width), _I(height), light, alb, _p(rgb), _p(depth), _p(normal), _p(mask))
        return {"rgb": rgb, "depth": depth, "normal": normal, "mask": mask}


def write_ppm(path: str, rgb: torch.Tensor, gamma: float = 2.2) -> None:
    """Linear ``[h, w, 3]`` -> 8-bit binary PPM."""
    img = (rgb.detach().float().cpu().clamp(0, 1) ** (1.0 / gamma) * 255.0 + 0.5).to(torch.uint8)
    with open(path, "wb") as fh:
        fh.write(b"P6\n%d %d\n255\n" % (img.shape[1], img.shape[0]))
        fh.write(img.numpy().tobytes())


# ------------------------------------------------------------------------------------------------------ dual grid
_EDGE_NEIGHBOURS = (((0, 0, 0), (0, 0, 1), (0, 1, 1), (0, 1, 0)),      # the four voxels (z, y, x offsets) around a voxel's x edge,
                    ((0, 0, 0), (1, 0, 0), (1, 0, 1), (0, 0, 1)),      # its y edge,
                    ((0, 0, 0), (0, 1, 0), (1, 1, 0), (1, 0, 0)))      # its z edge


def dual_grid_mesh(coords: torch.Tensor, feats: torch.Tensor, voxel_size: float, aabb: Sequence[float]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Mesh of a sparse "flexible dual grid" prediction (common/trellis2_fdg_mesh.h:139-222): ``coords`` int [N, 3] voxel indices
    (z, y, x), ``feats`` [N, 7] = vertex offset inside the voxel (x, y, z in 0..1), one crossing flag per axis (> 0: the voxel's edge
    along that axis crosses the surface), a split weight.  Every voxel contributes one vertex; every crossed edge whose four
    surrounding voxels all exist contributes a quad over their vertices, cut along the diagonal whose two split weights have the
    larger product.  Returns ``(vertices f32 [N, 3], triangles i32 [M, 3])`` in the reference's order (voxel by voxel, axis by axis).
    Sorting and binary search take the place of the reference's hash table, so the same code runs on a GPU."""
    c = coords.to(torch.int64)
    f = feats.to(torch.float32)
    n, dev = c.shape[0], c.device
    lo = torch.tensor([float(v) for v in aabb[:3]], dtype=torch.float32, device=dev)
    verts = (c[:, [2, 1, 0]].float() + f[:, :3]) * voxel_size + lo
    if n == 0:
        return verts, torch.zeros(0, 3, dtype=torch.int32, device=dev)
    key = lambda z, y, x: (z << 40) | ((y & 0xFFFFF) << 20) | (x & 0xFFFFF)
    keys, order = torch.sort(key(c[:, 0], c[:, 1], c[:, 2]))
    tris, tags = [], []
    for axis in range(3):
        rows = (f[:, 3 + axis] > 0).nonzero(as_tuple=True)[0]
        quad, ok = [], torch.ones(rows.numel(), dtype=torch.bool, device=dev)
        for dz, dy, dx in _EDGE_NEIGHBOURS[axis]:
            want = key(c[rows, 0] + dz, c[rows, 1] + dy, c[rows, 2] + dx)
            at = torch.searchsorted(keys, want).clamp_max(n - 1)
            ok &= keys[at] == want
            quad.append(order[at])
        q = torch.stack(quad, 1)[ok]
        rows = rows[ok]
        w = f[:, 6]
        first = (w[q[:, 0]] * w[q[:, 2]] > w[q[:, 1]] * w[q[:, 3]])[:, None]
        a = torch.where(first, q[:, [0, 1, 2]], q[:, [0, 1, 3]])
        b = torch.where(first, q[:, [0, 2, 3]], q[:, [3, 1, 2]])
        tris.append(torch.stack([a, b], 1).reshape(-1, 3))
        tags.append((rows * 3 + axis).repeat_interleave(2) * 2 + torch.arange(2, device=dev).repeat(rows.numel()))
    tris, tags = torch.cat(tris), torch.cat(tags)
    return verts, tris[torch.argsort(tags)].to(torch.int32).contiguous()
