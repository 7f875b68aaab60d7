// Geometry post-processing shared by the CUDA kernels (geometry.cu) and the host library (host/geometry_host.cc): every function
// here compiles for both, so the CPU path is the device code run in a loop and serves as its oracle.
//
//  * Gaussian-splat activations -> the 17 floats per splat of the INRIA PLY layout (the storage rules the reference's writer
//    documents, common/gs_ply_writer.h:1-22: opacity as a logit, scale as a logarithm, rotation un-normalised);
//  * iso-surface extraction from a scalar grid.  The reference extracts with table-driven marching cubes
//    (common/marching_cubes.h); here every cell is cut into the six tetrahedra of the Kuhn triangulation (one per order of the
//    axes, all sharing the cell's main diagonal), which needs no case tables, has no ambiguous cases and gives a closed surface
//    because neighbouring cells cut their shared face along the same diagonal.  Two passes: count the triangles of a cell, then
//    emit them at the cell's offset; a vertex is identified by the grid edge it lies on, so equal keys weld;
//  * rays and points against a triangle mesh through a bounding-volume hierarchy (the reference: common/lightrt.hh SBVH,
//    common/closest_point_bvh.h, common/preview_render.h): closest hit, any hit (shadows), closest point, and the preview
//    shading of a pixel (Lambert + a GGX lobe under a sun with hard shadows, plus a sky gradient; depth, normal and mask as side outputs).
#pragma once
#include <math.h>
#include <stdint.h>

#ifdef __CUDACC__
#define GB_HD __host__ __device__ __forceinline__
#else
#define GB_HD inline
#endif

namespace gbgeo {

// ------------------------------------------------------------------------------------------------------ splat rows
GB_HD float softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
GB_HD float inv_softplus(float y) { return y > 20.0f ? y : logf(expm1f(y)); }

// One splat: position, SH DC colour, raw opacity, raw scale [3], rotation [4] -> row[17] = x y z nx ny nz f_dc[3] opacity scale[3] rot[4].
// opacity_stored = raw + opacity_bias; scale_stored = log(softplus(raw + inv_softplus(scaling_bias))).
GB_HD void gs_row(const float* xyz, const float* f_dc, float raw_opacity, const float* raw_scale, const float* rot, float opacity_bias,
                  float scaling_bias, float* row) {
  row[0] = xyz[0]; row[1] = xyz[1]; row[2] = xyz[2];
  row[3] = 0.0f; row[4] = 0.0f; row[5] = 0.0f;
  row[6] = f_dc[0]; row[7] = f_dc[1]; row[8] = f_dc[2];
  row[9] = raw_opacity + opacity_bias;
  const float shift = inv_softplus(scaling_bias);
  for (int i = 0; i < 3; ++i) row[10 + i] = logf(softplus(raw_scale[i] + shift));
  for (int i = 0; i < 4; ++i) row[13 + i] = rot[i];
}

// ------------------------------------------------------------------------------------------------------ iso-surface
struct Grid {
  const float* v;       // [nx][ny][nz], z fastest
  int nx, ny, nz;
  float org[3], step[3];  // position of sample (i, j, k) = org + (i, j, k) * step
};

GB_HD long long grid_index(const Grid& g, int i, int j, int k) { return ((long long)i * g.ny + j) * g.nz + k; }

// Triangles of cell (i, j, k) for the level `iso` (inside: value < iso).  pos == nullptr: count only.  Otherwise writes, per
// triangle, 9 floats to pos and 3 vertex keys to key (key = lo * n_samples + hi of the grid edge's two sample indices; the point is
// interpolated from lo to hi, so equal keys carry equal bits).  Triangles face from inside to outside.  Returns the count (<= 12).
GB_HD int cell_triangles(const Grid& g, int i, int j, int k, float iso, float* pos, long long* key) {
  const long long n_samples = (long long)g.nx * g.ny * g.nz;
  float val[8], px[8], py[8], pz[8];
  long long idx[8];
  bool any_in = false, any_out = false;
  for (int c = 0; c < 8; ++c) {                                 // corner c = bits (x, y, z)
    const int ci = i + (c & 1), cj = j + ((c >> 1) & 1), ck = k + ((c >> 2) & 1);
    idx[c] = grid_index(g, ci, cj, ck);
    val[c] = g.v[idx[c]];
    px[c] = g.org[0] + ci * g.step[0]; py[c] = g.org[1] + cj * g.step[1]; pz[c] = g.org[2] + ck * g.step[2];
    if (val[c] < iso) any_in = true; else any_out = true;
  }
  if (!(any_in && any_out)) return 0;
  // the six orders of the axes: corner 0 -> +a -> +b -> corner 7
  const int perm[6][3] = {{0, 1, 2}, {0, 2, 1}, {1, 0, 2}, {1, 2, 0}, {2, 0, 1}, {2, 1, 0}};
  int n_tri = 0;
  for (int t = 0; t < 6; ++t) {
    int tv[4];
    tv[0] = 0; tv[1] = 1 << perm[t][0]; tv[2] = tv[1] | (1 << perm[t][1]); tv[3] = 7;
    int in_v[4], out_v[4], n_in = 0, n_out = 0;
    for (int q = 0; q < 4; ++q) { if (val[tv[q]] < iso) in_v[n_in++] = tv[q]; else out_v[n_out++] = tv[q]; }
    if (n_in == 0 || n_in == 4) continue;
    // crossing points: one per (inside, outside) pair of the tetrahedron, in an order that walks around the cut polygon
    int ea[4], eb[4], n_e = 0;
    if (n_in == 1) { for (int q = 0; q < 3; ++q) { ea[n_e] = in_v[0]; eb[n_e++] = out_v[q]; } }
    else if (n_in == 3) { for (int q = 0; q < 3; ++q) { ea[n_e] = in_v[q]; eb[n_e++] = out_v[0]; } }
    else { ea[0] = in_v[0]; eb[0] = out_v[0]; ea[1] = in_v[0]; eb[1] = out_v[1]; ea[2] = in_v[1]; eb[2] = out_v[1]; ea[3] = in_v[1]; eb[3] = out_v[0]; n_e = 4; }
    const int tris = n_e - 2;
    if (pos == nullptr) { n_tri += tris; continue; }
    float qx[4], qy[4], qz[4], mx[4], my[4], mz[4];
    long long qk[4];
    for (int e = 0; e < n_e; ++e) {
      int lo = ea[e], hi = eb[e];
      if (idx[lo] > idx[hi]) { const int s = lo; lo = hi; hi = s; }
      const float d = val[hi] - val[lo];
      float w = d != 0.0f ? (iso - val[lo]) / d : 0.5f;
      w = w < 0.0f ? 0.0f : (w > 1.0f ? 1.0f : w);
      qx[e] = px[lo] + w * (px[hi] - px[lo]); qy[e] = py[lo] + w * (py[hi] - py[lo]); qz[e] = pz[lo] + w * (pz[hi] - pz[lo]);
      mx[e] = 0.5f * (px[lo] + px[hi]); my[e] = 0.5f * (py[lo] + py[hi]); mz[e] = 0.5f * (pz[lo] + pz[hi]);
      qk[e] = idx[lo] * n_samples + idx[hi];
    }
    // direction from the inside corners to the outside corners
    float dx = 0.f, dy = 0.f, dz = 0.f;
    for (int q = 0; q < n_out; ++q) { dx += px[out_v[q]] / n_out; dy += py[out_v[q]] / n_out; dz += pz[out_v[q]] / n_out; }
    for (int q = 0; q < n_in; ++q) { dx -= px[in_v[q]] / n_in; dy -= py[in_v[q]] / n_in; dz -= pz[in_v[q]] / n_in; }
    // which way round the polygon runs is a property of the edges it crosses, not of where it crosses them: decide it on the
    // edge midpoints, which never coincide (a sample exactly on the level puts several crossings on one point, and a normal
    // taken from those would be zero)
    const int l = n_e - 1;
    const float ux = mx[1] - mx[0], uy = my[1] - my[0], uz = mz[1] - mz[0];
    const float vx = mx[l] - mx[0], vy = my[l] - my[0], vz = mz[l] - mz[0];
    const float nxn = uy * vz - uz * vy, nyn = uz * vx - ux * vz, nzn = ux * vy - uy * vx;
    const bool flip = nxn * dx + nyn * dy + nzn * dz < 0.0f;
    for (int f = 0; f < tris; ++f) {
      const int a = 0, b = flip ? f + 2 : f + 1, c = flip ? f + 1 : f + 2;
      float* p = pos + (size_t)(n_tri + f) * 9;
      long long* kk = key + (size_t)(n_tri + f) * 3;
      p[0] = qx[a]; p[1] = qy[a]; p[2] = qz[a]; p[3] = qx[b]; p[4] = qy[b]; p[5] = qz[b]; p[6] = qx[c]; p[7] = qy[c]; p[8] = qz[c];
      kk[0] = qk[a]; kk[1] = qk[b]; kk[2] = qk[c];
    }
    n_tri += tris;
  }
  return n_tri;
}

// ------------------------------------------------------------------------------------------------------ BVH queries
struct Node {           // 32 bytes.  count > 0: a leaf over tri_order[first .. first + count); count == 0: children `first` and `first + 1`
  float bmin[3]; int first;
  float bmax[3]; int count;
};

struct Mesh {
  const float* verts;   // [n_verts][3]
  const int* tris;      // [n_tris][3]
  const Node* nodes;    // nodes[0] is the root
  const int* tri_order; // leaf ranges index this permutation of the triangles
  int n_nodes;
};

struct Hit { float t, u, v; int tri; };   // point = (1 - u - v) v0 + u v1 + v v2

GB_HD void tri_corners(const Mesh& m, int tri, const float*& a, const float*& b, const float*& c) {
  a = m.verts + 3 * (size_t)m.tris[3 * (size_t)tri]; b = m.verts + 3 * (size_t)m.tris[3 * (size_t)tri + 1]; c = m.verts + 3 * (size_t)m.tris[3 * (size_t)tri + 2];
}

// Moeller-Trumbore; accepts t in (tmin, tmax).
GB_HD bool ray_triangle(const float* o, const float* d, const float* a, const float* b, const float* c, float tmin, float tmax, float* t, float* u, float* v) {
  const float e1[3] = {b[0] - a[0], b[1] - a[1], b[2] - a[2]}, e2[3] = {c[0] - a[0], c[1] - a[1], c[2] - a[2]};
  const float p[3] = {d[1] * e2[2] - d[2] * e2[1], d[2] * e2[0] - d[0] * e2[2], d[0] * e2[1] - d[1] * e2[0]};
  const float det = e1[0] * p[0] + e1[1] * p[1] + e1[2] * p[2];
  if (fabsf(det) < 1e-20f) return false;
  const float inv = 1.0f / det;
  const float s[3] = {o[0] - a[0], o[1] - a[1], o[2] - a[2]};
  const float uu = (s[0] * p[0] + s[1] * p[1] + s[2] * p[2]) * inv;
  if (uu < 0.0f || uu > 1.0f) return false;
  const float q[3] = {s[1] * e1[2] - s[2] * e1[1], s[2] * e1[0] - s[0] * e1[2], s[0] * e1[1] - s[1] * e1[0]};
  const float vv = (d[0] * q[0] + d[1] * q[1] + d[2] * q[2]) * inv;
  if (vv < 0.0f || uu + vv > 1.0f) return false;
  const float tt = (e2[0] * q[0] + e2[1] * q[1] + e2[2] * q[2]) * inv;
  if (!(tt > tmin && tt < tmax)) return false;
  *t = tt; *u = uu; *v = vv;
  return true;
}

GB_HD bool ray_box(const Node& n, const float* o, const float* inv_d, float tmin, float tmax) {
  for (int a = 0; a < 3; ++a) {
    float t0 = (n.bmin[a] - o[a]) * inv_d[a], t1 = (n.bmax[a] - o[a]) * inv_d[a];
    if (t0 > t1) { const float s = t0; t0 = t1; t1 = s; }
    tmin = t0 > tmin ? t0 : tmin; tmax = t1 < tmax ? t1 : tmax;
    if (tmin > tmax) return false;
  }
  return true;
}

// Closest hit in (tmin, tmax); any_hit stops at the first one (shadow rays).  hit.tri < 0: none.
GB_HD Hit trace(const Mesh& m, const float* o, const float* d, float tmin, float tmax, bool any_hit) {
  Hit h; h.t = tmax; h.u = 0.f; h.v = 0.f; h.tri = -1;
  if (m.n_nodes <= 0) return h;
  float inv_d[3];
  for (int a = 0; a < 3; ++a) inv_d[a] = 1.0f / (fabsf(d[a]) > 1e-30f ? d[a] : (d[a] < 0.0f ? -1e-30f : 1e-30f));
  int stack[64], sp = 0;
  stack[sp++] = 0;
  while (sp > 0) {
    const Node& n = m.nodes[stack[--sp]];
    if (!ray_box(n, o, inv_d, tmin, h.t)) continue;
    if (n.count > 0) {
      for (int q = 0; q < n.count; ++q) {
        const int tri = m.tri_order[n.first + q];
        const float *a, *b, *c;
        tri_corners(m, tri, a, b, c);
        float t, u, v;
        if (ray_triangle(o, d, a, b, c, tmin, h.t, &t, &u, &v)) { h.t = t; h.u = u; h.v = v; h.tri = tri; if (any_hit) return h; }
      }
    } else if (sp + 2 <= 64) {
      stack[sp++] = n.first; stack[sp++] = n.first + 1;
    }
  }
  return h;
}

GB_HD float dot3(const float* a, const float* b) { return a[0] * b[0] + a[1] * b[1] + a[2] * b[2]; }

// Closest point of triangle (a, b, c) to p, by the regions of the triangle's plane (vertex, edge, face).  Writes the point and its
// barycentric weights; returns the squared distance.
GB_HD float closest_on_triangle(const float* p, const float* a, const float* b, const float* c, float* out, float* w) {
  const float ab[3] = {b[0] - a[0], b[1] - a[1], b[2] - a[2]}, ac[3] = {c[0] - a[0], c[1] - a[1], c[2] - a[2]};
  const float ap[3] = {p[0] - a[0], p[1] - a[1], p[2] - a[2]};
  const float d1 = dot3(ab, ap), d2 = dot3(ac, ap);
  float w0, w1, w2;
  const float bp[3] = {p[0] - b[0], p[1] - b[1], p[2] - b[2]};
  const float d3 = dot3(ab, bp), d4 = dot3(ac, bp);
  const float cp[3] = {p[0] - c[0], p[1] - c[1], p[2] - c[2]};
  const float d5 = dot3(ab, cp), d6 = dot3(ac, cp);
  const float vc = d1 * d4 - d3 * d2, vb = d5 * d2 - d1 * d6, va = d3 * d6 - d5 * d4;
  if (d1 <= 0.0f && d2 <= 0.0f) { w0 = 1.f; w1 = 0.f; w2 = 0.f; }
  else if (d3 >= 0.0f && d4 <= d3) { w0 = 0.f; w1 = 1.f; w2 = 0.f; }
  else if (vc <= 0.0f && d1 >= 0.0f && d3 <= 0.0f) { const float t = d1 / (d1 - d3); w0 = 1.f - t; w1 = t; w2 = 0.f; }
  else if (d6 >= 0.0f && d5 <= d6) { w0 = 0.f; w1 = 0.f; w2 = 1.f; }
  else if (vb <= 0.0f && d2 >= 0.0f && d6 <= 0.0f) { const float t = d2 / (d2 - d6); w0 = 1.f - t; w1 = 0.f; w2 = t; }
  else if (va <= 0.0f && (d4 - d3) >= 0.0f && (d5 - d6) >= 0.0f) { const float t = (d4 - d3) / ((d4 - d3) + (d5 - d6)); w0 = 0.f; w1 = 1.f - t; w2 = t; }
  else { const float den = 1.0f / (va + vb + vc); w1 = vb * den; w2 = vc * den; w0 = 1.0f - w1 - w2; }
  float dist = 0.f;
  for (int i = 0; i < 3; ++i) { out[i] = w0 * a[i] + w1 * b[i] + w2 * c[i]; const float e = out[i] - p[i]; dist += e * e; }
  w[0] = w0; w[1] = w1; w[2] = w2;
  return dist;
}

GB_HD float box_dist2(const Node& n, const float* p) {
  float s = 0.f;
  for (int a = 0; a < 3; ++a) { const float e = p[a] < n.bmin[a] ? n.bmin[a] - p[a] : (p[a] > n.bmax[a] ? p[a] - n.bmax[a] : 0.0f); s += e * e; }
  return s;
}

// Closest point of the mesh to p: triangle index (or -1 for an empty mesh), squared distance, point [3], weights [3].
GB_HD int closest_point(const Mesh& m, const float* p, float* dist2, float* point, float* w) {
  int best = -1;
  float bd = INFINITY;
  if (m.n_nodes <= 0) { *dist2 = bd; return best; }
  int stack[64], sp = 0;
  stack[sp++] = 0;
  while (sp > 0) {
    const Node& n = m.nodes[stack[--sp]];
    if (box_dist2(n, p) >= bd) continue;
    if (n.count > 0) {
      for (int q = 0; q < n.count; ++q) {
        const int tri = m.tri_order[n.first + q];
        const float *a, *b, *c;
        tri_corners(m, tri, a, b, c);
        float cp[3], cw[3];
        const float d = closest_on_triangle(p, a, b, c, cp, cw);
        if (d < bd) { bd = d; best = tri; for (int i = 0; i < 3; ++i) { point[i] = cp[i]; w[i] = cw[i]; } }
      }
    } else if (sp + 2 <= 64) {                                  // nearer child last, so that it is popped first
      const float dl = box_dist2(m.nodes[n.first], p), dr = box_dist2(m.nodes[n.first + 1], p);
      if (dl < dr) { stack[sp++] = n.first + 1; stack[sp++] = n.first; } else { stack[sp++] = n.first; stack[sp++] = n.first + 1; }
    }
  }
  *dist2 = bd;
  return best;
}

// ------------------------------------------------------------------------------------------------------ preview shading
struct Camera {         // pinhole: pixel (x, y) of a width x height image looks along fwd + sx * right + sy * up
  float org[3], fwd[3], right[3], up[3];
  float tan_half_fov;   // of the vertical field of view
  int width, height;
};

struct Light { float sun_dir[3], sun_rgb[3], zenith_rgb[3], horizon_rgb[3]; };

// GGX microfacet lobe for light l, view v, normal n (unit vectors, n.l > 0): D G F / (4 n.l n.v) * n.l with the Trowbridge-Reitz
// distribution, the separable Smith-Schlick visibility term and Schlick's Fresnel term at a normal reflectance f0.
GB_HD float ggx_specular(const float* n, const float* v, const float* l, float roughness, float f0) {
  float h[3] = {v[0] + l[0], v[1] + l[1], v[2] + l[2]};
  const float hl = sqrtf(h[0] * h[0] + h[1] * h[1] + h[2] * h[2]);
  if (hl <= 0.0f) return 0.0f;
  for (int i = 0; i < 3; ++i) h[i] /= hl;
  const float nl = n[0] * l[0] + n[1] * l[1] + n[2] * l[2], nv = n[0] * v[0] + n[1] * v[1] + n[2] * v[2];
  if (nl <= 0.0f || nv <= 0.0f) return 0.0f;
  const float nh = n[0] * h[0] + n[1] * h[1] + n[2] * h[2], vh = v[0] * h[0] + v[1] * h[1] + v[2] * h[2];
  const float a = roughness * roughness, a2 = a * a;
  const float dd = nh * nh * (a2 - 1.0f) + 1.0f;
  const float D = a2 / (3.14159265f * dd * dd);
  const float k = (roughness + 1.0f) * (roughness + 1.0f) * 0.125f;
  const float G = (nl / (nl * (1.0f - k) + k)) * (nv / (nv * (1.0f - k) + k));
  const float m = 1.0f - (vh < 0.0f ? 0.0f : vh), m2 = m * m;
  const float F = f0 + (1.0f - f0) * m2 * m2 * m;
  return D * G * F / (4.0f * nv);
}

GB_HD void sky(const Light& l, const float* d, float* rgb) {
  float h = d[1] < 0.0f ? 0.0f : d[1];
  h = sqrtf(h);
  for (int i = 0; i < 3; ++i) rgb[i] = l.horizon_rgb[i] + h * (l.zenith_rgb[i] - l.horizon_rgb[i]);
}

// One pixel: rgb [3] (linear), depth (distance along the ray, 0 on a miss), normal [3] (facing the camera), mask (1 on a hit).
// albedo_rgb[3] is the diffuse colour; albedo_rgb[3] / [4] are the roughness (<= 0: no specular lobe) and the normal reflectance.
GB_HD void shade_pixel(const Mesh& m, const Camera& cam, const Light& l, const float* albedo_rgb, int x, int y, float* rgb, float* depth,
                       float* normal, float* mask) {
  const float aspect = (float)cam.width / (float)cam.height;
  const float sx = (2.0f * (x + 0.5f) / cam.width - 1.0f) * cam.tan_half_fov * aspect;
  const float sy = (1.0f - 2.0f * (y + 0.5f) / cam.height) * cam.tan_half_fov;
  float d[3];
  for (int i = 0; i < 3; ++i) d[i] = cam.fwd[i] + sx * cam.right[i] + sy * cam.up[i];
  const float len = sqrtf(dot3(d, d));
  for (int i = 0; i < 3; ++i) d[i] /= len;
  const Hit h = trace(m, cam.org, d, 1e-6f, 1e30f, false);
  if (h.tri < 0) { sky(l, d, rgb); *depth = 0.0f; normal[0] = normal[1] = normal[2] = 0.0f; *mask = 0.0f; return; }
  const float *a, *b, *c;
  tri_corners(m, h.tri, a, b, c);
  const float e1[3] = {b[0] - a[0], b[1] - a[1], b[2] - a[2]}, e2[3] = {c[0] - a[0], c[1] - a[1], c[2] - a[2]};
  float n[3] = {e1[1] * e2[2] - e1[2] * e2[1], e1[2] * e2[0] - e1[0] * e2[2], e1[0] * e2[1] - e1[1] * e2[0]};
  const float nl = sqrtf(dot3(n, n));
  for (int i = 0; i < 3; ++i) n[i] = nl > 0.0f ? n[i] / nl : 0.0f;
  if (dot3(n, d) > 0.0f) for (int i = 0; i < 3; ++i) n[i] = -n[i];
  float p[3];
  for (int i = 0; i < 3; ++i) p[i] = cam.org[i] + h.t * d[i] + 1e-4f * n[i];
  float cosl = dot3(n, l.sun_dir);
  cosl = cosl < 0.0f ? 0.0f : cosl;
  float lit = 0.0f;
  if (cosl > 0.0f && trace(m, p, l.sun_dir, 1e-5f, 1e30f, true).tri < 0) lit = cosl;
  float amb[3];
  sky(l, n, amb);
  float spec = 0.0f;
  if (lit > 0.0f && albedo_rgb[3] > 0.0f) {
    const float view[3] = {-d[0], -d[1], -d[2]};
    spec = ggx_specular(n, view, l.sun_dir, albedo_rgb[3], albedo_rgb[4]);
  }
  for (int i = 0; i < 3; ++i) rgb[i] = albedo_rgb[i] * (l.sun_rgb[i] * lit + 0.5f * amb[i]) + l.sun_rgb[i] * spec;
  *depth = h.t; *mask = 1.0f;
  for (int i = 0; i < 3; ++i) normal[i] = n[i];
}

}  // namespace gbgeo
