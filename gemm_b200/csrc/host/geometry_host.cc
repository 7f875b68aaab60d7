// Host side of the geometry helpers: the BVH builder, and the functions of kernels/geometry.cuh run in loops (the CPU path of
// gemm_b200.geometry and the oracle of the CUDA kernels, which instantiate the same inline code).
#include <algorithm>
#include <cstring>
#include <vector>

#include "../kernels/geometry.cuh"
#include "common.h"

using namespace gbgeo;

namespace {

struct Builder {
  const float* verts; const int* tris; int leaf;
  std::vector<Node> nodes; std::vector<int> order; std::vector<float> cen, lo, hi;

  void bounds(int first, int count, float* bmin, float* bmax) const {
    for (int a = 0; a < 3; ++a) { bmin[a] = INFINITY; bmax[a] = -INFINITY; }
    for (int q = first; q < first + count; ++q)
      for (int a = 0; a < 3; ++a) { bmin[a] = std::min(bmin[a], lo[3 * (size_t)order[q] + a]); bmax[a] = std::max(bmax[a], hi[3 * (size_t)order[q] + a]); }
  }

  // Median split of the centroids along the longest axis of their bounds; children sit next to each other.
  void split(int node, int first, int count) {
    float bmin[3], bmax[3];
    bounds(first, count, bmin, bmax);
    for (int a = 0; a < 3; ++a) { nodes[node].bmin[a] = bmin[a]; nodes[node].bmax[a] = bmax[a]; }
    if (count <= leaf) { nodes[node].first = first; nodes[node].count = count; return; }
    float cmin[3] = {INFINITY, INFINITY, INFINITY}, cmax[3] = {-INFINITY, -INFINITY, -INFINITY};
    for (int q = first; q < first + count; ++q)
      for (int a = 0; a < 3; ++a) { cmin[a] = std::min(cmin[a], cen[3 * (size_t)order[q] + a]); cmax[a] = std::max(cmax[a], cen[3 * (size_t)order[q] + a]); }
    int axis = 0;
    for (int a = 1; a < 3; ++a) if (cmax[a] - cmin[a] > cmax[axis] - cmin[axis]) axis = a;
    const int mid = first + count / 2;
    std::nth_element(order.begin() + first, order.begin() + mid, order.begin() + first + count,
                     [&](int x, int y) { const float cx = cen[3 * (size_t)x + axis], cy = cen[3 * (size_t)y + axis]; return cx < cy || (cx == cy && x < y); });
    const int left = (int)nodes.size();
    nodes.push_back(Node()); nodes.push_back(Node());
    nodes[node].first = left; nodes[node].count = 0;
    split(left, first, mid - first);
    split(left + 1, mid, first + count - mid);
  }
};

Mesh mesh_of(const float* verts, const int* tris, const void* nodes, const int* order, int n_nodes) {
  Mesh m; m.verts = verts; m.tris = tris; m.nodes = (const Node*)nodes; m.tri_order = order; m.n_nodes = n_nodes;
  return m;
}

}  // namespace

// Build the hierarchy over n_tris triangles (leaves of at most `leaf` triangles).  nodes_out holds 2 * n_tris nodes of 32 bytes,
// order_out n_tris ints.  Returns the number of nodes, -1 on a bad argument (an index outside the vertices, leaf < 1).
GBH_API int gbh_geo_bvh_build(const float* verts, int n_verts, const int* tris, int n_tris, int leaf, void* nodes_out, int* order_out) {
  if (n_tris < 0 || n_verts < 0 || leaf < 1) return gbh::fail("bvh build: bad sizes");
  if (n_tris == 0) return 0;
  for (size_t i = 0; i < 3 * (size_t)n_tris; ++i) if (tris[i] < 0 || tris[i] >= n_verts) return gbh::fail("bvh build: triangle %ld names vertex %d of %d", (long)(i / 3), tris[i], n_verts);
  Builder b; b.verts = verts; b.tris = tris; b.leaf = leaf;
  b.order.resize((size_t)n_tris); b.cen.resize(3 * (size_t)n_tris); b.lo.resize(3 * (size_t)n_tris); b.hi.resize(3 * (size_t)n_tris);
  for (int t = 0; t < n_tris; ++t) {
    b.order[(size_t)t] = t;
    for (int a = 0; a < 3; ++a) {
      const float x = verts[3 * (size_t)tris[3 * (size_t)t] + a], y = verts[3 * (size_t)tris[3 * (size_t)t + 1] + a], z = verts[3 * (size_t)tris[3 * (size_t)t + 2] + a];
      b.lo[3 * (size_t)t + a] = std::min(x, std::min(y, z)); b.hi[3 * (size_t)t + a] = std::max(x, std::max(y, z));
      b.cen[3 * (size_t)t + a] = (x + y + z) * (1.0f / 3.0f);
    }
  }
  b.nodes.reserve(2 * (size_t)n_tris);
  b.nodes.push_back(Node());
  b.split(0, 0, n_tris);
  memcpy(nodes_out, b.nodes.data(), b.nodes.size() * sizeof(Node));
  memcpy(order_out, b.order.data(), sizeof(int) * (size_t)n_tris);
  return (int)b.nodes.size();
}

GBH_API void gbh_geo_gs_rows(long n, const float* xyz, const float* f_dc, const float* opacity, const float* scale, const float* rot, float opacity_bias,
                             float scaling_bias, float* rows) {
  for (long i = 0; i < n; ++i) gs_row(xyz + 3 * i, f_dc + 3 * i, opacity[i], scale + 3 * i, rot + 4 * i, opacity_bias, scaling_bias, rows + 17 * i);
}

static Grid grid_of(const float* v, int nx, int ny, int nz, const float* org, const float* step) {
  Grid g; g.v = v; g.nx = nx; g.ny = ny; g.nz = nz;
  for (int a = 0; a < 3; ++a) { g.org[a] = org[a]; g.step[a] = step[a]; }
  return g;
}

// counts[cell] for the (nx - 1)(ny - 1)(nz - 1) cells, cell = (i * (ny - 1) + j) * (nz - 1) + k
GBH_API void gbh_geo_iso_count(const float* v, int nx, int ny, int nz, const float* org, const float* step, float iso, int* counts) {
  const Grid g = grid_of(v, nx, ny, nz, org, step);
  for (int i = 0; i + 1 < nx; ++i) for (int j = 0; j + 1 < ny; ++j) for (int k = 0; k + 1 < nz; ++k)
    counts[((size_t)i * (ny - 1) + j) * (nz - 1) + k] = cell_triangles(g, i, j, k, iso, nullptr, nullptr);
}

// offsets[cell]: index of the cell's first triangle (exclusive prefix sum of the counts)
GBH_API void gbh_geo_iso_emit(const float* v, int nx, int ny, int nz, const float* org, const float* step, float iso, const long long* offsets,
                              const int* counts, float* pos, long long* key) {
  const Grid g = grid_of(v, nx, ny, nz, org, step);
  for (int i = 0; i + 1 < nx; ++i) for (int j = 0; j + 1 < ny; ++j) for (int k = 0; k + 1 < nz; ++k) {
    const size_t cell = ((size_t)i * (ny - 1) + j) * (nz - 1) + k;
    if (counts[cell] > 0) cell_triangles(g, i, j, k, iso, pos + 9 * (size_t)offsets[cell], key + 3 * (size_t)offsets[cell]);
  }
}

GBH_API void gbh_geo_trace(const float* verts, const int* tris, const void* nodes, const int* order, int n_nodes, long n_rays, const float* org,
                           const float* dir, float tmin, float tmax, int any_hit, float* out_t, int* out_tri, float* out_uv) {
  const Mesh m = mesh_of(verts, tris, nodes, order, n_nodes);
  for (long r = 0; r < n_rays; ++r) {
    const Hit h = trace(m, org + 3 * r, dir + 3 * r, tmin, tmax, any_hit != 0);
    out_t[r] = h.tri >= 0 ? h.t : INFINITY; out_tri[r] = h.tri; out_uv[2 * r] = h.u; out_uv[2 * r + 1] = h.v;
  }
}

GBH_API void gbh_geo_closest(const float* verts, const int* tris, const void* nodes, const int* order, int n_nodes, long n_points, const float* pts,
                             float* out_dist, int* out_tri, float* out_point, float* out_w) {
  const Mesh m = mesh_of(verts, tris, nodes, order, n_nodes);
  for (long r = 0; r < n_points; ++r) {
    float d2 = INFINITY;
    out_tri[r] = closest_point(m, pts + 3 * r, &d2, out_point + 3 * r, out_w + 3 * r);
    out_dist[r] = sqrtf(d2);
  }
}

// cam: org fwd right up [12] + tan(fov / 2); light: sun_dir sun_rgb zenith_rgb horizon_rgb [12]; albedo: diffuse rgb, roughness,
// normal reflectance [5]; images are [height][width](x 3)
GBH_API void gbh_geo_render(const float* verts, const int* tris, const void* nodes, const int* order, int n_nodes, const float* cam, int width, int height,
                            const float* light, const float* albedo, float* rgb, float* depth, float* normal, float* mask) {
  const Mesh m = mesh_of(verts, tris, nodes, order, n_nodes);
  Camera c; Light l;
  memcpy(c.org, cam, sizeof(float) * 12); c.tan_half_fov = cam[12]; c.width = width; c.height = height;
  memcpy(l.sun_dir, light, sizeof(float) * 12);
  for (int y = 0; y < height; ++y) for (int x = 0; x < width; ++x) {
    const size_t px = (size_t)y * width + x;
    shade_pixel(m, c, l, albedo, x, y, rgb + 3 * px, depth + px, normal + 3 * px, mask + px);
  }
}
