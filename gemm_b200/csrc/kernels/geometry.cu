// CUDA kernels of the geometry helpers: one thread per splat / grid cell / ray / query point / pixel, each calling the inline
// function of geometry.cuh that the host library runs in a loop.  Plain CUDA-core work: gathers, a few dozen flops and a stack per
// thread; nothing here is shaped like a matrix product.  The hierarchy is built on the host (host/geometry_host.cc) and passed in.
#include "geometry.cuh"
#include "host_common.h"

using namespace gbgeo;

namespace {

struct GridArg { const float* v; int nx, ny, nz; float org[3], step[3]; };
struct MeshArg { const float* verts; const int* tris; const Node* nodes; const int* order; int n_nodes; };

__device__ __forceinline__ Grid grid_of(const GridArg& a) {
  Grid g; g.v = a.v; g.nx = a.nx; g.ny = a.ny; g.nz = a.nz;
  for (int i = 0; i < 3; ++i) { g.org[i] = a.org[i]; g.step[i] = a.step[i]; }
  return g;
}
__device__ __forceinline__ Mesh mesh_of(const MeshArg& a) {
  Mesh m; m.verts = a.verts; m.tris = a.tris; m.nodes = a.nodes; m.tri_order = a.order; m.n_nodes = a.n_nodes;
  return m;
}

__global__ void gs_rows_kernel(long n, const float* xyz, const float* f_dc, const float* opacity, const float* scale, const float* rot,
                               float opacity_bias, float scaling_bias, float* rows) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float row[17];
  gs_row(xyz + 3 * i, f_dc + 3 * i, opacity[i], scale + 3 * i, rot + 4 * i, opacity_bias, scaling_bias, row);
  for (int q = 0; q < 17; ++q) rows[17 * i + q] = row[q];
}

__device__ __forceinline__ bool cell_of(const GridArg& a, long cell, int* i, int* j, int* k) {
  const long cy = a.ny - 1, cz = a.nz - 1, n = (long)(a.nx - 1) * cy * cz;
  if (cell >= n) return false;
  *k = (int)(cell % cz); *j = (int)((cell / cz) % cy); *i = (int)(cell / (cz * cy));
  return true;
}

__global__ void iso_count_kernel(GridArg a, float iso, int* counts) {
  const long cell = (long)blockIdx.x * blockDim.x + threadIdx.x;
  int i, j, k;
  if (!cell_of(a, cell, &i, &j, &k)) return;
  counts[cell] = cell_triangles(grid_of(a), i, j, k, iso, nullptr, nullptr);
}

__global__ void iso_emit_kernel(GridArg a, float iso, const long long* offsets, const int* counts, float* pos, long long* key) {
  const long cell = (long)blockIdx.x * blockDim.x + threadIdx.x;
  int i, j, k;
  if (!cell_of(a, cell, &i, &j, &k) || counts[cell] <= 0) return;
  float p[12 * 9];
  long long kk[12 * 3];
  const int n = cell_triangles(grid_of(a), i, j, k, iso, p, kk);
  const long long o = offsets[cell];
  for (int q = 0; q < n * 9; ++q) pos[9 * o + q] = p[q];
  for (int q = 0; q < n * 3; ++q) key[3 * o + q] = kk[q];
}

__global__ void trace_kernel(MeshArg a, long n_rays, const float* org, const float* dir, float tmin, float tmax, int any_hit, float* out_t,
                             int* out_tri, float* out_uv) {
  const long r = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_rays) return;
  const float o[3] = {org[3 * r], org[3 * r + 1], org[3 * r + 2]}, d[3] = {dir[3 * r], dir[3 * r + 1], dir[3 * r + 2]};
  const Hit h = trace(mesh_of(a), o, d, tmin, tmax, any_hit != 0);
  out_t[r] = h.tri >= 0 ? h.t : INFINITY; out_tri[r] = h.tri; out_uv[2 * r] = h.u; out_uv[2 * r + 1] = h.v;
}

__global__ void closest_kernel(MeshArg a, long n_points, const float* pts, float* out_dist, int* out_tri, float* out_point, float* out_w) {
  const long r = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_points) return;
  const float p[3] = {pts[3 * r], pts[3 * r + 1], pts[3 * r + 2]};
  float d2 = INFINITY, cp[3] = {0.f, 0.f, 0.f}, w[3] = {0.f, 0.f, 0.f};
  out_tri[r] = closest_point(mesh_of(a), p, &d2, cp, w);
  out_dist[r] = sqrtf(d2);
  for (int i = 0; i < 3; ++i) { out_point[3 * r + i] = cp[i]; out_w[3 * r + i] = w[i]; }
}

struct RenderArg { Camera cam; Light light; float albedo[5]; };   // diffuse rgb, roughness, normal reflectance

__global__ void render_kernel(MeshArg a, RenderArg ra, float* rgb, float* depth, float* normal, float* mask) {
  const int x = blockIdx.x * blockDim.x + threadIdx.x, y = blockIdx.y * blockDim.y + threadIdx.y;
  if (x >= ra.cam.width || y >= ra.cam.height) return;
  const size_t px = (size_t)y * ra.cam.width + x;
  float c[3], n[3], dp, mk;
  shade_pixel(mesh_of(a), ra.cam, ra.light, ra.albedo, x, y, c, &dp, n, &mk);
  for (int i = 0; i < 3; ++i) { rgb[3 * px + i] = c[i]; normal[3 * px + i] = n[i]; }
  depth[px] = dp; mask[px] = mk;
}

inline unsigned blocks(long n, int per) { return (unsigned)((n + per - 1) / per); }

GridArg grid_arg(const float* v, int nx, int ny, int nz, const float* org, const float* step) {
  GridArg a; a.v = v; a.nx = nx; a.ny = ny; a.nz = nz;
  for (int i = 0; i < 3; ++i) { a.org[i] = org[i]; a.step[i] = step[i]; }
  return a;
}
MeshArg mesh_arg(const float* verts, const int* tris, const void* nodes, const int* order, int n_nodes) {
  MeshArg a; a.verts = verts; a.tris = tris; a.nodes = (const Node*)nodes; a.order = order; a.n_nodes = n_nodes;
  return a;
}

}  // namespace

// All pointers below are device pointers except org / step / cam / light / albedo (small host arrays passed by value).
GB_API int gb_geo_gs_rows(long n, const float* xyz, const float* f_dc, const float* opacity, const float* scale, const float* rot, float opacity_bias,
                          float scaling_bias, float* rows, cudaStream_t stream) {
  if (n <= 0) return 0;
  gs_rows_kernel<<<blocks(n, 256), 256, 0, stream>>>(n, xyz, f_dc, opacity, scale, rot, opacity_bias, scaling_bias, rows);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_geo_iso_count(const float* v, int nx, int ny, int nz, const float* org, const float* step, float iso, int* counts, cudaStream_t stream) {
  if (nx < 2 || ny < 2 || nz < 2) return gb::fail("iso-surface: the grid needs at least 2 samples per axis%s", "");
  const long cells = (long)(nx - 1) * (ny - 1) * (nz - 1);
  iso_count_kernel<<<blocks(cells, 128), 128, 0, stream>>>(grid_arg(v, nx, ny, nz, org, step), iso, counts);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_geo_iso_emit(const float* v, int nx, int ny, int nz, const float* org, const float* step, float iso, const long long* offsets,
                           const int* counts, float* pos, long long* key, cudaStream_t stream) {
  if (nx < 2 || ny < 2 || nz < 2) return gb::fail("iso-surface: the grid needs at least 2 samples per axis%s", "");
  const long cells = (long)(nx - 1) * (ny - 1) * (nz - 1);
  iso_emit_kernel<<<blocks(cells, 64), 64, 0, stream>>>(grid_arg(v, nx, ny, nz, org, step), iso, offsets, counts, pos, key);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_geo_trace(const float* verts, const int* tris, const void* nodes, const int* order, int n_nodes, long n_rays, const float* org,
                        const float* dir, float tmin, float tmax, int any_hit, float* out_t, int* out_tri, float* out_uv, cudaStream_t stream) {
  if (n_rays <= 0) return 0;
  trace_kernel<<<blocks(n_rays, 128), 128, 0, stream>>>(mesh_arg(verts, tris, nodes, order, n_nodes), n_rays, org, dir, tmin, tmax, any_hit, out_t,
                                                        out_tri, out_uv);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_geo_closest(const float* verts, const int* tris, const void* nodes, const int* order, int n_nodes, long n_points, const float* pts,
                          float* out_dist, int* out_tri, float* out_point, float* out_w, cudaStream_t stream) {
  if (n_points <= 0) return 0;
  closest_kernel<<<blocks(n_points, 128), 128, 0, stream>>>(mesh_arg(verts, tris, nodes, order, n_nodes), n_points, pts, out_dist, out_tri, out_point,
                                                            out_w);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_geo_render(const float* verts, const int* tris, const void* nodes, const int* order, int n_nodes, const float* cam, int width, int height,
                         const float* light, const float* albedo, float* rgb, float* depth, float* normal, float* mask, cudaStream_t stream) {
  if (width <= 0 || height <= 0) return gb::fail("render: empty image%s", "");
  RenderArg ra;
  memcpy(ra.cam.org, cam, sizeof(float) * 12); ra.cam.tan_half_fov = cam[12]; ra.cam.width = width; ra.cam.height = height;
  memcpy(ra.light.sun_dir, light, sizeof(float) * 12);
  for (int i = 0; i < 5; ++i) ra.albedo[i] = albedo[i];
  const dim3 block(16, 8), grid((width + 15) / 16, (height + 7) / 8);
  render_kernel<<<grid, block, 0, stream>>>(mesh_arg(verts, tris, nodes, order, n_nodes), ra, rgb, depth, normal, mask);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}
