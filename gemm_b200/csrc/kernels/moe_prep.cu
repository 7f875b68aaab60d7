// Everything between the RMSNorm in front of a MoE block and its grouped expert GEMM, in ONE launch, for decode-sized
// batches (at most 64 tokens, at most 128 experts):
//
//   router logits (tcgen05, K split over a thread-block cluster)  ->  top-k routing  ->  expert-sorted row plan  ->
//   gather of the token rows into expert order, quantised to MXFP8 (or copied as bf16)
//
// The chain used to be four launches (router projection, routing, plan, gather / quantise) of which three ran on one CTA or
// a handful; here the CTAs of one cluster share the work and hand each other their partial results through distributed
// shared memory, so nothing but the final plan and the gathered rows touches global memory.
//
// Cluster of C = hidden / 256 CTAs (1, 2, 4, 8 or 16).  CTA c
//   1. stages its K slice (256 columns) of the router matrix [128 x 256] and of the tokens [64 x 256] in shared memory in
//      the 128-byte-swizzled K-major layout, and issues 16 MMAs (M = 128 experts, N = 64 tokens, K = 16): a partial logit
//      tile [128 x 64] in TMEM;
//   2. sends the partial logits of token t to the CTA that owns the token (t / (64 / C)) with st.shared::cluster; after a
//      cluster barrier the owner adds the C partials in CTA order (fixed order: bit-identical from run to run), routes its
//      tokens (one warp each) and broadcasts the chosen expert ids to every CTA of the cluster;
//   3. after a second cluster barrier every CTA builds the same plan: a 64-bit token mask per expert gives the segment
//      sizes (popcount) and the rank of a token inside its expert's segment (popcount of the lower bits), i.e. rows are
//      ordered by token inside an expert, as the multi-kernel plan orders them;
//   4. serves the tokens it owns: a token's bf16 row is quantised once per 32 elements (E8M0 scale into the scale atoms of the
//      grouped GEMM) and the bytes are stored to the rows of all its picks in the expert-sorted buffer.
//
// With expert parallelism every rank runs this over ALL tokens of the step (gathered from the peers) and keeps only the
// experts it owns (id_shift / n_local); the kernel can wait for the peers' arrival flags before it touches the tokens.
//
// Replaces in the reference: the router GEMV + device-to-host copy + host top-k of cuda/llm/cuda_llm_runner.c:13611-13648,
// 14878-14881, moe_topk_kernel (:7958), gather_rows_f32 (:7931) and mmq_gather_quant_q8_1 (:5240); the routing rule is
// that of common/transformer.h:4050-4091 and common/m3_impl.h:692-698.
#include "sm100.cuh"
#include "host_common.h"
#include "../fabric/fabric.cuh"
#include "moe_route.cuh"
#include "mxq.cuh"

namespace gb {

constexpr int kPrepThreads = 512;      // 16 warps: the gather phase wants many rows in flight
constexpr int kPrepTok = 64;          // token capacity (N of the MMA tile)
constexpr int kPrepExp = 128;         // expert capacity (M of the MMA tile)
constexpr int kPrepKC = 256;          // K columns per CTA
constexpr int kPrepIdsLd = 16;        // ids per token in the shared id table (>= top-k)

struct MoePrepArgs {
  const __nv_bfloat16* h; int ld_h; int n_tok; int hidden;
  const __nv_bfloat16* w; int ld_w; int n_exp;
  const float* bias; int topk; int mode; int renorm; float routed_scale; int id_shift; int n_local;
  int plan_exp;                 // experts the plan covers: n_local when the ids are made local, else n_exp
  int align; int capacity;      // segment alignment (rows) and rows of the expert-sorted buffer
  int* ids; float* weights;     // [n_tok, topk]
  int* seg_start; int* seg_count; int* pair_row; int* row_token;
  uint8_t* xq; uint8_t* xsf; int sf32;      // MXFP8 rows + scale atoms (sf32: one atom per 32 rows), or
  __nv_bfloat16* xs;                        // bf16 rows (when xq is null)
  const uint32_t* wait_flags; int wait_n; const uint32_t* epoch_ptr;
  KernelStatus* status;
};

__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
  return r;
}
__device__ __forceinline__ void st_cluster_b32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.b32 [%0], %1;" :: "r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() { cluster_arrive(); cluster_wait(); }

// Copies rows [0, n_rows) x columns [k0, k0 + 256) of a row-major bf16 matrix into four 128-byte-swizzled K-major atoms
// (rows x 64 elements each, `atom_bytes` apart); rows in [n_rows, PAD_ROWS) are zero.  16-byte chunk c of row r lands at chunk
// c ^ (r & 7) of its 128-byte line: the layout a TMA box with SWIZZLE_128B writes and the MMA descriptor expects.
template <int PAD_ROWS, int U>      // U loads in flight per thread: the copy is latency-bound otherwise
__device__ __forceinline__ void stage_slice(uint8_t* dst, uint32_t atom_bytes, const __nv_bfloat16* __restrict__ src, int ld, int n_rows, int k0) {
  constexpr int CPR = kPrepKC / 8;                         // 16-byte chunks per row
  static_assert((PAD_ROWS * CPR) % (kPrepThreads * U) == 0, "slice must divide into whole batches");
#pragma unroll 1
  for (int q0 = threadIdx.x; q0 < PAD_ROWS * CPR; q0 += kPrepThreads * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int q = q0 + u * kPrepThreads, r = q / CPR, kc = q - r * CPR;
      v[u] = make_uint4(0, 0, 0, 0);
      if (r < n_rows) v[u] = *reinterpret_cast<const uint4*>(src + (size_t)r * ld + k0 + kc * 8);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int q = q0 + u * kPrepThreads, r = q / CPR, kc = q - r * CPR;
      const int atom = kc >> 3, c16 = kc & 7;
      *reinterpret_cast<uint4*>(dst + (size_t)atom * atom_bytes + r * 128 + ((c16 ^ (r & 7)) << 4)) = v[u];
    }
  }
}

__global__ void __launch_bounds__(kPrepThreads, 1)
moe_prep_kernel(const MoePrepArgs a) {
  static_assert(kPrepTok % (kPrepThreads / 32) == 0, "the gather phase gives every warp the same number of items");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int C = gridDim.x, c = blockIdx.x;                 // the grid is one cluster
  const int TPC = kPrepTok / C;                            // tokens owned per CTA
  uint8_t* Ws = smem;                                      // 4 atoms x [128][128 B]
  uint8_t* Xs = Ws + kPrepExp * kPrepKC * 2;               // 4 atoms x [64][128 B]
  float* part = reinterpret_cast<float*>(Xs + kPrepTok * kPrepKC * 2);      // [C][TPC][128] partial logits of MY tokens
  float* lg = part + kPrepTok * kPrepExp;                  // [TPC][128] summed logits
  int* ids_all = reinterpret_cast<int*>(lg + TPC * kPrepExp);               // [64][16] expert id of every pick (-1 = none / not local), later its row
  unsigned long long* mask = reinterpret_cast<unsigned long long*>(ids_all + kPrepTok * kPrepIdsLd);   // [128] tokens per expert
  int* seg0 = reinterpret_cast<int*>(mask + kPrepExp);     // [128] segment start
  int* wsum = seg0 + kPrepExp;                             // [8] scan scratch
  uint64_t* mma_bar = reinterpret_cast<uint64_t*>(wsum + 8);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = c * kPrepKC;

  if (threadIdx.x == 0) { mbar_init(mma_bar, 1); *abort_flag = 0; fence_barrier_init(); }
  if (warp == 1) { tmem_alloc(tmem_slot, 64); tmem_relinquish(); }
  for (int i = threadIdx.x; i < kPrepTok * kPrepIdsLd; i += kPrepThreads) ids_all[i] = -1;
  for (int i = threadIdx.x; i < kPrepExp; i += kPrepThreads) mask[i] = 0ull;
  // "this CTA runs and its tables are initialised": a peer may store into this CTA's shared memory only after it has seen
  // every CTA of the cluster arrive here (the matching wait sits in front of the first remote store)
  cluster_arrive();
  // the router matrix is a weight: its slice is staged while the kernel in front of this one still runs
  stage_slice<kPrepExp, 8>(Ws, kPrepExp * 128, a.w, a.ld_w, a.n_exp, k0);
  pdl_wait();
  pdl_trigger();
  if (a.wait_n > 0) {
    // the token rows were stored here by the peer GPUs: wait for every source's flag of this epoch
    if (threadIdx.x == 0) {
      const uint32_t want = *a.epoch_ptr;
      for (int i = 0; i < a.wait_n; ++i)
        if (!wait_flag_ge(a.wait_flags + i, want, a.status, 1100, i)) { *abort_flag = 1; break; }
    }
    __syncthreads();
  }
  bool ok = (*abort_flag == 0);
  if (ok) stage_slice<kPrepTok, 4>(Xs, kPrepTok * 128, a.h, a.ld_h, a.n_tok, k0);
  fence_proxy_async_smem();                                // generic-proxy stores above -> visible to the tensor core's reads
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // ---- 1. partial logits: D[expert, token] += W[expert, k] * X[token, k] over this CTA's 256 columns
  if (ok && warp == 0 && lane == 0) {
    constexpr uint32_t idesc = make_idesc(kPrepExp, kPrepTok, 1, 1);
#pragma unroll
    for (int at = 0; at < kPrepKC / 64; ++at)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        mma_f16_ss(tmem_base, make_sdesc_sw128(smem_u32(Ws) + at * (kPrepExp * 128) + j * 32),
                   make_sdesc_sw128(smem_u32(Xs) + at * (kPrepTok * 128) + j * 32), idesc, (at > 0 || j > 0) ? 1u : 0u);
    tc_commit(mma_bar);
  }
  if (ok && !mbar_wait(mma_bar, 0, abort_flag, a.status, 1101, c)) ok = false;
  tc_fence_after();
  __syncwarp();
  cluster_wait();                                          // all CTAs of the cluster have started (see cluster_arrive above)

  // ---- 2. every partial goes to the CTA that owns its token (warps 0-3: tokens 0..31, warps 4-7: tokens 32..63; a warp reads
  // the TMEM lane quarter warp % 4, i.e. experts 32 * (warp % 4) + lane)
  if (ok && warp < 8) {
    const int q = warp & 3, col0 = (warp >> 2) * 32;
    uint32_t r[32];
    tmem_ld_x32(tmem_base + ((uint32_t)(q * 32) << 16) + col0, r);
    tc_wait_ld();
    const int e = q * 32 + lane;
    const uint32_t part0 = smem_u32(part);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int t = col0 + j;
      const int owner = t / TPC, tl = t - owner * TPC;
      st_cluster_b32(mapa_u32(part0 + (uint32_t)(((c * TPC + tl) * kPrepExp + e) * 4), (uint32_t)owner), r[j]);
    }
  }
  tc_fence_before();
  cluster_sync_all();                                      // every CTA arrives, aborted or not

  // sum of the C partials in CTA order, then one warp per owned token routes it
  for (int i = threadIdx.x; i < TPC * kPrepExp; i += kPrepThreads) {
    float s = 0.f;
    for (int src = 0; src < C; ++src) s += part[(size_t)src * TPC * kPrepExp + i];
    lg[i] = s;
  }
  __syncthreads();
  {
    const uint32_t ids0 = smem_u32(ids_all);
    for (int tl = warp; tl < TPC; tl += kPrepThreads / 32) {
      const int t = c * TPC + tl;
      if (t >= a.n_tok || !ok) continue;
      const int id = route_row<4>(lg + tl * kPrepExp, a.bias, a.ids + (size_t)t * a.topk, a.weights + (size_t)t * a.topk, lane, a.n_exp, a.topk,
                                  a.mode, a.renorm, a.routed_scale, a.id_shift, a.n_local);
      if (lane < a.topk)
        for (int d = 0; d < C; ++d) st_cluster_b32(mapa_u32(ids0 + (uint32_t)((t * kPrepIdsLd + lane) * 4), (uint32_t)d), (uint32_t)id);
    }
  }
  cluster_sync_all();

  // ---- 3. the plan, computed identically by every CTA
  const int n_pairs = a.n_tok * a.topk;
  for (int i = threadIdx.x; i < n_pairs; i += kPrepThreads) {
    const int t = i / a.topk, j = i - t * a.topk;
    const int e = ids_all[t * kPrepIdsLd + j];
    if (e >= 0 && e < a.plan_exp) atomicOr(&mask[e], 1ull << t);
  }
  __syncthreads();
  if (threadIdx.x < kPrepExp) {
    const int e = threadIdx.x;
    const int cnt = e < a.plan_exp ? __popcll(mask[e]) : 0;
    const int padded = (cnt + a.align - 1) / a.align * a.align;
    int inc = padded;                                      // inclusive scan over the 128 experts: warp scan, then warp totals
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += v; }
    if (lane == 31) wsum[warp] = inc;
    asm volatile("bar.sync 1, 128;" ::: "memory");         // the four warps that scan
    int base = 0;
    for (int w2 = 0; w2 < warp; ++w2) base += wsum[w2];
    seg0[e] = base + inc - padded;
    if (c == 0 && e < a.plan_exp) { a.seg_start[e] = base + inc - padded; a.seg_count[e] = cnt; }
  }
  if (c == 0) for (int r = threadIdx.x; r < a.capacity; r += kPrepThreads) a.row_token[r] = -1;
  __syncthreads();
  // pair (token t, pick j) -> row = start of its expert + number of lower tokens that chose the expert.  One thread per pair;
  // the row replaces the expert id in the shared table (phase 4 reads rows only), CTA 0 also writes the tables out (its -1 fill
  // above is ordered before by the barrier).
  for (int i = threadIdx.x; i < n_pairs; i += kPrepThreads) {
    const int t = i / a.topk, j = i - t * a.topk;
    const int e = ids_all[t * kPrepIdsLd + j];
    int row = -1;
    if (e >= 0 && e < a.plan_exp) {
      row = seg0[e] + __popcll(mask[e] & ((1ull << t) - 1ull));
      if (row >= a.capacity) row = -1;
    }
    ids_all[t * kPrepIdsLd + j] = row;
    if (c == 0) { a.pair_row[i] = row; if (row >= 0) a.row_token[row] = t; }
  }
  __syncthreads();

  // ---- 4. the rows themselves.  Every CTA serves the tokens it owns: a token is quantised ONCE and its bytes are stored to the
  // rows of all its picks.  A work item is (owned token, slab of 32 vectors of 8 elements): 64 / C tokens x C slabs = 64 items,
  // four per warp, whose loads are all requested before the first is used.
  {
    constexpr int IPW = kPrepTok / (kPrepThreads / 32);     // items per warp
    uint4 raw[IPW];
    int tok[IPW], vec[IPW];
#pragma unroll
    for (int u = 0; u < IPW; ++u) {
      const int it = warp * IPW + u;
      const int tl = it / C, slab = it - tl * C;
      tok[u] = c * TPC + tl;
      vec[u] = slab * 32 + lane;
      raw[u] = make_uint4(0, 0, 0, 0);
      if (tok[u] < a.n_tok && ok) raw[u] = *reinterpret_cast<const uint4*>(a.h + (size_t)tok[u] * a.ld_h + vec[u] * 8);
    }
#pragma unroll
    for (int u = 0; u < IPW; ++u) {
      const int t = tok[u], v = vec[u];
      uint2 qv = make_uint2(0, 0);
      int ex = 127;
      if (a.xq != nullptr) {
        const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
        float y[8];
        float amax = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < 4; ++w2) {
          const float2 f = __bfloat1622float2(hv[w2]);
          y[2 * w2] = f.x; y[2 * w2 + 1] = f.y;
          amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));     // 4 consecutive lanes hold one 32-element block
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        ex = e8m0_amax(amax);
        const float inv = __uint_as_float((uint32_t)(254 - ex) << 23);
        qv.x = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(y[0] * inv, y[1] * inv), __NV_SATFINITE, __NV_E4M3) |
               ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(y[2] * inv, y[3] * inv), __NV_SATFINITE, __NV_E4M3) << 16);
        qv.y = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(y[4] * inv, y[5] * inv), __NV_SATFINITE, __NV_E4M3) |
               ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(y[6] * inv, y[7] * inv), __NV_SATFINITE, __NV_E4M3) << 16);
      }
      if (t >= a.n_tok || !ok) continue;
      for (int j = 0; j < a.topk; ++j) {
        const int row = ids_all[t * kPrepIdsLd + j];
        if (row < 0) continue;
        if (a.xq != nullptr) {
          *reinterpret_cast<uint2*>(a.xq + (size_t)row * a.hidden + v * 8) = qv;
          if ((v & 3) == 0) a.xsf[sf_atom_offset(row, v >> 2, a.hidden >> 7, a.sf32)] = (uint8_t)ex;
        } else {
          *reinterpret_cast<uint4*>(a.xs + (size_t)row * a.hidden + v * 8) = raw[u];
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 64); }
}

}  // namespace gb

using namespace gb;

// Cluster size for a hidden width, or 0 when the fused kernel does not take it.
static int prep_cluster(int hidden) {
  if (hidden % kPrepKC) return 0;
  const int c = hidden / kPrepKC;
  return (c == 1 || c == 2 || c == 4 || c == 8 || c == 16) ? c : 0;
}

// 1 when gb_moe_prep takes the shape.
GB_API int gb_moe_prep_supported(int n_tok, int hidden, int n_exp, int topk) {
  return (n_tok >= 1 && n_tok <= kPrepTok && n_exp >= 1 && n_exp <= kPrepExp && topk >= 1 && topk <= kPrepIdsLd && topk <= n_exp &&
          prep_cluster(hidden) != 0) ? 1 : 0;
}

// h bf16 [n_tok, hidden] (row stride ld_h), w bf16 [n_exp, hidden].  Outputs: ids / weights [n_tok, topk]; seg_start / seg_count
// [plan_exp]; pair_row [n_tok * topk]; row_token [capacity]; the gathered rows as MXFP8 (xq [capacity, hidden] + scale atoms xsf in
// the layout of `align`-row tiles: sf32 != 0 for 32-row atoms) or, with xq == NULL, as bf16 (xs [capacity, hidden]).
// id_shift / n_local as in gb_moe_route; plan_exp = n_local when n_local > 0, else n_exp.  Segments start at multiples of `align`.
GB_API int gb_moe_prep(const void* h, int ld_h, int n_tok, int hidden, const void* w, int ld_w, int n_exp, const float* bias, int topk,
                       int mode, int renorm, float routed_scale, int id_shift, int n_local, int align, int capacity, int* ids,
                       float* weights, int* seg_start, int* seg_count, int* pair_row, int* row_token, void* xq, void* xsf, int sf32,
                       void* xs, const void* wait_flags, int wait_n, const void* epoch_ptr, void* status, cudaStream_t stream) {
  if (!gb_moe_prep_supported(n_tok, hidden, n_exp, topk)) return fail("moe_prep: unsupported shape%s (tokens %ld, hidden %ld)", "", n_tok, hidden);
  if (ld_h % 8 || ld_w % 8 || ((uintptr_t)h & 15) || ((uintptr_t)w & 15)) return fail("moe_prep: rows must be 16-byte aligned%s");
  if (align < 1 || capacity < 1) return fail("moe_prep: bad plan geometry%s");
  if (xq == nullptr && xs == nullptr) return fail("moe_prep: no output buffer for the gathered rows%s");
  const int C = prep_cluster(hidden);
  MoePrepArgs a;
  memset(&a, 0, sizeof(a));
  a.h = (const __nv_bfloat16*)h; a.ld_h = ld_h; a.n_tok = n_tok; a.hidden = hidden; a.w = (const __nv_bfloat16*)w; a.ld_w = ld_w; a.n_exp = n_exp;
  a.bias = bias; a.topk = topk; a.mode = mode; a.renorm = renorm; a.routed_scale = routed_scale; a.id_shift = id_shift; a.n_local = n_local;
  a.plan_exp = n_local > 0 ? n_local : n_exp; a.align = align; a.capacity = capacity; a.ids = ids; a.weights = weights;
  a.seg_start = seg_start; a.seg_count = seg_count; a.pair_row = pair_row; a.row_token = row_token;
  a.xq = (uint8_t*)xq; a.xsf = (uint8_t*)xsf; a.sf32 = sf32; a.xs = (__nv_bfloat16*)xs;
  a.wait_flags = (const uint32_t*)wait_flags; a.wait_n = wait_n; a.epoch_ptr = (const uint32_t*)epoch_ptr; a.status = (KernelStatus*)status;
  const int tpc = kPrepTok / C;
  const size_t smem = 1024 + (size_t)kPrepExp * kPrepKC * 2 + (size_t)kPrepTok * kPrepKC * 2 + (size_t)kPrepTok * kPrepExp * 4 +
                      (size_t)tpc * kPrepExp * 4 + (size_t)kPrepTok * kPrepIdsLd * 4 + kPrepExp * 8 + kPrepExp * 4 + 64 + 64;
  auto kern = moe_prep_kernel;
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    GB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    attr_set = true;
  }
  GB_CUDA_OK(launch_k_cluster(kern, dim3((unsigned)C), kPrepThreads, smem, stream, (unsigned)C, a));
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}
