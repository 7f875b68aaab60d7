// Mixture-of-experts routing on the device, with no host synchronisation anywhere:
//   gb_moe_route   router logits -> (softmax | sigmoid+bias) -> top-k -> renormalised weights
//   gb_moe_plan    top-k ids -> per-expert row segments (aligned for the grouped GEMM), the row of every
//                  (token, k) pair in the expert-sorted buffer and the source token of every row;
//                  ordering inside an expert is by (token, k), so results are run-to-run identical
//   gb_moe_combine out[t] = sum_k w[t,k] * y[row(t,k)]   (fixed order -> deterministic)
//
// Router semantics follow common/transformer.h:4050-4091 (softmax over all experts, top-k, weights
// renormalised to sum 1; ties go to the lower index, NaN counts as -FLT_MAX as in
// cuda/llm/cuda_llm_runner.c:7958-8035) and common/m3_impl.h:692-698 for the sigmoid + bias variant.
// Replaces moe_topk_kernel (cuda_llm_runner.c:7958), the host-side moe_topk_softmax (:13611, a
// device->host sync per layer), gather_rows_f32 (:7931) and scatter_add_weighted_f32 (:7943).
#include "sm100.cuh"
#include "host_common.h"
#include "../fabric/fabric.cuh"
#include "moe_route.cuh"
#include <float.h>

namespace gb {

template <int MAXV>
__device__ __forceinline__ int route_token_n(const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ ids,
                                           float* __restrict__ weights, int w, int lane, int n_exp, int k, int mode, int renorm,
                                           float routed_scale, int ld, int id_shift, int n_local) {
  return route_row<MAXV>(logits + (size_t)w * ld, bias, ids + (size_t)w * k, weights + (size_t)w * k, lane, n_exp, k, mode, renorm,
                         routed_scale, id_shift, n_local);
}

// The per-lane expert slots are sized to the expert count, so a 128-expert router runs a quarter of the 512-expert code.
__device__ __forceinline__ int route_token(const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ ids,
                                           float* __restrict__ weights, int w, int lane, int n_exp, int k, int mode, int renorm,
                                           float routed_scale, int ld, int id_shift, int n_local) {
  if (n_exp <= 128) return route_token_n<4>(logits, bias, ids, weights, w, lane, n_exp, k, mode, renorm, routed_scale, ld, id_shift, n_local);
  if (n_exp <= 256) return route_token_n<8>(logits, bias, ids, weights, w, lane, n_exp, k, mode, renorm, routed_scale, ld, id_shift, n_local);
  return route_token_n<16>(logits, bias, ids, weights, w, lane, n_exp, k, mode, renorm, routed_scale, ld, id_shift, n_local);
}

// One warp per token.
__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ ids, float* __restrict__ weights,
                 int n_tok, int n_exp, int k, int mode, int renorm, float routed_scale, int ld, int id_shift, int n_local) {
  pdl_wait();
  pdl_trigger();
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (w >= n_tok) return;
  route_token(logits, bias, ids, weights, w, threadIdx.x & 31, n_exp, k, mode, renorm, routed_scale, ld, id_shift, n_local);
}

// Router logits for decode-sized batches on the CUDA cores: out[m, n] = sum_k x[m, k] * w[n, k] (bf16 in, fp32 out).
// A 128 x 2048 router matrix is one tensor-core tile, i.e. one CTA walking 32 k-steps (about 20 us); here 64 CTAs each take
// 8 tokens (staged in shared memory) x 16 experts and finish in a few microseconds.  k % 256 == 0, k <= 8192.
constexpr int kSlTok = 8, kSlRows = 16;
__global__ void __launch_bounds__(256)
small_linear_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, float* __restrict__ out, int m, int n, int k,
                    int ldx, int ldw, int ldo) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint4 sx[];                     // [kSlTok][k / 8] vectors of 8 bf16
  const int n0 = blockIdx.x * kSlRows, m0 = blockIdx.y * kSlTok;
  const int kv = k >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int RPW = kSlRows / 8;                  // rows per warp
  constexpr int MAXV = 8;                           // weight vectors per lane and row held in registers (k <= 2048); longer rows loop
  // the weight rows of this warp are requested first, so that their latency overlaps the staging of the token rows
  uint4 wr[RPW][MAXV];
#pragma unroll
  for (int rr = 0; rr < RPW; ++rr) {
    const int row = n0 + warp * RPW + rr;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + 32 * i;
      wr[rr][i] = (row < n && v < kv) ? *reinterpret_cast<const uint4*>(w + (size_t)row * ldw + v * 8) : make_uint4(0, 0, 0, 0);
    }
  }
  for (int i = threadIdx.x; i < kSlTok * kv; i += blockDim.x) {
    const int tk = i / kv, v = i - tk * kv;
    sx[i] = (m0 + tk < m) ? *reinterpret_cast<const uint4*>(x + (size_t)(m0 + tk) * ldx + v * 8) : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
#pragma unroll
  for (int rr = 0; rr < RPW; ++rr) {
    const int row = n0 + warp * RPW + rr;
    if (row >= n) continue;
    float acc[kSlTok];
#pragma unroll
    for (int i = 0; i < kSlTok; ++i) acc[i] = 0.f;
    auto fma_vec = [&](const uint4& wv, int v) {
      const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv);
      float wf[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(wh[i]); wf[2 * i] = f.x; wf[2 * i + 1] = f.y; }
#pragma unroll
      for (int tk = 0; tk < kSlTok; ++tk) {
        const uint4 xr = sx[tk * kv + v];
        const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xr);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(xh[i]); acc[tk] += wf[2 * i] * f.x + wf[2 * i + 1] * f.y; }
      }
    };
#pragma unroll
    for (int i = 0; i < MAXV; ++i) if (lane + 32 * i < kv) fma_vec(wr[rr][i], lane + 32 * i);
    for (int v = lane + 32 * MAXV; v < kv; v += 32) fma_vec(*reinterpret_cast<const uint4*>(w + (size_t)row * ldw + v * 8), v);
#pragma unroll
    for (int tk = 0; tk < kSlTok; ++tk) {
      const float s = warp_sum(acc[tk]);
      if (lane == 0 && m0 + tk < m) out[(size_t)(m0 + tk) * ldo + row] = s;
    }
  }
}

// Router projection and routing in one launch for decode-sized batches and up to 128 experts: the CTAs of `small_linear_kernel`
// that share a token group (one per 16 experts) form a thread-block cluster, leave their logits in the shared memory of the
// cluster's first CTA (distributed shared memory), and after the cluster barrier that CTA routes its 8 tokens, one warp each.
// The logits never go to global memory and the routing kernel's launch disappears.
__global__ void __launch_bounds__(256)
router_route_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, int m, int n, int k, int ldx, int ldw,
                    const float* __restrict__ bias, int* __restrict__ ids, float* __restrict__ weights, int topk, int mode, int renorm,
                    float routed_scale, int id_shift, int n_local) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint4 sx[];                     // [kSlTok][k / 8] vectors of 8 bf16
  __shared__ float lg[kSlTok][128];                 // used in the cluster's first CTA: logits of its 8 tokens
  const int n0 = blockIdx.x * kSlRows, m0 = blockIdx.y * kSlTok;
  const int kv = k >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int RPW = kSlRows / 8;
  constexpr int MAXV = 8;
  uint4 wr[RPW][MAXV];
#pragma unroll
  for (int rr = 0; rr < RPW; ++rr) {
    const int row = n0 + warp * RPW + rr;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + 32 * i;
      wr[rr][i] = (row < n && v < kv) ? *reinterpret_cast<const uint4*>(w + (size_t)row * ldw + v * 8) : make_uint4(0, 0, 0, 0);
    }
  }
  for (int i = threadIdx.x; i < kSlTok * kv; i += blockDim.x) {
    const int tk = i / kv, v = i - tk * kv;
    sx[i] = (m0 + tk < m) ? *reinterpret_cast<const uint4*>(x + (size_t)(m0 + tk) * ldx + v * 8) : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  // address of lg in the cluster's CTA 0 (the cluster spans blockIdx.x)
  uint32_t lg0;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(lg0) : "r"(smem_u32(&lg[0][0])), "r"(0));
#pragma unroll
  for (int rr = 0; rr < RPW; ++rr) {
    const int row = n0 + warp * RPW + rr;
    float acc[kSlTok];
#pragma unroll
    for (int i = 0; i < kSlTok; ++i) acc[i] = 0.f;
    auto fma_vec = [&](const uint4& wv, int v) {
      const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv);
      float wf[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(wh[i]); wf[2 * i] = f.x; wf[2 * i + 1] = f.y; }
#pragma unroll
      for (int tk = 0; tk < kSlTok; ++tk) {
        const uint4 xr = sx[tk * kv + v];
        const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xr);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(xh[i]); acc[tk] += wf[2 * i] * f.x + wf[2 * i + 1] * f.y; }
      }
    };
    if (row < n) {
#pragma unroll
      for (int i = 0; i < MAXV; ++i) if (lane + 32 * i < kv) fma_vec(wr[rr][i], lane + 32 * i);
      for (int v = lane + 32 * MAXV; v < kv; v += 32) fma_vec(*reinterpret_cast<const uint4*>(w + (size_t)row * ldw + v * 8), v);
    }
#pragma unroll
    for (int tk = 0; tk < kSlTok; ++tk) {
      const float s = warp_sum(acc[tk]);
      if (lane == 0 && row < n)
        asm volatile("st.shared::cluster.f32 [%0], %1;" :: "r"(lg0 + (uint32_t)(tk * 128 + row) * 4u), "f"(s) : "memory");
    }
  }
  // every CTA of the cluster arrives (no early exit above), so the barrier completes; release / acquire orders the remote stores
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (blockIdx.x != 0) return;
  const int tok = m0 + warp;                         // 8 warps, 8 tokens
  if (tok >= m) return;
  route_row<4>(&lg[warp][0], bias, ids + (size_t)tok * topk, weights + (size_t)tok * topk, lane, n, topk, mode, renorm, routed_scale,
               id_shift, n_local);
}

constexpr int kPlanBlock = 256;

// block_hist[b][e] = pairs of block b routed to expert e (pairs whose expert is outside [e_lo, e_hi) are dropped)
__global__ void __launch_bounds__(kPlanBlock)
moe_hist_kernel(const int* __restrict__ ids, int* __restrict__ block_hist, long n_pairs, int n_exp) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ int sh[];
  for (int e = threadIdx.x; e < n_exp; e += kPlanBlock) sh[e] = 0;
  __syncthreads();
  const long i = (long)blockIdx.x * kPlanBlock + threadIdx.x;
  if (i < n_pairs) { const int e = ids[i]; if (e >= 0 && e < n_exp) atomicAdd(&sh[e], 1); }
  __syncthreads();
  for (int e = threadIdx.x; e < n_exp; e += kPlanBlock) block_hist[(size_t)blockIdx.x * n_exp + e] = sh[e];
}

// One block per expert: exclusive scan of block_hist[:, e] over the blocks (in place) and seg_count[e].
__global__ void __launch_bounds__(256)
moe_scan_kernel(int* __restrict__ block_hist, int* __restrict__ seg_count, int n_blocks, int n_exp) {
  pdl_wait();
  pdl_trigger();
  __shared__ int part[256];
  const int e = blockIdx.x, t = threadIdx.x;
  const int per = (n_blocks + 255) / 256;
  const int b0 = t * per, b1 = min(n_blocks, b0 + per);
  int sum = 0;
  for (int b = b0; b < b1; ++b) sum += block_hist[(size_t)b * n_exp + e];
  part[t] = sum;
  __syncthreads();
  // Hillis-Steele inclusive scan over 256 partial sums
  for (int o = 1; o < 256; o <<= 1) {
    int v = (t >= o) ? part[t - o] : 0;
    __syncthreads();
    part[t] += v;
    __syncthreads();
  }
  int run = part[t] - sum;
  for (int b = b0; b < b1; ++b) { const int c = block_hist[(size_t)b * n_exp + e]; block_hist[(size_t)b * n_exp + e] = run; run += c; }
  if (t == 255) seg_count[e] = part[255];
}

// Experts are grouped into "regions" of experts_per_region consecutive experts (the experts of one
// destination rank); region r starts at row r * region_rows, segments inside are aligned to `align`.
__global__ void __launch_bounds__(512)
moe_seg_kernel(const int* __restrict__ seg_count, int* __restrict__ seg_start, int* __restrict__ region_rows_used,
               int n_exp, int experts_per_region, int region_rows, int align, unsigned* epoch_ctr) {
  pdl_wait();
  pdl_trigger();
  const int r = threadIdx.x;
  __shared__ int cnt[512], start[512];
  if (r == 0 && epoch_ctr != nullptr) *epoch_ctr = *epoch_ctr + 1;     // one tick per MoE layer call (expert-parallel epoch)
  if (r < n_exp) cnt[r] = seg_count[r];
  __syncthreads();
  if (r < n_exp / experts_per_region) {
    int pos = 0;
    for (int i = 0; i < experts_per_region; ++i) {
      const int ee = r * experts_per_region + i;
      start[ee] = r * region_rows + pos;
      pos += (cnt[ee] + align - 1) / align * align;
    }
    if (region_rows_used != nullptr) region_rows_used[r] = pos;
  }
  __syncthreads();
  if (r < n_exp) seg_start[r] = start[r];
}

__global__ void __launch_bounds__(kPlanBlock)
moe_scatter_kernel(const int* __restrict__ ids, const int* __restrict__ block_hist, const int* __restrict__ seg_start,
                   int* __restrict__ pair_row, int* __restrict__ row_token, long n_pairs, int n_exp, int k, long capacity) {
  pdl_wait();
  pdl_trigger();
  __shared__ int se[kPlanBlock];
  const long i = (long)blockIdx.x * kPlanBlock + threadIdx.x;
  int e = -1;
  if (i < n_pairs) { e = ids[i]; if (e < 0 || e >= n_exp) e = -1; }
  se[threadIdx.x] = e;
  __syncthreads();
  if (i >= n_pairs) return;
  if (e < 0) { pair_row[i] = -1; return; }
  int rank = 0;
  for (int j = 0; j < (int)threadIdx.x; ++j) rank += (se[j] == e);
  const long row = (long)seg_start[e] + block_hist[(size_t)blockIdx.x * n_exp + e] + rank;
  if (row < capacity) { pair_row[i] = (int)row; row_token[row] = (int)(i / k); }
  else pair_row[i] = -1;
}

// The whole plan in one CTA for decode-sized batches (n_pairs <= kSmallPairs): histogram, aligned segment starts,
// rank of every pair inside its expert (by pair index, so the order is the one of the multi-kernel path) and the
// scatter, all from shared memory.  Replaces one memset and four launches.
constexpr int kSmallPairs = 2048;
__global__ void __launch_bounds__(1024)
moe_plan_small_kernel(const int* __restrict__ ids, int* __restrict__ seg_start, int* __restrict__ seg_count,
                      int* __restrict__ region_rows_used, int* __restrict__ pair_row, int* __restrict__ row_token, int n_pairs,
                      int n_exp, int k, int experts_per_region, int region_rows, int align, int capacity, unsigned* epoch_ctr,
                      const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ ids_out,
                      float* __restrict__ weights_out, int n_route_exp, int mode, int renorm, float routed_scale, int ld, int id_shift,
                      int n_local) {
  pdl_wait();
  pdl_trigger();
  __shared__ int se[kSmallPairs];
  __shared__ int cnt[512], start[512];
  const int t = threadIdx.x;
  if (t == 0 && epoch_ctr != nullptr) *epoch_ctr = *epoch_ctr + 1;
  for (int e = t; e < n_exp; e += blockDim.x) cnt[e] = 0;
  for (int r = t; r < capacity; r += blockDim.x) row_token[r] = -1;
  __syncthreads();
  if (logits != nullptr) {
    // routing fused in: a warp per token picks the top-k and leaves the ids in shared memory for the plan
    const int lane = t & 31, n_tok = n_pairs / k;
    for (int w = t >> 5; w < n_tok; w += (int)(blockDim.x >> 5)) {
      int e = route_token(logits, bias, ids_out, weights_out, w, lane, n_route_exp, k, mode, renorm, routed_scale, ld, id_shift, n_local);
      if (lane < k) {
        if (e < 0 || e >= n_exp) e = -1;
        se[w * k + lane] = e;
        if (e >= 0) atomicAdd(&cnt[e], 1);
      }
    }
  } else {
    for (int i = t; i < n_pairs; i += blockDim.x) {
      int e = ids[i];
      if (e < 0 || e >= n_exp) e = -1;
      se[i] = e;
      if (e >= 0) atomicAdd(&cnt[e], 1);
    }
  }
  __syncthreads();
  // aligned segment starts: every expert sums the padded counts of the experts before it in its region (parallel, E <= 512)
  for (int e = t; e < n_exp; e += blockDim.x) {
    const int r = e / experts_per_region, e0 = r * experts_per_region;
    int pos = 0;
    for (int i = e0; i < e; ++i) pos += (cnt[i] + align - 1) / align * align;
    start[e] = r * region_rows + pos;
    if (region_rows_used != nullptr && e == e0 + experts_per_region - 1) region_rows_used[r] = pos + (cnt[e] + align - 1) / align * align;
  }
  __syncthreads();
  for (int e = t; e < n_exp; e += blockDim.x) { seg_start[e] = start[e]; seg_count[e] = cnt[e]; }
  for (int i = t; i < n_pairs; i += blockDim.x) {
    const int e = se[i];
    if (e < 0) { pair_row[i] = -1; continue; }
    int rank = 0;
    for (int j = 0; j < i; ++j) rank += (se[j] == e);
    const int row = start[e] + rank;
    if (row < capacity) { pair_row[i] = row; row_token[row] = i / k; }
    else pair_row[i] = -1;
  }
}

// out[t, :] = sum_j w[t, j] * y[pair_row[t*k + j], :]   (bf16 in / out, fp32 accumulate, fixed order)
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pair_row, const float* __restrict__ weights,
                   __nv_bfloat16* __restrict__ out, int hidden, int k, int ld_y, const uint32_t* wait_flags, int wait_n,
                   const uint32_t* epoch_ptr, KernelStatus* st) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  __shared__ int rows[kMaxTopK];
  __shared__ float ws[kMaxTopK];
  __shared__ int failed;
  if (wait_n > 0) {
    // expert outputs are stored into `y` by the GPUs that own the experts: wait for each one's completion flag
    if (threadIdx.x == 0) {
      failed = 0;
      const uint32_t want = *epoch_ptr;
      for (int i = 0; i < wait_n; ++i) if (!wait_flag_ge(wait_flags + i, want, st, 800, i)) { failed = 1; break; }
    }
    __syncthreads();
    if (failed) return;
  }
  if (threadIdx.x < k) { rows[threadIdx.x] = pair_row[(size_t)t * k + threadIdx.x]; ws[threadIdx.x] = weights ? weights[(size_t)t * k + threadIdx.x] : 1.0f; }
  __syncthreads();
  for (int v = threadIdx.x; v < hidden / 8; v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int r = rows[j];
      if (r < 0) continue;
      const uint4 raw = *reinterpret_cast<const uint4*>(y + (size_t)r * ld_y + v * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); acc[2 * i] += ws[j] * f.x; acc[2 * i + 1] += ws[j] * f.y; }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]); o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + (size_t)t * hidden + v * 8) = o;
  }
}

// Expert-parallel combine for decode-sized batches where every rank sees all tokens: this rank's experts contribute
//   partial[t, :] = sum_{j : expert of (t, j) is local} w[t, j] * y[pair_row[t * k + j], :]        (fp32, fixed order)
// and the row goes straight into slot `rank` of the token's home GPU (tokens_per_rank consecutive tokens per rank), where the
// next RMSNorm sums the ranks' slots.  The last CTA advances the epoch and raises this rank's flag on every GPU.
struct CombineScatterArgs {
  const __nv_bfloat16* y; const int* pair_row; const float* weights;
  int hidden, k, ld_y, tokens_per_rank;
  float* slot[kMaxRanks];          // slot[p] = start of this rank's slot in rank p's heap ([tokens_per_rank, hidden] fp32)
  uint32_t* flag[kMaxRanks];       // this rank's flag in rank p's heap
  int world;
  uint32_t* epoch_ctr; unsigned* done_ctr;
};
__global__ void __launch_bounds__(256)
moe_combine_scatter_kernel(const CombineScatterArgs a) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  __shared__ int rows[kMaxTopK];
  __shared__ float ws[kMaxTopK];
  if (threadIdx.x < a.k) {
    rows[threadIdx.x] = a.pair_row[(size_t)t * a.k + threadIdx.x];
    ws[threadIdx.x] = a.weights ? a.weights[(size_t)t * a.k + threadIdx.x] : 1.0f;
  }
  __syncthreads();
  // tokens_per_rank == 0: every rank holds every token (tensor-parallel attention in front of expert-parallel experts), the row
  // goes into this rank's slot on ALL GPUs
  const bool bcast = a.tokens_per_rank == 0;
  const int home = bcast ? 0 : t / a.tokens_per_rank, lr = bcast ? t : t - home * a.tokens_per_rank;
  float* dst = a.slot[home] + (size_t)lr * a.hidden;
  for (int v = threadIdx.x; v < a.hidden / 8; v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < a.k; ++j) {
      const int r = rows[j];
      if (r < 0) continue;
      const uint4 raw = *reinterpret_cast<const uint4*>(a.y + (size_t)r * a.ld_y + v * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); acc[2 * i] += ws[j] * f.x; acc[2 * i + 1] += ws[j] * f.y; }
    }
    reinterpret_cast<float4*>(dst + v * 8)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    reinterpret_cast<float4*>(dst + v * 8)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if (bcast)
      for (int p = 1; p < a.world; ++p) {
        float* d2 = a.slot[p] + (size_t)lr * a.hidden + v * 8;
        reinterpret_cast<float4*>(d2)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        reinterpret_cast<float4*>(d2)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
      }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // Every CTA orders its rows before its arrival at GPU scope; the last one to arrive has thereby observed all of them and
    // publishes with one system-scope fence + release stores (release is cumulative), instead of a system fence per CTA.
    __threadfence();
    if (atomicAdd(a.done_ctr, 1u) == gridDim.x - 1) {
      __threadfence_system();
      *a.done_ctr = 0;
      const uint32_t e = *a.epoch_ctr + 1;
      *a.epoch_ctr = e;
      for (int p = 0; p < a.world; ++p) st_release_sys(a.flag[p], e);
    }
  }
}

// Plain row gather (bf16): out[r] = in[src[r]] or zeros when src[r] < 0.
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ in, const int* __restrict__ src, __nv_bfloat16* __restrict__ out,
                                   long rows, int hidden, int ld_in) {
  pdl_wait();
  pdl_trigger();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const int vpr = hidden >> 3;
  if (idx >= rows * vpr) return;
  const long r = idx / vpr; const int v = (int)(idx % vpr);
  const int s = src[r];
  uint4 val = make_uint4(0, 0, 0, 0);
  if (s >= 0) val = *reinterpret_cast<const uint4*>(in + (size_t)s * ld_in + v * 8);
  *reinterpret_cast<uint4*>(out + r * hidden + v * 8) = val;
}

}  // namespace gb

using namespace gb;

// Router projection + routing for m <= 64 tokens and n_exp <= 128 experts (n_exp % 16 == 0): ids / weights [m, topk] as gb_moe_route
// writes them.  x bf16 [m, k], w bf16 [n_exp, k]; k % 256 == 0, k <= 8192.
GB_API int gb_router_route(const void* x, const void* w, int m, int n_exp, int k, int ldx, int ldw, const float* bias, int* ids, float* weights,
                           int topk, int mode, int renorm, float routed_scale, int id_shift, int n_local, cudaStream_t stream) {
  if (m <= 0) return 0;
  if (n_exp > 128 || n_exp % kSlRows != 0 || k % 256 != 0 || k > 8192 || topk > kMaxTopK || topk > 32 || ldx % 8 != 0 || ldw % 8 != 0)
    return fail("router_route: unsupported shape%s");
  const size_t smem = (size_t)kSlTok * (k / 8) * sizeof(uint4);
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA_OK(cudaFuncSetAttribute(router_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSlTok * (8192 / 8) * (int)sizeof(uint4)));
    attr_set = true;
  }
  const unsigned cx = (unsigned)(n_exp / kSlRows);
  GB_CUDA_OK(launch_k_cluster(router_route_kernel, dim3(cx, (unsigned)((m + kSlTok - 1) / kSlTok)), 256, smem, stream, cx,
                              (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, m, n_exp, k, ldx, ldw, bias, ids, weights, topk, mode, renorm,
                              routed_scale, id_shift, n_local));
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_small_linear(const void* x, const void* w, float* out, int m, int n, int k, int ldx, int ldw, int ldo, cudaStream_t stream) {
  if (k % 256 || k > 8192) return fail("small_linear: k must be a multiple of 256 and <= 8192%s");
  if (m <= 0 || n <= 0) return 0;
  const size_t smem = (size_t)kSlTok * k * 2;
  static bool attr_set = false;
  if (!attr_set) { GB_CUDA_OK(cudaFuncSetAttribute(small_linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 8192 * 2)); attr_set = true; }
  launch_k(small_linear_kernel, dim3((n + kSlRows - 1) / kSlRows, (m + kSlTok - 1) / kSlTok), 256, smem, stream, (const __nv_bfloat16*)x,
           (const __nv_bfloat16*)w, out, m, n, k, ldx, ldw, ldo);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_moe_route(const float* logits, const float* bias, int* ids, float* weights, int n_tok, int n_exp, int k, int mode,
                        int renorm, float routed_scale, int ld, int id_shift, int n_local, cudaStream_t stream) {
  if (n_exp > 512 || k > kMaxTopK || k > n_exp) return fail("moe_route: need n_exp <= 512 and k <= 16%s");
  if (n_tok <= 0) return 0;
  launch_k(moe_route_kernel, (n_tok + 7) / 8, 256, 0, stream, logits, bias, ids, weights, n_tok, n_exp, k, mode, renorm, routed_scale, ld, id_shift, n_local);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

// workspace: int32 [ceil(n_pairs / 256) * n_exp].  row_token must hold `capacity` ints (set to -1 here).
GB_API int gb_moe_plan(const int* ids, int* workspace, int* seg_start, int* seg_count, int* region_rows_used, int* pair_row,
                       int* row_token, long n_pairs, int n_exp, int k, int experts_per_region, int region_rows, int align,
                       long capacity, void* epoch_ctr, cudaStream_t stream) {
  if (n_exp > 512) return fail("moe_plan: n_exp > 512%s");
  if (n_exp % experts_per_region) return fail("moe_plan: n_exp %% experts_per_region != 0%s");
  if (n_pairs <= kSmallPairs && capacity < (1l << 30)) {
    launch_k(moe_plan_small_kernel, 1, 1024, 0, stream, ids, seg_start, seg_count, region_rows_used, pair_row, row_token, (int)n_pairs,
             n_exp, k, experts_per_region, region_rows, align, (int)capacity, (unsigned*)epoch_ctr, (const float*)nullptr,
             (const float*)nullptr, (int*)nullptr, (float*)nullptr, 0, 0, 0, 1.0f, 0, 0, 0);
    GB_CUDA_OK(cudaGetLastError());
    return 0;
  }
  const int nb = (int)((n_pairs + kPlanBlock - 1) / kPlanBlock);
  GB_CUDA_OK(cudaMemsetAsync(row_token, 0xff, (size_t)capacity * sizeof(int), stream));
  if (nb > 0) launch_k(moe_hist_kernel, nb, kPlanBlock, n_exp * sizeof(int), stream, ids, workspace, n_pairs, n_exp);
  launch_k(moe_scan_kernel, n_exp, 256, 0, stream, workspace, seg_count, nb, n_exp);
  launch_k(moe_seg_kernel, 1, 512, 0, stream, seg_count, seg_start, region_rows_used, n_exp, experts_per_region, region_rows, align, (unsigned*)epoch_ctr);
  if (nb > 0) launch_k(moe_scatter_kernel, nb, kPlanBlock, 0, stream, ids, workspace, seg_start, pair_row, row_token, n_pairs, n_exp, k, capacity);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Routing and plan in one launch for decode-sized batches (n_tok * k <= 2048): logits f32 [n_tok, n_route_exp] -> ids / weights
// [n_tok, k] plus every output of gb_moe_plan over `n_exp` plan experts (= n_local when the ids are made local, else n_route_exp).
GB_API int gb_moe_route_plan(const float* logits, const float* bias, int* ids, float* weights, int n_tok, int n_route_exp, int k, int mode,
                             int renorm, float routed_scale, int ld, int id_shift, int n_local, int* seg_start, int* seg_count,
                             int* region_rows_used, int* pair_row, int* row_token, int n_exp, int experts_per_region, int region_rows,
                             int align, long capacity, void* epoch_ctr, cudaStream_t stream) {
  if (n_route_exp > 512 || n_exp > 512 || k > kMaxTopK || k > n_route_exp) return fail("moe_route_plan: need n_exp <= 512 and k <= 16%s");
  if ((long)n_tok * k > kSmallPairs || n_tok <= 0) return fail("moe_route_plan: batch too large for the single-kernel path%s");
  if (n_exp % experts_per_region) return fail("moe_route_plan: n_exp %% experts_per_region != 0%s");
  launch_k(moe_plan_small_kernel, 1, 1024, 0, stream, (const int*)nullptr, seg_start, seg_count, region_rows_used, pair_row, row_token,
           n_tok * k, n_exp, k, experts_per_region, region_rows, align, (int)capacity, (unsigned*)epoch_ctr, logits, bias, ids, weights,
           n_route_exp, mode, renorm, routed_scale, ld, id_shift, n_local);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_moe_combine(const void* y, const int* pair_row, const float* weights, void* out, int n_tok, int hidden, int k, int ld_y,
                          const void* wait_flags, int wait_n, const void* epoch_ptr, void* status, cudaStream_t stream) {
  if (hidden % 8 || k > kMaxTopK) return fail("moe_combine: hidden %% 8 != 0 or k > 16%s");
  if (n_tok <= 0) return 0;
  launch_k(moe_combine_kernel, n_tok, 256, 0, stream, (const __nv_bfloat16*)y, pair_row, weights, (__nv_bfloat16*)out, hidden, k, ld_y,
                                               (const uint32_t*)wait_flags, wait_n, (const uint32_t*)epoch_ptr, (KernelStatus*)status);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

// slots[p] / flags[p]: device pointers (as mapped in this process) of this rank's slot and flag on rank p.
GB_API int gb_moe_combine_scatter(const void* y, const int* pair_row, const float* weights, int n_tok, int hidden, int k, int ld_y,
                                  int tokens_per_rank, void* const* slots, void* const* flags, int world, void* epoch_ctr, void* done_ctr,
                                  cudaStream_t stream) {
  if (hidden % 8 || k > kMaxTopK || world > kMaxRanks) return fail("moe_combine_scatter: hidden %% 8 != 0, k > 16 or world > 8%s");
  // tokens_per_rank == 0: broadcast mode (every token row goes to every rank)
  if (n_tok <= 0 || (tokens_per_rank != 0 && n_tok != tokens_per_rank * world)) return fail("moe_combine_scatter: n_tok must be tokens_per_rank * world%s");
  CombineScatterArgs a;
  memset(&a, 0, sizeof(a));
  a.y = (const __nv_bfloat16*)y; a.pair_row = pair_row; a.weights = weights; a.hidden = hidden; a.k = k; a.ld_y = ld_y;
  a.tokens_per_rank = tokens_per_rank; a.world = world; a.epoch_ctr = (uint32_t*)epoch_ctr; a.done_ctr = (unsigned*)done_ctr;
  for (int p = 0; p < world; ++p) { a.slot[p] = (float*)slots[p]; a.flag[p] = (uint32_t*)flags[p]; }
  launch_k(moe_combine_scatter_kernel, n_tok, 256, 0, stream, a);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_gather_rows(const void* in, const int* src, void* out, long rows, int hidden, int ld_in, cudaStream_t stream) {
  if (hidden % 8) return fail("gather_rows: hidden %% 8 != 0%s");
  const long n = rows * (hidden / 8);
  if (n <= 0) return 0;
  launch_k(gather_rows_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, (const __nv_bfloat16*)in, src, (__nv_bfloat16*)out, rows, hidden, ld_in);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}
