// Token sampling on the device: greedy arg-max and temperature / top-k / top-p sampling over f32 or
// bf16 logits, one CTA per sequence.  With a vocabulary-sharded LM head every rank runs the arg-max on
// its shard and the (value, index) pairs are merged by the fabric's arg-max all-reduce.
//
// Replaces the host-side transformer_sample_topk (common/transformer.h:5415-5467: top-k by repeated
// scan, softmax with temperature, inverse-CDF draw) and sample_token of server/server_llm.c:220-284
// (temperature + top-p through an O(V^2) selection sort).  Ties resolve to the lower token id, as the
// reference's arg-max does.
#include "sm100.cuh"
#include "host_common.h"
#include <float.h>

namespace gb {

template <typename T> __device__ __forceinline__ float ld_logit(const T* p, long i);
template <> __device__ __forceinline__ float ld_logit<float>(const float* p, long i) { return p[i]; }
template <> __device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, long i) { return __bfloat162float(p[i]); }

__device__ __forceinline__ void better(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

template <typename T>
__global__ void __launch_bounds__(1024)
argmax_kernel(const T* __restrict__ logits, int* __restrict__ out_idx, float* __restrict__ out_val, int vocab, long ld, int idx_offset) {
  pdl_wait();
  pdl_trigger();
  const T* row = logits + (size_t)blockIdx.x * ld;
  float bv = -FLT_MAX; int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = ld_logit(row, i);
    v = (v == v) ? fmaxf(v, -FLT_MAX) : -FLT_MAX; /* NaN and -inf count as the lowest finite value */
    better(bv, bi, v, i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  __shared__ float sv[32]; __shared__ int si[32];
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    bv = threadIdx.x < nw ? sv[threadIdx.x] : -FLT_MAX; bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (threadIdx.x == 0) { out_idx[blockIdx.x] = bi + idx_offset; if (out_val) out_val[blockIdx.x] = bv; }
  }
}

// Final step of the arg-max fused into the LM-head GEMM: reduce [parts][rows] (value, index) pairs per row.
__global__ void __launch_bounds__(256)
argmax_pairs_kernel(const float* __restrict__ val, const int* __restrict__ idx, int* __restrict__ out_idx, float* __restrict__ out_val,
                    int parts, int rows, int idx_offset) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  float bv = -FLT_MAX; int bi = 0x7fffffff;
  for (int p = threadIdx.x; p < parts; p += blockDim.x) better(bv, bi, val[(size_t)p * rows + r], idx[(size_t)p * rows + r]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  __shared__ float sv[8]; __shared__ int si[8];
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) better(bv, bi, sv[w], si[w]);
    out_idx[r] = bi + idx_offset;
    if (out_val) out_val[r] = bv;
  }
}

// Two-stage arg-max for wide rows: stage 1 covers a row with `chunks` CTAs.
template <typename T>
__global__ void __launch_bounds__(256)
argmax_chunk_kernel(const T* __restrict__ logits, float* __restrict__ pval, int* __restrict__ pidx, int vocab, long ld, int rows) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.y, c = blockIdx.x, chunks = gridDim.x;
  const int per = (vocab + chunks - 1) / chunks;
  const int i0 = c * per, i1 = min(vocab, i0 + per);
  const T* row = logits + (size_t)r * ld;
  float bv = -FLT_MAX; int bi = 0x7fffffff;
  for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) { float v = ld_logit(row, i); v = (v == v) ? fmaxf(v, -FLT_MAX) : -FLT_MAX; /* NaN and -inf count as the lowest finite value */ better(bv, bi, v, i); }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  __shared__ float sv[8]; __shared__ int si[8];
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) better(bv, bi, sv[w], si[w]);
    pval[(size_t)c * rows + r] = bv; pidx[(size_t)c * rows + r] = bi;
  }
}

// Counter-based generator: 64-bit mix of (seed, step, row) -> uniform in [0, 1).
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t step, uint64_t row) {
  uint64_t z = seed + 0x9E3779B97F4A7C15ull * (step + 1) + 0xBF58476D1CE4E5B9ull * (row + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

constexpr int kMaxCand = 1024;

// Sampling: keep the `top_k` (<= 1024; 0 means 1024) largest logits, softmax with temperature over
// them, cut the sorted tail once the cumulative probability passes top_p, draw by inverse CDF.
// The candidates are found with a 4-pass radix select on the order-preserving integer image of the
// floats, gathered into shared memory and bitonic-sorted (descending, ties by lower id).
template <typename T>
__global__ void __launch_bounds__(1024)
sample_kernel(const T* __restrict__ logits, int* __restrict__ out_idx, int vocab, long ld, float temperature, int top_k, float top_p,
              uint64_t seed, uint64_t step, const unsigned long long* __restrict__ step_ctr) {
  pdl_wait();
  pdl_trigger();
  // A decode step replayed from a CUDA graph carries the same kernel arguments every time: the part of the step number that
  // changes lives in device memory (advanced once per step by the decode bookkeeping kernel).
  if (step_ctr != nullptr) step += *step_ctr;
  const T* row = logits + (size_t)blockIdx.x * ld;
  __shared__ unsigned hist[256];
  __shared__ unsigned s_prefix, s_remaining;
  __shared__ float cv[kMaxCand];
  __shared__ int ci[kMaxCand];
  __shared__ int s_count;
  const int kk = (top_k <= 0 || top_k > kMaxCand) ? min(kMaxCand, vocab) : min(top_k, vocab);
  auto key_of = [](float v) -> unsigned {
    v = (v == v) ? fmaxf(v, -FLT_MAX) : -FLT_MAX; /* NaN and -inf count as the lowest finite value */
    unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);        // larger float -> larger key
  };
  // radix select of the kk-th largest key
  if (threadIdx.x == 0) { s_prefix = 0; s_remaining = (unsigned)kk; }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const unsigned prefix = s_prefix;
    const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const unsigned key = key_of(ld_logit(row, i));
      if ((key & mask) == (prefix & mask)) atomicAdd(&hist[(key >> shift) & 0xff], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned rem = s_remaining; int b = 255;
      for (; b > 0; --b) { if (hist[b] >= rem) break; rem -= hist[b]; }
      s_prefix = prefix | ((unsigned)b << shift);
      s_remaining = rem;
    }
    __syncthreads();
  }
  const unsigned thr = s_prefix;          // key of the kk-th largest element
  if (threadIdx.x == 0) s_count = 0;
  __syncthreads();
  // strictly greater first, then fill with equal keys (lowest ids first is not guaranteed among equals; harmless)
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = ld_logit(row, i);
    if (key_of(v) > thr) { const int p = atomicAdd(&s_count, 1); if (p < kMaxCand) { cv[p] = v; ci[p] = i; } }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = ld_logit(row, i);
    if (key_of(v) == thr) { const int p = atomicAdd(&s_count, 1); if (p < kk) { cv[p] = v; ci[p] = i; } }
  }
  __syncthreads();
  const int n = min(s_count, kk);
  for (int i = n + threadIdx.x; i < kMaxCand; i += blockDim.x) { cv[i] = -FLT_MAX; ci[i] = 0x7fffffff; }
  __syncthreads();
  // bitonic sort, descending by value then ascending id
  for (int size = 2; size <= kMaxCand; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int i = threadIdx.x;
      const int j = i ^ stride;
      if (j > i) {
        const bool up = (i & size) == 0;
        const bool i_first = cv[i] > cv[j] || (cv[i] == cv[j] && ci[i] < ci[j]);
        if (up != i_first) { float tv = cv[i]; cv[i] = cv[j]; cv[j] = tv; int ti = ci[i]; ci[i] = ci[j]; ci[j] = ti; }
      }
      __syncthreads();
    }
  }
  if (threadIdx.x == 0) {
    const float inv_t = 1.0f / fmaxf(temperature, 1e-6f);
    const float mx = cv[0];
    float sum = 0.f;
    for (int i = 0; i < n; ++i) sum += expf((cv[i] - mx) * inv_t);
    // top-p cut
    int keep = n; float cum = 0.f;
    if (top_p < 1.0f) {
      for (int i = 0; i < n; ++i) { cum += expf((cv[i] - mx) * inv_t) / sum; if (cum >= top_p) { keep = i + 1; break; } }
    }
    float ksum = 0.f;
    for (int i = 0; i < keep; ++i) ksum += expf((cv[i] - mx) * inv_t);
    const float u = uniform01(seed, step, blockIdx.x) * ksum;
    float acc = 0.f; int pick = ci[0];
    for (int i = 0; i < keep; ++i) { acc += expf((cv[i] - mx) * inv_t); pick = ci[i]; if (acc > u) break; }
    out_idx[blockIdx.x] = pick;
  }
}

}  // namespace gb

using namespace gb;

// dtype: 0 = f32, 1 = bf16.  idx_offset is added to the winning index (first vocabulary id of a shard).
GB_API int gb_argmax(const void* logits, int* out_idx, float* out_val, int rows, int vocab, long ld, int dtype, int idx_offset, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == 0) launch_k(argmax_kernel<float>, rows, 1024, 0, stream, (const float*)logits, out_idx, out_val, vocab, ld, idx_offset);
  else launch_k(argmax_kernel<__nv_bfloat16>, rows, 1024, 0, stream, (const __nv_bfloat16*)logits, out_idx, out_val, vocab, ld, idx_offset);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_argmax_pairs(const float* val, const int* idx, int* out_idx, float* out_val, int parts, int rows, int idx_offset, cudaStream_t stream) {
  if (rows <= 0) return 0;
  launch_k(argmax_pairs_kernel, rows, 256, 0, stream, val, idx, out_idx, out_val, parts, rows, idx_offset);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Wide-row arg-max in two stages; pval / pidx are scratch of chunks * rows entries.
GB_API int gb_argmax2(const void* logits, int* out_idx, float* out_val, float* pval, int* pidx, int rows, int vocab, long ld, int dtype,
                      int idx_offset, int chunks, cudaStream_t stream) {
  if (rows <= 0) return 0;
  dim3 grid(chunks, rows);
  if (dtype == 0) launch_k(argmax_chunk_kernel<float>, grid, 256, 0, stream, (const float*)logits, pval, pidx, vocab, ld, rows);
  else launch_k(argmax_chunk_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)logits, pval, pidx, vocab, ld, rows);
  launch_k(argmax_pairs_kernel, rows, 256, 0, stream, pval, pidx, out_idx, out_val, chunks, rows, idx_offset);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

// `step_ctr` (optional, device): a 64-bit counter added to `step`, so that a captured launch draws fresh numbers at every replay.
GB_API int gb_sample(const void* logits, int* out_idx, int rows, int vocab, long ld, int dtype, float temperature, int top_k, float top_p,
                     unsigned long long seed, unsigned long long step, const void* step_ctr, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const unsigned long long* sc = (const unsigned long long*)step_ctr;
  if (dtype == 0) launch_k(sample_kernel<float>, rows, 1024, 0, stream, (const float*)logits, out_idx, vocab, ld, temperature, top_k, top_p, seed, step, sc);
  else launch_k(sample_kernel<__nv_bfloat16>, rows, 1024, 0, stream, (const __nv_bfloat16*)logits, out_idx, vocab, ld, temperature, top_k, top_p, seed, step, sc);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}
