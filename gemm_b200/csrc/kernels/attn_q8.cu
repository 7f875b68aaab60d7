// Decode attention over an INT8 KV cache, and the store that fills it.
//
// Cache format: per cache slot and KV head 128 int8 values and one f32 scale, `x = scale * q`, `scale = amax / 127` (the rule of
// the reference's kv_cache_store_q8 / attn_decode_q8, cuda/llm/cuda_llm_runner.c:220-330, with the maximum taken over the whole
// head).  Half the bytes of the bf16 cache: a decode step at long context is bound by streaming K and V.
//
// gb_kv_store_q8        bf16 K / V rows of the new tokens (as the QK-norm + RoPE kernel leaves them) -> int8 + scale at their slots
// gb_attn_decode_q8     one query token per sequence, GQA, paged block table, optional split of the KV range
//
// The attention kernel runs on the CUDA cores: the scores are integer dot products (dp4a) of the int8 keys with the query
// quantised to int8 per head, a lane per KV position; the weighted sum of the values has a lane per four output features and
// accumulates a 32-position block in half2 before it is added to the fp32 sums.  K and V scales never touch the inner loops:
// the key's scale multiplies its score, the value's scale its probability.  Work item = (sequence, KV head, split); the four
// warps of a CTA take alternate 32-position blocks and are merged through shared memory; splits are merged by the
// flash-decode combine kernel.
#include "sm100.cuh"
#include "host_common.h"
#include <cuda_fp16.h>

namespace gb {

constexpr int kQ8D = 128;          // head dim
constexpr int kQ8MaxG = 16;        // query heads per KV head

// ------------------------------------------------------------------------------------------ store
// One warp per (token, KV head, K | V): 4 values per lane.
__global__ void __launch_bounds__(256)
kv_store_q8_kernel(const __nv_bfloat16* __restrict__ k_src, const __nv_bfloat16* __restrict__ v_src, const int* __restrict__ src_slots,
                   const int* __restrict__ dst_slots, int8_t* __restrict__ kq, int8_t* __restrict__ vq, float* __restrict__ ks,
                   float* __restrict__ vs, int n_tok, int hkv, long src_rows, long dst_rows) {
  pdl_wait();
  pdl_trigger();
  const long w = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long)n_tok * hkv * 2) return;
  const int which = (int)(w & 1);
  const long th = w >> 1;
  const int t = (int)(th / hkv), h = (int)(th - (long)t * hkv);
  const long ss = src_slots != nullptr ? src_slots[t] : t, ds = dst_slots[t];
  if (ds < 0 || ds >= dst_rows || ss < 0 || ss >= src_rows) return;          // a slot of -1 means "do not store"
  const __nv_bfloat16* src = (which ? v_src : k_src) + (ss * hkv + h) * kQ8D + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(hv[0]), b = __bfloat1622float2(hv[1]);
  const float amax = warp_max(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
  const float inv = amax > 0.f ? 127.0f / amax : 0.f;
  const int q0 = max(-127, min(127, __float2int_rn(a.x * inv))), q1 = max(-127, min(127, __float2int_rn(a.y * inv)));
  const int q2 = max(-127, min(127, __float2int_rn(b.x * inv))), q3 = max(-127, min(127, __float2int_rn(b.y * inv)));
  const uint32_t pk = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
  *reinterpret_cast<uint32_t*>((which ? vq : kq) + (ds * hkv + h) * kQ8D + lane * 4) = pk;
  if (lane == 0) (which ? vs : ks)[ds * hkv + h] = amax / 127.0f;
}

// ------------------------------------------------------------------------------------------ decode attention
struct AttnQ8Args {
  const __nv_bfloat16* q;        // [B, Hq, 128], pre-scaled by softmax_scale * log2(e)
  const int8_t* kq; const int8_t* vq; const float* ks; const float* vs;   // [slots, Hkv, 128] / [slots, Hkv]
  __nv_bfloat16* out;            // [B, Hq, 128] (num_splits == 1)
  float* part_o; float* part_lse;   // [S, B, Hq, 128] / [S, B, Hq] (num_splits > 1)
  const int* kv_len; const int* block_table;
  int max_pages, page_size, n_seq, hq, hkv, num_splits, window;
  long num_slots;
  KernelStatus* status;
};

__device__ __forceinline__ float q8_exp2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

template <int G>
__global__ void __launch_bounds__(128)
attn_decode_q8_kernel(const AttnQ8Args a) {
  pdl_wait();
  pdl_trigger();
  const int item = blockIdx.x, split = blockIdx.y;
  const int b = item / a.hkv, kvh = item - b * a.hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ __align__(16) uint32_t qi8[G][32];      // the query heads of this KV head as int8, 4 per word
  __shared__ float qsc[G];
  __shared__ float m_sh[4][G], l_sh[4][G];
  __shared__ __align__(16) float o_sh[4][G][kQ8D];

  // ---- the queries: one warp per head (round robin), 4 values per lane, int8 with one scale per head
  for (int g = warp; g < G; g += 4) {
    const __nv_bfloat16* qp = a.q + ((size_t)b * a.hq + (size_t)kvh * G + g) * kQ8D + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(qp);
    const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 x = __bfloat1622float2(hv[0]), y = __bfloat1622float2(hv[1]);
    const float amax = warp_max(fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(y.x), fabsf(y.y))));
    const float inv = amax > 0.f ? 127.0f / amax : 0.f;
    const int q0 = __float2int_rn(x.x * inv), q1 = __float2int_rn(x.y * inv), q2 = __float2int_rn(y.x * inv), q3 = __float2int_rn(y.y * inv);
    qi8[g][lane] = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
    if (lane == 0) qsc[g] = amax / 127.0f;
  }
  __syncthreads();

  const int n = a.kv_len[b];
  const int first = (a.window > 0 && n > a.window) ? n - a.window : 0;      // sliding window: the last `window` positions
  const int nblk = (n + 31) >> 5;
  const int blk0 = (int)(((long)nblk * split) / a.num_splits), blk1 = (int)(((long)nblk * (split + 1)) / a.num_splits);
  const int* bt = a.block_table + (size_t)b * a.max_pages;

  float m[G], l[G], o[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) { m[g] = -INFINITY; l[g] = 0.f; o[g][0] = o[g][1] = o[g][2] = o[g][3] = 0.f; }

  for (int blk = blk0 + warp; blk < blk1; blk += 4) {
    // ---- scores: this lane's position against all G heads
    const int pos = blk * 32 + lane;
    const bool live = pos < n && pos >= first;
    long slot = 0;
    if (live) {
      const int page = bt[pos / a.page_size];
      slot = (long)page * a.page_size + pos % a.page_size;
      if (slot < 0 || slot >= a.num_slots) { report_status(a.status, ST_BAD_ARG, 1400, b, pos, (int)slot); slot = 0; }
    }
    const size_t row = ((size_t)slot * a.hkv + kvh);
    uint4 kw[8];
    const uint4* kp = reinterpret_cast<const uint4*>(a.kq + row * kQ8D);
#pragma unroll
    for (int u = 0; u < 8; ++u) kw[u] = live ? kp[u] : make_uint4(0, 0, 0, 0);
    const float ksc = live ? a.ks[row] : 0.f;
    const float vsc = live ? a.vs[row] : 0.f;
    // the values' scales ride on the probabilities, normalised by the block's largest scale so that every half-precision term
    // stays below 127 and a block sum below 4096 whatever the magnitude of V; the block sum is multiplied back in fp32
    const float vmax = warp_max(vsc);
    const float vrel = vmax > 0.f ? vsc / vmax : 0.f;
    uint32_t p[G];                                           // this position's probability x value scale per head, as a half2 pair
#pragma unroll
    for (int g = 0; g < G; ++g) {
      int dot = 0;
      const uint4* qw = reinterpret_cast<const uint4*>(qi8[g]);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint4 qv = qw[u];
        dot = __dp4a((int)kw[u].x, (int)qv.x, dot); dot = __dp4a((int)kw[u].y, (int)qv.y, dot);
        dot = __dp4a((int)kw[u].z, (int)qv.z, dot); dot = __dp4a((int)kw[u].w, (int)qv.w, dot);
      }
      const float s = live ? (float)dot * ksc * qsc[g] : -INFINITY;
      // online softmax over the warp's 32 positions
      const float m_new = fmaxf(m[g], warp_max(s));
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = q8_exp2(m[g] - m_use);             // exp2(-inf) = 0 for the first block
      const float e = live ? q8_exp2(s - m_use) : 0.f;
      l[g] = l[g] * alpha + warp_sum(e);
      m[g] = m_new;
      o[g][0] *= alpha; o[g][1] *= alpha; o[g][2] *= alpha; o[g][3] *= alpha;
      const __half2 ph = __float2half2_rn(e * vrel);
      p[g] = *reinterpret_cast<const uint32_t*>(&ph);
    }
    // ---- values: lane = features 4 lane .. 4 lane + 3; the block's 32 positions one after the other, summed in half2
    __half2 acc01[G], acc23[G];
#pragma unroll
    for (int g = 0; g < G; ++g) { acc01[g] = __float2half2_rn(0.f); acc23[g] = __float2half2_rn(0.f); }
    const int cnt = min(32, n - blk * 32);
    const __half2 bias = __halves2half2(__ushort_as_half((unsigned short)0x6480), __ushort_as_half((unsigned short)0x6480));
#pragma unroll 4
    for (int j = 0; j < cnt; ++j) {
      const long sj = __shfl_sync(0xffffffffu, slot, j);
      const uint32_t vw = *reinterpret_cast<const uint32_t*>(a.vq + ((size_t)sj * a.hkv + kvh) * kQ8D + lane * 4);
      // int8 x4 -> half2 x2: byte b ^ 0x80 into the mantissa of 1024 (0x6400 | byte = 1024 + b + 128), minus 1152
      const uint32_t x = vw ^ 0x80808080u;
      const uint32_t lo = __byte_perm(x, 0x64646464u, 0x4140), hi = __byte_perm(x, 0x64646464u, 0x4342);
      const __half2 v01 = __hsub2(*reinterpret_cast<const __half2*>(&lo), bias), v23 = __hsub2(*reinterpret_cast<const __half2*>(&hi), bias);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const uint32_t pw = __shfl_sync(0xffffffffu, p[g], j);
        const __half2 ph = *reinterpret_cast<const __half2*>(&pw);
        acc01[g] = __hfma2(ph, v01, acc01[g]);
        acc23[g] = __hfma2(ph, v23, acc23[g]);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float2 f01 = __half22float2(acc01[g]), f23 = __half22float2(acc23[g]);
      o[g][0] += f01.x * vmax; o[g][1] += f01.y * vmax; o[g][2] += f23.x * vmax; o[g][3] += f23.y * vmax;
    }
  }

  // ---- merge the four warps
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) { m_sh[warp][g] = m[g]; l_sh[warp][g] = l[g]; }
    *reinterpret_cast<float4*>(&o_sh[warp][g][lane * 4]) = make_float4(o[g][0], o[g][1], o[g][2], o[g][3]);
  }
  __syncthreads();
  for (int g = warp; g < G; g += 4) {
    float mm = fmaxf(fmaxf(m_sh[0][g], m_sh[1][g]), fmaxf(m_sh[2][g], m_sh[3][g]));
    const float m_use = (mm == -INFINITY) ? 0.f : mm;
    float lt = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float sc = q8_exp2(m_sh[w][g] - m_use);
      lt += l_sh[w][g] * sc;
      const float4 v = *reinterpret_cast<const float4*>(&o_sh[w][g][lane * 4]);
      acc.x += v.x * sc; acc.y += v.y * sc; acc.z += v.z * sc; acc.w += v.w * sc;
    }
    const float inv = lt > 0.f ? 1.0f / lt : 0.f;
    const size_t head = (size_t)b * a.hq + (size_t)kvh * G + g;
    if (a.part_o == nullptr) {
      uint2 pk;
      pk.x = pack_bf16x2(acc.x * inv, acc.y * inv); pk.y = pack_bf16x2(acc.z * inv, acc.w * inv);
      *reinterpret_cast<uint2*>(a.out + head * kQ8D + lane * 4) = pk;
    } else {
      const size_t ph = (size_t)split * a.n_seq * a.hq + head;
      *reinterpret_cast<float4*>(a.part_o + ph * kQ8D + lane * 4) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
      if (lane == 0) a.part_lse[ph] = lt > 0.f ? mm + log2f(lt) : -INFINITY;
    }
  }
}

}  // namespace gb

using namespace gb;

// k_src / v_src: bf16 [src_rows, hkv, 128]; token t is read from row src_slots[t] (t when src_slots is null) and stored quantised
// at cache slot dst_slots[t] (negative: skipped) of kq / vq [dst_rows, hkv, 128] with scales ks / vs [dst_rows, hkv].
GB_API int gb_kv_store_q8(const void* k_src, const void* v_src, const int* src_slots, const int* dst_slots, void* kq, void* vq, float* ks,
                          float* vs, int n_tok, int hkv, int head_dim, long src_rows, long dst_rows, cudaStream_t stream) {
  if (head_dim != kQ8D) return fail("kv_store_q8: head_dim must be 128%s");
  if (n_tok <= 0) return 0;
  const long warps = (long)n_tok * hkv * 2;
  launch_k(kv_store_q8_kernel, (unsigned)((warps * 32 + 255) / 256), 256, 0, stream, (const __nv_bfloat16*)k_src, (const __nv_bfloat16*)v_src,
           src_slots, dst_slots, (int8_t*)kq, (int8_t*)vq, ks, vs, n_tok, hkv, src_rows, dst_rows);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

// One query token per sequence.  q bf16 [n_seq, hq, 128] pre-scaled by softmax_scale * log2(e); out bf16 [n_seq, hq, 128], or with
// num_splits > 1 the partials part_o f32 [splits, n_seq, hq, 128] (each normalised by its own sum) and part_lse f32
// [splits, n_seq, hq] (base-2 log-sum-exp), to be merged by gb_fa_combine.
GB_API int gb_attn_decode_q8(const void* q, const void* kq, const void* vq, const float* ks, const float* vs, void* out, float* part_o,
                             float* part_lse, const int* kv_len, const int* block_table, int max_pages, int page_size, long num_slots,
                             int n_seq, int hq, int hkv, int head_dim, int num_splits, int window, void* status, cudaStream_t stream) {
  if (head_dim != kQ8D) return fail("attn_decode_q8: head_dim must be 128%s");
  if (hkv <= 0 || hq % hkv) return fail("attn_decode_q8: Hq %% Hkv != 0%s");
  const int G = hq / hkv;
  if (n_seq <= 0) return 0;
  if (num_splits < 1 || (num_splits > 1 && (part_o == nullptr || part_lse == nullptr))) return fail("attn_decode_q8: splits need partial buffers%s");
  if (num_splits == 1 && out == nullptr) return fail("attn_decode_q8: no output buffer%s");
  AttnQ8Args a;
  memset(&a, 0, sizeof(a));
  a.q = (const __nv_bfloat16*)q; a.kq = (const int8_t*)kq; a.vq = (const int8_t*)vq; a.ks = ks; a.vs = vs; a.out = (__nv_bfloat16*)out;
  a.part_o = num_splits > 1 ? part_o : nullptr; a.part_lse = num_splits > 1 ? part_lse : nullptr; a.kv_len = kv_len; a.block_table = block_table;
  a.max_pages = max_pages; a.page_size = page_size; a.n_seq = n_seq; a.hq = hq; a.hkv = hkv; a.num_splits = num_splits; a.window = window;
  a.num_slots = num_slots; a.status = (KernelStatus*)status;
  const dim3 grid((unsigned)(n_seq * hkv), (unsigned)num_splits);
#define GB_Q8(GV) if (G == GV) { launch_k(attn_decode_q8_kernel<GV>, grid, dim3(128), 0, stream, a); GB_CUDA_OK(cudaGetLastError()); return 0; }
  GB_Q8(1) GB_Q8(2) GB_Q8(4) GB_Q8(7) GB_Q8(8) GB_Q8(16)
#undef GB_Q8
  return fail("attn_decode_q8: %sgroup size %ld not built (1, 2, 4, 7, 8, 16)", "", (long)G);
}
