// Memory-bound token-wise kernels: embedding gather, RMSNorm (+residual add, + MXFP8 quantisation of
// the normalised row), per-head QK-RMSNorm + NeoX RoPE + paged KV write, SiLU-gate, MXFP8 activation
// quantiser with optional row gather, dtype casts.  All are one pass over HBM with 16-byte accesses.
//
// Replaces in the reference (cuda/llm/cuda_llm_runner.c): embed_f16:79 / batch_embed_f16:4422,
// rmsnorm_f32:87 / batch_rmsnorm_f32:8291 / add_f32:465, qknorm_f32:151, rope_neox_f32:180 /
// batch_rope_neox_f32:8056, kv_cache_store_f16:209 / batch_kv_store_f16:8206, silu_mul_f32:455,
// quantize_to_fp8_e4m3 (cuda/cuda_fp8_mma_kernels.h).  Numerics follow common/transformer.h:593-637
// (RMSNorm), :1281-1315 (QK-norm) and :1183-1219 (NeoX RoPE, inv_freq = base^(-2j/d)).
#include "sm100.cuh"
#include "host_common.h"
#include "../fabric/fabric.cuh"
#include "mxq.cuh"
#include <algorithm>

namespace gb {

struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  bf16x8 r = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(r.v[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
  bf16x8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = r;
}

// ------------------------------------------------------------------------------------------ embed
__global__ void embed_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table, __nv_bfloat16* __restrict__ out,
                             int n_tok, int hidden, int vocab) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

// ------------------------------------------------------------------------------------------ rmsnorm
// Optional all-gather in the epilogue (expert-parallel decode): the normalised bf16 row also goes to `out[p]` on every GPU p (this
// rank's region of p's gather buffer), and the CTA that finishes last advances the epoch and raises this rank's flag on
// every GPU, so the kernel that consumes the gathered rows waits on flags instead of on an exchange kernel of its own.
struct RmsBcast {
  __nv_bfloat16* out[8];
  uint32_t* flag[8];
  int world;               // 0 = off
  int partials_bf16;       // != 0: the `partials` of this launch are bf16 rows (a reduce-scatter that travelled as bf16), not f32
  uint32_t* epoch_ctr;
  unsigned* done_ctr;
};

// One CTA per row.  Optional: residual[row] += delta[row] first (the sum is written back and is the
// normalised input); optional MXFP8 output (e4m3 bytes + scale atoms) beside / instead of bf16.
template <int VPT>   // 8-element vectors per thread (hidden <= 256 * 8 * VPT)
__global__ void __launch_bounds__(256)
rmsnorm_kernel(__nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ delta, const __nv_bfloat16* __restrict__ x_in,
               const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ out, uint8_t* __restrict__ out_q,
               uint8_t* __restrict__ out_sf, int hidden, float eps, int ld_in, int ld_out, int sf32,
               const float* __restrict__ partials, int n_partials, long partial_stride, const uint32_t* wait_flags, int wait_n,
               const uint32_t* epoch_ptr, KernelStatus* st, const __nv_bfloat16* __restrict__ comb_y, const int* __restrict__ comb_rows,
               const float* __restrict__ comb_w, int comb_k, int comb_ld, int part_inner, long part_inner_stride, const RmsBcast bc) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const int nvec = hidden >> 3;
  __shared__ int c_rows[16];
  __shared__ float c_w[16];
  if (comb_y != nullptr) {
    // MoE combine fused into its consumer: delta[row] = sum_j w[row, j] * y[pair_row[row, j]]
    if (threadIdx.x < comb_k) {
      c_rows[threadIdx.x] = comb_rows[(size_t)row * comb_k + threadIdx.x];
      c_w[threadIdx.x] = comb_w != nullptr ? comb_w[(size_t)row * comb_k + threadIdx.x] : 1.0f;
    }
  }
  if (wait_n > 0) {
    // the partial sums of a tensor-parallel projection are stored here by the peers: wait for every rank's flag
    __shared__ int failed;
    if (threadIdx.x == 0) {
      failed = 0;
      const uint32_t want = *epoch_ptr;
      for (int i = 0; i < wait_n; ++i) if (!wait_flag_ge(wait_flags + i, want, st, 900, i)) { failed = 1; break; }
    }
    __syncthreads();
    if (failed) {
      // nothing is published (the consumers' own waits run out), but the arrival counter is left at zero for the next launch
      if (bc.world > 0 && threadIdx.x == 0 && atomicAdd(bc.done_ctr, 1u) == gridDim.x - 1) *bc.done_ctr = 0;
      return;
    }
  }
  if (comb_y != nullptr) __syncthreads();
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
      if (residual != nullptr) {
        float r[8], d[8];
        load8(residual + (size_t)row * ld_in + vi * 8, r);
        if (partials != nullptr) {
          // all-reduce fused into its consumer: sum the ranks' fp32 partials in rank order (bit-identical everywhere)
#pragma unroll
          for (int j = 0; j < 8; ++j) d[j] = 0.f;
          // partial p = (rank, K split): ranks are partial_stride apart, the splits of one rank part_inner_stride
          if (bc.partials_bf16) {
            // a reduce-scatter that travelled as bf16 rows (prefill-sized tensor parallelism)
            for (int p = 0; p < n_partials; ++p) {
              float t8[8];
              load8(reinterpret_cast<const __nv_bfloat16*>(partials) + (size_t)p * partial_stride + (size_t)row * hidden + vi * 8, t8);
#pragma unroll
              for (int j = 0; j < 8; ++j) d[j] += t8[j];
            }
          } else {
            for (int p = 0; p < n_partials; ++p) {
              const int po = p / part_inner, pi = p - po * part_inner;
              const float4* src = reinterpret_cast<const float4*>(partials + (size_t)po * partial_stride + (size_t)pi * part_inner_stride +
                                                                  (size_t)row * hidden + vi * 8);
              const float4 a = src[0], b = src[1];
              d[0] += a.x; d[1] += a.y; d[2] += a.z; d[3] += a.w; d[4] += b.x; d[5] += b.y; d[6] += b.z; d[7] += b.w;
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) r[j] = __bfloat162float(__float2bfloat16(r[j] + d[j]));
          store8(residual + (size_t)row * ld_in + vi * 8, r);
        } else if (comb_y != nullptr) {
#pragma unroll
          for (int j = 0; j < 8; ++j) d[j] = 0.f;
          for (int c = 0; c < comb_k; ++c) {
            const int cr = c_rows[c];
            if (cr < 0) continue;
            float yv[8];
            load8(comb_y + (size_t)cr * comb_ld + vi * 8, yv);
#pragma unroll
            for (int j = 0; j < 8; ++j) d[j] += c_w[c] * yv[j];
          }
          // same roundings as the unfused pair of kernels: the combined row is bf16, then the residual sum is bf16
#pragma unroll
          for (int j = 0; j < 8; ++j) r[j] = __bfloat162float(__float2bfloat16(r[j] + __bfloat162float(__float2bfloat16(d[j]))));
          store8(residual + (size_t)row * ld_in + vi * 8, r);
        } else if (delta != nullptr) {
          load8(delta + (size_t)row * ld_in + vi * 8, d);
#pragma unroll
          for (int j = 0; j < 8; ++j) r[j] = __bfloat162float(__float2bfloat16(r[j] + d[j]));
          store8(residual + (size_t)row * ld_in + vi * 8, r);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = r[j];
      } else {
        load8(x_in + (size_t)row * ld_in + vi * 8, v[i]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  __shared__ float red[8];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float scale = rsqrtf(tot / (float)hidden + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * 256;
    float w[8], y[8];
    float amax = 0.f;
    if (vi < nvec) {
      load8(weight + vi * 8, w);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        y[j] = __bfloat162float(__float2bfloat16(v[i][j] * scale * w[j]));
        amax = fmaxf(amax, fabsf(y[j]));
      }
      if (out != nullptr) store8(out + (size_t)row * ld_out + vi * 8, y);
      for (int p = 0; p < bc.world; ++p) store8(bc.out[p] + (size_t)row * hidden + vi * 8, y);
    }
    if (out_q != nullptr) {
      // 4 consecutive threads hold one 32-element block
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      if (vi < nvec) {
        const int e = e8m0_amax(amax);
        const float inv = __uint_as_float((uint32_t)(254 - e) << 23);
        uint8_t q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { __nv_fp8_e4m3 f(y[j] * inv); q[j] = *reinterpret_cast<uint8_t*>(&f); }
        *reinterpret_cast<uint2*>(out_q + (size_t)row * hidden + vi * 8) = *reinterpret_cast<uint2*>(q);
        if ((vi & 3) == 0) out_sf[sf_atom_offset(row, vi >> 2, hidden >> 7, sf32)] = (uint8_t)e;
      }
    }
  }
  if (bc.world > 0) {
    __syncthreads();
    if (threadIdx.x == 0) {
      // every CTA orders its rows before its arrival; the last one publishes with one system fence + release stores
      __threadfence();
      if (atomicAdd(bc.done_ctr, 1u) == gridDim.x - 1) {
        __threadfence_system();
        *bc.done_ctr = 0;
        const uint32_t e = *bc.epoch_ctr + 1;
        *bc.epoch_ctr = e;
        for (int p = 0; p < bc.world; ++p) st_release_sys(bc.flag[p], e);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ qk-norm + rope + kv write
// One warp per (token, head) over the fused QKV row [Hq*D | Hkv*D | Hkv*D].  Q heads: RMSNorm over D
// (weight q_w, skipped if null), NeoX rotation of the first 2*rope_pairs dims, written to q_out.
// K heads: same with k_w, written into the paged cache slot of the token; V heads: copied to the cache.
// Cache layout: [num_slots, Hkv, D] for K and for V, slot = block * block_size + offset.
template <int D>
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
                    const __nv_bfloat16* __restrict__ q_w, const __nv_bfloat16* __restrict__ k_w, __nv_bfloat16* __restrict__ q_out,
                    __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int n_tok, int hq, int hkv,
                    int rope_pairs, float theta, float eps, int ld_qkv, float q_scale, const float2* __restrict__ rope_tab, int tab_len,
                    const int* __restrict__ pos3, int sec_h3, int sec_w3) {
  pdl_wait();
  pdl_trigger();
  constexpr int EPL = D / 32;            // elements per lane, index = lane + 32 * i
  // (cos, sin) of pair j at this token: from the precomputed table [position][pair] when there is one (exact range reduction,
  // no powf / sincosf in the hot path), else computed.  With M-RoPE (pos3 = [3][n_tok] temporal / height / width positions)
  // pair j takes the position of section j % 3 while j is inside that section's interleaved range, else the temporal one
  // (common/transformer.h:1227-1251).
  auto cos_sin = [&](int tok, int j, float denom, float& c, float& s) {
    int p = positions[tok];
    if (pos3 != nullptr) {
      const int m3 = j % 3;
      const int which = (m3 == 1 && j < sec_h3) ? 1 : (m3 == 2 && j < sec_w3) ? 2 : 0;
      p = pos3[(size_t)which * n_tok + tok];
    }
    if (rope_tab != nullptr && p >= 0 && p < tab_len) {
      const float2 cs = rope_tab[(size_t)p * rope_pairs + j];
      c = cs.x; s = cs.y;
    } else {
      const float inv_freq = powf(theta, -2.0f * (float)j / denom);
      sincosf((float)p * inv_freq, &s, &c);
    }
  };
  const int heads = hq + 2 * hkv;
  const long gw = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (gw >= (long)n_tok * heads) return;
  const int lane = threadIdx.x & 31;
  const int t = (int)(gw / heads), h = (int)(gw % heads);
  const __nv_bfloat16* src = qkv + (size_t)t * ld_qkv + (size_t)h * D;
  float x[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) x[i] = __bfloat162float(src[lane + 32 * i]);
  const bool is_q = h < hq, is_k = !is_q && h < hq + hkv;
  if (is_q || is_k) {
    const __nv_bfloat16* w = is_q ? q_w : k_w;
    if (w != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) ss += x[i] * x[i];
      ss = warp_sum(ss);
      const float sc = rsqrtf(ss / (float)D + eps);
#pragma unroll
      for (int i = 0; i < EPL; ++i) x[i] = x[i] * sc * __bfloat162float(w[lane + 32 * i]);
    }
    // pair (j, j + rope_pairs) for j < rope_pairs; with full rotary rope_pairs = D/2 = 32 * EPL/2
    if (2 * rope_pairs == D) {
#pragma unroll
      for (int i = 0; i < EPL / 2; ++i) {
        const int j = lane + 32 * i;
        float s, c;
        cos_sin(t, j, (float)D, c, s);
        const float a = x[i], b = x[i + EPL / 2];
        x[i] = a * c - b * s;
        x[i + EPL / 2] = a * s + b * c;
      }
    } else {
      // partial rotary: pairs may straddle lanes -> go through shuffles of the partner element
      const float rd = 2.0f * (float)rope_pairs;
      float xo[EPL];
#pragma unroll
      for (int i = 0; i < EPL; ++i) xo[i] = x[i];
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const int idx = lane + 32 * i;
        const bool lo = idx < rope_pairs, hi = idx >= rope_pairs && idx < 2 * rope_pairs;
        const int pidx = lo ? idx + rope_pairs : idx - rope_pairs;
        float partner = 0.f;
#pragma unroll
        for (int ii = 0; ii < EPL; ++ii) {
          const float cand = __shfl_sync(0xffffffffu, xo[ii], pidx & 31);
          if ((pidx >> 5) == ii) partner = cand;
        }
        if (lo || hi) {
          const int j = lo ? idx : idx - rope_pairs;
          float s, c;
          cos_sin(t, j, rd, c, s);
          x[i] = lo ? (xo[i] * c - partner * s) : (partner * s + xo[i] * c);
        }
      }
    }
  }
  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out + ((size_t)t * hq + h) * D;
#pragma unroll
    for (int i = 0; i < EPL; ++i) x[i] *= q_scale;
  } else {
    const int slot = slots[t];
    if (slot < 0) return;
    const int kh = is_k ? h - hq : h - hq - hkv;
    dst = (is_k ? k_cache : v_cache) + ((size_t)slot * hkv + kh) * D;
  }
#pragma unroll
  for (int i = 0; i < EPL; ++i) dst[lane + 32 * i] = __float2bfloat16(x[i]);
}

// The same for head_dim 128 with full rotary (the Qwen3 shape), 16 lanes per (token, head): lane l holds elements 4l..4l+3 and
// 64+4l..64+4l+3, i.e. both halves of four NeoX pairs, so that every access is an 8-byte vector and a warp moves 256
// contiguous bytes per instruction (the generic kernel moves 2 bytes per lane).
__global__ void __launch_bounds__(256)
qk_norm_rope128_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
                       const __nv_bfloat16* __restrict__ q_w, const __nv_bfloat16* __restrict__ k_w, __nv_bfloat16* __restrict__ q_out,
                       __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int n_tok, int hq, int hkv,
                       float theta, float eps, int ld_qkv, float q_scale, const float2* __restrict__ rope_tab, int tab_len,
                       const int* __restrict__ pos3, int sec_h3, int sec_w3, const float* __restrict__ part, int n_part,
                       long part_stride) {
  pdl_wait();
  pdl_trigger();
  constexpr int D = 128, PAIRS = 64;
  const int heads = hq + 2 * hkv;
  const long total = (long)n_tok * heads;
  long gh = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
  const bool active = gh < total;
  if (!active) gh = total - 1;                 // the idle half of the last warp computes along (shuffles use the full mask)
  const int l = threadIdx.x & 15;
  const int t = (int)(gh / heads), h = (int)(gh % heads);
  const __nv_bfloat16* src = qkv + (size_t)t * ld_qkv + (size_t)h * D;
  auto unpack4 = [](uint2 v, float* f) {
    const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&v);
    const float2 a = __bfloat1622float2(hp[0]), b = __bfloat1622float2(hp[1]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  };
  float xa[4], xb[4];
  if (part != nullptr) {
    // the projection arrives as K-split fp32 partial sums [n_part][n_tok][ld_qkv]: summed here in split order
#pragma unroll
    for (int i = 0; i < 4; ++i) { xa[i] = 0.f; xb[i] = 0.f; }
    const float* pp = part + (size_t)t * ld_qkv + (size_t)h * D + 4 * l;
    for (int p = 0; p < n_part; ++p, pp += part_stride) {
      const float4 a = *reinterpret_cast<const float4*>(pp), b = *reinterpret_cast<const float4*>(pp + PAIRS);
      xa[0] += a.x; xa[1] += a.y; xa[2] += a.z; xa[3] += a.w; xb[0] += b.x; xb[1] += b.y; xb[2] += b.z; xb[3] += b.w;
    }
  } else {
    unpack4(*reinterpret_cast<const uint2*>(src + 4 * l), xa);
    unpack4(*reinterpret_cast<const uint2*>(src + PAIRS + 4 * l), xb);
  }
  const bool is_q = h < hq, is_k = !is_q && h < hq + hkv;
  if (is_q || is_k) {
    const __nv_bfloat16* w = is_q ? q_w : k_w;
    if (w != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) ss += xa[i] * xa[i] + xb[i] * xb[i];
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float sc = rsqrtf(ss / (float)D + eps);
      float wa[4], wb[4];
      unpack4(*reinterpret_cast<const uint2*>(w + 4 * l), wa);
      unpack4(*reinterpret_cast<const uint2*>(w + PAIRS + 4 * l), wb);
#pragma unroll
      for (int i = 0; i < 4; ++i) { xa[i] = xa[i] * sc * wa[i]; xb[i] = xb[i] * sc * wb[i]; }
    }
    float c[4], sn[4];
    const int p0 = positions[t];
    if (pos3 == nullptr && rope_tab != nullptr && p0 >= 0 && p0 < tab_len) {
      const float4* tp = reinterpret_cast<const float4*>(rope_tab + (size_t)p0 * PAIRS + 4 * l);
      const float4 u = tp[0], v = tp[1];
      c[0] = u.x; sn[0] = u.y; c[1] = u.z; sn[1] = u.w; c[2] = v.x; sn[2] = v.y; c[3] = v.z; sn[3] = v.w;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = 4 * l + i;
        int p = p0;
        if (pos3 != nullptr) {
          const int m3 = j % 3;
          const int which = (m3 == 1 && j < sec_h3) ? 1 : (m3 == 2 && j < sec_w3) ? 2 : 0;
          p = pos3[(size_t)which * n_tok + t];
        }
        if (rope_tab != nullptr && p >= 0 && p < tab_len) { const float2 cs = rope_tab[(size_t)p * PAIRS + j]; c[i] = cs.x; sn[i] = cs.y; }
        else { const float inv_freq = powf(theta, -2.0f * (float)j / (float)D); sincosf((float)p * inv_freq, &sn[i], &c[i]); }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = xa[i], b = xb[i];
      xa[i] = a * c[i] - b * sn[i];
      xb[i] = a * sn[i] + b * c[i];
    }
  }
  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out + ((size_t)t * hq + h) * D;
#pragma unroll
    for (int i = 0; i < 4; ++i) { xa[i] *= q_scale; xb[i] *= q_scale; }
  } else {
    const int slot = slots[t];
    if (slot < 0) return;
    const int kh = is_k ? h - hq : h - hq - hkv;
    dst = (is_k ? k_cache : v_cache) + ((size_t)slot * hkv + kh) * D;
  }
  if (!active) return;
  uint2 oa, ob;
  oa.x = pack_bf16x2(xa[0], xa[1]); oa.y = pack_bf16x2(xa[2], xa[3]);
  ob.x = pack_bf16x2(xb[0], xb[1]); ob.y = pack_bf16x2(xb[2], xb[3]);
  *reinterpret_cast<uint2*>(dst + 4 * l) = oa;
  *reinterpret_cast<uint2*>(dst + PAIRS + 4 * l) = ob;
}

// ------------------------------------------------------------------------------------------ silu * up
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, long rows, int inter, int ld) {
  pdl_wait();
  pdl_trigger();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const int vec_per_row = inter >> 3;
  if (idx >= rows * vec_per_row) return;
  const long r = idx / vec_per_row;
  const int c = (int)(idx % vec_per_row) * 8;
  float g[8], u[8], y[8];
  load8(gate_up + r * ld + c, g);
  load8(gate_up + r * ld + inter + c, u);
#pragma unroll
  for (int j = 0; j < 8; ++j) y[j] = g[j] / (1.0f + __expf(-g[j])) * u[j];
  store8(out + r * inter + c, y);
}

// SiLU(gate) * up followed by MXFP8 quantisation: gate_up [rows, 2 * inter] bf16 -> e4m3 bytes [rows, inter] + scale atoms.
// Used after a plain (single-accumulator) gate/up GEMM for prefill-sized expert batches, where the two-accumulator GEMM
// with this math in its epilogue cannot double-buffer its accumulators in TMEM.  Rows whose row_valid entry is negative
// (padding of the expert-sorted buffer) are skipped.  8 elements per thread, 4 threads share a scale.
constexpr int kSiluU = 2;        // items per thread: the gate and up vectors of both are requested before the first use
__global__ void __launch_bounds__(256)
silu_mul_quant_kernel(const __nv_bfloat16* __restrict__ gate_up, const int* __restrict__ row_valid, uint8_t* __restrict__ out_q,
                      uint8_t* __restrict__ out_sf, long rows, int inter, int ld, int sf32) {
  pdl_wait();
  pdl_trigger();
  const int vec_per_row = inter >> 3;
  const long base = (long)blockIdx.x * (256 * kSiluU) + threadIdx.x;
  bf16x8 gr[kSiluU], ur[kSiluU];
  long rr[kSiluU];
  int vv[kSiluU];
  bool live[kSiluU];
#pragma unroll
  for (int u = 0; u < kSiluU; ++u) {
    const long idx = base + u * 256;
    rr[u] = idx / vec_per_row;
    vv[u] = (int)(idx - rr[u] * vec_per_row);
    live[u] = rr[u] < rows && (row_valid == nullptr || row_valid[rr[u]] >= 0);
    if (live[u]) {
      gr[u] = *reinterpret_cast<const bf16x8*>(gate_up + rr[u] * ld + vv[u] * 8);
      ur[u] = *reinterpret_cast<const bf16x8*>(gate_up + rr[u] * ld + inter + vv[u] * 8);
    }
  }
#pragma unroll
  for (int u = 0; u < kSiluU; ++u) {
    float y[8];
    float amax = 0.f;
    if (live[u]) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 g = __bfloat1622float2(gr[u].v[j]), up = __bfloat1622float2(ur[u].v[j]);
        y[2 * j] = __fdividef(g.x, 1.0f + __expf(-g.x)) * up.x;
        y[2 * j + 1] = __fdividef(g.y, 1.0f + __expf(-g.y)) * up.y;
        amax = fmaxf(amax, fmaxf(fabsf(y[2 * j]), fabsf(y[2 * j + 1])));
      }
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (!live[u]) continue;
    const int e = e8m0_amax(amax);
    const float inv = __uint_as_float((uint32_t)(254 - e) << 23);
    uint2 q;            // two values per conversion instruction
    q.x = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(y[0] * inv, y[1] * inv), __NV_SATFINITE, __NV_E4M3) |
          ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(y[2] * inv, y[3] * inv), __NV_SATFINITE, __NV_E4M3) << 16);
    q.y = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(y[4] * inv, y[5] * inv), __NV_SATFINITE, __NV_E4M3) |
          ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(y[6] * inv, y[7] * inv), __NV_SATFINITE, __NV_E4M3) << 16);
    *reinterpret_cast<uint2*>(out_q + rr[u] * inter + vv[u] * 8) = q;
    if ((vv[u] & 3) == 0) out_sf[sf_atom_offset(rr[u], vv[u] >> 2, inter >> 7, sf32)] = (uint8_t)e;
  }
}

// SiLU(gate) * up from K-split partial sums: part f32 [n_part][rows][2 * inter] (gate columns first).  The slabs are added in
// split order; the result goes out as bf16 and / or as MXFP8 with scale atoms.  8 elements per thread, 4 threads share a scale.
__global__ void __launch_bounds__(256)
silu_mul_partials_kernel(const float* __restrict__ part, int n_part, long part_stride, __nv_bfloat16* __restrict__ out, uint8_t* __restrict__ out_q,
                         uint8_t* __restrict__ out_sf, long rows, int inter, int sf32) {
  pdl_wait();
  pdl_trigger();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const int vec_per_row = inter >> 3;
  const long r = idx / vec_per_row;
  const int vi = (int)(idx - r * vec_per_row);
  const bool live = r < rows;
  float y[8];
  float amax = 0.f;
  if (live) {
    float g[8], u[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { g[j] = 0.f; u[j] = 0.f; }
    const float* pp = part + r * (2L * inter) + vi * 8;
    for (int p = 0; p < n_part; ++p, pp += part_stride) {
      const float4 g0 = *reinterpret_cast<const float4*>(pp), g1 = *reinterpret_cast<const float4*>(pp + 4);
      const float4 u0 = *reinterpret_cast<const float4*>(pp + inter), u1 = *reinterpret_cast<const float4*>(pp + inter + 4);
      g[0] += g0.x; g[1] += g0.y; g[2] += g0.z; g[3] += g0.w; g[4] += g1.x; g[5] += g1.y; g[6] += g1.z; g[7] += g1.w;
      u[0] += u0.x; u[1] += u0.y; u[2] += u0.z; u[3] += u0.w; u[4] += u1.x; u[5] += u1.y; u[6] += u1.z; u[7] += u1.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { y[j] = g[j] / (1.0f + __expf(-g[j])) * u[j]; amax = fmaxf(amax, fabsf(y[j])); }
    if (out != nullptr) store8(out + r * inter + vi * 8, y);
  }
  if (out_q == nullptr) return;
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  if (!live) return;
  const int e = e8m0_amax(amax);
  const float inv = __uint_as_float((uint32_t)(254 - e) << 23);
  uint8_t q[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { __nv_fp8_e4m3 f(y[j] * inv); q[j] = *reinterpret_cast<uint8_t*>(&f); }
  *reinterpret_cast<uint2*>(out_q + r * inter + vi * 8) = *reinterpret_cast<uint2*>(q);
  if ((vi & 3) == 0) out_sf[sf_atom_offset(r, vi >> 2, inter >> 7, sf32)] = (uint8_t)e;
}

// ------------------------------------------------------------------------------------------ mxfp8 quantiser
// out row r <- in row (src_rows ? src_rows[r] : r); rows whose source is negative are zero-filled with
// scale 1.  One warp per 256 elements: lane holds 8 elements, 4 lanes share a scale.
constexpr int kMxQuantU = 4;     // vectors per thread: all loads of a thread are issued before the first use
__global__ void __launch_bounds__(256)
mx_quant_kernel(const __nv_bfloat16* __restrict__ in, const int* __restrict__ src_rows, uint8_t* __restrict__ out_q,
                uint8_t* __restrict__ out_sf, long out_rows, int k, int ld_in, int sf32) {
  pdl_wait();
  pdl_trigger();
  const int vec_per_row = k >> 3;
  const long total = out_rows * vec_per_row;
  const long base = (long)blockIdx.x * (256 * kMxQuantU) + threadIdx.x;
  bf16x8 raw[kMxQuantU];
  long rr[kMxQuantU];
  int vv[kMxQuantU];
  bool act[kMxQuantU], have[kMxQuantU];
#pragma unroll
  for (int u = 0; u < kMxQuantU; ++u) {
    const long idx = base + u * 256;
    act[u] = idx < total;
    rr[u] = act[u] ? idx / vec_per_row : 0;
    vv[u] = act[u] ? (int)(idx - rr[u] * vec_per_row) : 0;
    long src = rr[u];
    if (act[u] && src_rows != nullptr) src = src_rows[rr[u]];
    have[u] = act[u] && src >= 0;
    if (have[u]) raw[u] = *reinterpret_cast<const bf16x8*>(in + src * ld_in + vv[u] * 8);
  }
#pragma unroll
  for (int u = 0; u < kMxQuantU; ++u) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t2 = have[u] ? __bfloat1622float2(raw[u].v[j]) : make_float2(0.f, 0.f);
      v[2 * j] = t2.x; v[2 * j + 1] = t2.y;
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (!act[u]) continue;
    const int e = e8m0_amax(amax);
    const float inv = __uint_as_float((uint32_t)(254 - e) << 23);
    uint2 q;
    q.x = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv, v[1] * inv), __NV_SATFINITE, __NV_E4M3) |
          ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv, v[3] * inv), __NV_SATFINITE, __NV_E4M3) << 16);
    q.y = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(v[4] * inv, v[5] * inv), __NV_SATFINITE, __NV_E4M3) |
          ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(v[6] * inv, v[7] * inv), __NV_SATFINITE, __NV_E4M3) << 16);
    *reinterpret_cast<uint2*>(out_q + rr[u] * k + vv[u] * 8) = q;
    if ((vv[u] & 3) == 0) out_sf[sf_atom_offset(rr[u], vv[u] >> 2, k >> 7, sf32)] = (uint8_t)e;
  }
}

// Gathering variant, one warp per output row: padding rows (source < 0) are skipped after one load, so a mostly
// empty expert-sorted buffer costs almost nothing.  Needs k % 256 == 0; the output must be pre-zeroed.
__global__ void __launch_bounds__(256)
mx_quant_rows_kernel(const __nv_bfloat16* __restrict__ in, const int* __restrict__ src_rows, uint8_t* __restrict__ out_q,
                     uint8_t* __restrict__ out_sf, long out_rows, int k, int ld_in, int sf32) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long warp0 = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, n_warps = ((long)gridDim.x * blockDim.x) >> 5;
  const int vec_per_row = k >> 3;
  for (long r = warp0; r < out_rows; r += n_warps) {
    const int src = src_rows[r];
    if (src < 0) continue;
    for (int vi = lane; vi < vec_per_row; vi += 32) {
      float v[8];
      load8(in + (size_t)src * ld_in + vi * 8, v);
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const int e = e8m0_amax(amax);
      const float inv = __uint_as_float((uint32_t)(254 - e) << 23);
      uint8_t q[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) { __nv_fp8_e4m3 f(v[j] * inv); q[j] = *reinterpret_cast<uint8_t*>(&f); }
      *reinterpret_cast<uint2*>(out_q + r * k + vi * 8) = *reinterpret_cast<uint2*>(q);
      if ((vi & 3) == 0) out_sf[sf_atom_offset(r, vi >> 2, k >> 7, sf32)] = (uint8_t)e;
    }
  }
}

// Gather of rows that are already MXFP8: output row r <- input row src_rows[r] (bytes and scales; the scale layouts of the
// two sides may differ), negative sources are skipped.  The MoE dispatch of a layer whose RMSNorm already produced the
// quantised tokens: every token is quantised once instead of once per selected expert.  One warp per output row, k % 128 == 0.
__global__ void __launch_bounds__(256)
mx_gather_rows_kernel(const uint8_t* __restrict__ in_q, const uint8_t* __restrict__ in_sf, const int* __restrict__ src_rows,
                      uint8_t* __restrict__ out_q, uint8_t* __restrict__ out_sf, long out_rows, int k, int in_sf32, int out_sf32) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long warp0 = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, n_warps = ((long)gridDim.x * blockDim.x) >> 5;
  const int vecs = k >> 4, k_atoms = k >> 7;
  // two rows per warp and step; the loads of both rows (4 vectors per lane and row at a time) are issued before the stores
  for (long r0 = warp0 * 2; r0 < out_rows; r0 += n_warps * 2) {
    int src[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) src[u] = (r0 + u < out_rows) ? src_rows[r0 + u] : -1;
    for (int v0 = 0; v0 < vecs; v0 += 128) {
      uint4 buf[2][4];
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int vi = v0 + lane + 32 * i;
          if (src[u] >= 0 && vi < vecs) buf[u][i] = reinterpret_cast<const uint4*>(in_q + (size_t)src[u] * k)[vi];
        }
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int vi = v0 + lane + 32 * i;
          if (src[u] >= 0 && vi < vecs) reinterpret_cast<uint4*>(out_q + (size_t)(r0 + u) * k)[vi] = buf[u][i];
        }
    }
    // the four scales of one 128-element block are four consecutive bytes in either layout
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (src[u] < 0) continue;
      for (int a = lane; a < k_atoms; a += 32)
        *reinterpret_cast<uint32_t*>(out_sf + sf_atom_offset(r0 + u, a * 4, k_atoms, out_sf32)) =
            *reinterpret_cast<const uint32_t*>(in_sf + sf_atom_offset(src[u], a * 4, k_atoms, in_sf32));
    }
  }
}

// ------------------------------------------------------------------------------------------ KV page copy
// cache page dst[i] <- cache page src[i] (16-byte vectors): the copy-on-write of a forked sequence's tail page
// (the reference's per-sequence KV arrays are copied whole on a clone: common/glm5.h:640).
__global__ void __launch_bounds__(256)
kv_copy_pages_kernel(uint4* __restrict__ cache, const int* __restrict__ src, const int* __restrict__ dst, int n_pages, long vec_per_page) {
  pdl_wait();
  pdl_trigger();
  const int s = src[blockIdx.x], d = dst[blockIdx.x];
  if (s < 0 || d < 0 || s >= n_pages || d >= n_pages || s == d) return;
  const uint4* sp = cache + (size_t)s * vec_per_page;
  uint4* dp = cache + (size_t)d * vec_per_page;
  for (long i = (long)blockIdx.y * blockDim.x + threadIdx.x; i < vec_per_page; i += (long)gridDim.y * blockDim.x) dp[i] = sp[i];
}

// ------------------------------------------------------------------------------------------ INT8 KV codec
// rows of head_dim bf16 values (one per cache slot and KV head) <-> int8 with one f32 scale per row: scale = amax / 127,
// q = round(x / scale) clamped to [-127, 127] (the rule of kv_cache_store_q8, cuda/llm/cuda_llm_runner.c:220-241, with the maximum
// taken over the whole head; the reference's reduction only spans a warp).  One warp per row, head_dim % 32 == 0, <= 256.
__global__ void __launch_bounds__(256)
kv_quant_q8_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scale, long rows, int d) {
  pdl_wait();
  pdl_trigger();
  const long r = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (r >= rows) return;
  const int lane = threadIdx.x & 31, per = d >> 5;
  float v[8];
  float amax = 0.f;
  for (int i = 0; i < per; ++i) { v[i] = __bfloat162float(x[r * d + lane * per + i]); amax = fmaxf(amax, fabsf(v[i])); }
  amax = warp_max(amax);
  const float inv = amax > 0.f ? 127.0f / amax : 0.f;
  if (lane == 0) scale[r] = amax / 127.0f;
  for (int i = 0; i < per; ++i) q[r * d + lane * per + i] = (int8_t)max(-127, min(127, __float2int_rn(v[i] * inv)));
}

__global__ void __launch_bounds__(256)
kv_dequant_q8_kernel(const int8_t* __restrict__ q, const float* __restrict__ scale, __nv_bfloat16* __restrict__ x, long rows, int d) {
  pdl_wait();
  pdl_trigger();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * d) return;
  x[i] = __float2bfloat16((float)q[i] * scale[i / d]);
}

// ------------------------------------------------------------------------------------------ casts
__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long n) {
  pdl_wait();
  pdl_trigger();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16(in[i]);
}

// Decode bookkeeping kept on the device so that a captured step can be replayed without the host:
// every live sequence advances by one position; its next slot comes from the block table.
__global__ void decode_advance_kernel(int* __restrict__ positions, int* __restrict__ kv_len, int* __restrict__ slots,
                                      const int* __restrict__ block_table, const int* __restrict__ live, int max_pages, int page_size, int n,
                                      unsigned long long* __restrict__ step_ctr) {
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b == 0 && step_ctr != nullptr) *step_ctr += 1;       // the step number the sampler of the NEXT step reads
  if (b >= n) return;
  if (live != nullptr && live[b] == 0) return;
  const int p = positions[b] + 1;
  positions[b] = p;
  kv_len[b] = p + 1;
  const int page = block_table[(size_t)b * max_pages + min(p / page_size, max_pages - 1)];
  slots[b] = page * page_size + p % page_size;
}

// The same under context parallelism (the positions of a sequence are dealt to the ranks page by page: page g of a sequence lives on
// rank g % world as that rank's page g / world): positions stay global, kv_len is the number of positions up to and including the new one
// that THIS rank stores, the slot is -1 where another rank stores the new position (the rope kernel then skips the cache write).
__global__ void decode_advance_cp_kernel(int* __restrict__ positions, int* __restrict__ kv_len, int* __restrict__ slots,
                                         const int* __restrict__ block_table, int max_pages, int page_size, int n, int world, int rank,
                                         unsigned long long* __restrict__ step_ctr) {
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b == 0 && step_ctr != nullptr) *step_ctr += 1;
  if (b >= n) return;
  const int p = positions[b] + 1;
  positions[b] = p;
  const int round = page_size * world;
  const int rem = (p + 1) % round - rank * page_size;
  kv_len[b] = (p + 1) / round * page_size + min(max(rem, 0), page_size);
  const int g = p / page_size;
  if (g % world != rank) {
    slots[b] = -1;
    return;
  }
  const int page = block_table[(size_t)b * max_pages + min(g / world, max_pages - 1)];
  slots[b] = page * page_size + p % page_size;
}

}  // namespace gb

using namespace gb;

GB_API int gb_decode_advance_cp(int* positions, int* kv_len, int* slots, const int* block_table, int max_pages, int page_size, int n,
                                int world, int rank, void* step_ctr, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (world < 1 || rank < 0 || rank >= world) return fail("decode_advance_cp: bad rank%s");
  launch_k(decode_advance_cp_kernel, (n + 127) / 128, 128, 0, stream, positions, kv_len, slots, block_table, max_pages, page_size, n, world,
           rank, (unsigned long long*)step_ctr);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_decode_advance(int* positions, int* kv_len, int* slots, const int* block_table, const int* live, int max_pages,
                             int page_size, int n, void* step_ctr, cudaStream_t stream) {
  if (n <= 0) return 0;
  launch_k(decode_advance_kernel, (n + 127) / 128, 128, 0, stream, positions, kv_len, slots, block_table, live, max_pages, page_size, n,
           (unsigned long long*)step_ctr);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_embed(const int* ids, const void* table, void* out, int n_tok, int hidden, int vocab, cudaStream_t stream) {
  if (hidden % 8) return fail("embed: hidden %% 8 != 0%s");
  if (n_tok <= 0) return 0;
  launch_k(embed_kernel, n_tok, 128, 0, stream, ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, n_tok, hidden, vocab);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

// residual (in/out, may be null) += delta (may be null); y = rmsnorm(residual or x_in) * weight.
// out (bf16) and out_q/out_sf (MXFP8) are optional outputs.
static int rmsnorm_launch(void* residual, const void* delta, const void* x_in, const void* weight, void* out, void* out_q, void* out_sf,
                          int rows, int hidden, float eps, int ld_in, int ld_out, int sf32, const float* partials, int n_partials,
                          long partial_stride, const void* wait_flags, int wait_n, const void* epoch_ptr, void* status, cudaStream_t stream,
                          const void* comb_y = nullptr, const int* comb_rows = nullptr, const float* comb_w = nullptr, int comb_k = 0,
                          int comb_ld = 0, int part_inner = 1, long part_inner_stride = 0, const RmsBcast* bcast = nullptr) {
  if (part_inner < 1) part_inner = 1;
  RmsBcast bc;
  memset(&bc, 0, sizeof(bc));
  if (bcast != nullptr) {
    bc = *bcast;
    if (bc.world < 0 || bc.world > 8 || bc.epoch_ctr == nullptr || bc.done_ctr == nullptr) return fail("rmsnorm: bad gather arguments%s");
  }
  if (comb_k > 16) return fail("rmsnorm: combine of more than 16 rows%s");
  if (hidden % 8 || hidden > 256 * 8 * 4) return fail("rmsnorm: hidden must be a multiple of 8 and <= 8192%s");
  if (out_q != nullptr && hidden % 128) return fail("rmsnorm: MXFP8 output needs hidden %% 128 == 0%s");
  if (rows <= 0) return 0;
  const int nvec = hidden / 8;
#define GB_RMS(V) launch_k(rmsnorm_kernel<V>, rows, 256, 0, stream, (__nv_bfloat16*)residual, (const __nv_bfloat16*)delta, \
    (const __nv_bfloat16*)x_in, (const __nv_bfloat16*)weight, (__nv_bfloat16*)out, (uint8_t*)out_q, (uint8_t*)out_sf, hidden, eps, ld_in, ld_out, sf32, \
    partials, n_partials, partial_stride, (const uint32_t*)wait_flags, wait_n, (const uint32_t*)epoch_ptr, (KernelStatus*)status, \
    (const __nv_bfloat16*)comb_y, comb_rows, comb_w, comb_k, comb_ld, part_inner, part_inner_stride, bc)
  if (nvec <= 256) GB_RMS(1); else if (nvec <= 512) GB_RMS(2); else if (nvec <= 768) GB_RMS(3); else GB_RMS(4);
#undef GB_RMS
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_rmsnorm(void* residual, const void* delta, const void* x_in, const void* weight, void* out, void* out_q, void* out_sf,
                      int rows, int hidden, float eps, int ld_in, int ld_out, int sf32, cudaStream_t stream) {
  return rmsnorm_launch(residual, delta, x_in, weight, out, out_q, out_sf, rows, hidden, eps, ld_in, ld_out, sf32, nullptr, 0, 0, nullptr, 0,
                        nullptr, nullptr, stream);
}

// residual += sum over ranks of partials[p] (fp32, [n_partials][partial_stride] with rows * hidden used), then RMSNorm.
// Waits (bounded) until wait_flags[i] >= *epoch_ptr for i < wait_n before reading the partials.
GB_API int gb_rmsnorm_reduce(void* residual, const float* partials, int n_partials, long partial_stride, const void* weight, void* out,
                             void* out_q, void* out_sf, int rows, int hidden, float eps, int sf32, const void* wait_flags, int wait_n,
                             const void* epoch_ptr, void* status, cudaStream_t stream) {
  return rmsnorm_launch(residual, nullptr, nullptr, weight, out, out_q, out_sf, rows, hidden, eps, hidden, hidden, sf32, partials, n_partials,
                        partial_stride, wait_flags, wait_n, epoch_ptr, status, stream);
}

// gb_rmsnorm_reduce whose bf16 result is also all-gathered: row r goes to bcast->out[p] + r * hidden on every GPU p and the flags
// bcast->flag[p] are raised with the advanced epoch once all rows are stored (see RmsBcast).  `out` may be null.
GB_API int gb_rmsnorm_reduce_bcast(void* residual, const float* partials, int n_partials, long partial_stride, const void* weight, void* out,
                                   void* out_q, void* out_sf, int rows, int hidden, float eps, int sf32, const void* wait_flags, int wait_n,
                                   const void* epoch_ptr, void* status, const RmsBcast* bcast, cudaStream_t stream) {
  return rmsnorm_launch(residual, nullptr, nullptr, weight, out, out_q, out_sf, rows, hidden, eps, hidden, hidden, sf32, partials, n_partials,
                        partial_stride, wait_flags, wait_n, epoch_ptr, status, stream, nullptr, nullptr, nullptr, 0, 0, 1, 0, bcast);
}

// A rank with no rows to contribute still has to advance the epoch and raise its flags (the others wait for every rank).
__global__ void bcast_signal_kernel(const RmsBcast bc) {
  pdl_wait();
  pdl_trigger();
  if (threadIdx.x == 0) {
    const uint32_t e = *bc.epoch_ctr + 1;
    *bc.epoch_ctr = e;
    for (int p = 0; p < bc.world; ++p) st_release_sys(bc.flag[p], e);
  }
}
GB_API int gb_bcast_signal(const RmsBcast* bcast, cudaStream_t stream) {
  if (bcast == nullptr || bcast->world < 1 || bcast->world > 8 || bcast->epoch_ctr == nullptr) return fail("bcast_signal: bad arguments%s");
  launch_k(bcast_signal_kernel, 1, 32, 0, stream, *bcast);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

// residual += delta, RMSNorm, MXFP8 copy (optional) and the all-gather of the bf16 rows (see RmsBcast).
GB_API int gb_rmsnorm_bcast(void* residual, const void* delta, const void* weight, void* out_q, void* out_sf, int rows, int hidden, float eps,
                            int ld_in, int sf32, const RmsBcast* bcast, cudaStream_t stream) {
  return rmsnorm_launch(residual, delta, nullptr, weight, nullptr, out_q, out_sf, rows, hidden, eps, ld_in, hidden, sf32, nullptr, 0, 0, nullptr, 0,
                        nullptr, nullptr, stream, nullptr, nullptr, nullptr, 0, 0, 1, 0, bcast);
}

// The same when every rank's slot holds `n_inner` K-split partials, `inner_stride` elements apart: n_ranks * n_inner slabs are summed
// (rank-major, split-minor order).
GB_API int gb_rmsnorm_reduce2(void* residual, const float* partials, int n_ranks, long rank_stride, int n_inner, long inner_stride,
                              const void* weight, void* out, void* out_q, void* out_sf, int rows, int hidden, float eps, int sf32,
                              const void* wait_flags, int wait_n, const void* epoch_ptr, void* status, cudaStream_t stream) {
  return rmsnorm_launch(residual, nullptr, nullptr, weight, out, out_q, out_sf, rows, hidden, eps, hidden, hidden, sf32, partials,
                        n_ranks * (n_inner < 1 ? 1 : n_inner), rank_stride, wait_flags, wait_n, epoch_ptr, status, stream, nullptr, nullptr, nullptr, 0,
                        0, n_inner, inner_stride);
}

// residual[t] += sum_j w[t, j] * y[pair_row[t * k + j]] (the MoE combine), then RMSNorm: the combine never makes a round trip
// through memory.  Optional bounded wait on wait_flags (expert-parallel: the rows of y are stored by the experts' GPUs).
GB_API int gb_rmsnorm_combine(void* residual, const void* y, const int* pair_row, const float* weights, int k, int ld_y, const void* weight,
                              void* out, void* out_q, void* out_sf, int rows, int hidden, float eps, int sf32, const void* wait_flags,
                              int wait_n, const void* epoch_ptr, void* status, cudaStream_t stream) {
  return rmsnorm_launch(residual, nullptr, nullptr, weight, out, out_q, out_sf, rows, hidden, eps, hidden, hidden, sf32, nullptr, 0, 0,
                        wait_flags, wait_n, epoch_ptr, status, stream, y, pair_row, weights, k, ld_y);
}

// Same with the fused QKV rows given as K-split fp32 partial sums `part` [n_part][n_tok][ld_qkv] (head_dim 128, full rotary only).
GB_API int gb_qk_norm_rope_partials(const float* part, int n_part, long part_stride, const int* positions, const int* slots, const void* q_w,
                                    const void* k_w, void* q_out, void* k_cache, void* v_cache, int n_tok, int hq, int hkv, float theta,
                                    float eps, int ld_qkv, float q_scale, const void* rope_tab, int tab_len, const int* pos3, int sec_h3,
                                    int sec_w3, cudaStream_t stream) {
  if (n_tok <= 0) return 0;
  const auto al = [](const void* p, int a) { return ((uintptr_t)p & (uintptr_t)(a - 1)) == 0; };
  if (n_part < 1 || ld_qkv % 4 != 0 || part_stride % 4 != 0 || !al(part, 16) || !al(q_w, 8) || !al(k_w, 8) || !al(q_out, 8) ||
      !al(k_cache, 8) || !al(v_cache, 8) || !al(rope_tab, 16))
    return fail("qk_norm_rope_partials: misaligned argument%s");
  const long warps = (long)n_tok * (hq + 2 * hkv);
  launch_k(qk_norm_rope128_kernel, (unsigned)((warps + 15) / 16), 256, 0, stream, (const __nv_bfloat16*)nullptr, positions, slots,
           (const __nv_bfloat16*)q_w, (const __nv_bfloat16*)k_w, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
           n_tok, hq, hkv, theta, eps, ld_qkv, q_scale, (const float2*)rope_tab, tab_len, pos3, sec_h3, sec_w3, part, n_part, part_stride);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_qk_norm_rope(const void* qkv, const int* positions, const int* slots, const void* q_w, const void* k_w, void* q_out,
                           void* k_cache, void* v_cache, int n_tok, int hq, int hkv, int head_dim, int rope_pairs, float theta,
                           float eps, int ld_qkv, float q_scale, const void* rope_tab, int tab_len, const int* pos3, int sec_h3, int sec_w3,
                           cudaStream_t stream) {
  if (n_tok <= 0) return 0;
  const long warps = (long)n_tok * (hq + 2 * hkv);
  const auto al8 = [](const void* p) { return ((uintptr_t)p & 7) == 0; };
  if (head_dim == 128 && rope_pairs == 64 && ld_qkv % 4 == 0 && al8(qkv) && al8(q_w) && al8(k_w) && al8(q_out) && al8(k_cache) &&
      al8(v_cache) && ((uintptr_t)rope_tab & 15) == 0) {
    launch_k(qk_norm_rope128_kernel, (unsigned)((warps + 15) / 16), 256, 0, stream, (const __nv_bfloat16*)qkv, positions, slots,
             (const __nv_bfloat16*)q_w, (const __nv_bfloat16*)k_w, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
             n_tok, hq, hkv, theta, eps, ld_qkv, q_scale, (const float2*)rope_tab, tab_len, pos3, sec_h3, sec_w3, (const float*)nullptr, 0, 0L);
    GB_CUDA_OK(cudaGetLastError());
    return 0;
  }
  const int blocks = (int)((warps + 7) / 8);
#define GB_QK(DV) launch_k(qk_norm_rope_kernel<DV>, blocks, 256, 0, stream, (const __nv_bfloat16*)qkv, positions, slots, \
    (const __nv_bfloat16*)q_w, (const __nv_bfloat16*)k_w, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, \
    n_tok, hq, hkv, rope_pairs, theta, eps, ld_qkv, q_scale, (const float2*)rope_tab, tab_len, pos3, sec_h3, sec_w3)
  if (head_dim == 64) GB_QK(64); else if (head_dim == 128) GB_QK(128); else if (head_dim == 256) GB_QK(256);
  else return fail("qk_norm_rope: head_dim must be 64, 128 or 256%s");
#undef GB_QK
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_silu_mul(const void* gate_up, void* out, long rows, int inter, int ld, cudaStream_t stream) {
  if (inter % 8) return fail("silu_mul: inter %% 8 != 0%s");
  const long n = rows * (inter / 8);
  if (n <= 0) return 0;
  launch_k(silu_mul_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, rows, inter, ld);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_silu_mul_quant(const void* gate_up, const int* row_valid, void* out_q, void* out_sf, long rows, int inter, int ld, int sf32,
                             cudaStream_t stream) {
  if (inter % 128) return fail("silu_mul_quant: inter %% 128 != 0%s");
  const long n = rows * (inter / 8);
  if (n <= 0) return 0;
  launch_k(silu_mul_quant_kernel, (unsigned)((n + 256 * kSiluU - 1) / (256 * kSiluU)), 256, 0, stream, (const __nv_bfloat16*)gate_up, row_valid, (uint8_t*)out_q,
           (uint8_t*)out_sf, rows, inter, ld, sf32);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_silu_mul_partials(const float* part, int n_part, long part_stride, void* out, void* out_q, void* out_sf, long rows, int inter,
                                int sf32, cudaStream_t stream) {
  if (inter % 8 || (out_q != nullptr && inter % 128)) return fail("silu_mul_partials: inter must be a multiple of 8 (128 with MXFP8 output)%s");
  if (part_stride % 4 != 0 || ((uintptr_t)part & 15) != 0) return fail("silu_mul_partials: misaligned partials%s");
  const long n = rows * (inter / 8);
  if (n <= 0) return 0;
  launch_k(silu_mul_partials_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, part, n_part, part_stride, (__nv_bfloat16*)out, (uint8_t*)out_q,
           (uint8_t*)out_sf, rows, inter, sf32);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_mx_quant(const void* in, const int* src_rows, void* out_q, void* out_sf, long out_rows, int k, int ld_in, int sf32, cudaStream_t stream) {
  if (k % 128) return fail("mx_quant: k %% 128 != 0%s");
  const long n = out_rows * (k / 8);
  if (n <= 0) return 0;
  if (src_rows != nullptr && k % 256 == 0) {
    const long blocks = std::min<long>((out_rows + 7) / 8, (long)sm_count() * 16);
    launch_k(mx_quant_rows_kernel, (unsigned)blocks, 256, 0, stream, (const __nv_bfloat16*)in, src_rows, (uint8_t*)out_q, (uint8_t*)out_sf, out_rows, k, ld_in, sf32);
    GB_CUDA_OK(cudaGetLastError());
    return 0;
  }
  launch_k(mx_quant_kernel, (unsigned)((n + 256 * kMxQuantU - 1) / (256 * kMxQuantU)), 256, 0, stream, (const __nv_bfloat16*)in, src_rows, (uint8_t*)out_q, (uint8_t*)out_sf, out_rows, k, ld_in, sf32);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_mx_gather_rows(const void* in_q, const void* in_sf, const int* src_rows, void* out_q, void* out_sf, long out_rows, int k,
                             int in_sf32, int out_sf32, cudaStream_t stream) {
  if (out_rows <= 0) return 0;
  if (k % 128 != 0) return fail("mx_gather_rows: k %% 128 != 0%s");
  const long blocks = std::min<long>((out_rows + 7) / 8, (long)sm_count() * 16);
  launch_k(mx_gather_rows_kernel, (unsigned)blocks, 256, 0, stream, (const uint8_t*)in_q, (const uint8_t*)in_sf, src_rows, (uint8_t*)out_q,
           (uint8_t*)out_sf, out_rows, k, in_sf32, out_sf32);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Copies `n` pages of `page_bytes` bytes inside one cache tensor; src / dst are device arrays of page indices.
GB_API int gb_kv_copy_pages(void* cache, const int* src, const int* dst, int n, int n_pages, long page_bytes, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (page_bytes % 16 != 0 || ((uintptr_t)cache & 15) != 0) return fail("kv_copy_pages: pages must be 16-byte aligned%s");
  const long vecs = page_bytes / 16;
  const unsigned by = (unsigned)std::min<long>((vecs + 255) / 256, 64);
  launch_k(kv_copy_pages_kernel, dim3((unsigned)n, by), 256, 0, stream, (uint4*)cache, src, dst, n_pages, vecs);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_kv_quant_q8(const void* x, void* q, float* scale, long rows, int d, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (d % 32 || d > 256) return fail("kv_quant_q8: head_dim must be a multiple of 32, at most 256%s");
  launch_k(kv_quant_q8_kernel, (unsigned)((rows * 32 + 255) / 256), 256, 0, stream, (const __nv_bfloat16*)x, (int8_t*)q, scale, rows, d);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_kv_dequant_q8(const void* q, const float* scale, void* x, long rows, int d, cudaStream_t stream) {
  if (rows <= 0) return 0;
  launch_k(kv_dequant_q8_kernel, (unsigned)((rows * d + 255) / 256), 256, 0, stream, (const int8_t*)q, scale, (__nv_bfloat16*)x, rows, d);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_cast_f32_bf16(const float* in, void* out, long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  launch_k(cast_f32_bf16_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, in, (__nv_bfloat16*)out, n);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}
