// Chunked scan of the gated Delta-Net recurrence for prefill (the per-token form and the math conventions are in deltanet.cu).
//
// Per value head the recurrence is  S_t = g_t S_{t-1} + u_t k_t^T,  u_t = beta_t (v_t - g_t S_{t-1} k_t),  o_t = S_t q_t
// with the scalar decay g_t = exp(a_t).  Over a chunk of C = 64 tokens, with c_i the running sum of a_t inside the chunk and S0 the
// state in front of it, the u_t solve a unit lower-triangular system, and everything else is matrix products:
//
//   L_ij   = beta_i exp(c_i - c_j) (k_i . k_j)   (j < i)          T = (I + L)^-1 diag(beta)
//   U      = T V - (T diag(exp c) K) S0^T                          (rows u_i)
//   O      = diag(exp c) Q S0^T + M U,   M_ij = exp(c_i - c_j) (q_i . k_j)  (j <= i)
//   S_end  = exp(c_last) S0 + U^T diag(exp(c_last - c_j)) K
//
// Two kernels.  dn_chunk_prep_kernel (one CTA per chunk and value head, all chunks of all sequences in parallel) computes what
// does not depend on the state: the normalised q / k, T (forward substitution, one thread per column), T V, -T diag(exp c) K, M,
// diag(exp c) Q and the decayed keys, all as bf16 tiles in a workspace.  dn_chunk_scan_kernel (one CTA per sequence and value head)
// walks the chunks in order with the state in registers as fp32 accumulator fragments: three products per chunk (U, O, the state
// update), the gated RMSNorm of O, and the output.  The products are 64 x 128 x 128 at most and sit on a serial chain, so they
// run on warp-level mma tiles with register accumulators (nvcuda::wmma, bf16 in, fp32 out) rather than on tcgen05: a TMEM round
// trip per link of the chain would cost more than the tiles themselves.
//
// The reference's counterpart is the chunked scan of cuda/llm/cuda_llm_runner.c:8128 (batch_deltanet_scan_f32) and its test
// cuda/llm/scan/deltanet_chunk_test.c; the per-token recurrence is common/transformer.h:2829-2851.

#include <mma.h>

#include "sm100.cuh"
#include "host_common.h"

namespace gb {

using namespace nvcuda;

constexpr int kDnC = 64;            // tokens per chunk
constexpr int kDnD = 128;           // d_state
constexpr int kDnLd = kDnD + 8;     // bf16 row stride of a 128-wide tile in shared memory (the pad spreads the rows over the banks)
constexpr int kDnLc = kDnC + 8;     // bf16 row stride of a 64-wide tile
constexpr int kDnLf = kDnD + 4;     // fp32 row stride of the 64 x 128 staging tile
constexpr int kDnLo = kDnC;         // L (64 x 64, fp32) lives in the columns 64 .. 127 of the staging tile while T is solved
constexpr int kDnThreads = 256;

struct DnChunkArgs {
  const __nv_bfloat16* qkv; int ld_qkv;
  const __nv_bfloat16* z; int ld_z;
  const float* ab; const float* a; const float* dt_bias; const float* norm_w;
  float* state; const int* cu_q; const int* seq_slots; __nv_bfloat16* out;
  int n_group, dt_rank, n_seqs; float eps;
  // workspace: entry (chunk, head) at index chunk * dt_rank + head
  __nv_bfloat16* gq;     // [64][128]  exp(c_i) q_i
  __nv_bfloat16* nw;     // [64][128]  -(T diag(exp c) K)
  __nv_bfloat16* uv;     // [64][128]  T V
  __nv_bfloat16* kdt;    // [128][64]  exp(c_last - c_j) k_j, transposed
  __nv_bfloat16* mqk;    // [64][64]   M
  float* glast;          // exp(c_last)
};

// chunk `cb` (numbered through the sequences in order) -> its sequence and token range
__device__ __forceinline__ bool dn_find_chunk(const int* __restrict__ cu_q, int n_seqs, int cb, int& t0, int& t1) {
  int acc = 0;
  for (int s = 0; s < n_seqs; ++s) {
    const int b = cu_q[s], e = cu_q[s + 1];
    const int n = (e - b + kDnC - 1) / kDnC;
    if (cb < acc + n) {
      t0 = b + (cb - acc) * kDnC;
      t1 = min(t0 + kDnC, e);
      return true;
    }
    acc += n;
  }
  return false;
}

__device__ __forceinline__ float dn_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

using FragA = wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major>;
using FragB = wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major>;     // B given as [n][k] rows
using FragC = wmma::fragment<wmma::accumulator, 16, 16, 16, float>;

// 112.5 KB: two CTAs per SM
constexpr int kPrepSmem = (2 * kDnC * kDnLd + 2 * kDnD * kDnLc + kDnC * kDnLc) * 2 + (kDnC * kDnLf + 2 * kDnC) * 4;

__global__ void __launch_bounds__(kDnThreads)
dn_chunk_prep_kernel(const DnChunkArgs a) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(128) uint8_t dn_smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(dn_smem);          // [64][kDnLd] normalised, scaled q
  __nv_bfloat16* sK = sQ + kDnC * kDnLd;                                   // [64][kDnLd] normalised k
  __nv_bfloat16* sVT = sK + kDnC * kDnLd;                                  // [128][kDnLc] v transposed
  __nv_bfloat16* sGKT = sVT + kDnD * kDnLc;                                // [128][kDnLc] exp(c_j) k_j transposed
  __nv_bfloat16* sT = sGKT + kDnD * kDnLc;                                 // [64][kDnLc]
  float* sF = reinterpret_cast<float*>(sT + kDnC * kDnLc);                 // [64][kDnLf]
  float* sL = sF + kDnLo;                                                  // [64][.. kDnLf], the right half of sF
  float* sc = sF + kDnC * kDnLf;                                           // [64] running log decay
  float* sb = sc + kDnC;                                                   // [64] beta

  const int cb = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int t0 = 0, t1 = 0;
  if (!dn_find_chunk(a.cu_q, a.n_seqs, cb, t0, t1)) return;
  const int g = h % a.n_group;
  const int q_off = g * kDnD, k_off = (a.n_group + g) * kDnD, v_off = 2 * a.n_group * kDnD + h * kDnD;
  const size_t ws = (size_t)cb * a.dt_rank + h;

  // rows of the chunk: L2-normalised q (scaled by 1 / sqrt(d)) and k, v transposed; tokens past the end are zero rows
  for (int i = warp; i < kDnC; i += kDnThreads / 32) {
    const int t = t0 + i;
    float q4[4] = {0.f, 0.f, 0.f, 0.f}, k4[4] = {0.f, 0.f, 0.f, 0.f}, v4[4] = {0.f, 0.f, 0.f, 0.f};
    if (t < t1) {
      const __nv_bfloat16* row = a.qkv + (size_t)t * a.ld_qkv;
      const uint2 qr = *reinterpret_cast<const uint2*>(row + q_off + 4 * lane);
      const uint2 kr = *reinterpret_cast<const uint2*>(row + k_off + 4 * lane);
      const uint2 vr = *reinterpret_cast<const uint2*>(row + v_off + 4 * lane);
      const __nv_bfloat16* qb = reinterpret_cast<const __nv_bfloat16*>(&qr);
      const __nv_bfloat16* kb = reinterpret_cast<const __nv_bfloat16*>(&kr);
      const __nv_bfloat16* vb = reinterpret_cast<const __nv_bfloat16*>(&vr);
#pragma unroll
      for (int e = 0; e < 4; ++e) { q4[e] = __bfloat162float(qb[e]); k4[e] = __bfloat162float(kb[e]); v4[e] = __bfloat162float(vb[e]); }
    }
    const float qs = dn_warp_sum(q4[0] * q4[0] + q4[1] * q4[1] + q4[2] * q4[2] + q4[3] * q4[3]);
    const float ks = dn_warp_sum(k4[0] * k4[0] + k4[1] * k4[1] + k4[2] * k4[2] + k4[3] * k4[3]);
    const float qsc = rsqrtf(qs + a.eps) * rsqrtf((float)kDnD), ksc = rsqrtf(ks + a.eps);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      sQ[i * kDnLd + 4 * lane + e] = __float2bfloat16(q4[e] * qsc);
      sK[i * kDnLd + 4 * lane + e] = __float2bfloat16(k4[e] * ksc);
      sVT[(4 * lane + e) * kDnLc + i] = __float2bfloat16(v4[e]);
    }
  }
  if (tid < kDnC) {
    const int t = t0 + tid;
    float al = 0.f, beta = 0.f;
    if (t < t1) {
      const float ar = a.ab[(size_t)t * 2 * a.dt_rank + h] + a.dt_bias[h];
      const float sp = ar > 20.0f ? ar : log1pf(__expf(ar));
      al = sp * a.a[h];
      beta = 1.0f / (1.0f + __expf(-a.ab[(size_t)t * 2 * a.dt_rank + a.dt_rank + h]));
    }
    sc[tid] = al;
    sb[tid] = beta;
  }
  __syncthreads();
  if (tid == 0) {
    float acc = 0.f;
    for (int i = 0; i < kDnC; ++i) { acc += sc[i]; sc[i] = acc; }
  }
  __syncthreads();
  const float c_last = sc[kDnC - 1];
  for (int idx = tid; idx < kDnC * kDnD; idx += kDnThreads) {
    const int j = idx / kDnD, c = idx % kDnD;
    sGKT[c * kDnLc + j] = __float2bfloat16(__expf(sc[j]) * __bfloat162float(sK[j * kDnLd + c]));
  }

  // K K^T and Q K^T (64 x 64 x 128): warp w computes the tiles (m = w & 3, n = 2 (w >> 2) and the next)
  const int tm = warp & 3, tn0 = (warp >> 2) * 2;
  for (int pass = 0; pass < 2; ++pass) {
    const __nv_bfloat16* sA = pass == 0 ? sK : sQ;
    FragC acc[2];
    wmma::fill_fragment(acc[0], 0.f);
    wmma::fill_fragment(acc[1], 0.f);
    for (int kk = 0; kk < kDnD / 16; ++kk) {
      FragA fa;
      wmma::load_matrix_sync(fa, sA + (16 * tm) * kDnLd + 16 * kk, kDnLd);
#pragma unroll
      for (int n2 = 0; n2 < 2; ++n2) {
        FragB fb;
        wmma::load_matrix_sync(fb, sK + (16 * (tn0 + n2)) * kDnLd + 16 * kk, kDnLd);
        wmma::mma_sync(acc[n2], fa, fb, acc[n2]);
      }
    }
    wmma::store_matrix_sync(sF + (16 * tm) * kDnLf + 16 * tn0, acc[0], kDnLf, wmma::mem_row_major);
    wmma::store_matrix_sync(sF + (16 * tm) * kDnLf + 16 * (tn0 + 1), acc[1], kDnLf, wmma::mem_row_major);
    __syncthreads();
    for (int idx = tid; idx < kDnC * kDnC; idx += kDnThreads) {
      const int i = idx / kDnC, j = idx % kDnC;
      if (pass == 0) {
        sL[i * kDnLf + j] = (j < i) ? sb[i] * __expf(sc[i] - sc[j]) * sF[i * kDnLf + j] : 0.f;
      } else {
        const float m = (j <= i) ? __expf(sc[i] - sc[j]) * sF[i * kDnLf + j] : 0.f;
        a.mqk[(ws * kDnC + i) * kDnC + j] = __float2bfloat16(m);
      }
    }
    __syncthreads();
  }

  // T = (I + L)^-1 diag(beta) by forward substitution, column by column: four adjacent lanes share a column (each a quarter of
  // the inner sum; x_j = 0 above the diagonal, so the sum starts at the column's block of four)
  {
    const int col = tid >> 2, q = tid & 3, j0 = (col & ~3) + q;
    const float bcol = sb[col];
    for (int i = 0; i < kDnC; ++i) {
      float part = 0.f;
      for (int j = j0; j < i; j += 4) part += sL[i * kDnLf + j] * sF[j * kDnLf + col];
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      if (q == 0) sF[i * kDnLf + col] = ((i == col) ? bcol : 0.f) - part;
      __syncwarp();
    }
  }
  __syncthreads();
  for (int idx = tid; idx < kDnC * kDnC; idx += kDnThreads) {
    const int i = idx / kDnC, j = idx % kDnC;
    sT[i * kDnLc + j] = __float2bfloat16(sF[i * kDnLf + j]);
  }
  __syncthreads();

  // T V and -(T diag(exp c) K) (64 x 128 x 64): warp w computes the 16 output columns 16 w ..
  for (int pass = 0; pass < 2; ++pass) {
    const __nv_bfloat16* sB = pass == 0 ? sVT : sGKT;
    FragC acc[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) wmma::fill_fragment(acc[m], 0.f);
    for (int kk = 0; kk < kDnC / 16; ++kk) {
      FragB fb;
      wmma::load_matrix_sync(fb, sB + (16 * warp) * kDnLc + 16 * kk, kDnLc);
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        FragA fa;
        wmma::load_matrix_sync(fa, sT + (16 * m) * kDnLc + 16 * kk, kDnLc);
        wmma::mma_sync(acc[m], fa, fb, acc[m]);
      }
    }
#pragma unroll
    for (int m = 0; m < 4; ++m) wmma::store_matrix_sync(sF + (16 * m) * kDnLf + 16 * warp, acc[m], kDnLf, wmma::mem_row_major);
    __syncthreads();
    __nv_bfloat16* dst = (pass == 0 ? a.uv : a.nw) + ws * kDnC * kDnD;
    const float sign = pass == 0 ? 1.0f : -1.0f;
    for (int idx = tid; idx < kDnC * kDnD; idx += kDnThreads) dst[idx] = __float2bfloat16(sign * sF[(idx / kDnD) * kDnLf + idx % kDnD]);
    __syncthreads();
  }

  for (int idx = tid; idx < kDnC * kDnD; idx += kDnThreads) {
    const int i = idx / kDnD, c = idx % kDnD;
    a.gq[ws * kDnC * kDnD + idx] = __float2bfloat16(__expf(sc[i]) * __bfloat162float(sQ[i * kDnLd + c]));
  }
  for (int idx = tid; idx < kDnD * kDnC; idx += kDnThreads) {
    const int c = idx / kDnC, j = idx % kDnC;
    a.kdt[ws * kDnD * kDnC + idx] = __float2bfloat16(__expf(c_last - sc[j]) * __bfloat162float(sK[j * kDnLd + c]));
  }
  if (tid == 0) a.glast[ws] = __expf(c_last);
}

constexpr int kDnLt = kDnC + 4;     // fp32 row stride of U stored transposed (128 x 64) in the staging tile
constexpr int kScanStage = (kDnC * kDnLf > kDnD * kDnLt ? kDnC * kDnLf : kDnD * kDnLt);
constexpr int kScanSmem = (2 * kDnC * kDnLd + 2 * kDnD * kDnLc + kDnC * kDnLc + kDnD * kDnLd) * 2 + (kScanStage + 8 * 256) * 4;

__global__ void __launch_bounds__(kDnThreads)
dn_chunk_scan_kernel(const DnChunkArgs a) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(128) uint8_t dn_smem[];
  __nv_bfloat16* sGQ = reinterpret_cast<__nv_bfloat16*>(dn_smem);         // [64][kDnLd]
  __nv_bfloat16* sNW = sGQ + kDnC * kDnLd;                                 // [64][kDnLd]
  __nv_bfloat16* sKdT = sNW + kDnC * kDnLd;                                // [128][kDnLc]
  __nv_bfloat16* sUT = sKdT + kDnD * kDnLc;                                // [128][kDnLc] U transposed
  __nv_bfloat16* sMqk = sUT + kDnD * kDnLc;                                // [64][kDnLc]
  __nv_bfloat16* sSb = sMqk + kDnC * kDnLc;                                // [128][kDnLd] the state as bf16, [value][key]
  float* sF = reinterpret_cast<float*>(sSb + kDnD * kDnLd);                // [64][kDnLf]
  float* sScr = sF + kScanStage;                                           // [8 warps][16 x 16]

  const int h = blockIdx.x, s = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq_t0 = a.cu_q[s], seq_t1 = a.cu_q[s + 1];
  if (seq_t1 <= seq_t0) return;
  int cb = 0;
  for (int i = 0; i < s; ++i) cb += (a.cu_q[i + 1] - a.cu_q[i] + kDnC - 1) / kDnC;
  const int n_chunks = (seq_t1 - seq_t0 + kDnC - 1) / kDnC;

  // state rows 16 warp .. of this head: eight 16 x 16 fp32 accumulator fragments per warp
  float* st = a.state + ((size_t)a.seq_slots[s] * a.dt_rank + h) * kDnD * kDnD;
  FragC S[8];
#pragma unroll
  for (int f = 0; f < 8; ++f) wmma::load_matrix_sync(S[f], st + (16 * warp) * kDnD + 16 * f, kDnD, wmma::mem_row_major);
  float* scr = sScr + warp * 256;

  for (int ci = 0; ci < n_chunks; ++ci, ++cb) {
    const size_t ws = (size_t)cb * a.dt_rank + h;
    const int t0 = seq_t0 + ci * kDnC, t1 = min(t0 + kDnC, seq_t1);
    // the chunk's tiles -> shared memory (16 bytes per copy); T V goes to the staging tile as fp32: it is where U accumulates
    {
      const uint4* gq = reinterpret_cast<const uint4*>(a.gq + ws * kDnC * kDnD);
      const uint4* nw = reinterpret_cast<const uint4*>(a.nw + ws * kDnC * kDnD);
      const uint4* uv = reinterpret_cast<const uint4*>(a.uv + ws * kDnC * kDnD);
      for (int idx = tid; idx < kDnC * kDnD / 8; idx += kDnThreads) {
        const int i = idx / (kDnD / 8), v = idx % (kDnD / 8);
        *reinterpret_cast<uint4*>(sGQ + i * kDnLd + 8 * v) = gq[idx];
        *reinterpret_cast<uint4*>(sNW + i * kDnLd + 8 * v) = nw[idx];
        const uint4 u = uv[idx];
        const __nv_bfloat16* ub = reinterpret_cast<const __nv_bfloat16*>(&u);
        float* d = sF + i * kDnLf + 8 * v;
#pragma unroll
        for (int e = 0; e < 8; ++e) d[e] = __bfloat162float(ub[e]);
      }
      const uint4* kd = reinterpret_cast<const uint4*>(a.kdt + ws * kDnD * kDnC);
      for (int idx = tid; idx < kDnD * kDnC / 8; idx += kDnThreads) {
        const int c = idx / (kDnC / 8), v = idx % (kDnC / 8);
        *reinterpret_cast<uint4*>(sKdT + c * kDnLc + 8 * v) = kd[idx];
      }
      const uint4* mq = reinterpret_cast<const uint4*>(a.mqk + ws * kDnC * kDnC);
      for (int idx = tid; idx < kDnC * kDnC / 8; idx += kDnThreads) {
        const int i = idx / (kDnC / 8), v = idx % (kDnC / 8);
        *reinterpret_cast<uint4*>(sMqk + i * kDnLc + 8 * v) = mq[idx];
      }
    }
    const float g_last = a.glast[ws];
    // the state in front of the chunk as a bf16 operand
#pragma unroll
    for (int f = 0; f < 8; ++f) {
      wmma::store_matrix_sync(scr, S[f], 16, wmma::mem_row_major);
      __syncwarp();
      for (int e = lane; e < 256; e += 32) sSb[(16 * warp + (e >> 4)) * kDnLd + 16 * f + (e & 15)] = __float2bfloat16(scr[e]);
      __syncwarp();
    }
    __syncthreads();

    // U = T V - (T diag(exp c) K) S0^T: warp w owns the value columns 16 w ..
    {
      FragC acc[4];
#pragma unroll
      for (int m = 0; m < 4; ++m) wmma::load_matrix_sync(acc[m], sF + (16 * m) * kDnLf + 16 * warp, kDnLf, wmma::mem_row_major);
      for (int kk = 0; kk < kDnD / 16; ++kk) {
        FragB fb;
        wmma::load_matrix_sync(fb, sSb + (16 * warp) * kDnLd + 16 * kk, kDnLd);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          FragA fa;
          wmma::load_matrix_sync(fa, sNW + (16 * m) * kDnLd + 16 * kk, kDnLd);
          wmma::mma_sync(acc[m], fa, fb, acc[m]);
        }
      }
      __syncthreads();        // every warp has taken its columns of T V out of the staging tile: U goes back transposed, [value][token]
#pragma unroll
      for (int m = 0; m < 4; ++m) wmma::store_matrix_sync(sF + (16 * warp) * kDnLt + 16 * m, acc[m], kDnLt, wmma::mem_col_major);
    }
    __syncthreads();
    for (int idx = tid; idx < kDnD * kDnC; idx += kDnThreads) {
      const int r = idx / kDnC, j = idx % kDnC;
      sUT[r * kDnLc + j] = __float2bfloat16(sF[r * kDnLt + j]);
    }
    __syncthreads();

    // O = diag(exp c) Q S0^T + M U
    {
      FragC acc[4];
#pragma unroll
      for (int m = 0; m < 4; ++m) wmma::fill_fragment(acc[m], 0.f);
      for (int kk = 0; kk < kDnD / 16; ++kk) {
        FragB fb;
        wmma::load_matrix_sync(fb, sSb + (16 * warp) * kDnLd + 16 * kk, kDnLd);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          FragA fa;
          wmma::load_matrix_sync(fa, sGQ + (16 * m) * kDnLd + 16 * kk, kDnLd);
          wmma::mma_sync(acc[m], fa, fb, acc[m]);
        }
      }
      for (int kk = 0; kk < kDnC / 16; ++kk) {
        FragB fb;
        wmma::load_matrix_sync(fb, sUT + (16 * warp) * kDnLc + 16 * kk, kDnLc);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          FragA fa;
          wmma::load_matrix_sync(fa, sMqk + (16 * m) * kDnLc + 16 * kk, kDnLc);
          wmma::mma_sync(acc[m], fa, fb, acc[m]);
        }
      }
#pragma unroll
      for (int m = 0; m < 4; ++m) wmma::store_matrix_sync(sF + (16 * m) * kDnLf + 16 * warp, acc[m], kDnLf, wmma::mem_row_major);
    }
    __syncthreads();

    // gated RMSNorm of the output rows: warp w takes the tokens 8 w .. 8 w + 7, a lane four features
    for (int i = 8 * warp; i < 8 * warp + 8; ++i) {
      const int t = t0 + i;
      if (t >= t1) break;
      const float4 o = *reinterpret_cast<const float4*>(sF + i * kDnLf + 4 * lane);
      const float ss = dn_warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w);
      const float sc = rsqrtf(ss / (float)kDnD + a.eps);
      const uint2 zr = *reinterpret_cast<const uint2*>(a.z + (size_t)t * a.ld_z + h * kDnD + 4 * lane);
      const __nv_bfloat16* zb = reinterpret_cast<const __nv_bfloat16*>(&zr);
      const float4 nw = *reinterpret_cast<const float4*>(a.norm_w + 4 * lane);
      const float ov[4] = {o.x, o.y, o.z, o.w}, nv[4] = {nw.x, nw.y, nw.z, nw.w};
      __nv_bfloat16 y[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float zv = __bfloat162float(zb[e]);
        y[e] = __float2bfloat16(ov[e] * sc * nv[e] * (zv / (1.0f + __expf(-zv))));
      }
      *reinterpret_cast<uint2*>(a.out + ((size_t)t * a.dt_rank + h) * kDnD + 4 * lane) = *reinterpret_cast<const uint2*>(y);
    }

    // S = exp(c_last) S + U^T diag(exp(c_last - c_j)) K
#pragma unroll
    for (int f = 0; f < 8; ++f)
#pragma unroll
      for (int e = 0; e < S[f].num_elements; ++e) S[f].x[e] *= g_last;
    for (int kk = 0; kk < kDnC / 16; ++kk) {
      FragA fa;
      wmma::load_matrix_sync(fa, sUT + (16 * warp) * kDnLc + 16 * kk, kDnLc);
#pragma unroll
      for (int f = 0; f < 8; ++f) {
        FragB fb;
        wmma::load_matrix_sync(fb, sKdT + (16 * f) * kDnLc + 16 * kk, kDnLc);
        wmma::mma_sync(S[f], fa, fb, S[f]);
      }
    }
    __syncthreads();          // the next chunk's tiles overwrite what this one still read
  }
#pragma unroll
  for (int f = 0; f < 8; ++f) wmma::store_matrix_sync(st + (16 * warp) * kDnD + 16 * f, S[f], kDnD, wmma::mem_row_major);
}

// bytes of one workspace entry (chunk, head): three 64 x 128 tiles, one 128 x 64, one 64 x 64 (bf16) and the chunk's total decay
constexpr size_t kDnEntryBf16 = 3 * (size_t)kDnC * kDnD + (size_t)kDnD * kDnC + (size_t)kDnC * kDnC;

}  // namespace gb

using namespace gb;

// Upper bound of the chunks of `total_tokens` tokens in `n_seqs` sequences (each sequence may end in a partial chunk), and the
// workspace the chunked scan needs for it.
GB_API long gb_deltanet_chunk_workspace(long total_tokens, int n_seqs, int dt_rank) {
  const long chunks = total_tokens / kDnC + n_seqs;
  return chunks * dt_rank * (long)(kDnEntryBf16 * 2 + 4) + 1024;
}

GB_API int gb_deltanet_chunked(const void* qkv, int ld_qkv, const void* z, int ld_z, const float* ab, const float* a, const float* dt_bias,
                               const float* norm_w, float* state, const int* cu_q, const int* seq_slots, void* out, int n_group, int dt_rank,
                               int d_state, float eps, int n_seqs, long total_tokens, void* workspace, long workspace_bytes,
                               cudaStream_t stream) {
  if (n_seqs <= 0 || total_tokens <= 0) return 0;
  if (d_state != kDnD) return fail("deltanet_chunked: d_state must be 128%s");
  if (n_group <= 0 || dt_rank % n_group) return fail("deltanet_chunked: dt_rank must be a multiple of n_group%s");
  if ((ld_qkv % 4) || (ld_z % 4) || ((uintptr_t)qkv % 8) || ((uintptr_t)z % 8) || ((uintptr_t)out % 8) || ((uintptr_t)norm_w % 16) ||
      ((uintptr_t)state % 32))
    return fail("deltanet_chunked: rows must be 8-byte aligned (state 32, norm weights 16)%s");
  if (workspace == nullptr || workspace_bytes < gb_deltanet_chunk_workspace(total_tokens, n_seqs, dt_rank) || ((uintptr_t)workspace % 256))
    return fail("deltanet_chunked: workspace too small or not 256-byte aligned%s");
  const long chunks = total_tokens / kDnC + n_seqs;
  const size_t entries = (size_t)chunks * dt_rank;
  DnChunkArgs g;
  g.qkv = (const __nv_bfloat16*)qkv; g.ld_qkv = ld_qkv; g.z = (const __nv_bfloat16*)z; g.ld_z = ld_z; g.ab = ab; g.a = a; g.dt_bias = dt_bias;
  g.norm_w = norm_w; g.state = state; g.cu_q = cu_q; g.seq_slots = seq_slots; g.out = (__nv_bfloat16*)out; g.n_group = n_group;
  g.dt_rank = dt_rank; g.n_seqs = n_seqs; g.eps = eps;
  __nv_bfloat16* w = (__nv_bfloat16*)workspace;
  g.gq = w; w += entries * kDnC * kDnD;
  g.nw = w; w += entries * kDnC * kDnD;
  g.uv = w; w += entries * kDnC * kDnD;
  g.kdt = w; w += entries * kDnD * kDnC;
  g.mqk = w; w += entries * kDnC * kDnC;
  g.glast = (float*)w;
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA_OK(cudaFuncSetAttribute(dn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmem));
    GB_CUDA_OK(cudaFuncSetAttribute(dn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanSmem));
    attr_set = true;
  }
  launch_k(dn_chunk_prep_kernel, dim3((unsigned)chunks, dt_rank), kDnThreads, kPrepSmem, stream, g);
  GB_CUDA_OK(cudaGetLastError());
  launch_k(dn_chunk_scan_kernel, dim3(dt_rank, n_seqs), kDnThreads, kScanSmem, stream, g);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}
