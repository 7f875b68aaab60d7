// ggml block formats on the device: an element decoder for every tensor type a GGUF file can hold (the 24
// named quantisation formats, F32/F16/BF16, plus Q8_1, Q8_K, MXFP4, NVFP4, Q1_0), a whole-tensor
// dequantiser to bf16 (load-time conversion and the feed of the tensor-core GEMM for large batches) and a
// generic fused dequant-GEMV for small batches (weights stay quantised in HBM, one warp per output row).
//
// Replaces the reference's per-type kernels of cuda/llm/cuda_llm_runner.c: matvec_<type>_f32 (:116-4053),
// batch_matvec_<type> (:4433-7768), dequant_<type>_to_f16 (:999-5447) and the embed_<type> gathers (:933-1769).
// The formats themselves are the file format's (decoders on the host: csrc/host/dequant.cc, bit-exact against
// common/ggml_dequant.h).  The IQ codebooks are uploaded once per device with gb_set_codebook.
#include "sm100.cuh"
#include "host_common.h"

namespace gb {

enum GgmlType : int {
  T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8, T_Q8_1 = 9, T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12,
  T_Q5_K = 13, T_Q6_K = 14, T_Q8_K = 15, T_IQ2_XXS = 16, T_IQ2_XS = 17, T_IQ3_XXS = 18, T_IQ1_S = 19, T_IQ4_NL = 20, T_IQ3_S = 21,
  T_IQ2_S = 22, T_IQ4_XS = 23, T_IQ1_M = 29, T_BF16 = 30, T_TQ1_0 = 34, T_TQ2_0 = 35, T_MXFP4 = 39, T_NVFP4 = 40, T_Q1_0 = 41
};

__device__ uint8_t d_iq2xxs[256 * 8];
__device__ uint8_t d_iq2xs[512 * 8];
__device__ uint8_t d_iq2s[1024 * 8];
__device__ uint8_t d_iq3xxs[256 * 4];
__device__ uint8_t d_iq3s[512 * 4];
__device__ int8_t d_iq1s[2048 * 8];
__device__ uint8_t d_ksigns[128];

__device__ __constant__ int8_t c_iq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
__device__ __constant__ int8_t c_fp4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

__host__ __device__ inline void type_geometry(int t, int* blk, int* bytes) {
  switch (t) {
    case T_F32: *blk = 1; *bytes = 4; break; case T_F16: case T_BF16: *blk = 1; *bytes = 2; break;
    case T_Q4_0: *blk = 32; *bytes = 18; break; case T_Q4_1: *blk = 32; *bytes = 20; break; case T_Q5_0: *blk = 32; *bytes = 22; break;
    case T_Q5_1: *blk = 32; *bytes = 24; break; case T_Q8_0: *blk = 32; *bytes = 34; break; case T_Q8_1: *blk = 32; *bytes = 36; break;
    case T_Q2_K: *blk = 256; *bytes = 84; break; case T_Q3_K: *blk = 256; *bytes = 110; break; case T_Q4_K: *blk = 256; *bytes = 144; break;
    case T_Q5_K: *blk = 256; *bytes = 176; break; case T_Q6_K: *blk = 256; *bytes = 210; break; case T_Q8_K: *blk = 256; *bytes = 292; break;
    case T_IQ2_XXS: *blk = 256; *bytes = 66; break; case T_IQ2_XS: *blk = 256; *bytes = 74; break; case T_IQ3_XXS: *blk = 256; *bytes = 98; break;
    case T_IQ1_S: *blk = 256; *bytes = 50; break; case T_IQ4_NL: *blk = 32; *bytes = 18; break; case T_IQ3_S: *blk = 256; *bytes = 110; break;
    case T_IQ2_S: *blk = 256; *bytes = 82; break; case T_IQ4_XS: *blk = 256; *bytes = 136; break; case T_IQ1_M: *blk = 256; *bytes = 56; break;
    case T_TQ1_0: *blk = 256; *bytes = 54; break; case T_TQ2_0: *blk = 256; *bytes = 66; break; case T_MXFP4: *blk = 32; *bytes = 17; break;
    case T_NVFP4: *blk = 64; *bytes = 36; break; case T_Q1_0: *blk = 128; *bytes = 18; break;
    default: *blk = 0; *bytes = 0;
  }
}

__device__ __forceinline__ uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
__device__ __forceinline__ uint32_t rd32(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
__device__ __forceinline__ float rdh(const uint8_t* p) { return __half2float(__ushort_as_half(rd16(p))); }
__device__ __forceinline__ float sgn(uint8_t signs, int j) { return ((signs >> j) & 1) ? -1.f : 1.f; }

__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, int* sc, int* mn) {
  if (j < 4) { *sc = q[j] & 63; *mn = q[j + 4] & 63; }
  else { *sc = (q[j + 4] & 15) | ((q[j - 4] >> 6) << 4); *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}
__device__ __forceinline__ int q3k_scale(const uint8_t* sp, int j) {
  if (j < 4) return (sp[j] & 15) | ((sp[8 + j] & 3) << 4);
  if (j < 8) return (sp[j] & 15) | (((sp[4 + j] >> 2) & 3) << 4);
  if (j < 12) return (sp[j - 8] >> 4) | (((sp[j] >> 4) & 3) << 4);
  return (sp[j - 8] >> 4) | (((sp[j - 4] >> 6) & 3) << 4);
}

// Value of element i (0 <= i < block size) of the block at b.
__device__ float block_elem(int type, const uint8_t* b, int i) {
  switch (type) {
    case T_F32: return __uint_as_float(rd32(b));
    case T_F16: return rdh(b);
    case T_BF16: return __uint_as_float((uint32_t)rd16(b) << 16);
    case T_Q4_0: { const int j = i & 15; const int q = (i < 16) ? (b[2 + j] & 15) : (b[2 + j] >> 4); return (q - 8) * rdh(b); }
    case T_Q4_1: { const int j = i & 15; const int q = (i < 16) ? (b[4 + j] & 15) : (b[4 + j] >> 4); return q * rdh(b) + rdh(b + 2); }
    case T_Q5_0: {
      const int j = i & 15; const uint32_t qh = rd32(b + 2);
      const int q = (i < 16) ? ((b[6 + j] & 15) | (((qh >> j) << 4) & 0x10)) : ((b[6 + j] >> 4) | ((qh >> (j + 12)) & 0x10));
      return (q - 16) * rdh(b);
    }
    case T_Q5_1: {
      const int j = i & 15; const uint32_t qh = rd32(b + 4);
      const int q = (i < 16) ? ((b[8 + j] & 15) | (((qh >> j) << 4) & 0x10)) : ((b[8 + j] >> 4) | ((qh >> (j + 12)) & 0x10));
      return q * rdh(b) + rdh(b + 2);
    }
    case T_Q8_0: return (int8_t)b[2 + i] * rdh(b);
    case T_Q8_1: return (int8_t)b[4 + i] * rdh(b);
    case T_Q2_K: {
      const int n = i >> 7, rem = i & 127, sh = rem >> 5, half = (rem & 31) >> 4, l = rem & 15;
      const uint8_t sc = b[n * 8 + sh * 2 + half];
      const int q = (b[16 + n * 32 + l + 16 * half] >> (2 * sh)) & 3;
      return rdh(b + 80) * (sc & 15) * q - rdh(b + 82) * (sc >> 4);
    }
    case T_Q3_K: {
      const int n = i >> 7, rem = i & 127, sh = rem >> 5, half = (rem & 31) >> 4, l = (rem & 15) + 16 * half;
      const int sc = q3k_scale(b + 96, n * 8 + sh * 2 + half) - 32;
      const int q = ((b[32 + n * 32 + l] >> (2 * sh)) & 3) - ((b[l] & (1 << (n * 4 + sh))) ? 0 : 4);
      return rdh(b + 108) * sc * q;
    }
    case T_Q4_K: {
      const int j = i >> 6, rem = i & 63, hi = rem >> 5, l = rem & 31;
      int sc, mn; scale_min_k4(2 * j + hi, b + 4, &sc, &mn);
      const int q = hi ? (b[16 + 32 * j + l] >> 4) : (b[16 + 32 * j + l] & 15);
      return rdh(b) * sc * q - rdh(b + 2) * mn;
    }
    case T_Q5_K: {
      const int j = i >> 6, rem = i & 63, hi = rem >> 5, l = rem & 31;
      int sc, mn; scale_min_k4(2 * j + hi, b + 4, &sc, &mn);
      int q = hi ? (b[48 + 32 * j + l] >> 4) : (b[48 + 32 * j + l] & 15);
      if (b[16 + l] & (1 << (2 * j + hi))) q += 16;
      return rdh(b) * sc * q - rdh(b + 2) * mn;
    }
    case T_Q6_K: {
      const int n = i >> 7, rem = i & 127, qt = rem >> 5, l = rem & 31;
      const uint8_t lo = b[n * 64 + l + ((qt & 1) ? 32 : 0)];
      const int q = (int)(((qt & 2) ? (lo >> 4) : (lo & 15)) | (((b[128 + n * 32 + l] >> (2 * qt)) & 3) << 4)) - 32;
      return rdh(b + 208) * (int8_t)b[192 + n * 8 + (l >> 4) + 2 * qt] * q;
    }
    case T_Q8_K: return __uint_as_float(rd32(b)) * (int8_t)b[4 + i];
    case T_IQ2_XXS: {
      const int ib = i >> 5, l = (i & 31) >> 3, j = i & 7;
      const uint8_t* p = b + 2 + 8 * ib; const uint32_t aux = rd32(p + 4);
      return rdh(b) * (0.5f + (aux >> 28)) * 0.25f * d_iq2xxs[p[l] * 8 + j] * sgn(d_ksigns[(aux >> (7 * l)) & 127], j);
    }
    case T_IQ2_XS: {
      const int ib = i >> 5, l = (i & 31) >> 3, j = i & 7;
      const uint16_t v = rd16(b + 2 + 2 * (4 * ib + l)); const uint8_t s = b[66 + ib];
      const float db = rdh(b) * (0.5f + ((l < 2) ? (s & 15) : (s >> 4))) * 0.25f;
      return db * d_iq2xs[(v & 511) * 8 + j] * sgn(d_ksigns[v >> 9], j);
    }
    case T_IQ2_S: {
      const int ib = i >> 5, l = (i & 31) >> 3, j = i & 7;
      const uint8_t s = b[74 + ib];
      const float db = rdh(b) * (0.5f + ((l < 2) ? (s & 15) : (s >> 4))) * 0.25f;
      const int idx = b[2 + 4 * ib + l] | ((b[66 + ib] << (8 - 2 * l)) & 0x300);
      return db * d_iq2s[idx * 8 + j] * sgn(b[34 + 4 * ib + l], j);
    }
    case T_IQ3_XXS: {
      const int ib = i >> 5, l = (i & 31) >> 3, j = i & 7;
      const uint32_t aux = rd32(b + 66 + 4 * ib);
      const uint8_t g = b[2 + 8 * ib + 2 * l + (j >> 2)];
      return rdh(b) * (0.5f + (aux >> 28)) * 0.5f * d_iq3xxs[g * 4 + (j & 3)] * sgn(d_ksigns[(aux >> (7 * l)) & 127], j);
    }
    case T_IQ3_S: {
      const int ib = i >> 5, l = (i & 31) >> 3, j = i & 7;
      const uint8_t s = b[106 + (ib >> 1)];
      const float db = rdh(b) * (1 + 2 * ((ib & 1) ? (s >> 4) : (s & 15)));
      const uint8_t qh = b[66 + ib];
      const int idx = b[2 + 8 * ib + 2 * l + (j >> 2)] | ((qh << ((j >> 2) ? (7 - 2 * l) : (8 - 2 * l))) & 256);
      return db * d_iq3s[idx * 4 + (j & 3)] * sgn(b[74 + 4 * ib + l], j);
    }
    case T_IQ1_S: {
      const int ib = i >> 5, l = (i & 31) >> 3, j = i & 7;
      const uint16_t qh = rd16(b + 34 + 2 * ib);
      const float dl = rdh(b) * (2 * ((qh >> 12) & 7) + 1), delta = (qh & 0x8000) ? -0.125f : 0.125f;
      return dl * (d_iq1s[(b[2 + 4 * ib + l] | (((qh >> (3 * l)) & 7) << 8)) * 8 + j] + delta);
    }
    case T_IQ1_M: {
      const int ib = i >> 5, l = (i & 31) >> 3, j = i & 7;
      const uint16_t s0 = rd16(b + 48), s1 = rd16(b + 50), s2 = rd16(b + 52), s3 = rd16(b + 54);
      const uint16_t su = (uint16_t)((s0 >> 12) | ((s1 >> 8) & 0x00f0) | ((s2 >> 4) & 0x0f00) | (s3 & 0xf000));
      const float d = __half2float(__ushort_as_half(su));
      const uint16_t sc = rd16(b + 48 + 2 * (ib >> 1));
      const float dl = d * (2 * ((sc >> (6 * (ib & 1) + (l < 2 ? 0 : 3))) & 7) + 1);
      const uint8_t qh = b[32 + 2 * ib + (l >> 1)];
      const int idx = b[4 * ib + l] | (((l & 1) ? (qh << 4) : (qh << 8)) & 0x700);
      const float delta = (qh & ((l & 1) ? 0x80 : 0x08)) ? -0.125f : 0.125f;
      return dl * (d_iq1s[idx * 8 + j] + delta);
    }
    case T_IQ4_NL: { const int j = i & 15; return rdh(b) * c_iq4nl[(i < 16) ? (b[2 + j] & 15) : (b[2 + j] >> 4)]; }
    case T_IQ4_XS: {
      const int ib = i >> 5, r = i & 31, j = r & 15;
      const int ls = ((b[4 + (ib >> 1)] >> (4 * (ib & 1))) & 15) | (((rd16(b + 2) >> (2 * ib)) & 3) << 4);
      const uint8_t q = b[8 + 16 * ib + j];
      return rdh(b) * (ls - 32) * c_iq4nl[(r < 16) ? (q & 15) : (q >> 4)];
    }
    case T_TQ1_0: {
      const uint8_t pow3[5] = {1, 3, 9, 27, 81};
      uint8_t q;
      if (i < 160) q = (uint8_t)(b[i & 31] * pow3[i >> 5]);
      else if (i < 240) { const int ii = i - 160; q = (uint8_t)(b[32 + (ii & 15)] * pow3[ii >> 4]); }
      else { const int ii = i - 240; q = (uint8_t)(b[48 + (ii & 3)] * pow3[ii >> 2]); }
      return (float)((((uint16_t)q * 3) >> 8) - 1) * rdh(b + 52);
    }
    case T_TQ2_0: { const int j = (i >> 7) * 32, l = (i & 127) >> 5, m = i & 31; return (float)(((b[j + m] >> (2 * l)) & 3) - 1) * rdh(b + 64); }
    case T_MXFP4: {
      const uint8_t e = b[0]; const uint32_t bits = e < 2 ? (0x00200000u << e) : ((uint32_t)(e - 1) << 23);
      const int j = i & 15; return c_fp4[(i < 16) ? (b[1 + j] & 15) : (b[1 + j] >> 4)] * __uint_as_float(bits);
    }
    case T_NVFP4: {
      const int s = i >> 4, r = i & 15, j = r & 7; const uint8_t x = b[s];
      float d = 0.f;
      if (x != 0 && x != 0x7f) { const int e = (x >> 3) & 15, m = x & 7; d = (e == 0 ? ldexpf((float)m, -9) : ldexpf(1.f + m / 8.f, e - 7)) * 0.5f; }
      const uint8_t q = b[4 + 8 * s + j];
      return c_fp4[(r < 8) ? (q & 15) : (q >> 4)] * d;
    }
    case T_Q1_0: return ((b[2 + (i >> 3)] >> (i & 7)) & 1) ? rdh(b) : -rdh(b);
    default: return 0.f;
  }
}

// Whole tensor -> bf16, one thread per element (coalesced writes; reads hit the same block within a warp).
__global__ void __launch_bounds__(256)
dequant_bf16_kernel(const uint8_t* __restrict__ src, __nv_bfloat16* __restrict__ dst, long n, int type, int blk, int bytes) {
  pdl_wait();
  pdl_trigger();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long bi = i / blk;
  const int e = (int)(i - bi * blk);
  const uint8_t* b = src + bi * bytes;
  dst[i] = __float2bfloat16(block_elem(type, b, e));
}

// y[m, r] = sum_k W[r, k] x[m, k] for m < M <= 8: one warp per weight row, lanes stride over k (x loads coalesce).
template <int M>
__global__ void __launch_bounds__(256)
gemv_quant_kernel(const uint8_t* __restrict__ w, const __nv_bfloat16* __restrict__ x, float* __restrict__ y, int rows, int k, int type, int blk,
                  int bytes, long row_bytes, int ldx, int ldy) {
  pdl_wait();
  pdl_trigger();
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint8_t* wr = w + (size_t)r * row_bytes;
  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  for (int kk = lane; kk < k; kk += 32) {
    const int bi = kk / blk;
    const float wv = block_elem(type, wr + (size_t)bi * bytes, kk - bi * blk);
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] += wv * __bfloat162float(x[(size_t)m * ldx + kk]);
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const float s = warp_sum(acc[m]);
    if (lane == 0) y[(size_t)m * ldy + r] = s;
  }
}

}  // namespace gb

using namespace gb;

// which: 0 iq2xxs, 1 iq2xs, 2 iq2s, 3 iq3xxs, 4 iq3s, 5 iq1s, 6 sign table.  Call once per device before IQ types are decoded.
GB_API int gb_set_codebook(int which, const void* data, long bytes) {
  switch (which) {
    case 0: if (bytes != sizeof(d_iq2xxs)) break; GB_CUDA_OK(cudaMemcpyToSymbol(d_iq2xxs, data, bytes)); return 0;
    case 1: if (bytes != sizeof(d_iq2xs)) break; GB_CUDA_OK(cudaMemcpyToSymbol(d_iq2xs, data, bytes)); return 0;
    case 2: if (bytes != sizeof(d_iq2s)) break; GB_CUDA_OK(cudaMemcpyToSymbol(d_iq2s, data, bytes)); return 0;
    case 3: if (bytes != sizeof(d_iq3xxs)) break; GB_CUDA_OK(cudaMemcpyToSymbol(d_iq3xxs, data, bytes)); return 0;
    case 4: if (bytes != sizeof(d_iq3s)) break; GB_CUDA_OK(cudaMemcpyToSymbol(d_iq3s, data, bytes)); return 0;
    case 5: if (bytes != sizeof(d_iq1s)) break; GB_CUDA_OK(cudaMemcpyToSymbol(d_iq1s, data, bytes)); return 0;
    case 6: if (bytes != sizeof(d_ksigns)) break; GB_CUDA_OK(cudaMemcpyToSymbol(d_ksigns, data, bytes)); return 0;
    default: break;
  }
  return fail("set_codebook: bad table index or size%s (%ld, %ld bytes)", "", (long)which, bytes);
}

GB_API int gb_dequant_bf16(const void* src, void* dst, long n, int type, cudaStream_t stream) {
  int blk, bytes;
  type_geometry(type, &blk, &bytes);
  if (blk == 0) return fail("dequant: unsupported ggml type%s %ld", "", (long)type);
  if (n % blk) return fail("dequant: element count is not a multiple of the block size%s");
  if (n <= 0) return 0;
  launch_k(dequant_bf16_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, (const uint8_t*)src, (__nv_bfloat16*)dst, n, type, blk, bytes);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

// w: rows x k in ggml type `type` (row-major blocks), x: bf16 [m, ldx], y: f32 [m, ldy]; m <= 8.
GB_API int gb_gemv_quant(const void* w, const void* x, float* y, int rows, int k, int m, int type, int ldx, int ldy, cudaStream_t stream) {
  int blk, bytes;
  type_geometry(type, &blk, &bytes);
  if (blk == 0) return fail("gemv_quant: unsupported ggml type%s %ld", "", (long)type);
  if (k % blk) return fail("gemv_quant: k is not a multiple of the block size%s");
  if (m < 1 || m > 8) return fail("gemv_quant: batch must be 1..8%s");
  if (rows <= 0) return 0;
  const long row_bytes = (long)(k / blk) * bytes;
  const int blocks = (rows + 7) / 8;
#define GB_GEMV(MV) launch_k(gemv_quant_kernel<MV>, blocks, 256, 0, stream, (const uint8_t*)w, (const __nv_bfloat16*)x, y, rows, k, type, blk, bytes, row_bytes, ldx, ldy)
  switch (m) { case 1: GB_GEMV(1); break; case 2: GB_GEMV(2); break; case 3: GB_GEMV(3); break; case 4: GB_GEMV(4); break;
               case 5: GB_GEMV(5); break; case 6: GB_GEMV(6); break; case 7: GB_GEMV(7); break; default: GB_GEMV(8); }
#undef GB_GEMV
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}
