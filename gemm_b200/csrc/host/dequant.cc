// CPU dequantisers for every ggml tensor type that GGUF checkpoints use (the 24 named quantisation
// formats plus F32/F16/BF16 and the three newer ones: MXFP4, NVFP4, Q1_0), and quantisers for the formats
// the synthetic checkpoints and the fused GPU kernels need (Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, Q4_K, Q5_K, Q6_K,
// Q2_K, Q3_K, IQ4_NL, TQ2_0, F16, BF16).
//
// The arithmetic of each format is fixed by the file format; the reference implements the same
// decoders in common/ggml_dequant.h:1479-3265 (dispatcher :3177) and has no quantiser at all.
// Everything here is written against the format definition: block layouts are read with byte offsets,
// the IQ codebooks are rebuilt at start-up from compact base-3 / base-8 codes (iq_codebooks.inc).
#include "common.h"
#include "ggml_types.h"
#include "iq_codebooks.inc"
#include <math.h>
#include <string.h>
#include <algorithm>
#include <mutex>
#include <vector>

namespace gbh {

// ------------------------------------------------------------------------------------------ codebooks
static uint8_t g_iq2xxs[256][8], g_iq2xs[512][8], g_iq2s[1024][8], g_iq3xxs[256][4], g_iq3s[512][4];
static int8_t g_iq1s[2048][8];
static uint8_t g_ksigns[128];
static std::once_flag g_cb_once;

template <int N, typename T>
static void expand(const uint16_t* codes, int count, const uint8_t* alphabet, int base, T (*out)[N]) {
  for (int i = 0; i < count; ++i) {
    int c = codes[i];
    for (int j = 0; j < N; ++j) { out[i][j] = (T)alphabet[c % base]; c /= base; }
  }
}
static void expand_codebooks() {
  expand<8>(k_iq2xxs_codes, 256, k_iq2xxs_alphabet, 3, g_iq2xxs);
  expand<8>(k_iq2xs_codes, 512, k_iq2xs_alphabet, 3, g_iq2xs);
  expand<8>(k_iq2s_codes, 1024, k_iq2s_alphabet, 3, g_iq2s);
  expand<4>(k_iq3xxs_codes, 256, k_iq3xxs_alphabet, 8, g_iq3xxs);
  expand<4>(k_iq3s_codes, 512, k_iq3s_alphabet, 8, g_iq3s);
  expand<8>(k_iq1s_codes, 2048, k_iq1s_alphabet, 3, g_iq1s);
  for (int i = 0; i < 128; ++i) g_ksigns[i] = (uint8_t)(i | ((__builtin_popcount(i) & 1) << 7));   // 8th bit = parity
}
static inline void need_codebooks() { std::call_once(g_cb_once, expand_codebooks); }

static const int8_t k_iq4nl_values[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
static const int8_t k_fp4_values[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};   // e2m1 times two

static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static inline uint32_t rd32(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
static inline float rdh(const uint8_t* p) { return fp16_to_f32(rd16(p)); }
static inline void wr16(uint8_t* p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }

// 6-bit (scale, min) pair j of the 12 packed bytes shared by Q4_K and Q5_K
static inline void scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* mn) {
  if (j < 4) { *sc = q[j] & 63; *mn = q[j + 4] & 63; }
  else { *sc = (uint8_t)((q[j + 4] & 0x0f) | ((q[j - 4] >> 6) << 4)); *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}

// ------------------------------------------------------------------------------------------ decoders (one block each)
static void dq_q4_0(const uint8_t* b, float* y) { const float d = rdh(b); for (int j = 0; j < 16; ++j) { y[j] = ((b[2 + j] & 15) - 8) * d; y[j + 16] = ((b[2 + j] >> 4) - 8) * d; } }
static void dq_q4_1(const uint8_t* b, float* y) { const float d = rdh(b), m = rdh(b + 2); for (int j = 0; j < 16; ++j) { y[j] = (b[4 + j] & 15) * d + m; y[j + 16] = (b[4 + j] >> 4) * d + m; } }
static void dq_q5_0(const uint8_t* b, float* y) {
  const float d = rdh(b); const uint32_t qh = rd32(b + 2);
  for (int j = 0; j < 16; ++j) {
    const int h0 = ((qh >> j) << 4) & 0x10, h1 = (qh >> (j + 12)) & 0x10;
    y[j] = (((b[6 + j] & 15) | h0) - 16) * d; y[j + 16] = (((b[6 + j] >> 4) | h1) - 16) * d;
  }
}
static void dq_q5_1(const uint8_t* b, float* y) {
  const float d = rdh(b), m = rdh(b + 2); const uint32_t qh = rd32(b + 4);
  for (int j = 0; j < 16; ++j) {
    const int h0 = ((qh >> j) << 4) & 0x10, h1 = (qh >> (j + 12)) & 0x10;
    y[j] = ((b[8 + j] & 15) | h0) * d + m; y[j + 16] = ((b[8 + j] >> 4) | h1) * d + m;
  }
}
static void dq_q8_0(const uint8_t* b, float* y) { const float d = rdh(b); for (int j = 0; j < 32; ++j) y[j] = (int8_t)b[2 + j] * d; }
static void dq_q8_1(const uint8_t* b, float* y) { const float d = rdh(b); for (int j = 0; j < 32; ++j) y[j] = (int8_t)b[4 + j] * d; }
static void dq_q2_K(const uint8_t* b, float* y) {
  const uint8_t* scales = b; const uint8_t* q = b + 16; const float d = rdh(b + 80), dmin = rdh(b + 82);
  int is = 0;
  for (int n = 0; n < 256; n += 128) {
    for (int shift = 0; shift < 8; shift += 2) {
      for (int half = 0; half < 2; ++half) {
        const uint8_t sc = scales[is++];
        const float dl = d * (sc & 15), ml = dmin * (sc >> 4);
        for (int l = 0; l < 16; ++l) *y++ = dl * ((q[l + 16 * half] >> shift) & 3) - ml;
      }
    }
    q += 32;
  }
}
static void dq_q3_K(const uint8_t* b, float* y) {
  const uint8_t* hm = b; const uint8_t* q = b + 32; const uint8_t* sp = b + 96; const float d_all = rdh(b + 108);
  uint32_t a0 = rd32(sp), a1 = rd32(sp + 4), t = rd32(sp + 8), aux[4];
  const uint32_t m1 = 0x03030303u, m2 = 0x0f0f0f0fu;
  aux[0] = (a0 & m2) | (((t >> 0) & m1) << 4); aux[1] = (a1 & m2) | (((t >> 2) & m1) << 4);
  aux[2] = ((a0 >> 4) & m2) | (((t >> 4) & m1) << 4); aux[3] = ((a1 >> 4) & m2) | (((t >> 6) & m1) << 4);
  int8_t scales[16];
  memcpy(scales, aux, 16);
  int is = 0; uint8_t m = 1;
  for (int n = 0; n < 256; n += 128) {
    for (int shift = 0; shift < 8; shift += 2) {
      for (int half = 0; half < 2; ++half) {
        const float dl = d_all * (scales[is++] - 32);
        for (int l = 0; l < 16; ++l) { const int li = l + 16 * half; *y++ = dl * ((int)((q[li] >> shift) & 3) - ((hm[li] & m) ? 0 : 4)); }
      }
      m <<= 1;
    }
    q += 32;
  }
}
static void dq_q4_K(const uint8_t* b, float* y) {
  const float d = rdh(b), dmin = rdh(b + 2); const uint8_t* sc = b + 4; const uint8_t* q = b + 16;
  int is = 0;
  for (int j = 0; j < 256; j += 64) {
    uint8_t s1, mn1, s2, mn2;
    scale_min_k4(is, sc, &s1, &mn1); scale_min_k4(is + 1, sc, &s2, &mn2);
    const float d1 = d * s1, m1 = dmin * mn1, d2 = d * s2, m2 = dmin * mn2;
    for (int l = 0; l < 32; ++l) *y++ = d1 * (q[l] & 15) - m1;
    for (int l = 0; l < 32; ++l) *y++ = d2 * (q[l] >> 4) - m2;
    q += 32; is += 2;
  }
}
static void dq_q5_K(const uint8_t* b, float* y) {
  const float d = rdh(b), dmin = rdh(b + 2); const uint8_t* sc = b + 4; const uint8_t* qh = b + 16; const uint8_t* ql = b + 48;
  int is = 0; uint8_t u1 = 1, u2 = 2;
  for (int j = 0; j < 256; j += 64) {
    uint8_t s1, mn1, s2, mn2;
    scale_min_k4(is, sc, &s1, &mn1); scale_min_k4(is + 1, sc, &s2, &mn2);
    const float d1 = d * s1, m1 = dmin * mn1, d2 = d * s2, m2 = dmin * mn2;
    for (int l = 0; l < 32; ++l) *y++ = d1 * ((ql[l] & 15) + ((qh[l] & u1) ? 16 : 0)) - m1;
    for (int l = 0; l < 32; ++l) *y++ = d2 * ((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
    ql += 32; is += 2; u1 <<= 2; u2 <<= 2;
  }
}
static void dq_q6_K(const uint8_t* b, float* y) {
  const uint8_t* ql = b; const uint8_t* qh = b + 128; const int8_t* sc = (const int8_t*)(b + 192); const float d = rdh(b + 208);
  for (int n = 0; n < 256; n += 128) {
    for (int l = 0; l < 32; ++l) {
      const int is = l / 16;
      const int q1 = (int)((ql[l] & 15) | (((qh[l] >> 0) & 3) << 4)) - 32, q2 = (int)((ql[l + 32] & 15) | (((qh[l] >> 2) & 3) << 4)) - 32;
      const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32, q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
      y[l] = d * sc[is] * q1; y[l + 32] = d * sc[is + 2] * q2; y[l + 64] = d * sc[is + 4] * q3; y[l + 96] = d * sc[is + 6] * q4;
    }
    y += 128; ql += 64; qh += 32; sc += 8;
  }
}
static void dq_q8_K(const uint8_t* b, float* y) { float d; memcpy(&d, b, 4); for (int j = 0; j < 256; ++j) y[j] = d * (int8_t)b[4 + j]; }
static void dq_iq2_xxs(const uint8_t* b, float* y) {
  const float d = rdh(b);
  for (int ib = 0; ib < 8; ++ib) {
    const uint8_t* p = b + 2 + 8 * ib;
    const uint32_t aux1 = rd32(p + 4);
    const float db = d * (0.5f + (aux1 >> 28)) * 0.25f;
    for (int l = 0; l < 4; ++l) {
      const uint8_t* grid = g_iq2xxs[p[l]];
      const uint8_t signs = g_ksigns[(aux1 >> (7 * l)) & 127];
      for (int j = 0; j < 8; ++j) *y++ = db * grid[j] * ((signs >> j) & 1 ? -1.f : 1.f);
    }
  }
}
static void dq_iq2_xs(const uint8_t* b, float* y) {
  const float d = rdh(b); const uint8_t* scales = b + 66;
  for (int ib = 0; ib < 8; ++ib) {
    const float db[2] = {d * (0.5f + (scales[ib] & 15)) * 0.25f, d * (0.5f + (scales[ib] >> 4)) * 0.25f};
    for (int l = 0; l < 4; ++l) {
      const uint16_t v = rd16(b + 2 + 2 * (4 * ib + l));
      const uint8_t* grid = g_iq2xs[v & 511];
      const uint8_t signs = g_ksigns[v >> 9];
      for (int j = 0; j < 8; ++j) *y++ = db[l / 2] * grid[j] * ((signs >> j) & 1 ? -1.f : 1.f);
    }
  }
}
static void dq_iq2_s(const uint8_t* b, float* y) {
  const float d = rdh(b); const uint8_t* qs = b + 2; const uint8_t* signs = qs + 32; const uint8_t* qh = b + 66; const uint8_t* scales = b + 74;
  for (int ib = 0; ib < 8; ++ib) {
    const float db[2] = {d * (0.5f + (scales[ib] & 15)) * 0.25f, d * (0.5f + (scales[ib] >> 4)) * 0.25f};
    for (int l = 0; l < 4; ++l) {
      const uint8_t* grid = g_iq2s[qs[l] | ((qh[ib] << (8 - 2 * l)) & 0x300)];
      for (int j = 0; j < 8; ++j) *y++ = db[l / 2] * grid[j] * ((signs[l] >> j) & 1 ? -1.f : 1.f);
    }
    qs += 4; signs += 4;
  }
}
static void dq_iq3_xxs(const uint8_t* b, float* y) {
  const float d = rdh(b); const uint8_t* qs = b + 2; const uint8_t* sas = b + 2 + 64;
  for (int ib = 0; ib < 8; ++ib) {
    const uint32_t aux = rd32(sas + 4 * ib);
    const float db = d * (0.5f + (aux >> 28)) * 0.5f;
    for (int l = 0; l < 4; ++l) {
      const uint8_t signs = g_ksigns[(aux >> (7 * l)) & 127];
      const uint8_t* g1 = g_iq3xxs[qs[2 * l]]; const uint8_t* g2 = g_iq3xxs[qs[2 * l + 1]];
      for (int j = 0; j < 4; ++j) { y[j] = db * g1[j] * ((signs >> j) & 1 ? -1.f : 1.f); y[j + 4] = db * g2[j] * ((signs >> (j + 4)) & 1 ? -1.f : 1.f); }
      y += 8;
    }
    qs += 8;
  }
}
static void dq_iq3_s(const uint8_t* b, float* y) {
  const float d = rdh(b); const uint8_t* qs = b + 2; const uint8_t* qh = b + 66; const uint8_t* signs = b + 74; const uint8_t* scales = b + 106;
  for (int ib = 0; ib < 8; ib += 2) {
    const float dbs[2] = {d * (1 + 2 * (scales[ib / 2] & 15)), d * (1 + 2 * (scales[ib / 2] >> 4))};
    for (int half = 0; half < 2; ++half) {
      for (int l = 0; l < 4; ++l) {
        const uint8_t* g1 = g_iq3s[qs[2 * l] | ((qh[half] << (8 - 2 * l)) & 256)];
        const uint8_t* g2 = g_iq3s[qs[2 * l + 1] | ((qh[half] << (7 - 2 * l)) & 256)];
        for (int j = 0; j < 4; ++j) { y[j] = dbs[half] * g1[j] * ((signs[l] >> j) & 1 ? -1.f : 1.f); y[j + 4] = dbs[half] * g2[j] * ((signs[l] >> (j + 4)) & 1 ? -1.f : 1.f); }
        y += 8;
      }
      qs += 8; signs += 4;
    }
    qh += 2;
  }
}
static void dq_iq1_s(const uint8_t* b, float* y) {
  const float d = rdh(b); const uint8_t* qs = b + 2;
  for (int ib = 0; ib < 8; ++ib) {
    const uint16_t qh = rd16(b + 34 + 2 * ib);
    const float dl = d * (2 * ((qh >> 12) & 7) + 1), delta = (qh & 0x8000) ? -0.125f : 0.125f;
    for (int l = 0; l < 4; ++l) {
      const int8_t* grid = g_iq1s[qs[l] | (((qh >> (3 * l)) & 7) << 8)];
      for (int j = 0; j < 8; ++j) *y++ = dl * (grid[j] + delta);
    }
    qs += 4;
  }
}
static void dq_iq1_m(const uint8_t* b, float* y) {
  const uint8_t* qs = b; const uint8_t* qh = b + 32;
  uint16_t sc[4];
  for (int i = 0; i < 4; ++i) sc[i] = rd16(b + 48 + 2 * i);
  const uint16_t su = (uint16_t)((sc[0] >> 12) | ((sc[1] >> 8) & 0x00f0) | ((sc[2] >> 4) & 0x0f00) | (sc[3] & 0xf000));
  const float d = fp16_to_f32(su);
  for (int ib = 0; ib < 8; ++ib) {
    const float dl1 = d * (2 * ((sc[ib / 2] >> (6 * (ib % 2) + 0)) & 7) + 1), dl2 = d * (2 * ((sc[ib / 2] >> (6 * (ib % 2) + 3)) & 7) + 1);
    const int idx[4] = {qs[0] | ((qh[0] << 8) & 0x700), qs[1] | ((qh[0] << 4) & 0x700), qs[2] | ((qh[1] << 8) & 0x700), qs[3] | ((qh[1] << 4) & 0x700)};
    const float delta[4] = {(qh[0] & 0x08) ? -0.125f : 0.125f, (qh[0] & 0x80) ? -0.125f : 0.125f, (qh[1] & 0x08) ? -0.125f : 0.125f, (qh[1] & 0x80) ? -0.125f : 0.125f};
    for (int l = 0; l < 4; ++l) {
      const int8_t* grid = g_iq1s[idx[l]];
      const float dl = l < 2 ? dl1 : dl2;
      for (int j = 0; j < 8; ++j) *y++ = dl * (grid[j] + delta[l]);
    }
    qs += 4; qh += 2;
  }
}
static void dq_iq4_nl(const uint8_t* b, float* y) { const float d = rdh(b); for (int j = 0; j < 16; ++j) { y[j] = d * k_iq4nl_values[b[2 + j] & 15]; y[j + 16] = d * k_iq4nl_values[b[2 + j] >> 4]; } }
static void dq_iq4_xs(const uint8_t* b, float* y) {
  const float d = rdh(b); const uint16_t sh = rd16(b + 2); const uint8_t* sl = b + 4; const uint8_t* qs = b + 8;
  for (int ib = 0; ib < 8; ++ib) {
    const int ls = ((sl[ib / 2] >> (4 * (ib % 2))) & 15) | (((sh >> (2 * ib)) & 3) << 4);
    const float dl = d * (ls - 32);
    for (int j = 0; j < 16; ++j) { y[j] = dl * k_iq4nl_values[qs[j] & 15]; y[j + 16] = dl * k_iq4nl_values[qs[j] >> 4]; }
    y += 32; qs += 16;
  }
}
static void dq_tq1_0(const uint8_t* b, float* y) {
  static const uint8_t pow3[5] = {1, 3, 9, 27, 81};
  const uint8_t* qs = b; const uint8_t* qh = b + 48; const float d = rdh(b + 52);
  for (int n = 0; n < 5; ++n) for (int m = 0; m < 32; ++m) { const uint8_t q = (uint8_t)(qs[m] * pow3[n]); *y++ = (float)((((uint16_t)q * 3) >> 8) - 1) * d; }
  for (int n = 0; n < 5; ++n) for (int m = 0; m < 16; ++m) { const uint8_t q = (uint8_t)(qs[32 + m] * pow3[n]); *y++ = (float)((((uint16_t)q * 3) >> 8) - 1) * d; }
  for (int n = 0; n < 4; ++n) for (int j = 0; j < 4; ++j) { const uint8_t q = (uint8_t)(qh[j] * pow3[n]); *y++ = (float)((((uint16_t)q * 3) >> 8) - 1) * d; }
}
static void dq_tq2_0(const uint8_t* b, float* y) {
  const float d = rdh(b + 64);
  for (int j = 0; j < 64; j += 32) for (int l = 0; l < 4; ++l) for (int m = 0; m < 32; ++m) *y++ = (float)(((b[j + m] >> (l * 2)) & 3) - 1) * d;
}
static inline float e8m0_half(uint8_t x) { const uint32_t bits = x < 2 ? (0x00200000u << x) : ((uint32_t)(x - 1) << 23); float f; memcpy(&f, &bits, 4); return f; }
static inline float ue4m3_half(uint8_t x) {
  if (x == 0 || x == 0x7f) return 0.f;
  const int e = (x >> 3) & 15, m = x & 7;
  return (e == 0 ? ldexpf((float)m, -9) : ldexpf(1.f + m / 8.f, e - 7)) * 0.5f;
}
static void dq_mxfp4(const uint8_t* b, float* y) { const float d = e8m0_half(b[0]); for (int j = 0; j < 16; ++j) { y[j] = k_fp4_values[b[1 + j] & 15] * d; y[j + 16] = k_fp4_values[b[1 + j] >> 4] * d; } }
static void dq_nvfp4(const uint8_t* b, float* y) {
  for (int s = 0; s < 4; ++s) {
    const float d = ue4m3_half(b[s]); const uint8_t* qs = b + 4 + 8 * s;
    for (int j = 0; j < 8; ++j) { y[16 * s + j] = k_fp4_values[qs[j] & 15] * d; y[16 * s + j + 8] = k_fp4_values[qs[j] >> 4] * d; }
  }
}
static void dq_q1_0(const uint8_t* b, float* y) { const float d = rdh(b); for (int j = 0; j < 128; ++j) y[j] = ((b[2 + (j >> 3)] >> (j & 7)) & 1) ? d : -d; }

typedef void (*BlockFn)(const uint8_t*, float*);
static BlockFn block_decoder(int t) {
  switch (t) {
    case T_Q4_0: return dq_q4_0; case T_Q4_1: return dq_q4_1; case T_Q5_0: return dq_q5_0; case T_Q5_1: return dq_q5_1;
    case T_Q8_0: return dq_q8_0; case T_Q8_1: return dq_q8_1; case T_Q2_K: return dq_q2_K; case T_Q3_K: return dq_q3_K;
    case T_Q4_K: return dq_q4_K; case T_Q5_K: return dq_q5_K; case T_Q6_K: return dq_q6_K; case T_Q8_K: return dq_q8_K;
    case T_IQ2_XXS: return dq_iq2_xxs; case T_IQ2_XS: return dq_iq2_xs; case T_IQ2_S: return dq_iq2_s; case T_IQ3_XXS: return dq_iq3_xxs;
    case T_IQ3_S: return dq_iq3_s; case T_IQ1_S: return dq_iq1_s; case T_IQ1_M: return dq_iq1_m; case T_IQ4_NL: return dq_iq4_nl;
    case T_IQ4_XS: return dq_iq4_xs; case T_TQ1_0: return dq_tq1_0; case T_TQ2_0: return dq_tq2_0; case T_MXFP4: return dq_mxfp4;
    case T_NVFP4: return dq_nvfp4; case T_Q1_0: return dq_q1_0;
    default: return nullptr;
  }
}

int dequant_row(int type, const void* src, float* dst, long n) {
  const TypeInfo* ti = type_info(type);
  if (!ti) return fail("dequant: unknown ggml type %d", type);
  if (n % ti->block) return fail("dequant: %ld elements is not a multiple of the %s block (%d)", n, ti->name, ti->block);
  const uint8_t* s = (const uint8_t*)src;
  switch (type) {
    case T_F32: memcpy(dst, src, (size_t)n * 4); return 0;
    case T_F16: for (long i = 0; i < n; ++i) dst[i] = fp16_to_f32(rd16(s + 2 * i)); return 0;
    case T_BF16: for (long i = 0; i < n; ++i) dst[i] = bf16_to_f32(rd16(s + 2 * i)); return 0;
    case T_I8: for (long i = 0; i < n; ++i) dst[i] = (int8_t)s[i]; return 0;
    case T_I16: for (long i = 0; i < n; ++i) dst[i] = (int16_t)rd16(s + 2 * i); return 0;
    case T_I32: for (long i = 0; i < n; ++i) dst[i] = (float)(int32_t)rd32(s + 4 * i); return 0;
    case T_F64: for (long i = 0; i < n; ++i) { double d; memcpy(&d, s + 8 * i, 8); dst[i] = (float)d; } return 0;
    default: break;
  }
  BlockFn fn = block_decoder(type);
  if (!fn) return fail("dequant: type %s has no decoder", ti->name);
  need_codebooks();
  const long nb = n / ti->block;
  for (long i = 0; i < nb; ++i) fn(s + (size_t)i * ti->bytes, dst + i * ti->block);
  return 0;
}

// ------------------------------------------------------------------------------------------ quantisers
static inline int nearest_int(float f) { return (int)lrintf(f); }

static void q_q8_0(const float* x, uint8_t* b) {
  float amax = 0.f;
  for (int j = 0; j < 32; ++j) amax = std::max(amax, fabsf(x[j]));
  const float d = amax / 127.f, id = d ? 1.f / d : 0.f;
  wr16(b, f32_to_fp16(d));
  for (int j = 0; j < 32; ++j) b[2 + j] = (uint8_t)(int8_t)nearest_int(x[j] * id);
}
static void q_q4_0(const float* x, uint8_t* b) {
  float amax = 0.f, mx = 0.f;
  for (int j = 0; j < 32; ++j) if (fabsf(x[j]) > amax) { amax = fabsf(x[j]); mx = x[j]; }
  const float d = mx / -8.f, id = d ? 1.f / d : 0.f;
  wr16(b, f32_to_fp16(d));
  for (int j = 0; j < 16; ++j) {
    const int a = std::min(15, (int)(x[j] * id + 8.5f)), c = std::min(15, (int)(x[j + 16] * id + 8.5f));
    b[2 + j] = (uint8_t)(a | (c << 4));
  }
}
static void q_q4_1(const float* x, uint8_t* b) {
  float mn = x[0], mx = x[0];
  for (int j = 1; j < 32; ++j) { mn = std::min(mn, x[j]); mx = std::max(mx, x[j]); }
  const float d = (mx - mn) / 15.f, id = d ? 1.f / d : 0.f;
  wr16(b, f32_to_fp16(d)); wr16(b + 2, f32_to_fp16(mn));
  for (int j = 0; j < 16; ++j) {
    const int a = std::min(15, (int)((x[j] - mn) * id + 0.5f)), c = std::min(15, (int)((x[j + 16] - mn) * id + 0.5f));
    b[4 + j] = (uint8_t)(a | (c << 4));
  }
}
static void q_q5_0(const float* x, uint8_t* b) {
  float amax = 0.f, mx = 0.f;
  for (int j = 0; j < 32; ++j) if (fabsf(x[j]) > amax) { amax = fabsf(x[j]); mx = x[j]; }
  const float d = mx / -16.f, id = d ? 1.f / d : 0.f;
  wr16(b, f32_to_fp16(d));
  uint32_t qh = 0;
  for (int j = 0; j < 16; ++j) {
    const int a = std::min(31, (int)(x[j] * id + 16.5f)), c = std::min(31, (int)(x[j + 16] * id + 16.5f));
    b[6 + j] = (uint8_t)((a & 15) | ((c & 15) << 4));
    qh |= (uint32_t)((a & 16) >> 4) << j;
    qh |= (uint32_t)((c & 16) >> 4) << (j + 16);
  }
  memcpy(b + 2, &qh, 4);
}
static void q_q5_1(const float* x, uint8_t* b) {
  float mn = x[0], mx = x[0];
  for (int j = 1; j < 32; ++j) { mn = std::min(mn, x[j]); mx = std::max(mx, x[j]); }
  const float d = (mx - mn) / 31.f, id = d ? 1.f / d : 0.f;
  wr16(b, f32_to_fp16(d)); wr16(b + 2, f32_to_fp16(mn));
  uint32_t qh = 0;
  for (int j = 0; j < 16; ++j) {
    const int a = std::min(31, (int)((x[j] - mn) * id + 0.5f)), c = std::min(31, (int)((x[j + 16] - mn) * id + 0.5f));
    b[8 + j] = (uint8_t)((a & 15) | ((c & 15) << 4));
    qh |= (uint32_t)((a & 16) >> 4) << j;
    qh |= (uint32_t)((c & 16) >> 4) << (j + 16);
  }
  memcpy(b + 4, &qh, 4);
}

// (scale, min) of one sub-block quantised to integers in [0, nmax]: least-squares refinement of min/max.
static float make_qkx(int n, int nmax, const float* x, uint8_t* L, float* the_min) {
  float mn = x[0], mx = x[0];
  for (int i = 1; i < n; ++i) { mn = std::min(mn, x[i]); mx = std::max(mx, x[i]); }
  if (mn > 0) mn = 0;
  if (mx == mn) { for (int i = 0; i < n; ++i) L[i] = 0; *the_min = -mn; return 0.f; }
  float iscale = nmax / (mx - mn), scale = 1 / iscale;
  for (int it = 0; it < 5; ++it) {
    float sumlx = 0; int suml2 = 0; bool changed = false;
    for (int i = 0; i < n; ++i) {
      int l = std::max(0, std::min(nmax, nearest_int(iscale * (x[i] - mn))));
      if (l != L[i]) { L[i] = (uint8_t)l; changed = true; }
      sumlx += (x[i] - mn) * l; suml2 += l * l;
    }
    scale = suml2 ? sumlx / suml2 : scale;
    float sum = 0;
    for (int i = 0; i < n; ++i) sum += x[i] - scale * L[i];
    mn = std::min(0.f, sum / n);
    iscale = scale ? 1 / scale : 0.f;
    if (!changed) break;
  }
  *the_min = -mn;
  return scale;
}

static void pack_scales_k4(const uint8_t* ls, const uint8_t* lm, uint8_t* out) {
  for (int j = 0; j < 8; ++j) {
    if (j < 4) { out[j] = ls[j]; out[j + 4] = lm[j]; }
    else { out[j + 4] = (uint8_t)((ls[j] & 15) | ((lm[j] & 15) << 4)); out[j - 4] |= (uint8_t)((ls[j] >> 4) << 6); out[j] |= (uint8_t)((lm[j] >> 4) << 6); }
  }
}

static void q_q4_K(const float* x, uint8_t* b) {
  uint8_t L[256], ls[8], lm[8];
  float scales[8], mins[8], max_scale = 0, max_min = 0;
  for (int j = 0; j < 8; ++j) {
    memset(L + 32 * j, 0, 32);
    scales[j] = make_qkx(32, 15, x + 32 * j, L + 32 * j, &mins[j]);
    max_scale = std::max(max_scale, scales[j]); max_min = std::max(max_min, mins[j]);
  }
  const float inv_s = max_scale > 0 ? 63.f / max_scale : 0.f, inv_m = max_min > 0 ? 63.f / max_min : 0.f;
  for (int j = 0; j < 8; ++j) { ls[j] = (uint8_t)std::min(63, nearest_int(inv_s * scales[j])); lm[j] = (uint8_t)std::min(63, nearest_int(inv_m * mins[j])); }
  const uint16_t dh = f32_to_fp16(max_scale / 63.f), mh = f32_to_fp16(max_min / 63.f);
  wr16(b, dh); wr16(b + 2, mh);
  memset(b + 4, 0, 12);
  pack_scales_k4(ls, lm, b + 4);
  const float d = fp16_to_f32(dh), dm = fp16_to_f32(mh);
  for (int j = 0; j < 8; ++j) {
    const float dd = d * ls[j], mm = dm * lm[j];
    if (!dd) { memset(L + 32 * j, 0, 32); continue; }
    for (int i = 0; i < 32; ++i) L[32 * j + i] = (uint8_t)std::max(0, std::min(15, nearest_int((x[32 * j + i] + mm) / dd)));
  }
  uint8_t* q = b + 16;
  for (int j = 0; j < 256; j += 64) { for (int l = 0; l < 32; ++l) q[l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 4)); q += 32; }
}
static void q_q5_K(const float* x, uint8_t* b) {
  uint8_t L[256], ls[8], lm[8];
  float scales[8], mins[8], max_scale = 0, max_min = 0;
  for (int j = 0; j < 8; ++j) {
    memset(L + 32 * j, 0, 32);
    scales[j] = make_qkx(32, 31, x + 32 * j, L + 32 * j, &mins[j]);
    max_scale = std::max(max_scale, scales[j]); max_min = std::max(max_min, mins[j]);
  }
  const float inv_s = max_scale > 0 ? 63.f / max_scale : 0.f, inv_m = max_min > 0 ? 63.f / max_min : 0.f;
  for (int j = 0; j < 8; ++j) { ls[j] = (uint8_t)std::min(63, nearest_int(inv_s * scales[j])); lm[j] = (uint8_t)std::min(63, nearest_int(inv_m * mins[j])); }
  const uint16_t dh = f32_to_fp16(max_scale / 63.f), mh = f32_to_fp16(max_min / 63.f);
  wr16(b, dh); wr16(b + 2, mh);
  memset(b + 4, 0, 12);
  pack_scales_k4(ls, lm, b + 4);
  const float d = fp16_to_f32(dh), dm = fp16_to_f32(mh);
  for (int j = 0; j < 8; ++j) {
    const float dd = d * ls[j], mm = dm * lm[j];
    if (!dd) { memset(L + 32 * j, 0, 32); continue; }
    for (int i = 0; i < 32; ++i) L[32 * j + i] = (uint8_t)std::max(0, std::min(31, nearest_int((x[32 * j + i] + mm) / dd)));
  }
  uint8_t* qh = b + 16; uint8_t* ql = b + 48;
  memset(qh, 0, 32);
  uint8_t m1 = 1, m2 = 2;
  for (int n = 0; n < 256; n += 64) {
    for (int j = 0; j < 32; ++j) {
      int l1 = L[n + j], l2 = L[n + j + 32];
      if (l1 > 15) { l1 -= 16; qh[j] |= m1; }
      if (l2 > 15) { l2 -= 16; qh[j] |= m2; }
      ql[j] = (uint8_t)(l1 | (l2 << 4));
    }
    m1 <<= 2; m2 <<= 2; ql += 32;
  }
}
// symmetric sub-block scale for integers in [-nmax, nmax-1]
static float make_qx(int n, int nmax, const float* x, int8_t* L) {
  float amax = 0, mx = 0;
  for (int i = 0; i < n; ++i) if (fabsf(x[i]) > amax) { amax = fabsf(x[i]); mx = x[i]; }
  if (amax < 1e-30f) { for (int i = 0; i < n; ++i) L[i] = 0; return 0.f; }
  const float iscale = -nmax / mx;
  float sumlx = 0, suml2 = 0;
  for (int i = 0; i < n; ++i) {
    const int l = std::max(-nmax, std::min(nmax - 1, nearest_int(iscale * x[i])));
    L[i] = (int8_t)l; sumlx += x[i] * l; suml2 += (float)l * l;
  }
  return suml2 ? sumlx / suml2 : 0.f;
}
static void q_q6_K(const float* x, uint8_t* b) {
  int8_t L[256]; float scales[16], max_scale = 0, max_abs = 0;
  for (int ib = 0; ib < 16; ++ib) {
    scales[ib] = make_qx(16, 32, x + 16 * ib, L + 16 * ib);
    if (fabsf(scales[ib]) > max_abs) { max_abs = fabsf(scales[ib]); max_scale = scales[ib]; }
  }
  uint8_t* ql = b; uint8_t* qh = b + 128; int8_t* sc = (int8_t*)(b + 192);
  if (max_abs < 1e-30f) { memset(b, 0, 210); return; }
  const float iscale = -128.f / max_scale;
  const uint16_t dh = f32_to_fp16(1 / iscale);
  wr16(b + 208, dh);
  for (int ib = 0; ib < 16; ++ib) sc[ib] = (int8_t)std::min(127, nearest_int(iscale * scales[ib]));
  const float dd = fp16_to_f32(dh);
  uint8_t Lu[256];
  for (int j = 0; j < 16; ++j) {
    const float d = dd * sc[j];
    for (int i = 0; i < 16; ++i) {
      int l = d ? nearest_int(x[16 * j + i] / d) : 0;
      Lu[16 * j + i] = (uint8_t)(std::max(-32, std::min(31, l)) + 32);
    }
  }
  for (int n = 0; n < 256; n += 128) {
    for (int l = 0; l < 32; ++l) {
      const uint8_t q1 = Lu[n + l] & 15, q2 = Lu[n + l + 32] & 15, q3 = Lu[n + l + 64] & 15, q4 = Lu[n + l + 96] & 15;
      ql[l] = (uint8_t)(q1 | (q3 << 4)); ql[l + 32] = (uint8_t)(q2 | (q4 << 4));
      qh[l] = (uint8_t)((Lu[n + l] >> 4) | ((Lu[n + l + 32] >> 4) << 2) | ((Lu[n + l + 64] >> 4) << 4) | ((Lu[n + l + 96] >> 4) << 6));
    }
    ql += 64; qh += 32;
  }
}
static void q_q2_K(const float* x, uint8_t* b) {
  uint8_t L[256]; float scales[16], mins[16], max_scale = 0, max_min = 0;
  for (int j = 0; j < 16; ++j) {
    memset(L + 16 * j, 0, 16);
    scales[j] = make_qkx(16, 3, x + 16 * j, L + 16 * j, &mins[j]);
    max_scale = std::max(max_scale, scales[j]); max_min = std::max(max_min, mins[j]);
  }
  uint8_t* sc = b; uint8_t* qs = b + 16;
  const float is = max_scale > 0 ? 15.f / max_scale : 0.f, im = max_min > 0 ? 15.f / max_min : 0.f;
  for (int j = 0; j < 16; ++j) sc[j] = (uint8_t)(std::min(15, nearest_int(is * scales[j])) | (std::min(15, nearest_int(im * mins[j])) << 4));
  const uint16_t dh = f32_to_fp16(max_scale / 15.f), mh = f32_to_fp16(max_min / 15.f);
  wr16(b + 80, dh); wr16(b + 82, mh);
  const float d = fp16_to_f32(dh), dm = fp16_to_f32(mh);
  for (int j = 0; j < 16; ++j) {
    const float dd = d * (sc[j] & 15), mm = dm * (sc[j] >> 4);
    for (int i = 0; i < 16; ++i) L[16 * j + i] = dd ? (uint8_t)std::max(0, std::min(3, nearest_int((x[16 * j + i] + mm) / dd))) : 0;
  }
  for (int n = 0; n < 256; n += 128) { for (int l = 0; l < 32; ++l) qs[l] = (uint8_t)(L[n + l] | (L[n + l + 32] << 2) | (L[n + l + 64] << 4) | (L[n + l + 96] << 6)); qs += 32; }
}
static void q_q3_K(const float* x, uint8_t* b) {
  int8_t L[256]; float scales[16], max_scale = 0, amax = 0;
  for (int j = 0; j < 16; ++j) {
    scales[j] = make_qx(16, 4, x + 16 * j, L + 16 * j);
    if (fabsf(scales[j]) > amax) { amax = fabsf(scales[j]); max_scale = scales[j]; }
  }
  uint8_t* hm = b; uint8_t* qs = b + 32; uint8_t* sp = b + 96;
  memset(b, 0, 110);
  if (amax < 1e-30f) return;
  const float iscale = -32.f / max_scale;
  int8_t ls[16];
  for (int j = 0; j < 16; ++j) {
    const int l = std::max(-32, std::min(31, nearest_int(iscale * scales[j]))) + 32;
    ls[j] = (int8_t)l;
    if (j < 8) sp[j] = (uint8_t)(l & 15); else sp[j - 8] |= (uint8_t)((l & 15) << 4);
    sp[8 + j % 4] |= (uint8_t)((l >> 4) << (2 * (j / 4)));
  }
  const uint16_t dh = f32_to_fp16(1 / iscale);
  wr16(b + 108, dh);
  const float dd = fp16_to_f32(dh);
  uint8_t Lu[256];
  for (int j = 0; j < 16; ++j) {
    const float d = dd * (ls[j] - 32);
    for (int i = 0; i < 16; ++i) { const int l = d ? nearest_int(x[16 * j + i] / d) : 0; Lu[16 * j + i] = (uint8_t)(std::max(-4, std::min(3, l)) + 4); }
  }
  int m = 0; uint8_t hb = 1;
  for (int j = 0; j < 256; ++j) { if (Lu[j] > 3) { hm[m] |= hb; Lu[j] -= 4; } if (++m == 32) { m = 0; hb <<= 1; } }
  for (int n = 0; n < 256; n += 128) { for (int l = 0; l < 32; ++l) qs[l] = (uint8_t)(Lu[n + l] | (Lu[n + l + 32] << 2) | (Lu[n + l + 64] << 4) | (Lu[n + l + 96] << 6)); qs += 32; }
}
static void q_iq4_nl(const float* x, uint8_t* b) {
  float amax = 0, mx = 0;
  for (int j = 0; j < 32; ++j) if (fabsf(x[j]) > amax) { amax = fabsf(x[j]); mx = x[j]; }
  const float d = mx / k_iq4nl_values[0], id = d ? 1.f / d : 0.f;
  wr16(b, f32_to_fp16(d));
  auto best = [&](float v) { int bi = 0; float bd = 1e30f; for (int k = 0; k < 16; ++k) { const float e = fabsf(v - k_iq4nl_values[k]); if (e < bd) { bd = e; bi = k; } } return bi; };
  for (int j = 0; j < 16; ++j) b[2 + j] = (uint8_t)(best(x[j] * id) | (best(x[j + 16] * id) << 4));
}
static void q_tq2_0(const float* x, uint8_t* b) {
  float amax = 0;
  for (int j = 0; j < 256; ++j) amax = std::max(amax, fabsf(x[j]));
  const float d = amax, id = d ? 1.f / d : 0.f;
  for (int j = 0; j < 64; j += 32)
    for (int m = 0; m < 32; ++m) {
      uint8_t q = 0;
      for (int l = 0; l < 4; ++l) q |= (uint8_t)((nearest_int(x[(j / 32) * 128 + l * 32 + m] * id) + 1) << (2 * l));
      b[j + m] = q;
    }
  wr16(b + 64, f32_to_fp16(d));
}

typedef void (*QuantFn)(const float*, uint8_t*);
static QuantFn block_encoder(int t) {
  switch (t) {
    case T_Q8_0: return q_q8_0; case T_Q4_0: return q_q4_0; case T_Q4_1: return q_q4_1; case T_Q5_0: return q_q5_0; case T_Q5_1: return q_q5_1;
    case T_Q4_K: return q_q4_K; case T_Q5_K: return q_q5_K; case T_Q6_K: return q_q6_K; case T_Q2_K: return q_q2_K; case T_Q3_K: return q_q3_K;
    case T_IQ4_NL: return q_iq4_nl; case T_TQ2_0: return q_tq2_0;
    default: return nullptr;
  }
}

int quantize_row(int type, const float* src, void* dst, long n) {
  const TypeInfo* ti = type_info(type);
  if (!ti) return fail("quantize: unknown ggml type %d", type);
  if (n % ti->block) return fail("quantize: %ld elements is not a multiple of the %s block (%d)", n, ti->name, ti->block);
  uint8_t* d = (uint8_t*)dst;
  switch (type) {
    case T_F32: memcpy(dst, src, (size_t)n * 4); return 0;
    case T_F16: for (long i = 0; i < n; ++i) wr16(d + 2 * i, f32_to_fp16(src[i])); return 0;
    case T_BF16: for (long i = 0; i < n; ++i) wr16(d + 2 * i, f32_to_bf16(src[i])); return 0;
    default: break;
  }
  QuantFn fn = block_encoder(type);
  if (!fn) return fail("quantize: no quantiser for type %s", ti->name);
  const long nb = n / ti->block;
  for (long i = 0; i < nb; ++i) fn(src + i * ti->block, d + (size_t)i * ti->bytes);
  return 0;
}

const void* codebook(int which, int* entries, int* width) {
  need_codebooks();
  switch (which) {
    case 0: *entries = 256; *width = 8; return g_iq2xxs;
    case 1: *entries = 512; *width = 8; return g_iq2xs;
    case 2: *entries = 1024; *width = 8; return g_iq2s;
    case 3: *entries = 256; *width = 4; return g_iq3xxs;
    case 4: *entries = 512; *width = 4; return g_iq3s;
    case 5: *entries = 2048; *width = 8; return g_iq1s;
    case 6: *entries = 128; *width = 1; return g_ksigns;
    default: return nullptr;
  }
}

}  // namespace gbh

// ------------------------------------------------------------------------------------------ C API
GBH_API int gbh_type_info(int type, int* block, int* bytes, char* name32) {
  const gbh::TypeInfo* ti = gbh::type_info(type);
  if (!ti) return gbh::fail("unknown ggml type %d", type);
  *block = ti->block; *bytes = ti->bytes;
  if (name32) snprintf(name32, 32, "%s", ti->name);
  return 0;
}
GBH_API long gbh_row_bytes(int type, long n) {
  const gbh::TypeInfo* ti = gbh::type_info(type);
  if (!ti || n % ti->block) return -1;
  return n / ti->block * ti->bytes;
}
GBH_API int gbh_dequant_row(int type, const void* src, float* dst, long n) { return gbh::dequant_row(type, src, dst, n); }
GBH_API int gbh_quantize_row(int type, const float* src, void* dst, long n) { return gbh::quantize_row(type, src, dst, n); }
GBH_API int gbh_can_quantize(int type) { return (type == gbh::T_F32 || type == gbh::T_F16 || type == gbh::T_BF16 || gbh::block_encoder(type)) ? 1 : 0; }
GBH_API int gbh_can_dequantize(int type) {
  return (type == gbh::T_F32 || type == gbh::T_F16 || type == gbh::T_BF16 || type == gbh::T_I8 || type == gbh::T_I16 || type == gbh::T_I32 ||
          type == gbh::T_F64 || gbh::block_decoder(type)) ? 1 : 0;
}
GBH_API const void* gbh_codebook(int which, int* entries, int* width) { return gbh::codebook(which, entries, width); }
