// ggml tensor types as stored in GGUF files: numeric ids, elements per block, bytes per block.
// Ids and sizes are fixed by the file format (the reference lists them in common/gguf_loader.h:45-84,185-223).
#pragma once
#include <stdint.h>

namespace gbh {

enum GgmlType : int {
  T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8, T_Q8_1 = 9,
  T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_Q8_K = 15,
  T_IQ2_XXS = 16, T_IQ2_XS = 17, T_IQ3_XXS = 18, T_IQ1_S = 19, T_IQ4_NL = 20, T_IQ3_S = 21, T_IQ2_S = 22, T_IQ4_XS = 23,
  T_I8 = 24, T_I16 = 25, T_I32 = 26, T_I64 = 27, T_F64 = 28, T_IQ1_M = 29, T_BF16 = 30,
  T_TQ1_0 = 34, T_TQ2_0 = 35, T_MXFP4 = 39, T_NVFP4 = 40, T_Q1_0 = 41, T_COUNT = 42
};

struct TypeInfo { const char* name; int block; int bytes; };

inline const TypeInfo* type_info(int t) {
  static const TypeInfo tab[T_COUNT] = {
      /*0*/ {"F32", 1, 4}, {"F16", 1, 2}, {"Q4_0", 32, 18}, {"Q4_1", 32, 20}, {nullptr, 0, 0}, {nullptr, 0, 0},
      /*6*/ {"Q5_0", 32, 22}, {"Q5_1", 32, 24}, {"Q8_0", 32, 34}, {"Q8_1", 32, 36},
      /*10*/ {"Q2_K", 256, 84}, {"Q3_K", 256, 110}, {"Q4_K", 256, 144}, {"Q5_K", 256, 176}, {"Q6_K", 256, 210}, {"Q8_K", 256, 292},
      /*16*/ {"IQ2_XXS", 256, 66}, {"IQ2_XS", 256, 74}, {"IQ3_XXS", 256, 98}, {"IQ1_S", 256, 50}, {"IQ4_NL", 32, 18},
      /*21*/ {"IQ3_S", 256, 110}, {"IQ2_S", 256, 82}, {"IQ4_XS", 256, 136},
      /*24*/ {"I8", 1, 1}, {"I16", 1, 2}, {"I32", 1, 4}, {"I64", 1, 8}, {"F64", 1, 8}, {"IQ1_M", 256, 56}, {"BF16", 1, 2},
      /*31*/ {nullptr, 0, 0}, {nullptr, 0, 0}, {nullptr, 0, 0},
      /*34*/ {"TQ1_0", 256, 54}, {"TQ2_0", 256, 66}, {nullptr, 0, 0}, {nullptr, 0, 0}, {nullptr, 0, 0},
      /*39*/ {"MXFP4", 32, 17}, {"NVFP4", 64, 36}, {"Q1_0", 128, 18}};
  if (t < 0 || t >= T_COUNT || tab[t].name == nullptr) return nullptr;
  return &tab[t];
}

// IEEE half <-> float, bit exact (subnormals included).
inline float fp16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff, bits;
  if (exp == 0) {
    if (man == 0) bits = sign;
    else {
      int e = -1;
      do { ++e; man <<= 1; } while ((man & 0x400) == 0);
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13);
    }
  } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
  else bits = sign | ((exp + 112) << 23) | (man << 13);
  float f;
  __builtin_memcpy(&f, &bits, 4);
  return f;
}
inline uint16_t f32_to_fp16(float f) {          // round to nearest even
  uint32_t x;
  __builtin_memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000;
  x &= 0x7fffffff;
  if (x >= 0x7f800000) return (uint16_t)(sign | 0x7c00 | ((x > 0x7f800000) ? 0x200 : 0));
  if (x >= 0x477ff000) return (uint16_t)(sign | 0x7c00);                // overflow -> inf
  if (x < 0x33000001) return (uint16_t)sign;                            // underflow -> 0
  int e = (int)(x >> 23) - 127;
  uint32_t m = (x & 0x7fffff) | 0x800000;
  if (e < -14) {
    const int shift = -14 - e + 13;
    uint32_t r = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (r & 1))) ++r;
    return (uint16_t)(sign | r);
  }
  uint32_t r = ((uint32_t)(e + 15) << 10) | ((m >> 13) & 0x3ff);
  const uint32_t rem = m & 0x1fff;
  if (rem > 0x1000 || (rem == 0x1000 && (r & 1))) ++r;
  return (uint16_t)(sign | r);
}
inline float bf16_to_f32(uint16_t h) {
  const uint32_t bits = (uint32_t)h << 16;
  float f;
  __builtin_memcpy(&f, &bits, 4);
  return f;
}
inline uint16_t f32_to_bf16(float f) {
  uint32_t x;
  __builtin_memcpy(&x, &f, 4);
  if ((x & 0x7fffffff) > 0x7f800000) return (uint16_t)((x >> 16) | 0x40);
  return (uint16_t)((x + 0x7fff + ((x >> 16) & 1)) >> 16);
}

}  // namespace gbh
