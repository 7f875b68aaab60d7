// MXFP8 activation quantiser pieces shared by the kernels that emit block-scaled fp8 rows: the E8M0 scale of a
// 32-element block and where that scale byte lives in the 512-byte scale atoms the block-scaled tcgen05 GEMM reads.
// Format: e4m3 values with one E8M0 scale per 1 x 32 block, w = e4m3 * 2^(s - 127) (common/glm5_mxfp8.h:25-35).
#pragma once
#include "sm100.cuh"

namespace gb {

__device__ __forceinline__ int e8m0_amax(float amax) {
  const float s = amax * (1.0f / 448.0f);
  const uint32_t bits = __float_as_uint(s);
  int e = (int)((bits >> 23) & 0xff);
  if (bits & 0x7fffffu) e += 1;
  return amax == 0.0f ? 127 : max(1, min(e, 254));   // an all-zero block gets scale 1
}
// Byte offset of the scale of (row, 32-element block) in the two atom layouts: one 512-byte atom per
// 128 rows (rows interleaved 32 x 4) or per 32 rows (bytes 0..3 of each 16-byte lane row).
__device__ __forceinline__ size_t sf_atom_offset(long row, int blk32, int k_atoms, int layout32 = 0) {
  if (layout32) return ((size_t)(row >> 5) * k_atoms + (blk32 >> 2)) * 512 + (row & 31) * 16 + (blk32 & 3);
  return ((size_t)(row >> 7) * k_atoms + (blk32 >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (blk32 & 3);
}

}  // namespace gb
