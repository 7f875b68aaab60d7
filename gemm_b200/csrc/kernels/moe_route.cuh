// Router arithmetic shared by the routing kernels: one warp turns a row of router logits into the top-k expert ids and
// their weights.  Semantics: common/transformer.h:4050-4091 (softmax over all experts, top-k, weights renormalised to sum 1;
// ties go to the lower index, NaN counts as -FLT_MAX as in cuda/llm/cuda_llm_runner.c:7958-8035) and
// common/m3_impl.h:692-698 for the sigmoid + selection-bias variant.
#pragma once
#include "sm100.cuh"
#include <float.h>

namespace gb {

constexpr int kMaxTopK = 16;

// Routing of token `w` by one warp (E <= 512): lane j < k ends with the j-th pick.  Returns the (possibly local) expert id.
template <int MAXV>
__device__ __forceinline__ int route_row(const float* row, const float* __restrict__ bias, int* __restrict__ ids_row,
                                         float* __restrict__ weights_row, int lane, int n_exp, int k, int mode, int renorm,
                                         float routed_scale, int id_shift, int n_local) {
  float p[MAXV], sel[MAXV];
  float mx = -FLT_MAX;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int e = lane + 32 * i;
    float v = -FLT_MAX;
    if (e < n_exp) { v = row[e]; if (!(v == v)) v = -FLT_MAX; }
    p[i] = v;
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  if (mode == 0) {
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) { const int e = lane + 32 * i; p[i] = (e < n_exp) ? expf(p[i] - mx) : 0.f; sum += p[i]; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) { p[i] *= inv; sel[i] = (lane + 32 * i < n_exp) ? p[i] : -FLT_MAX; }
  } else {
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int e = lane + 32 * i;
      p[i] = (e < n_exp) ? 1.0f / (1.0f + expf(-p[i])) : 0.f;
      sel[i] = (e < n_exp) ? p[i] + (bias != nullptr ? bias[e] : 0.f) : -FLT_MAX;
    }
  }
  float wsum = 0.f;
  float my_w = 0.f; int my_id = 0;      // lane j keeps the j-th pick
  for (int j = 0; j < k; ++j) {
    float best = -FLT_MAX; int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int e = lane + 32 * i;
      if (e < n_exp && (sel[i] > best || (sel[i] == best && e < bi))) { best = sel[i]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    // owner lane removes it and publishes its probability
    float pv = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) if (lane + 32 * i == bi) { pv = p[i]; sel[i] = -FLT_MAX; }
    pv = __shfl_sync(0xffffffffu, pv, bi & 31);
    wsum += pv;
    if (lane == j) { my_w = pv; my_id = bi; }
  }
  int out_id = -1;
  if (lane < k) {
    float wv = my_w;
    if (renorm) wv = wv / fmaxf(wsum, 1e-20f);
    // expert-parallel ranks that see every token keep only their own experts: ids become local, the others -1
    const int lid = my_id - id_shift;
    out_id = (n_local > 0 && (lid < 0 || lid >= n_local)) ? -1 : lid;
    ids_row[lane] = out_id;
    weights_row[lane] = wv * routed_scale;
  }
  return out_id;
}

}  // namespace gb
