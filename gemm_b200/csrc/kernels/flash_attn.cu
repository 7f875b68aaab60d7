// FlashAttention forward over a paged KV cache on tcgen05, one kernel for prefill and decode.
//
// A CTA owns one KV head of one sequence and a tile of 128 query ROWS, where a row is a
// (token, query-head-in-group) pair: with G = Hq / Hkv query heads per KV head the tile covers
// floor(128 / G) consecutive tokens.  Every K/V block is therefore fetched once for the whole GQA
// group.  Decode is the same kernel with one token per sequence (G valid rows) and, when the batch is
// small, the KV range split over several CTAs whose partial (O, log-sum-exp) results a second kernel
// merges (the same merge rule serves context parallelism across GPUs).
//
// Pipeline per 128-position KV block j (S, P, O live in TMEM; P overwrites S in place as packed bf16).  A CTA uses half of
// TMEM and 96 KB of shared memory, so two CTAs share an SM and one's tensor work runs under the other's softmax:
//   TMA warp   : K_j, V_j pages -> 128B-swizzled smem (one block each; K_{j+1} lands while softmax j runs), page ids from
//                the block table
//   MMA thread : S_j = Q K_j^T, then O += P_j V_j  (A operand = P from TMEM, B = V MN-major from smem)
//   softmax    : 128 threads, one per row: S row -> reference max / sum, P = exp2(S - m) -> TMEM; O is rescaled only when
//                a row's maximum has grown by more than 2^8; final O / l -> global
// Q arrives pre-multiplied by softmax_scale * log2(e) (done by the RoPE kernel) so exp2 is exact base.
//
// Replaces in the reference: fa2_attn_f (cuda/llm/fa2_kernels.cu:55), batch_attn_causal_f32
// (cuda/llm/cuda_llm_runner.c:8340), attn_decode_f32 (:391, which keeps seq_len scores in shared
// memory and so bounds the context), cuda/fa2/cuda_fa2_kernels.h.  Numerics: tf_attn_worker
// (common/transformer.h:1333-1530).
#include "sm100.cuh"
#include "host_common.h"

namespace gb {

constexpr int kFaThreads = 192;
constexpr int kBN = 128;            // KV positions per block
constexpr int kD = 128;             // head dim

struct FaArgs {
  const int* work;          // [n_work, 4] = {seq, kv_head, q_tok0 (within the sequence's chunk), split}
  const int* cu_q;          // [B+1] token offsets of each sequence's query chunk in Q / O
  const int* kv_len;        // [B] KV length of each sequence INCLUDING the chunk being processed
  const int* block_table;   // [B, max_pages]
  int max_pages;
  int page_size;            // positions per page (8..128, divides 128)
  int hq, hkv;
  int num_splits;
  int causal;
  int window;               // sliding window (0 = off): position p attends to (p - window, p]
  __nv_bfloat16* out;       // [T, Hq, D]                 (used when part_o is null)
  float* part_o;            // [splits, T, Hq, D] f32     (num_splits > 1, or 1 split whose partial a caller merges itself)
  float* part_lse;          // [splits, T, Hq] base-2 log-sum-exp
  int total_tokens;
  KernelStatus* status;
  // decode kernel only: MXFP8 copy of the output rows [T, Hq * 128] (e4m3 bytes + E8M0 scale atoms), the o_proj operand
  uint8_t* out_q;
  uint8_t* out_sf;
  int out_sf32;             // scale-atom layout: one atom per 32 rows (1) or per 128 rows (0)
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr int kFaSmem = 32768 * 3 + 256 + 1024;

__global__ void __launch_bounds__(kFaThreads, 2)
flash_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const FaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                       // 2 x [128 rows x 128 B]  (d halves)
  uint8_t* sK = smem + 32768;               // one block: 2 x [128 positions x 128 B]
  uint8_t* sV = smem + 32768 * 2;           // one block
  uint64_t* bars = (uint64_t*)(smem + 32768 * 3);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;
  uint64_t* p_ready = bars + 6;             // 128 arrivals
  uint64_t* o_ready = bars + 7;
  uint32_t* tmem_slot = (uint32_t*)(bars + 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Prologue that touches no global memory: it overlaps the tail of the previous kernel of the stream.
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(k_full, 1); mbar_init(k_empty, 1); mbar_init(v_full, 1); mbar_init(v_empty, 1);
    mbar_init(s_full, 1); mbar_init(p_ready, 128); mbar_init(o_ready, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  // Half of TMEM: S / P (128 columns, P overwrites S in place) and O (128 columns).  Two CTAs share an SM, so one CTA's MMAs
  // run under the other's softmax; inside a CTA the block loop is a plain chain S -> softmax -> P V.
  if (warp == 1) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 128;
  pdl_wait();
  pdl_trigger();

  const int G = a.hq / a.hkv;
  const int tpt = 128 / G;                  // tokens per tile
  const int* wk = a.work + (size_t)blockIdx.x * 4;
  const int seq = wk[0], kvh = wk[1], q_tok0 = wk[2], split = wk[3];
  const int q_begin = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_begin;
  const int kv_len = a.kv_len[seq];
  const int n_tok = min(tpt, q_len - q_tok0);            // valid tokens of this tile
  const int pos0 = kv_len - q_len + q_tok0;              // position of the tile's first token
  // KV block range of this CTA
  int last_pos = a.causal ? (pos0 + n_tok - 1) : (kv_len - 1);
  int first_pos = 0;
  if (a.window > 0) first_pos = max(0, pos0 - a.window + 1);
  int blk_lo = first_pos / kBN, blk_hi = last_pos / kBN + 1;     // [lo, hi)
  if (a.num_splits > 1) {
    const int nb = blk_hi - blk_lo, per = (nb + a.num_splits - 1) / a.num_splits;
    blk_lo = blk_lo + split * per;
    blk_hi = min(blk_hi, blk_lo + per);
  }
  int n_blk = max(0, blk_hi - blk_lo);
  // a work item that names a KV head this cache does not have (a work list built for other head counts): nothing of it is
  // touched, the tile is written as "no keys" and the status word says why
  const bool bad_item = kvh < 0 || kvh >= a.hkv || q_tok0 < 0 || q_len < 0;
  if (bad_item) {
    if (threadIdx.x == 0) report_status(a.status, ST_BAD_ARG, 640, kvh, a.hkv, q_tok0);
    n_blk = 0;
  }

  if (warp == 0) {
    if (lane == 0 && n_blk > 0) {
      // Q tile: box (64 d, G heads, tpt tokens), two d-halves
      mbar_expect_tx(q_full, (uint32_t)(2 * 128 * G * tpt));
      tma_load_3d(sQ, &tmQ, q_full, 0, kvh * G, q_begin + q_tok0);
      tma_load_3d(sQ + 16384, &tmQ, q_full, 64, kvh * G, q_begin + q_tok0);
      const int ppb = kBN / a.page_size;               // pages per KV block
      const uint32_t page_bytes = (uint32_t)a.page_size * 128;
      const int* bt = a.block_table + (size_t)seq * a.max_pages;
      const int last_page = (kv_len + a.page_size - 1) / a.page_size - 1;
      bool ok = true;
      for (int j = 0; j < n_blk && ok; ++j) {
        const uint32_t ph = j & 1;
        const int blk = blk_lo + j;
        // Pages past the end of the sequence are replaced by its last page: the tile is always filled with
        // finite cache contents (their scores are masked, and 0 * finite stays 0 in P V).
        // K_j may land as soon as S_{j-1} has been computed, V_j as soon as P_{j-1} V_{j-1} has: both long before they are needed.
        if (!mbar_wait(k_empty, ph ^ 1, abort_flag, a.status, 400, j)) { ok = false; break; }
        mbar_expect_tx(k_full, 32768u);
        for (int p = 0; p < ppb; ++p) {
          const int page = bt[min(blk * ppb + p, last_page)];
          uint8_t* dst = sK + p * page_bytes;
          tma_load_3d(dst, &tmK, k_full, 0, kvh, page * a.page_size);
          tma_load_3d(dst + 16384, &tmK, k_full, 64, kvh, page * a.page_size);
        }
        if (!mbar_wait(v_empty, ph ^ 1, abort_flag, a.status, 401, j)) { ok = false; break; }
        mbar_expect_tx(v_full, 32768u);
        for (int p = 0; p < ppb; ++p) {
          const int page = bt[min(blk * ppb + p, last_page)];
          uint8_t* dst = sV + p * page_bytes;
          tma_load_3d(dst, &tmV, v_full, 0, kvh, page * a.page_size);
          tma_load_3d(dst + 16384, &tmV, v_full, 64, kvh, page * a.page_size);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_blk > 0) {
      constexpr uint32_t idesc_s = make_idesc(128, 128, 1, 1, 0, 0);
      constexpr uint32_t idesc_o = make_idesc(128, 128, 1, 1, 0, 1);     // B (= V) is MN-major
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      bool ok = mbar_wait(q_full, 0, abort_flag, a.status, 500);
      for (int j = 0; j < n_blk && ok; ++j) {
        const uint32_t ph = j & 1;
        // S_j = Q K_j^T.  The tensor pipe runs this thread's MMAs in order, so S_j overwrites P_{j-1} only after
        // P_{j-1} V_{j-1} has read it, and a completed S_j implies that O holds every earlier product.
        if (!mbar_wait(k_full, ph, abort_flag, a.status, 501, j)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
          mma_f16_ss(tmem_base, make_sdesc_sw128(q_addr + off), make_sdesc_sw128(k_addr + off), idesc_s, ks > 0 ? 1u : 0u);
        }
        tc_commit(s_full);
        tc_commit(k_empty);
        if (!mbar_wait(p_ready, ph, abort_flag, a.status, 502, j)) { ok = false; break; }
        if (!mbar_wait(v_full, ph, abort_flag, a.status, 503, j)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_f16_ts(tmem_o, tmem_base + ks * 8, make_sdesc_sw128_mn(v_addr + ks * 2048, 16384), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
        tc_commit(v_empty);
        if (j == n_blk - 1) tc_commit(o_ready);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue, one row per thread
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int t_local = r / G, h_local = r - t_local * G;
    const bool row_valid = (t_local < n_tok) && (r < tpt * G) && !bad_item;
    const int qpos = pos0 + min(t_local, n_tok - 1);
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const uint32_t s_t = tmem_base + lane_off;
    // m is the maximum the exponents refer to; it follows the true running maximum only when that has moved by more
    // than 2^kTau, so that O and l are rarely rescaled (P stays below 2^kTau, harmless in bf16 with fp32 sums).
    constexpr float kTau = 8.0f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blk && ok; ++j) {
      if (!mbar_wait(s_full, j & 1, abort_flag, a.status, 600, j)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = (blk_lo + j) * kBN;
      int hi = kv_len - 1;
      if (a.causal) hi = min(hi, qpos);
      int lo = 0;
      if (a.window > 0) lo = max(0, qpos - a.window + 1);
      const bool edge = (kv0 + kBN - 1 > hi || kv0 < lo);
      // pass 1: row maximum (the scores are read again in pass 2 instead of being kept in 128 registers)
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float sv[32];
        tmem_ld_x32(s_t + c * 32, reinterpret_cast<uint32_t*>(sv));
        tc_wait_ld();
        if (edge) {
#pragma unroll
          for (int i = 0; i < 32; ++i) { const int kp = kv0 + c * 32 + i; if (kp > hi || kp < lo) sv[i] = -INFINITY; }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, sv[i]);
      }
      float alpha = 1.0f;
      const bool grow = mx > m + kTau || (m == -INFINITY && mx > -INFINITY);
      if (grow) { alpha = fast_exp2(m - mx); m = mx; }          // m = -inf -> alpha 0 (l and O are 0 then anyway)
      const float m_use = (m == -INFINITY) ? 0.f : m;
      // O holds all products up to block j - 1 (see the MMA thread): rescale it now if some row of this warp moved its reference
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld_x32(tmem_o + lane_off + c * 32, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_x32(tmem_o + lane_off + c * 32, o);
        }
      }
      // pass 2: P = exp2(S - m) as packed bf16 over the first half of the S columns (chunk c lands on columns that
      // chunks <= c have already been read from)
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float sv[32];
        tmem_ld_x32(s_t + c * 32, reinterpret_cast<uint32_t*>(sv));
        tc_wait_ld();
        if (edge) {
#pragma unroll
          for (int i = 0; i < 32; ++i) { const int kp = kv0 + c * 32 + i; if (kp > hi || kp < lo) sv[i] = -INFINITY; }
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = fast_exp2(sv[2 * i] - m_use), p1 = fast_exp2(sv[2 * i + 1] - m_use);
          rs += p0 + p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        tmem_st_x16(s_t + c * 16, pk);
      }
      l = l * alpha + rs;
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    if (ok && n_blk > 0) ok = mbar_wait(o_ready, 0, abort_flag, a.status, 602);
    if (ok) {
      tc_fence_after();
      const int tok = q_begin + q_tok0 + t_local;
      const int head = kvh * G + h_local;
      const float inv_l = (l > 0.f) ? 1.0f / l : 0.f;
      uint32_t sf_word = 0;                  // the row's four E8M0 scales (MXFP8 output)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        if (n_blk > 0) { tmem_ld_x32(tmem_o + lane_off + c * 32, o); tc_wait_ld(); }
        else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (row_valid) {
          if (a.out_q != nullptr) {
            // this thread holds a whole (token, head) row: its 32-feature scale blocks are thread-local
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(__uint_as_float(o[i]) * inv_l));
            const float sc = amax * (1.0f / 448.0f);
            const uint32_t bits = __float_as_uint(sc);
            int e = (int)((bits >> 23) & 0xff) + ((bits & 0x7fffffu) ? 1 : 0);
            e = amax == 0.0f ? 127 : max(1, min(e, 254));
            const float inv = __uint_as_float((uint32_t)(254 - e) << 23) * inv_l;
            sf_word |= (uint32_t)e << (8 * c);
            uint4* dst = reinterpret_cast<uint4*>(a.out_q + ((size_t)tok * a.hq + head) * kD + c * 32);
#pragma unroll
            for (int v = 0; v < 2; ++v) {
              uint32_t w4[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int b0 = v * 16 + i * 4;
                w4[i] = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(__uint_as_float(o[b0]) * inv, __uint_as_float(o[b0 + 1]) * inv), __NV_SATFINITE, __NV_E4M3) |
                        ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(__uint_as_float(o[b0 + 2]) * inv, __uint_as_float(o[b0 + 3]) * inv), __NV_SATFINITE, __NV_E4M3) << 16);
              }
              dst[v] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
          } else if (a.part_o == nullptr) {
            uint4* dst = reinterpret_cast<uint4*>(a.out + ((size_t)tok * a.hq + head) * kD + c * 32);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(o[v * 8 + 0]) * inv_l, __uint_as_float(o[v * 8 + 1]) * inv_l);
              w.y = pack_bf16x2(__uint_as_float(o[v * 8 + 2]) * inv_l, __uint_as_float(o[v * 8 + 3]) * inv_l);
              w.z = pack_bf16x2(__uint_as_float(o[v * 8 + 4]) * inv_l, __uint_as_float(o[v * 8 + 5]) * inv_l);
              w.w = pack_bf16x2(__uint_as_float(o[v * 8 + 6]) * inv_l, __uint_as_float(o[v * 8 + 7]) * inv_l);
              dst[v] = w;
            }
          } else {
            float4* dst = reinterpret_cast<float4*>(a.part_o + (((size_t)split * a.total_tokens + tok) * a.hq + head) * kD + c * 32);
#pragma unroll
            for (int v = 0; v < 8; ++v)
              dst[v] = make_float4(__uint_as_float(o[v * 4]) * inv_l, __uint_as_float(o[v * 4 + 1]) * inv_l,
                                   __uint_as_float(o[v * 4 + 2]) * inv_l, __uint_as_float(o[v * 4 + 3]) * inv_l);
          }
        }
      }
      if (row_valid && a.out_q != nullptr) {
        // blocks head*4 .. head*4+3 of the row [Hq * 128] share one atom column block: four consecutive bytes
        const int k_atoms = a.hq;
        const size_t off = a.out_sf32 ? ((size_t)(tok >> 5) * k_atoms + head) * 512 + (tok & 31) * 16
                                      : ((size_t)(tok >> 7) * k_atoms + head) * 512 + (tok & 31) * 16 + ((tok >> 5) & 3) * 4;
        *reinterpret_cast<uint32_t*>(a.out_sf + off) = sf_word;
      }
      if (row_valid && a.part_o != nullptr)
        a.part_lse[((size_t)split * a.total_tokens + tok) * a.hq + head] = (l > 0.f) ? (m + log2f(l)) : -INFINITY;
    }
  }

  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

// ------------------------------------------------------------------------------------------------------------------
// Decode-specialised flash kernel: one new token per sequence, so a GQA group has only G (<= 16) query rows.  Here the KV
// POSITIONS are the MMA M dimension and the query heads the N dimension (the same trick as the GEMM's "weights are M"):
//   S^T[128 pos x 16 heads] = K_j[128 x 128] Q^T          (A = K tile, K-major;  B = Q, 16 rows, K-major)
//   O^T[128 d   x 16 heads] += V_j^T[128 d x 128 pos] P_j  (A = V tile, MN-major; B = P^T written to smem as [head][pos])
// A softmax thread owns one KV position (S^T) or one output feature (O^T) and touches 16 values per block instead of the
// 128 of the prefill layout, where the 8 live rows of a decode tile sat in one warp that did all the exponentials.  Max and
// sum over the 128 positions of a block are warp shuffles plus a 4-entry shared-memory exchange.  Shared memory per CTA is
// about 107 KB (K and V tiles alternate through one ring of three 32 KB slots), so two CTAs share an SM: with 64 sequences x 4 KV heads all 256 work
// items are resident at once and there is no second, partly filled wave.
constexpr int kFdN = 16;                 // MMA N: query heads of one KV head, zero padded
constexpr int kFdThreads = 192;
constexpr int kFdSmem = 4096 + 3 * 32768 + 8192 + 2048 + 1024;   // Q, tile ring, P x2, barriers + reductions, alignment

// Reduce 16 per-lane values over the 32 lanes of a warp with 16 shuffles (a reduce-scatter: 8 + 4 + 2 + 1 exchanges, then one
// more between neighbours): lane L returns the result for index L >> 1.
#define GB_RS_STEP(IN, OUT, N, BIT, OP)                                                       \
  _Pragma("unroll") for (int i = 0; i < N; ++i) {                                            \
    const bool up = (lane & BIT) != 0;                                                       \
    const float send = up ? IN[i] : IN[N + i], keep = up ? IN[N + i] : IN[i];                 \
    OUT[i] = OP(keep, __shfl_xor_sync(0xffffffffu, send, BIT));                               \
  }
__device__ __forceinline__ float rs_max(float a, float b) { return fmaxf(a, b); }
__device__ __forceinline__ float rs_add(float a, float b) { return a + b; }
__device__ __forceinline__ float warp_reduce16_max(const float* v, int lane) {
  float a[8], b[4], c[2], d[1];
  GB_RS_STEP(v, a, 8, 16, rs_max) GB_RS_STEP(a, b, 4, 8, rs_max) GB_RS_STEP(b, c, 2, 4, rs_max) GB_RS_STEP(c, d, 1, 2, rs_max)
  return fmaxf(d[0], __shfl_xor_sync(0xffffffffu, d[0], 1));
}
__device__ __forceinline__ float warp_reduce16_sum(const float* v, int lane) {
  float a[8], b[4], c[2], d[1];
  GB_RS_STEP(v, a, 8, 16, rs_add) GB_RS_STEP(a, b, 4, 8, rs_add) GB_RS_STEP(b, c, 2, 4, rs_add) GB_RS_STEP(c, d, 1, 2, rs_add)
  return d[0] + __shfl_xor_sync(0xffffffffu, d[0], 1);
}

// Barrier over the 128 softmax threads (named barrier 1) that also ANDs a predicate: every thread learns whether all of them
// got through their bounded wait, so they leave the loop together and nobody is left standing at a barrier.
__device__ __forceinline__ bool softmax_bar_and(bool pred) {
  uint32_t r;
  asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(r) : "r"((uint32_t)pred) : "memory");
  return r != 0;
}

__global__ void __launch_bounds__(kFdThreads, 2)
flash_decode_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const FaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                          // 2 d-halves x [16 heads x 128 B]
  uint8_t* ring = smem + 4096;                 // 3 slots x 32 KB; tile t = 2j is K of block j, t = 2j + 1 is V of block j, slot = t % 3
  uint8_t* sP = ring + 3 * 32768;              // 2 buffers x 2 position-halves x [16 heads x 128 B] (bf16, 128B swizzle)
  uint64_t* bars = (uint64_t*)(sP + 8192);
  uint64_t* q_full = bars;                     // 1
  uint64_t* t_full = bars + 1;                 // 3
  uint64_t* t_empty = bars + 4;                // 3
  uint64_t* s_full = bars + 7;                 // 2
  // P of block j arrives at p_ready[j & 1] (128 arrivals).  Two barriers, not one: S(j + 1) is issued before the MMA thread waits
  // for P(j), so the softmax threads can finish block j + 1 while that thread is still parked in its wait for block j; on a single
  // barrier the phase would then flip twice, the parity the waiter looks for would never show, and the CTA would sit out its
  // wait budget (seen as one 1.1 s step in about one run in ten; the wait site reported was the producer's, whose budget
  // starts first).  With two barriers a second flip of the same one needs P(j + 2), which needs O(j), which needs this wait.
  uint64_t* p_ready = bars + 9;                // 2
  uint64_t* o_ready = bars + 11;               // 2: block j commits to o_ready[j & 1]
  uint32_t* tmem_slot = (uint32_t*)(bars + 13);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  float* red_max = (float*)(bars + 16);        // [2 (block parity)][4 warps][16 heads]
  float* red_sum = red_max + 2 * 4 * kFdN;     // [2][4][16]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 3; ++i) { mbar_init(&t_full[i], 1); mbar_init(&t_empty[i], 1); }
    for (int i = 0; i < 2; ++i) mbar_init(&s_full[i], 1);
    mbar_init(&p_ready[0], 128); mbar_init(&p_ready[1], 128); mbar_init(&o_ready[0], 1); mbar_init(&o_ready[1], 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  // rows of Q beyond the group size are never loaded: keep them finite (their columns of S and O are never stored)
  for (int i = threadIdx.x; i < 4096 / 16; i += kFdThreads) reinterpret_cast<uint4*>(sQ)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  if (warp == 1) { tmem_alloc(tmem_slot, 64); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 2 * kFdN;
  pdl_wait();

  const int G = a.hq / a.hkv;
  const int* wk = a.work + (size_t)blockIdx.x * 4;
  const int seq = wk[0], kvh = wk[1], split = wk[3];
  const int tok = a.cu_q[seq];
  const int kv_len = a.kv_len[seq];
  const int qpos = kv_len - 1;
  int first_pos = 0;
  if (a.window > 0) first_pos = max(0, qpos - a.window + 1);
  int blk_lo = first_pos / kBN, blk_hi = (kv_len > 0) ? (kv_len - 1) / kBN + 1 : 0;
  if (a.num_splits > 1) {
    const int nb = blk_hi - blk_lo, per = (nb + a.num_splits - 1) / a.num_splits;
    blk_lo = blk_lo + split * per;
    blk_hi = min(blk_hi, blk_lo + per);
  }
  int n_blk = max(0, blk_hi - blk_lo);
  const bool bad_item = kvh < 0 || kvh >= a.hkv || G > kFdN || (a.cu_q[seq + 1] - tok) != 1;
  if (bad_item) {
    if (threadIdx.x == 0) report_status(a.status, ST_BAD_ARG, 650, kvh, a.hkv, G);
    n_blk = 0;
  }

  if (warp == 0) {
    if (lane == 0 && n_blk > 0) {
      mbar_expect_tx(q_full, (uint32_t)(2 * 128 * G));
      tma_load_3d(sQ, &tmQ, q_full, 0, kvh * G, tok);
      tma_load_3d(sQ + 2048, &tmQ, q_full, 64, kvh * G, tok);
      const int ppb = kBN / a.page_size;
      const uint32_t page_bytes = (uint32_t)a.page_size * 128;
      const int* bt = a.block_table + (size_t)seq * a.max_pages;
      const int last_page = (kv_len + a.page_size - 1) / a.page_size - 1;
      bool ok = true;
      for (int t = 0; t < 2 * n_blk && ok; ++t) {
        const int slot = t % 3; const uint32_t ph = (uint32_t)(t / 3) & 1;
        const int blk = blk_lo + (t >> 1);
        const CUtensorMap* tm = (t & 1) ? &tmV : &tmK;
        if (!mbar_wait(&t_empty[slot], ph ^ 1, abort_flag, a.status, 410, t)) { ok = false; break; }
        mbar_expect_tx(&t_full[slot], 32768u);
        for (int p = 0; p < ppb; ++p) {
          const int page = bt[min(blk * ppb + p, last_page)];
          uint8_t* dst = ring + slot * 32768 + p * page_bytes;
          tma_load_3d(dst, tm, &t_full[slot], 0, kvh, page * a.page_size);
          tma_load_3d(dst + 16384, tm, &t_full[slot], 64, kvh, page * a.page_size);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_blk > 0) {
      constexpr uint32_t idesc_s = make_idesc(128, kFdN, 1, 1, 0, 0);
      constexpr uint32_t idesc_o = make_idesc(128, kFdN, 1, 1, 1, 0);      // A (= V^T) is MN-major
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, abort_flag, a.status, 510);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        const int t = 2 * j, slot = t % 3; const uint32_t ph = (uint32_t)(t / 3) & 1;
        if (!mbar_wait(&t_full[slot], ph, abort_flag, a.status, 511, j)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(ring + slot * 32768);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_f16_ss(tmem_base + s * kFdN, make_sdesc_sw128(k_addr + (ks >> 2) * 16384 + (ks & 3) * 32),
                     make_sdesc_sw128(q_addr + (ks >> 2) * 2048 + (ks & 3) * 32), idesc_s, ks > 0 ? 1u : 0u);
        tc_commit(&s_full[s]);
        tc_commit(&t_empty[slot]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_blk && ok; ++j) {
        if (j + 1 < n_blk) { if (!issue_s(j + 1)) { ok = false; break; } }
        const int tv = 2 * j + 1, vslot = tv % 3;
        if (!mbar_wait(&p_ready[j & 1], (uint32_t)(j >> 1) & 1, abort_flag, a.status, 512, j)) { ok = false; break; }
        if (!mbar_wait(&t_full[vslot], (uint32_t)(tv / 3) & 1, abort_flag, a.status, 513, j)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(ring + vslot * 32768);
        const uint32_t pj = p_addr + (j & 1) * 4096;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_f16_ss(tmem_o, make_sdesc_sw128_mn(v_addr + ks * 2048, 16384), make_sdesc_sw128(pj + (ks >> 2) * 2048 + (ks & 3) * 32),
                     idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
        tc_commit(&o_ready[j & 1]);
        tc_commit(&t_empty[vslot]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax: thread r = KV position r of the block / feature r of O
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    float m[kFdN], l[kFdN];          // m: the reference maximum the exponentials are taken against (may lag the true maximum by <= kTau)
                                     // l: THIS thread's share of the row sums (its positions only); the threads' shares are added once, at the end
#pragma unroll
    for (int h = 0; h < kFdN; ++h) { m[h] = -INFINITY; l[h] = 0.f; }
    constexpr float kTau = 8.0f;     // O and l are only rescaled when a block raises a maximum by more than 2^kTau
    bool ok = true, fail_o = false;  // fail_o: a wait for the second MMA ran out; it is put to the vote at the next barrier
    for (int j = 0; j < n_blk && ok; ++j) {
      const int s = j & 1;
      const bool got_s = mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag, a.status, 610, j);
      tc_fence_after();
      float sv[kFdN];
      tmem_ld_x16(tmem_base + s * kFdN + lane_off, reinterpret_cast<uint32_t*>(sv));
      tc_wait_ld();
      const int kp = (blk_lo + j) * kBN + r;
      const bool live = kp <= qpos && kp >= first_pos;
      float* rm = red_max + (j & 1) * 4 * kFdN;
#pragma unroll
      for (int h = 0; h < kFdN; ++h) if (!live || h >= G) sv[h] = -INFINITY;
      {
        const float v = warp_reduce16_max(sv, lane);            // lane L ends with head L >> 1
        if ((lane & 1) == 0) rm[q * kFdN + (lane >> 1)] = v;
      }
      if (!softmax_bar_and(got_s && !fail_o)) { ok = false; break; }   // maxima of all four warps are in rm; all 128 threads leave together
      float bm[kFdN];
      bool need = false;
#pragma unroll
      for (int h = 0; h < kFdN; ++h) {
        bm[h] = fmaxf(fmaxf(rm[h], rm[kFdN + h]), fmaxf(rm[2 * kFdN + h], rm[3 * kFdN + h]));
        need |= (h < G) && (bm[h] > m[h] + kTau);                  // also true for the first finite maximum (m = -inf)
      }
      float alpha[kFdN], pv[kFdN];
#pragma unroll
      for (int h = 0; h < kFdN; ++h) {
        const float m_new = need ? fmaxf(m[h], bm[h]) : m[h];
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[h] = need ? fast_exp2(m[h] - m_use) : 1.0f;
        m[h] = m_new;
        pv[h] = fast_exp2(sv[h] - m_use);
        l[h] = l[h] * alpha[h] + pv[h];
      }
      bool got_o = true;
      if (j >= 2) {
        // the P buffer of this parity was read by the second MMA of block j - 2
        got_o = mbar_wait(&o_ready[s], (uint32_t)((j - 2) >> 1) & 1, abort_flag, a.status, 611, j);
      }
      if (got_o && need && j > 0) {
        // rare: a maximum moved by more than 2^kTau.  All earlier P V products must have landed in O before it is rescaled.
        got_o = mbar_wait(&o_ready[(j - 1) & 1], (uint32_t)((j - 1) >> 1) & 1, abort_flag, a.status, 613, j);
        tc_fence_after();
        if (got_o) {
          uint32_t o[kFdN];
          tmem_ld_x16(tmem_o + lane_off, o);
          tc_wait_ld();
#pragma unroll
          for (int h = 0; h < kFdN; ++h) o[h] = __float_as_uint(__uint_as_float(o[h]) * alpha[h]);
          asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                       :: "r"(tmem_o + lane_off), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]),
                          "r"(o[8]), "r"(o[9]), "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]), "r"(o[14]), "r"(o[15]) : "memory");
          tc_wait_st();
        }
      }
      if (got_o) {
        // P^T into shared memory as [head][position] bf16, the K-major B operand of the second MMA (128-byte swizzle)
        uint8_t* pb = sP + s * 4096;
        const int half = r >> 6, chunk = (r & 63) >> 3;
#pragma unroll
        for (int h = 0; h < kFdN; ++h)
          *reinterpret_cast<__nv_bfloat16*>(pb + half * 2048 + h * 128 + ((chunk ^ (h & 7)) << 4) + (r & 7) * 2) = __float2bfloat16(pv[h]);
        fence_proxy_async_smem();                // P in shared memory -> visible to the tensor core's reads
        tc_fence_before();
        mbar_arrive(&p_ready[s]);
      }
      fail_o |= !got_o;
    }
    if (ok && !fail_o && n_blk > 0) ok = mbar_wait(&o_ready[(n_blk - 1) & 1], (uint32_t)((n_blk - 1) >> 1) & 1, abort_flag, a.status, 612);
    // row sums: add the 128 threads' shares (one reduce-scatter per warp, then the four warps through shared memory)
    {
      const float v = warp_reduce16_sum(l, lane);
      if ((lane & 1) == 0) red_sum[q * kFdN + (lane >> 1)] = v;
      ok = softmax_bar_and(ok && !fail_o);       // every softmax thread gets here exactly once, whatever happened in the loop
#pragma unroll
      for (int h = 0; h < kFdN; ++h) l[h] = red_sum[h] + red_sum[kFdN + h] + red_sum[2 * kFdN + h] + red_sum[3 * kFdN + h];
    }
    if (ok && !bad_item) {
      tc_fence_after();
      uint32_t o[kFdN];
      if (n_blk > 0) { tmem_ld_x16(tmem_o + lane_off, o); tc_wait_ld(); }
      else {
#pragma unroll
        for (int h = 0; h < kFdN; ++h) o[h] = 0u;
      }
#pragma unroll
      for (int h = 0; h < kFdN; ++h) {
        if (h >= G) continue;
        const float inv_l = (l[h] > 0.f) ? 1.0f / l[h] : 0.f;
        const int head = kvh * G + h;
        const float val = __uint_as_float(o[h]) * inv_l;
        if (a.out_q != nullptr) {
          // the 32 features of this warp are one scale block of the row: quantise here instead of in a kernel of its own
          const float amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(val))));
          const float sc = amax * (1.0f / 448.0f);
          const uint32_t bits = __float_as_uint(sc);
          int e = (int)((bits >> 23) & 0xff) + ((bits & 0x7fffffu) ? 1 : 0);
          e = amax == 0.0f ? 127 : max(1, min(e, 254));
          const float inv = __uint_as_float((uint32_t)(254 - e) << 23);
          __nv_fp8_e4m3 f8(val * inv);
          a.out_q[(size_t)tok * a.hq * kD + (size_t)head * kD + r] = *reinterpret_cast<uint8_t*>(&f8);
          if (lane == 0) {
            const int blk = head * 4 + q, k_atoms = a.hq;       // 128 features per head = one atom column block per head
            const size_t off = a.out_sf32 ? ((size_t)(tok >> 5) * k_atoms + (blk >> 2)) * 512 + (tok & 31) * 16 + (blk & 3)
                                          : ((size_t)(tok >> 7) * k_atoms + (blk >> 2)) * 512 + (tok & 31) * 16 + ((tok >> 5) & 3) * 4 + (blk & 3);
            a.out_sf[off] = (uint8_t)e;
          }
        } else if (a.part_o == nullptr) a.out[((size_t)tok * a.hq + head) * kD + r] = __float2bfloat16(val);
        else a.part_o[(((size_t)split * a.total_tokens + tok) * a.hq + head) * kD + r] = val;
        if (a.part_o != nullptr && r == 0)
          a.part_lse[((size_t)split * a.total_tokens + tok) * a.hq + head] = (l[h] > 0.f) ? (m[h] + log2f(l[h])) : -INFINITY;
      }
    }
  }

  pdl_trigger();           // a long kernel: its dependents are released at its end, not while it streams the cache
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 64); }
}

// Merge of split-KV partials: out = sum_s 2^(lse_s - lse_max) O_s / sum_s 2^(lse_s - lse_max).
// One warp per (token, head); D = 128 -> 4 floats per lane.
__global__ void fa_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, __nv_bfloat16* __restrict__ out,
                                  float* __restrict__ out_lse, int splits, long rows, uint8_t* __restrict__ out_q, uint8_t* __restrict__ out_sf,
                                  int out_sf32, int hq) {
  pdl_wait();
  pdl_trigger();
  const long w = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (w >= rows) return;
  const int lane = threadIdx.x & 31;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, part_lse[(size_t)s * rows + w]);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float den = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ls = part_lse[(size_t)s * rows + w];
    if (ls == -INFINITY) continue;
    const float wgt = exp2f(ls - mx);
    const float4 v = *reinterpret_cast<const float4*>(part_o + ((size_t)s * rows + w) * kD + lane * 4);
    acc[0] += wgt * v.x; acc[1] += wgt * v.y; acc[2] += wgt * v.z; acc[3] += wgt * v.w;
    den += wgt;
  }
  const float inv = den > 0.f ? 1.0f / den : 0.f;
  if (out_q != nullptr) {
    // MXFP8 row of the output projection's operand [T, Hq * 128]: eight lanes (32 features) share a scale
    float amax = fmaxf(fmaxf(fabsf(acc[0]), fabsf(acc[1])), fmaxf(fabsf(acc[2]), fabsf(acc[3]))) * inv;
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const uint32_t bits = __float_as_uint(amax * (1.0f / 448.0f));
    int e = (int)((bits >> 23) & 0xff) + ((bits & 0x7fffffu) ? 1 : 0);
    e = amax == 0.0f ? 127 : max(1, min(e, 254));
    const float sc = __uint_as_float((uint32_t)(254 - e) << 23) * inv;
    const uint32_t q4 = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(acc[0] * sc, acc[1] * sc), __NV_SATFINITE, __NV_E4M3) |
                        ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(acc[2] * sc, acc[3] * sc), __NV_SATFINITE, __NV_E4M3) << 16);
    *reinterpret_cast<uint32_t*>(out_q + (size_t)w * kD + lane * 4) = q4;
    if ((lane & 7) == 0) {
      const long tok = w / hq;
      const int head = (int)(w - tok * hq), sub = lane >> 3;
      const size_t off = out_sf32 ? ((size_t)(tok >> 5) * hq + head) * 512 + (tok & 31) * 16 + sub
                                  : ((size_t)(tok >> 7) * hq + head) * 512 + (tok & 31) * 16 + ((tok >> 5) & 3) * 4 + sub;
      out_sf[off] = (uint8_t)e;
    }
    if (out_lse != nullptr && lane == 0) out_lse[w] = den > 0.f ? mx + log2f(den) : -INFINITY;
    return;
  }
  uint2 o;
  o.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
  o.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
  *reinterpret_cast<uint2*>(out + (size_t)w * kD + lane * 4) = o;
  if (out_lse != nullptr && lane == 0) out_lse[w] = den > 0.f ? mx + log2f(den) : -INFINITY;
}

}  // namespace gb

using namespace gb;

// q [T, Hq, 128] bf16 (pre-scaled by softmax_scale * log2 e), k_cache / v_cache [num_slots, Hkv, 128] bf16,
// out [T, Hq, 128] bf16.  `work` is a device int32 [n_work, 4] list {seq, kv_head, q_tok0, split}.
// With num_splits > 1, part_o / part_lse receive the partials and gb_fa_combine finishes.
static int flash_attn_impl(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_lse,
                         const int* work, int n_work, const int* cu_q, const int* kv_len, const int* block_table, int max_pages,
                         int page_size, long num_slots, int total_tokens, int hq, int hkv, int head_dim, int num_splits, int causal,
                         int window, void* status, cudaStream_t stream, uint8_t* out_q, uint8_t* out_sf, int out_sf32) {
  if (head_dim != 128) return fail("flash_attn: head_dim must be 128%s");
  if (hq % hkv) return fail("flash_attn: Hq %% Hkv != 0%s");
  const int G = hq / hkv;
  if (G > 128) return fail("flash_attn: group size > 128%s");
  if (page_size < 8 || page_size > 128 || (128 % page_size) || (page_size % 8)) return fail("flash_attn: page_size must be 8..128, a multiple of 8 dividing 128%s");
  if (n_work <= 0) return 0;
  if (num_splits > 1 && part_o == nullptr) return fail("flash_attn: num_splits > 1 needs partial buffers%s");
  if (part_o == nullptr && out == nullptr) return fail("flash_attn: no output buffer%s");
  if (part_o != nullptr && part_lse == nullptr) return fail("flash_attn: partial output needs part_lse%s");
  const int tpt = 128 / G;
  CUtensorMap tmQ, tmK, tmV;
  {
    uint64_t dims[3] = {128, (uint64_t)hq, (uint64_t)total_tokens};
    uint64_t strides[2] = {256, (uint64_t)hq * 256};
    uint32_t box[3] = {64, (uint32_t)G, (uint32_t)tpt};
    if (make_tmap(&tmQ, q, TM_BF16, 3, dims, strides, box, TM_SW_128)) return -1;
  }
  {
    uint64_t dims[3] = {128, (uint64_t)hkv, (uint64_t)num_slots};
    uint64_t strides[2] = {256, (uint64_t)hkv * 256};
    uint32_t box[3] = {64, 1, (uint32_t)page_size};
    if (make_tmap(&tmK, k_cache, TM_BF16, 3, dims, strides, box, TM_SW_128)) return -1;
    if (make_tmap(&tmV, v_cache, TM_BF16, 3, dims, strides, box, TM_SW_128)) return -1;
  }
  FaArgs a;
  memset(&a, 0, sizeof(a));
  a.work = work; a.cu_q = cu_q; a.kv_len = kv_len; a.block_table = block_table; a.max_pages = max_pages; a.page_size = page_size;
  a.hq = hq; a.hkv = hkv; a.num_splits = num_splits; a.causal = causal; a.window = window; a.out = (__nv_bfloat16*)out;
  a.part_o = part_o; a.part_lse = part_lse; a.total_tokens = total_tokens; a.status = (KernelStatus*)status;
  a.out_q = out_q; a.out_sf = out_sf; a.out_sf32 = out_sf32;
  const int smem = kFaSmem;
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA_OK(cudaFuncSetAttribute(flash_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set = true;
  }
  launch_k(flash_attn_kernel, n_work, kFaThreads, smem, stream, tmQ, tmK, tmV, a);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_flash_attn(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_lse,
                         const int* work, int n_work, const int* cu_q, const int* kv_len, const int* block_table, int max_pages,
                         int page_size, long num_slots, int total_tokens, int hq, int hkv, int head_dim, int num_splits, int causal,
                         int window, void* status, cudaStream_t stream) {
  return flash_attn_impl(q, k_cache, v_cache, out, part_o, part_lse, work, n_work, cu_q, kv_len, block_table, max_pages, page_size, num_slots, total_tokens, hq, hkv, head_dim, num_splits, causal, window, status, stream, nullptr, nullptr, 0);
}

// gb_flash_attn with the output written as MXFP8 rows [T, Hq * 128] (one KV split): the operand of the output projection.
GB_API int gb_flash_attn_mx(const void* q, const void* k_cache, const void* v_cache, void* out_q, void* out_sf, int sf32, const int* work,
                            int n_work, const int* cu_q, const int* kv_len, const int* block_table, int max_pages, int page_size,
                            long num_slots, int total_tokens, int hq, int hkv, int head_dim, int causal, int window, void* status,
                            cudaStream_t stream) {
  if (out_q == nullptr || out_sf == nullptr) return fail("flash_attn_mx: no output buffer%s");
  return flash_attn_impl(q, k_cache, v_cache, out_q, nullptr, nullptr, work, n_work, cu_q, kv_len, block_table, max_pages, page_size, num_slots,
                         total_tokens, hq, hkv, head_dim, 1, causal, window, status, stream, (uint8_t*)out_q, (uint8_t*)out_sf, sf32);
}

// Decode form of gb_flash_attn: every sequence contributes exactly one query token (cu_q = 0, 1, 2, ...), Hq / Hkv <= 16.
// Same arguments and outputs; work items are {seq, kv_head, 0, split}.
static int flash_decode_impl(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_lse,
                           const int* work, int n_work, const int* cu_q, const int* kv_len, const int* block_table, int max_pages,
                           int page_size, long num_slots, int total_tokens, int hq, int hkv, int head_dim, int num_splits, int window,
                           void* status, cudaStream_t stream, uint8_t* out_q, uint8_t* out_sf, int out_sf32) {
  if (head_dim != 128) return fail("flash_decode: head_dim must be 128%s");
  if (hq % hkv || hq / hkv > kFdN) return fail("flash_decode: needs Hq %% Hkv == 0 and a group of at most 16 heads%s");
  if (page_size < 8 || page_size > 128 || (128 % page_size) || (page_size % 8)) return fail("flash_decode: page_size must be 8..128, a multiple of 8 dividing 128%s");
  if (n_work <= 0) return 0;
  if (num_splits > 1 && part_o == nullptr) return fail("flash_decode: num_splits > 1 needs partial buffers%s");
  if (part_o == nullptr && out == nullptr) return fail("flash_decode: no output buffer%s");
  const int G = hq / hkv;
  CUtensorMap tmQ, tmK, tmV;
  {
    uint64_t dims[3] = {128, (uint64_t)hq, (uint64_t)total_tokens};
    uint64_t strides[2] = {256, (uint64_t)hq * 256};
    uint32_t box[3] = {64, (uint32_t)G, 1};
    if (make_tmap(&tmQ, q, TM_BF16, 3, dims, strides, box, TM_SW_128)) return -1;
  }
  {
    uint64_t dims[3] = {128, (uint64_t)hkv, (uint64_t)num_slots};
    uint64_t strides[2] = {256, (uint64_t)hkv * 256};
    uint32_t box[3] = {64, 1, (uint32_t)page_size};
    if (make_tmap(&tmK, k_cache, TM_BF16, 3, dims, strides, box, TM_SW_128)) return -1;
    if (make_tmap(&tmV, v_cache, TM_BF16, 3, dims, strides, box, TM_SW_128)) return -1;
  }
  FaArgs a;
  memset(&a, 0, sizeof(a));
  a.work = work; a.cu_q = cu_q; a.kv_len = kv_len; a.block_table = block_table; a.max_pages = max_pages; a.page_size = page_size;
  a.hq = hq; a.hkv = hkv; a.num_splits = num_splits; a.causal = 1; a.window = window; a.out = (__nv_bfloat16*)out;
  a.part_o = part_o; a.part_lse = part_lse; a.total_tokens = total_tokens; a.status = (KernelStatus*)status;
  a.out_q = out_q; a.out_sf = out_sf; a.out_sf32 = out_sf32;
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA_OK(cudaFuncSetAttribute(flash_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFdSmem));
    attr_set = true;
  }
  launch_k(flash_decode_kernel, n_work, kFdThreads, kFdSmem, stream, tmQ, tmK, tmV, a);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_flash_decode(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_lse,
                           const int* work, int n_work, const int* cu_q, const int* kv_len, const int* block_table, int max_pages,
                           int page_size, long num_slots, int total_tokens, int hq, int hkv, int head_dim, int num_splits, int window,
                           void* status, cudaStream_t stream) {
  return flash_decode_impl(q, k_cache, v_cache, out, part_o, part_lse, work, n_work, cu_q, kv_len, block_table, max_pages, page_size, num_slots, total_tokens, hq, hkv, head_dim, num_splits, window, status, stream, nullptr, nullptr, 0);
}

// gb_flash_decode with the output written as MXFP8 rows [T, Hq * 128] (single split only): out_q e4m3 bytes, out_sf scale atoms in
// the 32-row (sf32 = 1) or 128-row layout.
GB_API int gb_flash_decode_mx(const void* q, const void* k_cache, const void* v_cache, void* out_q, void* out_sf, int sf32, const int* work,
                              int n_work, const int* cu_q, const int* kv_len, const int* block_table, int max_pages, int page_size,
                              long num_slots, int total_tokens, int hq, int hkv, int head_dim, int window, void* status, cudaStream_t stream) {
  if (out_q == nullptr || out_sf == nullptr) return fail("flash_decode_mx: no output buffer%s");
  return flash_decode_impl(q, k_cache, v_cache, out_q, nullptr, nullptr, work, n_work, cu_q, kv_len, block_table, max_pages, page_size,
                           num_slots, total_tokens, hq, hkv, head_dim, 1, window, status, stream, (uint8_t*)out_q, (uint8_t*)out_sf, sf32);
}

GB_API int gb_fa_combine(const float* part_o, const float* part_lse, void* out, float* out_lse, int splits, long rows, cudaStream_t stream) {
  if (rows <= 0) return 0;
  launch_k(fa_combine_kernel, (unsigned)((rows * 32 + 255) / 256), 256, 0, stream, part_o, part_lse, (__nv_bfloat16*)out, out_lse, splits, rows,
           (uint8_t*)nullptr, (uint8_t*)nullptr, 0, 1);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

// The same merge with the result written as MXFP8 rows [T, hq * 128] (rows = T * hq): the operand of the output projection.
GB_API int gb_fa_combine_mx(const float* part_o, const float* part_lse, void* out_q, void* out_sf, int sf32, int hq, int splits, long rows,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hq < 1 || rows % hq) return fail("fa_combine_mx: rows must be tokens * heads%s");
  launch_k(fa_combine_kernel, (unsigned)((rows * 32 + 255) / 256), 256, 0, stream, part_o, part_lse, (__nv_bfloat16*)nullptr, (float*)nullptr, splits,
           rows, (uint8_t*)out_q, (uint8_t*)out_sf, sf32, hq);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}
