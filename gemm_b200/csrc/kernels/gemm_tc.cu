// Persistent tcgen05 GEMM for linear layers:  Out[token, n] = sum_k X[token, k] * W[n, k].
//
// Orientation: the WEIGHT matrix is the MMA "A" operand (128 weight rows per tile fill the 128 TMEM
// lanes) and the TOKENS are the MMA "N" dimension (16..256 per tile).  Decode batches of 8..64
// tokens therefore waste no tensor-core work, and the same kernel serves prefill with 128/256-token
// tiles.  Both operands are K-major, staged by TMA into 128-byte-swizzled shared memory; accumulators
// live in TMEM (double buffered when they fit) and are drained by four epilogue warps.
//
// Variants (template parameters):
//   MODE 0  bf16 x bf16  (kind::f16)
//   MODE 1  MXFP8: e4m3 x e4m3 with one E8M0 scale per 32 K-elements on both operands
//           (kind::mxf8f6f4.block_scale; scale factors copied smem -> TMEM with tcgen05.cp)
//   DUAL    two weight tiles (gate rows, up rows) share one token tile; epilogue = SiLU(gate) * up
//   grouped (run time)  one weight matrix per group (expert); every group owns a row segment of X
//           described by device arrays, so no host synchronisation is needed after routing.
// Epilogues: bf16 / f32 store with optional bias, per-row scale and row scatter; or MXFP8
// re-quantisation (fp8 bytes + E8M0 scales in the layout MODE 1 consumes) so that the next GEMM
// reads what this one wrote.
//
// Replaces in the reference: the cuBLAS call sites of cuda/llm/cuda_llm_runner.c:15488-17418, the
// mma.sync GEMMs of cuda/cuda_kernels_common.h, silu_mul_f32 (cuda_llm_runner.c:455), the grouped
// expert GEMMs of mmq_*_grouped (cuda_llm_runner.c:5295-7329) and m3_gemm_mxfp8 (common/m3_impl.h:791-825).
#include "sm100.cuh"
#include "host_common.h"
#include <stdlib.h>
#include "../fabric/fabric.cuh"

namespace gb {

constexpr int kMaxGroups = 256;
constexpr int kGemmThreads = 192;

struct GemmArgs {
  int n_out;            // output features per group (weight rows of the gate half when DUAL)
  int k;                // reduction length in elements
  int m_tok;            // rows of X that exist (plain) / capacity of the segment buffer (grouped)
  int num_groups;       // 0 = plain GEMM
  int w_rows_per_group; // weight rows between consecutive groups
  int up_row_offset;    // DUAL: first "up" row inside a group
  const int* seg_start; // [G] first X row of each group (multiple of min(TN,128); of 128 for MX), device
  const int* seg_count; // [G] valid rows of each group, device
  const uint8_t* sfa;   // MODE 1: weight scales, 512-byte atoms [w_row/128][k/128]
  const uint8_t* sfb;   // MODE 1: activation scales, 512-byte atoms [x_row/128][k/128] (TN >= 128) or [x_row/32][k/128] (TN = 32)
  void* out;            // bf16 / f32 [rows, ldo]  or fp8 bytes [rows, ldo] for the quantising epilogue
  int ldo;
  int out_f32;
  uint8_t* out_sf;      // quantising epilogue: scale atoms [x_row/128][n/128]
  const float* bias;    // optional [n_out] (plain, per group not supported)
  const int* row_map;   // optional: output row of X row r (negative = drop)
  const float* row_scale; // optional: multiply row r of the result
  int stages;
  KernelStatus* status;
  // ---- expert-parallel extras (all optional) ----
  int w_group_mod;                 // > 0: the weights of group g are those of expert g % w_group_mod
  const uint32_t* wait_flags;      // wait until wait_flags[i] >= *epoch_ptr for i < wait_n before touching X / segments
  int wait_n;
  const uint32_t* epoch_ptr;
  void* peer_out[kMaxRanks];       // epilogue target per source rank: rows of region s go to peer_out[s]
  int peer_region_rows;            // > 0 enables the peer epilogue: X row r belongs to source r / region_rows and lands
  int peer_rank;                   //   at row peer_rank * region_rows + r % region_rows of that peer's buffer
  uint32_t* signal_flags[kMaxRanks];  // after the last tile of the grid: *signal_flags[p] = *epoch_ptr (release, system scope)
  int signal_n;
  unsigned* done_ctr;
  int peer_bcast;                  // > 0: tensor-parallel partial: every result row is stored to peer_out[p] for all p < peer_bcast
  int epoch_self_tick;             // != 0: signal *epoch_ptr + 1 and store it back (no separate tick kernel)
  // ---- split-K (plain GEMMs with few tiles): `splits` CTAs share one output tile, each reduces a K range into a
  // fp32 partial in sk_ws; the warp that arrives last at the tile's semaphore sums the partials in split order
  // (deterministic) and runs the normal epilogue.
  int splits;
  int tile_hint, m_tok_hint;       // host only: expected number of tiles and tokens per tile row (grid sizing of memory-bound launches)
  long partial_stride;             // > 0: no in-kernel reduction, split ks stores its fp32 partial at out + ks * partial_stride (elements)
  float* sk_ws;                    // [tiles][splits][NA * TN][128] fp32
  unsigned* sk_ctr;                // [tiles][4] self-resetting arrival counters (one per epilogue warp)
  // ---- arg-max epilogue: instead of storing the result, every epilogue warp writes the maximum of its 32 output
  // features and its feature index per token: amax_val / amax_idx [ceil(n_out/128) * 4][m_tok]
  float* amax_val;
  int* amax_idx;
  // ---- extents of the caller's buffers in bytes (0 = unknown): every global access of the kernel that is not a TMA
  // tile is checked against them; a violation is recorded in the status word (ST_BAD_ARG) and the access is skipped.
  size_t sfa_bytes, sfb_bytes, out_bytes, out_sf_bytes;
  // ---- weight layout: 0 = row-major [rows, k]; 1 = tiled [rows/128][k-blocks][128 rows][128 bytes], every 16 KB operand
  // tile of the main loop is one contiguous block of memory (one DRAM burst sequence instead of 128 strided lines)
  int early_weights;  // != 0: a plain decode-sized launch requests its first weight tiles before the dependency wait
  int dual_raw;  // DUAL without the activation: the second accumulator is the row block up_row_offset further down the same matrix
  int w_tiled;
};

// k-steps whose MXFP8 scale atoms are fetched by one bulk copy (2 for the widest tile, whose stages are short of room)
__host__ __device__ constexpr int sf_group(int tn) { return tn >= 256 ? 2 : tn >= 128 ? 4 : 1; }

struct Tile { int w_row0; int w_row1; int x_row0; int valid; int n0; int out_row0; int ks; int tile_id; };

// Maps the linear tile index of the persistent loop to a tile.  Every warp role walks the same
// sequence, so each keeps its own cursor.  n-blocks vary fastest: CTAs that run at the same time
// share one token tile (L2 reuse) and stream different weight rows.
template <int TN>
struct TileCursor {
  int g = 0, base = 0;
  __device__ __forceinline__ bool get(const GemmArgs& a, const int* s_start, const int* s_count, int t, Tile& o) {
    const int n_blocks = (a.n_out + 127) >> 7;
    if (a.num_groups == 0) {
      const int tok_blocks = (a.m_tok + TN - 1) / TN;
      const int sp = a.splits > 1 ? a.splits : 1;
      if (t >= n_blocks * tok_blocks * sp) return false;
      o.ks = t % sp; o.tile_id = t / sp;
      const int nb = o.tile_id % n_blocks, tb = o.tile_id / n_blocks;
      o.n0 = nb * 128; o.w_row0 = o.n0; o.w_row1 = a.up_row_offset + o.n0;
      o.x_row0 = tb * TN; o.valid = min(TN, a.m_tok - o.x_row0); o.out_row0 = o.x_row0;
      return true;
    }
    while (g < a.num_groups) {
      const int tiles_g = ((s_count[g] + TN - 1) / TN) * n_blocks;
      if (t < base + tiles_g) {
        const int lt = t - base;
        const int nb = lt % n_blocks, tb = lt / n_blocks;
        o.n0 = nb * 128;
        o.w_row0 = (a.w_group_mod > 0 ? g % a.w_group_mod : g) * a.w_rows_per_group + o.n0;
        o.w_row1 = o.w_row0 + a.up_row_offset;
        o.x_row0 = s_start[g] + tb * TN;
        o.valid = min(TN, s_count[g] - tb * TN);
        o.out_row0 = o.x_row0; o.ks = 0; o.tile_id = t;
        return true;
      }
      base += tiles_g; ++g;
    }
    return false;
  }
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// E8M0 exponent for a block whose absolute maximum is `amax`: the smallest power of two s with
// amax / s <= 448 (largest e4m3 magnitude), so quantisation never saturates.
__device__ __forceinline__ int e8m0_from_amax(float amax) {
  const float s = amax * (1.0f / 448.0f);
  uint32_t bits = __float_as_uint(s);
  int e = (int)((bits >> 23) & 0xff);
  if (bits & 0x7fffffu) e += 1;
  return amax == 0.0f ? 127 : max(1, min(e, 254));   // an all-zero block gets scale 1
}

template <int TN, int MODE, bool DUAL, bool QUANT_OUT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmArgs args) {
  constexpr int NA = DUAL ? 2 : 1;
  constexpr int A_BYTES = 128 * 128;                 // 128 rows x 128 bytes
  constexpr int B_BYTES = TN * 128;
  constexpr int SFB_ATOMS = (TN + 127) / 128;
  // Scale atoms travel and are copied to TMEM in groups of SFG k-steps: the atoms of consecutive k-steps are contiguous in
  // memory, so one bulk copy per operand and group replaces SFG copies of 512 bytes (which cost the producer thread
  // more issue time than the 16 KB operand tiles).  The group sits in the stage of its first k-step.
  constexpr int SFG = sf_group(TN);
  constexpr int SF_BYTES = (MODE == 1) ? (((NA + SFB_ATOMS) * 512 * SFG + 1023) & ~1023) : 0;
  constexpr int STAGE_BYTES = NA * A_BYTES + B_BYTES + SF_BYTES;
  constexpr int ACC_COLS = NA * TN;
  constexpr int SF_COLS = (MODE == 1) ? (NA * 4 + SFB_ATOMS * 4) * SFG : 0;
  constexpr int NACC = (2 * ACC_COLS + SF_COLS <= 512) ? 2 : 1;
  constexpr int NEED_COLS = NACC * ACC_COLS + SF_COLS;
  constexpr int TMEM_COLS = NEED_COLS <= 32 ? 32 : NEED_COLS <= 64 ? 64 : NEED_COLS <= 128 ? 128 : NEED_COLS <= 256 ? 256 : 512;
  static_assert(NEED_COLS <= 512, "accumulators do not fit TMEM");
  constexpr int KB_ELEMS = (MODE == 1) ? 128 : 64;   // K elements per 128-byte row

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int S = args.stages;
  uint8_t* tail = smem + (size_t)S * STAGE_BYTES;
  uint64_t* full_bar = (uint64_t*)tail;              // [S]
  uint64_t* empty_bar = full_bar + S;                // [S]
  uint64_t* accf_bar = empty_bar + S;                // [2] accumulator full
  uint64_t* acce_bar = accf_bar + 2;                 // [2] accumulator empty
  uint32_t* tmem_slot = (uint32_t*)(acce_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* s_start = (int*)(tmem_slot + 4);
  int* s_count = s_start + kMaxGroups;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (args.k + KB_ELEMS - 1) / KB_ELEMS;
  const int kb_per = (args.splits > 1) ? (num_kb + args.splits - 1) / args.splits : num_kb;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&accf_bar[i], 1); mbar_init(&acce_bar[i], 4); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmX);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  __syncthreads();                                   // barriers and the abort flag are initialised for everyone
  // Weights do not depend on the kernel in front of this one.  For a plain decode-sized GEMM (static tile sequence, one scale
  // group per k-step) the producer thread requests the weight tiles and weight scales of its first tile's first k-steps NOW,
  // before the dependency wait: the DRAM latency of the first loads and the fill of the ring overlap the previous kernel's
  // tail.  The stage's barrier gets the byte count of this part without an arrival; the token tile (and its arrival) follow
  // in the producer loop below.
  int pre_stages = 0;
  if (threadIdx.x == 0 && args.early_weights && args.num_groups == 0 && args.wait_n == 0 && SFG == 1) {
    TileCursor<TN> cur0; Tile t0;
    if (cur0.get(args, s_start, s_count, blockIdx.x, t0)) {
      const int kb0 = t0.ks * kb_per, kb1 = min(num_kb, kb0 + kb_per);
      const size_t row_bytes = (size_t)num_kb * 512;
      const size_t o0 = (size_t)(t0.w_row0 >> 7) * row_bytes, o1 = (size_t)(t0.w_row1 >> 7) * row_bytes;
      const bool sf_ok = MODE != 1 || args.sfa_bytes == 0 || (o0 + row_bytes <= args.sfa_bytes && (!DUAL || o1 + row_bytes <= args.sfa_bytes));
      if (sf_ok) {
        const int wy0 = ((t0.w_row0 >> 7) * num_kb) << 7, wy1 = ((t0.w_row1 >> 7) * num_kb) << 7;
        for (int kb = kb0; kb < kb1 && pre_stages < S; ++kb, ++pre_stages) {
          uint8_t* st = smem + (size_t)pre_stages * STAGE_BYTES;
          mbar_expect_tx_only(&full_bar[pre_stages], NA * A_BYTES + (MODE == 1 ? NA * 512 : 0));
          if (args.w_tiled) {
            tma_load_2d(st, &tmW, &full_bar[pre_stages], 0, wy0 + (kb << 7));
            if (DUAL) tma_load_2d(st + A_BYTES, &tmW, &full_bar[pre_stages], 0, wy1 + (kb << 7));
          } else {
            tma_load_2d(st, &tmW, &full_bar[pre_stages], kb * KB_ELEMS, t0.w_row0);
            if (DUAL) tma_load_2d(st + A_BYTES, &tmW, &full_bar[pre_stages], kb * KB_ELEMS, t0.w_row1);
          }
          if (MODE == 1) {
            uint8_t* sf = st + NA * A_BYTES + B_BYTES;
            bulk_load(sf, args.sfa + o0 + (size_t)kb * 512, 512, &full_bar[pre_stages]);
            if (DUAL) bulk_load(sf + SFG * 512, args.sfa + o1 + (size_t)kb * 512, 512, &full_bar[pre_stages]);
          }
        }
      }
    }
  }
  pdl_wait();                                        // everything above overlapped the previous kernel's tail
  pdl_trigger();                                     // at most one dependent grid is resident ahead of its turn
  if (args.wait_n > 0) {
    // Rows and segment tables are written by peer GPUs: wait for every source's flag of this epoch, then make the
    // observed data visible to the TMA (async proxy) reads that follow.
    if (threadIdx.x == 0) {
      const uint32_t want = *args.epoch_ptr;
      for (int i = 0; i < args.wait_n; ++i)
        if (!wait_flag_ge(args.wait_flags + i, want, args.status, 110, i)) { *abort_flag = 1; break; }
      asm volatile("fence.proxy.async.global;" ::: "memory");
    }
    __syncthreads();
  }
  if (!*abort_flag)
    for (int i = threadIdx.x; i < args.num_groups; i += blockDim.x) {
      // segment tables come from device memory: clamp them into the X buffer so that a corrupt table cannot walk off it
      const int st0 = args.seg_start[i], cn = args.seg_count[i];
      const bool sane = st0 >= 0 && cn >= 0 && st0 <= args.m_tok && cn <= args.m_tok - st0;
      if (!sane) report_status(args.status, ST_BAD_ARG, 130, i, st0, cn);
      s_start[i] = sane ? st0 : 0; s_count[i] = sane ? cn : 0;
    }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sf = tmem_base + NACC * ACC_COLS;   // SFA0 [, SFA1], SFB columns
  const bool run = (*abort_flag == 0);

  if (!run) {
    // a failed wait: nothing was issued, fall through to the teardown
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (one lane)
    if (lane == 0) {
      TileCursor<TN> cur; Tile t;
      int s = 0; uint32_t ph = 0;
      bool ok = true;
      for (int ti = blockIdx.x; ok && cur.get(args, s_start, s_count, ti, t); ti += gridDim.x) {
        const int kb0 = t.ks * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        // Per tile: the row coordinate of the (tiled) weight blocks and the start of each scale-atom stream.  The atoms of one
        // 128-row block are contiguous over k, so a stream is checked against its buffer's extent once, for the whole k range;
        // a bad one is reported and replaced by the buffer's first atoms.
        const int wy0 = ((t.w_row0 >> 7) * num_kb) << 7, wy1 = ((t.w_row1 >> 7) * num_kb) << 7;
        const uint8_t* sfa0 = nullptr; const uint8_t* sfa1 = nullptr; const uint8_t* sfbp[SFB_ATOMS];
        if (MODE == 1) {
          const size_t row_bytes = (size_t)num_kb * 512;
          auto stream_of = [&](const uint8_t* base, size_t extent, size_t atom_row, int where) -> const uint8_t* {
            const size_t off = atom_row * row_bytes;
            if (extent != 0 && off + row_bytes > extent) { report_status(args.status, ST_BAD_ARG, where, (int)atom_row, (int)(extent >> 9), ti); return base; }
            return base + off;
          };
          sfa0 = stream_of(args.sfa, args.sfa_bytes, (size_t)(t.w_row0 >> 7), 120);
          if (DUAL) sfa1 = stream_of(args.sfa, args.sfa_bytes, (size_t)(t.w_row1 >> 7), 121);
          if (TN == 32) {
            // narrow tiles use one atom per 32 rows (bytes 0..3 of each 16-byte lane row), so that the tile's
            // scales always land in column 0 of their TMEM block whatever 32-row boundary the tile starts on
            sfbp[0] = stream_of(args.sfb, args.sfb_bytes, (size_t)(t.x_row0 >> 5), 122);
          } else {
#pragma unroll
            for (int i = 0; i < SFB_ATOMS; ++i) {
              // a 256-token tile whose valid rows end in its first half has no second atom to fetch (it may lie past the
              // end of the scale buffer): the first one is fetched again so that the byte count of a stage stays fixed
              const int ai = (i * 128 < t.valid) ? i : 0;
              sfbp[i] = stream_of(args.sfb, args.sfb_bytes, (size_t)((t.x_row0 >> 7) + ai), 123);
            }
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, args.status, 100, s)) { ok = false; break; }
          uint8_t* st = smem + (size_t)s * STAGE_BYTES;
          // length of the scale group that starts at this k-step (0 = none starts here)
          const int glen = (MODE != 1) ? 0 : (SFG == 1) ? 1 : ((kb - kb0) % SFG == 0) ? min(SFG, kb1 - kb) : 0;
          // the weight part of this CTA's first k-steps was requested before the dependency wait (see above)
          const bool pre = ti == (int)blockIdx.x && kb - kb0 < pre_stages;
          mbar_expect_tx(&full_bar[s], pre ? B_BYTES + SFB_ATOMS * 512 * glen : NA * A_BYTES + B_BYTES + (NA + SFB_ATOMS) * 512 * glen);
          const int kx = kb * KB_ELEMS;
          if (pre) {
          } else if (args.w_tiled) {
            tma_load_2d(st, &tmW, &full_bar[s], 0, wy0 + (kb << 7));
            if (DUAL) tma_load_2d(st + A_BYTES, &tmW, &full_bar[s], 0, wy1 + (kb << 7));
          } else {
            tma_load_2d(st, &tmW, &full_bar[s], kx, t.w_row0);
            if (DUAL) tma_load_2d(st + A_BYTES, &tmW, &full_bar[s], kx, t.w_row1);
          }
          tma_load_2d(st + NA * A_BYTES, &tmX, &full_bar[s], kx, t.x_row0);
          if (MODE == 1 && glen > 0) {
            uint8_t* sf = st + NA * A_BYTES + B_BYTES;
            const uint32_t gbytes = (uint32_t)glen * 512;
            const size_t koff = (size_t)kb * 512;
            if (!pre) bulk_load(sf, sfa0 + koff, gbytes, &full_bar[s]);
            if (DUAL && !pre) bulk_load(sf + SFG * 512, sfa1 + koff, gbytes, &full_bar[s]);
#pragma unroll
            for (int i = 0; i < SFB_ATOMS; ++i) bulk_load(sf + (NA + i) * SFG * 512, sfbp[i] + koff, gbytes, &full_bar[s]);
          }
          if (++s == S) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (one lane)
    if (lane == 0) {
      TileCursor<TN> cur; Tile t;
      int s = 0; uint32_t ph = 0;
      int acc = 0; uint32_t acc_ph = 0;
      bool ok = true;
      for (int ti = blockIdx.x; ok && cur.get(args, s_start, s_count, ti, t); ti += gridDim.x) {
        if (!mbar_wait(&acce_bar[acc], acc_ph ^ 1, abort_flag, args.status, 200, acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * ACC_COLS;
        const int kb0 = t.ks * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, args.status, 201, s)) { ok = false; break; }
          tc_fence_after();
          const uint32_t st = smem_u32(smem + (size_t)s * STAGE_BYTES);
          uint32_t sfb_t = 0;
          uint32_t sfa_t = 0;
          if (MODE == 1) {
            const int kbi = kb - kb0, gj = kbi % SFG;
            if (gj == 0) {
              // the scale atoms of the next SFG k-steps came with this stage: copy them all into their TMEM columns
              const uint32_t sf = st + NA * A_BYTES + B_BYTES;
              const int glen = (SFG == 1) ? 1 : min(SFG, kb1 - kb);
#pragma unroll
              for (int g = 0; g < SFG; ++g) {
                if (g >= glen) break;
                tc_cp_32x128b_warpx4(tmem_sf + g * 4, make_sdesc_noswizzle(sf + g * 512, 0, 128));
                if (DUAL) tc_cp_32x128b_warpx4(tmem_sf + (SFG + g) * 4, make_sdesc_noswizzle(sf + (SFG + g) * 512, 0, 128));
#pragma unroll
                for (int i = 0; i < SFB_ATOMS; ++i)
                  tc_cp_32x128b_warpx4(tmem_sf + (NA * SFG + g * SFB_ATOMS + i) * 4, make_sdesc_noswizzle(sf + ((NA + i) * SFG + g) * 512, 0, 128));
              }
            }
            sfa_t = tmem_sf + gj * 4;
            // token tiles of MX GEMMs always start on a 128-row boundary; the atoms of a 256-token tile sit side by side
            sfb_t = tmem_sf + (NA * SFG + gj * SFB_ATOMS) * 4;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t a0 = make_sdesc_sw128(st + j * 32);
            const uint64_t b = make_sdesc_sw128(st + NA * A_BYTES + j * 32);
            const uint32_t accum = (kb > kb0 || j > 0) ? 1u : 0u;
            if (MODE == 0) {
              constexpr uint32_t idesc = make_idesc(128, TN, 1, 1);
              mma_f16_ss(d0, a0, b, idesc, accum);
              if (DUAL) mma_f16_ss(d0 + TN, make_sdesc_sw128(st + A_BYTES + j * 32), b, idesc, accum);
            } else {
              const uint32_t idesc = make_idesc_mx(128, TN, 0, 0, j, j);
              mma_mxf8_ss(d0, a0, b, idesc, accum, sfa_t, sfb_t);
              if (DUAL) mma_mxf8_ss(d0 + TN, make_sdesc_sw128(st + A_BYTES + j * 32), b, idesc, accum, sfa_t + SFG * 4, sfb_t);
            }
          }
          tc_commit(&empty_bar[s]);
          if (++s == S) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        tc_commit(&accf_bar[acc]);
        if (NACC == 2) { if (++acc == 2) { acc = 0; acc_ph ^= 1; } } else { acc_ph ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;                // weight row inside the tile == output feature
    TileCursor<TN> cur; Tile t;
    int acc = 0; uint32_t acc_ph = 0;
    bool ok = true;
    const bool simple_store = !QUANT_OUT && args.amax_val == nullptr && args.row_map == nullptr && args.peer_bcast == 0 &&
                              args.row_scale == nullptr && (args.splits <= 1 || args.partial_stride > 0);
    for (int ti = blockIdx.x; ok && cur.get(args, s_start, s_count, ti, t); ti += gridDim.x) {
      if (!mbar_wait(&accf_bar[acc], acc_ph, abort_flag, args.status, 300, acc)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tacc = tmem_base + acc * ACC_COLS + ((uint32_t)(q * 32) << 16);
      const int n = t.n0 + row;
      const bool n_ok = n < args.n_out;
      const float bias = (args.bias != nullptr && n_ok && (args.partial_stride == 0 || t.ks == 0)) ? args.bias[n] : 0.0f;
      // Everything after the accumulators are in registers: activation, bias, then one of the store forms.
      auto finish_chunk = [&](int c, const uint32_t* r0, const uint32_t* r1) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int xr = c + j;
          float v = __uint_as_float(r0[j]);
          if (DUAL) v = silu_f(v) * __uint_as_float(r1[j]);
          v += bias;
          const bool live = xr < t.valid;
          const int x_row = t.x_row0 + xr;
          if (QUANT_OUT) {
            // 32 lanes of this warp = one 32-wide block along n of one token: shared E8M0 scale.
            const float amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(n_ok ? fabsf(v) : 0.0f)));
            const int e = e8m0_from_amax(amax);
            const float inv = __uint_as_float((uint32_t)(254 - e) << 23);   // 2^(127-e)
            if (live) {
              if (n_ok) {
                __nv_fp8_e4m3 f8(v * inv);
                const size_t off = (size_t)x_row * args.ldo + n;
                if (args.out_bytes != 0 && off >= args.out_bytes) report_status(args.status, ST_BAD_ARG, 310, x_row, n, ti);
                else ((uint8_t*)args.out)[off] = *(uint8_t*)&f8;
              }
              if (lane == 0) {
                const size_t nkb = (size_t)((args.n_out + 127) >> 7);
                const size_t off = (TN == 32) ? ((size_t)(x_row >> 5) * nkb + (size_t)(t.n0 >> 7)) * 512 + (x_row & 31) * 16 + q
                                              : ((size_t)(x_row >> 7) * nkb + (size_t)(t.n0 >> 7)) * 512 + (x_row & 31) * 16 + ((x_row >> 5) & 3) * 4 + q;
                if (args.out_sf_bytes != 0 && off >= args.out_sf_bytes) report_status(args.status, ST_BAD_ARG, 311, x_row, (int)(off >> 9), ti);
                else args.out_sf[off] = (uint8_t)e;
              }
            }
          } else if (args.amax_val != nullptr) {
            // order-preserving integer image of the float, so that one redux gives the warp maximum; ties -> lowest feature
            float vv = (n_ok && v == v) ? v : -3.4e38f;
            uint32_t key = __float_as_uint(vv);
            key = (key & 0x80000000u) ? ~key : (key | 0x80000000u);
            const uint32_t kmax = __reduce_max_sync(0xffffffffu, key);
            const uint32_t who = __ballot_sync(0xffffffffu, key == kmax);
            if (live && lane == (int)__ffs(who) - 1) {
              const size_t slot = (size_t)((t.n0 >> 7) * 4 + q) * args.m_tok + x_row;
              args.amax_val[slot] = vv; args.amax_idx[slot] = n;
            }
          } else if (live && n_ok) {
            int orow = x_row;
            void* obase = args.out;
            if (args.peer_region_rows > 0) {
              const int src = x_row / args.peer_region_rows;
              obase = args.peer_out[src];
              orow = args.peer_rank * args.peer_region_rows + (x_row - src * args.peer_region_rows);
            }
            if (args.row_map != nullptr) orow = args.row_map[x_row];
            if (args.peer_bcast > 0) {
              // row-parallel partial result: the same value goes into this rank's slot on every GPU of the group
              const size_t po = (size_t)t.ks * (size_t)args.partial_stride;      // K-split partials: one slab per split inside the slot
              for (int p = 0; p < args.peer_bcast; ++p) {
                if (args.out_f32) ((float*)args.peer_out[p])[po + (size_t)orow * args.ldo + n] = v;
                else ((__nv_bfloat16*)args.peer_out[p])[(size_t)orow * args.ldo + n] = __float2bfloat16(v);
              }
            } else if (orow >= 0) {
              if (args.row_scale != nullptr) v *= args.row_scale[x_row];
              const size_t off = ((size_t)orow * args.ldo + n) * (args.out_f32 ? 4 : 2);
              if (args.out_bytes != 0 && args.peer_region_rows == 0 && off >= args.out_bytes) report_status(args.status, ST_BAD_ARG, 312, orow, n, ti);
              else if (args.out_f32) ((float*)obase)[(size_t)orow * args.ldo + n] = v;
              else ((__nv_bfloat16*)obase)[(size_t)orow * args.ldo + n] = __float2bfloat16(v);
            }
          }
        }
      };
      if (args.splits > 1 && args.partial_stride == 0) {
        // ---- split-K: park the partial, the last warp to arrive reduces
        float* ws = args.sk_ws + ((size_t)t.tile_id * args.splits) * (size_t)(NA * TN * 128);
        float* mine = ws + (size_t)t.ks * (NA * TN * 128);
#pragma unroll 1
        for (int c = 0; c < TN; c += 16) {
          uint32_t r0[16], r1[16];
          tmem_ld_x16(tacc + c, r0);
          if (DUAL) tmem_ld_x16(tacc + TN + c, r1);
          tc_wait_ld();
          if (c >= t.valid) continue;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            mine[(size_t)(c + j) * 128 + row] = __uint_as_float(r0[j]);
            if (DUAL) mine[(size_t)(TN + c + j) * 128 + row] = __uint_as_float(r1[j]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acce_bar[acc]);        // TMEM buffer is free again
        __threadfence();
        unsigned old = 0;
        if (lane == 0) old = atomicAdd(&args.sk_ctr[(size_t)t.tile_id * 4 + q], 1u);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == (unsigned)args.splits - 1) {
          if (lane == 0) args.sk_ctr[(size_t)t.tile_id * 4 + q] = 0;
          __threadfence();
#pragma unroll 1
          for (int c = 0; c < TN && c < t.valid; c += 16) {
            uint32_t r0[16], r1[16];
            float a0[16], a1[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) { a0[j] = 0.f; a1[j] = 0.f; }
            // split order is fixed (deterministic sum); the 16 (32) loads of one split are independent of each other
            for (int sidx = 0; sidx < args.splits; ++sidx) {
              const float* src = ws + (size_t)sidx * (NA * TN * 128);
              float l0[16], l1[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                l0[j] = __ldcg(src + (size_t)(c + j) * 128 + row);
                if (DUAL) l1[j] = __ldcg(src + (size_t)(TN + c + j) * 128 + row);
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) { a0[j] += l0[j]; if (DUAL) a1[j] += l1[j]; }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) { r0[j] = __float_as_uint(a0[j]); r1[j] = __float_as_uint(a1[j]); }
            finish_chunk(c, r0, r1);
          }
        }
        if (NACC == 2) { if (++acc == 2) { acc = 0; acc_ph ^= 1; } } else { acc_ph ^= 1; }
        continue;
      }
      if (simple_store) {
        // Common case (plain row-major bf16 / f32 result): every decision is made once per tile, the inner loop is
        // convert + store.  The tile's last element is checked against the buffer's extent.
        const size_t esz = args.out_f32 ? 4 : 2;
        const size_t part_off = (size_t)t.ks * (size_t)args.partial_stride;     // split-K partials: one output slab per split
        const size_t last = (part_off + (size_t)(t.x_row0 + t.valid - 1) * args.ldo + n) * esz;
        bool store_ok = n_ok;
        if (store_ok && args.out_bytes != 0 && args.peer_region_rows == 0 && last >= args.out_bytes) {
          report_status(args.status, ST_BAD_ARG, 312, t.x_row0 + t.valid - 1, n, ti);
          store_ok = false;
        }
        void* obase = args.out;
        size_t orow0 = (size_t)t.x_row0;
        if (args.peer_region_rows > 0) {
          // expert-parallel result rows go back to the GPU they came from; a tile never straddles two source regions
          const int src = t.x_row0 / args.peer_region_rows;
          obase = args.peer_out[src];
          orow0 = (size_t)args.peer_rank * args.peer_region_rows + (size_t)(t.x_row0 - src * args.peer_region_rows);
        }
        __nv_bfloat16* o16 = (__nv_bfloat16*)obase + part_off + orow0 * args.ldo + n;
        float* o32 = (float*)obase + part_off + orow0 * args.ldo + n;
        if constexpr (NACC == 1 && !DUAL) {
          if (!args.out_f32) {
            // One accumulator buffer (the widest tile with its scale columns fills TMEM): pull the whole row into registers
            // as packed bf16, hand the buffer back to the MMA thread, and only then store, so that the stores overlap the
            // next tile's MMAs.
            uint32_t pk[TN / 2];
#pragma unroll
            for (int c = 0; c < TN; c += 64) {
              uint32_t r[64];                      // two loads in flight per wait: the readout is latency-bound
              tmem_ld_x32(tacc + c, r);
              tmem_ld_x32(tacc + c + 32, r + 32);
              tc_wait_ld();
#pragma unroll
              for (int j = 0; j < 32; ++j) pk[c / 2 + j] = pack_bf16x2(__uint_as_float(r[2 * j]) + bias, __uint_as_float(r[2 * j + 1]) + bias);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acce_bar[acc]);
            if (store_ok) {
#pragma unroll
              for (int i = 0; i < TN / 2; ++i) {
                const int xr = 2 * i;
                if (xr < t.valid) ((unsigned short*)o16)[(size_t)xr * args.ldo] = (unsigned short)(pk[i] & 0xffffu);
                if (xr + 1 < t.valid) ((unsigned short*)o16)[(size_t)(xr + 1) * args.ldo] = (unsigned short)(pk[i] >> 16);
              }
            }
            acc_ph ^= 1;
            continue;
          }
        }
#pragma unroll 1
        for (int c = 0; c < TN; c += 16) {
          uint32_t r0[16], r1[16];
          tmem_ld_x16(tacc + c, r0);
          if (DUAL) tmem_ld_x16(tacc + TN + c, r1);
          tc_wait_ld();
          if (c >= t.valid) continue;
          if (!store_ok) continue;
          if (DUAL && args.dual_raw && args.partial_stride == 0) {
            // two row blocks of ONE projection share a token tile (rows n and up_row_offset + n): both plain results are stored.
            // Halves the tiles, the token-tile loads and the per-tile overhead of projections with a short K (expert down_proj).
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c + j < t.valid) {
                if (args.out_f32) {
                  o32[(size_t)(c + j) * args.ldo] = __uint_as_float(r0[j]);
                  o32[(size_t)(c + j) * args.ldo + args.up_row_offset] = __uint_as_float(r1[j]);
                } else {
                  o16[(size_t)(c + j) * args.ldo] = __float2bfloat16(__uint_as_float(r0[j]));
                  o16[(size_t)(c + j) * args.ldo + args.up_row_offset] = __float2bfloat16(__uint_as_float(r1[j]));
                }
              }
            continue;
          }
          if (DUAL && args.partial_stride > 0) {
            // K-split partials of a gate/up pair: both raw sums are stored (gate at column n, up at n_out + n of a 2 * n_out wide
            // slab); the activation needs the full sums and is applied by the kernel that adds the slabs
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c + j < t.valid) {
                o32[(size_t)(c + j) * args.ldo] = __uint_as_float(r0[j]);
                o32[(size_t)(c + j) * args.ldo + args.n_out] = __uint_as_float(r1[j]);
              }
            continue;
          }
          if (c + 16 <= t.valid) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float v = __uint_as_float(r0[j]);
              if (DUAL) v = silu_f(v) * __uint_as_float(r1[j]);
              v += bias;
              if (args.out_f32) o32[(size_t)(c + j) * args.ldo] = v;
              else o16[(size_t)(c + j) * args.ldo] = __float2bfloat16(v);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float v = __uint_as_float(r0[j]);
              if (DUAL) v = silu_f(v) * __uint_as_float(r1[j]);
              v += bias;
              if (c + j < t.valid) {
                if (args.out_f32) o32[(size_t)(c + j) * args.ldo] = v;
                else o16[(size_t)(c + j) * args.ldo] = __float2bfloat16(v);
              }
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < TN; c += 16) {
          uint32_t r0[16], r1[16];
          tmem_ld_x16(tacc + c, r0);
          if (DUAL) tmem_ld_x16(tacc + TN + c, r1);
          tc_wait_ld();
          if (c >= t.valid) continue;             // uniform across the CTA's epilogue warps
          finish_chunk(c, r0, r1);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acce_bar[acc]);
      if (NACC == 2) { if (++acc == 2) { acc = 0; acc_ph ^= 1; } } else { acc_ph ^= 1; }
    }
  }

  // Teardown.  After an abort, copies may still be landing in shared memory: give them a bounded
  // grace period before the CTA (and its shared memory) goes away.
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
  if (args.signal_n > 0 && threadIdx.x == 0) {
    // every store of this CTA happened before the barrier above; publish once the whole grid is done
    __threadfence_system();
    if (atomicAdd(args.done_ctr, 1u) == gridDim.x - 1) {
      *args.done_ctr = 0;
      uint32_t e = *args.epoch_ptr;
      if (args.epoch_self_tick) { e += 1; *const_cast<uint32_t*>(args.epoch_ptr) = e; }
      for (int p = 0; p < args.signal_n; ++p) st_release_sys(args.signal_flags[p], e);
    }
  }
}

template <int TN, int MODE, bool DUAL, bool QUANT_OUT>
static int launch_gemm(const CUtensorMap& tmW, const CUtensorMap& tmX, GemmArgs a, int max_tiles, cudaStream_t stream) {
  constexpr int NA = DUAL ? 2 : 1;
  constexpr int SFB_ATOMS = (TN + 127) / 128;
  constexpr int STAGE_BYTES = NA * 16384 + TN * 128 + ((MODE == 1) ? (((NA + SFB_ATOMS) * 512 * sf_group(TN) + 1023) & ~1023) : 0);
  const int tail = 1024 + 2 * kMaxGroups * 4 + 256;
  int stages = (int)((220 * 1024 - tail - 1024) / STAGE_BYTES);
  if (stages > 8) stages = 8;
  if (stages < 2) return fail("gemm: tile does not fit shared memory%s");
  a.stages = stages;
  const int smem = stages * STAGE_BYTES + tail + 1024;
  auto kern = gemm_tc_kernel<TN, MODE, DUAL, QUANT_OUT>;
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    attr_set = true;
  }
  int grid = sm_count();
  if (max_tiles > 0 && max_tiles < grid) grid = max_tiles;
  // Memory-bound (decode-sized) launches: all CTAs share the HBM stream, so a round of g tiles takes time proportional to g and the
  // kernel time goes with ceil(tiles / g) * g.  Take the g in [3/4 SMs, SMs] that wastes the fewest tile slots (768 equal tiles:
  // 128 CTAs x 6 rounds instead of 148 CTAs with a sixth round for 28 of them); ties go to more CTAs.
  static int even_waves = -1;
  if (even_waves < 0) { const char* e = getenv("GB_GEMM_EVEN_WAVES"); even_waves = (e != nullptr && atoi(e) == 0) ? 0 : 1; }
  if (even_waves && a.tile_hint > grid && a.m_tok_hint <= 64) {
    const int sms = grid;
    const long base = (long)((a.tile_hint + sms - 1) / sms) * sms;
    long best = base;
    for (int g = sms - 1; g >= sms * 3 / 4; --g) {
      const long slots = (long)((a.tile_hint + g - 1) / g) * g;
      if (slots < best && slots * 100 < base * 97) { best = slots; grid = g; }      // worth it from 3 % fewer slots on
    }
  }
  launch_k(kern, grid, kGemmThreads, smem, stream, tmW, tmX, a);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace gb

using namespace gb;

// Optional expert-parallel arguments of gb_gemm (host struct, mirrored by ctypes in parallel/fabric.py).
struct GemmExtras {
  int w_group_mod;
  int wait_n;
  const uint32_t* wait_flags;
  const uint32_t* epoch_ptr;
  void* peer_out[kMaxRanks];
  int peer_region_rows;
  int peer_rank;
  uint32_t* signal_flags[kMaxRanks];
  int signal_n;
  int pad;
  unsigned* done_ctr;
  int splits;
  int pad2;
  float* sk_ws;
  unsigned* sk_ctr;
  float* amax_val;
  int* amax_idx;
  long sk_ws_bytes;          // capacity of sk_ws
  long sk_ctr_count;         // capacity of sk_ctr (entries)
  int peer_bcast;
  int epoch_self_tick;
  size_t sfa_bytes, sfb_bytes, out_bytes, out_sf_bytes;
  long partial_stride;       // > 0 with splits > 1: every K split stores its fp32 partial into its own slab of `out` (the consumer sums them)
};

// Flags of gb_gemm.
enum { GEMM_MX = 1, GEMM_DUAL = 2, GEMM_QUANT_OUT = 4, GEMM_OUT_F32 = 8, GEMM_W_TILED = 16, GEMM_DUAL_RAW = 32 };

// Linear layer on tensor cores.
//   w        [w_rows, k] row-major (bf16, or e4m3 bytes when GEMM_MX), w_rows = groups * w_rows_per_group
//   x        [x_rows, k] row-major, same element type as w
//   out      [*, ldo]    bf16 (default), f32 (GEMM_OUT_F32) or e4m3 + out_sf (GEMM_QUANT_OUT)
//   tn       token tile: 16, 32, 64, 128 or 256 (256: non-DUAL without quantised output only)
// Grouped mode (num_groups > 0): seg_start / seg_count are device arrays; seg_start[g] must be a
// multiple of min(tn, 128); `max_rows` bounds the segment buffer (TMA extent).
GB_API int gb_gemm(const void* w, const void* x, void* out, int n_out, int k, int m_tok, int ldw, int ldx, int ldo,
                   int flags, int tn, int num_groups, int w_rows_per_group, int up_row_offset, const int* seg_start,
                   const int* seg_count, int x_rows, const void* sfa, const void* sfb, void* out_sf, const float* bias,
                   const int* row_map, const float* row_scale, const GemmExtras* ex, void* status, cudaStream_t stream) {
  const bool mx = flags & GEMM_MX, dual = flags & GEMM_DUAL, qo = flags & GEMM_QUANT_OUT;
  if (num_groups > kMaxGroups) return fail("gemm: too many groups%s");
  if (mx && (k % 128 != 0)) return fail("gemm: MXFP8 needs k %% 128 == 0%s");
  if (mx && tn < 32) return fail("gemm: MXFP8 needs a token tile of at least 32%s");
  // The scale factors of a token tile must start at column 0 of their 4-column TMEM block (an MMA whose
  // scale address pointed at column 1..3 raised "misaligned address"), so every MX token tile starts on a
  // 128-row boundary: narrow tiles only for a single token block, grouped segments 128-aligned with tn = 128.
  // tn = 32 reads activation scales in the one-atom-per-32-rows layout, tn = 128 in the 128-row layout; tn = 64
  // (128-row layout, second half at column 2) is kept to a single token block.
  if (mx && tn == 64 && (num_groups > 0 || m_tok > tn)) return fail("gemm: MXFP8 with tn = 64 needs a single token block%s");
  if (!mx && (k % 8 != 0)) return fail("gemm: bf16 needs k %% 8 == 0%s");
  if ((mx || num_groups > 0 || dual) && (n_out % 128 != 0)) return fail("gemm: n_out must be a multiple of 128 for MX / grouped / dual%s");
  const int esz = mx ? 1 : 2;
  const int w_groups = (ex != nullptr && ex->w_group_mod > 0) ? ex->w_group_mod : num_groups;
  const long w_rows = (num_groups > 0) ? (long)w_groups * w_rows_per_group : (dual ? (long)up_row_offset + n_out : (long)n_out);
  CUtensorMap tmW, tmX;
  const TmapDtype dt = mx ? TM_U8 : TM_BF16;
  const uint32_t box_k = mx ? 128 : 64;
  const bool w_tiled = flags & GEMM_W_TILED;
  if (w_tiled) {
    // tiled weights: [ceil(rows / 128)][ceil(k / box_k)][128][box_k]; a 2-D map whose rows are the 128-byte tile rows
    if (num_groups > 0 && (w_rows_per_group % 128 != 0 || up_row_offset % 128 != 0)) return fail("gemm: tiled weights need 128-row aligned groups%s");
    if (dual && up_row_offset % 128 != 0) return fail("gemm: tiled weights need a 128-row aligned up offset%s");
    const uint64_t kbs = ((uint64_t)k + box_k - 1) / box_k;
    const uint64_t rb = ((uint64_t)w_rows + 127) / 128;
    if (rb * kbs * 128 >= (1ull << 31)) return fail("gemm: tiled weight too large for 32-bit tile coordinates%s");
    if (make_tmap_2d(&tmW, w, dt, box_k, rb * kbs * 128, 128, box_k, 128, TM_SW_128)) return -1;
  } else if (make_tmap_2d(&tmW, w, dt, (uint64_t)k, (uint64_t)w_rows, (uint64_t)ldw * esz, box_k, 128, TM_SW_128)) return -1;
  if (make_tmap_2d(&tmX, x, dt, (uint64_t)k, (uint64_t)x_rows, (uint64_t)ldx * esz, box_k, (uint32_t)tn, TM_SW_128)) return -1;
  GemmArgs a;
  memset(&a, 0, sizeof(a));
  a.n_out = n_out; a.k = k; a.m_tok = m_tok; a.num_groups = num_groups; a.w_rows_per_group = w_rows_per_group;
  a.up_row_offset = up_row_offset; a.seg_start = seg_start; a.seg_count = seg_count;
  a.sfa = (const uint8_t*)sfa; a.sfb = (const uint8_t*)sfb; a.out = out; a.ldo = ldo; a.out_f32 = (flags & GEMM_OUT_F32) ? 1 : 0;
  a.w_tiled = w_tiled ? 1 : 0;
  {
    static int early = -1;                      // GB_GEMM_EARLY_WEIGHTS=0 switches the early weight requests off (A/B measurements)
    if (early < 0) { const char* e = getenv("GB_GEMM_EARLY_WEIGHTS"); early = (e != nullptr && atoi(e) == 0) ? 0 : 1; }
    a.early_weights = early;
  }
  a.dual_raw = (flags & GEMM_DUAL_RAW) ? 1 : 0;
  if (a.dual_raw && (!dual || qo)) return fail("gemm: GEMM_DUAL_RAW needs GEMM_DUAL without GEMM_QUANT_OUT%s");
  a.out_sf = (uint8_t*)out_sf; a.bias = bias; a.row_map = row_map; a.row_scale = row_scale; a.status = (KernelStatus*)status;
  if (ex != nullptr) {
    a.w_group_mod = ex->w_group_mod; a.wait_flags = ex->wait_flags; a.wait_n = ex->wait_n; a.epoch_ptr = ex->epoch_ptr;
    for (int i = 0; i < kMaxRanks; ++i) { a.peer_out[i] = ex->peer_out[i]; a.signal_flags[i] = ex->signal_flags[i]; }
    a.peer_region_rows = ex->peer_region_rows; a.peer_rank = ex->peer_rank; a.signal_n = ex->signal_n; a.done_ctr = ex->done_ctr;
    a.amax_val = ex->amax_val; a.amax_idx = ex->amax_idx; a.peer_bcast = ex->peer_bcast; a.epoch_self_tick = ex->epoch_self_tick;
    a.sfa_bytes = ex->sfa_bytes; a.sfb_bytes = ex->sfb_bytes; a.out_bytes = ex->out_bytes; a.out_sf_bytes = ex->out_sf_bytes;
    if (ex->splits > 1 && num_groups == 0 && ex->partial_stride > 0) {
      if (!(flags & GEMM_OUT_F32) || qo) return fail("gemm: split-K partials need a plain fp32 output%s");
      const int kb_elems = mx ? 128 : 64;
      const int num_kb = (k + kb_elems - 1) / kb_elems;
      const int kb_per = (num_kb + ex->splits - 1) / ex->splits;
      if ((num_kb + kb_per - 1) / kb_per != ex->splits) return fail("gemm: split-K partials: a split would be empty%s");
      a.splits = ex->splits; a.partial_stride = ex->partial_stride;
    } else if (ex->splits > 1 && num_groups == 0) {
      const int kb_elems = mx ? 128 : 64;
      const int num_kb = (k + kb_elems - 1) / kb_elems;
      int sp = ex->splits < num_kb ? ex->splits : num_kb;
      const int kb_per = (num_kb + sp - 1) / sp;
      sp = (num_kb + kb_per - 1) / kb_per;                    // no empty split
      const long tiles = (long)((n_out + 127) / 128) * ((m_tok + tn - 1) / tn);
      const long need = tiles * sp * (dual ? 2 : 1) * tn * 128 * 4;
      if (sp > 1 && ex->sk_ws != nullptr && need <= ex->sk_ws_bytes && tiles * 4 <= ex->sk_ctr_count) {
        a.splits = sp; a.sk_ws = ex->sk_ws; a.sk_ctr = ex->sk_ctr;
      }
    }
  }
  int max_tiles = 0;
  if (num_groups == 0) max_tiles = ((n_out + 127) / 128) * ((m_tok + tn - 1) / tn) * (a.splits > 1 ? a.splits : 1);
  // grouped launches do not know their tile count on the host; a decode-sized one (narrow token tile) has about one token tile
  // per group
  a.tile_hint = num_groups == 0 ? max_tiles : num_groups * ((n_out + 127) / 128);
  a.m_tok_hint = num_groups == 0 ? m_tok : (tn <= 32 ? tn : 1 << 20);
  if (num_groups == 0 && m_tok <= 0) return 0;

#define GB_DISPATCH(TNV)                                                                                      \
  if (tn == TNV) {                                                                                            \
    if (!mx && !dual && !qo) return launch_gemm<TNV, 0, false, false>(tmW, tmX, a, max_tiles, stream);        \
    if (!mx && dual && !qo) return launch_gemm<TNV, 0, true, false>(tmW, tmX, a, max_tiles, stream);          \
    if (mx && !dual && !qo) return launch_gemm<TNV, 1, false, false>(tmW, tmX, a, max_tiles, stream);         \
    if (mx && dual && qo) return launch_gemm<TNV, 1, true, true>(tmW, tmX, a, max_tiles, stream);             \
    if (mx && dual && !qo) return launch_gemm<TNV, 1, true, false>(tmW, tmX, a, max_tiles, stream);           \
    if (!mx && dual && qo) return launch_gemm<TNV, 0, true, true>(tmW, tmX, a, max_tiles, stream);            \
  }
  GB_DISPATCH(16)
  GB_DISPATCH(32)
  GB_DISPATCH(64)
  GB_DISPATCH(128)
  if (tn == 256 && !mx && !dual && !qo) return launch_gemm<256, 0, false, false>(tmW, tmX, a, max_tiles, stream);
  if (tn == 256 && mx && !dual && !qo) return launch_gemm<256, 1, false, false>(tmW, tmX, a, max_tiles, stream);
#undef GB_DISPATCH
  return fail("gemm: unsupported variant%s (tn=%ld flags=%ld)", "", (long)tn, (long)flags);
}
