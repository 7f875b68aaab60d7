// Expert FFN of a decode step in ONE persistent launch: gate/up projection + SiLU(gate) * up + MXFP8 re-quantisation, then the
// down projection, for every routed (token, expert) pair of a batch whose rows were already gathered into expert order.
//
// Why one kernel.  Run as two grouped GEMMs, each launch pays its own prologue, first-load latency and drain (about 10 us of an
// 85 us / 50 us pair), and each ends in a partial wave: 768 equal gate/up tiles are 5.19 rounds of 148 CTAs.  Here the two
// projections are one list of work: a CTA that has no tile left in the first list goes straight on to tiles of the second, whose
// weights do not depend on anything and whose activations were written (by other CTAs) a few microseconds earlier and are read
// back from L2.
//
//   phase 0 tile (b, nb): token block b (32 rows of one expert) x 128 gate rows + the matching 128 up rows, K = hidden;
//                         epilogue SiLU(gate) * up -> e4m3 bytes + E8M0 scales of block b in `hq` / `hsf`
//   phase 1 tile (b, nb): token block b x weight rows [128 nb, +128) and [hidden / 2 + 128 nb, +128) of the down projection,
//                         K = inter; epilogue bf16 stores into `y`
//
// Both phases have the same shape per k-step (two 128 x 128-byte weight tiles, one 32 x 128-byte token tile, three 512-byte
// scale atoms), so they share one shared-memory ring, one MMA loop and the TMEM accumulators.
//
// Order and dependencies.  Every CTA walks its phase-0 tiles first (tile index = CTA + i * grid), then its phase-1 tiles.  A
// phase-1 tile of block b reads what the `inter / 128` phase-0 tiles of block b wrote: every epilogue warp of such a tile bumps
// `ctr[b]` after its stores (fence + atomic), and the producer thread of the reading CTA waits (bounded) for the full count before
// it issues the first TMA load of that block's activations, followed by a proxy fence (generic writes -> async-proxy reads).  A
// phase-0 tile never waits, and every CTA finishes its phase-0 tiles before it can wait, so the waits always end.  CTAs that got
// one phase-0 tile more than the others skip the first rounds of phase 1 (about the cost of that tile), which keeps the
// finish times level (not when phase 0 is less than one round: then every CTA takes its share of phase 1).  The CTA that finishes last zeroes the counters for the next launch.
//
// Optional last phase (expert parallelism where every rank holds all tokens of the step): the router-weighted sum of a token's
// local expert rows, stored as an fp32 row into this rank's slot on the token's home GPU.  Token t is taken by CTA t % grid
// after its tiles; its epilogue warps wait (bounded) on per-block counters of the phase-1 tiles that produced the rows.  The last
// CTA advances the epoch and raises this rank's flag on every GPU, which is what the next RMSNorm (the consumer of the
// slots) waits for.  With it a layer's expert block is one launch and one flag round.
//
// Replaces in the reference: the per-expert loops over mmq_*_grouped + silu_mul + down GEMV of the MoE decode path
// (cuda/llm/cuda_llm_runner.c:5295-7329, 455).
#include "sm100.cuh"
#include "mxq.cuh"
#include "host_common.h"

namespace gb {

constexpr int kFfnThreads = 192;
constexpr int kFfnTN = 32;                         // token tile
constexpr int kFfnMaxBlocks = 512;                 // token blocks (32 rows each) the block table holds
constexpr int kFfnA = 128 * 128;                   // one weight tile
constexpr int kFfnB = kFfnTN * 128;                // one token tile
constexpr int kFfnStage = 2 * kFfnA + kFfnB + 2048;  // + three scale atoms (1536 bytes), padded to the 1 KB the swizzle needs
constexpr int kFfnTmemCols = 256;                  // 2 x (32 gate + 32 up) accumulator columns + 12 scale columns
constexpr int kFfnMaxGroups = 256;

struct FfnArgs {
  const uint8_t* sf13;   // scale atoms of the gate/up weights [rows / 128][hidden / 128] x 512 bytes
  const uint8_t* sf2;    // scale atoms of the down weights    [rows / 128][inter / 128]
  const uint8_t* xsf;    // scale atoms of the token rows, one atom per 32 rows: [capacity / 32][hidden / 128]
  uint8_t* hsf;          // written by phase 0, read by phase 1: [capacity / 32][inter / 128]
  uint8_t* hq;           // e4m3 activations [capacity, ldh]
  __nv_bfloat16* y;      // result rows [capacity, ldy]
  int ldh, ldy;
  int hidden, inter, num_groups, capacity;
  const int* seg_start;  // [G] first row of each expert's segment (multiple of 32; segments are packed in expert order)
  const int* seg_count;  // [G]
  unsigned* ctr;         // [kFfnMaxBlocks] phase-0 epilogue warps done per block, [kFfnMaxBlocks] the same for phase 1, then CTAs done, grid-wide abort
  int stages;
  KernelStatus* status;
  // ---- optional combine + scatter phase (world > 0)
  const int* pair_row;   // [n_tok * topk] row of y holding (token, j), negative = not computed here
  const float* pair_w;   // [n_tok * topk] router weights
  int n_tok, topk, tokens_per_rank, world;
  float* slot[8];        // this rank's slot on GPU p: fp32 [tokens_per_rank, hidden]
  uint32_t* flag[8];     // this rank's flag on GPU p
  uint32_t* epoch_ctr;
};

struct FfnTile { int phase, b, nb; };

// The tile sequence of one CTA; the three roles of a CTA walk it independently.
struct FfnCursor {
  int t1, t2, nb1, nb2, p, c, r, skip, i1, k2;
  __host__ __device__ __forceinline__ FfnCursor(int blocks, int nb1_, int nb2_, int k1, int k2_steps, int grid, int cta)
      : t1(blocks * nb1_), t2(blocks * nb2_), nb1(nb1_), nb2(nb2_), p(grid), c(cta), i1(0) {
    r = t1 % p;
    // One phase-0 tile costs about k1 / k2 phase-1 tiles: the CTAs without the extra tile run that many rounds of phase 1
    // ahead.  Only worth it when there is at least one full round of phase 0: the early phase-1 tiles then belong to token
    // blocks whose phase-0 tiles are finished.  With fewer phase-0 tiles than CTAs every phase-1 tile has to wait for
    // them anyway, and handing them all to the CTAs without a phase-0 tile would serialise them there.
    skip = (r && t1 >= p) ? (k1 + k2_steps / 2) / k2_steps : 0;
    k2 = (c < r) ? skip : 0;
  }
  __host__ __device__ __forceinline__ bool next(FfnTile& t) {
    const int a = c + i1 * p;
    if (a < t1) { ++i1; t.phase = 0; t.b = a / nb1; t.nb = a - t.b * nb1; return true; }
    const int u = (k2 < skip) ? k2 * (p - r) + (c - r) : skip * (p - r) + (k2 - skip) * p + c;
    if (u >= t2) return false;
    ++k2; t.phase = 1; t.b = u / nb2; t.nb = u - t.b * nb2;
    return true;
  }
};

__device__ __forceinline__ float ffn_silu(float x) { return x / (1.0f + __expf(-x)); }

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kFfnThreads, 1)
moe_ffn_kernel(const __grid_constant__ CUtensorMap tmW13, const __grid_constant__ CUtensorMap tmX,
               const __grid_constant__ CUtensorMap tmW2, const __grid_constant__ CUtensorMap tmH, const FfnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int S = a.stages;
  uint8_t* tail = smem + (size_t)S * kFfnStage;
  uint64_t* full_bar = (uint64_t*)tail;              // [S]
  uint64_t* empty_bar = full_bar + S;                // [S]
  uint64_t* accf_bar = empty_bar + S;                // [2]
  uint64_t* acce_bar = accf_bar + 2;                 // [2]
  uint32_t* tmem_slot = (uint32_t*)(acce_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* s_nb = (int*)(tmem_slot + 2);
  int* s_assigned = (int*)(tmem_slot + 3);
  short* blk_g = (short*)(tmem_slot + 4);            // [kFfnMaxBlocks] expert of each token block
  uint8_t* blk_valid = (uint8_t*)(blk_g + kFfnMaxBlocks);   // [kFfnMaxBlocks] live rows of each token block

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k1 = a.hidden >> 7, k2 = a.inter >> 7;   // k-steps of the two phases
  const int nb1 = a.inter >> 7, nb2 = a.hidden >> 8; // tiles per token block
  unsigned* ctr2 = a.ctr + kFfnMaxBlocks;
  unsigned* done_ctr = a.ctr + 2 * kFfnMaxBlocks;
  unsigned* grid_abort = done_ctr + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&accf_bar[i], 1); mbar_init(&acce_bar[i], 4); }
    *abort_flag = 0; *s_nb = 0; *s_assigned = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmW13); tma_prefetch_desc(&tmX); tma_prefetch_desc(&tmW2); tma_prefetch_desc(&tmH);
  }
  for (int i = threadIdx.x; i < kFfnMaxBlocks; i += blockDim.x) blk_g[i] = -1;
  if (warp == 1) { tmem_alloc(tmem_slot, kFfnTmemCols); tmem_relinquish(); }
  __syncthreads();
  pdl_wait();
  // Block table from the segment arrays: block seg_start / 32 + i belongs to the segment's expert.  The segments must tile
  // [0, 32 * blocks) without holes; anything else is reported and the launch does nothing.
  for (int g = threadIdx.x; g < a.num_groups; g += blockDim.x) {
    const int st0 = a.seg_start[g], cn = a.seg_count[g];
    const bool sane = st0 >= 0 && cn >= 0 && (st0 & 31) == 0 && st0 <= a.capacity && cn <= a.capacity - st0;
    if (!sane) { report_status(a.status, ST_BAD_ARG, 630, g, st0, cn); *abort_flag = 1; continue; }
    const int nblk = (cn + 31) >> 5;
    for (int i = 0; i < nblk; ++i) {
      const int b = (st0 >> 5) + i;
      blk_g[b] = (short)g;
      blk_valid[b] = (uint8_t)min(32, cn - i * 32);
    }
    if (nblk > 0) { atomicAdd(s_assigned, nblk); atomicMax(s_nb, (st0 >> 5) + nblk); }
  }
  __syncthreads();
  if (threadIdx.x == 0 && !*abort_flag && *s_assigned != *s_nb) {
    report_status(a.status, ST_BAD_ARG, 631, *s_assigned, *s_nb, 0);
    *abort_flag = 1;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sf = tmem_base + 128;          // gate scales, up scales, token scales: 4 columns each
  const int blocks = *s_nb;
  const bool run = (*abort_flag == 0);

  if (!run) {
    // bad segment tables: nothing was issued
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (one lane)
    if (lane == 0) {
      FfnCursor cur(blocks, nb1, nb2, k1, k2, (int)gridDim.x, (int)blockIdx.x); FfnTile t;
      int s = 0; uint32_t ph = 0;
      bool ok = true;
      while (ok && cur.next(t)) {
        const int g = blk_g[t.b];
        const bool p0 = t.phase == 0;
        const int nk = p0 ? k1 : k2;
        const CUtensorMap* tw = p0 ? &tmW13 : &tmW2;
        const CUtensorMap* tx = p0 ? &tmX : &tmH;
        const int row0 = p0 ? g * 2 * a.inter + t.nb * 128 : g * a.hidden + t.nb * 128;
        const int row1 = row0 + (p0 ? a.inter : (a.hidden >> 1));
        const int wy0 = ((row0 >> 7) * nk) << 7, wy1 = ((row1 >> 7) * nk) << 7;
        const uint8_t* sfw = p0 ? a.sf13 : a.sf2;
        const uint8_t* sfa0 = sfw + (size_t)(row0 >> 7) * nk * 512;
        const uint8_t* sfa1 = sfw + (size_t)(row1 >> 7) * nk * 512;
        const uint8_t* sfb = (p0 ? a.xsf : (const uint8_t*)a.hsf) + (size_t)t.b * nk * 512;
        bool ready = p0;
        for (int kb = 0; kb < nk; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, a.status, 600, s)) { ok = false; break; }
          uint8_t* st = smem + (size_t)s * kFfnStage;
          uint8_t* sf = st + 2 * kFfnA + kFfnB;
          mbar_expect_tx(&full_bar[s], 2 * kFfnA + kFfnB + 3 * 512);
          tma_load_2d(st, tw, &full_bar[s], 0, wy0 + (kb << 7));
          tma_load_2d(st + kFfnA, tw, &full_bar[s], 0, wy1 + (kb << 7));
          bulk_load(sf, sfa0 + (size_t)kb * 512, 512, &full_bar[s]);
          bulk_load(sf + 512, sfa1 + (size_t)kb * 512, 512, &full_bar[s]);
          if (!ready) {
            // the weights of this tile are on their way; its activations exist once every phase-0 tile of the block has stored
            const unsigned want = (unsigned)nb1 * 4u;
            const uint64_t t0 = globaltimer_ns();
            for (uint32_t it = 0; ld_acquire_gpu(a.ctr + t.b) < want; ++it) {
              if ((it & 63u) == 63u) {
                if (*abort_flag || ld_acquire_gpu(grid_abort) != 0) { *abort_flag = 1; ok = false; break; }
                if (globaltimer_ns() - t0 > kMbarBudgetNs) {
                  report_status(a.status, ST_TIMEOUT_FLAG, 610, t.b, (int)want, (int)ld_acquire_gpu(a.ctr + t.b));
                  *abort_flag = 1; atomicExch(grid_abort, 1u); ok = false; break;
                }
              }
            }
            if (!ok) break;      // the copies issued for this stage land during the teardown's grace period
            asm volatile("fence.proxy.async.global;" ::: "memory");
            ready = true;
          }
          tma_load_2d(st + 2 * kFfnA, tx, &full_bar[s], kb << 7, t.b << 5);
          bulk_load(sf + 1024, sfb + (size_t)kb * 512, 512, &full_bar[s]);
          if (++s == S) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (one lane)
    if (lane == 0) {
      FfnCursor cur(blocks, nb1, nb2, k1, k2, (int)gridDim.x, (int)blockIdx.x); FfnTile t;
      int s = 0; uint32_t ph = 0;
      int acc = 0; uint32_t acc_ph = 0;
      bool ok = true;
      while (ok && cur.next(t)) {
        if (!mbar_wait(&acce_bar[acc], acc_ph ^ 1, abort_flag, a.status, 601, acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * 64;
        const int nk = t.phase == 0 ? k1 : k2;
        for (int kb = 0; kb < nk; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, a.status, 602, s)) { ok = false; break; }
          tc_fence_after();
          const uint32_t st = smem_u32(smem + (size_t)s * kFfnStage);
          const uint32_t sf = st + 2 * kFfnA + kFfnB;
          tc_cp_32x128b_warpx4(tmem_sf, make_sdesc_noswizzle(sf, 0, 128));
          tc_cp_32x128b_warpx4(tmem_sf + 4, make_sdesc_noswizzle(sf + 512, 0, 128));
          tc_cp_32x128b_warpx4(tmem_sf + 8, make_sdesc_noswizzle(sf + 1024, 0, 128));
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t a0 = make_sdesc_sw128(st + j * 32);
            const uint64_t a1 = make_sdesc_sw128(st + kFfnA + j * 32);
            const uint64_t b = make_sdesc_sw128(st + 2 * kFfnA + j * 32);
            const uint32_t accum = (kb > 0 || j > 0) ? 1u : 0u;
            const uint32_t idesc = make_idesc_mx(128, kFfnTN, 0, 0, j, j);
            mma_mxf8_ss(d0, a0, b, idesc, accum, tmem_sf, tmem_sf + 8);
            mma_mxf8_ss(d0 + kFfnTN, a1, b, idesc, accum, tmem_sf + 4, tmem_sf + 8);
          }
          tc_commit(&empty_bar[s]);
          if (++s == S) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        tc_commit(&accf_bar[acc]);
        if (++acc == 2) { acc = 0; acc_ph ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;                // weight row inside the tile == output feature
    FfnCursor cur(blocks, nb1, nb2, k1, k2, (int)gridDim.x, (int)blockIdx.x); FfnTile t;
    int acc = 0; uint32_t acc_ph = 0;
    while (cur.next(t)) {
      if (!mbar_wait(&accf_bar[acc], acc_ph, abort_flag, a.status, 603, acc)) break;
      tc_fence_after();
      const uint32_t tacc = tmem_base + acc * 64 + ((uint32_t)(q * 32) << 16);
      const int valid = blk_valid[t.b];
      const int x0 = t.b << 5;
      const int n = t.nb * 128 + row;
      uint32_t r0[32], r1[32];
      tmem_ld_x32(tacc, r0);
      tmem_ld_x32(tacc + kFfnTN, r1);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acce_bar[acc]);      // the accumulators are in registers: the MMA thread may reuse the buffer
      if (t.phase == 0) {
        uint8_t* hrow = a.hq + (size_t)x0 * a.ldh + n;
        uint8_t* sfrow = a.hsf + ((size_t)t.b * nb1 + t.nb) * 512 + q;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float v = ffn_silu(__uint_as_float(r0[j])) * __uint_as_float(r1[j]);
          // the 32 lanes of this warp are one 32-wide block along the feature axis of token j: one shared E8M0 scale
          const float amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(v))));
          const int e = e8m0_amax(amax);
          const float inv = __uint_as_float((uint32_t)(254 - e) << 23);   // 2^(127-e)
          if (j < valid) {
            __nv_fp8_e4m3 f8(v * inv);
            hrow[(size_t)j * a.ldh] = *(uint8_t*)&f8;
            if (lane == 0) sfrow[j * 16] = (uint8_t)e;
          }
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(a.ctr + t.b, 1u);
      } else {
        __nv_bfloat16* o = a.y + (size_t)x0 * a.ldy + n;
        const int half = a.hidden >> 1;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < valid) {
            o[(size_t)j * a.ldy] = __float2bfloat16(__uint_as_float(r0[j]));
            o[(size_t)j * a.ldy + half] = __float2bfloat16(__uint_as_float(r1[j]));
          }
        if (a.world > 0) {
          __threadfence();
          __syncwarp();
          if (lane == 0) atomicAdd(ctr2 + t.b, 1u);
        }
      }
      if (++acc == 2) { acc = 0; acc_ph ^= 1; }
    }
    // ---------------------------------------------------------------- combine + scatter (the 128 epilogue threads, token by token)
    if (a.world > 0) {
      __shared__ int c_rows[16];
      __shared__ float c_w[16];
      __shared__ int c_fail[2];                     // by iteration parity: the reset of one iteration cannot overtake the readers of the one before
      const int te = threadIdx.x - 64;               // 0..127
      const unsigned want = (unsigned)nb2 * 4u;
      int par = 0;
      for (int tok = blockIdx.x; tok < a.n_tok; tok += gridDim.x, par ^= 1) {
        if (te == 0) c_fail[par] = *abort_flag ? 1 : 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (te < a.topk) {
          const int r = a.pair_row[(size_t)tok * a.topk + te];
          c_rows[te] = r;
          c_w[te] = a.pair_w[(size_t)tok * a.topk + te];
          if (r >= 0) {
            // the row exists once every phase-1 tile of its token block has stored
            const unsigned* c = ctr2 + (r >> 5);
            const uint64_t t0 = globaltimer_ns();
            for (uint32_t it = 0; ld_acquire_gpu(c) < want; ++it) {
              if ((it & 63u) == 63u) {
                if (*abort_flag || ld_acquire_gpu(grid_abort) != 0) { c_fail[par] = 1; break; }
                if (globaltimer_ns() - t0 > kMbarBudgetNs) {
                  report_status(a.status, ST_TIMEOUT_FLAG, 620, r >> 5, (int)want, (int)ld_acquire_gpu(c));
                  *abort_flag = 1; atomicExch(grid_abort, 1u); c_fail[par] = 1; break;
                }
              }
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (c_fail[par]) break;                       // uniform: every thread reads the same shared word after the barrier
        const int home = tok / a.tokens_per_rank, lr = tok - home * a.tokens_per_rank;
        float* dst = a.slot[home] + (size_t)lr * a.hidden;
        for (int v = te; v < (a.hidden >> 3); v += 128) {
          float accv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int j = 0; j < a.topk; ++j) {
            const int r = c_rows[j];
            if (r < 0) continue;
            const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(a.y + (size_t)r * a.ldy + v * 8));
            const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(hh[i]); accv[2 * i] += c_w[j] * f.x; accv[2 * i + 1] += c_w[j] * f.y; }
          }
          reinterpret_cast<float4*>(dst + v * 8)[0] = make_float4(accv[0], accv[1], accv[2], accv[3]);
          reinterpret_cast<float4*>(dst + v * 8)[1] = make_float4(accv[4], accv[5], accv[6], accv[7]);
        }
      }
    }
  }

  // The kernel behind this one may be scheduled now: released at the start, its CTAs would sit on the SMs for the whole
  // 100 us of this kernel (measured: the decode step is 0.4 ms slower with the early release).
  pdl_trigger();
  // Teardown.  After an abort, copies may still be landing in shared memory: give them a bounded grace period before the
  // CTA (and its shared memory) goes away.
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kFfnTmemCols); }
  if (threadIdx.x == 0) {
    // the last CTA to get here leaves the counters at zero for the next launch
    __threadfence();
    if (atomicAdd(done_ctr, 1u) == gridDim.x - 1) {
      __threadfence();
      const int nclr = min(kFfnMaxBlocks, (a.capacity + 31) >> 5);
      for (int i = 0; i < nclr; ++i) { a.ctr[i] = 0; ctr2[i] = 0; }
      *grid_abort = 0;
      *done_ctr = 0;
      if (a.world > 0) {
        // every CTA ordered its slot rows before its arrival (fence + atomic): publish them with one system-scope fence
        __threadfence_system();
        const uint32_t e = *a.epoch_ctr + 1;
        *a.epoch_ctr = e;
        for (int p = 0; p < a.world; ++p) {
          asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(a.flag[p]), "r"(e) : "memory");
        }
      }
    }
  }
}

}  // namespace gb

using namespace gb;

GB_API int gb_moe_ffn_supported(int hidden, int inter, int num_groups, int capacity) {
  return hidden >= 256 && hidden % 256 == 0 && inter >= 128 && inter % 128 == 0 && num_groups > 0 && num_groups <= kFfnMaxGroups &&
         capacity > 0 && capacity % 32 == 0 && capacity / 32 <= kFfnMaxBlocks;
}
// Number of 32-bit counters `ctr` must hold (zeroed once by the caller; the kernel leaves them zeroed).
GB_API int gb_moe_ffn_ctr_count() { return 2 * kFfnMaxBlocks + 2; }

// The tile sequence of CTA `cta` of a grid of `grid` CTAs, as the kernel walks it: out[3 * i + 0..2] = (phase, block, n-block).
// Returns the number of tiles (which may exceed `cap`; only `cap` are written).  Host-side: lets a test check that the
// sequences of all CTAs cover every tile exactly once and keep phase 0 ahead of phase 1.
GB_API int gb_moe_ffn_schedule(int blocks, int hidden, int inter, int grid, int cta, int* out, int cap) {
  FfnCursor cur(blocks, inter >> 7, hidden >> 8, hidden >> 7, inter >> 7, grid, cta);
  FfnTile t;
  int n = 0;
  while (cur.next(t)) {
    if (n < cap) { out[3 * n] = t.phase; out[3 * n + 1] = t.b; out[3 * n + 2] = t.nb; }
    ++n;
  }
  return n;
}

// Fused expert FFN over rows in expert order.
//   w13 / sf13  tiled e4m3 gate/up weights [G][2 * inter rows][hidden] + scale atoms; w2 / sf2 the down weights [G][hidden rows][inter]
//   xq / xsf    token rows [capacity, ldx] e4m3 + scale atoms in the one-atom-per-32-rows layout
//   hq / hsf    scratch for the activations (written and read inside the launch)
//   y           bf16 [capacity, ldy] result rows; rows of a segment beyond seg_count are not written
//   world > 0   adds the combine + scatter phase: pair_row / pair_w [n_tok * topk], n_tok = tokens_per_rank * world tokens, slots[p] /
//               flags[p] this rank's fp32 slot and flag on GPU p (as mapped here), epoch_ctr the exchange's epoch counter
GB_API int gb_moe_ffn(const void* w13, const void* sf13, long sf13_bytes, const void* w2, const void* sf2, long sf2_bytes,
                      const void* xq, int ldx, const void* xsf, long xsf_bytes, void* hq, int ldh, void* hsf, long hsf_bytes,
                      void* y, int ldy, long y_bytes, int hidden, int inter, int num_groups, const int* seg_start,
                      const int* seg_count, int capacity, unsigned* ctr, int ctr_count, const int* pair_row, const float* pair_w,
                      int n_tok, int topk, int tokens_per_rank, void* const* slots, void* const* flags, int world, void* epoch_ctr,
                      void* status, cudaStream_t stream) {
  if (!gb_moe_ffn_supported(hidden, inter, num_groups, capacity)) return fail("moe_ffn: unsupported shape%s (hidden=%ld inter=%ld)", "", hidden, inter);
  if (ctr == nullptr || ctr_count < gb_moe_ffn_ctr_count()) return fail("moe_ffn: counter buffer too small%s");
  const long k1 = hidden / 128, k2 = inter / 128, blocks = capacity / 32;
  if (sf13_bytes < (long)num_groups * (2 * inter / 128) * k1 * 512) return fail("moe_ffn: gate/up scale buffer too small%s");
  if (sf2_bytes < (long)num_groups * (hidden / 128) * k2 * 512) return fail("moe_ffn: down scale buffer too small%s");
  if (xsf_bytes < blocks * k1 * 512) return fail("moe_ffn: token scale buffer too small%s");
  if (hsf_bytes < blocks * k2 * 512) return fail("moe_ffn: activation scale buffer too small%s");
  if (ldx < hidden || ldh < inter || ldy < hidden || ldx % 16 || ldh % 16) return fail("moe_ffn: bad leading dimension%s");
  if (y_bytes < (long)capacity * ldy * 2) return fail("moe_ffn: result buffer too small%s");
  if (((uintptr_t)w13 | (uintptr_t)w2 | (uintptr_t)xq | (uintptr_t)hq | (uintptr_t)sf13 | (uintptr_t)sf2 | (uintptr_t)xsf | (uintptr_t)hsf) & 15)
    return fail("moe_ffn: operands must be 16-byte aligned%s");
  const uint64_t rows13 = (uint64_t)num_groups * (2 * inter / 128) * k1 * 128, rows2 = (uint64_t)num_groups * (hidden / 128) * k2 * 128;
  if (rows13 >= (1ull << 31) || rows2 >= (1ull << 31)) return fail("moe_ffn: tiled weight too large for 32-bit tile coordinates%s");
  CUtensorMap tmW13, tmX, tmW2, tmH;
  if (make_tmap_2d(&tmW13, w13, TM_U8, 128, rows13, 128, 128, 128, TM_SW_128)) return -1;
  if (make_tmap_2d(&tmW2, w2, TM_U8, 128, rows2, 128, 128, 128, TM_SW_128)) return -1;
  if (make_tmap_2d(&tmX, xq, TM_U8, (uint64_t)hidden, (uint64_t)capacity, (uint64_t)ldx, 128, kFfnTN, TM_SW_128)) return -1;
  if (make_tmap_2d(&tmH, hq, TM_U8, (uint64_t)inter, (uint64_t)capacity, (uint64_t)ldh, 128, kFfnTN, TM_SW_128)) return -1;
  FfnArgs a;
  memset(&a, 0, sizeof(a));
  a.sf13 = (const uint8_t*)sf13; a.sf2 = (const uint8_t*)sf2; a.xsf = (const uint8_t*)xsf; a.hsf = (uint8_t*)hsf;
  a.hq = (uint8_t*)hq; a.y = (__nv_bfloat16*)y; a.ldh = ldh; a.ldy = ldy;
  a.hidden = hidden; a.inter = inter; a.num_groups = num_groups; a.capacity = capacity;
  a.seg_start = seg_start; a.seg_count = seg_count; a.ctr = ctr; a.status = (KernelStatus*)status;
  if (world > 0) {
    if (world > 8 || pair_row == nullptr || pair_w == nullptr || slots == nullptr || flags == nullptr || epoch_ctr == nullptr || topk < 1 ||
        topk > 16 || tokens_per_rank < 1 || n_tok != tokens_per_rank * world || hidden % 8)
      return fail("moe_ffn: bad combine arguments%s");
    a.pair_row = pair_row; a.pair_w = pair_w; a.n_tok = n_tok; a.topk = topk; a.tokens_per_rank = tokens_per_rank; a.world = world;
    a.epoch_ctr = (uint32_t*)epoch_ctr;
    for (int p = 0; p < world; ++p) { a.slot[p] = (float*)slots[p]; a.flag[p] = (uint32_t*)flags[p]; }
  }
  const int tail = 1024 + kFfnMaxBlocks * 3 + 256;
  int stages = (220 * 1024 - tail - 1024) / kFfnStage;
  if (stages > 8) stages = 8;
  a.stages = stages;
  const int smem = stages * kFfnStage + tail + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA_OK(cudaFuncSetAttribute(moe_ffn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    attr_set = true;
  }
  // all CTAs must be resident at once (a CTA may wait for tiles of another): one per SM, never more than there are SMs
  launch_k(moe_ffn_kernel, sm_count(), kFfnThreads, smem, stream, tmW13, tmX, tmW2, tmH, a);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}
