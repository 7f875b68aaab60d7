// Fused dequant-GEMM for ggml-quantised weights (Q4_K, Q8_0) that stay quantised in HBM:
//   out[token, n] = sum_k W[n, k] * x[token, k],  five tokens and more (prefill, batched decode).
//
// The quantised blocks never become a bf16 matrix in memory.  Per 128-row x 256-column tile of W (one contiguous piece of the
// tiled layout of ops/ggml_torch.py) a bulk copy brings the raw blocks into shared memory; sixteen warps unpack them in registers
// (nibbles -> bf16 pairs with byte permutes, d * sc and dmin * m applied per 32-wide sub-block in packed bf16 arithmetic; int8 ->
// fp32 -> bf16 for Q8_0) and write the result straight into the 128-byte-swizzled K-major operand tile that tcgen05.mma reads;
// the tokens come in by TMA; the accumulator lives in TMEM.  Orientation as in the dense GEMM: W is the MMA A operand (128 rows
// = 128 TMEM lanes), the tokens are N (16 .. 128 per tile).
//
// Warp roles of a CTA (704 threads): warp 0 producer (bulk copies of raw tiles, TMA loads of token tiles), warp 1 MMA issuer,
// warps 2-5 epilogue (TMEM -> registers -> global), warps 6-21 unpack (a thread per 32-value sub-block and row).  Rings: raw tiles (2-4, what shared memory leaves), bf16 operand tiles of 128 x 128
// (2), token tiles (2-3), accumulators (2); all waits are bounded and report into the status word.
//
// A raw Q4_K tile is 18 KB for 64 KB of bf16 operand: at decode sizes the kernel is bound by the HBM stream of the quantised
// bytes, not by the four times larger operand it feeds to the tensor core.
//
// Replaces in the reference: mmq_q4_K_grouped and the other mma.sync MMQ kernels (cuda/llm/cuda_llm_runner.c:5295-7329,
// mmq/mmq_q4_K_test.cu:17-24 describes the scale handling), the dequant_*_to_f16 + cuBLAS pairs (:999-5447, :15488-17418) and
// batch_matvec_q4_K / q8_0 (:4433-4854); CPU oracle gemm_*_tokmajor of common/ggml_dequant.h:298-349.
#include "sm100.cuh"
#include "host_common.h"
#include <cuda_bf16.h>

namespace gb {

constexpr int kQgThreads = 704;
constexpr int kQgUnpackWarp0 = 6;          // first unpack warp
constexpr int kQgUnpackThreads = 512;   // 16 warps: a thread unpacks one 32-value sub-block of one row
constexpr int kQgA = 128 * 256;            // bytes of one bf16 operand stage: 2 atoms of [128 rows][64 k]

struct QGemmArgs {
  const uint8_t* w;                 // tiled weights [row_tiles][num_kb][tile bytes]
  void* out; int ldo; int out_f32;
  const float* bias;
  int n_out, m_tok, num_kb, row_tiles, tok_tiles;
  int splits, kb_per;            // K splits per output tile (>= 1) and 256-column blocks per split
  long partial_stride;           // splits > 1: split ks stores its fp32 partial at out + ks * partial_stride (elements)
  int b_stages, raw_stages;
  KernelStatus* status;
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) { return __byte_perm(a, b, sel); }

// One 32-value sub-block of a Q4_K chunk: the low (nib = 0) or high (nib = 1) nibbles of the 32 bytes `q0 q1`, scale a = d * sc
// and offset b = dmin * m  ->  four 16-byte chunks of bf16 (values 32 * nib + 8c .. + 7, c < 4) in the swizzled operand row.
__device__ __forceinline__ void unpack_q4k_sub(const uint4 q0, const uint4 q1, int nib, float a, float b, uint8_t* dst_row, int row) {
  const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
  const __nv_bfloat162 sixteen = __float2bfloat162_rn(16.0f);
  const __nv_bfloat162 a2 = __float2bfloat162_rn(a), b2 = __float2bfloat162_rn(-b);
  const int sh = nib ? 1 : 0;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 o;
    uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      // bf16(16 + q) = 0x4180 | (q << 3): exact for q < 16; the low byte carries 0x80 | q << 3, the high byte is 0x41
      const uint32_t x = w[2 * c + u];
      const uint32_t n3 = ((sh ? (x >> 1) : (x << 3)) & 0x78787878u) | 0x80808080u;
      uint32_t p0 = prmt(n3, 0x41414141u, 0x4140), p1 = prmt(n3, 0x41414141u, 0x4342);
      __nv_bfloat162 x0 = *reinterpret_cast<__nv_bfloat162*>(&p0), x1 = *reinterpret_cast<__nv_bfloat162*>(&p1);
      x0 = __hfma2(__hsub2(x0, sixteen), a2, b2);            // q * a - b, one rounding
      x1 = __hfma2(__hsub2(x1, sixteen), a2, b2);
      po[2 * u] = *reinterpret_cast<uint32_t*>(&x0); po[2 * u + 1] = *reinterpret_cast<uint32_t*>(&x1);
    }
    *reinterpret_cast<uint4*>(dst_row + (((4 * nib + c) ^ (row & 7)) << 4)) = o;
  }
}

// One Q8_0 block (32 int8 in two 16-byte vectors, scale d) -> four swizzled 16-byte chunks of bf16 (chunk index 4 * nib + c).
__device__ __forceinline__ void unpack_q80_sub(const uint4 qa, const uint4 qb, int nib, float d, uint8_t* dst_row, int row) {
  const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 o;
    uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const uint32_t x = w[2 * c + u];
      const float f0 = (float)(int)(int8_t)(x & 0xff), f1 = (float)(int)(int8_t)((x >> 8) & 0xff);
      const float f2 = (float)(int)(int8_t)((x >> 16) & 0xff), f3 = (float)(int)(int8_t)(x >> 24);
      po[2 * u] = pack_bf16x2(f0 * d, f1 * d); po[2 * u + 1] = pack_bf16x2(f2 * d, f3 * d);
    }
    *reinterpret_cast<uint4*>(dst_row + (((4 * nib + c) ^ (row & 7)) << 4)) = o;
  }
}

// TYPE: 0 = Q4_K, 1 = Q8_0.  TN: token tile.
template <int TYPE, int TN>
__global__ void __launch_bounds__(kQgThreads, 1)
qgemm_kernel(const __grid_constant__ CUtensorMap tmX, const QGemmArgs args) {
  constexpr int RAW = TYPE == 0 ? 128 * 144 : 128 * 272;                 // bytes of a raw tile (Q8_0 row: 256 values + 8 f16 scales)
  constexpr int RAW_PAD = (RAW + 1023) & ~1023;
  constexpr int B_BYTES = TN * 256;                                      // token stage: 2 atoms of [TN rows][64 k]
  constexpr int TMEM_COLS = 2 * TN < 32 ? 32 : 2 * TN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int BS = args.b_stages, RS = args.raw_stages;
  uint8_t* rawb = smem;                                  // [RS][RAW_PAD]
  uint8_t* Ab = rawb + (size_t)RS * RAW_PAD;             // [2][kQgA]
  uint8_t* Bb = Ab + 2 * kQgA;                           // [BS][B_BYTES]
  uint64_t* bars = reinterpret_cast<uint64_t*>(Bb + (size_t)BS * B_BYTES);
  uint64_t* raw_full = bars;            // [4]
  uint64_t* raw_empty = bars + 4;       // [4]  8 arrivals (unpack warps)
  uint64_t* a_full = bars + 8;          // [2]  8 arrivals
  uint64_t* a_empty = bars + 10;        // [2]  1 (tcgen05.commit)
  uint64_t* b_full = bars + 12;         // [4]
  uint64_t* b_empty = bars + 16;        // [4]  1 (commit)
  uint64_t* accf = bars + 20;           // [2]
  uint64_t* acce = bars + 22;           // [2]  4 arrivals (epilogue warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = args.row_tiles * args.tok_tiles * args.splits;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&a_full[i], kQgUnpackThreads / 32); mbar_init(&a_empty[i], 1); mbar_init(&accf[i], 1); mbar_init(&acce[i], 4); }
    for (int i = 0; i < 4; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], kQgUnpackThreads / 32); mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], 1); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  __syncthreads();
  pdl_wait();
  pdl_trigger();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int rs = 0; uint32_t rph = 0; int bs = 0; uint32_t bph = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x) {
        const int ksp = t % args.splits, tt = t / args.splits;
        const int rt = tt % args.row_tiles, tb = tt / args.row_tiles;
        const uint8_t* wt = args.w + (size_t)rt * args.num_kb * RAW;
        const int kb0 = ksp * args.kb_per, kb1 = min(args.num_kb, kb0 + args.kb_per);
        for (int kb = kb0; ok && kb < kb1; ++kb) {
          if (!mbar_wait(&raw_empty[rs], rph ^ 1, abort_flag, args.status, 1200, rs)) { ok = false; break; }
          mbar_expect_tx(&raw_full[rs], RAW);
          bulk_load(rawb + (size_t)rs * RAW_PAD, wt + (size_t)kb * RAW, RAW, &raw_full[rs]);
          if (++rs == RS) { rs = 0; rph ^= 1; }
          for (int h = 0; h < 2; ++h) {
            if (!mbar_wait(&b_empty[bs], bph ^ 1, abort_flag, args.status, 1201, bs)) { ok = false; break; }
            mbar_expect_tx(&b_full[bs], B_BYTES);
            uint8_t* dst = Bb + (size_t)bs * B_BYTES;
            const int kx = kb * 256 + h * 128;
            tma_load_2d(dst, &tmX, &b_full[bs], kx, tb * TN);
            tma_load_2d(dst + TN * 128, &tmX, &b_full[bs], kx + 64, tb * TN);
            if (++bs == BS) { bs = 0; bph ^= 1; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int as = 0; uint32_t aph = 0; int bs = 0; uint32_t bph = 0; int acc = 0; uint32_t acc_ph = 0;
      bool ok = true;
      constexpr uint32_t idesc = make_idesc(128, TN, 1, 1);
      for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x) {
        if (!mbar_wait(&acce[acc], acc_ph ^ 1, abort_flag, args.status, 1210, acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * TN;
        const int kb0 = (t % args.splits) * args.kb_per, nkb = min(args.num_kb, kb0 + args.kb_per) - kb0;
        for (int ks = 0; ok && ks < 2 * nkb; ++ks) {
          if (!mbar_wait(&a_full[as], aph, abort_flag, args.status, 1211, as)) { ok = false; break; }
          if (!mbar_wait(&b_full[bs], bph, abort_flag, args.status, 1212, bs)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a0 = smem_u32(Ab + (size_t)as * kQgA), b0 = smem_u32(Bb + (size_t)bs * B_BYTES);
#pragma unroll
          for (int at = 0; at < 2; ++at)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              mma_f16_ss(d0, make_sdesc_sw128(a0 + at * (128 * 128) + j * 32), make_sdesc_sw128(b0 + at * (TN * 128) + j * 32), idesc,
                         (ks > 0 || at > 0 || j > 0) ? 1u : 0u);
          tc_commit(&a_empty[as]);
          tc_commit(&b_empty[bs]);
          if (++as == 2) { as = 0; aph ^= 1; }
          if (++bs == BS) { bs = 0; bph ^= 1; }
        }
        if (!ok) break;
        tc_commit(&accf[acc]);
        if (++acc == 2) { acc = 0; acc_ph ^= 1; }
      }
    }
  } else if (warp < kQgUnpackWarp0) {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    const int row = q * 32 + lane;
    int acc = 0; uint32_t acc_ph = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x) {
      const int ksp = t % args.splits, tt = t / args.splits;
      const int rt = tt % args.row_tiles, tb = tt / args.row_tiles;
      if (!mbar_wait(&accf[acc], acc_ph, abort_flag, args.status, 1220, acc)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tacc = tmem_base + acc * TN + ((uint32_t)(q * 32) << 16);
      const int n = rt * 128 + row;
      const bool n_ok = n < args.n_out;
      const float bias = (args.bias != nullptr && n_ok && ksp == 0) ? args.bias[n] : 0.f;
      const int tok0 = tb * TN, valid = min(TN, args.m_tok - tok0);
      const size_t part = (size_t)ksp * (size_t)args.partial_stride;
#pragma unroll 1
      for (int c = 0; c < TN; c += 16) {
        uint32_t r[16];
        tmem_ld_x16(tacc + c, r);
        tc_wait_ld();
        if (c >= valid || !n_ok) continue;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c + j >= valid) break;
          const float v = __uint_as_float(r[j]) + bias;
          const size_t off = part + (size_t)(tok0 + c + j) * args.ldo + n;
          if (args.out_f32) reinterpret_cast<float*>(args.out)[off] = v;
          else reinterpret_cast<__nv_bfloat16*>(args.out)[off] = __float2bfloat16(v);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acce[acc]);
      if (++acc == 2) { acc = 0; acc_ph ^= 1; }
    }
  } else {
    // ------------------------------------------------------------------ unpack (warps 6..21): raw blocks -> swizzled bf16 operand
    const int ut = threadIdx.x - kQgUnpackWarp0 * 32;     // 0..511
    const int row = ut >> 2, cpar = (ut >> 1) & 1, nib = ut & 1;       // item: sub-block (2j + nib) of row `row`, atom cpar of every stage
    int rs = 0; uint32_t rph = 0; int as = 0; uint32_t aph = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x) {
      const int kb0 = (t % args.splits) * args.kb_per, kb1 = min(args.num_kb, kb0 + args.kb_per);
      for (int kb = kb0; ok && kb < kb1; ++kb) {
        if (!mbar_wait(&raw_full[rs], rph, abort_flag, args.status, 1230, rs)) { ok = false; break; }
        const uint8_t* rb = rawb + (size_t)rs * RAW_PAD;
        for (int h = 0; h < 2; ++h) {
          if (!mbar_wait(&a_empty[as], aph ^ 1, abort_flag, args.status, 1231, as)) { ok = false; break; }
          const int j = 2 * h + cpar;                      // 64-value chunk of the 256-column tile
          uint8_t* dst_row = Ab + (size_t)as * kQgA + cpar * (128 * 128) + row * 128;
          if (TYPE == 0) {
            const uint8_t* b = rb + row * 144;
            const uint4 hd = *reinterpret_cast<const uint4*>(b);
            const uint4 q0 = *reinterpret_cast<const uint4*>(b + 16 + 32 * j), q1 = *reinterpret_cast<const uint4*>(b + 32 + 32 * j);
            const __half2 dd = *reinterpret_cast<const __half2*>(&hd.x);
            const float d = __low2float(dd), dmin = __high2float(dd);
            const int bsh = 16 * cpar + 8 * nib;           // byte (2 * cpar + nib) of the scale words
            uint32_t sc, mn;
            if (h == 0) {                                  // sub-blocks 0..3: 6 bits straight from bytes 0..3 / 4..7
              sc = (hd.y >> bsh) & 63u; mn = (hd.z >> bsh) & 63u;
            } else {                                       // sub-blocks 4..7: low 4 bits in bytes 8..11, high 2 bits in the top of bytes 0..7
              const uint32_t x = (hd.w >> bsh) & 0xffu, y = (hd.y >> bsh) & 0xffu, z = (hd.z >> bsh) & 0xffu;
              sc = (x & 15u) | ((y >> 6) << 4); mn = (x >> 4) | ((z >> 6) << 4);
            }
            unpack_q4k_sub(q0, q1, nib, d * (float)sc, dmin * (float)mn, dst_row, row);
          } else {
            const uint4* qp = reinterpret_cast<const uint4*>(rb + row * 272 + 64 * j + 32 * nib);
            const __half dh = *reinterpret_cast<const __half*>(rb + row * 272 + 256 + (2 * j + nib) * 2);
            unpack_q80_sub(qp[0], qp[1], nib, __half2float(dh), dst_row, row);
          }
          fence_proxy_async_smem();                        // this thread's operand bytes -> visible to the tensor core
          __syncwarp();
          if (lane == 0) mbar_arrive(&a_full[as]);
          if (++as == 2) { as = 0; aph ^= 1; }
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(&raw_empty[rs]);
        if (++rs == RS) { rs = 0; rph ^= 1; }
      }
    }
  }

  if (*abort_flag) {                                       // copies may still be landing: bounded grace period
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

template <int TYPE, int TN>
static int launch_qgemm(const CUtensorMap& tmX, QGemmArgs a, cudaStream_t stream) {
  constexpr int RAW = TYPE == 0 ? 128 * 144 : 128 * 272;
  constexpr int RAW_PAD = (RAW + 1023) & ~1023;
  constexpr int B_BYTES = TN * 256;
  // token ring first (2 stages at least, 3 for wide tiles if they fit), the rest of shared memory buys depth for the raw-tile ring:
  // the quantised bytes in flight are what a decode-sized launch is bound by
  const int budget = 220 * 1024 - 2048 - 2 * kQgA;
  int bs = TN >= 128 ? 2 : 4;
  int rs = (budget - bs * B_BYTES) / RAW_PAD;
  if (rs > 4) rs = 4;
  if (rs >= 3 && TN >= 128 && budget - 3 * B_BYTES >= 2 * RAW_PAD) { bs = 3; rs = (budget - bs * B_BYTES) / RAW_PAD; if (rs > 4) rs = 4; }
  if (rs < 2) return fail("qgemm: token tile does not fit shared memory%s");
  a.b_stages = bs; a.raw_stages = rs;
  const int smem = 1024 + rs * RAW_PAD + 2 * kQgA + bs * B_BYTES + 512;
  auto kern = qgemm_kernel<TYPE, TN>;
  static bool attr_set = false;
  if (!attr_set) { GB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 222 * 1024)); attr_set = true; }
  int grid = sm_count();
  const int tiles = a.row_tiles * a.tok_tiles * a.splits;
  if (tiles < grid) grid = tiles;
  launch_k(kern, grid, kQgThreads, smem, stream, tmX, a);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace gb

using namespace gb;

// w: tiled Q4_K (ggml type 12) or Q8_0 (8) weights, ceil(n_out / 128) row tiles x k / 256 K tiles.  x bf16 [m, ldx].
// out bf16 (or f32) [m, ldo].  tn: token tile 16, 32, 64 or 128.  splits > 1 cuts K: `out` is then f32 [splits][m, ldo] (slabs
// m * ldo apart), one partial sum per split for the consumer to add; no split may be empty.
GB_API int gb_qgemm(const void* w, int ggml_type, const void* x, int ldx, void* out, int ldo, int out_f32, const float* bias, int n_out,
                    int k, int m, int tn, int splits, void* status, cudaStream_t stream) {
  if (ggml_type != 12 && ggml_type != 8) return fail("qgemm: only Q4_K and Q8_0 have a fused tensor-core path%s");
  if (k <= 0 || k % 256 || n_out <= 0) return fail("qgemm: k must be a positive multiple of 256%s");
  if (m <= 0) return 0;
  if (ldx % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail("qgemm: operands must be 16-byte aligned%s");
  CUtensorMap tmX;
  if (make_tmap_2d(&tmX, x, TM_BF16, (uint64_t)k, (uint64_t)m, (uint64_t)ldx * 2, 64, (uint32_t)tn, TM_SW_128)) return -1;
  QGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.w = (const uint8_t*)w; a.out = out; a.ldo = ldo; a.out_f32 = out_f32; a.bias = bias; a.n_out = n_out; a.m_tok = m; a.num_kb = k / 256;
  a.row_tiles = (n_out + 127) / 128; a.tok_tiles = (m + tn - 1) / tn; a.status = (KernelStatus*)status;
  a.splits = splits > 1 ? splits : 1;
  a.kb_per = (a.num_kb + a.splits - 1) / a.splits;
  if (a.splits > 1) {
    if (!out_f32) return fail("qgemm: K-split partials need an fp32 output%s");
    if ((a.num_kb + a.kb_per - 1) / a.kb_per != a.splits) return fail("qgemm: a K split would be empty%s");
    a.partial_stride = (long)m * ldo;
  }
  const int t = ggml_type == 12 ? 0 : 1;
#define GB_QG(TNV)                                                             \
  if (tn == TNV) return t == 0 ? launch_qgemm<0, TNV>(tmX, a, stream) : launch_qgemm<1, TNV>(tmX, a, stream);
  GB_QG(16) GB_QG(32) GB_QG(64) GB_QG(128)
#undef GB_QG
  return fail("qgemm: token tile must be 16, 32, 64 or 128%s");
}
