// Fused dequant-GEMV for ggml-quantised weights that stay quantised in HBM: out[m, n] = sum_k W[n, k] * x[m, k] for one to
// four tokens (latency-bound decode), W in Q4_K or Q8_0 blocks in the tiled layout of ops/ggml_torch.py (tiles of 128 rows x
// 256 columns, each one contiguous piece of memory).
//
// How the bytes become arithmetic.  The activations are quantised to int8 per 32 values inside the kernel (fp32 scale d8 and
// the block sum s8 = d8 * sum(q8) kept beside them in shared memory), so that a 32-bit word of weight nibbles / bytes meets a
// word of activations in one dp4a:
//   Q8_0:  acc += d * d8 * sum_i dp4a(q, q8)
//   Q4_K:  acc += (d * sc) * d8 * sum_i dp4a(nibbles, q8)  -  (dmin * m) * s8      per 32-wide sub-block
// (d * sc and dmin * m are applied once per sub-block, after the integer sum).  A weight word is unpacked once and used for every
// token and both rows of a thread; a CTA never reads a weight byte twice, and every 16-byte load of a warp falls into one
// contiguous stretch of its tile.
//
// Work split.  A CTA owns one row tile (128 output features) and a range of the K tiles (split-K: a projection with few rows still
// fills the GPU; every split writes its fp32 partial into its own slab and the consumer adds the slabs in split order, as the
// tensor-core GEMM's K-split does).  Inside a tile a lane owns one row and two of its four 64-value chunks; the activation words
// it needs are the same for all lanes of a half warp (a shared-memory broadcast).
//
// With tensor parallelism the result rows can go straight into this rank's slot on every GPU (peer stores) and the last CTA
// raises the arrival flags: the one-shot all-reduce of a row-parallel projection is the tail of the GEMV, its sum happens in the
// RMSNorm that follows (gb_rmsnorm_reduce2).
//
// Replaces in the reference: matvec_q4_K_q8_1_dp4a (cuda/llm/cuda_llm_runner.c:1307), quantize_f32_to_q8_1 (:1039),
// matvec_q8_0_dp4a / matvec_q8_0_f16act (:611, :711), the fused gate/up pair matvec_q8_0_dp4a_fused2 (:752) and the dispatcher
// launch_matvec_auto (:13363-13506); CPU counterpart tf_qmatvec_worker (common/transformer.h:648-738).
#include "sm100.cuh"
#include "host_common.h"
#include "../fabric/fabric.cuh"

namespace gb {

constexpr int kQvThreads = 256;
constexpr int kQ4KTileBytes = 128 * 144;
constexpr int kQ80RowBytes = 256 + 16;            // a row of a Q8_0 tile: 256 int8 values, then its eight f16 scales
constexpr int kQ80TileBytes = 128 * kQ80RowBytes;

struct QGemvArgs {
  const uint8_t* w;                 // tiled weights [row_tiles][num_kb][tile bytes]
  const __nv_bfloat16* x; int ldx;  // activations [m, k]
  float* out; int ldo;              // fp32 [splits][m][ldo]
  long partial_stride;              // elements between the slabs of two K splits
  const float* bias;                // optional [n_out], added by split 0
  int n_out, row_tiles, num_kb, kb_per, splits;
  void* peer_out[kMaxRanks];        // peer_bcast > 0: the slab goes to peer_out[p] for every p < peer_bcast instead of `out`
  int peer_bcast;
  uint32_t* signal_flags[kMaxRanks];
  int signal_n;
  unsigned* done_ctr;
  uint32_t* epoch_ptr;
  int epoch_self_tick;
  int stages;
  KernelStatus* status;
};

__device__ __forceinline__ int dp4a_s(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }
__device__ __forceinline__ uint32_t byte_of(uint32_t w, int i) { return (w >> (8 * i)) & 0xffu; }

// TYPE: 0 = Q4_K, 1 = Q8_0.  M tokens.  Persistent: CTA b walks a contiguous range of the work items (K split, row tile), which are
// ordered split-major, so its items mostly share their K range and the quantised activations are rebuilt only when the split
// changes.  Weight tiles travel through a ring of `stages` shared-memory slots filled by bulk copies (one elected thread issues
// them, an mbarrier per slot counts the bytes) that runs ahead across item boundaries: the bytes in flight per SM are what
// bounds a memory-bound GEMV, and registers alone cannot hold enough of them.
// Thread mapping inside a 128 x 256 tile: warp w owns rows 16 w .. 16 w + 15; lane l works on row 16 w + (l & 15) and on the two
// 64-value chunks 2 (l >> 4) and 2 (l >> 4) + 1, so a row's sum is one shuffle away and an item needs no block-wide step.
template <int TYPE, int M>
__global__ void __launch_bounds__(kQvThreads, 2)
qgemv_kernel(const QGemvArgs a) {
  extern __shared__ uint8_t qv_smem_raw[];
  uint8_t* qv_smem = (uint8_t*)(((uintptr_t)qv_smem_raw + 127) & ~(uintptr_t)127);
  constexpr int TILE = TYPE == 0 ? kQ4KTileBytes : kQ80TileBytes;
  const int S = a.stages;
  const int n_items = a.row_tiles * a.splits;
  const int it0 = (int)((long)blockIdx.x * n_items / gridDim.x), it1 = (int)((long)(blockIdx.x + 1) * n_items / gridDim.x);
  uint8_t* ring = qv_smem;                                                       // [S][TILE]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring + (size_t)S * TILE);     // [S]
  uint64_t* empty_bar = full_bar + S;                                            // [S] 8 arrivals (one per warp)
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + S);
  int8_t* aq = reinterpret_cast<int8_t*>(ring + (size_t)S * TILE + 128);         // [kb_per][M][256]
  float* ad = reinterpret_cast<float*>(aq + (size_t)a.kb_per * M * 256);         // [kb_per][M][8] block scales
  float* as = ad + (size_t)a.kb_per * M * 8;                                     // [kb_per][M][8] block sums (d8 * sum q8)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // producer cursor (thread 0 only): next tile to request = K tile p_kb of item p_it
  int p_it = it0, p_kb = 0, p_st = 0;
  auto item_range = [&](int it, int& tile_id, int& kb0, int& nkb) {
    const int ks = it / a.row_tiles;
    tile_id = it - ks * a.row_tiles;
    kb0 = ks * a.kb_per;
    nkb = min(a.num_kb, kb0 + a.kb_per) - kb0;
  };
  auto issue_next = [&]() {                                  // the slot p_st must be free
    int tile_id, kb0, nkb;
    item_range(p_it, tile_id, kb0, nkb);
    mbar_expect_tx(&full_bar[p_st], TILE);
    bulk_load(ring + (size_t)p_st * TILE, a.w + ((size_t)tile_id * a.num_kb + kb0 + p_kb) * TILE, TILE, &full_bar[p_st]);
    if (++p_kb == nkb) { p_kb = 0; ++p_it; }
    if (++p_st == S) p_st = 0;
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], kQvThreads / 32); }
    *abort_flag = 0;
    fence_barrier_init();
    // weights do not depend on the kernel in front of this one: the first tiles are requested before the dependency wait
    for (int s = 0; s < S && p_it < it1; ++s) issue_next();
  }
  pdl_wait();
  pdl_trigger();

  const int row = warp * 16 + (lane & 15), jh = lane >> 4;   // row inside the tile; chunks 2 jh and 2 jh + 1
  int st = 0; uint32_t ph = 0;
  int cur_ks = -1;
  bool ok = true;
  for (int it = it0; it < it1; ++it) {       // no early exit: every warp takes the same block-wide steps even after a failed wait
    int tile_id, kb0, nkb;
    item_range(it, tile_id, kb0, nkb);
    const int ks = it / a.row_tiles;
    if (ks != cur_ks) {
      // ---- activations of this K range -> int8 + scale + sum per 32 values (4 lanes x 8 values hold one block)
      cur_ks = ks;
      __syncthreads();                                       // every warp is done with the old tables (and sees the barrier initialisation)
      for (int q_it = threadIdx.x; q_it < nkb * M * 32; q_it += kQvThreads) {
        const int v = q_it & 31, m = (q_it >> 5) % M, kbi = (q_it >> 5) / M;
        const uint4 raw = *reinterpret_cast<const uint4*>(a.x + (size_t)m * a.ldx + (size_t)(kb0 + kbi) * 256 + v * 8);
        const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float f[8];
        float amax = 0.f;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float2 t = __bfloat1622float2(hv[u]);
          f[2 * u] = t.x; f[2 * u + 1] = t.y;
          amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float d = amax * (1.0f / 127.0f);
        const float inv = d > 0.f ? 1.0f / d : 0.f;
        int q[8], qsum = 0;
#pragma unroll
        for (int u = 0; u < 8; ++u) { q[u] = max(-127, min(127, __float2int_rn(f[u] * inv))); qsum += q[u]; }
        qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
        qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
        uint2 pk;
        pk.x = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
        pk.y = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
        *reinterpret_cast<uint2*>(aq + ((size_t)(kbi * M + m) * 256 + v * 8)) = pk;
        if ((v & 3) == 0) { ad[(kbi * M + m) * 8 + (v >> 2)] = d; as[(kbi * M + m) * 8 + (v >> 2)] = d * (float)qsum; }
      }
      __syncthreads();
    }

    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    for (int kbi = 0; kbi < nkb; ++kbi) {
      if (ok && !mbar_wait(&full_bar[st], ph, abort_flag, a.status, 1300, st)) ok = false;
      ok = __all_sync(0xffffffffu, ok);                      // warp-uniform
      if (!ok) continue;
      const uint8_t* t = ring + (size_t)st * TILE;
      // this lane's bytes of the tile: header + two 32-byte nibble chunks (Q4_K) / four 32-byte blocks + their four scales (Q8_0)
      uint4 hd, qw[8];
      if (TYPE == 0) {
        const uint8_t* b = t + row * 144;
        hd = *reinterpret_cast<const uint4*>(b);
#pragma unroll
        for (int u = 0; u < 4; ++u) qw[u] = *reinterpret_cast<const uint4*>(b + 16 + 64 * jh + 16 * u);
      } else {
        const uint8_t* b = t + row * kQ80RowBytes + 128 * jh;
#pragma unroll
        for (int u = 0; u < 8; ++u) qw[u] = *reinterpret_cast<const uint4*>(b + 16 * u);
        const uint2 sc = *reinterpret_cast<const uint2*>(t + row * kQ80RowBytes + 256 + 8 * jh);
        hd.x = sc.x; hd.y = sc.y;
      }
      // Q4_K: the 6-bit scales / offsets of this lane's four sub-blocks (4 jh .. 4 jh + 3) as bytes of two words, unpacked with
      // word-wide masks (sub-blocks 0..3: six bits straight from bytes 0..3 / 4..7; 4..7: low 4 bits in bytes 8..11, high 2 bits
      // on top of bytes 0..7), both forms computed and one selected: no divergence between the two half warps.
      uint32_t scw = 0, mnw = 0;
      float dq = 0.f, dminq = 0.f;
      if (TYPE == 0) {
        const __half2 dd = *reinterpret_cast<const __half2*>(&hd.x);
        dq = __low2float(dd); dminq = __high2float(dd);
        const uint32_t s0 = hd.y, s1 = hd.z, s2 = hd.w;
        const uint32_t sc_lo = s0 & 0x3f3f3f3fu, mn_lo = s1 & 0x3f3f3f3fu;
        const uint32_t sc_hi = (s2 & 0x0f0f0f0fu) | ((s0 >> 2) & 0x30303030u), mn_hi = ((s2 >> 4) & 0x0f0f0f0fu) | ((s1 >> 2) & 0x30303030u);
        scw = jh ? sc_hi : sc_lo; mnw = jh ? mn_hi : mn_lo;
      }
#pragma unroll
      for (int c = 0; c < 2; ++c) {                          // the two chunks of this lane
        const int j = 2 * jh + c;
        float s_lo, s_hi, o_lo = 0.f, o_hi = 0.f;
        uint32_t wlo[8], whi[8];
        if (TYPE == 0) {
          s_lo = dq * (float)byte_of(scw, 2 * c); s_hi = dq * (float)byte_of(scw, 2 * c + 1);
          o_lo = dminq * (float)byte_of(mnw, 2 * c); o_hi = dminq * (float)byte_of(mnw, 2 * c + 1);
          const uint32_t* qq = reinterpret_cast<const uint32_t*>(&qw[2 * c]);
#pragma unroll
          for (int i = 0; i < 8; ++i) { wlo[i] = qq[i] & 0x0f0f0f0fu; whi[i] = (qq[i] >> 4) & 0x0f0f0f0fu; }
        } else {
          const uint32_t sw = c == 0 ? hd.x : hd.y;
          const __half2 dd = *reinterpret_cast<const __half2*>(&sw);
          s_lo = __low2float(dd); s_hi = __high2float(dd);
          const uint32_t* qq = reinterpret_cast<const uint32_t*>(&qw[4 * c]);
#pragma unroll
          for (int i = 0; i < 8; ++i) { wlo[i] = qq[i]; whi[i] = qq[8 + i]; }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const uint4* ap = reinterpret_cast<const uint4*>(aq + ((size_t)(kbi * M + m) * 256 + 64 * j));
          const uint4 a0 = ap[0], a1 = ap[1], a2 = ap[2], a3 = ap[3];
          const uint32_t al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
          const uint32_t ah[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
          const float2 d8 = *reinterpret_cast<const float2*>(ad + (kbi * M + m) * 8 + 2 * j);      // block scales of the two sub-blocks
          int sl = 0, sh = 0;
#pragma unroll
          for (int i = 0; i < 8; ++i) { sl = dp4a_s(wlo[i], al[i], sl); sh = dp4a_s(whi[i], ah[i], sh); }
          float v = s_lo * d8.x * (float)sl + s_hi * d8.y * (float)sh;
          if (TYPE == 0) {
            const float2 t8 = *reinterpret_cast<const float2*>(as + (kbi * M + m) * 8 + 2 * j);    // block sums
            v -= o_lo * t8.x + o_hi * t8.y;
          }
          acc[m] += v;
        }
      }
      // Every word loaded from the slot has now been an operand of a dp4a, i.e. the shared-memory reads of this lane have returned.
      // (A release issued right behind the load instructions let the refill land under reads still in flight: seen as wrong
      // sums in a few lanes.)  Hand the slot back, and let the elected thread refill it with the next tile of the stream.
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[st]);
      if (threadIdx.x == 0 && p_it < it1) {
        if (mbar_wait(&empty_bar[st], ph, abort_flag, a.status, 1301, st)) issue_next();
        else ok = false;
      }
      if (++st == S) { st = 0; ph ^= 1; }
    }
    if (!ok) continue;

    // ---- a row's two half sums meet in lanes l and l + 16; lanes 0..15 store 16 consecutive output features
    const size_t slab = (size_t)ks * (size_t)a.partial_stride;
    const int n = tile_id * 128 + row;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float v = acc[m] + __shfl_xor_sync(0xffffffffu, acc[m], 16);
      if (jh == 0 && n < a.n_out) {
        if (a.bias != nullptr && ks == 0) v += a.bias[n];
        const size_t off = slab + (size_t)m * a.ldo + n;
        if (a.peer_bcast > 0) { for (int p = 0; p < a.peer_bcast; ++p) reinterpret_cast<float*>(a.peer_out[p])[off] = v; }
        else a.out[off] = v;
      }
    }
  }
  if (*abort_flag) {                                       // copies may still be landing: bounded grace period
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  if (a.signal_n > 0) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      if (atomicAdd(a.done_ctr, 1u) == gridDim.x - 1) {
        *a.done_ctr = 0;
        uint32_t e = *a.epoch_ptr;
        if (a.epoch_self_tick) { e += 1; *a.epoch_ptr = e; }
        for (int p = 0; p < a.signal_n; ++p) st_release_sys(a.signal_flags[p], e);
      }
    }
  }
}

}  // namespace gb

using namespace gb;

// Peer-store tail of gb_qgemv (all optional; mirrors the tensor-parallel fields of the GEMM's extras).
struct QGemvPeer {
  void* peer_out[kMaxRanks];
  uint32_t* signal_flags[kMaxRanks];
  int peer_bcast, signal_n;
  unsigned* done_ctr;
  uint32_t* epoch_ptr;
  int epoch_self_tick, pad;
};

// Shared memory of one CTA: a ring of weight tiles + the quantised activations of its K range.  Two CTAs share an SM.
constexpr int kQvSmemBudget = 110 * 1024;         // two CTAs per SM (three measured no faster: the kernel is not short of warps)
static int qgemv_stages(int type) { return type == 12 ? 4 : 2; }                 // 4 x 18 KB (Q4_K) / 2 x 34 KB (Q8_0)
static int qgemv_tile_bytes(int type) { return type == 12 ? kQ4KTileBytes : kQ80TileBytes; }
// Largest K range (in 256-column tiles) whose quantised activations fit beside the ring for `m` tokens.
static int qgemv_max_kb(int m, int type) {
  const int left = kQvSmemBudget - 1024 - qgemv_stages(type) * qgemv_tile_bytes(type);
  const int by_act = left / (m * (256 + 64));
  return by_act;
}

GB_API int gb_qgemv_supported(int ggml_type, int n_out, int k, int m) {
  return ((ggml_type == 12 || ggml_type == 8) && m >= 1 && m <= 4 && k > 0 && k % 256 == 0 && n_out > 0) ? 1 : 0;
}

// Smallest split count (>= want) whose K range fits shared memory and leaves no split empty; 0 if none.
GB_API int gb_qgemv_splits(int ggml_type, int k, int m, int want) {
  const int num_kb = k / 256;
  if (m < 1 || m > 4 || num_kb < 1 || (ggml_type != 12 && ggml_type != 8)) return 0;
  for (int sp = want < 1 ? 1 : want; sp <= num_kb; ++sp) {
    const int per = (num_kb + sp - 1) / sp;
    if ((num_kb + per - 1) / per != sp) continue;
    if (per <= qgemv_max_kb(m, ggml_type)) return sp;
  }
  return 0;
}

// w: tiled Q4_K (ggml_type 12) or Q8_0 (8) weights for ceil(n_out / 128) row tiles x k / 256 K tiles.  x bf16 [m, ldx], m <= 4.
// out fp32: slab s (s < splits) at out + s * partial_stride holds [m][ldo] partial sums over the K range of split s.
GB_API int gb_qgemv(const void* w, int ggml_type, const void* x, int ldx, float* out, int ldo, long partial_stride, const float* bias,
                    int n_out, int k, int m, int splits, const QGemvPeer* peer, void* status, cudaStream_t stream) {
  if (!gb_qgemv_supported(ggml_type, n_out, k, m)) return fail("qgemv: unsupported type / shape%s (type %ld, m %ld)", "", ggml_type, m);
  if (ldx % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail("qgemv: operands must be 16-byte aligned%s");
  const int num_kb = k / 256;
  if (splits < 1) splits = 1;
  const int kb_per = (num_kb + splits - 1) / splits;
  if ((num_kb + kb_per - 1) / kb_per != splits) return fail("qgemv: a K split would be empty%s");
  if (kb_per > qgemv_max_kb(m, ggml_type)) return fail("qgemv: K range per split too long for shared memory%s (%ld tiles)", "", kb_per);
  if (splits > 1 && partial_stride < (long)m * ldo) return fail("qgemv: partial slabs overlap%s");
  QGemvArgs a;
  memset(&a, 0, sizeof(a));
  a.w = (const uint8_t*)w; a.x = (const __nv_bfloat16*)x; a.ldx = ldx; a.out = out; a.ldo = ldo; a.partial_stride = partial_stride; a.bias = bias;
  a.n_out = n_out; a.row_tiles = (n_out + 127) / 128; a.num_kb = num_kb; a.kb_per = kb_per; a.splits = splits;
  if (peer != nullptr) {
    for (int i = 0; i < kMaxRanks; ++i) { a.peer_out[i] = peer->peer_out[i]; a.signal_flags[i] = peer->signal_flags[i]; }
    a.peer_bcast = peer->peer_bcast; a.signal_n = peer->signal_n; a.done_ctr = peer->done_ctr; a.epoch_ptr = peer->epoch_ptr;
    a.epoch_self_tick = peer->epoch_self_tick;
  }
  a.stages = qgemv_stages(ggml_type); a.status = (KernelStatus*)status;
  const size_t act = (size_t)kb_per * m * (256 + 64);
  const size_t smem = 128 + (size_t)a.stages * qgemv_tile_bytes(ggml_type) + 128 + act;
  int grid = a.row_tiles * splits;
  const int per_sm = 2;
  if (grid > per_sm * sm_count()) grid = per_sm * sm_count();      // persistent: the resident CTAs walk the items
  const int t = ggml_type == 12 ? 0 : 1;
#define GB_QV(TV, MV)                                                                                              \
  {                                                                                                                 \
    static bool attr = false;                                                                                       \
    if (!attr) { GB_CUDA_OK(cudaFuncSetAttribute(qgemv_kernel<TV, MV>, cudaFuncAttributeMaxDynamicSharedMemorySize, kQvSmemBudget)); attr = true; } \
    launch_k(qgemv_kernel<TV, MV>, grid, kQvThreads, smem, stream, a);                                              \
  }
  if (t == 0) { if (m == 1) GB_QV(0, 1) else if (m == 2) GB_QV(0, 2) else if (m == 3) GB_QV(0, 3) else GB_QV(0, 4) }
  else { if (m == 1) GB_QV(1, 1) else if (m == 2) GB_QV(1, 2) else if (m == 3) GB_QV(1, 3) else GB_QV(1, 4) }
#undef GB_QV
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}
