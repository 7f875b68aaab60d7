// NVLink fabric: symmetric heap management (CUDA IPC), and the stand-alone collectives written as
// kernels over peer memory: barrier, one-shot and two-shot all-reduce (sum, fixed rank order so every
// GPU computes bit-identical results), all-gather, reduce-scatter, all-to-all, arg-max all-reduce, and
// the expert-parallel dispatch (gather + MXFP8 quantise + store into the owning GPU's expert buffer).
//
// Replaces the reference's transports and collectives: common/comm.h (TCP mesh + POSIX shm,
// comm_allreduce_sum_f32:543, allgather:583, barrier:552), a64fx/utofu-tests/tp_allreduce.h
// (recursive-doubling all-reduce for SUM / MAX / ARGMAX:222-349) and the all-to-all dispatch of
// a64fx/utofu-tests/moe_dispatch_bench.c.  On NVSwitch every peer is one hop away, so the latency-bound
// collectives are single-step pushes; the bandwidth-bound one is reduce-scatter + all-gather.
//
// Protocol: every collective call has an epoch (a device-resident counter, so a captured CUDA graph can be
// replayed).  Data is stored into the peers' heaps, then a flag word per (source rank[, chunk]) is set to the
// epoch with release semantics at system scope; consumers poll with acquire loads under a time budget.
//
// Reuse of receive slots.  A flag proves that a peer has PUSHED call e, not that it has finished READING what it received
// in call e.  The collectives whose result leaves the slots inside the same kernel (one-shot all-reduce, arg-max all-reduce)
// therefore alternate between two slot sets by epoch parity: a rank can only start call e + 2 (the next writer of the
// parity-e set) after its own call e + 1 completed, which needed every peer's flag of call e + 1, which a peer raises only
// after its kernel of call e (and all its reads) ended.  The push exchange hands its receive buffer to later kernels of the
// caller, so its parity cannot alternate; its optional entry handshake (`ack`) makes every rank wait until all peers have
// ENTERED the same call (stream order puts their readers of the previous call before that) before the first store.
#include "fabric.cuh"
#include "../kernels/host_common.h"

namespace gb {

struct alignas(16) Vec16 { uint32_t x, y, z, w; };

__device__ __forceinline__ float4 bf16x4_to_f4(uint2 v) {
  const __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&v.x), b = *reinterpret_cast<__nv_bfloat162*>(&v.y);
  const float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
  return make_float4(fa.x, fa.y, fb.x, fb.y);
}

// ------------------------------------------------------------------------------------------ barrier
// flags: uint32 [world] in every heap at flags_off.  One thread per peer.
__global__ void fabric_barrier_kernel(PeerTable pt, size_t flags_off, uint32_t* epoch_ctr, KernelStatus* st) {
  pdl_wait();
  pdl_trigger();
  const uint32_t epoch = *epoch_ctr + 1;
  const int p = threadIdx.x;
  if (p < pt.world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>((char*)pt.base[p] + flags_off) + pt.rank, epoch);
    wait_flag_ge(reinterpret_cast<uint32_t*>((char*)pt.base[pt.rank] + flags_off) + p, epoch, st, 700, p);
  }
  __syncthreads();
  if (threadIdx.x == 0) *epoch_ctr = epoch;
}

// ------------------------------------------------------------------------------------------ one-shot all-reduce
// Each CTA owns one chunk of the vector: it pushes its chunk into slot[rank] of every peer, raises the
// chunk's flag there, waits for the same chunk from every peer and sums the slots in rank order.
//   slots: [world][max_elems] elements of T at data_off;  flags: uint32 [world][chunks] at flags_off.
template <typename T>
__global__ void __launch_bounds__(256)
allreduce_oneshot_kernel(PeerTable pt, size_t data_off, size_t flags_off, const T* __restrict__ in, T* __restrict__ out,
                         long n, long max_elems, uint32_t* epoch_ctr, unsigned* done_ctr, KernelStatus* st, size_t parity_stride) {
  pdl_wait();
  pdl_trigger();
  constexpr int EPV = 16 / sizeof(T);
  const uint32_t epoch = *epoch_ctr + 1;
  data_off += (size_t)(epoch & 1u) * parity_stride;          // two slot sets, alternating by call
  const int chunks = gridDim.x, c = blockIdx.x;
  const long nvec = (n + EPV - 1) / EPV;
  const long per = (nvec + chunks - 1) / chunks;
  const long v0 = c * per, v1 = min(nvec, v0 + per);
  for (int p = 0; p < pt.world; ++p) {
    Vec16* dst = reinterpret_cast<Vec16*>((char*)pt.base[p] + data_off) + (size_t)pt.rank * (max_elems / EPV);
    for (long v = v0 + threadIdx.x; v < v1; v += blockDim.x) dst[v] = reinterpret_cast<const Vec16*>(in)[v];
  }
  __syncthreads();
  if ((int)threadIdx.x < pt.world) {
    const int p = threadIdx.x;
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>((char*)pt.base[p] + flags_off) + (size_t)pt.rank * chunks + c, epoch);
    wait_flag_ge(reinterpret_cast<uint32_t*>((char*)pt.base[pt.rank] + flags_off) + (size_t)p * chunks + c, epoch, st, 710, p);
  }
  __syncthreads();
  const Vec16* slots = reinterpret_cast<const Vec16*>((char*)pt.base[pt.rank] + data_off);
  for (long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int p = 0; p < pt.world; ++p) {
      const Vec16 x = slots[(size_t)p * (max_elems / EPV) + v];
      if (sizeof(T) == 4) {
        acc[0] += __uint_as_float(x.x); acc[1] += __uint_as_float(x.y); acc[2] += __uint_as_float(x.z); acc[3] += __uint_as_float(x.w);
      } else {
        const float4 a = bf16x4_to_f4(make_uint2(x.x, x.y)), b = bf16x4_to_f4(make_uint2(x.z, x.w));
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w; acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      }
    }
    Vec16 o;
    if (sizeof(T) == 4) { o.x = __float_as_uint(acc[0]); o.y = __float_as_uint(acc[1]); o.z = __float_as_uint(acc[2]); o.w = __float_as_uint(acc[3]); }
    else { o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]); o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]); }
    reinterpret_cast<Vec16*>(out)[v] = o;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(done_ctr, 1u) == gridDim.x - 1) { *done_ctr = 0; *epoch_ctr = epoch; }
  }
}

// ------------------------------------------------------------------------------------------ two-shot all-reduce
// in_off / out_off: buffers of n elements inside every heap.  Rank r reduces slice r (reading its peers'
// inputs through NVLink once their "ready" flag of the chunk is up), pushes the reduced slice into every
// peer's output and raises "done"; every CTA leaves after the done flags of its chunk arrived from all ranks.
//   flags: uint32 [2][world][chunks]  (0 = ready, 1 = done)
template <typename T, int MW>      // MW: upper bound of the world size this instance is compiled for (sizes its register arrays)
__global__ void __launch_bounds__(256)
allreduce_twoshot_kernel(PeerTable pt, size_t in_off, size_t out_off, size_t flags_off, long n, uint32_t* epoch_ctr,
                         unsigned* done_ctr, KernelStatus* st) {
  pdl_wait();
  pdl_trigger();
  constexpr int EPV = 16 / sizeof(T);
  const uint32_t epoch = *epoch_ctr + 1;
  const int chunks = gridDim.x, c = blockIdx.x, W = pt.world;
  const long nvec = n / EPV;                       // n is a multiple of EPV * world
  const long slice = nvec / W;
  const long per = (slice + chunks - 1) / chunks;
  uint32_t* my_flags = reinterpret_cast<uint32_t*>((char*)pt.base[pt.rank] + flags_off);
  // "ready": the caller's stream already ordered the producer of `in` before this kernel
  if ((int)threadIdx.x < W) {
    const int p = threadIdx.x;
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>((char*)pt.base[p] + flags_off) + (size_t)pt.rank * chunks + c, epoch);
    wait_flag_ge(my_flags + (size_t)p * chunks + c, epoch, st, 720, p);
  }
  __syncthreads();
  const long s0 = (long)pt.rank * slice + c * per, s1 = min((long)(pt.rank + 1) * slice, s0 + per);
  // Four vectors per thread and step: all their peer loads (W each) are requested before the first sum, so that a CTA keeps
  // U * W * 256 * 16 bytes in flight over the links (one vector per thread left NVLink at a quarter of its bandwidth).
  constexpr int U = MW <= 4 ? 4 : 2;
  for (long vb = s0; vb < s1; vb += (long)U * blockDim.x) {
    Vec16 x[U][MW];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long v = vb + (long)u * blockDim.x + threadIdx.x;
#pragma unroll
      for (int p = 0; p < MW; ++p)
        if (p < W && v < s1) x[u][p] = reinterpret_cast<const Vec16*>((char*)pt.base[p] + in_off)[v];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long v = vb + (long)u * blockDim.x + threadIdx.x;
      if (v >= s1) continue;
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
      for (int p = 0; p < MW; ++p) {
        if (p >= W) continue;
        if (sizeof(T) == 4) {
          acc[0] += __uint_as_float(x[u][p].x); acc[1] += __uint_as_float(x[u][p].y); acc[2] += __uint_as_float(x[u][p].z); acc[3] += __uint_as_float(x[u][p].w);
        } else {
          const float4 a = bf16x4_to_f4(make_uint2(x[u][p].x, x[u][p].y)), b = bf16x4_to_f4(make_uint2(x[u][p].z, x[u][p].w));
          acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w; acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
        }
      }
      Vec16 o;
      if (sizeof(T) == 4) { o.x = __float_as_uint(acc[0]); o.y = __float_as_uint(acc[1]); o.z = __float_as_uint(acc[2]); o.w = __float_as_uint(acc[3]); }
      else { o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]); o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]); }
      for (int p = 0; p < W; ++p) reinterpret_cast<Vec16*>((char*)pt.base[p] + out_off)[v] = o;
    }
  }
  __syncthreads();
  if ((int)threadIdx.x < W) {
    const int p = threadIdx.x;
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>((char*)pt.base[p] + flags_off) + (size_t)(W + pt.rank) * chunks + c, epoch);
    wait_flag_ge(my_flags + (size_t)(W + p) * chunks + c, epoch, st, 721, p);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(done_ctr, 1u) == gridDim.x - 1) { *done_ctr = 0; *epoch_ctr = epoch; }
  }
}

// ------------------------------------------------------------------------------------------ all-gather / all-to-all (push)
// Rank r stores `bytes_per_dst` bytes starting at in + dst_stride_in * p into peer p's buffer at
// out_off + rank * bytes_per_dst.  dst_stride_in = 0 gives an all-gather, = bytes_per_dst an all-to-all.
__global__ void __launch_bounds__(256)
push_exchange_kernel(PeerTable pt, size_t out_off, size_t flags_off, const char* __restrict__ in, size_t bytes_per_dst,
                     size_t dst_stride_in, uint32_t* epoch_ctr, unsigned* done_ctr, KernelStatus* st, size_t ack_off) {
  pdl_wait();
  pdl_trigger();
  const uint32_t epoch = *epoch_ctr + 1;
  const int chunks = gridDim.x, c = blockIdx.x;
  if (ack_off != 0) {
    // entry handshake: nobody stores into a peer before that peer has entered this call (its readers of the previous call's
    // buffer precede this kernel in its stream).  CTA 0 announces, every CTA waits on the local copies.
    if ((int)threadIdx.x < pt.world) {
      const int p = threadIdx.x;
      if (c == 0) st_release_sys(reinterpret_cast<uint32_t*>((char*)pt.base[p] + ack_off) + pt.rank, epoch);
      wait_flag_ge(reinterpret_cast<uint32_t*>((char*)pt.base[pt.rank] + ack_off) + p, epoch, st, 731, p);
    }
    __syncthreads();
  }
  const size_t nvec = bytes_per_dst / 16, per = (nvec + chunks - 1) / chunks;
  const size_t v0 = c * per, v1 = min(nvec, v0 + per);
  for (int p = 0; p < pt.world; ++p) {
    const Vec16* src = reinterpret_cast<const Vec16*>(in + dst_stride_in * p);
    Vec16* dst = reinterpret_cast<Vec16*>((char*)pt.base[p] + out_off + (size_t)pt.rank * bytes_per_dst);
    for (size_t v = v0 + threadIdx.x; v < v1; v += blockDim.x) dst[v] = src[v];
  }
  __syncthreads();
  if ((int)threadIdx.x < pt.world) {
    const int p = threadIdx.x;
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>((char*)pt.base[p] + flags_off) + (size_t)pt.rank * chunks + c, epoch);
    wait_flag_ge(reinterpret_cast<uint32_t*>((char*)pt.base[pt.rank] + flags_off) + (size_t)p * chunks + c, epoch, st, 730, p);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(done_ctr, 1u) == gridDim.x - 1) { *done_ctr = 0; *epoch_ctr = epoch; }
  }
}

// ------------------------------------------------------------------------------------------ arg-max all-reduce
// Every rank contributes (value, index) per row; all ranks end with the same winner (ties: lower index).
// slots: [world][rows] of {float, int} at data_off.  One CTA.
__global__ void __launch_bounds__(256)
argmax_allreduce_kernel(PeerTable pt, size_t data_off, size_t flags_off, const float* __restrict__ val, const int* __restrict__ idx,
                        int* __restrict__ out_idx, float* __restrict__ out_val, int rows, int max_rows, uint32_t* epoch_ctr, KernelStatus* st,
                        size_t parity_stride) {
  pdl_wait();
  pdl_trigger();
  const uint32_t epoch = *epoch_ctr + 1;
  data_off += (size_t)(epoch & 1u) * parity_stride;
  for (int p = 0; p < pt.world; ++p) {
    int2* dst = reinterpret_cast<int2*>((char*)pt.base[p] + data_off) + (size_t)pt.rank * max_rows;
    for (int r = threadIdx.x; r < rows; r += blockDim.x) dst[r] = make_int2(__float_as_int(val[r]), idx[r]);
  }
  __syncthreads();
  if ((int)threadIdx.x < pt.world) {
    const int p = threadIdx.x;
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>((char*)pt.base[p] + flags_off) + pt.rank, epoch);
    wait_flag_ge(reinterpret_cast<uint32_t*>((char*)pt.base[pt.rank] + flags_off) + p, epoch, st, 740, p);
  }
  __syncthreads();
  const int2* slots = reinterpret_cast<const int2*>((char*)pt.base[pt.rank] + data_off);
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int p = 0; p < pt.world; ++p) {
      const int2 e = slots[(size_t)p * max_rows + r];
      const float v = __int_as_float(e.x);
      if (v > bv || (v == bv && e.y < bi)) { bv = v; bi = e.y; }
    }
    out_idx[r] = bi;
    if (out_val != nullptr) out_val[r] = bv;
  }
  __syncthreads();
  if (threadIdx.x == 0) *epoch_ctr = epoch;
}

// ------------------------------------------------------------------------------------------ EP dispatch
// For every row r of the sender's plan (regions = destination ranks, region_rows rows each): gather the
// token's hidden row, quantise to MXFP8 (or keep bf16) and store it into the destination rank's receive
// buffer at row  rank * region_rows + (r % region_rows); scales go to the matching atom of the receiver.
// The per-(destination, local expert) segment table goes to the receiver's meta arrays.  When the last
// CTA has finished, flag[rank] on every peer is set to the epoch.
struct EpDispatchArgs {
  const __nv_bfloat16* h; int ld_h; int hidden;
  const int* row_token;        // [world * region_rows]
  const int* seg_start;        // [E] rows in plan numbering
  const int* seg_count;        // [E]
  int region_rows; int experts_per_rank;
  size_t x_off;                // receive buffer (fp8 bytes or bf16) [world * region_rows, hidden]
  size_t sf_off;               // scale atoms of the receive buffer (mx only)
  size_t meta_off;             // int32 [2][world * experts_per_rank]: starts then counts
  size_t flags_off;            // uint32 [world]
  int mx; int sf32;
  uint32_t* epoch_ctr; unsigned* done_ctr; KernelStatus* st;
  // tokens that are already MXFP8 (the RMSNorm in front of the MoE block quantised them): rows and scale words are copied as
  // 16-byte / 4-byte stores instead of being quantised again per (token, expert) pair
  const uint8_t* hq; const uint8_t* hsf; int in_sf32;
};

__device__ __forceinline__ int ep_e8m0(float amax) {
  const float s = amax * (1.0f / 448.0f);
  const uint32_t bits = __float_as_uint(s);
  int e = (int)((bits >> 23) & 0xff);
  if (bits & 0x7fffffu) e += 1;
  return amax == 0.0f ? 127 : max(1, min(e, 254));
}

__global__ void __launch_bounds__(256)
ep_dispatch_kernel(PeerTable pt, EpDispatchArgs a) {
  pdl_wait();
  pdl_trigger();
  const uint32_t epoch = *a.epoch_ctr;          // the plan kernel advanced the epoch for this layer
  const int vec_per_row = a.hidden >> 3;
  const long total_rows = (long)pt.world * a.region_rows;
  const int lane = threadIdx.x & 31;
  const long warp0 = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long n_warps = ((long)gridDim.x * blockDim.x) >> 5;
  // one warp per plan row; padding rows (token < 0) cost one load
  for (long r = warp0; r < total_rows; r += n_warps) {
    const int tok = a.row_token[r];
    if (tok < 0) continue;
    const int dst = (int)(r / a.region_rows);
    const long drow = (long)pt.rank * a.region_rows + (r % a.region_rows);
    if (a.hq != nullptr) {
      const int katoms = a.hidden >> 7;
      const uint4* ip = reinterpret_cast<const uint4*>(a.hq + (size_t)tok * a.hidden);
      uint4* op = reinterpret_cast<uint4*>((uint8_t*)pt.base[dst] + a.x_off + (size_t)drow * a.hidden);
      for (int v0 = 0; v0 < (a.hidden >> 4); v0 += 128) {
        uint4 buf[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { const int vi = v0 + lane + 32 * i; if (vi < (a.hidden >> 4)) buf[i] = ip[vi]; }
#pragma unroll
        for (int i = 0; i < 4; ++i) { const int vi = v0 + lane + 32 * i; if (vi < (a.hidden >> 4)) op[vi] = buf[i]; }
      }
      uint8_t* sfb = (uint8_t*)pt.base[dst] + a.sf_off;
      for (int ka = lane; ka < katoms; ka += 32) {
        const size_t si = a.in_sf32 ? ((size_t)(tok >> 5) * katoms + ka) * 512 + (tok & 31) * 16
                                    : ((size_t)(tok >> 7) * katoms + ka) * 512 + (tok & 31) * 16 + ((tok >> 5) & 3) * 4;
        const size_t so = a.sf32 ? ((size_t)(drow >> 5) * katoms + ka) * 512 + (drow & 31) * 16
                                 : ((size_t)(drow >> 7) * katoms + ka) * 512 + (drow & 31) * 16 + ((drow >> 5) & 3) * 4;
        *reinterpret_cast<uint32_t*>(sfb + so) = *reinterpret_cast<const uint32_t*>(a.hsf + si);
      }
      continue;
    }
    for (int vi = lane; vi < vec_per_row; vi += 32) {
      const uint4 raw = *reinterpret_cast<const uint4*>(a.h + (size_t)tok * a.ld_h + vi * 8);
      if (a.mx) {
        float v[8];
        const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(hh[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const int e = ep_e8m0(amax);
        const float inv = __uint_as_float((uint32_t)(254 - e) << 23);
        uint8_t q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { __nv_fp8_e4m3 f(v[j] * inv); q[j] = *reinterpret_cast<uint8_t*>(&f); }
        uint8_t* xb = (uint8_t*)pt.base[dst] + a.x_off;
        *reinterpret_cast<uint2*>(xb + (size_t)drow * a.hidden + vi * 8) = *reinterpret_cast<uint2*>(q);
        if ((vi & 3) == 0) {
          uint8_t* sfb = (uint8_t*)pt.base[dst] + a.sf_off;
          const int blk = vi >> 2, katoms = a.hidden >> 7;
          if (a.sf32) sfb[((size_t)(drow >> 5) * katoms + (blk >> 2)) * 512 + (drow & 31) * 16 + (blk & 3)] = (uint8_t)e;
          else sfb[((size_t)(drow >> 7) * katoms + (blk >> 2)) * 512 + (drow & 31) * 16 + ((drow >> 5) & 3) * 4 + (blk & 3)] = (uint8_t)e;
        }
      } else {
        __nv_bfloat16* xb = reinterpret_cast<__nv_bfloat16*>((char*)pt.base[dst] + a.x_off);
        *reinterpret_cast<uint4*>(xb + (size_t)drow * a.hidden + vi * 8) = raw;
      }
    }
  }
  // segment table: entry (dst, e_local) lands at index rank * experts_per_rank + e_local on dst
  const int n_exp = pt.world * a.experts_per_rank;
  for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < n_exp; e += gridDim.x * blockDim.x) {
    const int dst = e / a.experts_per_rank, el = e % a.experts_per_rank;
    int* meta = reinterpret_cast<int*>((char*)pt.base[dst] + a.meta_off);
    const int g = pt.rank * a.experts_per_rank + el;
    meta[g] = pt.rank * a.region_rows + (a.seg_start[e] - dst * a.region_rows);
    meta[n_exp + g] = a.seg_count[e];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(a.done_ctr, 1u) == gridDim.x - 1) {
      *a.done_ctr = 0;
      for (int p = 0; p < pt.world; ++p)
        st_release_sys(reinterpret_cast<uint32_t*>((char*)pt.base[p] + a.flags_off) + pt.rank, epoch);
    }
  }
}

// Advances a device-resident epoch counter (one thread); used where no other kernel can carry the tick.
__global__ void epoch_tick_kernel(uint32_t* ctr) {
  pdl_wait();
  pdl_trigger(); *ctr = *ctr + 1; }

}  // namespace gb

using namespace gb;

// ------------------------------------------------------------------------------------------ host API
GB_API int gb_fabric_alloc(size_t bytes, void** out) {
  GB_CUDA_OK(cudaMalloc(out, bytes));
  GB_CUDA_OK(cudaMemset(*out, 0, bytes));
  GB_CUDA_OK(cudaDeviceSynchronize());
  return 0;
}
GB_API int gb_fabric_free(void* p) { GB_CUDA_OK(cudaFree(p)); return 0; }
GB_API int gb_ipc_get(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  GB_CUDA_OK(cudaIpcGetMemHandle(&h, p));
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
GB_API int gb_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  GB_CUDA_OK(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
GB_API int gb_ipc_close(void* p) { GB_CUDA_OK(cudaIpcCloseMemHandle(p)); return 0; }

static PeerTable make_table(void* const* bases, int world, int rank) {
  PeerTable pt;
  memset(&pt, 0, sizeof(pt));
  for (int i = 0; i < world && i < kMaxRanks; ++i) pt.base[i] = bases[i];
  pt.world = world; pt.rank = rank;
  return pt;
}

GB_API int gb_fabric_barrier(void* const* bases, int world, int rank, size_t flags_off, void* epoch_ctr, void* status, cudaStream_t stream) {
  if (world > kMaxRanks) return fail("fabric: world > 8%s");
  launch_k(fabric_barrier_kernel, 1, 32, 0, stream, make_table(bases, world, rank), flags_off, (uint32_t*)epoch_ctr, (KernelStatus*)status);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

// dtype: 0 = f32, 1 = bf16.  n elements (multiple of 16 bytes), slots hold max_elems each, flags [world][chunks].
// The slot area holds two sets of [world][max_elems] elements, `parity_stride` bytes apart (0 = a single set: the caller then has
// to keep consecutive calls apart itself).
GB_API int gb_allreduce_oneshot(void* const* bases, int world, int rank, size_t data_off, size_t flags_off, const void* in, void* out,
                                long n, long max_elems, int dtype, int chunks, void* epoch_ctr, void* done_ctr, void* status,
                                size_t parity_stride, cudaStream_t stream) {
  if (world > kMaxRanks) return fail("fabric: world > 8%s");
  const int esz = dtype == 0 ? 4 : 2;
  if ((n * esz) % 16 || n > max_elems || (max_elems * esz) % 16) return fail("allreduce_oneshot: size must be a multiple of 16 bytes and fit the slot%s");
  PeerTable pt = make_table(bases, world, rank);
  if (dtype == 0) launch_k(allreduce_oneshot_kernel<float>, chunks, 256, 0, stream, pt, data_off, flags_off, (const float*)in, (float*)out, n, max_elems, (uint32_t*)epoch_ctr, (unsigned*)done_ctr, (KernelStatus*)status, parity_stride);
  else launch_k(allreduce_oneshot_kernel<__nv_bfloat16>, chunks, 256, 0, stream, pt, data_off, flags_off, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, n, max_elems, (uint32_t*)epoch_ctr, (unsigned*)done_ctr, (KernelStatus*)status, parity_stride);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_allreduce_twoshot(void* const* bases, int world, int rank, size_t in_off, size_t out_off, size_t flags_off, long n, int dtype,
                                int chunks, void* epoch_ctr, void* done_ctr, void* status, cudaStream_t stream) {
  if (world > kMaxRanks) return fail("fabric: world > 8%s");
  const int esz = dtype == 0 ? 4 : 2;
  if ((n * esz) % (16 * world)) return fail("allreduce_twoshot: bytes must be a multiple of 16 * world%s");
  PeerTable pt = make_table(bases, world, rank);
#define GB_TWOSHOT(TT, MWV) launch_k(allreduce_twoshot_kernel<TT, MWV>, chunks, 256, 0, stream, pt, in_off, out_off, flags_off, n, \
                                      (uint32_t*)epoch_ctr, (unsigned*)done_ctr, (KernelStatus*)status)
  if (dtype == 0) { if (world <= 2) GB_TWOSHOT(float, 2); else if (world <= 4) GB_TWOSHOT(float, 4); else GB_TWOSHOT(float, 8); }
  else { if (world <= 2) GB_TWOSHOT(__nv_bfloat16, 2); else if (world <= 4) GB_TWOSHOT(__nv_bfloat16, 4); else GB_TWOSHOT(__nv_bfloat16, 8); }
#undef GB_TWOSHOT
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_push_exchange(void* const* bases, int world, int rank, size_t out_off, size_t flags_off, const void* in, size_t bytes_per_dst,
                            size_t dst_stride_in, int chunks, void* epoch_ctr, void* done_ctr, void* status, size_t ack_off,
                            cudaStream_t stream) {
  // ack_off: offset of uint32 [world] handshake flags in every heap, or 0 when the caller's own ordering keeps a rank from
  // overwriting a receive buffer that a peer still reads
  if (world > kMaxRanks) return fail("fabric: world > 8%s");
  if (bytes_per_dst % 16 || dst_stride_in % 16) return fail("push_exchange: sizes must be multiples of 16 bytes%s");
  launch_k(push_exchange_kernel, chunks, 256, 0, stream, make_table(bases, world, rank), out_off, flags_off, (const char*)in, bytes_per_dst,
                                                   dst_stride_in, (uint32_t*)epoch_ctr, (unsigned*)done_ctr, (KernelStatus*)status, ack_off);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_argmax_allreduce(void* const* bases, int world, int rank, size_t data_off, size_t flags_off, const float* val, const int* idx,
                               int* out_idx, float* out_val, int rows, int max_rows, void* epoch_ctr, void* status, size_t parity_stride,
                               cudaStream_t stream) {
  if (world > kMaxRanks) return fail("fabric: world > 8%s");
  if (rows > max_rows) return fail("argmax_allreduce: too many rows%s");
  launch_k(argmax_allreduce_kernel, 1, 256, 0, stream, make_table(bases, world, rank), data_off, flags_off, val, idx, out_idx, out_val, rows, max_rows,
                                                 (uint32_t*)epoch_ctr, (KernelStatus*)status, parity_stride);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_ep_dispatch(void* const* bases, int world, int rank, const void* h, int ld_h, int hidden, const int* row_token,
                          const int* seg_start, const int* seg_count, int region_rows, int experts_per_rank, size_t x_off, size_t sf_off,
                          size_t meta_off, size_t flags_off, int mx, int sf32, void* epoch_ctr, void* done_ctr, void* status, cudaStream_t stream) {
  if (world > kMaxRanks) return fail("fabric: world > 8%s");
  if (hidden % 128 || region_rows % 128) return fail("ep_dispatch: hidden and region_rows must be multiples of 128%s");
  EpDispatchArgs a;
  memset(&a, 0, sizeof(a));
  a.h = (const __nv_bfloat16*)h; a.ld_h = ld_h; a.hidden = hidden; a.row_token = row_token; a.seg_start = seg_start; a.seg_count = seg_count;
  a.region_rows = region_rows; a.experts_per_rank = experts_per_rank; a.x_off = x_off; a.sf_off = sf_off; a.meta_off = meta_off;
  a.flags_off = flags_off; a.mx = mx; a.sf32 = sf32; a.epoch_ctr = (uint32_t*)epoch_ctr; a.done_ctr = (unsigned*)done_ctr; a.st = (KernelStatus*)status;
  if ((hidden / 8) % 32) return fail("ep_dispatch: hidden must be a multiple of 256%s");
  const long total_rows = (long)world * region_rows;
  int grid = (int)std::min<long>((total_rows + 7) / 8, (long)sm_count() * 8);
  if (grid < 1) grid = 1;
  launch_k(ep_dispatch_kernel, grid, 256, 0, stream, make_table(bases, world, rank), a);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

// gb_ep_dispatch for tokens that are already MXFP8: hq e4m3 bytes [T, hidden], hsf their scale atoms (in_sf32: 32-row layout).
GB_API int gb_ep_dispatch_mx(void* const* bases, int world, int rank, const void* hq, const void* hsf, int in_sf32, int hidden,
                             const int* row_token, const int* seg_start, const int* seg_count, int region_rows, int experts_per_rank,
                             size_t x_off, size_t sf_off, size_t meta_off, size_t flags_off, int sf32, void* epoch_ctr, void* done_ctr,
                             void* status, cudaStream_t stream) {
  if (world > kMaxRanks) return fail("fabric: world > 8%s");
  if (hidden % 128 || region_rows % 128 || ((uintptr_t)hq & 15) || ((uintptr_t)hsf & 3)) return fail("ep_dispatch_mx: bad shape or alignment%s");
  EpDispatchArgs a;
  memset(&a, 0, sizeof(a));
  a.hidden = hidden; a.row_token = row_token; a.seg_start = seg_start; a.seg_count = seg_count;
  a.region_rows = region_rows; a.experts_per_rank = experts_per_rank; a.x_off = x_off; a.sf_off = sf_off; a.meta_off = meta_off;
  a.flags_off = flags_off; a.mx = 1; a.sf32 = sf32; a.epoch_ctr = (uint32_t*)epoch_ctr; a.done_ctr = (unsigned*)done_ctr; a.st = (KernelStatus*)status;
  a.hq = (const uint8_t*)hq; a.hsf = (const uint8_t*)hsf; a.in_sf32 = in_sf32;
  const long total_rows = (long)world * region_rows;
  int grid = (int)std::min<long>((total_rows + 7) / 8, (long)sm_count() * 8);
  if (grid < 1) grid = 1;
  launch_k(ep_dispatch_kernel, grid, 256, 0, stream, make_table(bases, world, rank), a);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_epoch_tick(void* ctr, cudaStream_t stream) {
  launch_k(epoch_tick_kernel, 1, 1, 0, stream, (uint32_t*)ctr);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}
