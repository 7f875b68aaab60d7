// Allocation-free variant of the two-stage arg-max (see argmax_noalloc.h for who needs it and the rules).
// The partial (value, index) pairs of stage one live in a file-scope device array instead of a caller buffer.
#include "argmax_noalloc.h"
#include "host_common.h"
#include <cuda_bf16.h>
#include <float.h>
#include <mutex>

namespace {

constexpr int kChunks = 64;                                   // CTAs per row in stage one
constexpr int kMaxRows = GB_ARGMAX_NOALLOC_MAX_ROWS;
struct Partial { float val; int idx; };

// The scratch: kChunks x kMaxRows partial results = 512 KiB, resident on every device that loads the library.
static __device__ __align__(256) unsigned char g_scratch[kChunks * kMaxRows * sizeof(Partial)];

__device__ __forceinline__ void take_better(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}
template <typename T> __device__ __forceinline__ float load_logit(const T* p, long i);
template <> __device__ __forceinline__ float load_logit<float>(const float* p, long i) { return p[i]; }
template <> __device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* p, long i) { return __bfloat162float(p[i]); }

template <typename T>
__global__ void __launch_bounds__(256)
stage_one(const T* __restrict__ logits, Partial* __restrict__ part, int vocab, long ld, int rows) {
  const int r = blockIdx.y, c = blockIdx.x;
  const int per = (vocab + kChunks - 1) / kChunks;
  const int i0 = c * per, i1 = min(vocab, i0 + per);
  const T* row = logits + (size_t)r * ld;
  float bv = -FLT_MAX; int bi = 0x7fffffff;
  for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) { float v = load_logit(row, i); v = (v == v) ? fmaxf(v, -FLT_MAX) : -FLT_MAX; /* NaN and -inf count as the lowest finite value */ take_better(bv, bi, v, i); }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) take_better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  __shared__ float sv[8]; __shared__ int si[8];
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) take_better(bv, bi, sv[w], si[w]);
    part[(size_t)c * rows + r] = Partial{bv, bi};           // every entry stage two reads is written here first
  }
}

__global__ void __launch_bounds__(64)
stage_two(const Partial* __restrict__ part, int* __restrict__ out_idx, float* __restrict__ out_val, int rows, int idx_offset) {
  const int r = blockIdx.x;
  float bv = -FLT_MAX; int bi = 0x7fffffff;
  if (threadIdx.x < kChunks) { const Partial p = part[(size_t)threadIdx.x * rows + r]; bv = p.val; bi = p.idx; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) take_better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  __shared__ float sv[2]; __shared__ int si[2];
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    take_better(bv, bi, sv[1], si[1]);
    out_idx[r] = bi + idx_offset;
    if (out_val != nullptr) out_val[r] = bv;
  }
}

// Device address of g_scratch per device.  In host code the name g_scratch is only a handle for the runtime, not a
// device address, so it is resolved once per device with that device current.
std::mutex g_mu;
void* g_scratch_addr[64] = {nullptr};

int scratch_for_current_device(void** out) {
  int dev = 0;
  GB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return gb::fail("argmax_noalloc: device index %s%ld is out of range", "", (long)dev);
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    GB_CUDA_OK(cudaGetSymbolAddress(&p, g_scratch));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int gb_argmax_noalloc(const void* logits, int* out_idx, float* out_val, int rows, int vocab, long ld, int dtype, int idx_offset,
                      cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (rows > kMaxRows) return gb::fail("argmax_noalloc: %s%ld rows exceed the built-in scratch (at most %ld rows per call)", "", (long)rows, (long)kMaxRows);
  if (vocab <= 0 || ld < vocab) return gb::fail("argmax_noalloc: bad row geometry%s (vocab %ld, ld %ld)", "", (long)vocab, (long)ld);
  if (dtype != 0 && dtype != 1) return gb::fail("argmax_noalloc: dtype must be 0 (float32) or 1 (bfloat16)%s");
  void* scratch = nullptr;
  if (scratch_for_current_device(&scratch) != 0) return -1;
  Partial* part = static_cast<Partial*>(scratch);
  const dim3 grid(kChunks, rows);
  if (dtype == 0) stage_one<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(logits), part, vocab, ld, rows);
  else stage_one<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), part, vocab, ld, rows);
  stage_two<<<rows, 64, 0, stream>>>(part, out_idx, out_val, rows, idx_offset);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}
