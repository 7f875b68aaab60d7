// Host-side helpers shared by the kernel launchers: error strings, TMA descriptor encoding through
// the driver entry point (no link-time dependency on libcuda), launch configuration.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#define GB_API extern "C" __attribute__((visibility("default")))

namespace gb {

// Last error message of this thread; returned by gb_last_error().
char* last_error_buf();

inline int fail(const char* fmt, const char* a = "", long b = 0, long c = 0) {
  snprintf(last_error_buf(), 512, fmt, a, b, c);
  return -1;
}

#define GB_CUDA_OK(expr)                                                                    \
  do {                                                                                      \
    cudaError_t _e = (expr);                                                                \
    if (_e != cudaSuccess) {                                                                \
      snprintf(gb::last_error_buf(), 512, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return -1;                                                                            \
    }                                                                                       \
  } while (0)

enum TmapDtype { TM_U8 = 0, TM_BF16 = 1, TM_F16 = 2, TM_F32 = 3, TM_U32 = 4 };
enum TmapSwizzle { TM_SW_NONE = 0, TM_SW_32 = 1, TM_SW_64 = 2, TM_SW_128 = 3 };

// Encode a tiled tensor map of rank 2..4.  dims / box are in elements, innermost first; strides are in
// bytes for dims 1.. (dim 0 is contiguous).  Returns 0 on success.
int make_tmap(CUtensorMap* out, const void* base, TmapDtype dt, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, TmapSwizzle sw);

inline int make_tmap_2d(CUtensorMap* out, const void* base, TmapDtype dt, uint64_t inner, uint64_t outer,
                        uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, TmapSwizzle sw) {
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[1] = {row_stride_bytes};
  uint32_t box[2] = {box_inner, box_outer};
  return make_tmap(out, base, dt, 2, dims, strides, box, sw);
}

int sm_count();   // SMs of the current device (cached per device)

// Programmatic dependent launch: when on (default; gb_set_pdl(0) or GB_PDL=0 turns it off), every kernel of this library
// is launched with the "programmatic stream serialization" attribute.  Each kernel signals
// griddepcontrol.launch_dependents as soon as it starts and executes griddepcontrol.wait before its first access to
// global memory, so the launch latency and the prologue (barrier init, TMEM allocation, descriptor prefetch) of kernel
// N+1 overlap the tail of kernel N while all memory dependencies stay those of a plain stream.
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<Args&&>(args)...);
}

// The same with a thread-block cluster of `cluster_x` CTAs along x (distributed shared memory between them).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster_x,
                                    Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = cluster_x; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<Args&&>(args)...);
}

}  // namespace gb
