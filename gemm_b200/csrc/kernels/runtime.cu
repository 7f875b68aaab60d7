// Process-wide runtime pieces of the kernel library: last-error string, the status word that
// bounded waits report into, TMA descriptor encoding, device properties.
#include "host_common.h"
#include <stdlib.h>
#include "sm100.cuh"
#include <cudaTypedefs.h>
#include <mutex>

namespace gb {

char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
static std::once_flag g_encode_once;

static void load_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) g_encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
}

int make_tmap(CUtensorMap* out, const void* base, TmapDtype dt, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, TmapSwizzle sw) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return fail("cuTensorMapEncodeTiled entry point not available%s");
  static const CUtensorMapDataType dts[] = {CU_TENSOR_MAP_DATA_TYPE_UINT8, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                            CU_TENSOR_MAP_DATA_TYPE_FLOAT16, CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                                            CU_TENSOR_MAP_DATA_TYPE_UINT32};
  static const CUtensorMapSwizzle sws[] = {CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_SWIZZLE_32B,
                                           CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_SWIZZLE_128B};
  if (((uintptr_t)base & 15) != 0) return fail("tensor map base %s is not 16-byte aligned");
  cuuint64_t gdim[5]; cuuint64_t gstr[4]; cuuint32_t gbox[5]; cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; gbox[i] = box[i]; estr[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) {
    gstr[i] = strides_bytes[i];
    if (gstr[i] % 16 != 0) return fail("tensor map stride%s %ld is not a multiple of 16 bytes", "", (long)gstr[i]);
  }
  CUresult r = g_encode(out, dts[dt], (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, gbox, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, sws[sw], CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed%s code %ld", "", (long)r);
  return 0;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, dev) == cudaSuccess) cached[dev] = p.multiProcessorCount;
    else cached[dev] = 148;
  }
  return cached[dev];
}

static int g_pdl = -1;
bool pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("GB_PDL");
    g_pdl = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return g_pdl != 0;
}

static __device__ KernelStatus g_status;

}  // namespace gb

GB_API const char* gb_last_error() { return gb::last_error_buf(); }

// Device address of the per-device status word (one per device that loaded the library).
GB_API void* gb_status_ptr() {
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, gb::g_status) != cudaSuccess) return nullptr;
  return p;
}

// Copies the status word to `out16` (16 ints) and optionally clears it.  Synchronises the device.
GB_API int gb_status_read(int* out16, int clear) {
  GB_CUDA_OK(cudaDeviceSynchronize());
  GB_CUDA_OK(cudaMemcpyFromSymbol(out16, gb::g_status, sizeof(gb::KernelStatus)));
  if (clear) {
    gb::KernelStatus z;
    memset(&z, 0, sizeof(z));
    GB_CUDA_OK(cudaMemcpyToSymbol(gb::g_status, &z, sizeof(z)));
  }
  return 0;
}

GB_API int gb_sm_count() { return gb::sm_count(); }

// Turn programmatic dependent launch on (1) or off (0) for every later launch of this library; returns the old setting.
GB_API int gb_set_pdl(int on) {
  const int old = gb::pdl_enabled() ? 1 : 0;
  gb::g_pdl = on ? 1 : 0;
  return old;
}
