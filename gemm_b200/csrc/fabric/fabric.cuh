// NVLink fabric primitives used from inside kernels: peer pointer tables, system-scope flag stores and
// bounded flag waits.  A "flag" is a 32-bit word in a peer's symmetric heap that only ever grows (epoch
// numbers), as the reference's one-sided Put protocol does with its sequence trailer
// (a64fx/utofu-tests/tp_allreduce.h:90-97); unlike it, an expired wait returns an error status and the
// kernel finishes normally (the reference exits the process, tp_allreduce.h:122-134).
#pragma once
#include "../kernels/sm100.cuh"

namespace gb {

constexpr int kMaxRanks = 8;

struct PeerTable {
  void* base[kMaxRanks];     // base address of every rank's symmetric heap as mapped in THIS process
  int world;
  int rank;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Wait until *flag >= want (wrap-safe signed difference).  One thread calls this; returns false after
// the wall-clock budget and records (rank waited for, wanted, seen) in the status word.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want, KernelStatus* st, int where, int peer,
                                             uint64_t budget_ns = kPeerBudgetNs) {
  uint32_t v = ld_acquire_sys(flag);
  if ((int32_t)(v - want) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    v = ld_acquire_sys(flag);
    if ((int32_t)(v - want) >= 0) return true;
    if ((it & 0xff) == 0) {
      if (globaltimer_ns() - t0 > budget_ns) {
        report_status(st, ST_TIMEOUT_FLAG, where, peer, (int)want, (int)v);
        return false;
      }
      __nanosleep(64);
    }
  }
}

}  // namespace gb
