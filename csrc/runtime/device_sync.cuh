// Device-side synchronisation primitives shared by every kernel that talks to another GPU.
//
// * system-scope release/acquire accessors for flags that live in a peer's memory;
// * bounded waits: every spin has a wall-clock limit (globaltimer); when it runs out the kernel
//   records WHERE it gave up in a status block, raises a local abort flag so that sibling CTAs
//   stop too, and returns normally. Nothing here traps or spins forever.
// The reference's flag helpers (nvidia/src/fast_alltoall/flash_alltoall_nvshmem.cu:5-52) and its
// unbounded nvshmem_uint64_wait_until / while(true) waits (:1645-1689, :2451-2482) are the
// behaviour this replaces.
#pragma once
#include <cstdint>

namespace fastb {

// Written by the device (first error wins), read by the host after the stream is idle.
struct DeviceStatus {
  unsigned long long code;    // 0 = ok, see kStatus*
  unsigned long long site;    // which wait gave up (kSite*)
  unsigned long long detail;  // peer rank / stage / item index, site specific
  unsigned long long seen;    // last value observed
  unsigned long long want;    // value waited for
  unsigned long long abort;   // non-zero once any CTA of this rank has given up
};

constexpr unsigned long long kStatusOk = 0, kStatusTimeout = 1, kStatusBadArg = 2;
enum WaitSite : unsigned long long {
  kSiteEntryReady = 1, kSiteBalanceArrive = 2, kSiteRailArrive = 3, kSiteOutputArrive = 4,
  kSiteCountsArrive = 5, kSiteCombineReady = 6, kSiteReuse = 7, kSiteMbarrier = 8, kSiteTest = 9, kSiteCapacity = 10, kSiteExpertId = 11,
};

#ifdef __CUDACC__
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void report_failure(DeviceStatus* st, unsigned long long code, unsigned long long site,
                                               unsigned long long detail, unsigned long long seen, unsigned long long want) {
  if (atomicCAS(&st->code, 0ull, code) == 0ull) {
    st->site = site; st->detail = detail; st->seen = seen; st->want = want;
  }
  atomicExch(&st->abort, 1ull);
  __threadfence_system();
}

// Waits until *flag >= want (acquire). Returns false after timeout_ns or once a sibling aborted.
__device__ __forceinline__ bool wait_ge_bounded(const unsigned long long* flag, unsigned long long want, DeviceStatus* st,
                                                unsigned long long site, unsigned long long detail, unsigned long long timeout_ns) {
  unsigned long long v = ld_acquire_sys(flag);
  if (v >= want) return true;
  const unsigned long long t0 = global_timer_ns();
  unsigned int spins = 0;
  while (true) {
    v = ld_acquire_sys(flag);
    if (v >= want) return true;
    if ((++spins & 63u) == 0u) {
      if (*reinterpret_cast<volatile unsigned long long*>(&st->abort) != 0ull) return false;
      if (global_timer_ns() - t0 > timeout_ns) {
        report_failure(st, kStatusTimeout, site, detail, v, want);
        return false;
      }
      __nanosleep(32);
    }
  }
}

#endif  // __CUDACC__

}  // namespace fastb
