// Device-side primitives for kernels that talk to another GPU (or another CTA) through memory:
// system-scope acquire loads / release stores / release reductions on 32-bit flag words, and the
// one bounded wait that every such kernel uses.
//
// Conventions shared by all kernel families (fused GEMM + collective, context-parallel attention,
// data-parallel optimizer, expert-parallel dispatch / combine, stand-alone collectives):
//   * flag words only ever grow; a call knows the value that means "this call's data has arrived"
//     (an epoch or a running count), so nothing is reset between calls;
//   * data is written with plain stores, then made visible with __threadfence_system() followed
//     by a release store / reduction on the flag; the consumer acquires the flag, then reads;
//   * a wait gives up after `limit_ns` of wall time (host-settable, lb_set_flag_wait_ns; default
//     20 s because ranks may be seconds apart at start-up) and returns false.  The caller records
//     a status word that the host reads (lb_*_status), stops consuming the data it waited for and
//     leaves; it never spins forever and never traps.
#pragma once
#include "common.cuh"

namespace lbcomm {

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Waits until *f >= target (wrap-around safe).  False when `limit_ns` ran out first.
__device__ __forceinline__ bool flag_wait_ge(const unsigned int* f, unsigned int target, unsigned long long limit_ns) {
  if ((int)(ld_acquire_sys(f) - target) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  while (true) {
    for (int i = 0; i < 64; i++) {
      if ((int)(ld_acquire_sys(f) - target) >= 0) return true;
      __nanosleep(64);
    }
    if (globaltimer_ns() - t0 > limit_ns) return false;
  }
}

// 16-byte peer / local copies that never go through a cache line that could be stale.
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) { return __ldcv(reinterpret_cast<const uint4*>(p)); }

}  // namespace lbcomm
