// Flag words shared between GPUs: system-scope release stores, acquire loads
// and a wait that is bounded by a wall-clock deadline.  A wait that runs out
// records kStatusPeerTimeout in the status word and returns false; it also
// returns false as soon as any other kernel has recorded a failure, so that
// one lost peer does not cost one timeout per waiting kernel.
#pragma once
#include <stdint.h>

#include "ptx.cuh"

namespace piper {

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ unsigned long long ld_acquire_sys(const uint64_t* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(uint64_t* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Waits until flags[0..n) are all >= value.  The status word is the first of four ints: a wait that runs out
// also leaves (tag of the wait, index of the flag it was waiting for, value it wanted) in the other three.
__device__ inline bool wait_flags(const uint64_t* flags, int n, unsigned long long value,
                                  unsigned long long timeout_ns, int* status, int tag = 0) {
  const unsigned long long t0 = globaltimer_ns();
  for (int p = 0; p < n; ++p) {
    unsigned spins = 0;
    while (ld_acquire_sys(flags + p) < value) {
      if ((++spins & 255u) == 0) {
        if (*reinterpret_cast<volatile int*>(status) != 0) return false;
        if (globaltimer_ns() - t0 > timeout_ns) {
          if (atomicCAS(status, 0, kStatusPeerTimeout) == 0) {
            status[1] = tag;
            status[2] = p;
            status[3] = static_cast<int>(value);
          }
          return false;
        }
      }
      __nanosleep(64);
    }
  }
  return true;
}

}  // namespace piper
