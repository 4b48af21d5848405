// peer.cuh — device-side halves of the small all-reduce over mapped peer memory (see PeerXchg
// in runtime.h and PeerPush in kernels.h): a bounded wait on a flag another GPU raises, and
// the "last CTA raises the flags" tail of a pushing kernel.
#pragma once

#include "kernels.h"

namespace cg {

// Bounded wait until a flag written by another GPU reaches `want`; on expiry raises the
// context's error word and gives up (the caller carries on with whatever data is there).  Once a
// timeout has been reported in this context, every later wait gives up at its first slow-path
// check: a rank that stopped pushing costs the others one limit in total, not one per hand-over.
// The limit is the 64-bit word at byte offset 8 of the error block (nanoseconds, 0 = 1 s).
__device__ __forceinline__ bool peer_wait_flag(const uint32_t* f, uint32_t want, int32_t* err) {
  unsigned long long t0 = 0, limit = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if (v == want) return true;
    if ((it & 0xFF) == 0xFF) {
      if (*(volatile int32_t*)err == DEV_TIMEOUT) return false;
      unsigned long long now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (t0 == 0) {
        t0 = now;
        limit = *(const volatile unsigned long long*)(err + 2);
        if (limit == 0) limit = 1000000000ull;
      } else if (now - t0 > limit) { *err = DEV_TIMEOUT; return false; }
    }
  }
}

// Parity of the reduction a pushing kernel contributes to: one more than the last one this
// rank pushed.  Read after the kernel's dependency wait; stable until the kernel's last CTA
// has seen every other CTA finish.
__device__ __forceinline__ uint32_t peer_push_parity(const PeerPush& px) {
  return (*(volatile uint32_t*)px.epoch + 1u) & 1u;
}

// Tail of a pushing kernel, called by ONE thread per CTA after a CTA-wide barrier that
// follows the CTA's last push: the fence orders the CTA's pushes (system wide) before its
// ticket, and the CTA that draws the last ticket raises this rank's flag on every rank.
__device__ __forceinline__ void peer_push_done(const PeerPush& px, unsigned total_ctas) {
  __threadfence_system();
  const unsigned t = atomicAdd(px.ticket, 1u);
  if (t == total_ctas - 1u) {
    *px.ticket = 0u;
    const uint32_t e = *(volatile uint32_t*)px.epoch + 1u;
    __threadfence_system();
    for (int r = 0; r < px.world; ++r)
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(px.flags[r] + (e & 1u) * px.world + px.rank), "r"(e) : "memory");
    *(volatile uint32_t*)px.epoch = e;
  }
}

}  // namespace cg
