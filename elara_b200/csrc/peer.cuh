// What the kernels that talk to other ranks' GPUs share: the table of peer pointers a kernel receives by value, the
// bounded barrier lane, and the containment of a failed exchange.
#pragma once
#include "common.cuh"

namespace srm2 {

constexpr int kMaxPeers = 16;
struct PeerPtrs { void* p[kMaxPeers]; };

// Lane r < world of one warp: arrive at rank r, then wait for rank r.  Callers make their earlier stores visible first
// (__threadfence_system by every writing thread, then a warp or CTA barrier).
// A rank that leaves a barrier with its error word set (a peer that never arrived, an overflowed receive buffer, now or
// in an earlier step: the word is sticky) must not feed what it received to the update kernels: with n_recv != nullptr the
// lane then sets the count of received lookups to zero, so dedup, index and the fused reduce + Adam of that step see an
// empty batch and leave the shard untouched.
__device__ __forceinline__ void contain_failure(const uint32_t* err, int64_t* n_recv) {
  if (n_recv != nullptr && *reinterpret_cast<const volatile uint32_t*>(err) != 0u) *n_recv = 0;
}

__device__ __forceinline__ void peer_barrier_lane(const PeerPtrs& sig, int rank, int r, unsigned long long ticket, uint32_t* __restrict__ err,
                                                  long long timeout_ns) {
  unsigned long long* dst = static_cast<unsigned long long*>(sig.p[r]) + rank;
  __threadfence_system();
  asm volatile("st.release.sys.global.u64 [%0], %1;\n" ::"l"(dst), "l"(ticket) : "memory");
  const unsigned long long* src = static_cast<const unsigned long long*>(sig.p[rank]) + r;
  long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t0));
  for (uint32_t it = 0; it < (1u << 27); ++it) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];\n" : "=l"(v) : "l"(src) : "memory");
    if (v >= ticket) return;
    if ((it & 15u) == 15u) {
      long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t1));
      if (t1 - t0 > timeout_ns) break;
    }
    __nanosleep(40);
  }
  atomicOr(err, 2u);
}

}  // namespace srm2
