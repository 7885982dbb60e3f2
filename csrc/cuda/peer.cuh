// Peer-memory helpers shared by the in-kernel collectives: the per-rank pointer table passed by value to kernels and
// system-scope release / acquire accesses for flag words that another GPU reads or writes.
#pragma once
#include "common.cuh"

namespace rbpeer {

constexpr int MAX_RANKS = 16;

struct PeerPtrs {
  unsigned long long p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

inline PeerPtrs to_ptrs(const unsigned long long* host_ptrs, int world) {
  PeerPtrs p;
  for (int i = 0; i < MAX_RANKS; ++i) p.p[i] = (i < world) ? host_ptrs[i] : 0ull;
  return p;
}

}  // namespace rbpeer
