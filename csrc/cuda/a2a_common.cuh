// Control-block layout, flag waits and signalling shared by the push-exchange kernels (a2a_push.cu, a2a_dynamic.cu).
#pragma once
#include "common.cuh"
#include "peer.cuh"

namespace rba2a {

using namespace rbpeer;

constexpr int A2A_PHASES = 4;
// control block of one rank (peer-mapped, ints): counts[W_MAX src][W_MAX dst] then flags[A2A_PHASES][W_MAX src]
constexpr int CTL_COUNTS = 0;
constexpr int CTL_FLAGS = MAX_RANKS * MAX_RANKS;
constexpr int CTL_INTS = CTL_FLAGS + A2A_PHASES * MAX_RANKS;

// local (not peer-visible) state, ints
constexpr int LOC_EPOCH = 0;                    // [A2A_PHASES] epoch of each signalling kernel
constexpr int LOC_TICKET = 8;                   // [A2A_PHASES] last-block tickets
constexpr int LOC_CNT = 16;                     // [W_MAX] entries this rank sends to each owner (this step)
constexpr int LOC_CURSOR = 32;                  // [W_MAX] running position while scattering
constexpr int LOC_BASE = 48;                    // [W_MAX] first position of this rank's entries in each owner's list
constexpr int LOC_SRC_PREFIX = 64;              // [W_MAX + 1] prefix of the sources in this rank's own receive list
constexpr int LOC_N_OWNED = 96;                 // entries in this rank's receive list (clamped to the capacity)
constexpr int LOC_INTS = 128;

constexpr long long META_J_MASK = 0xFFFFFFFFll;
__device__ __forceinline__ long long make_meta(long long j, int f, int src) {
  return j | (static_cast<long long>(f) << 32) | (static_cast<long long>(src) << 48);
}
__device__ __forceinline__ int meta_f(long long m) { return static_cast<int>((m >> 32) & 0xFFFF); }
__device__ __forceinline__ int meta_src(long long m) { return static_cast<int>((m >> 48) & 0xFF); }

__device__ __forceinline__ bool wait_flags(const int* ctl_local, int phase, int e, int world, int* status,
                                           unsigned long long limit_ns, int* s_ok) {
  if (threadIdx.x < world) {
    const int* f = ctl_local + CTL_FLAGS + phase * MAX_RANKS + threadIdx.x;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    bool ok = false;
    for (unsigned it = 0;; ++it) {
      if (ld_acquire_sys(f) - e >= 0) { ok = true; break; }
      if ((it & 63) == 63) {
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > limit_ns) break;
      }
    }
    if (!ok) {
      *s_ok = 0;
      if (status) atomicCAS(status, 0, RB_ERR_PEER_TIMEOUT);
    }
  }
  __syncthreads();
  return *s_ok != 0;
}

// Every block calls this after its last global store of the kernel; true in the block that finishes last.
// One system-scope fence per block, issued by the thread that takes the ticket after the block barrier: the barrier
// orders every thread's stores before that thread, and its fence is cumulative over them (a fence in every thread would
// cost one membar.sys per thread for the same guarantee).
__device__ __forceinline__ bool is_last_block(int* loc, int phase) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int t = atomicAdd(loc + LOC_TICKET + phase, 1);
    s_last = (t == static_cast<int>(gridDim.x) - 1);
  }
  __syncthreads();
  return s_last != 0;
}

// Last block only: raise flags[phase][me] = e at every rank and publish the epoch locally.  The release store at system
// scope orders everything this block has observed (all blocks' tickets, hence their fenced stores) before the flag.
__device__ __forceinline__ void signal_all(const PeerPtrs& ctl, int* loc, int phase, int e, int me, int world) {
  __syncthreads();
  if (threadIdx.x < world) {
    __threadfence_system();      // at most 16 threads of one block: cheap, and keeps the acquire side of the ticket chain explicit
    st_release_sys(reinterpret_cast<int*>(ctl.p[threadIdx.x]) + CTL_FLAGS + phase * MAX_RANKS + me, e);
  }
  if (threadIdx.x == 0) {
    loc[LOC_TICKET + phase] = 0;
    __threadfence();
    *reinterpret_cast<volatile int*>(loc + LOC_EPOCH + phase) = e;
  }
}

__device__ __forceinline__ int table_of(const long long* cumsum, int n, long long key) {
  int lo = 0, hi = n;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (cumsum[mid] <= key) lo = mid; else hi = mid; }
  return lo;
}

}  // namespace rba2a
