// In-kernel collectives over NVLink peer mappings (and NVSwitch multimem where a multicast
// mapping exists).  These replace the library collectives on the hot path:
//
//   rb_peer_barrier        device-side barrier of all ranks (flag words in each rank's peer-mapped
//                          signal pad, monotonically increasing epoch kept on the device so that a
//                          captured CUDA graph replays correctly).
//   rb_allgather_push      every rank stores its slab into all peers' copy of a gathered buffer
//                          (used for the id exchange that precedes the owner-side gradient update).
//   rb_allreduce_f32       two-shot all-reduce of the flat fp32 dense-gradient buffer with the
//                          1/world scale fused: each rank reduces its slice by reading every peer
//                          (or one multimem.ld_reduce through the switch) and writes the result to
//                          every peer (or one multimem.st).  Barriers before/between/after are part
//                          of the same launch.
//
// Every flag wait is bounded; on expiry the kernel records RB_ERR_PEER_TIMEOUT and returns.
// The reference's counterpart is its LCCL layer (cust_op/ascendc_op/ai_core_op/lccl/v220/op_kernel/
// all2all.h, sync_collectives.h), whose waits are unbounded.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

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

// One warp-sized team signals every peer and waits for every peer.  `slot` selects one of several
// independent flag rows so different barriers of a step never alias.  Returns false on timeout.
__device__ bool barrier_team(const PeerPtrs& pads, int* epoch_word, int rank, int world, int slot,
                             int* status, unsigned long long limit_ns) {
  __shared__ int s_epoch;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_epoch = *epoch_word + 1;
    s_ok = 1;
  }
  __syncthreads();
  const int e = s_epoch;
  if (threadIdx.x < world) {
    const int peer = threadIdx.x;
    int* remote = reinterpret_cast<int*>(pads.p[peer]) + slot * MAX_RANKS + rank;
    __threadfence_system();
    st_release_sys(remote, e);
    const int* mine = reinterpret_cast<const int*>(pads.p[rank]) + slot * MAX_RANKS + peer;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    bool ok = false;
    for (unsigned long long it = 0;; ++it) {
      if (ld_acquire_sys(mine) - e >= 0) { ok = true; break; }
      if ((it & 255) == 255) {
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > limit_ns) break;
        __nanosleep(100);
      }
    }
    if (!ok) {
      s_ok = 0;
      if (status) atomicCAS(status, 0, RB_ERR_PEER_TIMEOUT);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *epoch_word = e;
  __syncthreads();
  return s_ok != 0;
}

__global__ void peer_barrier_kernel(PeerPtrs pads, int* epoch_word, int rank, int world, int slot, int* status,
                                    unsigned long long limit_ns) {
  barrier_team(pads, epoch_word, rank, world, slot, status, limit_ns);
}

// dst_r[dst_offset + i] = src[i] for every rank r (16-byte vectors)
__global__ void allgather_push_kernel(PeerPtrs dst, const uint4* __restrict__ src, long long n_vec,
                                      long long dst_offset_vec, int world) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    const uint4 v = src[i];
#pragma unroll 1
    for (int r = 0; r < world; ++r) reinterpret_cast<uint4*>(dst.p[r])[dst_offset_vec + i] = v;
  }
}

// strided variant: src is [rows, cols_vec] contiguous, destination row stride dst_ld_vec, column
// offset dst_col_vec (gathers per-feature id slabs into a [T, world * B_local] matrix).
__global__ void allgather_push_2d_kernel(PeerPtrs dst, const uint4* __restrict__ src, int rows, long long cols_vec,
                                         long long dst_ld_vec, long long dst_col_vec, int world) {
  const long long total = static_cast<long long>(rows) * cols_vec;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r_ = i / cols_vec, c = i % cols_vec;
    const uint4 v = src[i];
#pragma unroll 1
    for (int r = 0; r < world; ++r) reinterpret_cast<uint4*>(dst.p[r])[r_ * dst_ld_vec + dst_col_vec + c] = v;
  }
}

__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_f32x4(float* mc_addr, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_addr), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

// Cooperative launch: grid-wide syncs separate the three phases.
//   phase 0: barrier (all ranks finished producing gradients)
//   phase 1: rank r reduces slice r (sum over peers * scale) and stores it to every peer
//   phase 2: barrier (all slices landed everywhere)
__global__ void allreduce_f32_kernel(PeerPtrs bufs, float* mc_buf, PeerPtrs pads, int* epoch_word, long long n,
                                     float scale, int rank, int world, int slot, int* status,
                                     unsigned long long limit_ns, int* abort_word) {
  cg::grid_group grid = cg::this_grid();
  if (blockIdx.x == 0) {
    const bool ok = barrier_team(pads, epoch_word, rank, world, slot, status, limit_ns);
    if (!ok && threadIdx.x == 0) *abort_word = 1;
  }
  grid.sync();
  const bool aborted = *reinterpret_cast<volatile int*>(abort_word) != 0;
  if (!aborted) {
    const long long n_vec = n / 4;
    const long long per = (n_vec + world - 1) / world;
    const long long beg = per * rank;
    const long long end = (beg + per < n_vec) ? beg + per : n_vec;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = beg + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < end; i += stride) {
      float4 acc;
      if (mc_buf) {
        acc = multimem_ld_reduce_f32x4(mc_buf + i * 4);
      } else {
        acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int r = 0; r < world; ++r) {
          const float4 v = reinterpret_cast<const float4*>(bufs.p[r])[i];
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
      }
      acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
      if (mc_buf) {
        multimem_st_f32x4(mc_buf + i * 4, acc);
      } else {
#pragma unroll 1
        for (int r = 0; r < world; ++r) reinterpret_cast<float4*>(bufs.p[r])[i] = acc;
      }
    }
    __threadfence_system();
  }
  grid.sync();
  if (blockIdx.x == 0 && !aborted) barrier_team(pads, epoch_word, rank, world, slot + 1, status, limit_ns);
}

inline PeerPtrs to_ptrs(const unsigned long long* host_ptrs, int world) {
  PeerPtrs p;
  for (int i = 0; i < MAX_RANKS; ++i) p.p[i] = (i < world) ? host_ptrs[i] : 0ull;
  return p;
}

}  // namespace

// pads[r]: device address (in this process) of rank r's signal pad, at least 64 * 16 ints, zeroed once.
RB_API int rb_peer_barrier(const unsigned long long* pads, int* epoch_word, int rank, int world, int slot,
                           int* status, long long timeout_ms, cudaStream_t st) {
  if (world > MAX_RANKS) return -1;
  peer_barrier_kernel<<<1, 32, 0, st>>>(to_ptrs(pads, world), epoch_word, rank, world, slot, status,
                                        static_cast<unsigned long long>(timeout_ms) * 1000000ull);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_allgather_push(const unsigned long long* dst_ptrs, const void* src, long long bytes,
                             long long dst_offset_bytes, int world, int num_sms, cudaStream_t st) {
  if (world > MAX_RANKS || (bytes % 16) || (dst_offset_bytes % 16)) return -1;
  if (bytes == 0) return 0;
  const long long n_vec = bytes / 16;
  long long blocks = (n_vec + 255) / 256;
  const long long cap = (num_sms > 0 ? num_sms : 148) * 4;
  if (blocks > cap) blocks = cap;
  allgather_push_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(to_ptrs(dst_ptrs, world),
                                                                 reinterpret_cast<const uint4*>(src), n_vec,
                                                                 dst_offset_bytes / 16, world);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_allgather_push_2d(const unsigned long long* dst_ptrs, const void* src, int rows, long long row_bytes,
                                long long dst_row_bytes, long long dst_col_bytes, int world, int num_sms,
                                cudaStream_t st) {
  if (world > MAX_RANKS || (row_bytes % 16) || (dst_row_bytes % 16) || (dst_col_bytes % 16)) return -1;
  if (rows == 0 || row_bytes == 0) return 0;
  const long long total = static_cast<long long>(rows) * (row_bytes / 16);
  long long blocks = (total + 255) / 256;
  const long long cap = (num_sms > 0 ? num_sms : 148) * 4;
  if (blocks > cap) blocks = cap;
  allgather_push_2d_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
      to_ptrs(dst_ptrs, world), reinterpret_cast<const uint4*>(src), rows, row_bytes / 16, dst_row_bytes / 16,
      dst_col_bytes / 16, world);
  return static_cast<int>(cudaGetLastError());
}

// In-place averaged all-reduce of n fp32 values held at the same offset of every rank's peer-mapped
// buffer.  n must be a multiple of 4; mc_buf is the multicast mapping of the same buffer or null.
// Uses barrier slots `slot` and `slot + 1`.  abort_word is one zeroed int of scratch.
RB_API int rb_allreduce_f32(const unsigned long long* buf_ptrs, void* mc_buf, const unsigned long long* pads,
                            int* epoch_word, long long n, float scale, int rank, int world, int slot, int* status,
                            long long timeout_ms, int* abort_word, int num_sms, cudaStream_t st) {
  if (world > MAX_RANKS || (n % 4)) return -1;
  if (n == 0) return 0;
  PeerPtrs bufs = to_ptrs(buf_ptrs, world);
  PeerPtrs pd = to_ptrs(pads, world);
  float* mc = reinterpret_cast<float*>(mc_buf);
  unsigned long long limit = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
  long long per_rank_vec = (n / 4 + world - 1) / world;
  int blocks = static_cast<int>((per_rank_vec + 255) / 256);
  const int cap = (num_sms > 0 ? num_sms : 148);
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  void* args[] = {&bufs, &mc, &pd, &epoch_word, &n, &scale, &rank, &world, &slot, &status, &limit, &abort_word};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(allreduce_f32_kernel), dim3(blocks),
                                                      dim3(256), args, 0, st));
}
