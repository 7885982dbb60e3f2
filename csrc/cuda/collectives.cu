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
#include "peer.cuh"

using namespace rbpeer;

namespace cg = cooperative_groups;

namespace {

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

// ---------------------------------------------------------------------------------------------
// Dense-gradient all-reduce, push design (fused cast + scale, 16-bit on the wire).
//
// Every rank holds n fp32 gradients.  The averaged result is written back in place.  Data crosses
// NVLink as bf16 (or fp32 when wire_bf16 == 0): each rank converts while it pushes, sums arrive in
// fp32 registers, the 1/world scale is applied once on the reduced value.
//
//   two-shot   slice s of the vector belongs to rank s.
//              loop 1  block b converts its chunks of every slice and STORES them into the owner's
//                      staging[me][...] (posted stores over NVLink), then raises flag1[me][b] at every peer
//              loop 2  waits for flag1[src][b] of every source, sums the W staged copies of its chunks
//                      of slice `me` from LOCAL memory, scales, and stores the result into every peer's
//                      result[me][...]; raises flag2[me][b]
//              loop 3  waits for flag2, converts its chunks of every slice of the local result buffer
//                      back into the fp32 gradient buffer
//   one-shot   (small vectors) every rank pushes its whole converted vector to every peer's
//              staging[parity][me][...] and reduces all W copies locally: one flag round trip.
//
// Flags are per (source rank, block): a block only ever waits for the block of the same index on the
// other ranks, whose pushes depend on nothing, so no grid-wide synchronisation and no cooperative launch
// is needed and the kernel can share the GPU with the backward GEMMs.  The epoch lives on the device
// (bumped by the last block to leave), so a captured CUDA graph replays correctly.  Waits are bounded.
// Role in the reference: LCCL all-reduce / ping-pong flag words
// (cust_op/ascendc_op/ai_core_op/lccl/v220/op_kernel/all2all.h:30-140, sync_collectives.h:66-263).
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int AR_THREADS = 512;
constexpr int AR_VEC = 8;                          // elements per thread per chunk
constexpr int AR_CHUNK = AR_THREADS * AR_VEC;      // elements per block iteration

struct ArArgs {
  float* grad;                 // local fp32 vector, n elements (n % 8 == 0)
  long long n;
  PeerPtrs staging;            // per rank: wire-typed staging area
  PeerPtrs result;             // per rank: wire-typed result area (two-shot only)
  PeerPtrs flags;              // per rank: int[2][MAX_RANKS][grid]
  int* epoch_word;             // [0] epoch, [1] ticket
  float scale;
  int rank, world;
  int* status;
  unsigned long long limit_ns;
};

template <bool BF16> struct Wire;
template <> struct Wire<true> {
  using T = uint4;                                 // 8 x bf16
  static constexpr int BYTES = 2;
  static constexpr int GROUP = 8;
  static __device__ __forceinline__ void to_f32(const uint4& u, float (&v)[8]) {
    float2 a = rb::unpack_bf16(u.x), b = rb::unpack_bf16(u.y), c = rb::unpack_bf16(u.z), d = rb::unpack_bf16(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
  static __device__ __forceinline__ uint4 from_f32(const float (&v)[8]) {
    return make_uint4(rb::pack_bf16(v[0], v[1]), rb::pack_bf16(v[2], v[3]), rb::pack_bf16(v[4], v[5]),
                      rb::pack_bf16(v[6], v[7]));
  }
  // peers wrote this memory: read it at L2, never from a stale L1 line
  static __device__ __forceinline__ uint4 ld(const uint4* p) { return __ldcg(p); }
};
struct F32x8 { float4 a, b; };
template <> struct Wire<false> {
  using T = F32x8;                                 // 8 x fp32
  static constexpr int BYTES = 4;
  static constexpr int GROUP = 4;
  static __device__ __forceinline__ void to_f32(const F32x8& u, float (&v)[8]) {
    v[0] = u.a.x; v[1] = u.a.y; v[2] = u.a.z; v[3] = u.a.w; v[4] = u.b.x; v[5] = u.b.y; v[6] = u.b.z; v[7] = u.b.w;
  }
  static __device__ __forceinline__ F32x8 from_f32(const float (&v)[8]) {
    return F32x8{make_float4(v[0], v[1], v[2], v[3]), make_float4(v[4], v[5], v[6], v[7])};
  }
  static __device__ __forceinline__ F32x8 ld(const F32x8* p) {
    const float4* q = reinterpret_cast<const float4*>(p);
    return F32x8{__ldcg(q), __ldcg(q + 1)};
  }
};

__device__ __forceinline__ void ld_grad8(const float* g, long long idx, long long n, float (&v)[8]) {
  if (idx + 8 <= n) {
    const float4 a = *reinterpret_cast<const float4*>(g + idx), b = *reinterpret_cast<const float4*>(g + idx + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
  }
}
__device__ __forceinline__ void st_grad8(float* g, long long idx, long long n, const float (&v)[8]) {
  if (idx + 8 <= n) {
    *reinterpret_cast<float4*>(g + idx) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(g + idx + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
}

// raise flags[phase][me][block] = e at every rank
__device__ __forceinline__ void ar_signal(const ArArgs& a, int phase, int e) {
  __syncthreads();          // every thread's stores are ordered before the releasing threads; st.release.sys carries the fence
  if (threadIdx.x < a.world) {
    int* f = reinterpret_cast<int*>(a.flags.p[threadIdx.x]) +
             (static_cast<long long>(phase) * MAX_RANKS + a.rank) * gridDim.x + blockIdx.x;
    st_release_sys(f, e);
  }
}
// wait until flags[phase][src][block] >= e for every src; false on timeout
__device__ __forceinline__ bool ar_wait(const ArArgs& a, int phase, int e, int* s_ok) {
  if (threadIdx.x < a.world) {
    const int* f = reinterpret_cast<const int*>(a.flags.p[a.rank]) +
                   (static_cast<long long>(phase) * MAX_RANKS + threadIdx.x) * gridDim.x + blockIdx.x;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    bool ok = false;
    for (unsigned it = 0;; ++it) {
      if (ld_acquire_sys(f) - e >= 0) { ok = true; break; }
      if ((it & 63) == 63) {
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > a.limit_ns) break;
      }
    }
    if (!ok) {
      *s_ok = 0;
      if (a.status) atomicCAS(a.status, 0, RB_ERR_PEER_TIMEOUT);
    }
  }
  __syncthreads();
  return *s_ok != 0;
}

__device__ __forceinline__ void ar_leave(const ArArgs& a, int e) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int t = atomicAdd(a.epoch_word + 1, 1);
    if (t == static_cast<int>(gridDim.x) - 1) {
      a.epoch_word[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(a.epoch_word) = e;
    }
  }
}

template <bool BF16>
__global__ void __launch_bounds__(AR_THREADS) allreduce_twoshot_kernel(const ArArgs a) {
  using W = Wire<BF16>;
  using WT = typename W::T;
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  const int e = *reinterpret_cast<volatile int*>(a.epoch_word) + 1;
  __syncthreads();
  const int world = a.world, me = a.rank;
  const long long slice = ((a.n + world - 1) / world + AR_VEC - 1) / AR_VEC * AR_VEC;   // elements per slice
  const long long step = static_cast<long long>(gridDim.x) * (blockDim.x * AR_VEC);
  const long long first = static_cast<long long>(blockIdx.x) * (blockDim.x * AR_VEC) + threadIdx.x * AR_VEC;
  // loop 1: convert and push my contribution to every slice owner
  for (int k = 0; k < world; ++k) {
    const int p = (me + k) % world;
    WT* dst = reinterpret_cast<WT*>(a.staging.p[p]) + (static_cast<long long>(me) * slice) / AR_VEC;
    const long long base = static_cast<long long>(p) * slice;
    for (long long el = first; el < slice; el += 4 * step) {      // four independent 32-byte loads in flight per thread
      float v[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (el + u * step < slice) ld_grad8(a.grad, base + el + u * step, a.n, v[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (el + u * step < slice) dst[(el + u * step) / AR_VEC] = W::from_f32(v[u]);
    }
  }
  ar_signal(a, 0, e);
  // loop 2: reduce my slice from local staging, scale, push the result to everyone
  if (ar_wait(a, 0, e, &s_ok)) {
    const WT* src = reinterpret_cast<const WT*>(a.staging.p[me]);
    for (long long el = first; el < slice; el += step) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int r0 = 0; r0 < world; r0 += W::GROUP) {      // GROUP independent 16/32-byte loads in flight
        WT u[W::GROUP];
#pragma unroll
        for (int r = 0; r < W::GROUP; ++r)
          if (r0 + r < world) u[r] = W::ld(src + (static_cast<long long>(r0 + r) * slice + el) / AR_VEC);
#pragma unroll
        for (int r = 0; r < W::GROUP; ++r)
          if (r0 + r < world) {
            float v[8];
            W::to_f32(u[r], v);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += v[i];
          }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] *= a.scale;
      const WT out = W::from_f32(acc);
      for (int k = 0; k < world; ++k) {
        const int p = (me + k) % world;
        reinterpret_cast<WT*>(a.result.p[p])[(static_cast<long long>(me) * slice + el) / AR_VEC] = out;
      }
    }
    ar_signal(a, 1, e);
    // loop 3: result buffer (local) -> fp32 gradients
    if (ar_wait(a, 1, e, &s_ok)) {
      const WT* res = reinterpret_cast<const WT*>(a.result.p[me]);
      for (int s = 0; s < world; ++s) {
        const long long base = static_cast<long long>(s) * slice;
        for (long long el = first; el < slice; el += step) {
          float v[8];
          W::to_f32(W::ld(res + (base + el) / AR_VEC), v);
          st_grad8(a.grad, base + el, a.n, v);
        }
      }
    }
  }
  ar_leave(a, e);
}

// staging per rank: [2 parity][world][n_pad] wire elements
template <bool BF16>
__global__ void __launch_bounds__(AR_THREADS) allreduce_oneshot_kernel(const ArArgs a) {
  using W = Wire<BF16>;
  using WT = typename W::T;
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  const int e = *reinterpret_cast<volatile int*>(a.epoch_word) + 1;
  __syncthreads();
  const int world = a.world, me = a.rank;
  const long long n_pad = (a.n + AR_VEC - 1) / AR_VEC * AR_VEC;
  const long long half = static_cast<long long>(e & 1) * world * n_pad;
  const long long step = static_cast<long long>(gridDim.x) * (blockDim.x * AR_VEC);
  const long long first = static_cast<long long>(blockIdx.x) * (blockDim.x * AR_VEC) + threadIdx.x * AR_VEC;
  for (long long el = first; el < n_pad; el += step) {
    float v[8];
    ld_grad8(a.grad, el, a.n, v);
    const WT w = W::from_f32(v);
    for (int k = 0; k < world; ++k) {
      const int p = (me + k) % world;
      reinterpret_cast<WT*>(a.staging.p[p])[(half + static_cast<long long>(me) * n_pad + el) / AR_VEC] = w;
    }
  }
  ar_signal(a, 0, e);
  if (ar_wait(a, 0, e, &s_ok)) {
    const WT* src = reinterpret_cast<const WT*>(a.staging.p[me]) + half / AR_VEC;
    for (long long el = first; el < n_pad; el += step) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int r0 = 0; r0 < world; r0 += W::GROUP) {      // GROUP independent 16/32-byte loads in flight
        WT u[W::GROUP];
#pragma unroll
        for (int r = 0; r < W::GROUP; ++r)
          if (r0 + r < world) u[r] = W::ld(src + (static_cast<long long>(r0 + r) * n_pad + el) / AR_VEC);
#pragma unroll
        for (int r = 0; r < W::GROUP; ++r)
          if (r0 + r < world) {
            float v[8];
            W::to_f32(u[r], v);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += v[i];
          }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] *= a.scale;
      st_grad8(a.grad, el, a.n, acc);
    }
  }
  ar_leave(a, e);
}

}  // namespace

// Bytes of peer-mapped staging / result area and flag ints that rb_allreduce_push needs for vectors of up to n elements.
RB_API long long rb_allreduce_push_staging_bytes(long long n, int world, int wire_bf16) {
  const long long wb = wire_bf16 ? 2 : 4;
  const long long slice = ((n + world - 1) / world + AR_VEC - 1) / AR_VEC * AR_VEC;
  const long long two = slice * world * wb;
  const long long n_pad = (n + AR_VEC - 1) / AR_VEC * AR_VEC;
  const long long one = 2 * n_pad * world * wb;
  return (two > one ? two : one) + 256;
}

RB_API int rb_allreduce_push_max_blocks(void) { return 512; }

// In-place averaged (x scale) all-reduce of the n fp32 values at `grad` on every rank.  staging / result / flags are
// arrays of `world` peer addresses (this rank's view) of areas sized by rb_allreduce_push_staging_bytes (result may
// be null for one_shot) and of an int[2][16][rb_allreduce_push_max_blocks()] flag area zeroed once; epoch_word is
// int[2] local, zeroed once.  Each concurrently running reduction needs its own staging, result, flags and epoch_word.
// `blocks` must be the same on every rank (0 = default).
RB_API int rb_allreduce_push(float* grad, long long n, const unsigned long long* staging,
                             const unsigned long long* result, const unsigned long long* flags, int* epoch_word,
                             float scale, int rank, int world, int wire_bf16, int one_shot, int blocks, int* status,
                             long long timeout_ms, cudaStream_t st) {
  if (world > MAX_RANKS || (n % AR_VEC) || world < 1) return -1;
  if (n == 0) return 0;
  ArArgs a;
  a.grad = grad; a.n = n;
  a.staging = to_ptrs(staging, world);
  a.result = result ? to_ptrs(result, world) : to_ptrs(staging, world);
  a.flags = to_ptrs(flags, world);
  a.epoch_word = epoch_word; a.scale = scale; a.rank = rank; a.world = world; a.status = status;
  a.limit_ns = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
  const long long work = one_shot ? n : ((n + world - 1) / world);
  // threads per block: 512, or 256 (RECSDK_B200_ALLREDUCE_THREADS; must be the same on every rank) for blocks small
  // enough to share an SM with a GEMM CTA of the backward they overlap
  static const int threads = [] {
    const char* e = getenv("RECSDK_B200_ALLREDUCE_THREADS");
    const int t = e ? atoi(e) : AR_THREADS;
    return (t == 256 || t == 128) ? t : AR_THREADS;
  }();
  const long long chunk = static_cast<long long>(threads) * AR_VEC;
  long long want = (work + chunk - 1) / chunk;
  const int cap = blocks > 0 ? blocks : 128 * (AR_THREADS / threads);
  if (want > cap) want = cap;
  if (blocks > 0) want = blocks;             // the grid is part of the flag layout: identical on every rank
  if (want > rb_allreduce_push_max_blocks()) return -1;
  if (want < 1) want = 1;
  const int g = static_cast<int>(want);
  if (one_shot) {
    if (wire_bf16) allreduce_oneshot_kernel<true><<<g, threads, 0, st>>>(a);
    else allreduce_oneshot_kernel<false><<<g, threads, 0, st>>>(a);
  } else {
    if (!result) return -1;
    if (wire_bf16) allreduce_twoshot_kernel<true><<<g, threads, 0, st>>>(a);
    else allreduce_twoshot_kernel<false><<<g, threads, 0, st>>>(a);
  }
  return static_cast<int>(cudaGetLastError());
}
