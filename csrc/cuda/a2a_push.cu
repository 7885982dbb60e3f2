// Push-based sparse exchange over NVLink peer memory: the variable-size all-to-all of a sharded embedding
// lookup, fused with the work on either side of it.
//
// One train step of a sharded embedding collection, seen from rank `me` (W ranks):
//
//   rb_a2a_route         (sample side)  every local id -> (owner rank, key on the owner); per-owner counts; the last
//                        block pushes the count row into every rank's W x W count matrix and raises flag phase 0.
//   rb_a2a_scatter       (sample side)  waits for all count rows, derives from the matrix where this rank's entries
//                        start in every owner's receive list (exclusive prefix over the sources), and STORES
//                        (key, meta) into the owner's list: the receive list of an owner is dense and holds exactly
//                        the ids it owns, O(owned) instead of O(global batch).  Raises flag phase 1.
//   rb_a2a_serve_rows    (owner side)   waits for the payload of all sources, reads each requested row from LOCAL
//                        HBM and stores it straight into the requesting GPU's output: for one-hot features that is
//                        the feature-interaction input [B, sum(D)] (id exchange + gather + pooled-output exchange in
//                        one kernel, with coalesced posted stores over NVLink instead of dependent remote loads),
//                        otherwise a per-id row list that the requester pools or returns as a sequence.
//                        Raises flag phase 2.
//   rb_a2a_push_grads    (sample side, backward)  stores the gradient row of every local id into the owner's
//                        gradient list at the position its key was given in the forward.  Raises flag phase 3.
//   rb_a2a_wait          waits for one phase of all sources (before a consumer that is not one of these kernels).
//
// The owner then sorts its received keys and runs the fused segment-sum + optimizer kernel of embedding.cu over
// local memory only.  Flags carry a per-kernel epoch kept on the device (a captured CUDA graph replays correctly);
// every wait is bounded and reports RB_ERR_PEER_TIMEOUT, a receive list that would overflow reports RB_ERR_CAPACITY
// and the surplus is dropped on every rank consistently.
//
// Counterparts in the reference: the LCCL kernels gather_all.h (row gather fused with all-to-all over a lookup index
// list), all2all.h (variable send_count_matrix) and all2all_uss.h (gradient all-to-all fused with the segment sum),
// cust_op/ascendc_op/ai_core_op/lccl/v220/op_kernel/.
#include "common.cuh"
#include "peer.cuh"
#include "a2a_common.cuh"
#include "tbe_common.cuh"

using namespace rbpeer;
using namespace rbtbe;
using namespace rba2a;

namespace {

// ---------------------------------------------------------------------------------------------
// phase 0: route
// ---------------------------------------------------------------------------------------------
struct RouteArgs {
  const TableShard* shards;       // per feature; nullptr = dynamic keys (owner = key mod world, key kept as is)
  const long long* key_base_all;  // [world][n_tables] first linear key of each table on each rank (static tables)
  const int* feature_table;       // [T]
  int n_tables;
  const void* indices;
  int idx64;
  const long long* offsets;       // [T*B+1] or null (one id per bag)
  int T, B;
  long long nnz;
  int world, me;
  long long* entry_key;           // [nnz]
  long long* entry_meta;          // [nnz]
  int* entry_dst;                 // [nnz]
  int* entry_bag;                 // [nnz] or null
  PeerPtrs ctl;
  int* loc;
  int* status;
};

__global__ void __launch_bounds__(256) a2a_route_kernel(const RouteArgs a) {
  __shared__ int s_cnt[MAX_RANKS];
  if (threadIdx.x < MAX_RANKS) s_cnt[threadIdx.x] = 0;
  const int e = *reinterpret_cast<volatile int*>(a.loc + LOC_EPOCH + 0) + 1;
  __syncthreads();
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long j = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; j < a.nnz; j += stride) {
    long long bag = j;
    if (a.offsets) {
      long long lo = 0, hi = static_cast<long long>(a.T) * a.B;
      while (hi - lo > 1) { const long long mid = (lo + hi) >> 1; if (a.offsets[mid] <= j) lo = mid; else hi = mid; }
      bag = lo;
    }
    const int f = static_cast<int>(bag / a.B);
    const long long id = a.idx64 ? reinterpret_cast<const long long*>(a.indices)[j]
                                 : static_cast<long long>(reinterpret_cast<const int*>(a.indices)[j]);
    int dst = -1;
    long long key = -1;
    if (a.shards) {
      const TableShard ts = a.shards[f];
      int rank; long long row;
      if (locate_row(ts, id, a.world, a.me, rank, row)) {
        dst = rank;
        key = a.key_base_all[static_cast<long long>(rank) * a.n_tables + a.feature_table[f]] + row;
      } else if (a.status) {
        atomicCAS(a.status, 0, RB_ERR_BOUNDS);
      }
    } else {
      dst = static_cast<int>(static_cast<unsigned long long>(id) % static_cast<unsigned long long>(a.world));
      key = id;
    }
    a.entry_key[j] = key;
    a.entry_meta[j] = make_meta(j, f, a.me);
    a.entry_dst[j] = dst;
    if (a.entry_bag) a.entry_bag[j] = static_cast<int>(bag);
    if (dst >= 0) atomicAdd(&s_cnt[dst], 1);
  }
  __syncthreads();
  if (threadIdx.x < a.world && s_cnt[threadIdx.x]) atomicAdd(a.loc + LOC_CNT + threadIdx.x, s_cnt[threadIdx.x]);
  if (is_last_block(a.loc, 0)) {
    // publish this rank's row of the count matrix everywhere, then the flag
    for (int i = threadIdx.x; i < a.world * a.world; i += blockDim.x) {
      const int peer = i / a.world, d = i % a.world;
      const int c = *reinterpret_cast<volatile int*>(a.loc + LOC_CNT + d);
      reinterpret_cast<int*>(a.ctl.p[peer])[CTL_COUNTS + a.me * MAX_RANKS + d] = c;
    }
    __syncthreads();
    if (threadIdx.x < MAX_RANKS) { a.loc[LOC_CNT + threadIdx.x] = 0; a.loc[LOC_CURSOR + threadIdx.x] = 0; }
    signal_all(a.ctl, a.loc, 0, e, a.me, a.world);
  }
}

// ---------------------------------------------------------------------------------------------
// phase 1: scatter the (key, meta) pairs into the owners' receive lists
// ---------------------------------------------------------------------------------------------
struct ScatterArgs {
  const long long* entry_key;
  const long long* entry_meta;
  const int* entry_dst;
  int* entry_pos;                 // [nnz] position in the owner's list (-1: dropped / invalid)
  long long nnz;
  PeerPtrs recv_keys;             // per rank: long long[cap]
  PeerPtrs recv_meta;             // per rank: long long[cap]
  int cap;
  PeerPtrs ctl;
  int* loc;
  int world, me;
  int* status;
  unsigned long long limit_ns;
};

__global__ void __launch_bounds__(256) a2a_scatter_kernel(const ScatterArgs a) {
  __shared__ int s_ok;
  __shared__ int s_base[MAX_RANKS];
  if (threadIdx.x == 0) s_ok = 1;
  const int e_wait = *reinterpret_cast<volatile int*>(a.loc + LOC_EPOCH + 0);
  const int e = *reinterpret_cast<volatile int*>(a.loc + LOC_EPOCH + 1) + 1;
  __syncthreads();
  const int* ctl = reinterpret_cast<const int*>(a.ctl.p[a.me]);
  const bool ok = wait_flags(ctl, 0, e_wait, a.world, a.status, a.limit_ns, &s_ok);
  if (ok) {
    if (threadIdx.x < a.world) {
      const int d = threadIdx.x;
      int base = 0, tot = 0;
      for (int s_ = 0; s_ < a.world; ++s_) {
        const int c = __ldcg(ctl + CTL_COUNTS + s_ * MAX_RANKS + d);
        if (s_ < a.me) base += c;
        tot += c;
      }
      s_base[d] = base;
      if (tot > a.cap && a.status) atomicCAS(a.status, 0, RB_ERR_CAPACITY);
      if (blockIdx.x == 0) a.loc[LOC_BASE + d] = base;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      int run = 0;
      for (int s_ = 0; s_ < a.world; ++s_) {
        a.loc[LOC_SRC_PREFIX + s_] = run;
        run += __ldcg(ctl + CTL_COUNTS + s_ * MAX_RANKS + a.me);
      }
      a.loc[LOC_SRC_PREFIX + a.world] = run;
      a.loc[LOC_N_OWNED] = run < a.cap ? run : a.cap;
    }
    __syncthreads();
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long n_round = (a.nnz + 31) / 32 * 32;          // whole warps stay together for the vote below
    const unsigned lane = threadIdx.x & 31;
    for (long long j = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; j < n_round; j += stride) {
      const int dst = j < a.nnz ? a.entry_dst[j] : -1;
      const unsigned peers = __match_any_sync(0xFFFFFFFFu, dst);
      const int leader = __ffs(peers) - 1;
      int rel0 = 0;
      if (dst >= 0 && static_cast<int>(lane) == leader) rel0 = atomicAdd(a.loc + LOC_CURSOR + dst, __popc(peers));
      rel0 = __shfl_sync(0xFFFFFFFFu, rel0, leader);
      if (j < a.nnz) {
        int pos = -1;
        if (dst >= 0) {
          pos = s_base[dst] + rel0 + __popc(peers & ((1u << lane) - 1u));
          if (pos < a.cap) {
            reinterpret_cast<long long*>(a.recv_keys.p[dst])[pos] = a.entry_key[j];
            reinterpret_cast<long long*>(a.recv_meta.p[dst])[pos] = a.entry_meta[j];
          } else {
            pos = -1;
          }
        }
        a.entry_pos[j] = pos;
      }
    }
  } else {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long j = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; j < a.nnz; j += stride)
      a.entry_pos[j] = -1;
  }
  if (is_last_block(a.loc, 1)) signal_all(a.ctl, a.loc, 1, e, a.me, a.world);
}

// ---------------------------------------------------------------------------------------------
// phase 2 (owner): gather the requested rows from local HBM and store them into the requester's output
// ---------------------------------------------------------------------------------------------
struct ServeArgs {
  const long long* recv_keys;     // local list
  const long long* recv_meta;
  long long* recv_keys_rw;        // same list, for the -1 tail fill
  int cap;
  const long long* key_cumsum;    // [n_tables + 1] this rank's linear key ranges
  const long long* w_offsets;     // [n_tables] element offsets in `weights`
  const int* table_dims;          // [n_tables]
  const int* f_Doff;              // [T] column offset of each feature in the pooled output (one-hot mode)
  int n_tables, T;
  const void* weights;
  PeerPtrs out;                   // per rank: requester's output buffer
  long long ld_out;               // elements between rows of the output
  int one_hot;                    // 1: out[b, Doff[f] ...] with j = f * B + b;  0: out[j, ...]
  int B;
  PeerPtrs ctl;
  int* loc;
  int world, me;
  int* status;
  unsigned long long limit_ns;
};

template <typename WT, typename OT, int G>
__global__ void __launch_bounds__(256) a2a_serve_rows_kernel(const ServeArgs a) {
  extern __shared__ long long sm_serve[];
  __shared__ int s_ok;
  long long* kc = sm_serve;                         // [n_tables + 1]
  long long* wo = kc + a.n_tables + 1;              // [n_tables]
  int* td = reinterpret_cast<int*>(wo + a.n_tables);   // [n_tables]
  int* fo = td + a.n_tables;                        // [T]
  for (int i = threadIdx.x; i <= a.n_tables; i += blockDim.x) kc[i] = a.key_cumsum[i];
  for (int i = threadIdx.x; i < a.n_tables; i += blockDim.x) { wo[i] = a.w_offsets[i]; td[i] = a.table_dims[i]; }
  for (int i = threadIdx.x; i < a.T; i += blockDim.x) fo[i] = a.f_Doff ? a.f_Doff[i] : 0;
  if (threadIdx.x == 0) s_ok = 1;
  const int e_wait = *reinterpret_cast<volatile int*>(a.loc + LOC_EPOCH + 1);
  const int e = *reinterpret_cast<volatile int*>(a.loc + LOC_EPOCH + 2) + 1;
  __syncthreads();
  const int* ctl = reinterpret_cast<const int*>(a.ctl.p[a.me]);
  if (wait_flags(ctl, 1, e_wait, a.world, a.status, a.limit_ns, &s_ok)) {
    const int n = *reinterpret_cast<volatile int*>(a.loc + LOC_N_OWNED);
    // keys beyond the received count read as "not owned" for the sort that follows
    for (int i = n + blockIdx.x * blockDim.x + threadIdx.x; i < a.cap; i += gridDim.x * blockDim.x) a.recv_keys_rw[i] = -1;
    const int hl = threadIdx.x & 15;
    const int halves = gridDim.x * (blockDim.x >> 4);
    const long long total_keys = kc[a.n_tables];
    for (int i0 = (blockIdx.x * (blockDim.x >> 4) + (threadIdx.x >> 4)) * G; i0 < n; i0 += halves * G) {
      const WT* src[G];
      OT* dst[G];
      int D[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        src[g] = nullptr; dst[g] = nullptr; D[g] = 0;
        const int i = i0 + g;
        if (i < n) {
          const long long key = __ldcg(a.recv_keys + i);
          const long long meta = __ldcg(a.recv_meta + i);
          if (key < 0 || key >= total_keys) {
            if (hl == 0 && a.status) atomicCAS(a.status, 0, RB_ERR_BOUNDS);
            continue;
          }
          const int t = table_of(kc, a.n_tables, key);
          D[g] = td[t];
          src[g] = reinterpret_cast<const WT*>(a.weights) + wo[t] + (key - kc[t]) * D[g];
          const int r = meta_src(meta), f = meta_f(meta);
          const long long j = meta & META_J_MASK;
          OT* base = reinterpret_cast<OT*>(a.out.p[r]);
          dst[g] = a.one_hot ? base + (j - static_cast<long long>(f) * a.B) * a.ld_out + fo[f] : base + j * a.ld_out;
        }
      }
      int maxD = 0;
#pragma unroll
      for (int g = 0; g < G; ++g) maxD = D[g] > maxD ? D[g] : maxD;
      for (int d0 = hl * 8; d0 < maxD; d0 += 128) {
        float v[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g)
          if (src[g] && d0 < D[g]) Vec8<WT>::ld(src[g] + d0, v[g]);
#pragma unroll
        for (int g = 0; g < G; ++g)
          if (src[g] && d0 < D[g]) Vec8<OT>::st(dst[g] + d0, v[g]);
      }
    }
  }
  if (is_last_block(a.loc, 2)) signal_all(a.ctl, a.loc, 2, e, a.me, a.world);
}

// ---------------------------------------------------------------------------------------------
// phase 3 (sample side, backward): store each id's gradient row into its owner's gradient list
// ---------------------------------------------------------------------------------------------
struct GradArgs {
  const long long* entry_meta;
  const int* entry_dst;
  const int* entry_pos;
  const int* entry_bag;           // pooled mode: bag of each id (f * B + b)
  const long long* offsets;       // pooled mean: bag offsets
  long long nnz;
  const int* f_D;                 // [T]
  const int* f_Doff;              // [T]
  int T, B;
  int mode;                       // 0: one-hot (j = f*B + b, grad = dout[b, Doff[f]..]); 1: per-id rows (grad = dout[j, ..]);
                                  // 2: pooled (grad = dout[b(bag), Doff[f]..], scaled by 1/len for mean)
  int mean;
  const void* dout;
  long long ld_dout;
  PeerPtrs grad_recv;             // per rank: gradient list, rows of g_ld elements
  long long g_ld;
  PeerPtrs ctl;
  int* loc;
  int world, me;
};

template <typename GT, int G>
__global__ void __launch_bounds__(256) a2a_push_grads_kernel(const GradArgs a) {
  extern __shared__ int sm_grad[];
  int* fD = sm_grad;
  int* fO = fD + a.T;
  for (int i = threadIdx.x; i < a.T; i += blockDim.x) { fD[i] = a.f_D[i]; fO[i] = a.f_Doff ? a.f_Doff[i] : 0; }
  const int e = *reinterpret_cast<volatile int*>(a.loc + LOC_EPOCH + 3) + 1;
  __syncthreads();
  const int hl = threadIdx.x & 15;
  const long long halves = static_cast<long long>(gridDim.x) * (blockDim.x >> 4);
  for (long long j0 = (static_cast<long long>(blockIdx.x) * (blockDim.x >> 4) + (threadIdx.x >> 4)) * G; j0 < a.nnz;
       j0 += halves * G) {
    const GT* src[G];
    GT* dst[G];
    int D[G];
    float scale[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      src[g] = nullptr; dst[g] = nullptr; D[g] = 0; scale[g] = 1.f;
      const long long j = j0 + g;
      if (j < a.nnz) {
        const int pos = a.entry_pos[j];
        if (pos < 0) continue;
        const int f = meta_f(a.entry_meta[j]);
        D[g] = fD[f];
        const GT* base = reinterpret_cast<const GT*>(a.dout);
        if (a.mode == 0) {
          src[g] = base + (j - static_cast<long long>(f) * a.B) * a.ld_dout + fO[f];
        } else if (a.mode == 1) {
          src[g] = base + j * a.ld_dout;
        } else {
          const long long bag = a.entry_bag[j];
          src[g] = base + (bag - static_cast<long long>(f) * a.B) * a.ld_dout + fO[f];
          if (a.mean && a.offsets) {
            const long long len = a.offsets[bag + 1] - a.offsets[bag];
            scale[g] = len > 0 ? 1.f / static_cast<float>(len) : 0.f;
          }
        }
        dst[g] = reinterpret_cast<GT*>(a.grad_recv.p[a.entry_dst[j]]) + static_cast<long long>(pos) * a.g_ld;
      }
    }
    int maxD = 0;
#pragma unroll
    for (int g = 0; g < G; ++g) maxD = D[g] > maxD ? D[g] : maxD;
    for (int d0 = hl * 8; d0 < maxD; d0 += 128) {
      float v[G][8];
#pragma unroll
      for (int g = 0; g < G; ++g)
        if (src[g] && d0 < D[g]) Vec8<GT>::ld(src[g] + d0, v[g]);
#pragma unroll
      for (int g = 0; g < G; ++g)
        if (src[g] && d0 < D[g]) {
          if (scale[g] != 1.f) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[g][i] *= scale[g];
          }
          Vec8<GT>::st(dst[g] + d0, v[g]);
        }
    }
  }
  if (is_last_block(a.loc, 3)) signal_all(a.ctl, a.loc, 3, e, a.me, a.world);
}

__global__ void a2a_wait_kernel(PeerPtrs ctl, int* loc, int phase, int world, int me, int* status,
                                unsigned long long limit_ns) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  const int e = *reinterpret_cast<volatile int*>(loc + LOC_EPOCH + phase);
  __syncthreads();
  wait_flags(reinterpret_cast<const int*>(ctl.p[me]), phase, e, world, status, limit_ns, &s_ok);
}

// Requester side, variable-length bags: pooled[b, Doff[f] ..] = sum (or mean) of the per-id rows of bag (f, b), which the
// owners stored into rows[j, :D] in id order.  One half-warp per bag, fp32 accumulation.
template <typename RT, typename OT>
__global__ void __launch_bounds__(256) pool_rows_kernel(const RT* __restrict__ rows, long long ld_rows,
                                                        const long long* __restrict__ offsets, int T, int B,
                                                        const int* __restrict__ f_D, const int* __restrict__ f_Doff,
                                                        int mean, OT* __restrict__ out, long long ld_out) {
  const int hl = threadIdx.x & 15;
  const long long bag = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  if (bag >= static_cast<long long>(T) * B) return;
  const int f = static_cast<int>(bag / B);
  const int b = static_cast<int>(bag - static_cast<long long>(f) * B);
  const int D = f_D[f];
  const long long beg = offsets[bag], end = offsets[bag + 1];
  const float inv = (mean && end > beg) ? 1.f / static_cast<float>(end - beg) : 1.f;
  for (int d0 = hl * 8; d0 < D; d0 += 128) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (long long j = beg; j < end; ++j) {
      float v[8];
      Vec8<RT>::ld(rows + j * ld_rows + d0, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= inv;
    Vec8<OT>::st(out + static_cast<long long>(b) * ld_out + f_Doff[f] + d0, acc);
  }
}

inline int grid_for(long long work_items, int per_block, int num_sms, int per_sm) {
  long long b = (work_items + per_block - 1) / per_block;
  const long long cap = static_cast<long long>(num_sms > 0 ? num_sms : 148) * per_sm;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace

// Sizes (in ints) of the peer-mapped control block and of the local state block; both zeroed once.
RB_API int rb_a2a_ctl_ints(void) { return CTL_INTS; }
RB_API int rb_a2a_loc_ints(void) { return LOC_INTS; }
// index of the "entries in my receive list" word inside the local state block
RB_API int rb_a2a_loc_n_owned_index(void) { return LOC_N_OWNED; }

RB_API int rb_a2a_route(const void* shards, const long long* key_base_all, const int* feature_table, int n_tables,
                        const void* indices, int idx64, const long long* offsets, int T, int B, long long nnz,
                        int world, int me, long long* entry_key, long long* entry_meta, int* entry_dst,
                        int* entry_bag, const unsigned long long* ctl, int* loc, int num_sms, int* status,
                        cudaStream_t st) {
  if (world > MAX_RANKS || T >= 65536 || nnz > META_J_MASK) return -1;
  RouteArgs a;
  a.shards = reinterpret_cast<const TableShard*>(shards);
  a.key_base_all = key_base_all; a.feature_table = feature_table; a.n_tables = n_tables;
  a.indices = indices; a.idx64 = idx64; a.offsets = offsets; a.T = T; a.B = B; a.nnz = nnz;
  a.world = world; a.me = me; a.entry_key = entry_key; a.entry_meta = entry_meta; a.entry_dst = entry_dst;
  a.entry_bag = entry_bag; a.ctl = to_ptrs(ctl, world); a.loc = loc; a.status = status;
  a2a_route_kernel<<<grid_for(nnz, 256, num_sms, 8), 256, 0, st>>>(a);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_a2a_scatter(const long long* entry_key, const long long* entry_meta, const int* entry_dst,
                          int* entry_pos, long long nnz, const unsigned long long* recv_keys,
                          const unsigned long long* recv_meta, int cap, const unsigned long long* ctl, int* loc,
                          int world, int me, int num_sms, int* status, long long timeout_ms, cudaStream_t st) {
  if (world > MAX_RANKS) return -1;
  ScatterArgs a;
  a.entry_key = entry_key; a.entry_meta = entry_meta; a.entry_dst = entry_dst; a.entry_pos = entry_pos; a.nnz = nnz;
  a.recv_keys = to_ptrs(recv_keys, world); a.recv_meta = to_ptrs(recv_meta, world); a.cap = cap;
  a.ctl = to_ptrs(ctl, world); a.loc = loc; a.world = world; a.me = me; a.status = status;
  a.limit_ns = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
  a2a_scatter_kernel<<<grid_for(nnz, 256, num_sms, 8), 256, 0, st>>>(a);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_a2a_serve_rows(const long long* recv_keys, const long long* recv_meta, int cap,
                             const long long* key_cumsum, const long long* w_offsets, const int* table_dims,
                             const int* f_Doff, int n_tables, int T, const void* weights, int w_dtype,
                             const unsigned long long* out_ptrs, int out_dtype, long long ld_out, int one_hot, int B,
                             const unsigned long long* ctl, int* loc, int world, int me, int num_sms, int* status,
                             long long timeout_ms, cudaStream_t st) {
  if (world > MAX_RANKS) return -1;
  ServeArgs a;
  a.recv_keys = recv_keys; a.recv_meta = recv_meta; a.recv_keys_rw = const_cast<long long*>(recv_keys); a.cap = cap;
  a.key_cumsum = key_cumsum; a.w_offsets = w_offsets; a.table_dims = table_dims; a.f_Doff = f_Doff;
  a.n_tables = n_tables; a.T = T; a.weights = weights; a.out = to_ptrs(out_ptrs, world); a.ld_out = ld_out;
  a.one_hot = one_hot; a.B = B; a.ctl = to_ptrs(ctl, world); a.loc = loc; a.world = world; a.me = me;
  a.status = status; a.limit_ns = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
  const size_t smem = sizeof(long long) * (2 * static_cast<size_t>(n_tables) + 1) + sizeof(int) * (n_tables + T) + 16;
  if (smem > 48 * 1024) return -6;
  constexpr int G = 4;
  const int grid = grid_for((static_cast<long long>(cap) + G - 1) / G, 16, num_sms, 8);
#define RB_SERVE(WT_, OT_) a2a_serve_rows_kernel<WT_, OT_, G><<<grid, 256, smem, st>>>(a)
  switch (w_dtype * 3 + out_dtype) {
    case DT_F32 * 3 + DT_F32: RB_SERVE(float, float); break;
    case DT_F32 * 3 + DT_F16: RB_SERVE(float, __half); break;
    case DT_F32 * 3 + DT_BF16: RB_SERVE(float, __nv_bfloat16); break;
    case DT_F16 * 3 + DT_F32: RB_SERVE(__half, float); break;
    case DT_F16 * 3 + DT_F16: RB_SERVE(__half, __half); break;
    case DT_F16 * 3 + DT_BF16: RB_SERVE(__half, __nv_bfloat16); break;
    case DT_BF16 * 3 + DT_F32: RB_SERVE(__nv_bfloat16, float); break;
    case DT_BF16 * 3 + DT_F16: RB_SERVE(__nv_bfloat16, __half); break;
    case DT_BF16 * 3 + DT_BF16: RB_SERVE(__nv_bfloat16, __nv_bfloat16); break;
    default: return -1;
  }
#undef RB_SERVE
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_a2a_push_grads(const long long* entry_meta, const int* entry_dst, const int* entry_pos,
                             const int* entry_bag, const long long* offsets, long long nnz, const int* f_D,
                             const int* f_Doff, int T, int B, int mode, int mean, const void* dout, int g_dtype,
                             long long ld_dout, const unsigned long long* grad_recv, long long g_ld,
                             const unsigned long long* ctl, int* loc, int world, int me, int num_sms,
                             cudaStream_t st) {
  if (world > MAX_RANKS || (mode == 2 && !entry_bag)) return -1;
  GradArgs a;
  a.entry_meta = entry_meta; a.entry_dst = entry_dst; a.entry_pos = entry_pos; a.entry_bag = entry_bag;
  a.offsets = offsets; a.nnz = nnz; a.f_D = f_D; a.f_Doff = f_Doff; a.T = T; a.B = B; a.mode = mode; a.mean = mean;
  a.dout = dout; a.ld_dout = ld_dout; a.grad_recv = to_ptrs(grad_recv, world); a.g_ld = g_ld;
  a.ctl = to_ptrs(ctl, world); a.loc = loc; a.world = world; a.me = me;
  constexpr int G = 4;
  const int grid = grid_for((nnz + G - 1) / G, 16, num_sms, 8);
  const size_t smem = sizeof(int) * 2 * static_cast<size_t>(T) + 16;
  if (smem > 48 * 1024) return -6;
  switch (g_dtype) {
    case DT_F32: a2a_push_grads_kernel<float, G><<<grid, 256, smem, st>>>(a); break;
    case DT_F16: a2a_push_grads_kernel<__half, G><<<grid, 256, smem, st>>>(a); break;
    case DT_BF16: a2a_push_grads_kernel<__nv_bfloat16, G><<<grid, 256, smem, st>>>(a); break;
    default: return -1;
  }
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_a2a_wait(const unsigned long long* ctl, int* loc, int phase, int world, int me, int* status,
                       long long timeout_ms, cudaStream_t st) {
  if (world > MAX_RANKS || phase < 0 || phase >= A2A_PHASES) return -1;
  a2a_wait_kernel<<<1, 32, 0, st>>>(to_ptrs(ctl, world), loc, phase, world, me, status,
                                    static_cast<unsigned long long>(timeout_ms) * 1000000ull);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_pool_rows(const void* rows, int rows_dtype, long long ld_rows, const long long* offsets, int T, int B,
                        const int* f_D, const int* f_Doff, int mean, void* out, int out_dtype, long long ld_out,
                        cudaStream_t st) {
  const long long bags = static_cast<long long>(T) * B;
  if (bags == 0) return 0;
  const long long blocks = (bags * 16 + 255) / 256;
#define RB_POOL(RT_, OT_) pool_rows_kernel<RT_, OT_><<<blocks, 256, 0, st>>>(                                       \
      reinterpret_cast<const RT_*>(rows), ld_rows, offsets, T, B, f_D, f_Doff, mean, reinterpret_cast<OT_*>(out), ld_out)
  switch (rows_dtype * 3 + out_dtype) {
    case DT_F32 * 3 + DT_F32: RB_POOL(float, float); break;
    case DT_F32 * 3 + DT_F16: RB_POOL(float, __half); break;
    case DT_F32 * 3 + DT_BF16: RB_POOL(float, __nv_bfloat16); break;
    case DT_F16 * 3 + DT_F32: RB_POOL(__half, float); break;
    case DT_F16 * 3 + DT_F16: RB_POOL(__half, __half); break;
    case DT_F16 * 3 + DT_BF16: RB_POOL(__half, __nv_bfloat16); break;
    case DT_BF16 * 3 + DT_F32: RB_POOL(__nv_bfloat16, float); break;
    case DT_BF16 * 3 + DT_F16: RB_POOL(__nv_bfloat16, __half); break;
    case DT_BF16 * 3 + DT_BF16: RB_POOL(__nv_bfloat16, __nv_bfloat16); break;
    default: return -1;
  }
#undef RB_POOL
  return static_cast<int>(cudaGetLastError());
}
