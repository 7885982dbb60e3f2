// Table-batched embedding kernels for sm_100a.
//
//  * rb_tbe_forward       pooled (sum/mean) or per-id lookup over many tables in one launch.
//                         Each table is described by a TableShard record; its rows may live on
//                         this GPU or on a peer GPU (NVLink peer pointers), sharded table-wise,
//                         row-wise (round-robin or block) or replicated.  The kernel pulls rows
//                         straight from the owner's HBM and writes the pooled result into the
//                         caller's feature-interaction input buffer, so the id exchange and the
//                         pooled-embedding exchange of a classic sharded lookup never exist.
//  * rb_tbe_linearize     (table,id) -> one sortable row key + bag id.
//  * rb_sort_segments     radix sort + run-length encode (CUB) -> unique rows and their segments.
//  * rb_tbe_backward_update  per unique row: sum the gradients of every bag that used it
//                         (reading them from whichever GPU holds that sample), then apply
//                         SGD / Adagrad / row-wise Adagrad / Adam in place.  This is the
//                         gradient exchange + dedup/segment-sum + sparse update in one kernel.
//
// Semantics follow FBGEMM's "exact" table-batched embedding as adopted by the reference
// (cust_op/ascendc_op/ai_core_op/recops_backward_codegen_adagrad_unweighted_exact/v220/README.md,
//  cust_op/framework/torch_plugin/torch_library/split_embedding_codegen_forward_unweighted/).
#include <cub/cub.cuh>

#include <cstdlib>

#include "common.cuh"
#include "tbe_common.cuh"

using namespace rbtbe;

namespace {

// ---------------------------------------------------------------------------
// forward: one warp per bag (pooled) or per id (POOL_NONE)
// ---------------------------------------------------------------------------
template <typename WT, typename OT, typename IT>
__global__ void tbe_forward_kernel(const TableShard* __restrict__ shards, const long long* __restrict__ ptrs,
                                   const IT* __restrict__ indices, const long long* __restrict__ offsets,
                                   int T, int B, int world, int self, int pooling, OT* __restrict__ out,
                                   long long ld_out, int* status) {
  const long long warp_global = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long n_bags = static_cast<long long>(T) * B;
  if (warp_global >= n_bags) return;
  const int t = static_cast<int>(warp_global / B);
  const int b = static_cast<int>(warp_global % B);
  const TableShard ts = shards[t];
  long long beg, end;
  if (offsets) { beg = offsets[warp_global]; end = offsets[warp_global + 1]; }
  else { beg = warp_global; end = warp_global + 1; }
  OT* o = out + static_cast<long long>(b) * ld_out + ts.D_offset;
  for (int d0 = lane * 4; d0 < ts.D; d0 += 128) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long j = beg; j < end; ++j) {
      const long long id = static_cast<long long>(indices[j]);
      int rank; long long row;
      if (!locate_row(ts, id, world, self, rank, row)) {
        if (lane == 0 && status) atomicCAS(status, 0, RB_ERR_BOUNDS);
        continue;
      }
      const WT* base = reinterpret_cast<const WT*>(ptrs[ts.ptr_index + rank]);
      const float4 v = Ld4<WT>::ld(base + row * ts.D + d0);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (pooling == POOL_MEAN && end > beg) {
      const float inv = 1.f / static_cast<float>(end - beg);
      acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    }
    Ld4<OT>::st(o + d0, acc);
  }
}

// per-id (sequence) lookup: out[j, :D] = row(indices[j]); table of position j given by a
// per-table range array pos_offsets[T+1] (positions are grouped by table).
template <typename WT, typename OT, typename IT>
__global__ void tbe_sequence_kernel(const TableShard* __restrict__ shards, const long long* __restrict__ ptrs,
                                    const IT* __restrict__ indices, const long long* __restrict__ pos_offsets,
                                    int T, long long nnz, int world, int self, OT* __restrict__ out,
                                    long long ld_out, int* status) {
  const long long j = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (j >= nnz) return;
  int lo = 0, hi = T;  // last t with pos_offsets[t] <= j
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (pos_offsets[mid] <= j) lo = mid; else hi = mid; }
  const TableShard ts = shards[lo];
  const long long id = static_cast<long long>(indices[j]);
  int rank; long long row;
  OT* o = out + j * ld_out;
  if (!locate_row(ts, id, world, self, rank, row)) {
    if (lane == 0 && status) atomicCAS(status, 0, RB_ERR_BOUNDS);
    for (int d0 = lane * 4; d0 < ts.D; d0 += 128) Ld4<OT>::st(o + d0, make_float4(0.f, 0.f, 0.f, 0.f));
    return;
  }
  const WT* base = reinterpret_cast<const WT*>(ptrs[ts.ptr_index + rank]);
  for (int d0 = lane * 4; d0 < ts.D; d0 += 128) Ld4<OT>::st(o + d0, Ld4<WT>::ld(base + row * ts.D + d0));
}

// ---------------------------------------------------------------------------
// linearize: key = key_base + local row on the owner; only ids this rank owns are kept (others
// get key = -1; the sort looks at the low key bits only, so they land in one run at the end, which
// the update kernel skips).
// ---------------------------------------------------------------------------
template <typename IT>
__global__ void tbe_linearize_kernel(const TableShard* __restrict__ shards, const IT* __restrict__ indices,
                                     const long long* __restrict__ offsets, int T, int B, long long nnz,
                                     int world, int self, long long* __restrict__ keys,
                                     int* __restrict__ bags) {
  const long long j = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j >= nnz) return;
  long long bag;
  if (offsets) {
    long long lo = 0, hi = static_cast<long long>(T) * B;
    while (hi - lo > 1) { const long long mid = (lo + hi) >> 1; if (offsets[mid] <= j) lo = mid; else hi = mid; }
    bag = lo;
  } else {
    bag = j;
  }
  const int t = static_cast<int>(bag / B);
  const TableShard ts = shards[t];
  int rank; long long row;
  long long key = -1;
  if (locate_row(ts, static_cast<long long>(indices[j]), world, self, rank, row) && rank == self)
    key = ts.key_base + row;
  keys[j] = key;
  bags[j] = static_cast<int>(bag);
}

// ---------------------------------------------------------------------------
// one-hot fast forward: a half-warp per bag with 16-byte loads, G bags in flight per half-warp
// ---------------------------------------------------------------------------
template <typename WT, typename OT, typename IT, int G>
__global__ void __launch_bounds__(256)
tbe_forward_onehot_kernel(const TableShard* __restrict__ shards, const long long* __restrict__ ptrs,
                          const IT* __restrict__ indices, int T, int B, int world, int self,
                          OT* __restrict__ out, long long ld_out, int* status) {
  const int hl = threadIdx.x & 15;
  const long long half_id = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  const int groups_per_t = (B + G - 1) / G;
  if (half_id >= static_cast<long long>(T) * groups_per_t) return;
  const int t = static_cast<int>(half_id / groups_per_t);
  const int b0 = static_cast<int>(half_id % groups_per_t) * G;
  const TableShard ts = shards[t];
  const WT* src[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    src[g] = nullptr;
    if (b0 + g < B) {
      const long long id = static_cast<long long>(indices[static_cast<long long>(t) * B + b0 + g]);
      int rank; long long row;
      if (locate_row(ts, id, world, self, rank, row))
        src[g] = reinterpret_cast<const WT*>(ptrs[ts.ptr_index + rank]) + row * ts.D;
      else if (hl == 0 && status) atomicCAS(status, 0, RB_ERR_BOUNDS);
    }
  }
  for (int d0 = hl * 8; d0 < ts.D; d0 += 128) {
    float v[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (src[g]) Vec8<WT>::ld(src[g] + d0, v[g]);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[g][i] = 0.f;
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g)
      if (b0 + g < B) Vec8<OT>::st(out + static_cast<long long>(b0 + g) * ld_out + ts.D_offset + d0, v[g]);
  }
}

// ---------------------------------------------------------------------------
// backward + optimizer
// ---------------------------------------------------------------------------
struct OptArgs {
  int type;
  float lr, eps, beta1, beta2, weight_decay;
  float bias_c1, bias_c2;  // 1-beta1^t, 1-beta2^t
};

constexpr int LONG_CHUNK = 32;   // entries summed by one half-warp of the long-segment kernel

struct BwdArgs {
  const TableShard* shards;
  const long long* key_cumsum;   // [n_tables+1] linear key range of each table on this rank
  const long long* w_offsets;    // [n_tables] element offset of each table in `weights`
  const long long* s_offsets;    // [n_tables] offset of each table in the state arrays (rows or elements)
  int T, n_tables, B_local, world;   // T = features (bag groups); n_tables = physical tables
  const long long* grad_ptrs;    // [world] base of each rank's pooled-gradient buffer
  long long ld_g;
  const long long* offsets;      // bag offsets for mean pooling (nullable), over the global bag index
  int pooling;
  const int* sorted_bags;        // bag index (f * B_global + b_global)
  const long long* unique_keys;
  const int* seg_offsets;        // [num_runs + 1]
  const int* num_runs;
  void* weights;
  float* state1;
  float* state2;
  OptArgs opt;
  // long-segment machinery (scratch)
  int* long_list;      // [long_cap] segment index of each long segment
  int* counters;       // [0] = number of long segments, [1] = number of chunks
  int2* chunk_list;    // [chunk_cap] (long index, chunk index)
  float* long_accum;   // [long_cap][accum_ld] fp32 partial sums, all zero between launches
  int long_cap, chunk_cap, accum_ld, long_threshold;
  int* status;
  // direct mode (push exchange): the gradient row of sorted entry j is direct_rows + sorted_bags[j] * direct_ld,
  // in local memory; table_dims[n_tables] gives the row width
  const void* direct_rows;
  long long direct_ld;
  const int* table_dims;
};

// per-kernel shared-memory copy of the small lookup tables
struct Tabs {
  const long long* key_cumsum;
  const long long* w_off;
  const long long* s_off;
  const long long* gptr;
  const int* f_D;
  const int* f_Doff;
};

__device__ __forceinline__ Tabs load_tabs(const BwdArgs& a, long long* sm) {
  long long* kc = sm;
  long long* wo = kc + a.n_tables + 1;
  long long* so = wo + a.n_tables;
  long long* gp = so + a.n_tables;
  int* fD = reinterpret_cast<int*>(gp + a.world);
  int* fO = fD + a.T;
  for (int i = threadIdx.x; i <= a.n_tables; i += blockDim.x) kc[i] = a.key_cumsum[i];
  for (int i = threadIdx.x; i < a.n_tables; i += blockDim.x) { wo[i] = a.w_offsets[i]; so[i] = a.s_offsets[i]; }
  for (int i = threadIdx.x; i < a.world; i += blockDim.x) gp[i] = a.grad_ptrs[i];
  for (int i = threadIdx.x; i < a.T; i += blockDim.x) { fD[i] = a.shards[i].D; fO[i] = a.shards[i].D_offset; }
  __syncthreads();
  return Tabs{kc, wo, so, gp, fD, fO};
}

inline size_t tabs_bytes(int n_tables, int T, int world) {
  return sizeof(long long) * (3 * static_cast<size_t>(n_tables) + 1 + world) + sizeof(int) * 2 * static_cast<size_t>(T) + 16;
}

__device__ __forceinline__ int table_of_key(const long long* cumsum, int n, long long key) {
  int lo = 0, hi = n;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (cumsum[mid] <= key) lo = mid; else hi = mid; }
  return lo;
}

__device__ __forceinline__ float half_sum(float v, unsigned mask) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(mask, v, o, 16);
  return v;
}

// sum the gradient rows of entries [beg, end) into acc; 4 rows in flight per half-warp
template <typename GT, int NCH>
__device__ __forceinline__ void accumulate_range(const BwdArgs& a, const Tabs& tb, int D, int beg, int end,
                                                 unsigned B_global, float (&acc)[NCH][8], int hl) {
  for (int j = beg; j < end; j += 4) {
    const GT* g[4];
    float scale[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      g[u] = nullptr;
      scale[u] = 1.f;
      if (j + u < end && a.direct_rows) {
        g[u] = reinterpret_cast<const GT*>(a.direct_rows) + static_cast<long long>(a.sorted_bags[j + u]) * a.direct_ld + hl * 8;
      } else if (j + u < end) {
        const unsigned bag = static_cast<unsigned>(a.sorted_bags[j + u]);
        const unsigned f = bag / B_global;
        const unsigned bg = bag - f * B_global;
        const unsigned r = bg / static_cast<unsigned>(a.B_local);
        const unsigned bl = bg - r * static_cast<unsigned>(a.B_local);
        g[u] = reinterpret_cast<const GT*>(tb.gptr[r]) + static_cast<long long>(bl) * a.ld_g + tb.f_Doff[f] + hl * 8;
        if (a.pooling == POOL_MEAN && a.offsets) {
          const long long len = a.offsets[bag + 1] - a.offsets[bag];
          scale[u] = len > 0 ? 1.f / static_cast<float>(len) : 0.f;
        }
      }
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      if (hl * 8 + c * 128 >= D) continue;
      float v[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (g[u]) Vec8<GT>::ld(g[u] + c * 128, v[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (g[u]) {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[c][i] += v[u][i] * scale[u];
        }
    }
  }
}

// The row's weights (and its row-wise state) are loaded by the caller BEFORE it sums the gradients,
// so those loads overlap the gradient gathers instead of extending the dependent chain.
template <typename WT, int NCH>
__device__ __forceinline__ void preload_row(const BwdArgs& a, const Tabs& tb, int t, long long local_row, int D,
                                            float (&wv)[NCH][8], float& row_state, int hl) {
  const WT* w = reinterpret_cast<const WT*>(a.weights) + tb.w_off[t] + local_row * D;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int d0 = hl * 8 + c * 128;
    if (d0 < D) Vec8<WT>::ld(w + d0, wv[c]);
  }
  row_state = (a.opt.type == OPT_ROWWISE_ADAGRAD) ? a.state1[tb.s_off[t] + local_row] : 0.f;
}

template <typename WT, int NCH>
__device__ __forceinline__ void apply_row_update(const BwdArgs& a, const Tabs& tb, int t, long long local_row, int D,
                                                 float (&acc)[NCH][8], float (&wpre)[NCH][8], float row_state,
                                                 int hl, unsigned hmask) {
  WT* w = reinterpret_cast<WT*>(a.weights) + tb.w_off[t] + local_row * D;
  const OptArgs& o = a.opt;
  if (o.type == OPT_ROWWISE_ADAGRAD) {
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c)
      if (hl * 8 + c * 128 < D) {
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += acc[c][i] * acc[c][i];
      }
    ss = half_sum(ss, hmask);
    const float g2 = row_state + ss / static_cast<float>(D);
    if (hl == 0) a.state1[tb.s_off[t] + local_row] = g2;
    const float mult = o.lr / (sqrtf(g2) + o.eps);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int d0 = hl * 8 + c * 128;
      if (d0 < D) {
#pragma unroll
        for (int i = 0; i < 8; ++i) wpre[c][i] -= mult * acc[c][i];
        Vec8<WT>::st(w + d0, wpre[c]);
      }
    }
    return;
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int d0 = hl * 8 + c * 128;
    if (d0 >= D) continue;
    float (&wv)[8] = wpre[c];
    if (o.type == OPT_SGD) {
#pragma unroll
      for (int i = 0; i < 8; ++i) wv[i] -= o.lr * (acc[c][i] + o.weight_decay * wv[i]);
    } else if (o.type == OPT_ADAGRAD) {
      float* st = a.state1 + tb.s_off[t] + local_row * D + d0;
      float sv[8];
      Vec8<float>::ld(st, sv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sv[i] += acc[c][i] * acc[c][i];
        wv[i] -= o.lr * acc[c][i] / (sqrtf(sv[i]) + o.eps);
      }
      Vec8<float>::st(st, sv);
    } else {  // Adam
      float* m = a.state1 + tb.s_off[t] + local_row * D + d0;
      float* vv = a.state2 + tb.s_off[t] + local_row * D + d0;
      float mv[8], vs[8];
      Vec8<float>::ld(m, mv);
      Vec8<float>::ld(vv, vs);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float gi = acc[c][i] + o.weight_decay * wv[i];
        mv[i] = o.beta1 * mv[i] + (1.f - o.beta1) * gi;
        vs[i] = o.beta2 * vs[i] + (1.f - o.beta2) * gi * gi;
        wv[i] -= (o.lr / o.bias_c1) * mv[i] / (sqrtf(vs[i] / o.bias_c2) + o.eps);
      }
      Vec8<float>::st(m, mv);
      Vec8<float>::st(vv, vs);
    }
    Vec8<WT>::st(w + d0, wv);
  }
}

// (1) one half-warp per unique row; segments longer than long_threshold are split into chunks of
//     LONG_CHUNK entries and queued for kernels (2) and (3).
template <typename WT, typename GT, int NCH, int MINB>
__global__ void __launch_bounds__(256, MINB) tbe_bwd_short_kernel(const BwdArgs a) {
  extern __shared__ long long sm_tabs[];
  const Tabs tb = load_tabs(a, sm_tabs);
  const int hl = threadIdx.x & 15;
  const unsigned hmask = (threadIdx.x & 16) ? 0xFFFF0000u : 0x0000FFFFu;
  const int groups_total = gridDim.x * (blockDim.x >> 4);
  const int n = *a.num_runs;
  const unsigned B_global = static_cast<unsigned>(a.B_local) * static_cast<unsigned>(a.world);
  for (int s = blockIdx.x * (blockDim.x >> 4) + (threadIdx.x >> 4); s < n; s += groups_total) {
    const long long key = a.unique_keys[s];
    if (key < 0) continue;
    const int beg = a.seg_offsets[s], end = a.seg_offsets[s + 1];
    const int len = end - beg;
    if (len > a.long_threshold) {
      int li = 0, base = 0;
      const int nch = (len + LONG_CHUNK - 1) / LONG_CHUNK;
      if (hl == 0) {
        li = atomicAdd(a.counters, 1);
        if (li < a.long_cap) {
          a.long_list[li] = s;
          base = atomicAdd(a.counters + 1, nch);
        } else if (a.status) {
          atomicCAS(a.status, 0, RB_ERR_CAPACITY);
        }
      }
      li = __shfl_sync(hmask, li, threadIdx.x & 16);
      base = __shfl_sync(hmask, base, threadIdx.x & 16);
      if (li < a.long_cap) {
        for (int c = hl; c < nch; c += 16) {
          if (base + c < a.chunk_cap) a.chunk_list[base + c] = make_int2(li, c);
          else if (a.status) atomicCAS(a.status, 0, RB_ERR_CAPACITY);
        }
      }
      continue;
    }
    const int t = table_of_key(tb.key_cumsum, a.n_tables, key);
    const int D = a.direct_rows ? a.table_dims[t] : tb.f_D[static_cast<unsigned>(a.sorted_bags[beg]) / B_global];
    float acc[NCH][8], wpre[NCH][8], row_state;
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[c][i] = 0.f;
    preload_row<WT, NCH>(a, tb, t, key - tb.key_cumsum[t], D, wpre, row_state, hl);
    accumulate_range<GT, NCH>(a, tb, D, beg, end, B_global, acc, hl);
    apply_row_update<WT, NCH>(a, tb, t, key - tb.key_cumsum[t], D, acc, wpre, row_state, hl, hmask);
  }
}

// (2) one half-warp per chunk of a long segment: partial sum -> fp32 atomics into the segment's scratch row
template <typename GT, int NCH>
__global__ void __launch_bounds__(256) tbe_bwd_long_chunk_kernel(const BwdArgs a) {
  extern __shared__ long long sm_tabs[];
  const Tabs tb = load_tabs(a, sm_tabs);
  const int hl = threadIdx.x & 15;
  const int groups_total = gridDim.x * (blockDim.x >> 4);
  int n_chunks = a.counters[1];
  if (n_chunks > a.chunk_cap) n_chunks = a.chunk_cap;
  const unsigned B_global = static_cast<unsigned>(a.B_local) * static_cast<unsigned>(a.world);
  for (int ci = blockIdx.x * (blockDim.x >> 4) + (threadIdx.x >> 4); ci < n_chunks; ci += groups_total) {
    const int2 item = a.chunk_list[ci];
    const int s = a.long_list[item.x];
    const int seg_beg = a.seg_offsets[s], seg_end = a.seg_offsets[s + 1];
    const int beg = seg_beg + item.y * LONG_CHUNK;
    const int end = min(seg_end, beg + LONG_CHUNK);
    const int D = a.direct_rows ? a.table_dims[table_of_key(tb.key_cumsum, a.n_tables, a.unique_keys[s])]
                                : tb.f_D[static_cast<unsigned>(a.sorted_bags[seg_beg]) / B_global];
    float acc[NCH][8];
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[c][i] = 0.f;
    accumulate_range<GT, NCH>(a, tb, D, beg, end, B_global, acc, hl);
    float* dst = a.long_accum + static_cast<long long>(item.x) * a.accum_ld;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int d0 = hl * 8 + c * 128;
      if (d0 < D) {
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(dst + d0 + i, acc[c][i]);
      }
    }
  }
}

// (3) one half-warp per long segment: read its scratch row, clear it for the next launch, update
template <typename WT, int NCH>
__global__ void __launch_bounds__(256) tbe_bwd_long_final_kernel(const BwdArgs a) {
  extern __shared__ long long sm_tabs[];
  const Tabs tb = load_tabs(a, sm_tabs);
  const int hl = threadIdx.x & 15;
  const unsigned hmask = (threadIdx.x & 16) ? 0xFFFF0000u : 0x0000FFFFu;
  const int groups_total = gridDim.x * (blockDim.x >> 4);
  int n_long = a.counters[0];
  if (n_long > a.long_cap) n_long = a.long_cap;
  const unsigned B_global = static_cast<unsigned>(a.B_local) * static_cast<unsigned>(a.world);
  for (int li = blockIdx.x * (blockDim.x >> 4) + (threadIdx.x >> 4); li < n_long; li += groups_total) {
    const int s = a.long_list[li];
    const long long key = a.unique_keys[s];
    const int t = table_of_key(tb.key_cumsum, a.n_tables, key);
    const int D = a.direct_rows ? a.table_dims[t] : tb.f_D[static_cast<unsigned>(a.sorted_bags[a.seg_offsets[s]]) / B_global];
    float* src = a.long_accum + static_cast<long long>(li) * a.accum_ld;
    float acc[NCH][8], wpre[NCH][8], row_state;
    preload_row<WT, NCH>(a, tb, t, key - tb.key_cumsum[t], D, wpre, row_state, hl);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int d0 = hl * 8 + c * 128;
      if (d0 < D) {
        Vec8<float>::ld(src + d0, acc[c]);
        const float z[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        Vec8<float>::st(src + d0, z);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[c][i] = 0.f;
      }
    }
    apply_row_update<WT, NCH>(a, tb, t, key - tb.key_cumsum[t], D, acc, wpre, row_state, hl, hmask);
  }
}

template <typename WT, typename GT, int NCH>
int launch_bwd(const BwdArgs& a, int max_runs, int num_sms, cudaStream_t st) {
  const size_t smem = tabs_bytes(a.n_tables, a.T, a.world);
  if (smem > 48 * 1024) return -6;
  int blocks = (max_runs + 15) / 16;
  const int cap = num_sms * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  // resident CTAs per SM the kernel is compiled for: the kernel is bound by the latency of its dependent loads, so more
  // half-warps in flight beat a spill-free register allocation (measured 2.94 -> 2.80 ms per DLRM-large step from 2 to 4);
  // RECSDK_B200_TBE_BWD_MINB = 2 | 3 | 4 overrides it for tuning
  static const int minb = [] { const char* e = getenv("RECSDK_B200_TBE_BWD_MINB"); return e ? atoi(e) : 4; }();
  if (blocks == cap) blocks = num_sms * (minb >= 4 ? 16 : (minb == 3 ? 12 : 8));
  if (blocks > (max_runs + 15) / 16) blocks = (max_runs + 15) / 16;
  if (minb >= 4) tbe_bwd_short_kernel<WT, GT, NCH, 4><<<blocks, 256, smem, st>>>(a);
  else if (minb == 3) tbe_bwd_short_kernel<WT, GT, NCH, 3><<<blocks, 256, smem, st>>>(a);
  else tbe_bwd_short_kernel<WT, GT, NCH, 2><<<blocks, 256, smem, st>>>(a);
  tbe_bwd_long_chunk_kernel<GT, NCH><<<num_sms * 4, 256, smem, st>>>(a);
  tbe_bwd_long_final_kernel<WT, NCH><<<num_sms, 256, smem, st>>>(a);
  return static_cast<int>(cudaGetLastError());
}

template <typename WT, typename GT>
int dispatch_nch(const BwdArgs& a, int max_D, int max_runs, int num_sms, cudaStream_t st) {
  if (max_D <= 128) return launch_bwd<WT, GT, 1>(a, max_runs, num_sms, st);
  if (max_D <= 256) return launch_bwd<WT, GT, 2>(a, max_runs, num_sms, st);
  if (max_D <= 512) return launch_bwd<WT, GT, 4>(a, max_runs, num_sms, st);
  if (max_D <= 1024) return launch_bwd<WT, GT, 8>(a, max_runs, num_sms, st);
  return -5;
}

// generic row gather / scatter (HBM cache <-> staging buffers of the host tier)
template <typename T4>
__global__ void gather_rows_kernel(const T4* __restrict__ src, const long long* __restrict__ idx, long long n,
                                   int vec_per_row, T4* __restrict__ dst) {
  const long long total = n * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row);
    dst[i] = src[idx[r] * vec_per_row + c];
  }
}
template <typename T4>
__global__ void scatter_rows_kernel(const T4* __restrict__ src, const long long* __restrict__ idx, long long n,
                                    int vec_per_row, T4* __restrict__ dst) {
  const long long total = n * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row);
    dst[idx[r] * vec_per_row + c] = src[i];
  }
}

}  // namespace

#define RB_W_DISPATCH(wd, ...)                                        \
  switch (wd) {                                                       \
    case DT_F32: { using WT = float; __VA_ARGS__; } break;            \
    case DT_F16: { using WT = __half; __VA_ARGS__; } break;           \
    case DT_BF16: { using WT = __nv_bfloat16; __VA_ARGS__; } break;   \
    default: return -1;                                               \
  }
#define RB_O_DISPATCH(od, ...)                                        \
  switch (od) {                                                       \
    case DT_F32: { using OT = float; __VA_ARGS__; } break;            \
    case DT_F16: { using OT = __half; __VA_ARGS__; } break;           \
    case DT_BF16: { using OT = __nv_bfloat16; __VA_ARGS__; } break;   \
    default: return -1;                                               \
  }

RB_API int rb_tbe_forward(const void* shards, const long long* ptrs, const void* indices, int idx64,
                          const long long* offsets, int T, int B, int world, int self, int pooling,
                          int w_dtype, void* out, int out_dtype, long long ld_out, int vec8_ok, int* status,
                          cudaStream_t st) {
  const long long n_warps = static_cast<long long>(T) * B;
  if (n_warps == 0) return 0;
  const int threads = 256;
  const TableShard* sh = reinterpret_cast<const TableShard*>(shards);
  if (offsets == nullptr && vec8_ok) {
    // one id per bag, every D a multiple of 8 and 16-byte aligned rows: half-warp fast path
    constexpr int G = 4;
    const long long halves = static_cast<long long>(T) * ((B + G - 1) / G);
    const long long fblocks = (halves * 16 + threads - 1) / threads;
    RB_W_DISPATCH(w_dtype, RB_O_DISPATCH(out_dtype, {
      if (idx64)
        tbe_forward_onehot_kernel<WT, OT, long long, G><<<fblocks, threads, 0, st>>>(
            sh, ptrs, reinterpret_cast<const long long*>(indices), T, B, world, self, reinterpret_cast<OT*>(out),
            ld_out, status);
      else
        tbe_forward_onehot_kernel<WT, OT, int, G><<<fblocks, threads, 0, st>>>(
            sh, ptrs, reinterpret_cast<const int*>(indices), T, B, world, self, reinterpret_cast<OT*>(out), ld_out,
            status);
    }))
    return static_cast<int>(cudaGetLastError());
  }
  const long long blocks = (n_warps * 32 + threads - 1) / threads;
  RB_W_DISPATCH(w_dtype, RB_O_DISPATCH(out_dtype, {
    if (idx64)
      tbe_forward_kernel<WT, OT, long long><<<blocks, threads, 0, st>>>(
          sh, ptrs, reinterpret_cast<const long long*>(indices), offsets, T, B, world, self, pooling,
          reinterpret_cast<OT*>(out), ld_out, status);
    else
      tbe_forward_kernel<WT, OT, int><<<blocks, threads, 0, st>>>(
          sh, ptrs, reinterpret_cast<const int*>(indices), offsets, T, B, world, self, pooling,
          reinterpret_cast<OT*>(out), ld_out, status);
  }))
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_tbe_sequence(const void* shards, const long long* ptrs, const void* indices, int idx64,
                           const long long* pos_offsets, int T, long long nnz, int world, int self,
                           int w_dtype, void* out, int out_dtype, long long ld_out, int* status,
                           cudaStream_t st) {
  if (nnz == 0) return 0;
  const int threads = 256;
  const long long blocks = (nnz * 32 + threads - 1) / threads;
  const TableShard* sh = reinterpret_cast<const TableShard*>(shards);
  RB_W_DISPATCH(w_dtype, RB_O_DISPATCH(out_dtype, {
    if (idx64)
      tbe_sequence_kernel<WT, OT, long long><<<blocks, threads, 0, st>>>(
          sh, ptrs, reinterpret_cast<const long long*>(indices), pos_offsets, T, nnz, world, self,
          reinterpret_cast<OT*>(out), ld_out, status);
    else
      tbe_sequence_kernel<WT, OT, int><<<blocks, threads, 0, st>>>(
          sh, ptrs, reinterpret_cast<const int*>(indices), pos_offsets, T, nnz, world, self,
          reinterpret_cast<OT*>(out), ld_out, status);
  }))
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_tbe_linearize(const void* shards, const void* indices, int idx64, const long long* offsets,
                            int T, int B, long long nnz, int world, int self, long long* keys, int* bags,
                            cudaStream_t st) {
  if (nnz == 0) return 0;
  const int threads = 256;
  const long long blocks = (nnz + threads - 1) / threads;
  const TableShard* sh = reinterpret_cast<const TableShard*>(shards);
  if (idx64)
    tbe_linearize_kernel<long long><<<blocks, threads, 0, st>>>(
        sh, reinterpret_cast<const long long*>(indices), offsets, T, B, nnz, world, self, keys, bags);
  else
    tbe_linearize_kernel<int><<<blocks, threads, 0, st>>>(sh, reinterpret_cast<const int*>(indices), offsets,
                                                          T, B, nnz, world, self, keys, bags);
  return static_cast<int>(cudaGetLastError());
}

struct IsOwnedKey {
  __host__ __device__ __forceinline__ bool operator()(const long long& k) const { return k >= 0; }
};

// Temp-storage size for rb_sort_segments / rb_compact_owned with up to n keys.
RB_API long long rb_sort_segments_temp_bytes(long long n) {
  size_t a = 0, b = 0, c = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, a, (long long*)nullptr, (long long*)nullptr, (int*)nullptr,
                                  (int*)nullptr, static_cast<int>(n), 0, 64);
  cub::DeviceRunLengthEncode::Encode(nullptr, b, (long long*)nullptr, (long long*)nullptr, (int*)nullptr,
                                     (int*)nullptr, static_cast<int>(n));
  cub::DeviceScan::ExclusiveSum(nullptr, c, (int*)nullptr, (int*)nullptr, static_cast<int>(n) + 1);
  size_t d = 0, e = 0;
  cub::DeviceSelect::If(nullptr, d, (long long*)nullptr, (long long*)nullptr, (int*)nullptr, static_cast<int>(n), IsOwnedKey());
  cub::DeviceSelect::FlaggedIf(nullptr, e, (int*)nullptr, (long long*)nullptr, (int*)nullptr, (int*)nullptr, static_cast<int>(n),
                               IsOwnedKey());
  size_t m = a > b ? a : b;
  m = m > c ? m : c;
  m = m > d ? m : d;
  m = m > e ? m : e;
  return static_cast<long long>(m + 256);
}

// Keep the (key, bag) pairs this rank owns (key >= 0), in their original order, in the first `count` entries of the
// outputs and fill entries [count, cap) with the "not owned" key -1, so that a sort of `cap` entries replaces a sort
// of all n.  cap is a host-side bound on the owned count; if it is exceeded the surplus pairs are dropped and
// status[0] becomes RB_ERR_CAPACITY.  Outputs must have room for n entries.  No host synchronisation.
__global__ void pad_owned_tail_kernel(long long* __restrict__ keys, int* __restrict__ bags, const int* __restrict__ count, int cap,
                                      int* __restrict__ status) {
  const int c = *count;
  if (c > cap && blockIdx.x == 0 && threadIdx.x == 0) atomicExch(status, RB_ERR_CAPACITY);
  for (int i = c + blockIdx.x * blockDim.x + threadIdx.x; i < cap; i += gridDim.x * blockDim.x) { keys[i] = -1; bags[i] = 0; }
}

RB_API int rb_compact_owned(const long long* keys, const int* bags, long long n, long long* keys_out, int* bags_out, int* count,
                            int cap, void* temp, long long temp_bytes, int* status, cudaStream_t st) {
  if (n == 0) return static_cast<int>(cudaMemsetAsync(count, 0, sizeof(int), st));
  size_t tb = static_cast<size_t>(temp_bytes);
  RB_CUDA_CHECK(cub::DeviceSelect::If(temp, tb, keys, keys_out, count, static_cast<int>(n), IsOwnedKey(), st));
  tb = static_cast<size_t>(temp_bytes);
  RB_CUDA_CHECK(cub::DeviceSelect::FlaggedIf(temp, tb, bags, keys, bags_out, count, static_cast<int>(n), IsOwnedKey(), st));
  pad_owned_tail_kernel<<<64, 256, 0, st>>>(keys_out, bags_out, count, cap, status);
  return static_cast<int>(cudaGetLastError());
}

// keys/vals -> sorted keys/vals, unique keys, segment offsets (exclusive scan of run lengths,
// with seg_offsets[num_runs] = n) and the run count, all on the device, no host sync.
// `counts` is scratch of n+1 ints.  Keys are signed 64-bit; sorting uses bits [0, end_bit) plus
// the sign bit when end_bit == 64.
RB_API int rb_sort_segments(const long long* keys_in, const int* vals_in, long long n, int end_bit,
                            long long* keys_out, int* vals_out, long long* unique_out, int* counts,
                            int* seg_offsets, int* num_runs, void* temp, long long temp_bytes,
                            cudaStream_t st) {
  if (n == 0) { return static_cast<int>(cudaMemsetAsync(num_runs, 0, sizeof(int), st)); }
  size_t tb = static_cast<size_t>(temp_bytes);
  // keys may be -1 (not owned): sort all 64 bits in that case so they group together.
  RB_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(temp, tb, keys_in, keys_out, vals_in, vals_out,
                                                static_cast<int>(n), 0, end_bit, st));
  tb = static_cast<size_t>(temp_bytes);
  RB_CUDA_CHECK(cudaMemsetAsync(counts, 0, sizeof(int) * (n + 1), st));
  RB_CUDA_CHECK(cub::DeviceRunLengthEncode::Encode(temp, tb, keys_out, unique_out, counts, num_runs,
                                                   static_cast<int>(n), st));
  tb = static_cast<size_t>(temp_bytes);
  RB_CUDA_CHECK(cub::DeviceScan::ExclusiveSum(temp, tb, counts, seg_offsets, static_cast<int>(n) + 1, st));
  return 0;
}

static int tbe_backward_update_impl(
    const void* shards, const long long* key_cumsum, const long long* w_offsets, const long long* s_offsets,
    int T, int n_tables, int B_local, int world, const long long* grad_ptrs, long long ld_g, int g_dtype,
    const long long* offsets, int pooling, const int* sorted_bags, const long long* unique_keys,
    const int* seg_offsets, const int* num_runs, int max_runs, void* weights, int w_dtype, float* state1,
    float* state2, int opt_type, float lr, float eps, float beta1, float beta2, float weight_decay,
    float bias_c1, float bias_c2, int max_D, int* long_list, int* counters, void* chunk_list, float* long_accum,
    int long_cap, int chunk_cap, int accum_ld, int long_threshold, int num_sms, int* status, cudaStream_t st,
    const void* direct_rows, long long direct_ld, const int* table_dims) {
  if (max_runs <= 0) return 0;
  BwdArgs a;
  a.shards = reinterpret_cast<const TableShard*>(shards);
  a.key_cumsum = key_cumsum; a.w_offsets = w_offsets; a.s_offsets = s_offsets;
  a.T = T; a.n_tables = n_tables; a.B_local = B_local; a.world = world; a.grad_ptrs = grad_ptrs; a.ld_g = ld_g;
  a.offsets = offsets; a.pooling = pooling; a.sorted_bags = sorted_bags; a.unique_keys = unique_keys;
  a.seg_offsets = seg_offsets; a.num_runs = num_runs; a.weights = weights; a.state1 = state1;
  a.state2 = state2;
  a.opt.type = opt_type; a.opt.lr = lr; a.opt.eps = eps; a.opt.beta1 = beta1; a.opt.beta2 = beta2;
  a.opt.weight_decay = weight_decay; a.opt.bias_c1 = bias_c1; a.opt.bias_c2 = bias_c2;
  a.long_list = long_list; a.counters = counters; a.chunk_list = reinterpret_cast<int2*>(chunk_list);
  a.long_accum = long_accum; a.long_cap = long_cap; a.chunk_cap = chunk_cap; a.accum_ld = accum_ld;
  a.long_threshold = long_threshold; a.status = status;
  a.direct_rows = direct_rows; a.direct_ld = direct_ld; a.table_dims = table_dims;
  if (num_sms <= 0) num_sms = 148;
  if (max_D % 8 || accum_ld < max_D) return -7;
  RB_CUDA_CHECK(cudaMemsetAsync(counters, 0, 2 * sizeof(int), st));
#define RB_G_DISPATCH(...)                                                  \
  switch (g_dtype) {                                                        \
    case DT_F32: { using GT = float; __VA_ARGS__; } break;                  \
    case DT_F16: { using GT = __half; __VA_ARGS__; } break;                 \
    case DT_BF16: { using GT = __nv_bfloat16; __VA_ARGS__; } break;         \
    default: return -1;                                                     \
  }
  RB_W_DISPATCH(w_dtype, RB_G_DISPATCH(return dispatch_nch<WT, GT>(a, max_D, max_runs, num_sms, st)))
  return 0;
}

RB_API int rb_tbe_backward_update(
    const void* shards, const long long* key_cumsum, const long long* w_offsets, const long long* s_offsets,
    int T, int n_tables, int B_local, int world, const long long* grad_ptrs, long long ld_g, int g_dtype,
    const long long* offsets, int pooling, const int* sorted_bags, const long long* unique_keys,
    const int* seg_offsets, const int* num_runs, int max_runs, void* weights, int w_dtype, float* state1,
    float* state2, int opt_type, float lr, float eps, float beta1, float beta2, float weight_decay,
    float bias_c1, float bias_c2, int max_D, int* long_list, int* counters, void* chunk_list, float* long_accum,
    int long_cap, int chunk_cap, int accum_ld, int long_threshold, int num_sms, int* status, cudaStream_t st) {
  return tbe_backward_update_impl(shards, key_cumsum, w_offsets, s_offsets, T, n_tables, B_local, world, grad_ptrs, ld_g, g_dtype, offsets,
                                 pooling, sorted_bags, unique_keys, seg_offsets, num_runs, max_runs, weights, w_dtype, state1, state2,
                                 opt_type, lr, eps, beta1, beta2, weight_decay, bias_c1, bias_c2, max_D, long_list, counters,
                                 chunk_list, long_accum, long_cap, chunk_cap, accum_ld, long_threshold, num_sms, status, st, nullptr, 0, nullptr);
}

// Same update with the gradient rows already in local memory (push exchange): the gradient of sorted entry j is the
// row sorted_bags[j] of `direct_rows` (rows of direct_ld elements of g_dtype); table_dims[n_tables] = row widths.
RB_API int rb_tbe_backward_update_rows(
    const void* shards, const long long* key_cumsum, const long long* w_offsets, const long long* s_offsets,
    int T, int n_tables, int B_local, int world, const long long* grad_ptrs, long long ld_g, int g_dtype,
    const long long* offsets, int pooling, const int* sorted_bags, const long long* unique_keys,
    const int* seg_offsets, const int* num_runs, int max_runs, void* weights, int w_dtype, float* state1,
    float* state2, int opt_type, float lr, float eps, float beta1, float beta2, float weight_decay,
    float bias_c1, float bias_c2, int max_D, int* long_list, int* counters, void* chunk_list, float* long_accum,
    int long_cap, int chunk_cap, int accum_ld, int long_threshold, int num_sms, int* status, cudaStream_t st,
    const void* direct_rows, long long direct_ld, const int* table_dims) {
  if (!direct_rows || !table_dims) return -1;
  return tbe_backward_update_impl(shards, key_cumsum, w_offsets, s_offsets, T, n_tables, B_local, world, grad_ptrs, ld_g, g_dtype, offsets,
                                 pooling, sorted_bags, unique_keys, seg_offsets, num_runs, max_runs, weights, w_dtype, state1, state2,
                                 opt_type, lr, eps, beta1, beta2, weight_decay, bias_c1, bias_c2, max_D, long_list, counters,
                                 chunk_list, long_accum, long_cap, chunk_cap, accum_ld, long_threshold, num_sms, status, st, direct_rows, direct_ld, table_dims);
}

RB_API int rb_gather_rows(const void* src, const long long* idx, long long n, long long row_bytes, void* dst,
                          cudaStream_t st) {
  if (n == 0) return 0;
  if (row_bytes % 16 == 0) {
    const int v = static_cast<int>(row_bytes / 16);
    const long long total = n * v;
    const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
    gather_rows_kernel<uint4><<<blocks, 256, 0, st>>>(reinterpret_cast<const uint4*>(src), idx, n, v,
                                                      reinterpret_cast<uint4*>(dst));
  } else if (row_bytes % 4 == 0) {
    const int v = static_cast<int>(row_bytes / 4);
    const long long total = n * v;
    const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
    gather_rows_kernel<uint32_t><<<blocks, 256, 0, st>>>(reinterpret_cast<const uint32_t*>(src), idx, n, v,
                                                         reinterpret_cast<uint32_t*>(dst));
  } else {
    return -1;
  }
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_scatter_rows(const void* src, const long long* idx, long long n, long long row_bytes, void* dst,
                           cudaStream_t st) {
  if (n == 0) return 0;
  if (row_bytes % 16 == 0) {
    const int v = static_cast<int>(row_bytes / 16);
    const long long total = n * v;
    const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
    scatter_rows_kernel<uint4><<<blocks, 256, 0, st>>>(reinterpret_cast<const uint4*>(src), idx, n, v,
                                                       reinterpret_cast<uint4*>(dst));
  } else if (row_bytes % 4 == 0) {
    const int v = static_cast<int>(row_bytes / 4);
    const long long total = n * v;
    const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
    scatter_rows_kernel<uint32_t><<<blocks, 256, 0, st>>>(reinterpret_cast<const uint32_t*>(src), idx, n, v,
                                                          reinterpret_cast<uint32_t*>(dst));
  } else {
    return -1;
  }
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// dst[dst_idx[i]] = src[src_idx[i]] for rows of row_bytes (a multiple of 16).  Either side may be pinned
// host memory (mapped into the device address space), so one launch moves a whole layer of KV pages between the
// host chunk pool and the paged device cache without a staging buffer.
__global__ void copy_rows_kernel(const uint4* __restrict__ src, const long long* __restrict__ src_idx,
                                 uint4* __restrict__ dst, const long long* __restrict__ dst_idx, long long n, int v) {
  const long long total = n * v;
  for (long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; t < total;
       t += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = t / v;
    const int c = static_cast<int>(t - r * v);
    dst[dst_idx[r] * v + c] = src[src_idx[r] * v + c];
  }
}

RB_API int rb_copy_rows(const void* src, const long long* src_idx, void* dst, const long long* dst_idx, long long n,
                        long long row_bytes, int num_sms, cudaStream_t st) {
  if (n == 0) return 0;
  if (row_bytes % 16) return -1;
  if (num_sms <= 0) num_sms = 148;
  const int v = static_cast<int>(row_bytes / 16);
  const long long total = n * v;
  const long long want = (total + 255) / 256;
  const int blocks = static_cast<int>(want < num_sms * 8LL ? want : num_sms * 8LL);
  copy_rows_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const uint4*>(src), src_idx, reinterpret_cast<uint4*>(dst),
                                           dst_idx, n, v);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// Pooled gather / scatter-add over the unique rows of a dynamic (hash) table:
//   out[bag, :] = sum (or mean) over j in [offsets[bag], offsets[bag+1]) of rows[inverse[j], :]
//   red[inverse[j], :] += g[bag, :] (/ len for mean)
// rows / red are fp32 [n_unique, D] (D a multiple of 4); a group of G = min(32, pow2 >= D/4) lanes serves one bag,
// 32 / G bags per warp, so the per-id rows are never materialised.
// (dynamic_emb lookup_forward / lookup_backward of the reference: csrc/ops/pooling_embeddings, csrc/ops/look_backward.)
template <typename OT>
__global__ void pooled_gather_kernel(const float* __restrict__ rows, const long long* __restrict__ inverse,
                                     const long long* __restrict__ offsets, long long bags, long long B, int D, int G, int mean,
                                     OT* __restrict__ out, long long ld_out) {
  const int lane = threadIdx.x & 31;
  const int gl = lane & (G - 1);
  const long long group = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) / G;
  if (group >= bags) return;
  const long long beg = offsets[group], end = offsets[group + 1];
  const float inv_len = (mean && end > beg) ? 1.f / static_cast<float>(end - beg) : 1.f;
  for (int c = gl; c * 4 < D; c += G) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    long long j = beg;
    for (; j + 1 < end; j += 2) {                                    // two rows in flight
      const float4 a = *reinterpret_cast<const float4*>(rows + inverse[j] * D + c * 4);
      const float4 b = *reinterpret_cast<const float4*>(rows + inverse[j + 1] * D + c * 4);
      acc.x += a.x + b.x; acc.y += a.y + b.y; acc.z += a.z + b.z; acc.w += a.w + b.w;
    }
    if (j < end) {
      const float4 a = *reinterpret_cast<const float4*>(rows + inverse[j] * D + c * 4);
      acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
    }
    OT* o = out + (group % B) * ld_out + (group / B) * D + c * 4;            // bag = feature * B + sample
    o[0] = static_cast<OT>(acc.x * inv_len); o[1] = static_cast<OT>(acc.y * inv_len);
    o[2] = static_cast<OT>(acc.z * inv_len); o[3] = static_cast<OT>(acc.w * inv_len);
  }
}

template <typename GT>
__global__ void pooled_scatter_add_kernel(const GT* __restrict__ g, long long ld_g, const long long* __restrict__ inverse,
                                          const long long* __restrict__ offsets, long long bags, long long B, int D, int G, int mean,
                                          float* __restrict__ red) {
  const int lane = threadIdx.x & 31;
  const int gl = lane & (G - 1);
  const long long group = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) / G;
  if (group >= bags) return;
  const long long beg = offsets[group], end = offsets[group + 1];
  const float inv_len = (mean && end > beg) ? 1.f / static_cast<float>(end - beg) : 1.f;
  for (int c = gl; c * 4 < D; c += G) {
    const GT* gp = g + (group % B) * ld_g + (group / B) * D + c * 4;
    const float x = static_cast<float>(gp[0]) * inv_len, y = static_cast<float>(gp[1]) * inv_len,
                z = static_cast<float>(gp[2]) * inv_len, w = static_cast<float>(gp[3]) * inv_len;
    for (long long j = beg; j < end; ++j) rb::red_add_v4(red + inverse[j] * D + c * 4, x, y, z, w);
  }
}

// Sorted form of the same reduction: the (unique row, bag) pairs arrive sorted by row, every group of G lanes owns CH
// consecutive pairs and keeps a running sum while the row stays the same.  A row whose pairs all lie inside one group's
// range is written with a plain store; only rows that span groups (the hot keys of a skewed batch) are accumulated with
// vector reductions, one per group instead of one per id.  `red` must be zero where rows span groups (the caller zeroes it).
template <typename GT, int CH>
__global__ void pooled_segment_add_kernel(const GT* __restrict__ g, long long ld_g, const long long* __restrict__ keys,
                                          const int* __restrict__ bags_sorted, const long long* __restrict__ offsets, long long n,
                                          long long B, int D, int G, int mean, float* __restrict__ red) {
  const int gl = threadIdx.x & (G - 1);
  const long long group = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) / G;
  const long long p0 = group * CH;
  if (p0 >= n) return;
  const long long p1 = (p0 + CH < n) ? p0 + CH : n;
  for (int c = gl; c * 4 < D; c += G) {
    long long cur = keys[p0];
    bool starts_here = (p0 == 0) || (keys[p0 - 1] != cur);
    float ax = 0.f, ay = 0.f, az = 0.f, aw = 0.f;
#pragma unroll 4
    for (long long p = p0; p < p1; ++p) {
      const long long k = keys[p];
      if (k != cur) {
        float* o = red + cur * D + c * 4;
        if (starts_here) *reinterpret_cast<float4*>(o) = make_float4(ax, ay, az, aw);
        else rb::red_add_v4(o, ax, ay, az, aw);
        cur = k; starts_here = true;
        ax = ay = az = aw = 0.f;
      }
      const long long bag = bags_sorted[p];
      float sc = 1.f;
      if (mean) { const long long len = offsets[bag + 1] - offsets[bag]; sc = len > 0 ? 1.f / static_cast<float>(len) : 1.f; }
      const GT* gp = g + (bag % B) * ld_g + (bag / B) * D + c * 4;
      ax += static_cast<float>(gp[0]) * sc; ay += static_cast<float>(gp[1]) * sc;
      az += static_cast<float>(gp[2]) * sc; aw += static_cast<float>(gp[3]) * sc;
    }
    const bool ends_here = (p1 == n) || (keys[p1] != cur);
    float* o = red + cur * D + c * 4;
    if (starts_here && ends_here) *reinterpret_cast<float4*>(o) = make_float4(ax, ay, az, aw);
    else rb::red_add_v4(o, ax, ay, az, aw);
  }
}

static int pooled_group(int D) {
  int g = 1;
  while (g < 32 && g * 4 < D) g <<= 1;
  return g;
}

// bags = F * B (feature-major); the pooled row of bag f * B + b is written to out[b * ld_out + f * D ...]
RB_API int rb_pooled_gather(const float* rows, const long long* inverse, const long long* offsets, long long bags, long long B, int D,
                            int mean, void* out, int out_dtype, long long ld_out, cudaStream_t st) {
  if (bags == 0) return 0;
  if (B <= 0) B = bags;
  if (D % 4) return -1;
  const int G = pooled_group(D);
  const long long threads = bags * G;
  const unsigned blocks = static_cast<unsigned>((threads + 255) / 256);
  RB_O_DISPATCH(out_dtype, pooled_gather_kernel<OT><<<blocks, 256, 0, st>>>(rows, inverse, offsets, bags, B, D, G, mean,
                                                                            reinterpret_cast<OT*>(out), ld_out));
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_pooled_scatter_add(const void* g, int g_dtype, long long ld_g, const long long* inverse, const long long* offsets,
                                 long long bags, long long B, int D, int mean, float* red, cudaStream_t st) {
  if (bags == 0) return 0;
  if (B <= 0) B = bags;
  if (D % 4) return -1;
  const int G = pooled_group(D);
  const long long threads = bags * G;
  const unsigned blocks = static_cast<unsigned>((threads + 255) / 256);
  switch (g_dtype) {
    case DT_F32: pooled_scatter_add_kernel<float><<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(g), ld_g, inverse, offsets, bags, B, D, G, mean, red); break;
    case DT_F16: pooled_scatter_add_kernel<__half><<<blocks, 256, 0, st>>>(reinterpret_cast<const __half*>(g), ld_g, inverse, offsets, bags, B, D, G, mean, red); break;
    case DT_BF16: pooled_scatter_add_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(g), ld_g, inverse, offsets, bags, B, D, G, mean, red); break;
    default: return -1;
  }
  return static_cast<int>(cudaGetLastError());
}

// Radix sort of (row, bag) pairs on the low `end_bit` bits of the row index; temp size: rb_sort_segments_temp_bytes(n).
RB_API int rb_sort_pairs_i64_i32(const long long* keys_in, const int* vals_in, long long n, int end_bit, long long* keys_out,
                                 int* vals_out, void* temp, long long temp_bytes, cudaStream_t st) {
  if (n == 0) return 0;
  size_t tb = static_cast<size_t>(temp_bytes);
  return static_cast<int>(cub::DeviceRadixSort::SortPairs(temp, tb, keys_in, keys_out, vals_in, vals_out, static_cast<int>(n), 0,
                                                          end_bit, st));
}

// red[row] (+)= sum of the gradients of the bags that used the row; keys / bags sorted by row (see the kernel above)
RB_API int rb_pooled_segment_add(const void* g, int g_dtype, long long ld_g, const long long* keys_sorted, const int* bags_sorted,
                                 const long long* offsets, long long n, long long B, int D, int mean, float* red, cudaStream_t st) {
  if (n == 0) return 0;
  if (D % 4) return -1;
  constexpr int CH = 64;
  const int G = pooled_group(D);
  const long long groups = (n + CH - 1) / CH;
  const unsigned blocks = static_cast<unsigned>((groups * G + 255) / 256);
  switch (g_dtype) {
    case DT_F32: pooled_segment_add_kernel<float, CH><<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(g), ld_g, keys_sorted, bags_sorted, offsets, n, B, D, G, mean, red); break;
    case DT_F16: pooled_segment_add_kernel<__half, CH><<<blocks, 256, 0, st>>>(reinterpret_cast<const __half*>(g), ld_g, keys_sorted, bags_sorted, offsets, n, B, D, G, mean, red); break;
    case DT_BF16: pooled_segment_add_kernel<__nv_bfloat16, CH><<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(g), ld_g, keys_sorted, bags_sorted, offsets, n, B, D, G, mean, red); break;
    default: return -1;
  }
  return static_cast<int>(cudaGetLastError());
}
