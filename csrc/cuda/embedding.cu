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

#include "common.cuh"

namespace {

enum ShardKind : int { SH_LOCAL = 0, SH_TABLE_WISE = 1, SH_ROW_MOD = 2, SH_ROW_BLOCK = 3 };
enum Pooling : int { POOL_SUM = 0, POOL_MEAN = 1, POOL_NONE = 2 };
enum WDtype : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };
enum OptType : int { OPT_SGD = 0, OPT_ROWWISE_ADAGRAD = 1, OPT_ADAGRAD = 2, OPT_ADAM = 3 };

// One record per feature (bag group); features that share a table carry the same table fields.
// `ptr_index` points into the flat pointer table
// ptrs[ptr_index + rank]; for SH_LOCAL / SH_TABLE_WISE only entry `owner` is used.
struct TableShard {
  int kind;
  int owner;
  int D;
  int D_offset;          // column offset of this table in the pooled output
  long long rows;        // logical row count (bounds check)
  long long block;       // rows per rank for SH_ROW_BLOCK
  long long ptr_index;
  long long key_base;    // first linear key of this table on its owner (backward)
};

template <typename T> struct Ld4;
template <> struct Ld4<float> {
  static __device__ __forceinline__ float4 ld(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void st(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Ld4<__half> {
  static __device__ __forceinline__ float4 ld(const __half* p) {
    uint2 u = *reinterpret_cast<const uint2*>(p);
    float2 a = rb::unpack_f16(u.x), b = rb::unpack_f16(u.y);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void st(__half* p, float4 v) {
    *reinterpret_cast<uint2*>(p) = make_uint2(rb::pack_f16(v.x, v.y), rb::pack_f16(v.z, v.w));
  }
};
template <> struct Ld4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 ld(const __nv_bfloat16* p) {
    uint2 u = *reinterpret_cast<const uint2*>(p);
    float2 a = rb::unpack_bf16(u.x), b = rb::unpack_bf16(u.y);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float4 v) {
    *reinterpret_cast<uint2*>(p) = make_uint2(rb::pack_bf16(v.x, v.y), rb::pack_bf16(v.z, v.w));
  }
};

__device__ __forceinline__ bool locate_row(const TableShard& ts, long long id, int world, int self,
                                           int& rank, long long& row) {
  if (id < 0 || id >= ts.rows) return false;
  switch (ts.kind) {
    case SH_ROW_MOD: rank = static_cast<int>(id % world); row = id / world; break;
    case SH_ROW_BLOCK: rank = static_cast<int>(id / ts.block); row = id % ts.block; break;
    case SH_TABLE_WISE: rank = ts.owner; row = id; break;
    default: rank = self; row = id; break;
  }
  return true;
}

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
// backward + optimizer
// ---------------------------------------------------------------------------
struct OptArgs {
  int type;
  float lr, eps, beta1, beta2, weight_decay;
  float bias_c1, bias_c2;  // 1-beta1^t, 1-beta2^t
};

struct BwdArgs {
  const TableShard* shards;
  const long long* key_cumsum;   // [T+1] linear key range of each table on this rank
  const long long* w_offsets;    // [T] element offset of each table in `weights`
  const long long* s_offsets;    // [T] offset of each table in the state arrays (rows or elements)
  int T, n_tables, B_local, world;   // T = features (bag groups); n_tables = physical tables
  const long long* grad_ptrs;    // [world] base of each rank's pooled-gradient buffer
  long long ld_g;
  const long long* offsets;      // bag offsets for mean pooling (nullable), over the global bag index
  int pooling;
  const int* sorted_bags;        // bag index (t * B_global + b_global)
  const long long* unique_keys;
  const int* seg_offsets;        // [num_runs + 1]
  const int* num_runs;
  void* weights;
  float* state1;
  float* state2;
  OptArgs opt;
  int* long_list;
  int* long_count;
  int long_cap;
  int long_threshold;
  int* status;
};

template <typename WT, int NCH>
__device__ __forceinline__ void apply_row_update(const BwdArgs& a, int t, long long local_row, int D,
                                                 float4 (&acc)[NCH], int lane) {
  WT* w = reinterpret_cast<WT*>(a.weights) + a.w_offsets[t] + local_row * D;
  const OptArgs& o = a.opt;
  if (o.type == OPT_ROWWISE_ADAGRAD) {
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c)
      if (lane * 4 + c * 128 < D) ss += acc[c].x * acc[c].x + acc[c].y * acc[c].y + acc[c].z * acc[c].z + acc[c].w * acc[c].w;
    ss = rb::warp_sum(ss);
    float* st = a.state1 + a.s_offsets[t] + local_row;
    const float g2 = *st + ss / static_cast<float>(D);
    __syncwarp();
    if (lane == 0) *st = g2;
    const float mult = o.lr / (sqrtf(g2) + o.eps);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int d0 = lane * 4 + c * 128;
      if (d0 < D) {
        float4 v = Ld4<WT>::ld(w + d0);
        v.x -= mult * acc[c].x; v.y -= mult * acc[c].y; v.z -= mult * acc[c].z; v.w -= mult * acc[c].w;
        Ld4<WT>::st(w + d0, v);
      }
    }
    return;
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int d0 = lane * 4 + c * 128;
    if (d0 >= D) continue;
    float4 v = Ld4<WT>::ld(w + d0);
    float g[4] = {acc[c].x, acc[c].y, acc[c].z, acc[c].w};
    float wv[4] = {v.x, v.y, v.z, v.w};
    if (o.type == OPT_SGD) {
#pragma unroll
      for (int i = 0; i < 4; ++i) wv[i] -= o.lr * (g[i] + o.weight_decay * wv[i]);
    } else if (o.type == OPT_ADAGRAD) {
      float* st = a.state1 + a.s_offsets[t] + local_row * D + d0;
      float4 s = *reinterpret_cast<float4*>(st);
      float sv[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) { sv[i] += g[i] * g[i]; wv[i] -= o.lr * g[i] / (sqrtf(sv[i]) + o.eps); }
      *reinterpret_cast<float4*>(st) = make_float4(sv[0], sv[1], sv[2], sv[3]);
    } else {  // Adam
      float* m = a.state1 + a.s_offsets[t] + local_row * D + d0;
      float* vv = a.state2 + a.s_offsets[t] + local_row * D + d0;
      float4 m4 = *reinterpret_cast<float4*>(m), v4 = *reinterpret_cast<float4*>(vv);
      float mv[4] = {m4.x, m4.y, m4.z, m4.w}, vvv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float gi = g[i] + o.weight_decay * wv[i];
        mv[i] = o.beta1 * mv[i] + (1.f - o.beta1) * gi;
        vvv[i] = o.beta2 * vvv[i] + (1.f - o.beta2) * gi * gi;
        wv[i] -= (o.lr / o.bias_c1) * mv[i] / (sqrtf(vvv[i] / o.bias_c2) + o.eps);
      }
      *reinterpret_cast<float4*>(m) = make_float4(mv[0], mv[1], mv[2], mv[3]);
      *reinterpret_cast<float4*>(vv) = make_float4(vvv[0], vvv[1], vvv[2], vvv[3]);
    }
    Ld4<WT>::st(w + d0, make_float4(wv[0], wv[1], wv[2], wv[3]));
  }
}

__device__ __forceinline__ int table_of_key(const long long* cumsum, int T, long long key) {
  int lo = 0, hi = T;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (cumsum[mid] <= key) lo = mid; else hi = mid; }
  return lo;
}

template <typename GT, int NCH>
__device__ __forceinline__ void accumulate_entry(const BwdArgs& a, int D, int bag, long long B_global,
                                                 float4 (&acc)[NCH], int lane) {
  const int f = static_cast<int>(bag / B_global);
  const int D_offset = a.shards[f].D_offset;
  const long long bg = bag - static_cast<long long>(f) * B_global;
  const int r = static_cast<int>(bg / a.B_local);
  const long long bl = bg % a.B_local;
  const GT* g = reinterpret_cast<const GT*>(a.grad_ptrs[r]) + bl * a.ld_g + D_offset;
  float scale = 1.f;
  if (a.pooling == POOL_MEAN && a.offsets) {
    const long long len = a.offsets[bag + 1] - a.offsets[bag];
    scale = len > 0 ? 1.f / static_cast<float>(len) : 0.f;
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int d0 = lane * 4 + c * 128;
    if (d0 < D) {
      const float4 v = Ld4<GT>::ld(g + d0);
      acc[c].x += v.x * scale; acc[c].y += v.y * scale; acc[c].z += v.z * scale; acc[c].w += v.w * scale;
    }
  }
}

// one warp per unique row; rows with very long segments are deferred to the block kernel
template <typename WT, typename GT, int NCH>
__global__ void tbe_backward_warp_kernel(const BwdArgs a) {
  const int lane = threadIdx.x & 31;
  const int warps_total = (gridDim.x * blockDim.x) >> 5;
  const int n = *a.num_runs;
  const long long B_global = static_cast<long long>(a.B_local) * a.world;
  for (int s = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; s < n; s += warps_total) {
    const long long key = a.unique_keys[s];
    if (key < 0) continue;
    const int beg = a.seg_offsets[s], end = a.seg_offsets[s + 1];
    if (end - beg > a.long_threshold) {
      if (lane == 0) {
        const int slot = atomicAdd(a.long_count, 1);
        if (slot < a.long_cap) a.long_list[slot] = s;
        else if (a.status) atomicCAS(a.status, 0, RB_ERR_CAPACITY);
      }
      continue;
    }
    const int t = table_of_key(a.key_cumsum, a.n_tables, key);
    const int D = a.shards[a.sorted_bags[beg] / B_global].D;
    float4 acc[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = beg; j < end; ++j) accumulate_entry<GT, NCH>(a, D, a.sorted_bags[j], B_global, acc, lane);
    apply_row_update<WT, NCH>(a, t, key - a.key_cumsum[t], D, acc, lane);
  }
}

// one CTA (8 warps) per long segment: warps stride over the entries, partial sums meet in
// shared memory, warp 0 applies the optimizer.
template <typename WT, typename GT, int NCH>
__global__ void __launch_bounds__(256) tbe_backward_block_kernel(const BwdArgs a) {
  __shared__ float4 red[8][NCH * 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int n_long = *a.long_count;
  if (n_long > a.long_cap) n_long = a.long_cap;
  const long long B_global = static_cast<long long>(a.B_local) * a.world;
  for (int li = blockIdx.x; li < n_long; li += gridDim.x) {
    const int s = a.long_list[li];
    const long long key = a.unique_keys[s];
    const int beg = a.seg_offsets[s], end = a.seg_offsets[s + 1];
    const int t = table_of_key(a.key_cumsum, a.n_tables, key);
    const int D = a.shards[a.sorted_bags[beg] / B_global].D;
    float4 acc[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = beg + warp; j < end; j += 8) accumulate_entry<GT, NCH>(a, D, a.sorted_bags[j], B_global, acc, lane);
#pragma unroll
    for (int c = 0; c < NCH; ++c) red[warp][c * 32 + lane] = acc[c];
    __syncthreads();
    if (warp == 0) {
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        float4 sum = red[0][c * 32 + lane];
        for (int w = 1; w < 8; ++w) {
          const float4 v = red[w][c * 32 + lane];
          sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        acc[c] = sum;
      }
      apply_row_update<WT, NCH>(a, t, key - a.key_cumsum[t], D, acc, lane);
    }
    __syncthreads();
  }
}

template <typename WT, typename GT, int NCH>
int launch_bwd(const BwdArgs& a, int max_runs, int num_sms, cudaStream_t st) {
  int blocks = (max_runs + 7) / 8;
  const int cap = num_sms * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  tbe_backward_warp_kernel<WT, GT, NCH><<<blocks, 256, 0, st>>>(a);
  tbe_backward_block_kernel<WT, GT, NCH><<<num_sms * 2, 256, 0, st>>>(a);
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
                          int w_dtype, void* out, int out_dtype, long long ld_out, int* status,
                          cudaStream_t st) {
  const long long n_warps = static_cast<long long>(T) * B;
  if (n_warps == 0) return 0;
  const int threads = 256;
  const long long blocks = (n_warps * 32 + threads - 1) / threads;
  const TableShard* sh = reinterpret_cast<const TableShard*>(shards);
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

// Temp-storage size for rb_sort_segments with up to n keys.
RB_API long long rb_sort_segments_temp_bytes(long long n) {
  size_t a = 0, b = 0, c = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, a, (long long*)nullptr, (long long*)nullptr, (int*)nullptr,
                                  (int*)nullptr, static_cast<int>(n), 0, 64);
  cub::DeviceRunLengthEncode::Encode(nullptr, b, (long long*)nullptr, (long long*)nullptr, (int*)nullptr,
                                     (int*)nullptr, static_cast<int>(n));
  cub::DeviceScan::ExclusiveSum(nullptr, c, (int*)nullptr, (int*)nullptr, static_cast<int>(n) + 1);
  size_t m = a > b ? a : b;
  m = m > c ? m : c;
  return static_cast<long long>(m + 256);
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

RB_API int rb_tbe_backward_update(
    const void* shards, const long long* key_cumsum, const long long* w_offsets, const long long* s_offsets,
    int T, int n_tables, int B_local, int world, const long long* grad_ptrs, long long ld_g, int g_dtype,
    const long long* offsets, int pooling, const int* sorted_bags, const long long* unique_keys,
    const int* seg_offsets, const int* num_runs, int max_runs, void* weights, int w_dtype, float* state1,
    float* state2, int opt_type, float lr, float eps, float beta1, float beta2, float weight_decay,
    float bias_c1, float bias_c2, int max_D, int* long_list, int* long_count, int long_cap,
    int long_threshold, int num_sms, int* status, cudaStream_t st) {
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
  a.long_list = long_list; a.long_count = long_count; a.long_cap = long_cap;
  a.long_threshold = long_threshold; a.status = status;
  if (num_sms <= 0) num_sms = 148;
  RB_CUDA_CHECK(cudaMemsetAsync(long_count, 0, sizeof(int), st));
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
