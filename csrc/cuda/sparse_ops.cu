// Device-side sparse preprocessing: segmented hash unique (unique keys / inverse / counts per table),
// row-wise bucketisation of a jagged batch (round robin or contiguous blocks), order-preserving compaction,
// per-table ranges and the post-dedup lengths.  These replace the reference's host-side id processing and its
// AscendC kernels (dynamic_emb csrc/ops/unique_op/unique_op_kernel.h:57-172, csrc/dynamic_emb_op.cpp:1001-1124,
// csrc/ops/block_bucketsize_sparse_features, csrc/ops/maskselect_op, csrc/ops/get_table_range_op,
// csrc/ops/get_new_length_and_offsets_op) so the whole input path stays on the GPU and can be graph-captured.
#include <cub/cub.cuh>
#include <thrust/iterator/counting_iterator.h>

#include "common.cuh"

namespace {

constexpr long long kEmpty = static_cast<long long>(0x8000000000000000ULL);

__device__ __forceinline__ unsigned long long mix64(unsigned long long k) {
  k ^= k >> 33; k *= 0xff51afd7ed558ccdULL; k ^= k >> 33; k *= 0xc4ceb9fe1a85ec53ULL; k ^= k >> 33;
  return k;
}

// largest t with offs[t] <= i  (offs has T + 1 entries, offs[0] == 0)
__device__ __forceinline__ int seg_of(const long long* __restrict__ offs, int T, long long i) {
  int lo = 0, hi = T;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (offs[mid] <= i) lo = mid; else hi = mid;
  }
  return lo;
}

// ---- segmented unique --------------------------------------------------------------------------------------
// Hash set with one region per table: region t = slots [2*offs[t], 2*offs[t+1]) (load factor <= 0.5); the
// sentinel key (INT64_MIN) of table t lives in the reserved slot 2n + t.
__global__ void seg_unique_insert(const long long* __restrict__ keys, long long n, const long long* __restrict__ offs, int T,
                                  long long* __restrict__ table, int* __restrict__ pos, int* __restrict__ count,
                                  int* __restrict__ status) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = seg_of(offs, T, i);
    const long long key = keys[i];
    if (key == kEmpty) {
      const long long old = atomicExch(reinterpret_cast<unsigned long long*>(table + 2 * n + t), 0ULL);
      if (old == kEmpty) atomicAdd(count + t, 1);
      pos[i] = static_cast<int>(2 * n + t);
      continue;
    }
    const long long base = 2 * offs[t];
    const long long size = 2 * (offs[t + 1] - offs[t]);
    long long p = static_cast<long long>(mix64(static_cast<unsigned long long>(key)) % static_cast<unsigned long long>(size));
    bool done = false;
    for (long long probe = 0; probe < size; ++probe) {
      const long long cur = table[base + p];
      if (cur == key) { done = true; break; }
      if (cur == kEmpty) {
        const long long old = static_cast<long long>(atomicCAS(reinterpret_cast<unsigned long long*>(table + base + p),
                                                               static_cast<unsigned long long>(kEmpty),
                                                               static_cast<unsigned long long>(key)));
        if (old == kEmpty) { atomicAdd(count + t, 1); done = true; break; }
        if (old == key) { done = true; break; }
      }
      if (++p == size) p = 0;
    }
    if (!done) { atomicExch(status, RB_ERR_CAPACITY); p = 0; }
    pos[i] = static_cast<int>(base + p);
  }
}

// one block: exclusive scan of the per-table counts -> unique_offsets[T + 1]; clears the cursors
__global__ void seg_unique_scan(const int* __restrict__ count, int T, long long* __restrict__ unique_offsets, int* __restrict__ cursor) {
  if (threadIdx.x == 0) {
    long long acc = 0;
    for (int t = 0; t < T; ++t) { unique_offsets[t] = acc; acc += count[t]; cursor[t] = 0; }
    unique_offsets[T] = acc;
  }
}

__global__ void seg_unique_assign(const long long* __restrict__ table, long long n, const long long* __restrict__ offs, int T,
                                  const long long* __restrict__ unique_offsets, int* __restrict__ cursor, int* __restrict__ slots,
                                  long long* __restrict__ unique_out) {
  const long long total = 2 * n + T;
  for (long long p = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; p < total;
       p += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long v = table[p];
    if (v == kEmpty) continue;
    const bool reserved = p >= 2 * n;
    const int t = reserved ? static_cast<int>(p - 2 * n) : seg_of(offs, T, p >> 1);
    const long long idx = unique_offsets[t] + atomicAdd(cursor + t, 1);
    slots[p] = static_cast<int>(idx);
    unique_out[idx] = reserved ? kEmpty : v;
  }
}

__global__ void seg_unique_inverse(const int* __restrict__ pos, long long n, const int* __restrict__ slots,
                                   long long* __restrict__ inverse, int* __restrict__ counts) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int idx = slots[pos[i]];
    inverse[i] = idx;
    if (counts) atomicAdd(counts + idx, 1);
  }
}

__global__ void fill_i64(long long* __restrict__ p, long long n, long long v) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) p[i] = v;
}

// ---- bucketize ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int bucket_of(long long id, int world, long long block) {
  if (block > 0) { const long long w = id / block; return static_cast<int>(w < world - 1 ? w : world - 1); }
  long long m = id % world;
  return static_cast<int>(m < 0 ? m + world : m);
}

// one warp per bag: lanes stride over the bag's ids and count per bucket with warp votes
__global__ void bucketize_count(const long long* __restrict__ offsets, const long long* __restrict__ indices, long long FB,
                                long long B, int world, const long long* __restrict__ block_sizes, long long* __restrict__ new_lengths) {
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= FB) return;
  const long long block = block_sizes ? block_sizes[warp / B] : 0;
  const long long s = offsets[warp], e = offsets[warp + 1];
  for (int w0 = 0; w0 < world; w0 += 32) {
    int mine = 0;                                     // lane l counts bucket w0 + l
    for (long long j = s; j < e; j += 32) {
      const long long jj = j + lane;
      const int w = jj < e ? bucket_of(indices[jj], world, block) : -1;
      for (int l = 0; l < 32; ++l) {
        const int wl = __shfl_sync(0xffffffffu, w, l);
        if (wl == w0 + lane) ++mine;
      }
    }
    if (w0 + lane < world) new_lengths[(w0 + lane) * FB + warp] = mine;
  }
}

// one warp per bag; order inside a bucket follows the input order (stable), like the host implementation
__global__ void bucketize_fill(const long long* __restrict__ offsets, const long long* __restrict__ indices,
                               const float* __restrict__ weights, long long FB, long long B, int world,
                               const long long* __restrict__ block_sizes, int local_rows, const long long* __restrict__ new_offsets,
                               long long* __restrict__ new_indices, float* __restrict__ new_weights,
                               long long* __restrict__ unbucketize_permute) {
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= FB) return;
  const long long block = block_sizes ? block_sizes[warp / B] : 0;
  const long long s = offsets[warp], e = offsets[warp + 1];
  for (int w = 0; w < world; ++w) {
    long long cursor = new_offsets[w * FB + warp];
    for (long long j = s; j < e; j += 32) {
      const long long jj = j + lane;
      const bool in = jj < e;
      const long long id = in ? indices[jj] : 0;
      const bool hit = in && bucket_of(id, world, block) == w;
      const unsigned m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const long long p = cursor + __popc(m & ((1u << lane) - 1u));
        long long v = id;
        if (local_rows) v = block > 0 ? id - w * block : id / world;
        new_indices[p] = v;
        if (new_weights) new_weights[p] = weights[jj];
        if (unbucketize_permute) unbucketize_permute[jj] = p;
      }
      cursor += __popc(m);
    }
  }
}

// ---- small helpers ------------------------------------------------------------------------------------------
__global__ void table_range_kernel(const long long* __restrict__ offsets, const int* __restrict__ feature_offsets, int T, long long B,
                                   long long* __restrict__ out) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t <= T) out[t] = offsets[static_cast<long long>(feature_offsets[t]) * B];
}

// After per-table dedup the table's unique keys are spread evenly over its (feature, sample) bags:
// bag j of table t gets floor(u_t / bags_t) keys, the first (u_t mod bags_t) bags one more.
__global__ void new_lengths_kernel(const long long* __restrict__ unique_offsets, const int* __restrict__ feature_offsets, int T,
                                   long long B, long long* __restrict__ new_lengths, long long* __restrict__ new_offsets) {
  const long long FB = static_cast<long long>(feature_offsets[T]) * B;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i <= FB;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    if (i == FB) { new_offsets[FB] = unique_offsets[T]; continue; }
    int lo = 0, hi = T;
    while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (static_cast<long long>(feature_offsets[mid]) * B <= i) lo = mid; else hi = mid; }
    const long long first = static_cast<long long>(feature_offsets[lo]) * B;
    const long long bags = static_cast<long long>(feature_offsets[lo + 1]) * B - first;
    const long long u = unique_offsets[lo + 1] - unique_offsets[lo];
    const long long j = i - first, q = u / bags, r = u % bags;
    new_lengths[i] = q + (j < r ? 1 : 0);
    new_offsets[i] = unique_offsets[lo] + j * q + (j < r ? j : r);
  }
}

inline int grid_for(long long n, int num_sms) {
  if (num_sms <= 0) num_sms = 148;
  const long long want = (n + 255) / 256;
  return static_cast<int>(want < 1 ? 1 : (want < num_sms * 16LL ? want : num_sms * 16LL));
}

}  // namespace

// Workspace: table int64 [2n + T], slots int32 [2n + T], count int32 [T], cursor int32 [T]; `inverse` doubles as
// the probe-position scratch (int32 view) while the kernels run.  `unique_offsets` [T + 1] receives the per-table
// ranges of `unique_out`; `counts` (optional, int32 [n], zeroed here) the multiplicity of every unique key.
RB_API int rb_segmented_unique(const long long* keys, long long n, const long long* table_offsets, int T, long long* table,
                               int* slots, int* count, int* cursor, int* pos, long long* unique_out, long long* inverse,
                               int* counts, long long* unique_offsets, int* status, int num_sms, cudaStream_t st) {
  if (T <= 0) return -1;
  if (2 * n + T > 0x7fffffffLL) return -2;
  RB_CUDA_CHECK(cudaMemsetAsync(count, 0, sizeof(int) * T, st));
  fill_i64<<<grid_for(2 * n + T, num_sms), 256, 0, st>>>(table, 2 * n + T, kEmpty);
  if (counts && n) RB_CUDA_CHECK(cudaMemsetAsync(counts, 0, sizeof(int) * n, st));
  if (n) seg_unique_insert<<<grid_for(n, num_sms), 256, 0, st>>>(keys, n, table_offsets, T, table, pos, count, status);
  seg_unique_scan<<<1, 32, 0, st>>>(count, T, unique_offsets, cursor);
  seg_unique_assign<<<grid_for(2 * n + T, num_sms), 256, 0, st>>>(table, n, table_offsets, T, unique_offsets, cursor, slots, unique_out);
  if (n) seg_unique_inverse<<<grid_for(n, num_sms), 256, 0, st>>>(pos, n, slots, inverse, counts);
  return static_cast<int>(cudaGetLastError());
}

// offsets [F*B + 1] = exclusive cumsum of lengths.  Step 1 writes new_lengths [world*F*B]; the caller turns them
// into new_offsets (a cumsum) and calls step 2.
RB_API int rb_block_bucketize_count(const long long* offsets, const long long* indices, long long F, long long B, int world,
                                    const long long* block_sizes, long long* new_lengths, cudaStream_t st) {
  const long long FB = F * B;
  if (FB == 0) return 0;
  const long long blocks = (FB * 32 + 255) / 256;
  bucketize_count<<<static_cast<unsigned>(blocks), 256, 0, st>>>(offsets, indices, FB, B, world, block_sizes, new_lengths);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_block_bucketize_fill(const long long* offsets, const long long* indices, const float* weights, long long F, long long B,
                                   int world, const long long* block_sizes, int local_rows, const long long* new_offsets,
                                   long long* new_indices, float* new_weights, long long* unbucketize_permute, cudaStream_t st) {
  const long long FB = F * B;
  if (FB == 0) return 0;
  const long long blocks = (FB * 32 + 255) / 256;
  bucketize_fill<<<static_cast<unsigned>(blocks), 256, 0, st>>>(offsets, indices, weights, FB, B, world, block_sizes, local_rows,
                                                               new_offsets, new_indices, new_weights, unbucketize_permute);
  return static_cast<int>(cudaGetLastError());
}

// Order-preserving compaction: out = values[flags != 0] (values == nullptr: the positions themselves);
// num_out (device int64) receives the count.  Query the temp size with temp == nullptr.
RB_API long long rb_compact_select_temp_bytes(long long n) {
  size_t bytes = 0;
  cub::DeviceSelect::Flagged(nullptr, bytes, static_cast<const long long*>(nullptr), static_cast<const unsigned char*>(nullptr),
                             static_cast<long long*>(nullptr), static_cast<long long*>(nullptr), n);
  size_t b2 = 0;
  thrust::counting_iterator<long long> it(0);
  cub::DeviceSelect::Flagged(nullptr, b2, it, static_cast<const unsigned char*>(nullptr), static_cast<long long*>(nullptr),
                             static_cast<long long*>(nullptr), n);
  return static_cast<long long>(bytes > b2 ? bytes : b2);
}

RB_API int rb_compact_select(const long long* values, const unsigned char* flags, long long n, long long* out, long long* num_out,
                             void* temp, long long temp_bytes, cudaStream_t st) {
  size_t bytes = static_cast<size_t>(temp_bytes);
  if (values) {
    RB_CUDA_CHECK(cub::DeviceSelect::Flagged(temp, bytes, values, flags, out, num_out, n, st));
  } else {
    thrust::counting_iterator<long long> it(0);
    RB_CUDA_CHECK(cub::DeviceSelect::Flagged(temp, bytes, it, flags, out, num_out, n, st));
  }
  return 0;
}

// out[t] = offsets[feature_offsets[t] * B]: the range of table t's ids in the KJT values (feature_offsets [T + 1]).
RB_API int rb_table_range(const long long* offsets, const int* feature_offsets, int T, long long B, long long* out, cudaStream_t st) {
  table_range_kernel<<<(T + 1 + 127) / 128, 128, 0, st>>>(offsets, feature_offsets, T, B, out);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_new_lengths_offsets(const long long* unique_offsets, const int* feature_offsets, int T, long long B, long long total_bags,
                                  long long* new_lengths, long long* new_offsets, int num_sms, cudaStream_t st) {
  new_lengths_kernel<<<grid_for(total_bags + 1, num_sms), 256, 0, st>>>(unique_offsets, feature_offsets, T, B, new_lengths, new_offsets);
  return static_cast<int>(cudaGetLastError());
}
