// Owner-side kernels of the push exchange for dynamic (hash-table backed) embeddings: the received raw keys are
// de-duplicated (sort + run-length encode), probed / inserted in the hash table once per unique key, and the rows are
// stored into the requesters' outputs by slot; in the backward the received gradient rows are summed per unique key
// from local memory and handed to the fused optimizer on slots.  Together with a2a_push.cu this is the id exchange
// fused with the hash probe and the row gather on the owning GPU, and the gradient exchange fused with the
// de-duplicating segment sum and the sparse update.
//
//   rb_a2a_pad_keys        keys beyond the received count <- EMPTY (so that the sort sees one run of empties)
//   rb_fill_tail_i64       buf[i] = value for i >= *n_dev (unique-key list beyond the number of runs)
//   rb_expand_runs         run index of every sorted entry; slot of every received position (through its run)
//   rb_a2a_serve_slots     row(slot) -> requester's output, fp32 table rows converted on the fly
//   rb_rows_segment_add    red[run] = sum of the gradient rows of the run's entries (vector reductions only where a
//                          run spans several thread groups)
//
// Reference flow: training/torch_rec_v2/dynamic_emb/dynamic_emb/distributed/sharding/rw_sharding.py:222-263 (bucketize,
// all-to-all, owner-side unique + find_or_insert + gather, all-to-all back) and batched_dynamicemb_function.py:344-432.
#include "common.cuh"
#include "peer.cuh"
#include "a2a_common.cuh"
#include "tbe_common.cuh"

using namespace rbpeer;
using namespace rbtbe;
using namespace rba2a;

namespace {

constexpr long long EMPTY = -1;

__global__ void pad_keys_kernel(long long* keys, const int* n_dev, int cap) {
  const int n = *n_dev;
  for (int i = n + blockIdx.x * blockDim.x + threadIdx.x; i < cap; i += gridDim.x * blockDim.x) keys[i] = EMPTY;
}

__global__ void fill_tail_kernel(long long* buf, const int* n_dev, int cap, long long value) {
  const int n = *n_dev;
  for (int i = (n < 0 ? 0 : n) + blockIdx.x * blockDim.x + threadIdx.x; i < cap; i += gridDim.x * blockDim.x) buf[i] = value;
}

// one thread per sorted entry: its run (binary search in seg_offsets) -> run_of_sorted[j], slot_of_pos[pos_sorted[j]]
__global__ void expand_runs_kernel(const int* __restrict__ seg_offsets, const int* __restrict__ num_runs,
                                   const int* __restrict__ pos_sorted, const long long* __restrict__ slots_u, int n,
                                   long long* __restrict__ run_of_sorted, long long* __restrict__ slot_of_pos) {
  const int runs = *num_runs;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < n; j += gridDim.x * blockDim.x) {
    int lo = 0, hi = runs;                       // last r with seg_offsets[r] <= j
    while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (seg_offsets[mid] <= j) lo = mid; else hi = mid; }
    run_of_sorted[j] = lo;
    if (slot_of_pos) slot_of_pos[pos_sorted[j]] = slots_u[lo];
  }
}

struct HkvRows {        // where the value rows live (see hkv.cu): slot < hbm_rows in HBM, the rest in mapped host memory
  const float* hbm;
  const float* host;
  long long hbm_rows;
  int row_dim, emb_dim;
};

struct ServeSlotsArgs {
  const long long* slot_of_pos;   // [cap] slot of each received entry (-1: not resident -> default value)
  const long long* recv_meta;
  const int* n_dev;               // entries received
  HkvRows rows;
  float missing_value;
  PeerPtrs out;                   // requester's per-id row list
  long long ld_out;
  PeerPtrs ctl;
  int* loc;
  int world, me;
};

template <typename OT, int G>
__global__ void __launch_bounds__(256) a2a_serve_slots_kernel(const ServeSlotsArgs a) {
  const int e = *reinterpret_cast<volatile int*>(a.loc + LOC_EPOCH + 2) + 1;
  const int n = *a.n_dev;
  const int hl = threadIdx.x & 15;
  const int halves = gridDim.x * (blockDim.x >> 4);
  const int D = a.rows.emb_dim;
  for (int i0 = (blockIdx.x * (blockDim.x >> 4) + (threadIdx.x >> 4)) * G; i0 < n; i0 += halves * G) {
    const float* src[G];
    OT* dst[G];
    bool live[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      src[g] = nullptr; dst[g] = nullptr; live[g] = false;
      const int i = i0 + g;
      if (i < n) {
        const long long s = a.slot_of_pos[i];
        const long long meta = __ldcg(a.recv_meta + i);
        const int r = meta_src(meta);
        const long long j = meta & META_J_MASK;
        dst[g] = reinterpret_cast<OT*>(a.out.p[r]) + j * a.ld_out;
        live[g] = true;
        if (s >= 0) src[g] = (s < a.rows.hbm_rows ? a.rows.hbm + s * a.rows.row_dim
                                                  : a.rows.host + (s - a.rows.hbm_rows) * a.rows.row_dim);
      }
    }
    for (int d0 = hl * 8; d0 < D; d0 += 128) {
      float v[G][8];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        if (src[g]) Vec8<float>::ld(src[g] + d0, v[g]);
        else {
#pragma unroll
          for (int k = 0; k < 8; ++k) v[g][k] = a.missing_value;
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g)
        if (live[g]) Vec8<OT>::st(dst[g] + d0, v[g]);
    }
  }
  if (is_last_block(a.loc, 2)) signal_all(a.ctl, a.loc, 2, e, a.me, a.world);     // phase 2: rows are there
}

// Sorted entries p (grouped by run): red[run_of_sorted[p], :D] += rows[pos_sorted[p], :D].  Every group of G lanes owns CH
// consecutive entries and keeps a running sum while the run stays the same; a run inside one group's range is written
// with a plain store, runs that span groups are accumulated with vector reductions (red must be zero there; the
// caller zeroes it).  Entries whose key is EMPTY (the padded tail of the receive list) are skipped.
template <typename GT, int CH>
__global__ void rows_segment_add_kernel(const GT* __restrict__ rows, long long ld_rows, const long long* __restrict__ run_of,
                                        const int* __restrict__ pos_sorted, const long long* __restrict__ keys_sorted, int n,
                                        int D, int G, float* __restrict__ red) {
  const int gl = threadIdx.x & (G - 1);
  const long long group = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) / G;
  const long long p0 = group * CH;
  if (p0 >= n) return;
  const long long p1 = (p0 + CH < n) ? p0 + CH : n;
  for (int c = gl; c * 4 < D; c += G) {
    long long cur = run_of[p0];
    bool starts_here = (p0 == 0) || (run_of[p0 - 1] != cur);
    bool cur_live = keys_sorted[p0] != EMPTY;
    float ax = 0.f, ay = 0.f, az = 0.f, aw = 0.f;
    for (long long p = p0; p < p1; ++p) {
      const long long k = run_of[p];
      if (k != cur) {
        if (cur_live) {
          float* o = red + cur * D + c * 4;
          if (starts_here) *reinterpret_cast<float4*>(o) = make_float4(ax, ay, az, aw);
          else rb::red_add_v4(o, ax, ay, az, aw);
        }
        cur = k; starts_here = true; cur_live = keys_sorted[p] != EMPTY;
        ax = ay = az = aw = 0.f;
      }
      if (cur_live) {
        const GT* gp = rows + static_cast<long long>(pos_sorted[p]) * ld_rows + c * 4;
        ax += static_cast<float>(gp[0]); ay += static_cast<float>(gp[1]);
        az += static_cast<float>(gp[2]); aw += static_cast<float>(gp[3]);
      }
    }
    if (cur_live) {
      const bool ends_here = (p1 == n) || (run_of[p1] != cur);
      float* o = red + cur * D + c * 4;
      if (starts_here && ends_here) *reinterpret_cast<float4*>(o) = make_float4(ax, ay, az, aw);
      else rb::red_add_v4(o, ax, ay, az, aw);
    }
  }
}

}  // namespace

RB_API int rb_a2a_pad_keys(long long* keys, const int* n_dev, int cap, cudaStream_t st) {
  if (cap <= 0) return 0;
  pad_keys_kernel<<<64, 256, 0, st>>>(keys, n_dev, cap);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_fill_tail_i64(long long* buf, const int* n_dev, int cap, long long value, cudaStream_t st) {
  if (cap <= 0) return 0;
  fill_tail_kernel<<<64, 256, 0, st>>>(buf, n_dev, cap, value);
  return static_cast<int>(cudaGetLastError());
}

// n sorted entries; seg_offsets / num_runs from rb_sort_segments.  slot_of_pos / slots_u may be null (runs only).
RB_API int rb_expand_runs(const int* seg_offsets, const int* num_runs, const int* pos_sorted, const long long* slots_u, int n,
                          long long* run_of_sorted, long long* slot_of_pos, cudaStream_t st) {
  if (n <= 0) return 0;
  int blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  expand_runs_kernel<<<blocks, 256, 0, st>>>(seg_offsets, num_runs, pos_sorted, slots_u, n, run_of_sorted,
                                            slots_u ? slot_of_pos : nullptr);
  return static_cast<int>(cudaGetLastError());
}

// Stores row(slot_of_pos[i])[:emb_dim] of a hash table (fp32 rows of row_dim floats; slots >= hbm_rows live in the mapped
// host tier) into the requester named by recv_meta[i], for the first *n_dev received entries, and raises the exchange's
// "rows" flag.  Must be ordered after the payload wait (rb_a2a_wait phase 1).
RB_API int rb_a2a_serve_slots(const long long* slot_of_pos, const long long* recv_meta, const int* n_dev, int cap,
                              const float* values_hbm, const float* values_host, long long hbm_rows, int row_dim, int emb_dim,
                              float missing_value, const unsigned long long* out_ptrs, int out_dtype, long long ld_out,
                              const unsigned long long* ctl, int* loc, int world, int me, int num_sms, cudaStream_t st) {
  if (world > MAX_RANKS || emb_dim % 8 || row_dim % 4) return -1;
  ServeSlotsArgs a;
  a.slot_of_pos = slot_of_pos; a.recv_meta = recv_meta; a.n_dev = n_dev;
  a.rows = HkvRows{values_hbm, values_host, hbm_rows, row_dim, emb_dim};
  a.missing_value = missing_value; a.out = to_ptrs(out_ptrs, world); a.ld_out = ld_out;
  a.ctl = to_ptrs(ctl, world); a.loc = loc; a.world = world; a.me = me;
  constexpr int G = 4;
  long long b = ((static_cast<long long>(cap) + G - 1) / G + 15) / 16;
  const long long cap_b = static_cast<long long>(num_sms > 0 ? num_sms : 148) * 8;
  if (b > cap_b) b = cap_b;
  if (b < 1) b = 1;
  const int grid = static_cast<int>(b);
  switch (out_dtype) {
    case DT_F32: a2a_serve_slots_kernel<float, G><<<grid, 256, 0, st>>>(a); break;
    case DT_F16: a2a_serve_slots_kernel<__half, G><<<grid, 256, 0, st>>>(a); break;
    case DT_BF16: a2a_serve_slots_kernel<__nv_bfloat16, G><<<grid, 256, 0, st>>>(a); break;
    default: return -1;
  }
  return static_cast<int>(cudaGetLastError());
}

// red[run, :D] = sum over the run's entries of rows[pos_sorted[p], :D]; red (fp32, [>= runs][D]) must be zeroed by the caller.
RB_API int rb_rows_segment_add(const void* rows, int g_dtype, long long ld_rows, const long long* run_of_sorted,
                               const int* pos_sorted, const long long* keys_sorted, int n, int D, float* red,
                               cudaStream_t st) {
  if (n <= 0) return 0;
  if (D % 4) return -1;
  constexpr int CH = 64;
  int G = 1;
  while (G < 32 && G * 4 < D) G <<= 1;
  const long long groups = (static_cast<long long>(n) + CH - 1) / CH;
  const unsigned blocks = static_cast<unsigned>((groups * G + 255) / 256);
  switch (g_dtype) {
    case DT_F32: rows_segment_add_kernel<float, CH><<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(rows), ld_rows, run_of_sorted, pos_sorted, keys_sorted, n, D, G, red); break;
    case DT_F16: rows_segment_add_kernel<__half, CH><<<blocks, 256, 0, st>>>(reinterpret_cast<const __half*>(rows), ld_rows, run_of_sorted, pos_sorted, keys_sorted, n, D, G, red); break;
    case DT_BF16: rows_segment_add_kernel<__nv_bfloat16, CH><<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(rows), ld_rows, run_of_sorted, pos_sorted, keys_sorted, n, D, G, red); break;
    default: return -1;
  }
  return static_cast<int>(cudaGetLastError());
}
