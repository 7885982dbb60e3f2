// HKV-style dynamic embedding hash table on the GPU.
//
// Layout: `capacity` slots grouped in buckets of 128.  Per slot: 64-bit key, 64-bit score, 8-bit
// digest; the value row of slot s ([embedding | optimizer state], row_dim floats) lives at a fixed
// address (values_hbm for s < hbm_rows, else a host-mapped pinned buffer), so slot numbers double as
// stable row pointers for the gather and the fused optimizer kernels.
//
// One warp serves one key under a per-bucket lock (bounded acquire): the 128 digests of the bucket are
// read as one 4-byte word per lane, candidates are confirmed against the key, an empty slot is
// claimed, or - when the bucket is full - the lowest-score slot is evicted (its key / score / row are
// appended to the caller's eviction buffers so a storage tier below can take them).  New rows are
// initialised in the same kernel by a counter-based generator keyed on (seed, key, column), so a
// key's initial vector does not depend on insertion order or sharding.
//
// Reference API surface (the implementation is an absent submodule there):
// training/torch_rec_v2/dynamic_emb/csrc/hkv_variable.cpp:353-717 (find, find_or_insert,
// insert_and_evict, assign, accum_or_assign, erase, clear, reserve, export_batch[_if], size),
// csrc/ops/{load_from_pointer,load_or_initialize_embeddings,Rowwise_adagrad_update,Adam_update,
// Adagrad_update,sgd_update,device_timestamp}, csrc/initializer_generators.h.
#include "common.cuh"

namespace {

constexpr int BUCKET = 128;
constexpr unsigned long long EMPTY_KEY = 0xFFFFFFFFFFFFFFFFull;
constexpr unsigned EMPTY_DIGEST = 0xFFu;

enum EvictStrategy : int { EV_LRU = 0, EV_LFU = 1, EV_EPOCH_LRU = 2, EV_EPOCH_LFU = 3, EV_CUSTOMIZED = 4 };
enum InitMode : int { INIT_UNIFORM = 0, INIT_NORMAL = 1, INIT_TRUNC_NORMAL = 2, INIT_CONSTANT = 3, INIT_DEBUG = 4 };
enum OptType : int { OPT_SGD = 0, OPT_ROWWISE_ADAGRAD = 1, OPT_ADAGRAD = 2, OPT_ADAM = 3 };
enum KeyStatus : unsigned char { ST_FOUND = 0, ST_INSERTED = 1, ST_EVICTED_OTHER = 2, ST_REJECTED = 3, ST_MISSING = 4,
                                 ST_LOCK_TIMEOUT = 5 };

struct HkvTable {
  unsigned long long* keys;
  unsigned long long* scores;
  unsigned char* digests;
  int* locks;
  float* values_hbm;
  float* values_host;
  long long hbm_rows;
  long long capacity;
  long long num_buckets;
  int row_dim;
  int emb_dim;
  int evict_strategy;
  unsigned long long* size;
  // Launch stamps: find_or_insert writes `epoch` into touch[slot] of every slot it returns, and never evicts a slot
  // stamped with the current epoch.  Slot numbers handed out by one launch therefore stay valid for the kernels that
  // consume them (gather, scatter, update): a later warp of the same launch cannot evict a key inserted or found by
  // an earlier one.  touch may be null (no protection).
  unsigned* touch;
  unsigned epoch;
  // counters[0..3]: keys inserted into an empty slot, keys that displaced a resident key, keys rejected, bucket-lock
  // timeouts - accumulated over the table's life (may be null)
  unsigned long long* counters;
};

constexpr unsigned LOCKED_STAMP = 0xFFFFFFFFu;     // touch value of a slot pinned by rb_hkv_lock: never a victim

struct InitArgs {
  int mode;
  float lower, upper, mean, stddev, value;
  unsigned long long seed;
  float state_init;   // initial value of the optimizer-state columns
};

__device__ __forceinline__ unsigned long long hash64(unsigned long long k) {
  k ^= k >> 33; k *= 0xff51afd7ed558ccdull; k ^= k >> 33; k *= 0xc4ceb9fe1a85ec53ull; k ^= k >> 33;
  return k;
}
__device__ __forceinline__ unsigned digest_of(unsigned long long h) {
  unsigned d = static_cast<unsigned>(h >> 32) & 0xFFu;
  return d == EMPTY_DIGEST ? 0xFEu : d;
}
__device__ __forceinline__ float* row_ptr(const HkvTable& t, long long slot) {
  return slot < t.hbm_rows ? t.values_hbm + slot * t.row_dim : t.values_host + (slot - t.hbm_rows) * t.row_dim;
}
__device__ __forceinline__ unsigned long long device_timestamp() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// one prefetch per 128 bytes of the `n_floats` floats starting at p, never beyond them (lanes 0..)
__device__ __forceinline__ void prefetch_row(const float* p, int n_floats, int lane) {
  if (lane * 128 < n_floats * 4) asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(p) + lane * 128));
}
// keys a warp takes per step: 32 when there is enough work for every warp, fewer (a power of two) for short lists so
// that the keys still spread over all warps
__device__ __forceinline__ int chunk_width(long long n, long long warps_total) {
  int cw = 32;
  while (cw > 1 && static_cast<long long>(cw) * warps_total > n) cw >>= 1;
  return cw;
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
__device__ __forceinline__ float u01(unsigned long long seed, unsigned long long key, unsigned col, unsigned stream) {
  unsigned long long x = hash64(key ^ (seed * 0x9E3779B97F4A7C15ull) ^ (static_cast<unsigned long long>(col) << 32) ^ stream);
  return (static_cast<float>(x >> 40) + 0.5f) * (1.0f / 16777216.0f);
}
__device__ __forceinline__ float init_value(const InitArgs& a, unsigned long long key, int col) {
  switch (a.mode) {
    case INIT_UNIFORM: return a.lower + (a.upper - a.lower) * u01(a.seed, key, col, 0);
    case INIT_NORMAL: {
      const float r = sqrtf(-2.f * __logf(u01(a.seed, key, col, 1)));
      return a.mean + a.stddev * r * __cosf(6.2831853f * u01(a.seed, key, col, 2));
    }
    case INIT_TRUNC_NORMAL: {
      float v = 0.f;
      for (unsigned it = 0; it < 8; ++it) {
        const float r = sqrtf(-2.f * __logf(u01(a.seed, key, col, 1 + 2 * it)));
        v = r * __cosf(6.2831853f * u01(a.seed, key, col, 2 + 2 * it));
        if (fabsf(v) <= 2.f) break;
        v = fminf(fmaxf(v, -2.f), 2.f);
      }
      return a.mean + a.stddev * v;
    }
    case INIT_CONSTANT: return a.value;
    default: return static_cast<float>(key % 100000ull);   // debug: value = key % 100000
  }
}

__device__ __forceinline__ bool lock_bucket(int* lock, int lane, int* status) {
  int ok = 0;
  if (lane == 0) {
    for (int it = 0; it < (1 << 20); ++it) {
      if (atomicCAS(lock, 0, 1) == 0) { ok = 1; break; }
      __nanosleep(64);
    }
    if (!ok && status) atomicCAS(status, 0, RB_ERR_PEER_TIMEOUT);
    __threadfence();
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void unlock_bucket(int* lock, int lane) {
  __syncwarp();
  if (lane == 0) { __threadfence(); atomicExch(lock, 0); }
}

// position of `key` in bucket b, or -1 (warp-uniform result)
__device__ __forceinline__ int find_in_bucket(const HkvTable& t, long long b, unsigned long long key, unsigned dg,
                                              unsigned d4, int lane) {
  int mine = -1;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (((d4 >> (8 * j)) & 0xFFu) == dg && __ldcg(t.keys + b * BUCKET + lane * 4 + j) == key) mine = lane * 4 + j;
  const unsigned m = __ballot_sync(0xffffffffu, mine >= 0);
  if (!m) return -1;
  return __shfl_sync(0xffffffffu, mine, __ffs(m) - 1);
}

__device__ __forceinline__ unsigned long long new_score(int strategy, unsigned long long old, bool is_new,
                                                        const unsigned long long* scores_in, long long i) {
  switch (strategy) {
    case EV_LRU: return device_timestamp();
    case EV_LFU: return (is_new ? 0ull : old) + (scores_in ? scores_in[i] : 1ull);
    default: return scores_in ? scores_in[i] : (is_new ? 1ull : old);
  }
}

// ---------------------------------------------------------------------------
// find / find_or_insert  (mode: 0 = find only, 1 = find or insert)
// ---------------------------------------------------------------------------
struct EvictOut {
  unsigned long long* keys;
  unsigned long long* scores;
  float* values;          // [cap][row_dim]
  int* count;
  int cap;
};

__global__ void __launch_bounds__(256)
hkv_find_or_insert_kernel(HkvTable t, const unsigned long long* __restrict__ keys, long long n, int insert,
                          int update_score, const unsigned long long* __restrict__ scores_in,
                          long long* __restrict__ out_slots, unsigned char* __restrict__ out_status, InitArgs init,
                          EvictOut ev, int* status, const int* __restrict__ n_dev) {
  const int lane = threadIdx.x & 31;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  if (n_dev && *n_dev < n) n = *n_dev;          // the number of keys may live on the device (no host read)
  // A find-only launch changes no key, digest or slot, so it takes no bucket lock even when it refreshes scores or
  // stamps the slots it found (callers keep launches on one table in one stream).
  const bool need_lock = insert != 0;
  const bool stamp = insert || (update_score & 2);
  const bool upd_score = (update_score & 1) != 0;
  long long d_size = 0;                          // lane 0: outcome counts of this warp, flushed once at the end
  unsigned long long c_out[4] = {0ull, 0ull, 0ull, 0ull};
  // Keys are taken 32 at a time (one coalesced load; empty keys cost nothing more) and every lane prefetches the
  // bucket head of its key, so the dependent loads of the serial per-key work below mostly hit L2.
  const int cw = chunk_width(n, warps_total);
  for (long long base = ((static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5) * cw; base < n;
       base += warps_total * cw) {
    const long long il = base + lane;
    const bool mine = lane < cw && il < n;
    const unsigned long long kl = mine ? keys[il] : EMPTY_KEY;
    if (kl == EMPTY_KEY) {
      if (mine) { out_slots[il] = -1; if (out_status) out_status[il] = ST_MISSING; }
    } else {
      const long long bl = static_cast<long long>(hash64(kl) & static_cast<unsigned long long>(t.num_buckets - 1));
      prefetch_l2(t.digests + bl * BUCKET);
      if (need_lock) prefetch_l2(t.locks + bl);
    }
    unsigned pending = __ballot_sync(0xffffffffu, kl != EMPTY_KEY);
  while (pending) {
    const int src = __ffs(pending) - 1;
    pending &= pending - 1;
    const unsigned long long key = __shfl_sync(0xffffffffu, kl, src);
    const long long i = base + src;
    const unsigned long long h = hash64(key);
    const long long b = static_cast<long long>(h & static_cast<unsigned long long>(t.num_buckets - 1));
    const unsigned dg = digest_of(h);
    if (need_lock && !lock_bucket(t.locks + b, lane, status)) {
      if (lane == 0) { out_slots[i] = -1; if (out_status) out_status[i] = ST_LOCK_TIMEOUT; c_out[3] += 1; }
      continue;
    }
    const unsigned d4 = __ldcg(reinterpret_cast<const unsigned*>(t.digests + b * BUCKET) + lane);  // L2: L1 may be stale
    int pos = find_in_bucket(t, b, key, dg, d4, lane);
    unsigned char st = ST_FOUND;
    if (pos >= 0) {
      if (lane == 0) {
        const long long s = b * BUCKET + pos;
        if (upd_score) t.scores[s] = new_score(t.evict_strategy, __ldcg(t.scores + s), false, scores_in, i);
        if (stamp && t.touch && t.touch[s] != LOCKED_STAMP) t.touch[s] = t.epoch;
      }
    } else if (!insert) {
      st = ST_MISSING;
    } else {
      // ---- claim an empty slot
      int mine = -1;
#pragma unroll
      for (int j = 3; j >= 0; --j)
        if (((d4 >> (8 * j)) & 0xFFu) == EMPTY_DIGEST) mine = lane * 4 + j;
      unsigned m = __ballot_sync(0xffffffffu, mine >= 0);
      const unsigned long long sc_new = new_score(t.evict_strategy, 0ull, true, scores_in, i);
      if (m) {
        pos = __shfl_sync(0xffffffffu, mine, __ffs(m) - 1);
        st = ST_INSERTED;
        if (lane == 0) d_size += 1;
      } else {
        // ---- bucket full: evict the lowest score
        unsigned long long best = ~0ull;
        int best_pos = lane * 4;
        bool any_free = false;                   // a slot not handed out by this launch
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const long long sl = b * BUCKET + lane * 4 + j;
          if (t.touch) { const unsigned tv = __ldcg(t.touch + sl); if (tv == t.epoch || tv == LOCKED_STAMP) continue; }
          const unsigned long long s = __ldcg(t.scores + sl);
          if (!any_free || s < best) { best = s; best_pos = lane * 4 + j; }
          any_free = true;
        }
        if (!any_free) best = ~0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const unsigned long long ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int op = __shfl_xor_sync(0xffffffffu, best_pos, o);
          if (ob < best || (ob == best && op < best_pos)) { best = ob; best_pos = op; }
        }
        const bool all_stamped = __ballot_sync(0xffffffffu, any_free) == 0u;
        if (all_stamped || (t.evict_strategy != EV_LRU && sc_new < best)) {
          st = ST_REJECTED;    // the newcomer scores lower than everything resident, or every slot was handed out by this launch
        } else {
          pos = best_pos;
          st = ST_EVICTED_OTHER;
          const long long s = b * BUCKET + pos;
          int slot_out = -1;
          if (ev.count) {
            if (lane == 0) slot_out = atomicAdd(ev.count, 1);
            slot_out = __shfl_sync(0xffffffffu, slot_out, 0);
            if (slot_out < ev.cap) {
              if (lane == 0) { ev.keys[slot_out] = __ldcg(t.keys + s); ev.scores[slot_out] = __ldcg(t.scores + s); }
              const float* src = row_ptr(t, s);
              for (int c = lane; c < t.row_dim; c += 32) ev.values[static_cast<long long>(slot_out) * t.row_dim + c] = src[c];
            } else if (lane == 0 && status) {
              atomicCAS(status, 0, RB_ERR_CAPACITY);
            }
          }
        }
      }
      if (st == ST_INSERTED || st == ST_EVICTED_OTHER) {
        const long long s = b * BUCKET + pos;
        float* row = row_ptr(t, s);
        for (int c = lane; c < t.row_dim; c += 32) row[c] = c < t.emb_dim ? init_value(init, key, c) : init.state_init;
        if (lane == 0) {
          t.keys[s] = key;
          t.scores[s] = sc_new;
          t.digests[s] = static_cast<unsigned char>(dg);
          if (t.touch) t.touch[s] = t.epoch;
        }
      }
    }
    if (need_lock) unlock_bucket(t.locks + b, lane);
    if (lane == 0) {
      out_slots[i] = (st == ST_MISSING || st == ST_REJECTED) ? -1 : b * BUCKET + pos;
      if (out_status) out_status[i] = st;
      c_out[0] += st == ST_INSERTED; c_out[1] += st == ST_EVICTED_OTHER; c_out[2] += st == ST_REJECTED;
    }
  }
  }
  if (lane == 0) {
    if (d_size) atomicAdd(t.size, static_cast<unsigned long long>(d_size));
    if (t.counters) {
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (c_out[c]) atomicAdd(t.counters + c, c_out[c]);
    }
  }
}

// erase keys (slot becomes empty; value row is left as is)
__global__ void __launch_bounds__(256)
hkv_erase_kernel(HkvTable t, const unsigned long long* __restrict__ keys, long long n, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  long long erased = 0;                           // lane 0
  const int cw = chunk_width(n, warps_total);
  for (long long base = ((static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5) * cw; base < n;
       base += warps_total * cw) {
    const long long il = base + lane;
    const unsigned long long kl = (lane < cw && il < n) ? keys[il] : EMPTY_KEY;
    if (kl != EMPTY_KEY) {
      const long long bl = static_cast<long long>(hash64(kl) & static_cast<unsigned long long>(t.num_buckets - 1));
      prefetch_l2(t.digests + bl * BUCKET);
      prefetch_l2(t.locks + bl);
    }
    unsigned pending = __ballot_sync(0xffffffffu, kl != EMPTY_KEY);
    while (pending) {
      const int src = __ffs(pending) - 1;
      pending &= pending - 1;
      const unsigned long long key = __shfl_sync(0xffffffffu, kl, src);
      const unsigned long long h = hash64(key);
      const long long b = static_cast<long long>(h & static_cast<unsigned long long>(t.num_buckets - 1));
      if (!lock_bucket(t.locks + b, lane, status)) continue;
      const unsigned d4 = __ldcg(reinterpret_cast<const unsigned*>(t.digests + b * BUCKET) + lane);  // L2: L1 may be stale
      const int pos = find_in_bucket(t, b, key, digest_of(h), d4, lane);
      if (pos >= 0 && lane == 0) {
        const long long s = b * BUCKET + pos;
        t.keys[s] = EMPTY_KEY;
        t.scores[s] = 0ull;
        t.digests[s] = static_cast<unsigned char>(EMPTY_DIGEST);
        erased += 1;
      }
      unlock_bucket(t.locks + b, lane);
    }
  }
  if (lane == 0 && erased) atomicAdd(t.size, static_cast<unsigned long long>(-erased));
}

// pin == 1: resident keys become ineligible as eviction victims until unpinned (flags[i] = found; slots[i] = slot or -1);
// pin == 0: the pin is lifted.  The reference's lock / unlock hide a key from concurrent writers for the same purpose:
// rows that a caller holds pointers to must not be recycled under it (csrc/hkv_variable.h:178-190).
__global__ void __launch_bounds__(256)
hkv_pin_kernel(HkvTable t, const unsigned long long* __restrict__ keys, long long n, int pin, long long* __restrict__ out_slots,
               unsigned char* __restrict__ flags, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; i < n; i += warps_total) {
    const unsigned long long key = keys[i];
    long long slot = -1;
    if (key != EMPTY_KEY && t.touch) {
      const unsigned long long h = hash64(key);
      const long long b = static_cast<long long>(h & static_cast<unsigned long long>(t.num_buckets - 1));
      if (lock_bucket(t.locks + b, lane, status)) {
        const unsigned d4 = __ldcg(reinterpret_cast<const unsigned*>(t.digests + b * BUCKET) + lane);
        const int pos = find_in_bucket(t, b, key, digest_of(h), d4, lane);
        if (pos >= 0) {
          slot = b * BUCKET + pos;
          if (lane == 0) t.touch[slot] = pin ? LOCKED_STAMP : 0u;
        }
        unlock_bucket(t.locks + b, lane);
      }
    }
    if (lane == 0) {
      if (out_slots) out_slots[i] = slot;
      if (flags) flags[i] = slot >= 0 ? 1 : 0;
    }
  }
}

__global__ void hkv_clear_kernel(HkvTable t) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long s = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; s < t.capacity; s += stride) {
    t.keys[s] = EMPTY_KEY;
    t.scores[s] = 0ull;
    t.digests[s] = static_cast<unsigned char>(EMPTY_DIGEST);
    if (t.touch) t.touch[s] = 0u;
    if (s < t.num_buckets) t.locks[s] = 0;
    if (s == 0) *t.size = 0ull;
  }
}

// ---------------------------------------------------------------------------
// rows by slot: gather (optionally a column window) and scatter-assign / accumulate
// ---------------------------------------------------------------------------
template <typename OT>
__global__ void hkv_gather_kernel(HkvTable t, const long long* __restrict__ slots, long long n, int col0, int cols,
                                  OT* __restrict__ out, long long ld_out, float missing_value) {
  const int lane = threadIdx.x & 31;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  // rows sit at random places of a table far larger than the TLB reach: the slot of the row after next is loaded and
  // the next row's lines are prefetched while the current row is copied
  long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  long long s = i < n ? slots[i] : -1;
  long long s_next = i + warps_total < n ? slots[i + warps_total] : -1;
  for (; i < n; i += warps_total) {
    const long long s_after = i + 2 * warps_total < n ? slots[i + 2 * warps_total] : -1;
    if (s_next >= 0) prefetch_row(row_ptr(t, s_next) + col0, cols, lane);
    OT* o = out + i * ld_out;
    if (s < 0) {
      for (int c = lane; c < cols; c += 32) o[c] = static_cast<OT>(missing_value);
    } else {
      const float* src = row_ptr(t, s) + col0;
      for (int c = lane; c < cols; c += 32) o[c] = static_cast<OT>(src[c]);
    }
    s = s_next;
    s_next = s_after;
  }
}

// mode 0: row[col0:col0+cols] = in ; mode 1: += in
__global__ void hkv_scatter_kernel(HkvTable t, const long long* __restrict__ slots, long long n, int col0, int cols,
                                   const float* __restrict__ in, long long ld_in, int mode) {
  const int lane = threadIdx.x & 31;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; i < n; i += warps_total) {
    const long long s = slots[i];
    if (s < 0) continue;
    float* dst = row_ptr(t, s) + col0;
    const float* src = in + i * ld_in;
    for (int c = lane; c < cols; c += 32) dst[c] = mode ? dst[c] + src[c] : src[c];
  }
}

// ---------------------------------------------------------------------------
// fused optimizer on row pointers: row = [w (dim) | state]
//   SGD: no state; row-wise Adagrad: state[0] = sum of mean(g^2); Adagrad: state[dim]; Adam: m[dim], v[dim]
// ---------------------------------------------------------------------------
struct OptArgs { int type; float lr, eps, beta1, beta2, weight_decay, bc1, bc2; };

template <typename GT>
__global__ void hkv_update_kernel(HkvTable t, const long long* __restrict__ slots, long long n,
                                  const GT* __restrict__ grads, long long ld_g, OptArgs o) {
  const int lane = threadIdx.x & 31;
  const int D = t.emb_dim;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  long long s_cur = i < n ? slots[i] : -1;
  long long s_next = i + warps_total < n ? slots[i + warps_total] : -1;
  for (; i < n; i += warps_total) {
    const long long s = s_cur;
    const long long s_after = i + 2 * warps_total < n ? slots[i + 2 * warps_total] : -1;
    if (s_next >= 0) prefetch_row(row_ptr(t, s_next), t.row_dim, lane);     // next row's lines while this one is updated
    s_cur = s_next;
    s_next = s_after;
    if (s < 0) continue;
    float* row = row_ptr(t, s);
    const GT* g = grads + i * ld_g;
    if (o.type == OPT_ROWWISE_ADAGRAD) {
      float ss = 0.f;
      for (int c = lane; c < D; c += 32) { const float gv = static_cast<float>(g[c]); ss += gv * gv; }
      ss = rb::warp_sum(ss);
      const float acc = row[D] + ss / static_cast<float>(D);
      __syncwarp();
      if (lane == 0) row[D] = acc;
      const float mult = o.lr / (sqrtf(acc) + o.eps);
      for (int c = lane; c < D; c += 32) row[c] -= mult * static_cast<float>(g[c]);
    } else if (o.type == OPT_SGD) {
      for (int c = lane; c < D; c += 32) row[c] -= o.lr * (static_cast<float>(g[c]) + o.weight_decay * row[c]);
    } else if (o.type == OPT_ADAGRAD) {
      for (int c = lane; c < D; c += 32) {
        const float gv = static_cast<float>(g[c]);
        const float a = row[D + c] + gv * gv;
        row[D + c] = a;
        row[c] -= o.lr * gv / (sqrtf(a) + o.eps);
      }
    } else {
      // Adam with decoupled weight decay, as the reference's Adam optimizer applies it
      // (dynamic_emb csrc/dynamic_emb_op.cpp:1602 decay_factor = 1 - lr * weight_decay; csrc/ops/AdamW_update/AdamW_update_kernel.h:74)
      const float decay = 1.f - o.lr * o.weight_decay;
      for (int c = lane; c < D; c += 32) {
        const float gv = static_cast<float>(g[c]);
        const float m = o.beta1 * row[D + c] + (1.f - o.beta1) * gv;
        const float v = o.beta2 * row[2 * D + c] + (1.f - o.beta2) * gv * gv;
        row[D + c] = m;
        row[2 * D + c] = v;
        row[c] = row[c] * decay - (o.lr / o.bc1) * m / (sqrtf(v / o.bc2) + o.eps);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// export: compact occupied slots of [slot0, slot0 + count) whose score >= min_score
// ---------------------------------------------------------------------------
__global__ void hkv_export_kernel(HkvTable t, long long slot0, long long count, unsigned long long min_score,
                                  unsigned long long* __restrict__ out_keys, unsigned long long* __restrict__ out_scores,
                                  float* __restrict__ out_values, long long* __restrict__ out_slots, int* counter,
                                  int out_cap) {
  const int lane = threadIdx.x & 31;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; w * 32 < count; w += warps_total) {
    const long long s = slot0 + w * 32 + lane;
    const bool live = (w * 32 + lane < count) && s < t.capacity && t.keys[s] != EMPTY_KEY && t.scores[s] >= min_score;
    const unsigned m = __ballot_sync(0xffffffffu, live);
    if (!m) continue;
    int base = 0;
    if (lane == 0) base = atomicAdd(counter, __popc(m));
    base = __shfl_sync(0xffffffffu, base, 0);
    const int my = base + __popc(m & ((1u << lane) - 1));
    if (live && my < out_cap) {
      out_keys[my] = t.keys[s];
      if (out_scores) out_scores[my] = t.scores[s];
      if (out_slots) out_slots[my] = s;
    }
    if (out_values) {
      for (int l = 0; l < 32; ++l) {
        if (!((m >> l) & 1u)) continue;
        const int dst = base + __popc(m & ((1u << l) - 1));
        if (dst >= out_cap) continue;
        const float* src = row_ptr(t, slot0 + w * 32 + l);
        for (int c = lane; c < t.row_dim; c += 32) out_values[static_cast<long long>(dst) * t.row_dim + c] = src[c];
      }
    }
  }
}

// re-insert every live entry of `src` into the (larger, empty) table `dst` keeping value rows and scores
__global__ void __launch_bounds__(256) hkv_rehash_kernel(HkvTable src, HkvTable dst, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long s = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; s < src.capacity; s += warps_total) {
    const unsigned long long key = src.keys[s];
    if (key == EMPTY_KEY) continue;
    const unsigned long long h = hash64(key);
    const long long b = static_cast<long long>(h & static_cast<unsigned long long>(dst.num_buckets - 1));
    if (!lock_bucket(dst.locks + b, lane, status)) continue;
    const unsigned d4 = __ldcg(reinterpret_cast<const unsigned*>(dst.digests + b * BUCKET) + lane);
    int mine = -1;
#pragma unroll
    for (int j = 3; j >= 0; --j)
      if (((d4 >> (8 * j)) & 0xFFu) == EMPTY_DIGEST) mine = lane * 4 + j;
    const unsigned m = __ballot_sync(0xffffffffu, mine >= 0);
    if (m) {
      const int pos = __shfl_sync(0xffffffffu, mine, __ffs(m) - 1);
      const long long d = b * BUCKET + pos;
      const float* from = row_ptr(src, s);
      float* to = row_ptr(dst, d);
      for (int c = lane; c < src.row_dim; c += 32) to[c] = from[c];
      if (lane == 0) {
        dst.keys[d] = key;
        dst.scores[d] = src.scores[s];
        dst.digests[d] = static_cast<unsigned char>(digest_of(h));
        atomicAdd(dst.size, 1ull);
      }
    } else if (lane == 0 && status) {
      atomicCAS(status, 0, RB_ERR_CAPACITY);
    }
    unlock_bucket(dst.locks + b, lane);
  }
}

__global__ void device_timestamp_kernel(unsigned long long* out) { *out = device_timestamp(); }

inline int warp_grid(long long n, int num_sms) {
  long long b = (n * 32 + 255) / 256;
  const long long cap = static_cast<long long>(num_sms > 0 ? num_sms : 148) * 8;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace

// The table descriptor is passed as a flat array of 16 64-bit words (see recsdk_b200/dynamic/hkv.py):
// keys, scores, digests, locks, values_hbm, values_host, hbm_rows, capacity, num_buckets, row_dim, emb_dim,
// evict_strategy, size, touch (launch stamps, may be 0), epoch (stamp of the current launch), counters (may be 0)
static HkvTable unpack(const long long* d) {
  HkvTable t;
  t.keys = reinterpret_cast<unsigned long long*>(d[0]);
  t.scores = reinterpret_cast<unsigned long long*>(d[1]);
  t.digests = reinterpret_cast<unsigned char*>(d[2]);
  t.locks = reinterpret_cast<int*>(d[3]);
  t.values_hbm = reinterpret_cast<float*>(d[4]);
  t.values_host = reinterpret_cast<float*>(d[5]);
  t.hbm_rows = d[6]; t.capacity = d[7]; t.num_buckets = d[8];
  t.row_dim = static_cast<int>(d[9]); t.emb_dim = static_cast<int>(d[10]); t.evict_strategy = static_cast<int>(d[11]);
  t.size = reinterpret_cast<unsigned long long*>(d[12]);
  t.touch = reinterpret_cast<unsigned*>(d[13]);
  t.epoch = static_cast<unsigned>(d[14]);
  t.counters = reinterpret_cast<unsigned long long*>(d[15]);
  return t;
}

RB_API int rb_hkv_clear(const long long* desc, int num_sms, cudaStream_t st) {
  HkvTable t = unpack(desc);
  hkv_clear_kernel<<<(num_sms > 0 ? num_sms : 148) * 4, 256, 0, st>>>(t);
  return static_cast<int>(cudaGetLastError());
}

// insert == 0: find (out_slots = -1 for missing keys).  insert == 1: find_or_insert; rows of new keys are
// initialised; when a full bucket forces an eviction the victim is appended to ev_* (ev_count may be null).
RB_API int rb_hkv_find_or_insert(const long long* desc, const void* keys, long long n, int insert, int update_score,
                                 const void* scores_in, long long* out_slots, void* out_status, int init_mode,
                                 float lower, float upper, float mean, float stddev, float value,
                                 long long seed, float state_init, void* ev_keys, void* ev_scores, float* ev_values,
                                 int* ev_count, int ev_cap, int num_sms, int* status, cudaStream_t st) {
  if (n == 0) return 0;
  HkvTable t = unpack(desc);
  InitArgs ia{init_mode, lower, upper, mean, stddev, value, static_cast<unsigned long long>(seed), state_init};
  EvictOut ev{reinterpret_cast<unsigned long long*>(ev_keys), reinterpret_cast<unsigned long long*>(ev_scores), ev_values,
              ev_count, ev_cap};
  hkv_find_or_insert_kernel<<<warp_grid(n, num_sms), 256, 0, st>>>(
      t, reinterpret_cast<const unsigned long long*>(keys), n, insert, update_score,
      reinterpret_cast<const unsigned long long*>(scores_in), out_slots, reinterpret_cast<unsigned char*>(out_status), ia,
      ev, status, nullptr);
  return static_cast<int>(cudaGetLastError());
}

// Same with the key count on the device: the first min(n_max, *n_dev) keys are served (no host synchronisation between
// the de-duplication that produced the count and the probe).
RB_API int rb_hkv_find_or_insert_n(const long long* desc, const void* keys, long long n_max, const int* n_dev, int insert,
                                   int update_score, const void* scores_in, long long* out_slots, void* out_status,
                                   int init_mode, float lower, float upper, float mean, float stddev, float value,
                                   long long seed, float state_init, void* ev_keys, void* ev_scores, float* ev_values,
                                   int* ev_count, int ev_cap, int num_sms, int* status, cudaStream_t st) {
  if (n_max == 0) return 0;
  HkvTable t = unpack(desc);
  InitArgs ia{init_mode, lower, upper, mean, stddev, value, static_cast<unsigned long long>(seed), state_init};
  EvictOut ev{reinterpret_cast<unsigned long long*>(ev_keys), reinterpret_cast<unsigned long long*>(ev_scores), ev_values,
              ev_count, ev_cap};
  hkv_find_or_insert_kernel<<<warp_grid(n_max, num_sms), 256, 0, st>>>(
      t, reinterpret_cast<const unsigned long long*>(keys), n_max, insert, update_score,
      reinterpret_cast<const unsigned long long*>(scores_in), out_slots, reinterpret_cast<unsigned char*>(out_status), ia,
      ev, status, n_dev);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_hkv_pin(const long long* desc, const void* keys, long long n, int pin, long long* out_slots, void* flags,
                      int num_sms, int* status, cudaStream_t st) {
  if (n == 0) return 0;
  hkv_pin_kernel<<<warp_grid(n, num_sms), 256, 0, st>>>(unpack(desc), reinterpret_cast<const unsigned long long*>(keys), n, pin,
                                                       out_slots, reinterpret_cast<unsigned char*>(flags), status);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_hkv_erase(const long long* desc, const void* keys, long long n, int num_sms, int* status, cudaStream_t st) {
  if (n == 0) return 0;
  hkv_erase_kernel<<<warp_grid(n, num_sms), 256, 0, st>>>(unpack(desc), reinterpret_cast<const unsigned long long*>(keys),
                                                         n, status);
  return static_cast<int>(cudaGetLastError());
}

// out[i, 0:cols] = row(slots[i])[col0 : col0+cols]; out dtype 0 = fp32, 2 = bf16, 1 = fp16
RB_API int rb_hkv_gather(const long long* desc, const long long* slots, long long n, int col0, int cols, void* out,
                         int out_dtype, long long ld_out, float missing_value, int num_sms, cudaStream_t st) {
  if (n == 0) return 0;
  HkvTable t = unpack(desc);
  const int g = warp_grid(n, num_sms);
  if (out_dtype == 0) hkv_gather_kernel<float><<<g, 256, 0, st>>>(t, slots, n, col0, cols, reinterpret_cast<float*>(out), ld_out, missing_value);
  else if (out_dtype == 2) hkv_gather_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(t, slots, n, col0, cols, reinterpret_cast<__nv_bfloat16*>(out), ld_out, missing_value);
  else if (out_dtype == 1) hkv_gather_kernel<__half><<<g, 256, 0, st>>>(t, slots, n, col0, cols, reinterpret_cast<__half*>(out), ld_out, missing_value);
  else return -1;
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_hkv_scatter(const long long* desc, const long long* slots, long long n, int col0, int cols,
                          const float* in, long long ld_in, int accumulate, int num_sms, cudaStream_t st) {
  if (n == 0) return 0;
  hkv_scatter_kernel<<<warp_grid(n, num_sms), 256, 0, st>>>(unpack(desc), slots, n, col0, cols, in, ld_in, accumulate);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_hkv_update(const long long* desc, const long long* slots, long long n, const void* grads, int g_dtype,
                         long long ld_g, int opt_type, float lr, float eps, float beta1, float beta2, float weight_decay,
                         float bc1, float bc2, int num_sms, cudaStream_t st) {
  if (n == 0) return 0;
  HkvTable t = unpack(desc);
  OptArgs o{opt_type, lr, eps, beta1, beta2, weight_decay, bc1, bc2};
  const int g = warp_grid(n, num_sms);
  if (g_dtype == 0) hkv_update_kernel<float><<<g, 256, 0, st>>>(t, slots, n, reinterpret_cast<const float*>(grads), ld_g, o);
  else if (g_dtype == 2) hkv_update_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(t, slots, n, reinterpret_cast<const __nv_bfloat16*>(grads), ld_g, o);
  else if (g_dtype == 1) hkv_update_kernel<__half><<<g, 256, 0, st>>>(t, slots, n, reinterpret_cast<const __half*>(grads), ld_g, o);
  else return -1;
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_hkv_export(const long long* desc, long long slot0, long long count, long long min_score, void* out_keys,
                         void* out_scores, float* out_values, long long* out_slots, int* counter, int out_cap,
                         int num_sms, cudaStream_t st) {
  if (count == 0) return 0;
  hkv_export_kernel<<<warp_grid((count + 31) / 32, num_sms), 256, 0, st>>>(
      unpack(desc), slot0, count, static_cast<unsigned long long>(min_score), reinterpret_cast<unsigned long long*>(out_keys),
      reinterpret_cast<unsigned long long*>(out_scores), out_values, out_slots, counter, out_cap);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_hkv_rehash(const long long* src_desc, const long long* dst_desc, int num_sms, int* status, cudaStream_t st) {
  HkvTable s = unpack(src_desc);
  hkv_rehash_kernel<<<warp_grid(s.capacity, num_sms), 256, 0, st>>>(s, unpack(dst_desc), status);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_device_timestamp(void* out, cudaStream_t st) {
  device_timestamp_kernel<<<1, 1, 0, st>>>(reinterpret_cast<unsigned long long*>(out));
  return static_cast<int>(cudaGetLastError());
}
