// CPU id processing: id -> slot mapping with fused unique, sort-based parallel unique, and row-wise
// bucketisation of KJT values.  Behavioural spec: hybrid_torchrec/src/ids_process/ids_mapper.{h,cpp}
// (FindOrInsert, UniqueAndLookupOut, ParallelUniqueHashOut), unique.cpp:55-129, bucketize.cpp:35-305.
#pragma once
#include <omp.h>

#include <algorithm>
#include <numeric>

#include "common.h"

namespace rbh {

// Maps raw int64 ids to dense slots [0, size) in first-seen order (monotone allocation); keeps the
// reverse slot -> id vector.  Insertions are serialised by a mutex; lookups of an unchanged map are
// safe from many threads.
class IdsMapper {
 public:
  explicit IdsMapper(int64_t max_slots, size_t reserve = 1024) : max_slots_(max_slots), map_(reserve) {}

  int64_t size() const { return static_cast<int64_t>(slot2id_.size()); }
  int64_t capacity() const { return max_slots_; }

  // slot of id, inserting when new; throws when the table is full
  int64_t find_or_insert(int64_t id) {
    std::lock_guard<std::mutex> lk(mu_);
    return find_or_insert_unlocked(id);
  }

  int64_t find(int64_t id) const {
    const int64_t* p = map_.find(id);
    return p ? *p : -1;
  }

  // ids[n] -> out[n] slots (inserting new ids)
  void ids2indices(const int64_t* ids, int64_t n, int64_t* out) {
    std::lock_guard<std::mutex> lk(mu_);
    for (int64_t i = 0; i < n; ++i) out[i] = find_or_insert_unlocked(ids[i]);
  }

  // Fused unique + lookup for one table's ids:
  //   unique_ids[u]   distinct raw ids in first-seen order
  //   unique[u]       their slots
  //   inverse[i]      position of ids[i] in unique_ids
  //   hash_indices[i] slot of ids[i]
  // Returns u.  Uses a per-call scratch map keyed by raw id.
  int64_t unique_and_lookup(const int64_t* ids, int64_t n, int64_t* hash_indices, int64_t* unique,
                            int64_t* unique_ids, int64_t* inverse) {
    std::lock_guard<std::mutex> lk(mu_);
    const int threads = std::max(1, std::min<int>(omp_get_max_threads(), static_cast<int>(n / 16384)));
    if (threads <= 1) return unique_and_lookup_serial(ids, n, hash_indices, unique, unique_ids, inverse);
    // Parallel form with the same outputs (distinct ids in first-seen order, slots handed out in that order):
    //   1. every thread de-duplicates its contiguous chunk with a small private map (cache resident) and looks its
    //      distinct ids up in the table map (read-only while this call holds the lock),
    //   2. one pass over the chunks' distinct ids in chunk order assigns global positions: known ids are recognised
    //      through a slot-indexed stamp array (no hashing), new ids are inserted,
    //   3. every thread translates its chunk's local positions into global ones and fills the per-id outputs.
    struct Chunk { std::vector<int64_t> uniq, slot, gpos; std::vector<int32_t> inv; };
    std::vector<Chunk> ch(threads);
    const int64_t per = (n + threads - 1) / threads;
#pragma omp parallel for num_threads(threads) schedule(static, 1)
    for (int t = 0; t < threads; ++t) {
      const int64_t b = t * per, e = std::min<int64_t>(n, b + per);
      Chunk& c = ch[t];
      if (b >= e) continue;
      FlatMap<int32_t> seen(static_cast<size_t>(e - b) + 1);
      c.inv.resize(e - b);
      c.uniq.reserve((e - b) / 2 + 16);
      for (int64_t i = b; i < e; ++i) {
        auto r = seen.insert(ids[i], static_cast<int32_t>(c.uniq.size()));
        if (r.second) c.uniq.push_back(ids[i]);
        c.inv[i - b] = *r.first;
      }
      c.slot.resize(c.uniq.size());
      for (size_t k = 0; k < c.uniq.size(); ++k) {
        const int64_t* p = map_.find(c.uniq[k]);
        c.slot[k] = p ? *p : -1;
      }
    }
    ++stamp_;
    if (stamp_ == 0) { std::fill(slot_stamp_.begin(), slot_stamp_.end(), 0u); stamp_ = 1; }
    int64_t u = 0;
    for (int t = 0; t < threads; ++t) {
      Chunk& c = ch[t];
      c.gpos.resize(c.uniq.size());
      for (size_t k = 0; k < c.uniq.size(); ++k) {
        int64_t slot = c.slot[k];
        if (slot < 0) slot = find_or_insert_unlocked(c.uniq[k]);   // new here, or inserted by an earlier chunk of this call
        if (static_cast<size_t>(slot) >= slot_stamp_.size()) {
          const size_t want = std::max<size_t>(slot2id_.size(), static_cast<size_t>(slot) + 1);
          slot_stamp_.resize(want + want / 4 + 16, 0u);
          slot_pos_.resize(slot_stamp_.size(), 0);
        }
        if (slot_stamp_[slot] == stamp_) {
          c.gpos[k] = slot_pos_[slot];
        } else {
          slot_stamp_[slot] = stamp_;
          slot_pos_[slot] = u;
          unique_ids[u] = c.uniq[k];
          unique[u] = slot;
          c.gpos[k] = u++;
        }
      }
    }
#pragma omp parallel for num_threads(threads) schedule(static, 1)
    for (int t = 0; t < threads; ++t) {
      const int64_t b = t * per, e = std::min<int64_t>(n, b + per);
      const Chunk& c = ch[t];
      for (int64_t i = b; i < e; ++i) {
        const int64_t pos = c.gpos[c.inv[i - b]];
        inverse[i] = pos;
        hash_indices[i] = unique[pos];
      }
    }
    return u;
  }

  int64_t unique_and_lookup_serial(const int64_t* ids, int64_t n, int64_t* hash_indices, int64_t* unique,
                                   int64_t* unique_ids, int64_t* inverse) {
    FlatMap<int64_t> seen(static_cast<size_t>(n) + 1);
    int64_t u = 0;
    for (int64_t i = 0; i < n; ++i) {
      auto r = seen.insert(ids[i], u);
      if (r.second) {
        unique_ids[u] = ids[i];
        unique[u] = find_or_insert_unlocked(ids[i]);
        ++u;
      }
      const int64_t pos = *r.first;
      inverse[i] = pos;
      hash_indices[i] = unique[pos];
    }
    return u;
  }

  const std::vector<int64_t>& slot2id() const { return slot2id_; }

  // bulk restore (checkpoint): ids in slot order
  void load(const int64_t* ids, int64_t n) {
    std::lock_guard<std::mutex> lk(mu_);
    map_.clear();
    slot2id_.clear();
    for (int64_t i = 0; i < n; ++i) find_or_insert_unlocked(ids[i]);
  }

 private:
  int64_t find_or_insert_unlocked(int64_t id) {
    int64_t* p = map_.find(id);
    if (p) return *p;
    const int64_t slot = static_cast<int64_t>(slot2id_.size());
    if (slot >= max_slots_) throw std::runtime_error("IdsMapper: table is full (" + std::to_string(max_slots_) + " slots)");
    map_.insert(id, slot);
    slot2id_.push_back(id);
    return slot;
  }
  int64_t max_slots_;
  FlatMap<int64_t> map_;
  std::vector<int64_t> slot2id_;
  std::vector<uint32_t> slot_stamp_;        // per slot: the call that last listed it among its distinct ids
  std::vector<int64_t> slot_pos_;           // ... and its position in that call's distinct list
  uint32_t stamp_ = 0;
  mutable std::mutex mu_;
};

// Sort-based unique with inverse (stable w.r.t. value order): out_unique sorted ascending.
// Parallel: chunks are sorted by OpenMP threads and merged.
inline int64_t unique_parallel(const int64_t* in, int64_t n, int64_t* out_unique, int64_t* out_inverse,
                               int64_t* out_counts) {
  if (n == 0) return 0;
  std::vector<int64_t> order(n);
  std::iota(order.begin(), order.end(), 0);
  const int threads = std::max(1, std::min<int>(omp_get_max_threads(), static_cast<int>(n / 65536) + 1));
  if (threads == 1) {
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return in[a] < in[b]; });
  } else {
    const int64_t chunk = (n + threads - 1) / threads;
#pragma omp parallel for num_threads(threads) schedule(static, 1)
    for (int t = 0; t < threads; ++t) {
      const int64_t b = t * chunk, e = std::min<int64_t>(n, b + chunk);
      if (b < e)
        std::stable_sort(order.begin() + b, order.begin() + e, [&](int64_t x, int64_t y) { return in[x] < in[y]; });
    }
    for (int64_t width = chunk; width < n; width *= 2)
      for (int64_t b = 0; b + width < n; b += 2 * width)
        std::inplace_merge(order.begin() + b, order.begin() + b + width, order.begin() + std::min<int64_t>(n, b + 2 * width),
                           [&](int64_t x, int64_t y) { return in[x] < in[y]; });
  }
  int64_t u = 0;
  for (int64_t i = 0; i < n; ++i) {
    const int64_t v = in[order[i]];
    if (i == 0 || v != out_unique[u - 1]) {
      out_unique[u] = v;
      if (out_counts) out_counts[u] = 0;
      ++u;
    }
    if (out_inverse) out_inverse[order[i]] = u - 1;
    if (out_counts) ++out_counts[u - 1];
  }
  return u;
}

// Row-wise bucketisation of a KJT.  lengths [F*B], indices [nnz] (key-major).  Bucket of an id:
//   block_sizes == nullptr : id % world                         (round robin; the reference's default)
//   block_sizes[f] > 0     : min(id / block_sizes[f], world-1)  (contiguous ranges)
// Outputs (bucket-major then feature-major, like fbgemm's block_bucketize_sparse_features):
//   new_lengths [world*F*B], new_indices [nnz] (the id, or the id's local row when `local_rows`),
//   unbucketize_permute [nnz] (position of input element i in new_indices), optional new_weights.
inline void block_bucketize(const int64_t* lengths, const int64_t* indices, const float* weights, int64_t F,
                            int64_t B, int64_t world, const int64_t* block_sizes, bool local_rows,
                            int64_t* new_lengths, int64_t* new_indices, float* new_weights,
                            int64_t* unbucketize_permute) {
  const int64_t FB = F * B;
  // scratch that keeps its pages between calls (a fresh 8 * world * F * B byte vector per batch costs more in page
  // faults than the bucketize itself)
  static thread_local std::vector<int64_t> offsets_tl, new_offsets_tl;
  offsets_tl.resize(FB + 1);
  new_offsets_tl.resize(world * FB + 1);
  int64_t* const offsets = offsets_tl.data();          // plain pointers: the OpenMP workers must see THIS thread's buffers
  int64_t* const new_offsets = new_offsets_tl.data();
  offsets[0] = 0;
  for (int64_t i = 0; i < FB; ++i) offsets[i + 1] = offsets[i] + lengths[i];
  std::fill(new_lengths, new_lengths + world * FB, 0);
  auto bucket_of = [&](int64_t f, int64_t id) -> int64_t {
    if (block_sizes && block_sizes[f] > 0) return std::min<int64_t>(id / block_sizes[f], world - 1);
    int64_t m = id % world;
    return m < 0 ? m + world : m;
  };
#pragma omp parallel for schedule(static)
  for (int64_t fb = 0; fb < FB; ++fb) {
    const int64_t f = fb / B;
    for (int64_t j = offsets[fb]; j < offsets[fb + 1]; ++j) ++new_lengths[bucket_of(f, indices[j]) * FB + fb];
  }
  // exclusive prefix over world*FB counts: per-thread partial sums, then a short serial carry
  const int64_t total = world * FB;
  new_offsets[0] = 0;
  {
    const int nt = std::max(1, std::min<int>(omp_get_max_threads(), static_cast<int>(total / 65536) + 1));
    const int64_t per = (total + nt - 1) / nt;
    std::vector<int64_t> carry(nt + 1, 0);
#pragma omp parallel for num_threads(nt) schedule(static, 1)
    for (int t = 0; t < nt; ++t) {
      int64_t run = 0;
      for (int64_t i = t * per; i < std::min<int64_t>(total, (t + 1) * per); ++i) { new_offsets[i + 1] = run += new_lengths[i]; }
      carry[t + 1] = run;
    }
    for (int t = 0; t < nt; ++t) carry[t + 1] += carry[t];
#pragma omp parallel for num_threads(nt) schedule(static, 1)
    for (int t = 1; t < nt; ++t)
      for (int64_t i = t * per; i < std::min<int64_t>(total, (t + 1) * per); ++i) new_offsets[i + 1] += carry[t];
  }
#pragma omp parallel for schedule(static)
  for (int64_t fb = 0; fb < FB; ++fb) {
    const int64_t f = fb / B;
    int64_t cursor_small[64];                                  // no heap allocation per bag
    std::vector<int64_t> cursor_big;
    int64_t* cursor = cursor_small;
    if (world > 64) { cursor_big.resize(world); cursor = cursor_big.data(); }
    for (int64_t w = 0; w < world; ++w) cursor[w] = new_offsets[w * FB + fb];
    for (int64_t j = offsets[fb]; j < offsets[fb + 1]; ++j) {
      const int64_t id = indices[j];
      const int64_t w = bucket_of(f, id);
      const int64_t pos = cursor[w]++;
      int64_t v = id;
      if (local_rows) v = (block_sizes && block_sizes[f] > 0) ? id - w * block_sizes[f] : id / world;
      new_indices[pos] = v;
      if (new_weights && weights) new_weights[pos] = weights[j];
      if (unbucketize_permute) unbucketize_permute[j] = pos;
    }
  }
}

// Rebuild the per-id device-cache offsets after the swap planner assigned an offset to every unique key:
// hash_indices[r] = unique_indices[unique_inverse[r] + unique_offset[t]] for the ids r of table t
// (offsets_per_table[t] .. offsets_per_table[t+1]).  Returns the first bad position (or -1); nothing is written past it
// for that table (the reference: torchrec_embcache csrc/ops/restore.cpp:17-70).
inline int64_t restore_hash_indices(const int64_t* unique_indices, int64_t n_unique, const int64_t* unique_inverse, int64_t n_ids,
                                    const int64_t* unique_offset, const int64_t* offsets_per_table, int64_t n_tables,
                                    int64_t* hash_indices) {
  int64_t bad = -1;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t t = 0; t < n_tables; ++t) {
    const int64_t shift = unique_offset[t];
    const int64_t r0 = offsets_per_table[t], r1 = offsets_per_table[t + 1];
    if (r0 < 0 || r1 > n_ids || r0 > r1) {
#pragma omp critical
      bad = bad < 0 ? r0 : bad;
      continue;
    }
    for (int64_t r = r0; r < r1; ++r) {
      const int64_t g = unique_inverse[r] + shift;
      if (g < 0 || g >= n_unique) {
#pragma omp critical
        bad = bad < 0 ? r : bad;
        break;
      }
      hash_indices[r] = unique_indices[g];
    }
  }
  return bad;
}

}  // namespace rbh
