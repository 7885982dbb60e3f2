// Multi-tier embedding cache engines (host side): device-cache slot allocator, host-DRAM embedding
// table with slab pool and initialisers, admission/eviction filter, checkpoint files, and the manager
// that ties them together per table and runs its work on a thread pool.
//
// Behavioural spec (reference, torchrec_embcache/csrc): embedding_cache/swap_manager.{h,cpp},
// emb_table/{emb_table,emb_memory_pool,initializer}.h, hash_table/fast_hashmap.h,
// feature_filter/feature_filter.{h,cpp}, embedding_cache/embcache_manager.{h,cpp} (Save :549-618,
// MergeFiles :620-800, attribute files :868-903, Load :905-981), file_system/.
#pragma once
#include <sys/stat.h>
#include <sys/types.h>

#include <algorithm>
#include <cstdlib>
#include <unordered_map>
#include <thread>
#include <condition_variable>
#include <cmath>
#include <fstream>
#include <random>
#include <set>
#include <unordered_set>

#include "common.h"
#include "file_system.h"

namespace rbh {

// ============================================================================ SwapManager
struct SwapInfo {
  std::vector<int64_t> swapout_keys, swapout_offs, swapin_keys, swapin_offs, batch_offs;
};

// Slot allocator of the HBM cache of one table.  Every slot remembers its last three (key, version)
// owners so a host update that arrives a step later can still resolve which key a slot held.
class SwapManager {
 public:
  SwapManager(int64_t cache_size, bool reserve_slot0)
      : cache_size_(cache_size), first_(reserve_slot0 ? 1 : 0), next_free_(first_), hand_(first_),
        slot_key_(cache_size, kNone), slot_version_(cache_size, -1), history_(cache_size) {
    if (cache_size <= first_) throw std::invalid_argument("SwapManager: cache size too small");
  }

  // keys: de-duplicated ids of this table for batch `version`; -1 = not admitted -> offset 0.
  SwapInfo compute_swap_info(const int64_t* keys, int64_t n, int64_t version) {
    SwapInfo out;
    out.batch_offs.resize(n);
    for (int64_t i = 0; i < n; ++i) {
      const int64_t k = keys[i];
      if (k < 0) { out.batch_offs[i] = 0; continue; }
      int64_t* hit = key2off_.find(k);
      if (hit) {
        slot_version_[*hit] = version;
        out.batch_offs[i] = *hit;
        continue;
      }
      int64_t off;
      if (!free_list_.empty()) {
        off = free_list_.back();
        free_list_.pop_back();
      } else if (next_free_ < cache_size_) {
        off = next_free_++;
      } else {
        off = find_victim(version);
        const int64_t old = slot_key_[off];
        key2off_.erase(old);
        out.swapout_keys.push_back(old);
        out.swapout_offs.push_back(off);
      }
      slot_key_[off] = k;
      slot_version_[off] = version;
      push_history(off, k, version);
      key2off_.insert(k, off);
      out.swapin_keys.push_back(k);
      out.swapin_offs.push_back(off);
      out.batch_offs[i] = off;
    }
    return out;
  }

  // key that occupied `off` at `version` (latest owner with owner.version <= version), or -1
  int64_t get_key(int64_t off, int64_t version) const {
    const auto& h = history_[off];
    int64_t best = -1, best_v = -1;
    for (int i = 0; i < 3; ++i)
      if (h.key[i] != kNone && h.ver[i] <= version && h.ver[i] > best_v) { best = h.key[i]; best_v = h.ver[i]; }
    return best;
  }

  // drop keys from the cache; evicted keys free their slot without write-back
  void remove_keys(const int64_t* keys, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
      int64_t* off = key2off_.find(keys[i]);
      if (!off) continue;
      const int64_t o = *off;
      key2off_.erase(keys[i]);
      slot_key_[o] = kNone;
      slot_version_[o] = -1;
      free_list_.push_back(o);
    }
  }

  int64_t offset_of(int64_t key) const { const int64_t* p = key2off_.find(key); return p ? *p : -1; }
  int64_t size() const { return static_cast<int64_t>(key2off_.size()); }
  int64_t capacity() const { return cache_size_; }

  // all resident (key, offset) pairs (used to flush the device cache at checkpoint time)
  void resident(std::vector<int64_t>& keys, std::vector<int64_t>& offs) const {
    key2off_.for_each([&](int64_t k, const int64_t& o) { keys.push_back(k); offs.push_back(o); });
  }

 private:
  static constexpr int64_t kNone = INT64_MIN;
  struct History { int64_t key[3] = {kNone, kNone, kNone}; int64_t ver[3] = {-1, -1, -1}; int pos = 0; };

  void push_history(int64_t off, int64_t key, int64_t ver) {
    auto& h = history_[off];
    h.key[h.pos] = key; h.ver[h.pos] = ver; h.pos = (h.pos + 1) % 3;
  }
  // clock hand: first slot not used by the current or the previous (possibly in-flight) batch
  int64_t find_victim(int64_t version) {
    const int64_t span = cache_size_ - first_;
    for (int64_t step = 0; step < span; ++step) {
      const int64_t off = hand_;
      hand_ = hand_ + 1 >= cache_size_ ? first_ : hand_ + 1;
      if (slot_key_[off] != kNone && slot_version_[off] < version - 1) return off;
    }
    throw std::runtime_error("SwapManager: cacheSize_ too small (no evictable slot for this batch)");
  }

  int64_t cache_size_, first_, next_free_, hand_;
  FlatMap<int64_t> key2off_;
  std::vector<int64_t> slot_key_, slot_version_, free_list_;
  std::vector<History> history_;
};

// ============================================================================ initialisers
enum class InitializerType : int { LINEAR = 0, TRUNCATED_NORMAL = 1, UNIFORM = 2, CONSTANT = 3 };

struct InitializerConfig {
  InitializerType type = InitializerType::UNIFORM;
  float min = -0.05f, max = 0.05f, mean = 0.f, stddev = 0.05f, value = 0.f;
  uint64_t seed = 0;
};

class Initializer {
 public:
  explicit Initializer(const InitializerConfig& c) : c_(c), rng_(c.seed ? c.seed : 0x9E3779B97F4A7C15ULL) {}
  void fill(float* row, int dim) {
    std::lock_guard<std::mutex> lk(mu_);
    switch (c_.type) {
      case InitializerType::LINEAR:
        for (int i = 0; i < dim; ++i) row[i] = dim > 1 ? c_.min + (c_.max - c_.min) * i / (dim - 1) : c_.min;
        break;
      case InitializerType::TRUNCATED_NORMAL: {
        std::normal_distribution<float> nd(c_.mean, c_.stddev);
        for (int i = 0; i < dim; ++i) {
          float v = nd(rng_);
          int tries = 0;
          while (std::fabs(v - c_.mean) > 2.f * c_.stddev && tries++ < 64) v = nd(rng_);
          row[i] = v;
        }
        break;
      }
      case InitializerType::UNIFORM: {
        std::uniform_real_distribution<float> ud(c_.min, c_.max);
        for (int i = 0; i < dim; ++i) row[i] = ud(rng_);
        break;
      }
      case InitializerType::CONSTANT:
        for (int i = 0; i < dim; ++i) row[i] = c_.value;
        break;
    }
  }
  // Counter-based variant: the values are a pure function of (seed, key, column), so they depend neither on the order
  // in which threads insert keys nor on how the table is sharded, and no generator state is shared between threads.
  void fill_keyed(float* row, int dim, int64_t key) const {
    const uint64_t base = mix64(static_cast<uint64_t>(key) ^ (c_.seed * 0x9E3779B97F4A7C15ULL + 0x632BE59BD9B4E019ULL));
    auto u01 = [&](int col, uint32_t stream) {
      const uint64_t x = mix64(base ^ (static_cast<uint64_t>(col) << 32) ^ stream);
      return (static_cast<float>(x >> 40) + 0.5f) * (1.0f / 16777216.0f);
    };
    switch (c_.type) {
      case InitializerType::LINEAR:
        for (int i = 0; i < dim; ++i) row[i] = dim > 1 ? c_.min + (c_.max - c_.min) * i / (dim - 1) : c_.min;
        break;
      case InitializerType::TRUNCATED_NORMAL:
        for (int i = 0; i < dim; ++i) {
          float v = 0.f;
          for (uint32_t t = 0; t < 16; ++t) {
            v = std::sqrt(-2.f * std::log(u01(i, 1 + 2 * t))) * std::cos(6.2831853f * u01(i, 2 + 2 * t));
            if (std::fabs(v) <= 2.f) break;
            v = std::fmin(std::fmax(v, -2.f), 2.f);
          }
          row[i] = c_.mean + c_.stddev * v;
        }
        break;
      case InitializerType::UNIFORM:
        for (int i = 0; i < dim; ++i) row[i] = c_.min + (c_.max - c_.min) * u01(i, 0);
        break;
      case InitializerType::CONSTANT:
        for (int i = 0; i < dim; ++i) row[i] = c_.value;
        break;
    }
  }
 private:
  InitializerConfig c_;
  std::mt19937_64 rng_;
  std::mutex mu_;
};

// ============================================================================ row memory pool
// Slab allocator for fixed-width rows with a recycle bin; slabs are never returned to the OS while the
// pool lives, so row pointers stay stable.  EMB_MEMORY_POOL_SIZE rows per slab (default 102400).
class EmbMemoryPool {
 public:
  explicit EmbMemoryPool(int row_floats)
      : row_floats_(row_floats), rows_per_slab_(env_int("EMB_MEMORY_POOL_SIZE", 102400, 1024, 1 << 24)) {
    // EMB_MEMORY_POOL_THREAD_NUM (1..1024, default 1) background threads keep spare slabs allocated and page-touched, so
    // that the thread that exhausts a slab under a table lock never pays for the allocation and its page faults.
    const char* e = std::getenv("EMB_MEMORY_POOL_THREAD_NUM");
    int n = 1;
    if (e && *e) {
      char* end = nullptr;
      const long v = std::strtol(e, &end, 10);
      if (end == e || *end != '\0') throw std::runtime_error("env EMB_MEMORY_POOL_THREAD_NUM is not a valid number");
      if (v < 1 || v > 1024) throw std::runtime_error("env EMB_MEMORY_POOL_THREAD_NUM should be in [1, 1024]");
      n = static_cast<int>(v);
    }
    spare_target_ = static_cast<size_t>(n);
    for (int i = 0; i < n; ++i) workers_.emplace_back([this] { refill_loop(); });
  }
  ~EmbMemoryPool() {
    { std::lock_guard<std::mutex> lk(mu_); stop_ = true; }
    cv_.notify_all();
    for (auto& w : workers_) w.join();
  }
  EmbMemoryPool(const EmbMemoryPool&) = delete;
  EmbMemoryPool& operator=(const EmbMemoryPool&) = delete;

  float* alloc() {
    std::unique_lock<std::mutex> lk(mu_);
    if (!recycle_.empty()) { float* p = recycle_.back(); recycle_.pop_back(); return p; }
    if (slabs_.empty() || used_in_last_ == rows_per_slab_) {
      if (!spares_.empty()) {
        slabs_.push_back(std::move(spares_.back()));
        spares_.pop_back();
      } else {
        slabs_.emplace_back(new float[slab_floats()]);        // the refill threads fell behind: allocate in place
      }
      used_in_last_ = 0;
      cv_.notify_one();
    } else if (used_in_last_ * 2 == rows_per_slab_) {
      cv_.notify_one();                                       // half way through the slab: make sure a spare is on its way
    }
    return slabs_.back().get() + static_cast<size_t>(used_in_last_++) * row_floats_;
  }
  void free(float* p) { std::lock_guard<std::mutex> lk(mu_); recycle_.push_back(p); }
  size_t bytes() const {
    std::lock_guard<std::mutex> lk(mu_);
    return (slabs_.size() + spares_.size()) * slab_floats() * sizeof(float);
  }
  int refill_threads() const { return static_cast<int>(workers_.size()); }

 private:
  size_t slab_floats() const { return static_cast<size_t>(rows_per_slab_) * row_floats_; }
  void refill_loop() {
    std::unique_lock<std::mutex> lk(mu_);
    for (;;) {
      cv_.wait(lk, [this] { return stop_ || (!slabs_.empty() && spares_.size() + pending_ < spare_target_); });
      if (stop_) return;
      ++pending_;
      lk.unlock();
      std::unique_ptr<float[]> slab(new float[slab_floats()]);
      std::memset(slab.get(), 0, slab_floats() * sizeof(float));   // touch every page now, off the critical path
      lk.lock();
      --pending_;
      spares_.push_back(std::move(slab));
    }
  }
  int row_floats_, rows_per_slab_, used_in_last_ = 0;
  std::vector<std::unique_ptr<float[]>> slabs_, spares_;
  std::vector<float*> recycle_;
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::vector<std::thread> workers_;
  size_t spare_target_ = 1, pending_ = 0;
  bool stop_ = false;
};

// key -> row pointer map of one table shard.  ENABLE_FAST_HASHMAP (default on here; "0" / "false" selects
// std::unordered_map, which is what the reference uses when the variable is unset) picks the open-addressing map;
// FAST_HASHMAP_RESERVE_BUCKET_NUM (whole table; split evenly over the shards) pre-sizes it so that a table that is
// expected to hold that many keys never rehashes under a lock.
class RowMap {
 public:
  RowMap() : fast_(env_flag("ENABLE_FAST_HASHMAP", true)), flat_(reserve_per_shard()) {
    if (!fast_) std_.reserve(reserve_per_shard());
  }
  float** find(int64_t k) {
    if (fast_) return flat_.find(k);
    auto it = std_.find(k);
    return it == std_.end() ? nullptr : &it->second;
  }
  float* const* find(int64_t k) const { return const_cast<RowMap*>(this)->find(k); }
  void insert(int64_t k, float* v) { if (fast_) flat_.insert(k, v); else std_[k] = v; }
  void erase(int64_t k) { if (fast_) flat_.erase(k); else std_.erase(k); }
  size_t size() const { return fast_ ? flat_.size() : std_.size(); }
  void clear() { if (fast_) flat_.clear(); else std_.clear(); }
  template <typename F>
  void for_each(F&& f) const {
    if (fast_) flat_.for_each(f);
    else for (const auto& kv : std_) f(kv.first, kv.second);
  }
  bool fast() const { return fast_; }

 private:
  static bool env_flag(const char* name, bool def) {
    const char* e = std::getenv(name);
    if (!e || !*e) return def;
    const std::string v(e);
    return !(v == "0" || v == "false" || v == "False" || v == "FALSE" || v == "no");
  }
  static size_t reserve_per_shard() {
    const char* e = std::getenv("FAST_HASHMAP_RESERVE_BUCKET_NUM");
    if (!e || !*e) return 1024;
    char* end = nullptr;
    const unsigned long long v = std::strtoull(e, &end, 10);
    if (end == e || *end != '\0') throw std::runtime_error("env FAST_HASHMAP_RESERVE_BUCKET_NUM is not a valid number");
    return static_cast<size_t>(v / 16 + 16);
  }
  bool fast_;
  FlatMap<float*> flat_;
  std::unordered_map<int64_t, float*> std_;
};

// ============================================================================ host embedding table
// Full table in host DRAM: key -> [embedding | optimizer state 1 | optimizer state 2] contiguous.
// 16 independently locked sub-maps give concurrent lookups/updates from the manager's thread pool.
class HostEmbTable {
 public:
  HostEmbTable(int dim, int optim_num, const InitializerConfig& init)
      : dim_(dim), optim_num_(optim_num), row_floats_(dim * (1 + optim_num)), pool_(row_floats_), init_(init) {}

  int dim() const { return dim_; }
  int optim_num() const { return optim_num_; }
  int row_floats() const { return row_floats_; }
  int64_t size() const { int64_t s = 0; for (auto& sh : shards_) { std::lock_guard<std::mutex> lk(sh.mu); s += sh.map.size(); } return s; }

  // rows_out [n, row_floats]; new keys get an initialised embedding and zero optimizer state
  void find_or_insert(const int64_t* keys, int64_t n, float* rows_out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
      Shard& sh = shard_of(keys[i]);
      float* row;
      {
        std::lock_guard<std::mutex> lk(sh.mu);
        float** p = sh.map.find(keys[i]);
        if (p) row = *p;
        else {
          row = pool_.alloc();
          init_.fill_keyed(row, dim_, keys[i]);          // per-key values: no shared generator under the shard locks
          std::fill(row + dim_, row + row_floats_, 0.f);
          sh.map.insert(keys[i], row);
        }
        std::memcpy(rows_out + i * row_floats_, row, sizeof(float) * row_floats_);
      }
    }
  }

  // found[i] = 1 and the row copied when present; missing rows are zero-filled
  void find(const int64_t* keys, int64_t n, float* rows_out, uint8_t* found) const {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
      const Shard& sh = shard_of(keys[i]);
      std::lock_guard<std::mutex> lk(sh.mu);
      float* const* p = sh.map.find(keys[i]);
      if (p) { std::memcpy(rows_out + i * row_floats_, *p, sizeof(float) * row_floats_); if (found) found[i] = 1; }
      else { std::fill(rows_out + i * row_floats_, rows_out + (i + 1) * row_floats_, 0.f); if (found) found[i] = 0; }
    }
  }

  void insert_or_assign(const int64_t* keys, int64_t n, const float* rows) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
      Shard& sh = shard_of(keys[i]);
      std::lock_guard<std::mutex> lk(sh.mu);
      float** p = sh.map.find(keys[i]);
      float* row;
      if (p) row = *p;
      else { row = pool_.alloc(); sh.map.insert(keys[i], row); }
      std::memcpy(row, rows + i * row_floats_, sizeof(float) * row_floats_);
    }
  }

  void erase(const int64_t* keys, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
      Shard& sh = shard_of(keys[i]);
      std::lock_guard<std::mutex> lk(sh.mu);
      float** p = sh.map.find(keys[i]);
      if (p) { pool_.free(*p); sh.map.erase(keys[i]); }
    }
  }

  // drop every key (rows go back to the pool's recycle bin)
  void clear() {
    for (auto& sh : shards_) {
      std::lock_guard<std::mutex> lk(sh.mu);
      sh.map.for_each([&](int64_t, float* const& r) { pool_.free(r); });
      sh.map.clear();
    }
  }

  void export_all(std::vector<int64_t>& keys, std::vector<float>& rows) const {
    for (auto& sh : shards_) {
      std::lock_guard<std::mutex> lk(sh.mu);
      sh.map.for_each([&](int64_t k, float* const& r) { keys.push_back(k); rows.insert(rows.end(), r, r + row_floats_); });
    }
  }

 private:
  struct Shard { mutable std::mutex mu; RowMap map; };
  Shard& shard_of(int64_t k) { return shards_[mix64(static_cast<uint64_t>(k)) >> 60]; }
  const Shard& shard_of(int64_t k) const { return shards_[mix64(static_cast<uint64_t>(k)) >> 60]; }
  int dim_, optim_num_, row_floats_;
  EmbMemoryPool pool_;
  Initializer init_;
  Shard shards_[16];
};

// ============================================================================ feature filter
struct AdmitEvictConfig {
  int64_t admit_threshold = -1;          // count policy: admit when count >= threshold (-1 = off)
  int64_t evict_threshold = -1;          // seconds since last seen (-1 = off)
  int policy = 0;                        // 0 = count, 1 = show-click
  float alpha = 1.f, beta = 1.f, sc_admit_threshold = 0.f, evict_percentage = 0.f, score_decay = 1.f;
  bool admit_enabled() const { return policy == 0 ? admit_threshold > 0 : sc_admit_threshold > 0.f; }
  bool evict_enabled() const { return policy == 0 ? evict_threshold > 0 : evict_percentage > 0.f; }
};

class FeatureFilter {
 public:
  explicit FeatureFilter(const AdmitEvictConfig& c) : c_(c) {}

  // counts how often each key of the batch appeared (counts may be null = 1 each; clicks for show-click)
  void statistics_key_count(const int64_t* keys, int64_t n, const int64_t* counts, const int64_t* clicks) {
    std::lock_guard<std::mutex> lk(mu_);
    for (int64_t i = 0; i < n; ++i) {
      if (keys[i] < 0) continue;
      Stat& s = *stats_.insert(keys[i], Stat()).first;
      const int64_t c = counts ? counts[i] : 1;
      s.count += c;
      if (c_.policy == 1) s.score = (s.score + c_.alpha * c + c_.beta * (clicks ? clicks[i] : 0)) * c_.score_decay;
    }
  }

  // replaces not-yet-admitted keys by -1 in place
  void filter(int64_t* keys, int64_t n) {
    if (!c_.admit_enabled()) return;
    std::lock_guard<std::mutex> lk(mu_);
    for (int64_t i = 0; i < n; ++i) {
      if (keys[i] < 0) continue;
      const Stat* s = stats_.find(keys[i]);
      const bool ok = s && (c_.policy == 0 ? s->count >= c_.admit_threshold : s->score >= c_.sc_admit_threshold);
      if (!ok) keys[i] = -1;
    }
  }

  void record_timestamp(const int64_t* keys, int64_t n, const int64_t* ts) {
    std::lock_guard<std::mutex> lk(mu_);
    for (int64_t i = 0; i < n; ++i) {
      if (keys[i] < 0) continue;
      Stat& s = *stats_.insert(keys[i], Stat()).first;
      s.ts = std::max(s.ts, ts[i]);
      latest_ts_ = std::max(latest_ts_, ts[i]);
    }
  }

  // keys to evict now; they are also dropped from the filter's own statistics
  std::vector<int64_t> evict() {
    std::lock_guard<std::mutex> lk(mu_);
    std::vector<int64_t> out;
    if (!c_.evict_enabled()) return out;
    if (c_.policy == 0) {
      stats_.for_each([&](int64_t k, const Stat& s) { if (s.ts >= 0 && latest_ts_ - s.ts > c_.evict_threshold) out.push_back(k); });
    } else {
      std::vector<std::pair<float, int64_t>> scored;
      stats_.for_each([&](int64_t k, const Stat& s) { scored.emplace_back(s.score, k); });
      const size_t m = static_cast<size_t>(scored.size() * static_cast<double>(c_.evict_percentage));
      std::partial_sort(scored.begin(), scored.begin() + std::min(m, scored.size()), scored.end());
      for (size_t i = 0; i < m && i < scored.size(); ++i) out.push_back(scored[i].second);
    }
    for (int64_t k : out) stats_.erase(k);
    return out;
  }

  void export_state(std::vector<int64_t>& keys, std::vector<int64_t>& counts, std::vector<int64_t>& ts) const {
    std::lock_guard<std::mutex> lk(mu_);
    stats_.for_each([&](int64_t k, const Stat& s) { keys.push_back(k); counts.push_back(s.count); ts.push_back(s.ts); });
  }
  void import_state(const int64_t* keys, const int64_t* counts, const int64_t* ts, int64_t n) {
    std::lock_guard<std::mutex> lk(mu_);
    for (int64_t i = 0; i < n; ++i) {
      Stat s; s.count = counts ? counts[i] : 0; s.ts = ts ? ts[i] : -1;
      *stats_.insert(keys[i], s).first = s;
      if (ts) latest_ts_ = std::max(latest_ts_, ts[i]);
    }
  }
  int64_t size() const { std::lock_guard<std::mutex> lk(mu_); return static_cast<int64_t>(stats_.size()); }
  void clear() { std::lock_guard<std::mutex> lk(mu_); stats_.clear(); latest_ts_ = 0; }
  void erase(const int64_t* keys, int64_t n) {
    std::lock_guard<std::mutex> lk(mu_);
    for (int64_t i = 0; i < n; ++i) stats_.erase(keys[i]);
  }

 private:
  struct Stat { int64_t count = 0; int64_t ts = -1; float score = 0.f; };
  AdmitEvictConfig c_;
  FlatMap<Stat> stats_;
  int64_t latest_ts_ = 0;
  mutable std::mutex mu_;
};

// ============================================================================ files
namespace fs {
// Every checkpoint file goes through the FileSystem layer (file_system.h): validated paths, no symbolic links, 0750 /
// 0640 modes, 32 KiB chunked IO.  RECSDK_B200_FS_STRICT=0 relaxes the ownership checks (shared scratch directories).
inline FileSystem& local() {
  static LocalFileSystem inst(env_int("RECSDK_B200_FS_STRICT", 1, 0, 1) != 0);
  return inst;
}
inline bool exists(const std::string& p) { return local().exists(p); }
inline void mkdirs(const std::string& p) { local().create_dir(p); }
inline void check_path(const std::string& p) { validate_path_text(p); }
inline void write_file(const std::string& p, const void* data, size_t bytes, bool append = false) {
  local().write(p, data, bytes, append);
}
inline std::vector<char> read_file(const std::string& p) { return local().read_all(p); }
}  // namespace fs

// One "slice" = <dir>/slice.attribute (raw int64s) + <dir>/slice.data (raw little-endian payload).
//   key dirs        attribute = [8, count]            data = int64 keys
//   row dirs        attribute = [4, count, dim]       data = fp32 rows
inline void write_slice_i64(const std::string& dir, const std::vector<int64_t>& v, bool append) {
  fs::mkdirs(dir);
  int64_t count = static_cast<int64_t>(v.size());
  if (append && fs::exists(dir + "/slice.attribute")) {
    auto a = fs::read_file(dir + "/slice.attribute");
    if (a.size() >= 16) count += reinterpret_cast<const int64_t*>(a.data())[1];
  }
  const int64_t attr[2] = {8, count};
  fs::write_file(dir + "/slice.attribute", attr, sizeof(attr));
  fs::write_file(dir + "/slice.data", v.data(), v.size() * sizeof(int64_t), append);
}
inline void write_slice_f32(const std::string& dir, const float* rows, int64_t count, int64_t dim, bool append) {
  fs::mkdirs(dir);
  int64_t total = count;
  if (append && fs::exists(dir + "/slice.attribute")) {
    auto a = fs::read_file(dir + "/slice.attribute");
    if (a.size() >= 24) total += reinterpret_cast<const int64_t*>(a.data())[1];
  }
  const int64_t attr[3] = {4, total, dim};
  fs::write_file(dir + "/slice.attribute", attr, sizeof(attr));
  fs::write_file(dir + "/slice.data", rows, static_cast<size_t>(count * dim) * sizeof(float), append);
}
inline std::vector<int64_t> read_slice_i64(const std::string& dir) {
  if (!fs::exists(dir + "/slice.data")) return {};
  auto d = fs::read_file(dir + "/slice.data");
  std::vector<int64_t> v(d.size() / sizeof(int64_t));
  std::memcpy(v.data(), d.data(), v.size() * sizeof(int64_t));
  return v;
}
inline std::vector<float> read_slice_f32(const std::string& dir, int64_t* count, int64_t* dim) {
  *count = 0; *dim = 0;
  if (!fs::exists(dir + "/slice.data")) return {};
  auto a = fs::read_file(dir + "/slice.attribute");
  if (a.size() >= 24) { *count = reinterpret_cast<const int64_t*>(a.data())[1]; *dim = reinterpret_cast<const int64_t*>(a.data())[2]; }
  auto d = fs::read_file(dir + "/slice.data");
  std::vector<float> v(d.size() / sizeof(float));
  std::memcpy(v.data(), d.data(), v.size() * sizeof(float));
  return v;
}

// ============================================================================ manager
struct EmbConfig {
  std::string table_name;
  int emb_dim = 0;
  int optim_num = 1;
  int64_t cache_size = 0;
  InitializerConfig init;
  AdmitEvictConfig admit_evict;
  bool is_incremental = false;
};

class EmbcacheManager {
 public:
  EmbcacheManager(const std::vector<EmbConfig>& cfgs, int threads) : cfgs_(cfgs), pool_(threads > 0 ? threads : 4) {
    for (const auto& c : cfgs_) {
      tables_.emplace_back(new Table(c));
    }
  }
  size_t num_tables() const { return tables_.size(); }
  const EmbConfig& config(size_t t) const { return cfgs_.at(t); }

  // ---- per-step operations (synchronous cores; *_async wrap them on the pool)
  SwapInfo compute_swap_info(size_t t, std::vector<int64_t> keys, int64_t step) {
    Table& tb = *tables_.at(t);
    TimeCost tc;
    tb.filter.filter(keys.data(), static_cast<int64_t>(keys.size()));
    SwapInfo si = tb.swap.compute_swap_info(keys.data(), static_cast<int64_t>(keys.size()), step);
    if (cfgs_[t].is_incremental) { std::lock_guard<std::mutex> lk(tb.mu); for (int64_t k : keys) if (k >= 0) tb.touched.insert(k); }
    log(LOG_DEBUG, "ComputeSwapInfo table %zu: %zu keys, %zu in, %zu out, %.3f ms", t, keys.size(), si.swapin_keys.size(),
        si.swapout_keys.size(), tc.ms());
    return si;
  }
  // One native call per table and batch: distinct keys with their counts (admission statistics, last-seen timestamps),
  // then the swap plan.  Replaces a host-side unique + per-key bookkeeping in the caller.
  SwapInfo plan_batch(size_t t, std::vector<int64_t> keys, int64_t step, bool count_stats, bool stamp, int64_t now) {
    if ((count_stats || stamp) && !keys.empty()) {
      FlatMap<int64_t> cnt(keys.size() * 2 + 16);
      std::vector<int64_t> uniq;
      uniq.reserve(keys.size());
      for (int64_t k : keys) {
        int64_t* c = cnt.find(k);
        if (c) ++*c;
        else { cnt.insert(k, 1); uniq.push_back(k); }
      }
      if (count_stats) {
        std::vector<int64_t> counts(uniq.size());
        for (size_t i = 0; i < uniq.size(); ++i) counts[i] = *cnt.find(uniq[i]);
        statistics_key_count(t, uniq.data(), static_cast<int64_t>(uniq.size()), counts.data(), nullptr);
      }
      if (stamp) {
        std::vector<int64_t> ts(uniq.size(), now);
        record_timestamp(t, uniq.data(), static_cast<int64_t>(uniq.size()), ts.data());
      }
    }
    return compute_swap_info(t, std::move(keys), step);
  }
  std::future<SwapInfo> plan_batch_async(size_t t, std::vector<int64_t> keys, int64_t step, bool count_stats, bool stamp,
                                         int64_t now) {
    return pool_.submit([this, t, keys = std::move(keys), step, count_stats, stamp, now]() mutable {
      return plan_batch(t, std::move(keys), step, count_stats, stamp, now);
    });
  }
  std::future<SwapInfo> compute_swap_info_async(size_t t, std::vector<int64_t> keys, int64_t step) {
    return pool_.submit([this, t, keys = std::move(keys), step]() mutable { return compute_swap_info(t, std::move(keys), step); });
  }
  // rows [n, dim*(1+optim_num)] for swap-in (host FindOrInsert)
  void embedding_lookup(size_t t, const int64_t* keys, int64_t n, float* rows_out) { tables_.at(t)->host.find_or_insert(keys, n, rows_out); }
  // host InsertOrAssign of rows swapped out of the device cache
  void embedding_update(size_t t, const int64_t* keys, int64_t n, const float* rows) { tables_.at(t)->host.insert_or_assign(keys, n, rows); }
  void statistics_key_count(size_t t, const int64_t* keys, int64_t n, const int64_t* counts, const int64_t* clicks) {
    tables_.at(t)->filter.statistics_key_count(keys, n, counts, clicks);
  }
  void record_timestamp(size_t t, const int64_t* keys, int64_t n, const int64_t* ts) { tables_.at(t)->filter.record_timestamp(keys, n, ts); }
  // evicted keys leave the filter, the device cache (slot freed, no write-back) and the host table
  std::vector<int64_t> evict_features(size_t t) {
    Table& tb = *tables_.at(t);
    std::vector<int64_t> ev = tb.filter.evict();
    tb.swap.remove_keys(ev.data(), static_cast<int64_t>(ev.size()));
    tb.host.erase(ev.data(), static_cast<int64_t>(ev.size()));
    if (cfgs_[t].is_incremental) {                 // replaying incremental checkpoints must not bring these keys back
      std::lock_guard<std::mutex> lk(tb.mu);
      for (int64_t k : ev) { tb.evicted.insert(k); tb.touched.erase(k); }
    }
    return ev;
  }
  // forget every device-resident row of table t without writing it back (after a checkpoint load)
  void invalidate_cache(size_t t) {
    std::vector<int64_t> k, o;
    tables_.at(t)->swap.resident(k, o);
    tables_.at(t)->swap.remove_keys(k.data(), static_cast<int64_t>(k.size()));
  }
  SwapManager& swap_manager(size_t t) { return tables_.at(t)->swap; }
  HostEmbTable& host_table(size_t t) { return tables_.at(t)->host; }
  FeatureFilter& feature_filter(size_t t) { return tables_.at(t)->filter; }
  ThreadPool& pool() { return pool_; }

  // ---- checkpoint.  The caller first writes the device-resident rows back with embedding_update
  // (Embedding2Host), then every rank saves its keys under <path>/<table>/rank<r>/..., rank 0 merges.
  void save(const std::string& path, int rank, bool incremental) {
    fs::check_path(path);
    for (size_t t = 0; t < tables_.size(); ++t) {
      Table& tb = *tables_[t];
      std::vector<int64_t> keys;
      std::vector<float> rows;
      tb.host.export_all(keys, rows);
      const int rf = tb.host.row_floats(), dim = tb.host.dim();
      if (incremental) {
        std::vector<int64_t> k2; std::vector<float> r2;
        std::lock_guard<std::mutex> lk(tb.mu);
        for (size_t i = 0; i < keys.size(); ++i)
          if (tb.touched.count(keys[i])) { k2.push_back(keys[i]); r2.insert(r2.end(), rows.begin() + i * rf, rows.begin() + (i + 1) * rf); }
        keys.swap(k2); rows.swap(r2);
      }
      std::vector<int64_t> gone;
      {
        std::lock_guard<std::mutex> lk(tb.mu);
        tb.touched.clear();
        if (incremental) gone.assign(tb.evicted.begin(), tb.evicted.end());
        tb.evicted.clear();
      }
      const std::string base = path + "/" + cfgs_[t].table_name + "/rank" + std::to_string(rank);
      write_slice_i64(base + "/key", keys, false);
      write_slice_i64(base + "/evicted_key", gone, false);    // incremental only: keys to erase when this delta is replayed
      const int64_t n = static_cast<int64_t>(keys.size());
      std::vector<float> col(static_cast<size_t>(n) * dim);
      static const char* names[3] = {"embedding", "momentum1", "momentum2"};
      for (int part = 0; part < 1 + tb.host.optim_num() && part < 3; ++part) {
        for (int64_t i = 0; i < n; ++i) std::memcpy(col.data() + i * dim, rows.data() + i * rf + part * dim, sizeof(float) * dim);
        write_slice_f32(base + "/" + names[part], col.data(), n, dim, false);
      }
      std::vector<int64_t> fk, fc, fts;
      tb.filter.export_state(fk, fc, fts);
      write_slice_i64(base + "/admit_count/key", fk, false);
      write_slice_i64(base + "/admit_count", fc, false);
      write_slice_i64(base + "/evict_timestamp", fts, false);
    }
  }

  // rank 0: concatenate <table>/rank*/<part> into <table>/<part>
  void merge_files(const std::string& path, int world) {
    for (size_t t = 0; t < tables_.size(); ++t) {
      const std::string tdir = path + "/" + cfgs_[t].table_name;
      const int dim = tables_[t]->host.dim();
      static const char* i64_parts[] = {"key", "evicted_key", "admit_count/key", "admit_count", "evict_timestamp"};
      for (const char* part : i64_parts) {
        for (int r = 0; r < world; ++r) {
          auto v = read_slice_i64(tdir + "/rank" + std::to_string(r) + "/" + part);
          write_slice_i64(tdir + "/" + part, v, r > 0);
        }
      }
      static const char* f32_parts[] = {"embedding", "momentum1", "momentum2"};
      for (int p = 0; p < 1 + tables_[t]->host.optim_num() && p < 3; ++p) {
        for (int r = 0; r < world; ++r) {
          int64_t c, d;
          auto v = read_slice_f32(tdir + "/rank" + std::to_string(r) + "/" + f32_parts[p], &c, &d);
          write_slice_f32(tdir + "/" + f32_parts[p], v.data(), static_cast<int64_t>(v.size()) / dim, dim, r > 0);
        }
      }
    }
  }

  // every rank reads the merged files and keeps key % world == rank (world-size-elastic reload)
  // `incremental` false: a full restore - the host table and the filter state are reset first, so keys that are not in
  // the checkpoint do not survive it.  true: a delta on top of the current state - its rows are inserted or overwritten
  // and the keys it lists as evicted are erased.
  void load(const std::string& path, int rank, int world, bool incremental = false) {
    for (size_t t = 0; t < tables_.size(); ++t) {
      Table& tb = *tables_[t];
      const std::string tdir = path + "/" + cfgs_[t].table_name;
      if (!incremental) {
        tb.host.clear();
        tb.filter.clear();
        std::lock_guard<std::mutex> lk(tb.mu);
        tb.touched.clear();
        tb.evicted.clear();
      } else {
        auto gone = read_slice_i64(tdir + "/evicted_key");
        std::vector<int64_t> mine_gone;
        for (int64_t k : gone) { int64_t m = k % world; if (m < 0) m += world; if (m == rank) mine_gone.push_back(k); }
        tb.host.erase(mine_gone.data(), static_cast<int64_t>(mine_gone.size()));
        tb.filter.erase(mine_gone.data(), static_cast<int64_t>(mine_gone.size()));
      }
      auto keys = read_slice_i64(tdir + "/key");
      const int dim = tb.host.dim(), rf = tb.host.row_floats();
      std::vector<std::vector<float>> parts;
      static const char* f32_parts[] = {"embedding", "momentum1", "momentum2"};
      for (int p = 0; p < 1 + tb.host.optim_num() && p < 3; ++p) {
        int64_t c, d;
        parts.push_back(read_slice_f32(tdir + "/" + f32_parts[p], &c, &d));
        if (!parts.back().empty() && d != dim) throw std::runtime_error("checkpoint dim mismatch for " + cfgs_[t].table_name);
      }
      std::vector<int64_t> mine;
      std::vector<float> rows;
      for (size_t i = 0; i < keys.size(); ++i) {
        int64_t m = keys[i] % world; if (m < 0) m += world;
        if (m != rank) continue;
        mine.push_back(keys[i]);
        const size_t base = rows.size();
        rows.resize(base + rf, 0.f);
        for (size_t p = 0; p < parts.size(); ++p)
          if (parts[p].size() >= (i + 1) * static_cast<size_t>(dim))
            std::memcpy(rows.data() + base + p * dim, parts[p].data() + i * dim, sizeof(float) * dim);
      }
      tb.host.insert_or_assign(mine.data(), static_cast<int64_t>(mine.size()), rows.data());
      auto fk = read_slice_i64(tdir + "/admit_count/key");
      auto fc = read_slice_i64(tdir + "/admit_count");
      auto fts = read_slice_i64(tdir + "/evict_timestamp");
      std::vector<int64_t> k2, c2, t2;
      for (size_t i = 0; i < fk.size(); ++i) {
        int64_t m = fk[i] % world; if (m < 0) m += world;
        if (m != rank) continue;
        k2.push_back(fk[i]); c2.push_back(i < fc.size() ? fc[i] : 0); t2.push_back(i < fts.size() ? fts[i] : -1);
      }
      tb.filter.import_state(k2.data(), c2.data(), t2.data(), static_cast<int64_t>(k2.size()));
    }
  }

 private:
  struct Table {
    explicit Table(const EmbConfig& c)
        : swap(c.cache_size, c.admit_evict.admit_enabled()), host(c.emb_dim, c.optim_num, c.init), filter(c.admit_evict) {}
    SwapManager swap;
    HostEmbTable host;
    FeatureFilter filter;
    std::mutex mu;
    std::unordered_set<int64_t> touched;
    std::unordered_set<int64_t> evicted;       // keys evicted / erased since the last save (incremental checkpoints)
  };
  std::vector<EmbConfig> cfgs_;
  std::vector<std::unique_ptr<Table>> tables_;
  ThreadPool pool_;
};

}  // namespace rbh
