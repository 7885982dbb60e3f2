// Shared host utilities: flat hash map, thread pool with futures, logger, stopwatch.
// Counterparts in the reference: torchrec_embcache/csrc/utils/*.h (AsyncTask, ThreadPool, SafeQueue,
// Logger with GLOG_stderrthreshold levels, TimeCost).
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <future>
#include <memory>
#include <mutex>
#include <queue>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace rbh {

// ----------------------------------------------------------------------------- logging
enum LogLevel : int { LOG_TRACE = -2, LOG_DEBUG = -1, LOG_INFO = 0, LOG_WARN = 1, LOG_ERROR = 2 };

inline int log_threshold() {
  static int lvl = [] {
    const char* e = std::getenv("GLOG_stderrthreshold");
    if (!e) return static_cast<int>(LOG_WARN);
    int v = std::atoi(e);
    if (v < LOG_TRACE) v = LOG_TRACE;
    if (v > LOG_ERROR) v = LOG_ERROR;
    return v;
  }();
  return lvl;
}

template <typename... Args>
inline void log(LogLevel lvl, const char* fmt, Args... args) {
  if (static_cast<int>(lvl) < log_threshold()) return;
  static const char* names[] = {"TRACE", "DEBUG", "INFO", "WARN", "ERROR"};
  std::fprintf(stderr, "[recsdk_b200][%s] ", names[static_cast<int>(lvl) + 2]);
  if constexpr (sizeof...(args) == 0) std::fputs(fmt, stderr);
  else std::fprintf(stderr, fmt, args...);
  std::fputc('\n', stderr);
}

class TimeCost {
 public:
  TimeCost() : t0_(std::chrono::steady_clock::now()) {}
  double ms() const {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0_).count();
  }
 private:
  std::chrono::steady_clock::time_point t0_;
};

// ----------------------------------------------------------------------------- hashing
inline uint64_t mix64(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33;
  return x;
}

// Open-addressing map int64 -> V with linear probing and tombstone-free backward-shift deletion.
// The empty key is INT64_MIN (never a valid id).
template <typename V>
class FlatMap {
 public:
  static constexpr int64_t kEmpty = INT64_MIN;
  explicit FlatMap(size_t reserve = 16) { rehash(cap_for(reserve)); }
  size_t size() const { return size_; }
  bool empty() const { return size_ == 0; }
  void clear() { std::fill(keys_.begin(), keys_.end(), kEmpty); size_ = 0; }
  void reserve(size_t n) { if (cap_for(n) > keys_.size()) rehash(cap_for(n)); }

  V* find(int64_t k) {
    size_t i = mix64(static_cast<uint64_t>(k)) & mask_;
    while (keys_[i] != kEmpty) {
      if (keys_[i] == k) return &vals_[i];
      i = (i + 1) & mask_;
    }
    return nullptr;
  }
  const V* find(int64_t k) const { return const_cast<FlatMap*>(this)->find(k); }

  // returns (slot pointer, inserted)
  std::pair<V*, bool> insert(int64_t k, const V& v) {
    if ((size_ + 1) * 10 > keys_.size() * 7) rehash(keys_.size() * 2);
    size_t i = mix64(static_cast<uint64_t>(k)) & mask_;
    while (keys_[i] != kEmpty) {
      if (keys_[i] == k) return {&vals_[i], false};
      i = (i + 1) & mask_;
    }
    keys_[i] = k; vals_[i] = v; ++size_;
    return {&vals_[i], true};
  }

  bool erase(int64_t k) {
    size_t i = mix64(static_cast<uint64_t>(k)) & mask_;
    while (keys_[i] != kEmpty && keys_[i] != k) i = (i + 1) & mask_;
    if (keys_[i] == kEmpty) return false;
    size_t j = i;
    for (;;) {                                   // backward-shift the cluster
      j = (j + 1) & mask_;
      if (keys_[j] == kEmpty) break;
      const size_t home = mix64(static_cast<uint64_t>(keys_[j])) & mask_;
      const bool movable = (i <= j) ? (home <= i || home > j) : (home <= i && home > j);
      if (movable) { keys_[i] = keys_[j]; vals_[i] = std::move(vals_[j]); i = j; }
    }
    keys_[i] = kEmpty; --size_;
    return true;
  }

  template <typename F>
  void for_each(F&& f) const {
    for (size_t i = 0; i < keys_.size(); ++i)
      if (keys_[i] != kEmpty) f(keys_[i], vals_[i]);
  }
  template <typename F>
  void for_each_mut(F&& f) {
    for (size_t i = 0; i < keys_.size(); ++i)
      if (keys_[i] != kEmpty) f(keys_[i], vals_[i]);
  }

 private:
  static size_t cap_for(size_t n) { size_t c = 16; while (c * 7 < n * 10 + 10) c <<= 1; return c; }
  void rehash(size_t cap) {
    std::vector<int64_t> ok = std::move(keys_);
    std::vector<V> ov = std::move(vals_);
    keys_.assign(cap, kEmpty); vals_.assign(cap, V()); mask_ = cap - 1; size_ = 0;
    for (size_t i = 0; i < ok.size(); ++i)
      if (ok[i] != kEmpty) {
        size_t j = mix64(static_cast<uint64_t>(ok[i])) & mask_;
        while (keys_[j] != kEmpty) j = (j + 1) & mask_;
        keys_[j] = ok[i]; vals_[j] = std::move(ov[i]); ++size_;
      }
  }
  std::vector<int64_t> keys_;
  std::vector<V> vals_;
  size_t mask_ = 0, size_ = 0;
};

// ----------------------------------------------------------------------------- thread pool
class ThreadPool {
 public:
  explicit ThreadPool(size_t n) : stop_(false) {
    if (n == 0) n = 1;
    for (size_t i = 0; i < n; ++i)
      workers_.emplace_back([this] {
        for (;;) {
          std::function<void()> job;
          {
            std::unique_lock<std::mutex> lk(mu_);
            cv_.wait(lk, [this] { return stop_ || !jobs_.empty(); });
            if (stop_ && jobs_.empty()) return;
            job = std::move(jobs_.front());
            jobs_.pop();
          }
          job();
        }
      });
  }
  ~ThreadPool() {
    { std::lock_guard<std::mutex> lk(mu_); stop_ = true; }
    cv_.notify_all();
    for (auto& w : workers_) w.join();
  }
  template <typename F>
  auto submit(F&& f) -> std::future<decltype(f())> {
    using R = decltype(f());
    auto task = std::make_shared<std::packaged_task<R()>>(std::forward<F>(f));
    std::future<R> fut = task->get_future();
    { std::lock_guard<std::mutex> lk(mu_); jobs_.emplace([task] { (*task)(); }); }
    cv_.notify_one();
    return fut;
  }
  size_t size() const { return workers_.size(); }
 private:
  std::vector<std::thread> workers_;
  std::queue<std::function<void()>> jobs_;
  std::mutex mu_;
  std::condition_variable cv_;
  bool stop_;
};

inline int env_int(const char* name, int def, int lo, int hi) {
  const char* e = std::getenv(name);
  if (!e) return def;
  int v = std::atoi(e);
  if (v < lo) v = lo;
  if (v > hi) v = hi;
  return v;
}

}  // namespace rbh
