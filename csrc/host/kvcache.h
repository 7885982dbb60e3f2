// Host-side bookkeeping of the paged KV cache used by HSTU ranking inference.
//
//   KVPageAllocator  which device page holds which token range of which user; LRU order; pages of
//                    prefixes already offloaded to the host can be reclaimed before whole users are
//                    evicted; per-user offload locks; fills the packed metadata the kernels consume.
//   HostChunkIndex   which pinned host chunk holds which token range of which user (LRU, capacity).
//
// Behavioural spec (reference): inference/kvcache_manager/src/npu_kvcache_manager_impl.{h,cpp}
// (lookup :100-125, alloc_single_sequence :206-303, allocate :305-438, check_for_offload :440-500,
// acquire/release_offload_pages :554-691), native_host_kvcache_manager_impl.cpp :367-483 (chunk
// allocation), docs/codeview.md.  Metadata layout: kvcache_metadata.py:66-126.
#pragma once
#include <deque>
#include <list>
#include <unordered_map>
#include <unordered_set>

#include "common.h"

namespace rbh {

struct KVAllocResult {
  std::vector<int32_t> page_indices;   // concatenated page ids of every sequence of the batch
  std::vector<int32_t> metadata;       // 5B + 4 ints (the device appends 2 * new_tokens more)
  int32_t new_tokens = 0;
};

class KVPageAllocator {
 public:
  KVPageAllocator(int page_size, int chunk_size, int num_primary_pages, int num_buffer_pages, int max_batch,
                  int max_seq_len)
      : page_(page_size), chunk_(chunk_size), n_pages_(num_primary_pages), n_buffer_(num_buffer_pages),
        max_batch_(max_batch), max_seq_(max_seq_len) {
    if (page_size <= 0 || chunk_size % page_size != 0) throw std::invalid_argument("chunk size must be a multiple of page size");
    evict_all();
  }

  int page_size() const { return page_; }
  int free_pages() const { return static_cast<int>(free_.size()); }
  int total_offloaded_pages() const { return offloaded_pages_; }
  int64_t num_users() const { return static_cast<int64_t>(users_.size()); }

  // (cached start position, cached length) on the device per uid; (0, 0) when unknown
  void lookup(const int64_t* uids, int n, int32_t* start, int32_t* length) const {
    for (int i = 0; i < n; ++i) {
      auto it = users_.find(uids[i]);
      start[i] = it == users_.end() ? 0 : it->second.start;
      length[i] = it == users_.end() ? 0 : it->second.length;
    }
  }

  void evict(int64_t uid) {
    auto it = users_.find(uid);
    if (it == users_.end()) return;
    for (int p : it->second.pages) free_.push_back(p);
    offloaded_pages_ -= offloaded_pages_of(it->second);
    lru_.erase(it->second.lru);
    users_.erase(it);
  }

  // give back the pages whose tokens already live on the host
  void evict_offloaded(int64_t uid) {
    auto it = users_.find(uid);
    if (it == users_.end()) return;
    User& u = it->second;
    const int n = offloaded_pages_of(u);
    if (n == 0) return;
    for (int i = 0; i < n; ++i) free_.push_back(u.pages[i]);
    u.pages.erase(u.pages.begin(), u.pages.begin() + n);
    u.start += n * page_;
    u.length -= n * page_;
    offloaded_pages_ -= n;
  }

  // forget the tokens at and beyond new_total (e.g. scratch tokens that were appended for one request only)
  void truncate(int64_t uid, int new_total) {
    auto it = users_.find(uid);
    if (it == users_.end()) return;
    User& u = it->second;
    if (new_total <= u.start) { if (u.offload_lock == 0) evict(uid); return; }
    if (new_total >= u.start + u.length) return;
    const int keep = ceil_div(new_total - u.start, page_);
    for (size_t p = static_cast<size_t>(keep); p < u.pages.size(); ++p) free_.push_back(u.pages[p]);
    u.pages.resize(static_cast<size_t>(keep));
    u.length = new_total - u.start;
    if (u.offloaded > new_total) {
      offloaded_pages_ -= offloaded_pages_of(u);
      u.offloaded = new_total;
      offloaded_pages_ += offloaded_pages_of(u);
    }
  }

  void evict_all() {
    users_.clear();
    lru_.clear();
    free_.clear();
    offloaded_pages_ = 0;
    for (int p = 0; p < n_pages_; ++p) free_.push_back(p);
  }

  // Pages for one user so that tokens [0, new_total) are addressable: pages for the host-cached prefix
  // that must be brought on board, the pages the user already holds, and pages for appended tokens.
  std::vector<int32_t> alloc_single_sequence(int64_t uid, int new_total, int host_cached_len,
                                             const std::unordered_set<int64_t>& frozen) {
    if (new_total < 0 || new_total > max_seq_) throw std::invalid_argument("new_total_length must be in [0, max_sequence_length]");
    if (host_cached_len < 0 || host_cached_len > new_total) throw std::invalid_argument("host_cached_length must be in [0, new_total_length]");
    const int total_pages = ceil_div(new_total, page_);
    const bool known = touch(uid);
    User& u = users_[uid];
    int onload_pages = 0;
    if (!known || u.length == 0) onload_pages = ceil_div(host_cached_len, page_);
    else if (u.start > 0) onload_pages = u.start / page_;
    const int cur_pages = ceil_div(u.length, page_);
    if (onload_pages + cur_pages > total_pages) throw std::runtime_error("cached sequence is longer than the requested total length");
    const int append_pages = total_pages - onload_pages - cur_pages;
    const int need = onload_pages + append_pages;

    // 1) reclaim offloaded prefixes of other unlocked users, oldest first
    for (auto it = lru_.begin(); it != lru_.end() && need > static_cast<int>(free_.size());) {
      const int64_t other = *it;
      ++it;
      if (other == uid || frozen.count(other) || locked(other)) continue;
      evict_offloaded(other);
      auto uo = users_.find(other);
      if (uo != users_.end() && uo->second.length == 0) { lru_.erase(uo->second.lru); users_.erase(uo); }
    }
    // 2) evict whole users in LRU order
    while (need > static_cast<int>(free_.size())) {
      int64_t victim = 0;
      bool found = false;
      for (int64_t cand : lru_)
        if (cand != uid && !frozen.count(cand) && !locked(cand)) { victim = cand; found = true; break; }
      if (!found) throw std::runtime_error("No evictable UID: all cached UIDs are frozen or offload-locked");
      evict(victim);
    }
    std::vector<int32_t> pages(static_cast<size_t>(total_pages));
    int w = 0;
    for (int i = 0; i < onload_pages; ++i) pages[w++] = pop_free();
    for (int i = 0; i < cur_pages; ++i) pages[w++] = u.pages[i];
    for (int i = 0; i < append_pages; ++i) pages[w++] = pop_free();
    u.pages = pages;
    u.start = 0;
    u.length = new_total;
    return pages;
  }

  // Allocate for a batch and build the packed int32 metadata:
  //   [0, B]            page_indptr            [B+1, 2B]       last_page_len
  //   [2B+1, 3B]        total_history_lengths  [3B+1, 4B+1]    total_history_offsets
  //   [4B+2]            new_history_nnz        [4B+3, 5B+3]    new_history_offsets
  // (batch_indices and positions of the new tokens are appended on the device by a kernel).
  KVAllocResult allocate(const int64_t* uids, const int32_t* total_lens, const int32_t* host_cached_lens, int B) {
    if (B > max_batch_) throw std::invalid_argument("batch size exceeds max_batch_size");
    KVAllocResult r;
    r.metadata.assign(static_cast<size_t>(5 * B + 4), 0);
    int32_t* indptr = r.metadata.data();
    int32_t* last_len = indptr + B + 1;
    int32_t* tot_len = indptr + 2 * B + 1;
    int32_t* tot_off = indptr + 3 * B + 1;
    int32_t* nnz = indptr + 4 * B + 2;
    int32_t* new_off = indptr + 4 * B + 3;
    std::vector<int> cached(B);
    for (int i = 0; i < B; ++i) {
      if (total_lens[i] < 0 || total_lens[i] > max_seq_) throw std::invalid_argument("total history length out of range");
      if (host_cached_lens[i] < 0 || host_cached_lens[i] > total_lens[i]) throw std::invalid_argument("host cached length out of range");
      int dev_end = 0;
      auto it = users_.find(uids[i]);
      if (it != users_.end()) {
        dev_end = it->second.start + it->second.length;
        if (dev_end > total_lens[i]) throw std::runtime_error("device cached range exceeds total history length");
      }
      cached[i] = std::max<int>(host_cached_lens[i], dev_end);
    }
    for (int i = 0; i < B; ++i) {
      bool was_known = users_.count(uids[i]) > 0;
      User& u = users_[uids[i]];
      if (!was_known) { lru_.push_back(uids[i]); u.lru = std::prev(lru_.end()); }
      offloaded_pages_ -= offloaded_pages_of(u);
      u.offloaded = host_cached_lens[i];
      offloaded_pages_ += offloaded_pages_of(u);
    }
    const std::unordered_set<int64_t> frozen(uids, uids + B);
    for (int i = 0; i < B; ++i) {
      std::vector<int32_t> pages = alloc_single_sequence(uids[i], total_lens[i], host_cached_lens[i], frozen);
      r.page_indices.insert(r.page_indices.end(), pages.begin(), pages.end());
      indptr[i + 1] = indptr[i] + static_cast<int32_t>(pages.size());
      int ll = users_[uids[i]].length % page_;
      last_len[i] = ll == 0 ? page_ : ll;
      tot_len[i] = total_lens[i];
      tot_off[i + 1] = tot_off[i] + total_lens[i];
      new_off[i + 1] = new_off[i] + total_lens[i] - cached[i];
    }
    *nnz = new_off[B];
    r.new_tokens = new_off[B];
    return r;
  }

  // users that hold at least one full chunk of tokens not yet on the host (batch users first, then
  // others in LRU order while the buffer-page budget is exceeded)
  std::vector<int64_t> check_for_offload(const int64_t* uids, int n, int max_offload_pages) const {
    std::vector<int64_t> out;
    std::unordered_set<int64_t> chosen;
    int64_t pages = 0;
    for (int i = 0; i < n; ++i) {
      auto it = users_.find(uids[i]);
      if (it == users_.end()) continue;
      const User& u = it->second;
      const int end = u.start + u.length;
      if (end - u.offloaded >= chunk_ && chosen.insert(uids[i]).second) out.push_back(uids[i]);
      pages += std::max(0, (end - u.offloaded) / page_);
    }
    for (int64_t uid : lru_) {
      if (static_cast<int64_t>(offloaded_pages_) + pages + static_cast<int64_t>(free_.size()) > n_buffer_) break;
      if (chosen.count(uid)) continue;
      const User& u = users_.at(uid);
      if (u.offloaded < u.start) continue;
      const int end = u.start + u.length;
      if (end - u.offloaded >= chunk_) {
        pages += (end - u.offloaded) / page_;
        if (pages > max_offload_pages) break;
        out.push_back(uid);
        chosen.insert(uid);
      }
    }
    return out;
  }

  struct OffloadPlan { std::vector<int64_t> uids; std::vector<int32_t> start; std::vector<std::vector<int32_t>> pages; };

  // lock users and return the pages of their not-yet-offloaded full pages
  OffloadPlan acquire_offload_pages(const int64_t* uids, int n, const int32_t* offloaded_lengths, bool always) {
    OffloadPlan plan;
    for (int i = 0; i < n; ++i) {
      auto it = users_.find(uids[i]);
      if (always) {
        plan.uids.push_back(uids[i]);
        plan.start.push_back(0);
        plan.pages.emplace_back(it == users_.end() ? std::vector<int32_t>() : it->second.pages);
        if (it != users_.end()) ++it->second.offload_lock;
        continue;
      }
      if (it == users_.end()) continue;
      User& u = it->second;
      if (offloaded_lengths) {
        offloaded_pages_ -= offloaded_pages_of(u);
        u.offloaded = offloaded_lengths[i];
        offloaded_pages_ += offloaded_pages_of(u);
      }
      if (u.offloaded < u.start) continue;
      const int end = u.start + u.length;
      if (end - u.offloaded < chunk_) continue;
      const int first = (u.offloaded - u.start) / page_;
      const int count = (end - u.offloaded) / page_;
      plan.uids.push_back(uids[i]);
      plan.start.push_back(u.offloaded);
      plan.pages.emplace_back(u.pages.begin() + first, u.pages.begin() + first + count);
      ++u.offload_lock;
    }
    return plan;
  }

  void release_offload_pages(const int64_t* uids, const int32_t* start, const int32_t* length, const uint8_t* done, int n) {
    for (int i = 0; i < n; ++i) {
      auto it = users_.find(uids[i]);
      if (it == users_.end() || it->second.offload_lock == 0) continue;
      User& u = it->second;
      if (done[i]) {
        offloaded_pages_ -= offloaded_pages_of(u);
        u.offloaded = start[i] + length[i];
        offloaded_pages_ += offloaded_pages_of(u);
      }
      --u.offload_lock;
    }
  }

  // an onboard (host -> device) that failed: forget the prefix pages that were reserved for it
  void revoke_onboard_pages(const int64_t* uids, const int32_t* onboard_start, const int32_t* onboard_len, int n) {
    for (int i = 0; i < n; ++i) {
      auto it = users_.find(uids[i]);
      if (it == users_.end() || onboard_len[i] <= 0) continue;
      User& u = it->second;
      const int drop = std::min<int>(ceil_div(onboard_start[i] + onboard_len[i] - u.start, page_), static_cast<int>(u.pages.size()));
      if (drop <= 0) continue;
      for (int p = 0; p < drop; ++p) free_.push_back(u.pages[p]);
      u.pages.erase(u.pages.begin(), u.pages.begin() + drop);
      const int tokens = std::min(drop * page_, u.length);
      u.start += tokens;
      u.length -= tokens;
    }
  }

  std::vector<int32_t> pages_of(int64_t uid) const {
    auto it = users_.find(uid);
    return it == users_.end() ? std::vector<int32_t>() : it->second.pages;
  }

 private:
  struct User {
    std::vector<int32_t> pages;
    int start = 0, length = 0, offloaded = 0, offload_lock = 0;
    std::list<int64_t>::iterator lru;
  };
  static int ceil_div(int a, int b) { return a <= 0 ? 0 : (a + b - 1) / b; }
  int offloaded_pages_of(const User& u) const { return std::max(0, (u.offloaded - u.start) / page_); }
  bool locked(int64_t uid) const { auto it = users_.find(uid); return it != users_.end() && it->second.offload_lock > 0; }
  int pop_free() { int p = free_.front(); free_.pop_front(); return p; }
  // move to the most-recently-used end; returns whether the user was already known
  bool touch(int64_t uid) {
    auto it = users_.find(uid);
    const bool known = it != users_.end();
    if (known) lru_.erase(it->second.lru);
    lru_.push_back(uid);
    users_[uid].lru = std::prev(lru_.end());
    return known;
  }

  int page_, chunk_, n_pages_, n_buffer_, max_batch_, max_seq_;
  int offloaded_pages_ = 0;
  std::deque<int> free_;
  std::list<int64_t> lru_;
  std::unordered_map<int64_t, User> users_;
};

// Index of the pinned host chunk pool: chunk c holds tokens [k*chunk, (k+1)*chunk) of one user for
// all layers.  LRU over users; a user's chunks are contiguous in token order starting at token 0.
class HostChunkIndex {
 public:
  HostChunkIndex(int64_t num_chunks, int chunk_tokens) : chunk_(chunk_tokens) {
    for (int64_t c = 0; c < num_chunks; ++c) free_.push_back(c);
  }
  int64_t free_chunks() const { return static_cast<int64_t>(free_.size()); }
  int chunk_tokens() const { return chunk_; }

  // (start, length) of host-resident tokens per uid (start is always 0)
  void lookup(const int64_t* uids, int n, int32_t* start, int32_t* length) {
    for (int i = 0; i < n; ++i) {
      auto it = users_.find(uids[i]);
      start[i] = 0;
      length[i] = it == users_.end() ? 0 : static_cast<int32_t>(it->second.chunks.size()) * chunk_;
      if (it != users_.end()) touch(it);
    }
  }
  // chunk ids holding tokens [first_token, first_token + n_tokens) of uid (both multiples of chunk)
  std::vector<int64_t> chunks_of(int64_t uid, int first_token, int n_tokens) const {
    std::vector<int64_t> out;
    auto it = users_.find(uid);
    if (it == users_.end()) return out;
    for (int c = first_token / chunk_; c < (first_token + n_tokens) / chunk_ && c < static_cast<int>(it->second.chunks.size()); ++c)
      out.push_back(it->second.chunks[c]);
    return out;
  }
  // reserve chunks so that uid holds tokens [0, start + n_tokens); start must equal the current length.
  // Evicts least-recently-used other users when the pool is full; returns the new chunk ids, or an
  // empty vector when the request cannot be satisfied (caller reports "no space").
  std::vector<int64_t> append(int64_t uid, int start_token, int n_tokens, const std::unordered_set<int64_t>& pinned) {
    auto it = users_.find(uid);
    const int have = it == users_.end() ? 0 : static_cast<int>(it->second.chunks.size()) * chunk_;
    if (start_token != have || n_tokens % chunk_ != 0) return {};
    const int need = n_tokens / chunk_;
    while (static_cast<int>(free_.size()) < need) {
      bool found = false;
      for (int64_t cand : lru_)
        if (cand != uid && !pinned.count(cand)) { evict(cand); found = true; break; }
      if (!found) return {};
    }
    if (it == users_.end()) { lru_.push_back(uid); it = users_.emplace(uid, User()).first; it->second.lru = std::prev(lru_.end()); }
    else touch(it);
    std::vector<int64_t> out;
    for (int i = 0; i < need; ++i) { out.push_back(free_.front()); it->second.chunks.push_back(free_.front()); free_.pop_front(); }
    return out;
  }
  // undo an append whose copy failed or timed out
  void rollback(int64_t uid, int n_chunks) {
    auto it = users_.find(uid);
    if (it == users_.end()) return;
    for (int i = 0; i < n_chunks && !it->second.chunks.empty(); ++i) { free_.push_back(it->second.chunks.back()); it->second.chunks.pop_back(); }
    if (it->second.chunks.empty()) { lru_.erase(it->second.lru); users_.erase(it); }
  }
  void evict(int64_t uid) {
    auto it = users_.find(uid);
    if (it == users_.end()) return;
    for (int64_t c : it->second.chunks) free_.push_back(c);
    lru_.erase(it->second.lru);
    users_.erase(it);
  }
  void evict_all() { std::vector<int64_t> all(lru_.begin(), lru_.end()); for (int64_t u : all) evict(u); }
  int64_t num_users() const { return static_cast<int64_t>(users_.size()); }

 private:
  struct User { std::vector<int64_t> chunks; std::list<int64_t>::iterator lru; };
  void touch(std::unordered_map<int64_t, User>::iterator it) {
    lru_.erase(it->second.lru);
    lru_.push_back(it->first);
    it->second.lru = std::prev(lru_.end());
  }
  int chunk_;
  std::deque<int64_t> free_;
  std::list<int64_t> lru_;
  std::unordered_map<int64_t, User> users_;
};

}  // namespace rbh
