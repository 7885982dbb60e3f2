// Log-structured disk tier for embedding rows (the third tier below HBM and host DRAM).
//
// Each table appends rows to data files (<dir>/<table>.<n>.data, records = [int64 key | fp32 row]) and
// keeps an in-memory key -> (file, offset) map.  Overwritten or deleted records become stale; when the
// stale fraction of a table exceeds the threshold a compaction rewrites the live rows into fresh files.
// When a path fills up (write error / size budget) the table spills to the next configured path.
// Save writes a step-stamped meta file; Load rebuilds the map from it.  A monitor thread compacts in
// the background.
//
// Behavioural spec (reference, TensorFlow stack): training/tf_rec_v1/src/core/ssd_engine/
// {ssd_engine.h:33-83, table.h:41-88, table.cpp:31-120, file.h:33-96} and l3_storage/cache_manager.h:49-55
// (return codes).
#pragma once
#include <atomic>
#include <fstream>
#include <map>
#include <unordered_map>

#include "common.h"
#include "embcache.h"

namespace rbh {

enum DiskRc : int { DISK_OK = 0, DISK_ERROR = 1, DISK_SPACE_NOT_ENOUGH = 2 };

class DiskTable {
 public:
  DiskTable(std::string name, std::vector<std::string> paths, int row_floats, int64_t max_bytes_per_path)
      : name_(std::move(name)), paths_(std::move(paths)), rf_(row_floats), budget_(max_bytes_per_path),
        rec_bytes_(sizeof(int64_t) + sizeof(float) * static_cast<size_t>(row_floats)) {
    if (paths_.empty()) throw std::invalid_argument("DiskTable needs at least one path");
    for (auto& p : paths_) { fs::check_path(p); fs::mkdirs(p); }
    used_.assign(paths_.size(), 0);
  }

  int64_t size() const { std::lock_guard<std::mutex> lk(mu_); return static_cast<int64_t>(loc_.size()); }
  int64_t stale() const { std::lock_guard<std::mutex> lk(mu_); return stale_; }
  int64_t bytes_used() const { std::lock_guard<std::mutex> lk(mu_); int64_t s = 0; for (auto u : used_) s += u; return s; }
  bool contains(int64_t key) const { std::lock_guard<std::mutex> lk(mu_); return loc_.find(key) != nullptr; }

  int insert(const int64_t* keys, int64_t n, const float* rows) {
    std::lock_guard<std::mutex> lk(mu_);
    for (int64_t i = 0; i < n; ++i) {
      Loc l;
      const int rc = append_record(keys[i], rows + i * rf_, l);
      if (rc != DISK_OK) return rc;
      auto r = loc_.insert(keys[i], l);
      if (!r.second) { *r.first = l; ++stale_; }
    }
    return DISK_OK;
  }

  // found[i] = 1 when present; rows of missing keys are left untouched
  int fetch(const int64_t* keys, int64_t n, float* rows_out, uint8_t* found) const {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& f : files_) if (f.out.is_open()) f.out.flush();
    for (int64_t i = 0; i < n; ++i) {
      const Loc* l = loc_.find(keys[i]);
      if (!l) { if (found) found[i] = 0; continue; }
      std::ifstream in(files_[l->file].path, std::ios::binary);
      if (!in) return DISK_ERROR;
      in.seekg(static_cast<std::streamoff>(l->offset + sizeof(int64_t)));
      in.read(reinterpret_cast<char*>(rows_out + i * rf_), sizeof(float) * rf_);
      if (!in) return DISK_ERROR;
      if (found) found[i] = 1;
    }
    return DISK_OK;
  }

  void erase(const int64_t* keys, int64_t n) {
    std::lock_guard<std::mutex> lk(mu_);
    for (int64_t i = 0; i < n; ++i)
      if (loc_.erase(keys[i])) ++stale_;
  }

  std::vector<int64_t> export_keys() const {
    std::lock_guard<std::mutex> lk(mu_);
    std::vector<int64_t> out;
    loc_.for_each([&](int64_t k, const Loc&) { out.push_back(k); });
    return out;
  }

  double stale_fraction() const {
    std::lock_guard<std::mutex> lk(mu_);
    const double total = static_cast<double>(loc_.size()) + stale_;
    return total > 0 ? stale_ / total : 0.0;
  }

  // rewrite live rows into new files and delete the old ones
  int compact() {
    std::lock_guard<std::mutex> lk(mu_);
    if (stale_ == 0) return DISK_OK;
    for (auto& f : files_) if (f.out.is_open()) f.out.close();
    std::vector<File> old;
    old.swap(files_);
    std::vector<int64_t> old_used = used_;
    std::fill(used_.begin(), used_.end(), 0);
    FlatMap<Loc> fresh(loc_.size() + 1);
    std::vector<float> row(rf_);
    int rc = DISK_OK;
    loc_.for_each([&](int64_t k, const Loc& l) {
      if (rc != DISK_OK) return;
      std::ifstream in(old[l.file].path, std::ios::binary);
      in.seekg(static_cast<std::streamoff>(l.offset + sizeof(int64_t)));
      in.read(reinterpret_cast<char*>(row.data()), sizeof(float) * rf_);
      if (!in) { rc = DISK_ERROR; return; }
      Loc nl;
      rc = append_record(k, row.data(), nl);
      if (rc == DISK_OK) fresh.insert(k, nl);
    });
    if (rc != DISK_OK) return rc;
    for (auto& f : files_) if (f.out.is_open()) f.out.flush();
    for (auto& f : old) std::remove(f.path.c_str());
    loc_ = std::move(fresh);
    stale_ = 0;
    return DISK_OK;
  }

  // <path0>/<table>.meta.<step>: [count][key, file, offset]* + the list of data files
  void save(int64_t step) {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& f : files_) if (f.out.is_open()) f.out.flush();
    std::vector<int64_t> blob;
    blob.push_back(static_cast<int64_t>(files_.size()));
    blob.push_back(static_cast<int64_t>(loc_.size()));
    loc_.for_each([&](int64_t k, const Loc& l) { blob.push_back(k); blob.push_back(l.file); blob.push_back(l.offset); });
    fs::write_file(meta_path(step), blob.data(), blob.size() * sizeof(int64_t));
    std::string names;
    for (auto& f : files_) names += f.path + "\n";
    fs::write_file(meta_path(step) + ".files", names.data(), names.size());
  }

  void load(int64_t step) {
    std::lock_guard<std::mutex> lk(mu_);
    auto raw = fs::read_file(meta_path(step));
    const int64_t* b = reinterpret_cast<const int64_t*>(raw.data());
    const int64_t nfiles = b[0], count = b[1];
    auto names = fs::read_file(meta_path(step) + ".files");
    files_.clear();
    std::string cur;
    for (char c : names) {
      if (c == '\n') { File f; f.path = cur; f.path_idx = 0; files_.push_back(std::move(f)); cur.clear(); }
      else cur.push_back(c);
    }
    if (static_cast<int64_t>(files_.size()) != nfiles) throw std::runtime_error("disk tier meta/file list mismatch");
    loc_.clear();
    for (int64_t i = 0; i < count; ++i) loc_.insert(b[2 + 3 * i], Loc{static_cast<int32_t>(b[3 + 3 * i]), b[4 + 3 * i]});
    stale_ = 0;
    next_file_id_ = nfiles;
  }

 private:
  struct Loc { int32_t file = 0; int64_t offset = 0; };
  struct File { std::string path; std::ofstream out; int64_t bytes = 0; size_t path_idx = 0; };
  static constexpr int64_t kMaxFileBytes = 256ll << 20;

  std::string meta_path(int64_t step) const { return paths_[0] + "/" + name_ + ".meta." + std::to_string(step); }

  int open_new_file() {
    for (size_t attempt = 0; attempt < paths_.size(); ++attempt) {
      const size_t pi = (cur_path_ + attempt) % paths_.size();
      if (budget_ > 0 && used_[pi] + static_cast<int64_t>(rec_bytes_) > budget_) continue;
      File f;
      f.path = paths_[pi] + "/" + name_ + "." + std::to_string(next_file_id_++) + ".data";
      f.out.open(f.path, std::ios::binary | std::ios::trunc);
      if (!f.out) continue;
      f.path_idx = pi;
      cur_path_ = pi;
      files_.push_back(std::move(f));
      return DISK_OK;
    }
    return DISK_SPACE_NOT_ENOUGH;
  }

  int append_record(int64_t key, const float* row, Loc& l) {
    if (files_.empty() || !files_.back().out.is_open() || files_.back().bytes + static_cast<int64_t>(rec_bytes_) > kMaxFileBytes ||
        (budget_ > 0 && used_[files_.back().path_idx] + static_cast<int64_t>(rec_bytes_) > budget_)) {
      if (!files_.empty() && budget_ > 0 && used_[files_.back().path_idx] + static_cast<int64_t>(rec_bytes_) > budget_)
        cur_path_ = (files_.back().path_idx + 1) % paths_.size();
      const int rc = open_new_file();
      if (rc != DISK_OK) return rc;
    }
    File& f = files_.back();
    l.file = static_cast<int32_t>(files_.size() - 1);
    l.offset = f.bytes;
    f.out.write(reinterpret_cast<const char*>(&key), sizeof(key));
    f.out.write(reinterpret_cast<const char*>(row), sizeof(float) * rf_);
    if (!f.out) return DISK_ERROR;
    f.bytes += static_cast<int64_t>(rec_bytes_);
    used_[f.path_idx] += static_cast<int64_t>(rec_bytes_);
    return DISK_OK;
  }

  std::string name_;
  std::vector<std::string> paths_;
  int rf_;
  int64_t budget_;
  size_t rec_bytes_;
  mutable std::mutex mu_;
  FlatMap<Loc> loc_;
  mutable std::vector<File> files_;
  std::vector<int64_t> used_;
  size_t cur_path_ = 0;
  int64_t next_file_id_ = 0;
  int64_t stale_ = 0;
};

// Tables + a monitor thread that compacts tables whose stale fraction exceeds the threshold.
class DiskEngine {
 public:
  explicit DiskEngine(double compact_threshold = 0.5, int period_ms = 60000)
      : threshold_(compact_threshold), period_ms_(period_ms) {}
  ~DiskEngine() { stop(); }

  void create_table(const std::string& name, const std::vector<std::string>& paths, int row_floats, int64_t max_bytes_per_path) {
    std::lock_guard<std::mutex> lk(mu_);
    if (tables_.count(name)) throw std::invalid_argument("disk table exists: " + name);
    tables_[name].reset(new DiskTable(name, paths, row_floats, max_bytes_per_path));
  }
  DiskTable& table(const std::string& name) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = tables_.find(name);
    if (it == tables_.end()) throw std::invalid_argument("no such disk table: " + name);
    return *it->second;
  }
  bool has_table(const std::string& name) { std::lock_guard<std::mutex> lk(mu_); return tables_.count(name) > 0; }

  void start() {
    if (running_.exchange(true)) return;
    monitor_ = std::thread([this] {
      while (running_) {
        compact_once();
        std::unique_lock<std::mutex> lk(cv_mu_);
        cv_.wait_for(lk, std::chrono::milliseconds(period_ms_), [this] { return !running_.load(); });
      }
    });
  }
  void stop() {
    if (!running_.exchange(false)) return;
    cv_.notify_all();
    if (monitor_.joinable()) monitor_.join();
  }
  int compact_once() {
    std::vector<DiskTable*> ts;
    { std::lock_guard<std::mutex> lk(mu_); for (auto& kv : tables_) ts.push_back(kv.second.get()); }
    int n = 0;
    for (DiskTable* t : ts)
      if (t->stale_fraction() > threshold_) { t->compact(); ++n; }
    return n;
  }
  void save(int64_t step) { std::lock_guard<std::mutex> lk(mu_); for (auto& kv : tables_) kv.second->save(step); }
  void load(int64_t step) { std::lock_guard<std::mutex> lk(mu_); for (auto& kv : tables_) kv.second->load(step); }

 private:
  double threshold_;
  int period_ms_;
  std::mutex mu_, cv_mu_;
  std::condition_variable cv_;
  std::map<std::string, std::unique_ptr<DiskTable>> tables_;
  std::atomic<bool> running_{false};
  std::thread monitor_;
};

}  // namespace rbh
