// Concurrency / memory-safety driver for the host engines, built with -fsanitize=thread or
// -fsanitize=address,undefined by tests/test_host_sanitizers.py (no Python, no OpenMP runtime: plain std::thread, so the
// sanitizers see every synchronisation).  Several threads hammer one HostEmbTable (find_or_insert / find /
// insert_or_assign / erase / export_all on overlapping key ranges), one EmbMemoryPool and one flat map guarded the way
// the engines guard theirs; the driver then checks the invariants that must hold whatever the interleaving.
// The reference ships no sanitizer run for its host engines (training/torch_rec_v1/torchrec_embcache/src/.../csrc).
#include <atomic>
#include <cstdio>
#include <thread>
#include <vector>

#include "../embcache.h"
#include "../ids_process.h"

using namespace rbh;

static int fail(const char* what) {
  std::fprintf(stderr, "host_stress: FAILED: %s\n", what);
  return 1;
}

int main() {
  const int kThreads = 8, kRounds = 40, kKeys = 512, dim = 8;
  InitializerConfig ic;
  ic.type = InitializerType::UNIFORM;
  ic.seed = 7;
  HostEmbTable table(dim, 1, ic);
  const int rf = table.row_floats();
  std::atomic<int> bad{0};
  std::vector<std::thread> th;
  for (int t = 0; t < kThreads; ++t) {
    th.emplace_back([&, t] {
      std::vector<int64_t> keys(kKeys);
      std::vector<float> rows(static_cast<size_t>(kKeys) * rf);
      std::vector<uint8_t> found(kKeys);
      for (int r = 0; r < kRounds; ++r) {
        for (int i = 0; i < kKeys; ++i) keys[i] = (static_cast<int64_t>(i) * 37 + t * 11 + r * 5) % 2000;   // overlapping
        table.find_or_insert(keys.data(), kKeys, rows.data());
        // a freshly initialised or previously assigned row: embedding within the initializer's range or the marker 3.0
        for (int i = 0; i < kKeys; ++i) {
          const float v = rows[static_cast<size_t>(i) * rf];
          if (!((v >= -0.05f && v <= 0.05f) || v == 3.0f)) bad.fetch_add(1);
        }
        if ((r + t) % 3 == 0) {
          for (auto& x : rows) x = 3.0f;
          table.insert_or_assign(keys.data(), kKeys / 4, rows.data());
        }
        if ((r + t) % 5 == 0) table.erase(keys.data() + kKeys / 2, kKeys / 8);
        table.find(keys.data(), kKeys, rows.data(), found.data());
        if ((r + t) % 7 == 0) {
          std::vector<int64_t> ek;
          std::vector<float> er;
          table.export_all(ek, er);
          if (er.size() != ek.size() * static_cast<size_t>(rf)) bad.fetch_add(1);
        }
      }
    });
  }
  for (auto& x : th) x.join();
  if (bad.load()) return fail("a row held values that no writer stored");
  if (table.size() <= 0 || table.size() > 2000) return fail("table size outside the key range");

  // same key -> same initial row, whichever thread inserts it first (counter-based initializer)
  HostEmbTable a(dim, 0, ic), b(dim, 0, ic);
  std::vector<int64_t> ks(1000);
  for (int i = 0; i < 1000; ++i) ks[i] = i * 3 + 1;
  std::vector<float> ra(1000 * dim), rb(1000 * dim);
  std::thread t1([&] { a.find_or_insert(ks.data(), 1000, ra.data()); });
  std::vector<int64_t> rev(ks.rbegin(), ks.rend());
  std::vector<float> rrev(1000 * dim);
  std::thread t2([&] { b.find_or_insert(rev.data(), 1000, rrev.data()); });
  t1.join();
  t2.join();
  b.find_or_insert(ks.data(), 1000, rb.data());
  if (ra != rb) return fail("initial rows depend on the insertion order");

  // one id mapper shared by several threads (insertions are serialised inside)
  IdsMapper mapper(1 << 12);
  std::vector<std::thread> tm;
  std::atomic<int> bad2{0};
  for (int t = 0; t < 4; ++t) {
    tm.emplace_back([&, t] {
      std::vector<int64_t> ids(3000), out(3000);
      for (int i = 0; i < 3000; ++i) ids[i] = (i * 7 + t) % 900 + 100000;
      mapper.ids2indices(ids.data(), 3000, out.data());
      for (int i = 0; i < 3000; ++i)
        if (out[i] < 0 || out[i] >= 900) bad2.fetch_add(1);
    });
  }
  for (auto& x : tm) x.join();
  if (bad2.load() || mapper.size() != 900) return fail("id mapper produced an index outside [0, distinct ids)");
  std::printf("host_stress: ok (table size %lld)\n", static_cast<long long>(table.size()));
  return 0;
}
