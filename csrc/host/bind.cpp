// pybind11 module recsdk_b200._C_host: the host engines exposed to Python over NumPy buffers
// (CPU torch tensors are passed zero-copy through tensor.numpy()).
// Reference counterparts: hybrid_torchrec/src/bind_torch_lib.cpp, torchrec_embcache/csrc/bind.cpp,
// inference/kvcache_manager/src/pybind.cpp.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "disk_tier.h"
#include "embcache.h"
#include "ids_process.h"
#include "kvcache.h"

namespace py = pybind11;
using namespace rbh;

using I64 = py::array_t<int64_t, py::array::c_style | py::array::forcecast>;
using I32 = py::array_t<int32_t, py::array::c_style | py::array::forcecast>;
using F32 = py::array_t<float, py::array::c_style | py::array::forcecast>;
using U8 = py::array_t<uint8_t, py::array::c_style | py::array::forcecast>;

template <typename T>
static py::array_t<T> to_array(const std::vector<T>& v) {
  py::array_t<T> a(static_cast<py::ssize_t>(v.size()));
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(T));
  return a;
}

static py::dict swap_info_to_dict(const SwapInfo& s) {
  py::dict d;
  d["swapout_keys"] = to_array(s.swapout_keys);
  d["swapout_offs"] = to_array(s.swapout_offs);
  d["swapin_keys"] = to_array(s.swapin_keys);
  d["swapin_offs"] = to_array(s.swapin_offs);
  d["batch_offs"] = to_array(s.batch_offs);
  return d;
}

// future handle for asynchronous swap planning
struct SwapInfoFuture {
  std::future<SwapInfo> fut;
  py::dict get() {
    SwapInfo s;
    { py::gil_scoped_release rel; s = fut.get(); }
    return swap_info_to_dict(s);
  }
  bool ready() { return fut.wait_for(std::chrono::seconds(0)) == std::future_status::ready; }
};

// future of a restore running on the shared helper pool; keeps the arrays alive until it finishes
struct RestoreFuture {
  std::future<int64_t> fut;
  I64 unique_indices, unique_inverse, unique_offset;
  py::array_t<int64_t> hash_indices;
  void get() {
    if (!fut.valid()) return;                      // already collected
    int64_t bad;
    { py::gil_scoped_release rel; bad = fut.get(); }
    if (bad >= 0) throw std::out_of_range("restore: index out of range at position " + std::to_string(bad));
  }
  bool ready() { return !fut.valid() || fut.wait_for(std::chrono::seconds(0)) == std::future_status::ready; }
};

static ThreadPool& helper_pool() {
  static ThreadPool pool(2);
  return pool;
}

static void check_restore_args(const I64& ui, const I64& inv, const I64& uo, const std::vector<int64_t>& opt,
                               const py::array_t<int64_t>& out) {
  if (ui.ndim() != 1 || inv.ndim() != 1 || uo.ndim() != 1 || out.ndim() != 1) throw std::invalid_argument("restore: tensors must be 1-D");
  if (out.size() != inv.size()) throw std::invalid_argument("restore: hash_indices length must equal unique_inverse length");
  if (static_cast<size_t>(uo.size()) != opt.size() || opt.empty())
    throw std::invalid_argument("restore: unique_offset length must equal offsets_per_table length");
}

PYBIND11_MODULE(_C_host, m) {
  m.doc() = "recsdk_b200 host engines";

  // file-system layer under the checkpoint writers (file_system.h)
  py::class_<LocalFileSystem>(m, "LocalFileSystem")
      .def(py::init<bool>(), py::arg("strict_owner") = true)
      .def("create_dir", &LocalFileSystem::create_dir)
      .def("exists", &LocalFileSystem::exists)
      .def("list_dir", &LocalFileSystem::list_dir)
      .def("file_size", &LocalFileSystem::file_size)
      .def("remove", &LocalFileSystem::remove)
      .def("write", [](LocalFileSystem& fs, const std::string& path, py::bytes data, bool append) {
        const std::string d = data;
        fs.write(path, d.data(), d.size(), append);
      }, py::arg("path"), py::arg("data"), py::arg("append") = false)
      .def("read", [](LocalFileSystem& fs, const std::string& path, long long bytes, long long offset) {
        const size_t n = bytes < 0 ? fs.file_size(path) - static_cast<size_t>(offset) : static_cast<size_t>(bytes);
        std::string buf(n, '\0');
        const size_t got = fs.read(path, buf.data(), n, static_cast<size_t>(offset));
        buf.resize(got);
        return py::bytes(buf);
      }, py::arg("path"), py::arg("bytes") = -1, py::arg("offset") = 0);
  m.def("validate_path", &validate_path_text);
  m.def("file_system_for", [](const std::string& uri) {
    std::string path;
    make_file_system(uri, &path);
    return path;
  }, "path part of a checkpoint URI; raises for schemes without a registered file system");

  m.def("restore", [](I64 ui, I64 inv, I64 uo, std::vector<int64_t> opt, py::array_t<int64_t, py::array::c_style> out) {
    check_restore_args(ui, inv, uo, opt, out);
    int64_t bad;
    {
      const int64_t* a = ui.data(); const int64_t* b = inv.data(); const int64_t* c = uo.data(); int64_t* o = out.mutable_data();
      const int64_t nu = ui.size(), ni = inv.size(), nt = static_cast<int64_t>(opt.size()) - 1;
      py::gil_scoped_release rel;
      bad = restore_hash_indices(a, nu, b, ni, c, opt.data(), nt, o);
    }
    if (bad >= 0) throw std::out_of_range("restore: index out of range at position " + std::to_string(bad));
  });
  py::class_<RestoreFuture>(m, "RestoreFuture").def("get", &RestoreFuture::get).def("ready", &RestoreFuture::ready);
  m.def("restore_async", [](I64 ui, I64 inv, I64 uo, std::vector<int64_t> opt, py::array_t<int64_t, py::array::c_style> out) {
    check_restore_args(ui, inv, uo, opt, out);
    auto f = std::make_unique<RestoreFuture>();
    f->unique_indices = ui; f->unique_inverse = inv; f->unique_offset = uo; f->hash_indices = out;
    const int64_t* a = ui.data(); const int64_t* b = inv.data(); const int64_t* c = uo.data(); int64_t* o = out.mutable_data();
    const int64_t nu = ui.size(), ni = inv.size(), nt = static_cast<int64_t>(opt.size()) - 1;
    f->fut = helper_pool().submit([=]() { return restore_hash_indices(a, nu, b, ni, c, opt.data(), nt, o); });
    return f;
  });

  // ------------------------------------------------------------------ ids processing
  py::class_<IdsMapper>(m, "IdsMapper")
      .def(py::init<int64_t, size_t>(), py::arg("max_slots"), py::arg("reserve") = 1024)
      .def("size", &IdsMapper::size)
      .def("capacity", &IdsMapper::capacity)
      .def("find", &IdsMapper::find)
      .def("find_or_insert", &IdsMapper::find_or_insert)
      .def("ids2indices", [](IdsMapper& self, I64 ids) {
        py::array_t<int64_t> out(ids.size());
        { py::gil_scoped_release rel; self.ids2indices(ids.data(), ids.size(), out.mutable_data()); }
        return out;
      })
      .def("ids2indices_unique_out", [](IdsMapper& self, I64 ids) {
        const int64_t n = ids.size();
        py::array_t<int64_t> hash_indices(n), unique(n), unique_ids(n), inverse(n);
        int64_t u;
        { py::gil_scoped_release rel;
          u = self.unique_and_lookup(ids.data(), n, hash_indices.mutable_data(), unique.mutable_data(),
                                     unique_ids.mutable_data(), inverse.mutable_data()); }
        unique.resize({u});
        unique_ids.resize({u});
        return py::make_tuple(hash_indices, unique, unique_ids, inverse);
      })
      .def("slot2id", [](const IdsMapper& self) { return to_array(self.slot2id()); })
      .def("load", [](IdsMapper& self, I64 ids) { self.load(ids.data(), ids.size()); });

  // table-parallel fused unique+lookup over several mappers (ENABLE_PARALLEL_GLOBAL_UNIQUE path)
  m.def("parallel_unique_hash_out", [](std::vector<IdsMapper*> mappers, std::vector<I64> ids_per_table) {
    const size_t T = mappers.size();
    std::vector<py::array_t<int64_t>> hi(T), un(T), ui(T), inv(T);
    std::vector<int64_t> counts(T, 0);
    for (size_t t = 0; t < T; ++t) {
      const int64_t n = ids_per_table[t].size();
      hi[t] = py::array_t<int64_t>(n); un[t] = py::array_t<int64_t>(n);
      ui[t] = py::array_t<int64_t>(n); inv[t] = py::array_t<int64_t>(n);
    }
    std::vector<const int64_t*> in(T);
    std::vector<int64_t*> p_hi(T), p_un(T), p_ui(T), p_inv(T);
    std::vector<int64_t> ns(T);
    for (size_t t = 0; t < T; ++t) {
      in[t] = ids_per_table[t].data(); ns[t] = ids_per_table[t].size();
      p_hi[t] = hi[t].mutable_data(); p_un[t] = un[t].mutable_data();
      p_ui[t] = ui[t].mutable_data(); p_inv[t] = inv[t].mutable_data();
    }
    {
      py::gil_scoped_release rel;
#pragma omp parallel for schedule(dynamic, 1)
      for (long t = 0; t < static_cast<long>(T); ++t)
        counts[t] = mappers[t]->unique_and_lookup(in[t], ns[t], p_hi[t], p_un[t], p_ui[t], p_inv[t]);
    }
    py::list out;
    for (size_t t = 0; t < T; ++t) {
      un[t].resize({counts[t]});
      ui[t].resize({counts[t]});
      out.append(py::make_tuple(hi[t], un[t], ui[t], inv[t]));
    }
    return out;
  });

  m.def("unique_parallel", [](I64 in, bool with_counts) {
    const int64_t n = in.size();
    py::array_t<int64_t> uniq(n), inv(n), cnt(with_counts ? n : 0);
    int64_t u;
    { py::gil_scoped_release rel;
      u = unique_parallel(in.data(), n, uniq.mutable_data(), inv.mutable_data(), with_counts ? cnt.mutable_data() : nullptr); }
    uniq.resize({u});
    if (with_counts) cnt.resize({u});
    return py::make_tuple(uniq, inv, cnt);
  }, py::arg("input"), py::arg("with_counts") = false);

  m.def("block_bucketize_sparse_features",
        [](I64 lengths, I64 indices, py::object weights, int64_t F, int64_t B, int64_t world, py::object block_sizes,
           bool local_rows) {
          const int64_t nnz = indices.size();
          py::array_t<int64_t> new_lengths(world * F * B), new_indices(nnz), permute(nnz);
          F32 w;
          py::array_t<float> new_w(0);
          const float* wp = nullptr;
          float* nwp = nullptr;
          if (!weights.is_none()) { w = weights.cast<F32>(); new_w = py::array_t<float>(nnz); wp = w.data(); nwp = new_w.mutable_data(); }
          I64 bs;
          const int64_t* bsp = nullptr;
          if (!block_sizes.is_none()) { bs = block_sizes.cast<I64>(); bsp = bs.data(); }
          { py::gil_scoped_release rel;
            block_bucketize(lengths.data(), indices.data(), wp, F, B, world, bsp, local_rows, new_lengths.mutable_data(),
                            new_indices.mutable_data(), nwp, permute.mutable_data()); }
          return py::make_tuple(new_lengths, new_indices, new_w, permute);
        },
        py::arg("lengths"), py::arg("indices"), py::arg("weights"), py::arg("num_features"), py::arg("batch_size"),
        py::arg("world_size"), py::arg("block_sizes") = py::none(), py::arg("local_rows") = false);

  // ------------------------------------------------------------------ embcache
  py::class_<SwapManager>(m, "SwapManager")
      .def(py::init<int64_t, bool>(), py::arg("cache_size"), py::arg("reserve_slot0") = false)
      .def("compute_swap_info", [](SwapManager& s, I64 keys, int64_t version) {
        return swap_info_to_dict(s.compute_swap_info(keys.data(), keys.size(), version));
      })
      .def("get_key", &SwapManager::get_key)
      .def("offset_of", &SwapManager::offset_of)
      .def("remove_keys", [](SwapManager& s, I64 keys) { s.remove_keys(keys.data(), keys.size()); })
      .def("size", &SwapManager::size)
      .def("capacity", &SwapManager::capacity)
      .def("resident", [](const SwapManager& s) {
        std::vector<int64_t> k, o;
        s.resident(k, o);
        return py::make_tuple(to_array(k), to_array(o));
      });

  py::enum_<InitializerType>(m, "InitializerType")
      .value("LINEAR", InitializerType::LINEAR)
      .value("TRUNCATED_NORMAL", InitializerType::TRUNCATED_NORMAL)
      .value("UNIFORM", InitializerType::UNIFORM)
      .value("CONSTANT", InitializerType::CONSTANT);

  py::class_<InitializerConfig>(m, "InitializerConfig")
      .def(py::init<>())
      .def_readwrite("type", &InitializerConfig::type)
      .def_readwrite("min", &InitializerConfig::min)
      .def_readwrite("max", &InitializerConfig::max)
      .def_readwrite("mean", &InitializerConfig::mean)
      .def_readwrite("stddev", &InitializerConfig::stddev)
      .def_readwrite("value", &InitializerConfig::value)
      .def_readwrite("seed", &InitializerConfig::seed);

  py::class_<AdmitEvictConfig>(m, "AdmitEvictConfig")
      .def(py::init<>())
      .def_readwrite("admit_threshold", &AdmitEvictConfig::admit_threshold)
      .def_readwrite("evict_threshold", &AdmitEvictConfig::evict_threshold)
      .def_readwrite("policy", &AdmitEvictConfig::policy)
      .def_readwrite("alpha", &AdmitEvictConfig::alpha)
      .def_readwrite("beta", &AdmitEvictConfig::beta)
      .def_readwrite("sc_admit_threshold", &AdmitEvictConfig::sc_admit_threshold)
      .def_readwrite("evict_percentage", &AdmitEvictConfig::evict_percentage)
      .def_readwrite("score_decay", &AdmitEvictConfig::score_decay)
      .def("admit_enabled", &AdmitEvictConfig::admit_enabled)
      .def("evict_enabled", &AdmitEvictConfig::evict_enabled);

  py::class_<EmbConfig>(m, "EmbConfig")
      .def(py::init<>())
      .def_readwrite("table_name", &EmbConfig::table_name)
      .def_readwrite("emb_dim", &EmbConfig::emb_dim)
      .def_readwrite("optim_num", &EmbConfig::optim_num)
      .def_readwrite("cache_size", &EmbConfig::cache_size)
      .def_readwrite("init", &EmbConfig::init)
      .def_readwrite("admit_evict", &EmbConfig::admit_evict)
      .def_readwrite("is_incremental", &EmbConfig::is_incremental);

  py::class_<FeatureFilter>(m, "FeatureFilter")
      .def(py::init<const AdmitEvictConfig&>())
      .def("statistics_key_count", [](FeatureFilter& f, I64 keys, py::object counts, py::object clicks) {
        I64 c, k2;
        const int64_t *cp = nullptr, *kp = nullptr;
        if (!counts.is_none()) { c = counts.cast<I64>(); cp = c.data(); }
        if (!clicks.is_none()) { k2 = clicks.cast<I64>(); kp = k2.data(); }
        f.statistics_key_count(keys.data(), keys.size(), cp, kp);
      }, py::arg("keys"), py::arg("counts") = py::none(), py::arg("clicks") = py::none())
      .def("filter", [](FeatureFilter& f, I64 keys) {
        py::array_t<int64_t> out(keys.size());
        std::memcpy(out.mutable_data(), keys.data(), sizeof(int64_t) * keys.size());
        f.filter(out.mutable_data(), out.size());
        return out;
      })
      .def("record_timestamp", [](FeatureFilter& f, I64 keys, I64 ts) { f.record_timestamp(keys.data(), keys.size(), ts.data()); })
      .def("evict", [](FeatureFilter& f) { return to_array(f.evict()); })
      .def("size", &FeatureFilter::size);

  py::class_<HostEmbTable>(m, "HostEmbTable")
      .def(py::init<int, int, const InitializerConfig&>())
      .def("size", &HostEmbTable::size)
      .def("row_floats", &HostEmbTable::row_floats)
      .def("find_or_insert", [](HostEmbTable& t, I64 keys) {
        py::array_t<float> rows({static_cast<py::ssize_t>(keys.size()), static_cast<py::ssize_t>(t.row_floats())});
        { py::gil_scoped_release rel; t.find_or_insert(keys.data(), keys.size(), rows.mutable_data()); }
        return rows;
      })
      .def("find", [](HostEmbTable& t, I64 keys) {
        py::array_t<float> rows({static_cast<py::ssize_t>(keys.size()), static_cast<py::ssize_t>(t.row_floats())});
        py::array_t<uint8_t> found(keys.size());
        { py::gil_scoped_release rel; t.find(keys.data(), keys.size(), rows.mutable_data(), found.mutable_data()); }
        return py::make_tuple(rows, found);
      })
      .def("insert_or_assign", [](HostEmbTable& t, I64 keys, F32 rows) {
        if (rows.size() != keys.size() * t.row_floats()) throw std::invalid_argument("rows shape mismatch");
        py::gil_scoped_release rel;
        t.insert_or_assign(keys.data(), keys.size(), rows.data());
      })
      .def("erase", [](HostEmbTable& t, I64 keys) { t.erase(keys.data(), keys.size()); })
      .def("export_all", [](HostEmbTable& t) {
        std::vector<int64_t> k;
        std::vector<float> r;
        t.export_all(k, r);
        py::array_t<float> rows({static_cast<py::ssize_t>(k.size()), static_cast<py::ssize_t>(t.row_floats())});
        if (!r.empty()) std::memcpy(rows.mutable_data(), r.data(), r.size() * sizeof(float));
        return py::make_tuple(to_array(k), rows);
      });

  py::class_<SwapInfoFuture>(m, "SwapInfoFuture").def("get", &SwapInfoFuture::get).def("ready", &SwapInfoFuture::ready);

  py::class_<EmbcacheManager>(m, "EmbcacheManager")
      .def(py::init<const std::vector<EmbConfig>&, int>(), py::arg("emb_configs"), py::arg("threads") = 4)
      .def("num_tables", &EmbcacheManager::num_tables)
      .def("compute_swap_info", [](EmbcacheManager& mg, size_t t, I64 keys, int64_t step) {
        std::vector<int64_t> k(keys.data(), keys.data() + keys.size());
        SwapInfo s;
        { py::gil_scoped_release rel; s = mg.compute_swap_info(t, std::move(k), step); }
        return swap_info_to_dict(s);
      })
      .def("compute_swap_info_async", [](EmbcacheManager& mg, size_t t, I64 keys, int64_t step) {
        std::vector<int64_t> k(keys.data(), keys.data() + keys.size());
        auto f = new SwapInfoFuture{mg.compute_swap_info_async(t, std::move(k), step)};
        return std::unique_ptr<SwapInfoFuture>(f);
      })
      .def("plan_batch_async", [](EmbcacheManager& mg, size_t t, I64 keys, int64_t step, bool count_stats, bool stamp, int64_t now) {
        std::vector<int64_t> k(keys.data(), keys.data() + keys.size());
        auto f = new SwapInfoFuture{mg.plan_batch_async(t, std::move(k), step, count_stats, stamp, now)};
        return std::unique_ptr<SwapInfoFuture>(f);
      })
      // rows of `keys` written into caller memory (a pinned staging buffer): dst = address of [len(keys), row_floats] floats
      .def("embedding_lookup_into", [](EmbcacheManager& mg, size_t t, I64 keys, uintptr_t dst, int64_t capacity_rows) {
        if (keys.size() > capacity_rows) throw std::invalid_argument("staging buffer too small for this swap-in");
        py::gil_scoped_release rel;
        mg.embedding_lookup(t, keys.data(), keys.size(), reinterpret_cast<float*>(dst));
      })
      // host InsertOrAssign straight from caller memory (the pinned buffer a device-to-host copy filled)
      .def("embedding_update_from", [](EmbcacheManager& mg, size_t t, I64 keys, uintptr_t src) {
        py::gil_scoped_release rel;
        mg.embedding_update(t, keys.data(), keys.size(), reinterpret_cast<const float*>(src));
      })
      .def("embedding_lookup", [](EmbcacheManager& mg, size_t t, I64 keys) {
        const int rf = mg.host_table(t).row_floats();
        py::array_t<float> rows({static_cast<py::ssize_t>(keys.size()), static_cast<py::ssize_t>(rf)});
        { py::gil_scoped_release rel; mg.embedding_lookup(t, keys.data(), keys.size(), rows.mutable_data()); }
        return rows;
      })
      .def("embedding_update", [](EmbcacheManager& mg, size_t t, I64 keys, F32 rows) {
        if (rows.size() != keys.size() * mg.host_table(t).row_floats()) throw std::invalid_argument("rows shape mismatch");
        py::gil_scoped_release rel;
        mg.embedding_update(t, keys.data(), keys.size(), rows.data());
      })
      .def("statistics_key_count", [](EmbcacheManager& mg, size_t t, I64 keys, py::object counts, py::object clicks) {
        I64 c, k2;
        const int64_t *cp = nullptr, *kp = nullptr;
        if (!counts.is_none()) { c = counts.cast<I64>(); cp = c.data(); }
        if (!clicks.is_none()) { k2 = clicks.cast<I64>(); kp = k2.data(); }
        mg.statistics_key_count(t, keys.data(), keys.size(), cp, kp);
      }, py::arg("table"), py::arg("keys"), py::arg("counts") = py::none(), py::arg("clicks") = py::none())
      .def("record_timestamp", [](EmbcacheManager& mg, size_t t, I64 keys, I64 ts) { mg.record_timestamp(t, keys.data(), keys.size(), ts.data()); })
      .def("evict_features", [](EmbcacheManager& mg, size_t t) { return to_array(mg.evict_features(t)); })
      .def("resident", [](EmbcacheManager& mg, size_t t) {
        std::vector<int64_t> k, o;
        mg.swap_manager(t).resident(k, o);
        return py::make_tuple(to_array(k), to_array(o));
      })
      .def("get_key", [](EmbcacheManager& mg, size_t t, int64_t off, int64_t version) { return mg.swap_manager(t).get_key(off, version); })
      .def("host_size", [](EmbcacheManager& mg, size_t t) { return mg.host_table(t).size(); })
      .def("invalidate_cache", &EmbcacheManager::invalidate_cache)
      .def("cache_capacity", [](EmbcacheManager& mg, size_t t) { return mg.swap_manager(t).capacity(); })
      .def("cache_size", [](EmbcacheManager& mg, size_t t) { return mg.swap_manager(t).size(); })
      .def("host_export", [](EmbcacheManager& mg, size_t t) {
        std::vector<int64_t> k;
        std::vector<float> r;
        mg.host_table(t).export_all(k, r);
        const int rf = mg.host_table(t).row_floats();
        py::array_t<float> rows({static_cast<py::ssize_t>(k.size()), static_cast<py::ssize_t>(rf)});
        if (!r.empty()) std::memcpy(rows.mutable_data(), r.data(), r.size() * sizeof(float));
        return py::make_tuple(to_array(k), rows);
      })
      .def("save", [](EmbcacheManager& mg, const std::string& p, int rank, bool inc) { py::gil_scoped_release rel; mg.save(p, rank, inc); })
      .def("merge_files", [](EmbcacheManager& mg, const std::string& p, int world) { py::gil_scoped_release rel; mg.merge_files(p, world); })
      .def("load", [](EmbcacheManager& mg, const std::string& p, int rank, int world, bool incremental) {
        py::gil_scoped_release rel;
        mg.load(p, rank, world, incremental);
      }, py::arg("path"), py::arg("rank"), py::arg("world"), py::arg("incremental") = false);

  // ------------------------------------------------------------------ kv cache
  py::class_<KVPageAllocator>(m, "KVPageAllocator")
      .def(py::init<int, int, int, int, int, int>(), py::arg("page_size"), py::arg("chunk_size"), py::arg("num_primary_pages"),
           py::arg("num_buffer_pages"), py::arg("max_batch_size"), py::arg("max_seq_len"))
      .def("free_pages", &KVPageAllocator::free_pages)
      .def("num_users", &KVPageAllocator::num_users)
      .def("total_offloaded_pages", &KVPageAllocator::total_offloaded_pages)
      .def("lookup", [](const KVPageAllocator& a, I64 uids) {
        py::array_t<int32_t> s(uids.size()), l(uids.size());
        a.lookup(uids.data(), static_cast<int>(uids.size()), s.mutable_data(), l.mutable_data());
        return py::make_tuple(s, l);
      })
      .def("allocate", [](KVPageAllocator& a, I64 uids, I32 total, I32 host_cached) {
        KVAllocResult r = a.allocate(uids.data(), total.data(), host_cached.data(), static_cast<int>(uids.size()));
        return py::make_tuple(to_array(r.page_indices), to_array(r.metadata), r.new_tokens);
      })
      .def("alloc_single_sequence", [](KVPageAllocator& a, int64_t uid, int total, int host_cached, std::vector<int64_t> frozen) {
        return to_array(a.alloc_single_sequence(uid, total, host_cached, std::unordered_set<int64_t>(frozen.begin(), frozen.end())));
      })
      .def("check_for_offload", [](const KVPageAllocator& a, I64 uids, int max_pages) {
        return to_array(a.check_for_offload(uids.data(), static_cast<int>(uids.size()), max_pages));
      })
      .def("acquire_offload_pages", [](KVPageAllocator& a, I64 uids, py::object offloaded, bool always) {
        I32 o;
        const int32_t* op = nullptr;
        if (!offloaded.is_none()) { o = offloaded.cast<I32>(); if (o.size() == uids.size()) op = o.data(); }
        auto plan = a.acquire_offload_pages(uids.data(), static_cast<int>(uids.size()), op, always);
        py::list pages;
        for (auto& p : plan.pages) pages.append(to_array(p));
        return py::make_tuple(to_array(plan.uids), to_array(plan.start), pages);
      }, py::arg("uids"), py::arg("offloaded_lengths") = py::none(), py::arg("always_offload") = false)
      .def("release_offload_pages", [](KVPageAllocator& a, I64 uids, I32 start, I32 length, U8 done) {
        a.release_offload_pages(uids.data(), start.data(), length.data(), done.data(), static_cast<int>(uids.size()));
      })
      .def("revoke_onboard_pages", [](KVPageAllocator& a, I64 uids, I32 start, I32 length) {
        a.revoke_onboard_pages(uids.data(), start.data(), length.data(), static_cast<int>(uids.size()));
      })
      .def("pages_of", [](const KVPageAllocator& a, int64_t uid) { return to_array(a.pages_of(uid)); })
      .def("evict", &KVPageAllocator::evict)
      .def("truncate", &KVPageAllocator::truncate)
      .def("evict_offloaded", &KVPageAllocator::evict_offloaded)
      .def("evict_all", &KVPageAllocator::evict_all);

  py::class_<HostChunkIndex>(m, "HostChunkIndex")
      .def(py::init<int64_t, int>(), py::arg("num_chunks"), py::arg("chunk_tokens"))
      .def("free_chunks", &HostChunkIndex::free_chunks)
      .def("num_users", &HostChunkIndex::num_users)
      .def("lookup", [](HostChunkIndex& h, I64 uids) {
        py::array_t<int32_t> s(uids.size()), l(uids.size());
        h.lookup(uids.data(), static_cast<int>(uids.size()), s.mutable_data(), l.mutable_data());
        return py::make_tuple(s, l);
      })
      .def("chunks_of", [](const HostChunkIndex& h, int64_t uid, int first, int n) { return to_array(h.chunks_of(uid, first, n)); })
      .def("append", [](HostChunkIndex& h, int64_t uid, int start, int n, std::vector<int64_t> pinned) {
        return to_array(h.append(uid, start, n, std::unordered_set<int64_t>(pinned.begin(), pinned.end())));
      }, py::arg("uid"), py::arg("start_token"), py::arg("n_tokens"), py::arg("pinned") = std::vector<int64_t>())
      .def("rollback", &HostChunkIndex::rollback)
      .def("evict", &HostChunkIndex::evict)
      .def("evict_all", &HostChunkIndex::evict_all);

  // ------------------------------------------------------------------ disk tier
  py::class_<DiskEngine>(m, "DiskEngine")
      .def(py::init<double, int>(), py::arg("compact_threshold") = 0.5, py::arg("period_ms") = 60000)
      .def("create_table", &DiskEngine::create_table, py::arg("name"), py::arg("paths"), py::arg("row_floats"),
           py::arg("max_bytes_per_path") = 0)
      .def("has_table", &DiskEngine::has_table)
      .def("insert", [](DiskEngine& e, const std::string& name, I64 keys, F32 rows) {
        py::gil_scoped_release rel;
        return e.table(name).insert(keys.data(), keys.size(), rows.data());
      })
      .def("fetch", [](DiskEngine& e, const std::string& name, I64 keys, int row_floats) {
        py::array_t<float> rows({static_cast<py::ssize_t>(keys.size()), static_cast<py::ssize_t>(row_floats)});
        py::array_t<uint8_t> found(keys.size());
        std::memset(rows.mutable_data(), 0, sizeof(float) * rows.size());
        int rc;
        { py::gil_scoped_release rel; rc = e.table(name).fetch(keys.data(), keys.size(), rows.mutable_data(), found.mutable_data()); }
        return py::make_tuple(rc, rows, found);
      })
      .def("erase", [](DiskEngine& e, const std::string& name, I64 keys) { e.table(name).erase(keys.data(), keys.size()); })
      .def("size", [](DiskEngine& e, const std::string& name) { return e.table(name).size(); })
      .def("stale", [](DiskEngine& e, const std::string& name) { return e.table(name).stale(); })
      .def("bytes_used", [](DiskEngine& e, const std::string& name) { return e.table(name).bytes_used(); })
      .def("export_keys", [](DiskEngine& e, const std::string& name) { return to_array(e.table(name).export_keys()); })
      .def("compact", [](DiskEngine& e, const std::string& name) { return e.table(name).compact(); })
      .def("compact_once", &DiskEngine::compact_once)
      .def("start", &DiskEngine::start)
      .def("stop", &DiskEngine::stop)
      .def("save", &DiskEngine::save)
      .def("load", &DiskEngine::load);

  m.attr("DISK_OK") = static_cast<int>(DISK_OK);
  m.attr("DISK_ERROR") = static_cast<int>(DISK_ERROR);
  m.attr("DISK_SPACE_NOT_ENOUGH") = static_cast<int>(DISK_SPACE_NOT_ENOUGH);
}
