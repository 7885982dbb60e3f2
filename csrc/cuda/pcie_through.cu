// Row swap between device tables and host memory that the GPU addresses directly ("PCIe-through"), and the host side
// that provides such memory: POSIX shared-memory segments mapped into the process and registered with CUDA so that a
// kernel reads / writes them through the unified address space (another process - a data loader, a parameter server
// shim - attaches to the same segment by name).
//
//   rb_shm_open / rb_shm_close      create or attach a named segment, optionally registered (mapped + portable)
//   rb_swap_multi_tables            for up to 8 tables in one call: rows listed in `out_idx` are copied device -> host,
//                                   then rows listed in `in_idx` are copied host -> device (16-byte vectors; no staging
//                                   copy, no copy-engine launch per table)
//
// Role in the reference: training/common/src/core/pcie_through/rma_shm_svm.{h,cpp} (shared-memory / SVM mapping) and the
// `RmaSwapMultiTables` operator (cust_op/ai_core_op/pcie_through: swap_in_index, swap_out_index, table_a..table_f,
// shm_swap_in, shm_swap_out).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <new>
#include <string>

#include "common.cuh"

namespace {

constexpr int SWAP_MAX_TABLES = 8;

struct ShmSegment {
  std::string name;
  void* ptr = nullptr;
  size_t bytes = 0;
  int fd = -1;
  bool registered = false;
  bool owner = false;
};

struct SwapArgs {
  char* table[SWAP_MAX_TABLES];
  const long long* idx[SWAP_MAX_TABLES];
  char* host[SWAP_MAX_TABLES];
  long long n[SWAP_MAX_TABLES];
  long long rows[SWAP_MAX_TABLES];       // rows of the table (bounds check)
  int vec_per_row[SWAP_MAX_TABLES];      // row bytes / 16
  long long vec_prefix[SWAP_MAX_TABLES + 1];
  int n_tables;
  int to_host;                           // 1: host[i] = table[idx[i]], 0: table[idx[i]] = host[i]
  int* status;
};

__global__ void __launch_bounds__(256) swap_rows_kernel(const SwapArgs a) {
  const long long total = a.vec_prefix[a.n_tables];
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < total;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    int t = 0;
    while (t + 1 < a.n_tables && v >= a.vec_prefix[t + 1]) ++t;
    const long long lv = v - a.vec_prefix[t];
    const long long i = lv / a.vec_per_row[t];
    const long long c = lv - i * a.vec_per_row[t];
    const long long r = a.idx[t][i];
    if (r < 0) continue;                                    // -1 = empty entry
    if (r >= a.rows[t]) {
      if (a.status) atomicCAS(a.status, 0, RB_ERR_BOUNDS);
      continue;
    }
    uint4* dev = reinterpret_cast<uint4*>(a.table[t]) + r * a.vec_per_row[t] + c;
    uint4* hst = reinterpret_cast<uint4*>(a.host[t]) + i * a.vec_per_row[t] + c;
    if (a.to_host) *hst = *dev;
    else *dev = *hst;
  }
}

}  // namespace

// create != 0: create (or truncate) the segment `name` with `bytes`; else attach to an existing one (bytes = its size,
// or 0 to take the size from the segment).  register_cuda != 0: page-lock and map it for the current device.
RB_API int rb_shm_open(const char* name, long long bytes, int create, int register_cuda, void** handle, void** host_ptr,
                       long long* bytes_out) {
  if (!name || !handle || !host_ptr || name[0] != '/' || std::strchr(name + 1, '/') != nullptr) return -1;
  const int fd = ::shm_open(name, create ? (O_CREAT | O_RDWR) : O_RDWR, 0600);
  if (fd < 0) return -2;
  if (create) {
    if (bytes <= 0 || ::ftruncate(fd, static_cast<off_t>(bytes)) != 0) { ::close(fd); ::shm_unlink(name); return -3; }
  } else {
    struct stat st;
    if (::fstat(fd, &st) != 0 || st.st_size <= 0 || (bytes > 0 && st.st_size < bytes)) { ::close(fd); return -4; }
    if (bytes <= 0) bytes = static_cast<long long>(st.st_size);
  }
  void* p = ::mmap(nullptr, static_cast<size_t>(bytes), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) { ::close(fd); if (create) ::shm_unlink(name); return -5; }
  ShmSegment* s = new (std::nothrow) ShmSegment();
  if (!s) { ::munmap(p, static_cast<size_t>(bytes)); ::close(fd); return -6; }
  s->name = name; s->ptr = p; s->bytes = static_cast<size_t>(bytes); s->fd = fd; s->owner = create != 0;
  if (register_cuda) {
    const cudaError_t e = cudaHostRegister(p, s->bytes, cudaHostRegisterPortable | cudaHostRegisterMapped);
    if (e != cudaSuccess) {
      ::munmap(p, s->bytes); ::close(fd); if (create) ::shm_unlink(name);
      delete s;
      return static_cast<int>(e);
    }
    s->registered = true;
  }
  *handle = s; *host_ptr = p;
  if (bytes_out) *bytes_out = bytes;
  return 0;
}

// unlink != 0 also removes the name (the creator does this once every user has attached or is done)
RB_API int rb_shm_close(void* handle, int unlink) {
  ShmSegment* s = static_cast<ShmSegment*>(handle);
  if (!s) return 0;
  int rc = 0;
  if (s->registered) rc = static_cast<int>(cudaHostUnregister(s->ptr));
  ::munmap(s->ptr, s->bytes);
  ::close(s->fd);
  if (unlink) ::shm_unlink(s->name.c_str());
  delete s;
  return rc;
}

// tables / host_out / host_in: host arrays of n_tables addresses (device tables; host buffers the device can address);
// out_idx / in_idx: host arrays of n_tables device pointers to int64 row lists (-1 entries are skipped) with n_out /
// n_in entries each; row_bytes (multiples of 16) and table_rows per table.  Swap-out runs before swap-in, so a slot may
// be listed in both: its old row goes to the host, the new one takes its place.
RB_API int rb_swap_multi_tables(const unsigned long long* tables, const long long* table_rows, const long long* row_bytes,
                                int n_tables, const unsigned long long* out_idx, const long long* n_out,
                                const unsigned long long* host_out, const unsigned long long* in_idx, const long long* n_in,
                                const unsigned long long* host_in, int num_sms, int* status, cudaStream_t st) {
  if (n_tables <= 0 || n_tables > SWAP_MAX_TABLES) return -1;
  for (int dir = 0; dir < 2; ++dir) {
    const unsigned long long* idx = dir == 0 ? out_idx : in_idx;
    const long long* n = dir == 0 ? n_out : n_in;
    const unsigned long long* host = dir == 0 ? host_out : host_in;
    if (!idx || !n || !host) continue;
    SwapArgs a;
    a.n_tables = n_tables; a.to_host = dir == 0 ? 1 : 0; a.status = status;
    long long total = 0;
    for (int t = 0; t < n_tables; ++t) {
      if (row_bytes[t] <= 0 || (row_bytes[t] % 16) || n[t] < 0) return -2;
      a.table[t] = reinterpret_cast<char*>(tables[t]);
      a.idx[t] = reinterpret_cast<const long long*>(idx[t]);
      a.host[t] = reinterpret_cast<char*>(host[t]);
      a.n[t] = n[t]; a.rows[t] = table_rows[t];
      a.vec_per_row[t] = static_cast<int>(row_bytes[t] / 16);
      a.vec_prefix[t] = total;
      total += n[t] * a.vec_per_row[t];
      if (n[t] > 0 && (!a.idx[t] || !a.host[t] || !a.table[t])) return -3;
    }
    for (int t = n_tables; t <= SWAP_MAX_TABLES; ++t) a.vec_prefix[t] = total;
    if (total == 0) continue;
    long long blocks = (total + 255) / 256;
    const long long cap = static_cast<long long>(num_sms > 0 ? num_sms : 148) * 8;
    if (blocks > cap) blocks = cap;
    swap_rows_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(a);
    RB_CUDA_CHECK(cudaGetLastError());
  }
  return 0;
}
