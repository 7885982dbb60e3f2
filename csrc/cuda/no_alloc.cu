// Implementation of rb_sort_segments_noalloc: see no_alloc.h for who needs it and the rules of use.
#include <cub/cub.cuh>

#include <mutex>

#include "common.cuh"
#include "no_alloc.h"

namespace {

// The only scratch this entry point ever uses.  In host code this name is just a handle for the
// runtime, not an address a kernel could use: the device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[RB_NOALLOC_SCRATCH_BYTES];

constexpr size_t COUNTS_BYTES = (static_cast<size_t>(RB_NOALLOC_MAX_KEYS) + 1) * sizeof(int);
constexpr size_t COUNTS_OFFSET = 0;
constexpr size_t TEMP_OFFSET = (COUNTS_BYTES + 255) / 256 * 256;
constexpr size_t TEMP_BYTES = RB_NOALLOC_SCRATCH_BYTES - TEMP_OFFSET;

constexpr int MAX_DEVICES = RB_NOALLOC_MAX_DEVICES;
std::mutex g_mu;
unsigned char* g_scratch_ptr[MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the current device (resolved on first use per device).
int scratch_for_current_device(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= MAX_DEVICES) return RB_NOALLOC_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" int rb_sort_segments_noalloc(const long long* keys_in, const int* vals_in, long long n, int end_bit,
                                        long long* keys_out, int* vals_out, long long* unique_out,
                                        int* seg_offsets, int* num_runs, cudaStream_t stream) {
  if (n < 0 || end_bit < 1 || end_bit > 64 || !num_runs || !seg_offsets) return RB_NOALLOC_ERR_BAD_ARG;
  if (n > RB_NOALLOC_MAX_KEYS) return RB_NOALLOC_ERR_TOO_LARGE;
  if (n > 0 && (!keys_in || !vals_in || !keys_out || !vals_out || !unique_out)) return RB_NOALLOC_ERR_BAD_ARG;
  unsigned char* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  if (n == 0) {
    RB_CUDA_CHECK(cudaMemsetAsync(num_runs, 0, sizeof(int), stream));
    return static_cast<int>(cudaMemsetAsync(seg_offsets, 0, sizeof(int), stream));
  }
  int* counts = reinterpret_cast<int*>(scratch + COUNTS_OFFSET);
  void* temp = scratch + TEMP_OFFSET;
  const int ni = static_cast<int>(n);

  // every stage must fit the static workspace (size queries run on the host, no allocation)
  size_t need_sort = 0, need_rle = 0, need_scan = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, need_sort, keys_in, keys_out, vals_in, vals_out, ni, 0, end_bit, stream);
  cub::DeviceRunLengthEncode::Encode(nullptr, need_rle, keys_out, unique_out, counts, num_runs, ni, stream);
  cub::DeviceScan::ExclusiveSum(nullptr, need_scan, counts, seg_offsets, ni + 1, stream);
  if (need_sort > TEMP_BYTES || need_rle > TEMP_BYTES || need_scan > TEMP_BYTES) return RB_NOALLOC_ERR_SCRATCH;

  size_t tb = TEMP_BYTES;
  RB_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(temp, tb, keys_in, keys_out, vals_in, vals_out, ni, 0, end_bit, stream));
  // run lengths beyond the last run must read as zero for the scan: the previous call's counts are
  // still in the shared scratch, so clear them here
  RB_CUDA_CHECK(cudaMemsetAsync(counts, 0, sizeof(int) * (static_cast<size_t>(n) + 1), stream));
  tb = TEMP_BYTES;
  RB_CUDA_CHECK(cub::DeviceRunLengthEncode::Encode(temp, tb, keys_out, unique_out, counts, num_runs, ni, stream));
  tb = TEMP_BYTES;
  RB_CUDA_CHECK(cub::DeviceScan::ExclusiveSum(temp, tb, counts, seg_offsets, ni + 1, stream));
  return 0;
}
