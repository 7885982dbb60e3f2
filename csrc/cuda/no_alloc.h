// Allocation-free variant of the id de-duplication step (sort + run-length encode).
//
// This entry point has no counterpart in the reference SDK.  It exists for callers that must not
// (or cannot) allocate device memory at the moment they need to de-duplicate a batch of ids:
//
//   * a serving process whose memory pool has already claimed the whole GPU (KV-cache pages,
//     embedding caches), so a late cudaMalloc for sort workspace would simply fail;
//   * a latency-critical request thread for which the device-wide synchronisation and the driver
//     lock taken by cudaMalloc / cudaFree are not acceptable;
//   * plain C / C++ hosts that link this library without PyTorch and therefore have no caching
//     allocator to borrow workspace from.
//
// What the regular entry point (rb_sort_segments) takes from the caller as `temp` and `counts`
// lives here in ONE file-scope device array of RB_NOALLOC_SCRATCH_BYTES (8 MiB) that every GPU
// loading the library holds until the process exits.  The caller still provides all inputs and
// outputs.  Nothing in this call allocates or frees memory, on the host or on the device.
//
// Limits and rules
//   * n <= RB_NOALLOC_MAX_KEYS (262,144).  Larger n returns RB_NOALLOC_ERR_TOO_LARGE and does nothing.
//   * The first call on a device resolves the scratch array's device address
//     (cudaGetSymbolAddress with that device current).  Make that first call before starting any
//     stream capture on that device; later calls only enqueue work on `stream`.
//   * All calls on one device share the scratch array, and it keeps whatever the previous call left
//     in it.  The call clears the part that must start at zero itself.  Two calls whose GPU work can
//     overlap (different streams without an ordering between them, or several host threads) race on
//     the scratch and give wrong results: order them on one stream or with events.
#pragma once
#include <cuda_runtime.h>

#define RB_NOALLOC_MAX_KEYS (1 << 18)
#define RB_NOALLOC_SCRATCH_BYTES (8u << 20)
#define RB_NOALLOC_ERR_TOO_LARGE (-20)   /* n exceeds RB_NOALLOC_MAX_KEYS */
#define RB_NOALLOC_ERR_SCRATCH (-21)     /* the sort needs more workspace than the static array holds */
#define RB_NOALLOC_ERR_BAD_ARG (-22)     /* null pointer / negative n / bad end_bit */
#define RB_NOALLOC_ERR_DEVICE (-23)      /* the current device's ordinal is RB_NOALLOC_MAX_DEVICES or more */
#define RB_NOALLOC_MAX_DEVICES 64        /* device ordinals served (one resolved scratch address each) */

#ifdef __cplusplus
extern "C" {
#endif

// keys_in/vals_in [n] -> keys_out/vals_out [n] sorted by the low `end_bit` key bits (stable),
// unique_out [<= n] distinct keys in sorted order, seg_offsets [n + 1] with seg_offsets[i] the start of
// run i and seg_offsets[num_runs] = n (entries past num_runs also hold n), num_runs [1].
// All pointers are device pointers owned by the caller.  Returns 0, a cudaError_t (> 0) or one of the
// RB_NOALLOC_ERR_* codes (< 0).  For n > 0 the output is identical to rb_sort_segments.  For n == 0 this call
// writes num_runs[0] = 0 and also seg_offsets[0] = 0 (rb_sort_segments leaves seg_offsets untouched then).
__attribute__((visibility("default")))
int rb_sort_segments_noalloc(const long long* keys_in, const int* vals_in, long long n, int end_bit,
                             long long* keys_out, int* vals_out, long long* unique_out, int* seg_offsets,
                             int* num_runs, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
