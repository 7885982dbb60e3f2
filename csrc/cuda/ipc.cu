// Own inter-process memory sharing below the peer group: device allocations that other ranks of the node map into
// their address space through CUDA IPC handles (the handles travel over the job's key-value store, see
// recsdk_b200/parallel/ipc.py).  The mappings are ordinary device pointers: every kernel of this library that takes a
// table of peer pointers (exchange, all-reduce, barriers) works on them with plain loads and stores.
// Role in the reference: the LCAL communicator's own shared-memory bootstrap and IPC buffer exchange
// (cust_op/ai_core_op/lccl: lcal_comm.cpp / lcal_sock_exchange.cpp).
#include <cstring>

#include "common.cuh"

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are exchanged as 64-byte blobs");

RB_API int rb_ipc_handle_bytes() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

// zero-filled device allocation that can be exported
RB_API int rb_ipc_alloc(long long bytes, void** out) {
  if (!out || bytes <= 0) return -1;
  void* p = nullptr;
  RB_CUDA_CHECK(cudaMalloc(&p, static_cast<size_t>(bytes)));
  const cudaError_t e = cudaMemset(p, 0, static_cast<size_t>(bytes));
  if (e != cudaSuccess) { cudaFree(p); return static_cast<int>(e); }
  RB_CUDA_CHECK(cudaDeviceSynchronize());     // set-up path: the zeros are visible before any peer maps the buffer
  *out = p;
  return 0;
}

RB_API int rb_ipc_export(void* ptr, void* handle64) {
  if (!ptr || !handle64) return -1;
  cudaIpcMemHandle_t h;
  RB_CUDA_CHECK(cudaIpcGetMemHandle(&h, ptr));
  std::memcpy(handle64, &h, sizeof(h));
  return 0;
}

// map another process's allocation (peer access between the two devices is enabled on first use)
RB_API int rb_ipc_open(const void* handle64, void** out) {
  if (!handle64 || !out) return -1;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  RB_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out = p;
  return 0;
}

RB_API int rb_ipc_close(void* mapped) { return mapped ? static_cast<int>(cudaIpcCloseMemHandle(mapped)) : 0; }

RB_API int rb_ipc_free(void* ptr) { return ptr ? static_cast<int>(cudaFree(ptr)) : 0; }

// 1 when `device` can map memory of `peer_device` (same device counts), 0 when not, negative on error
RB_API int rb_ipc_can_access(int device, int peer_device) {
  if (device == peer_device) return 1;
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, device, peer_device) != cudaSuccess) return -2;
  return ok;
}
