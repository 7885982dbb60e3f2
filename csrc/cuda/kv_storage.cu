// Host tier of the paged KV cache: a pinned chunk pool and the transfer engine between it and the device page tables.
//
// Layout of the pool: [chunk][layer][row] with `rows_per_cl` rows of `row_bytes` per (chunk, layer) - a row is one K or V
// page, the same unit as a row of a layer's device cache table, so one (chunk, layer) is ONE contiguous DMA transfer.
//
// Four streams, two staging buffers per direction, an event per layer:
//
//   onload :  pool --cudaMemcpyAsync H2D (onload stream)--> staging slot --scatter kernel (scatter stream)--> cache rows
//   offload:  cache rows --gather kernel (gather stream)--> staging slot --cudaMemcpyAsync D2H (offload stream)--> pool
//
// Layer l + 1's DMA runs while layer l's scatter kernel does (slots alternate; a slot is reused only after the event of
// its last consumer), and the caller's compute stream can wait for a single layer (`rb_kvs_task_stream_wait`) instead of
// the whole transfer.  The DMA engines move the bytes: no SM reads host memory.  Row lists travel through a small
// pinned index buffer per task.  Nothing here blocks the host; completion is polled (`rb_kvs_task_query`).
//
// Failure injection for tests is on the host: `rb_kvs_inject_failure(n)` makes the n-th following copy call report an
// error instead of being issued; the task then carries the error and the caller rolls back.
// Role in the reference: inference/kvcache_manager/src/native_host_kvcache_manager_impl.h:41-214 (handles with per-layer
// events, four streams, staging buffers, pinned chunk storage).
#include <mutex>
#include <new>
#include <vector>

#include "common.cuh"

namespace {

constexpr int KVS_SLOTS = 2;
constexpr int KVS_TASKS = 16;
constexpr int KVS_MAX_LAYERS = 256;

struct KvTask {
  std::vector<cudaEvent_t> layer_ev;
  long long* h_idx = nullptr;        // pinned row list of this task
  long long* d_idx = nullptr;
  long long idx_cap = 0;
  int busy = 0;
  int error = 0;                     // first cudaError_t seen while launching (0 = none)
  int layers_issued = 0;
};

struct KvStorage {
  int device = 0, num_layers = 0, rows_per_cl = 0;
  long long num_chunks = 0, row_bytes = 0, stage_rows = 0;
  char* pool = nullptr;
  std::vector<void*> cache;
  cudaStream_t s_onload = nullptr, s_scatter = nullptr, s_gather = nullptr, s_offload = nullptr;
  char* stage_on[KVS_SLOTS] = {nullptr, nullptr};
  char* stage_off[KVS_SLOTS] = {nullptr, nullptr};
  cudaEvent_t on_copied[KVS_SLOTS], on_free[KVS_SLOTS], off_gathered[KVS_SLOTS], off_free[KVS_SLOTS];
  cudaEvent_t ev_after = nullptr;
  unsigned on_use = 0, off_use = 0;
  KvTask tasks[KVS_TASKS];
  long long fail_countdown = -1;     // >= 0: copies until the injected failure
  long long stats[4] = {0, 0, 0, 0}; // bytes H2D, bytes D2H, copy calls, kernels
  std::mutex mu;
};

// rows of 16-byte vectors; scatter: dst[rows[i]] = src[i], gather: dst[i] = src[rows[i]]
__global__ void __launch_bounds__(256) kvs_move_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                             const long long* __restrict__ rows, long long n_rows,
                                                             long long vec_per_row, int scatter) {
  const long long total = n_rows * vec_per_row;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < total;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long i = v / vec_per_row, c = v - i * vec_per_row;
    const long long r = rows[i];
    if (r < 0) continue;
    if (scatter) dst[r * vec_per_row + c] = src[v];
    else dst[v] = src[r * vec_per_row + c];
  }
}

// every copy goes through here so that a test can make one of them fail without touching the GPU
cudaError_t kvs_copy(KvStorage* s, void* dst, const void* src, size_t bytes, cudaMemcpyKind kind, cudaStream_t st) {
  if (s->fail_countdown >= 0) {
    if (s->fail_countdown == 0) {
      s->fail_countdown = -1;
      return cudaErrorUnknown;
    }
    --s->fail_countdown;
  }
  s->stats[kind == cudaMemcpyHostToDevice ? 0 : 1] += static_cast<long long>(bytes);
  s->stats[2] += 1;
  return cudaMemcpyAsync(dst, src, bytes, kind, st);
}

int kvs_take_task(KvStorage* s, long long n_rows) {
  for (int t = 0; t < KVS_TASKS; ++t) {
    KvTask& k = s->tasks[t];
    if (k.busy) continue;
    if (k.idx_cap < n_rows) {
      if (k.h_idx) cudaFreeHost(k.h_idx);
      if (k.d_idx) cudaFree(k.d_idx);
      k.h_idx = nullptr; k.d_idx = nullptr; k.idx_cap = 0;
      const long long cap = n_rows < 1024 ? 1024 : n_rows;
      if (cudaHostAlloc(reinterpret_cast<void**>(&k.h_idx), sizeof(long long) * cap, cudaHostAllocDefault) != cudaSuccess) return -1;
      if (cudaMalloc(reinterpret_cast<void**>(&k.d_idx), sizeof(long long) * cap) != cudaSuccess) return -1;
      k.idx_cap = cap;
    }
    k.busy = 1; k.error = 0; k.layers_issued = 0;
    return t;
  }
  return -1;
}

#define KVS_TRY(expr)                                     \
  do {                                                    \
    const cudaError_t e_ = (expr);                        \
    if (e_ != cudaSuccess) { task.error = static_cast<int>(e_); goto done; } \
  } while (0)

}  // namespace

// stage_rows: rows per staging slot (a transfer with more rows per layer goes through the slot in pieces of whole chunks)
RB_API int rb_kvs_create(int device, int num_layers, long long num_chunks, int rows_per_chunk_layer, long long row_bytes,
                         long long stage_rows, void** out) {
  if (!out || num_layers <= 0 || num_layers > KVS_MAX_LAYERS || num_chunks <= 0 || rows_per_chunk_layer <= 0 || row_bytes <= 0 ||
      (row_bytes % 16))
    return -1;
  if (stage_rows < rows_per_chunk_layer) stage_rows = rows_per_chunk_layer;
  stage_rows -= stage_rows % rows_per_chunk_layer;
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return static_cast<int>(e);
  KvStorage* s = new (std::nothrow) KvStorage();
  if (!s) return -2;
  s->device = device; s->num_layers = num_layers; s->num_chunks = num_chunks; s->rows_per_cl = rows_per_chunk_layer;
  s->row_bytes = row_bytes; s->stage_rows = stage_rows;
  s->cache.assign(num_layers, nullptr);
  const size_t pool_bytes = static_cast<size_t>(num_chunks) * num_layers * rows_per_chunk_layer * row_bytes;
  e = cudaHostAlloc(reinterpret_cast<void**>(&s->pool), pool_bytes, cudaHostAllocPortable);
  if (e != cudaSuccess) { delete s; return static_cast<int>(e); }
  bool ok = true;
  ok &= cudaStreamCreateWithFlags(&s->s_onload, cudaStreamNonBlocking) == cudaSuccess;
  ok &= cudaStreamCreateWithFlags(&s->s_scatter, cudaStreamNonBlocking) == cudaSuccess;
  ok &= cudaStreamCreateWithFlags(&s->s_gather, cudaStreamNonBlocking) == cudaSuccess;
  ok &= cudaStreamCreateWithFlags(&s->s_offload, cudaStreamNonBlocking) == cudaSuccess;
  for (int i = 0; i < KVS_SLOTS && ok; ++i) {
    ok &= cudaMalloc(reinterpret_cast<void**>(&s->stage_on[i]), static_cast<size_t>(stage_rows) * row_bytes) == cudaSuccess;
    ok &= cudaMalloc(reinterpret_cast<void**>(&s->stage_off[i]), static_cast<size_t>(stage_rows) * row_bytes) == cudaSuccess;
    ok &= cudaEventCreateWithFlags(&s->on_copied[i], cudaEventDisableTiming) == cudaSuccess;
    ok &= cudaEventCreateWithFlags(&s->on_free[i], cudaEventDisableTiming) == cudaSuccess;
    ok &= cudaEventCreateWithFlags(&s->off_gathered[i], cudaEventDisableTiming) == cudaSuccess;
    ok &= cudaEventCreateWithFlags(&s->off_free[i], cudaEventDisableTiming) == cudaSuccess;
  }
  ok = ok && cudaEventCreateWithFlags(&s->ev_after, cudaEventDisableTiming) == cudaSuccess;
  for (int t = 0; t < KVS_TASKS && ok; ++t) {
    s->tasks[t].layer_ev.resize(num_layers);
    for (int l = 0; l < num_layers && ok; ++l)
      ok &= cudaEventCreateWithFlags(&s->tasks[t].layer_ev[l], cudaEventDisableTiming) == cudaSuccess;
  }
  if (!ok) return -3;     // the partially built object is leaked on purpose: the context is in an unknown state
  *out = s;
  return 0;
}

RB_API int rb_kvs_destroy(void* h) {
  KvStorage* s = static_cast<KvStorage*>(h);
  if (!s) return 0;
  cudaSetDevice(s->device);
  cudaStreamSynchronize(s->s_onload); cudaStreamSynchronize(s->s_scatter);
  cudaStreamSynchronize(s->s_gather); cudaStreamSynchronize(s->s_offload);
  for (int t = 0; t < KVS_TASKS; ++t) {
    for (cudaEvent_t ev : s->tasks[t].layer_ev) cudaEventDestroy(ev);
    if (s->tasks[t].h_idx) cudaFreeHost(s->tasks[t].h_idx);
    if (s->tasks[t].d_idx) cudaFree(s->tasks[t].d_idx);
  }
  for (int i = 0; i < KVS_SLOTS; ++i) {
    cudaFree(s->stage_on[i]); cudaFree(s->stage_off[i]);
    cudaEventDestroy(s->on_copied[i]); cudaEventDestroy(s->on_free[i]);
    cudaEventDestroy(s->off_gathered[i]); cudaEventDestroy(s->off_free[i]);
  }
  cudaEventDestroy(s->ev_after);
  cudaStreamDestroy(s->s_onload); cudaStreamDestroy(s->s_scatter); cudaStreamDestroy(s->s_gather); cudaStreamDestroy(s->s_offload);
  cudaFreeHost(s->pool);
  delete s;
  return 0;
}

RB_API long long rb_kvs_pool(void* h) { return static_cast<long long>(reinterpret_cast<uintptr_t>(static_cast<KvStorage*>(h)->pool)); }

RB_API long long rb_kvs_pool_bytes(void* h) {
  KvStorage* s = static_cast<KvStorage*>(h);
  return s->num_chunks * s->num_layers * s->rows_per_cl * s->row_bytes;
}

RB_API int rb_kvs_register_cache(void* h, int layer, void* cache_rows) {
  KvStorage* s = static_cast<KvStorage*>(h);
  if (layer < 0 || layer >= s->num_layers) return -1;
  s->cache[layer] = cache_rows;
  return 0;
}

// the `countdown`-th copy call from now (0 = the next one) reports an error instead of being issued; -1 disarms
RB_API int rb_kvs_inject_failure(void* h, long long countdown) {
  static_cast<KvStorage*>(h)->fail_countdown = countdown;
  return 0;
}

RB_API int rb_kvs_stats(void* h, long long* out4) {
  KvStorage* s = static_cast<KvStorage*>(h);
  for (int i = 0; i < 4; ++i) out4[i] = s->stats[i];
  return 0;
}

// Move `n_chunks` chunks between the pool and the device tables of all layers.  `rows` (host, n_chunks * rows_per_cl
// entries) lists the cache row of every pool row in chunk order; -1 skips a row.  The work is ordered after everything
// enqueued on `after` so far.  -> task id in *task_out (>= 0); the return value is 0, a negative argument error, or the
// cudaError_t of the call that failed (the task then exists, carries the error, and must still be released).
static int kvs_transfer(KvStorage* s, int onload, const long long* chunk_ids, long long n_chunks, const long long* rows,
                        cudaStream_t after, int* task_out) {
  if (!s || !task_out || n_chunks <= 0 || !chunk_ids || !rows) return -1;
  std::lock_guard<std::mutex> lock(s->mu);
  for (long long c = 0; c < n_chunks; ++c)
    if (chunk_ids[c] < 0 || chunk_ids[c] >= s->num_chunks) return -4;
  for (int l = 0; l < s->num_layers; ++l)
    if (!s->cache[l]) return -5;
  cudaSetDevice(s->device);
  const long long n_rows = n_chunks * s->rows_per_cl;
  const int t = kvs_take_task(s, n_rows);
  if (t < 0) return -6;
  KvTask& task = s->tasks[t];
  *task_out = t;
  const size_t cl_bytes = static_cast<size_t>(s->rows_per_cl) * s->row_bytes;
  const long long vec_per_row = s->row_bytes / 16;
  const long long chunks_per_piece = s->stage_rows / s->rows_per_cl;
  cudaStream_t s_dma = onload ? s->s_onload : s->s_offload;
  cudaStream_t s_krn = onload ? s->s_scatter : s->s_gather;
  for (long long i = 0; i < n_rows; ++i) task.h_idx[i] = rows[i];
  KVS_TRY(cudaEventRecord(s->ev_after, after));
  KVS_TRY(cudaStreamWaitEvent(s_krn, s->ev_after, 0));
  KVS_TRY(cudaStreamWaitEvent(s_dma, s->ev_after, 0));
  KVS_TRY(cudaMemcpyAsync(task.d_idx, task.h_idx, sizeof(long long) * n_rows, cudaMemcpyHostToDevice, s_krn));
  for (int l = 0; l < s->num_layers; ++l) {
    for (long long c0 = 0; c0 < n_chunks; c0 += chunks_per_piece) {
      const long long nc = (n_chunks - c0) < chunks_per_piece ? (n_chunks - c0) : chunks_per_piece;
      const long long piece_rows = nc * s->rows_per_cl;
      const long long total_vec = piece_rows * vec_per_row;
      const int grid = static_cast<int>(total_vec / 256 + 1 < 148 * 8 ? total_vec / 256 + 1 : 148 * 8);
      if (onload) {
        const unsigned slot = s->on_use++ % KVS_SLOTS;
        KVS_TRY(cudaStreamWaitEvent(s_dma, s->on_free[slot], 0));
        for (long long c = 0; c < nc; ++c)
          KVS_TRY(kvs_copy(s, s->stage_on[slot] + c * cl_bytes,
                           s->pool + (static_cast<size_t>(chunk_ids[c0 + c]) * s->num_layers + l) * cl_bytes, cl_bytes,
                           cudaMemcpyHostToDevice, s_dma));
        KVS_TRY(cudaEventRecord(s->on_copied[slot], s_dma));
        KVS_TRY(cudaStreamWaitEvent(s_krn, s->on_copied[slot], 0));
        kvs_move_rows_kernel<<<grid, 256, 0, s_krn>>>(reinterpret_cast<const uint4*>(s->stage_on[slot]),
                                                      reinterpret_cast<uint4*>(s->cache[l]),
                                                      task.d_idx + c0 * s->rows_per_cl, piece_rows, vec_per_row, 1);
        KVS_TRY(cudaGetLastError());
        s->stats[3] += 1;
        KVS_TRY(cudaEventRecord(s->on_free[slot], s_krn));
      } else {
        const unsigned slot = s->off_use++ % KVS_SLOTS;
        KVS_TRY(cudaStreamWaitEvent(s_krn, s->off_free[slot], 0));
        kvs_move_rows_kernel<<<grid, 256, 0, s_krn>>>(reinterpret_cast<const uint4*>(s->cache[l]),
                                                      reinterpret_cast<uint4*>(s->stage_off[slot]),
                                                      task.d_idx + c0 * s->rows_per_cl, piece_rows, vec_per_row, 0);
        KVS_TRY(cudaGetLastError());
        s->stats[3] += 1;
        KVS_TRY(cudaEventRecord(s->off_gathered[slot], s_krn));
        KVS_TRY(cudaStreamWaitEvent(s_dma, s->off_gathered[slot], 0));
        for (long long c = 0; c < nc; ++c)
          KVS_TRY(kvs_copy(s, s->pool + (static_cast<size_t>(chunk_ids[c0 + c]) * s->num_layers + l) * cl_bytes,
                           s->stage_off[slot] + c * cl_bytes, cl_bytes, cudaMemcpyDeviceToHost, s_dma));
        KVS_TRY(cudaEventRecord(s->off_free[slot], s_dma));
      }
    }
    KVS_TRY(cudaEventRecord(task.layer_ev[l], onload ? s_krn : s_dma));
    task.layers_issued = l + 1;
  }
done:
  return task.error;
}

RB_API int rb_kvs_onload(void* h, const long long* chunk_ids, long long n_chunks, const long long* dst_rows,
                         cudaStream_t after, int* task_out) {
  return kvs_transfer(static_cast<KvStorage*>(h), 1, chunk_ids, n_chunks, dst_rows, after, task_out);
}

RB_API int rb_kvs_offload(void* h, const long long* chunk_ids, long long n_chunks, const long long* src_rows,
                          cudaStream_t after, int* task_out) {
  return kvs_transfer(static_cast<KvStorage*>(h), 0, chunk_ids, n_chunks, src_rows, after, task_out);
}

// layer < 0: the whole task.  -> 0 done, 1 still running, 2 this layer was never issued (the launch failed before it),
// negative: bad argument
RB_API int rb_kvs_task_query(void* h, int task, int layer) {
  KvStorage* s = static_cast<KvStorage*>(h);
  if (task < 0 || task >= KVS_TASKS || layer >= s->num_layers) return -1;
  KvTask& k = s->tasks[task];
  if (!k.busy) return -2;
  const int last = layer < 0 ? k.layers_issued - 1 : layer;
  if (layer < 0 && k.error) return 2;
  if (last < 0 || last >= k.layers_issued) return 2;
  const cudaError_t e = cudaEventQuery(k.layer_ev[last]);
  if (e == cudaSuccess) return 0;
  if (e == cudaErrorNotReady) return 1;
  return -static_cast<int>(e) - 100;
}

// make `st` wait until `layer` of the task has arrived (no host blocking)
RB_API int rb_kvs_task_stream_wait(void* h, int task, int layer, cudaStream_t st) {
  KvStorage* s = static_cast<KvStorage*>(h);
  if (task < 0 || task >= KVS_TASKS || layer < 0 || layer >= s->num_layers) return -1;
  KvTask& k = s->tasks[task];
  if (!k.busy || layer >= k.layers_issued) return -2;
  return static_cast<int>(cudaStreamWaitEvent(st, k.layer_ev[layer], 0));
}

RB_API int rb_kvs_task_error(void* h, int task) {
  KvStorage* s = static_cast<KvStorage*>(h);
  if (task < 0 || task >= KVS_TASKS) return -1;
  return s->tasks[task].error;
}

// Give the task slot back.  `drain` != 0 first waits on the host for whatever of the task was issued (needed before the
// chunks of a failed or timed-out offload can be reused).  Without `drain` a task that is still running is NOT released
// (-> 1): its row list and events are in use.
RB_API int rb_kvs_task_release(void* h, int task, int drain) {
  KvStorage* s = static_cast<KvStorage*>(h);
  if (task < 0 || task >= KVS_TASKS) return -1;
  KvTask& k = s->tasks[task];
  if (!k.busy) return 0;
  int rc = 0;
  if (drain) {
    cudaSetDevice(s->device);
    // everything issued for the task sits on these four streams
    cudaError_t e = cudaStreamSynchronize(s->s_onload);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->s_scatter);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->s_gather);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->s_offload);
    rc = static_cast<int>(e);
  } else if (k.layers_issued > 0 && cudaEventQuery(k.layer_ev[k.layers_issued - 1]) == cudaErrorNotReady) {
    return 1;
  }
  std::lock_guard<std::mutex> lock(s->mu);
  k.busy = 0;
  return rc;
}
