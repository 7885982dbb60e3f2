// Row IO by raw device address and the sparse optimizers that go with it.
//
//   rb_rows_gather_by_address   out[i, :] = fp32 row at address[i]                (address 0: zeros)
//   rb_rows_update_by_address   row at address[i] += values[i, :] (update_type 0, atomic: an address may repeat) or
//                               = values[i, :] (any other type)                   (address 0: skipped)
//   rb_rows_sgd                 var[idx[i]] -= lr * (g[i] + weight_decay * var[idx[i]])
//   rb_rows_lazy_adam           Adam moments and variable of the listed rows only (rows must be distinct)
//
// Addresses are what `HKVTable.find_pointers` hands out (value rows of a dynamic table).  Every address is checked
// against the caller's region [lo, hi) and 4-byte alignment before it is dereferenced; one that fails is skipped and
// RB_ERR_BOUNDS is written to the status word - a bad address never reaches the memory system.
// Role in the reference: cust_op/framework/tf_plugin/src/{cust_embedding_by_address,lazy_adam,sgd}.cpp and
// ai_core_op/cust_op_by_addr (EmbeddingLookupByAddress, EmbeddingUpdateByAddress, LazyAdam, Sgd).
#include "common.cuh"

namespace {

__device__ __forceinline__ bool addr_ok(unsigned long long a, long long row_bytes, unsigned long long lo, unsigned long long hi) {
  return a >= lo && a + static_cast<unsigned long long>(row_bytes) <= hi && (a & 3ull) == 0;
}

__global__ void __launch_bounds__(256) gather_by_address_kernel(const long long* __restrict__ addr, long long n, int D,
                                                                float* __restrict__ out, unsigned long long lo,
                                                                unsigned long long hi, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
    const unsigned long long a = static_cast<unsigned long long>(addr[i]);
    float* o = out + i * D;
    if (a == 0 || !addr_ok(a, static_cast<long long>(D) * 4, lo, hi)) {
      if (a != 0 && lane == 0 && status) atomicCAS(status, 0, RB_ERR_BOUNDS);
      for (int c = lane; c < D; c += 32) o[c] = 0.f;
      continue;
    }
    const float* src = reinterpret_cast<const float*>(a);
    for (int c = lane; c < D; c += 32) o[c] = src[c];
  }
}

__global__ void __launch_bounds__(256) update_by_address_kernel(const long long* __restrict__ addr, long long n, int D,
                                                                const float* __restrict__ values, int add,
                                                                unsigned long long lo, unsigned long long hi, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
    const unsigned long long a = static_cast<unsigned long long>(addr[i]);
    if (a == 0) continue;
    if (!addr_ok(a, static_cast<long long>(D) * 4, lo, hi)) {
      if (lane == 0 && status) atomicCAS(status, 0, RB_ERR_BOUNDS);
      continue;
    }
    float* dst = reinterpret_cast<float*>(a);
    const float* v = values + i * D;
    if (add) { for (int c = lane; c < D; c += 32) atomicAdd(dst + c, v[c]); }
    else { for (int c = lane; c < D; c += 32) dst[c] = v[c]; }
  }
}

// mode 0: SGD, 1: lazy Adam
__global__ void __launch_bounds__(256) rows_optimizer_kernel(float* __restrict__ var, float* __restrict__ m, float* __restrict__ v,
                                                             const long long* __restrict__ idx, const float* __restrict__ g,
                                                             long long n, int D, long long rows, int mode, float lr, float wd,
                                                             float b1, float b2, float eps, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
    const long long r = idx[i];
    if (r < 0) continue;
    if (r >= rows) {
      if (lane == 0 && status) atomicCAS(status, 0, RB_ERR_BOUNDS);
      continue;
    }
    float* w = var + r * D;
    const float* gi = g + i * D;
    if (mode == 0) {
      if (wd == 0.f) { for (int c = lane; c < D; c += 32) atomicAdd(w + c, -lr * gi[c]); }     // an index may repeat
      else { for (int c = lane; c < D; c += 32) w[c] -= lr * (gi[c] + wd * w[c]); }
    } else {
      float* mr = m + r * D;
      float* vr = v + r * D;
      for (int c = lane; c < D; c += 32) {
        const float gv = gi[c];
        const float mn = b1 * mr[c] + (1.f - b1) * gv;
        const float vn = b2 * vr[c] + (1.f - b2) * gv * gv;
        mr[c] = mn; vr[c] = vn;
        w[c] -= lr * mn / (sqrtf(vn) + eps);
      }
    }
  }
}

inline int warp_grid_n(long long n, int num_sms) {
  long long b = (n * 32 + 255) / 256;
  const long long cap = static_cast<long long>(num_sms > 0 ? num_sms : 148) * 8;
  if (b > cap) b = cap;
  return static_cast<int>(b < 1 ? 1 : b);
}

}  // namespace

RB_API int rb_rows_gather_by_address(const long long* addr, long long n, int D, float* out, unsigned long long region_lo,
                                     unsigned long long region_hi, int num_sms, int* status, cudaStream_t st) {
  if (n == 0) return 0;
  if (D <= 0 || region_hi <= region_lo) return -1;
  gather_by_address_kernel<<<warp_grid_n(n, num_sms), 256, 0, st>>>(addr, n, D, out, region_lo, region_hi, status);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_rows_update_by_address(const long long* addr, long long n, int D, const float* values, int update_type,
                                     unsigned long long region_lo, unsigned long long region_hi, int num_sms, int* status,
                                     cudaStream_t st) {
  if (n == 0) return 0;
  if (D <= 0 || region_hi <= region_lo) return -1;
  update_by_address_kernel<<<warp_grid_n(n, num_sms), 256, 0, st>>>(addr, n, D, values, update_type == 0 ? 1 : 0, region_lo,
                                                                   region_hi, status);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_rows_sgd(float* var, long long rows, int D, const long long* idx, const float* grads, long long n, float lr,
                       float weight_decay, int num_sms, int* status, cudaStream_t st) {
  if (n == 0) return 0;
  if (D <= 0 || rows <= 0) return -1;
  rows_optimizer_kernel<<<warp_grid_n(n, num_sms), 256, 0, st>>>(var, nullptr, nullptr, idx, grads, n, D, rows, 0, lr,
                                                                weight_decay, 0.f, 0.f, 0.f, status);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_rows_lazy_adam(float* var, float* m, float* v, long long rows, int D, const long long* idx, const float* grads,
                             long long n, float lr, float beta1, float beta2, float eps, int num_sms, int* status,
                             cudaStream_t st) {
  if (n == 0) return 0;
  if (D <= 0 || rows <= 0 || !m || !v) return -1;
  rows_optimizer_kernel<<<warp_grid_n(n, num_sms), 256, 0, st>>>(var, m, v, idx, grads, n, D, rows, 1, lr, 0.f, beta1, beta2,
                                                                eps, status);
  return static_cast<int>(cudaGetLastError());
}
