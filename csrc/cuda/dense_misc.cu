// Small dense-side kernels that surround the tcgen05 GEMMs:
//   * rb_bce_head       last linear layer (N = 1) + sigmoid + BCE-with-logits loss + its full backward
//                       (dH, dw, db) in one pass over the activations,
//   * rb_colsum16       bias gradient (column sums of a 16-bit matrix) with fp32 accumulation,
//   * rb_adam_flat / rb_sgd_flat  one launch over all dense parameters (fp32 master + 16-bit shadow),
//   * rb_cast_pad_f32_to_16  dense-feature cast with zero padding to a TMA-friendly row stride,
//   * rb_scale_cast_f32_to_bf16 / rb_axpy helpers used by the gradient all-reduce path.
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------
// fused logit head: z = h . w + b ; loss = BCEWithLogits(z, y) ; backward
// ---------------------------------------------------------------------------
template <int KMAX_PER_LANE>
__global__ void __launch_bounds__(256)
bce_head_kernel(const __nv_bfloat16* __restrict__ H, long long ldh, int B, int K, const float* __restrict__ w,
                const float* __restrict__ bias, const float* __restrict__ labels, float inv_batch,
                float* __restrict__ logits, float* __restrict__ loss_sum, __nv_bfloat16* __restrict__ dH,
                long long lddh, float* __restrict__ dw, float* __restrict__ db, int relu_mask) {
  __shared__ float red[8][KMAX_PER_LANE * 32 + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float wl[KMAX_PER_LANE], dwl[KMAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < KMAX_PER_LANE; ++i) {
    const int k = lane * 2 + (i >> 1) * 64 + (i & 1);
    wl[i] = (k < K) ? w[k] : 0.f;
    dwl[i] = 0.f;
  }
  const float b0 = bias ? bias[0] : 0.f;
  float db_l = 0.f, loss_l = 0.f;
  for (int b = blockIdx.x * 8 + warp; b < B; b += gridDim.x * 8) {
    const __nv_bfloat16* h = H + static_cast<long long>(b) * ldh;
    float hv[KMAX_PER_LANE];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < KMAX_PER_LANE; i += 2) {
      const int k = lane * 2 + (i >> 1) * 64;
      float2 v = make_float2(0.f, 0.f);
      if (k < K) v = rb::unpack_bf16(*reinterpret_cast<const uint32_t*>(h + k));
      hv[i] = v.x; hv[i + 1] = v.y;
      dot += v.x * wl[i] + v.y * wl[i + 1];
    }
    dot = rb::warp_sum(dot);
    const float z = dot + b0;
    const float y = labels[b];
    const float sig = 1.f / (1.f + __expf(-z));
    const float dz = (sig - y) * inv_batch;
    if (lane == 0) {
      if (logits) logits[b] = z;
      loss_l += fmaxf(z, 0.f) - z * y + log1pf(__expf(-fabsf(z)));
      db_l += dz;
    }
#pragma unroll
    for (int i = 0; i < KMAX_PER_LANE; i += 2) {
      const int k = lane * 2 + (i >> 1) * 64;
      dwl[i] += dz * hv[i];
      dwl[i + 1] += dz * hv[i + 1];
      if (dH && k < K) {
        float g0 = dz * wl[i], g1 = dz * wl[i + 1];
        if (relu_mask) { g0 = hv[i] > 0.f ? g0 : 0.f; g1 = hv[i + 1] > 0.f ? g1 : 0.f; }
        *reinterpret_cast<uint32_t*>(dH + static_cast<long long>(b) * lddh + k) = rb::pack_bf16(g0, g1);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < KMAX_PER_LANE; ++i) red[warp][i * 32 + lane] = dwl[i];
  __syncthreads();
  for (int e = threadIdx.x; e < KMAX_PER_LANE * 32; e += 256) {
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < 8; ++wv) s += red[wv][e];
    const int i = e / 32, ln = e % 32;
    const int k = ln * 2 + (i >> 1) * 64 + (i & 1);
    if (k < K && dw) atomicAdd(dw + k, s);
  }
  if (lane == 0) {
    atomicAdd(loss_sum, loss_l * inv_batch);
    if (db) atomicAdd(db, db_l);
  }
}

// column sums: out[n] += sum_m A[m][n], A 16-bit (bf16 or f16), block = 32 x 8 threads, each
// thread owns two adjacent columns.
__global__ void __launch_bounds__(256)
colsum16_kernel(const uint16_t* __restrict__ A, long long lda, int M, int N, int rows_per_block, int is_bf16,
                float* __restrict__ out) {
  __shared__ float red[8][64];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int n = blockIdx.x * 64 + tx * 2;
  const int m0 = blockIdx.y * rows_per_block;
  const int m1 = min(M, m0 + rows_per_block);
  float s0 = 0.f, s1 = 0.f;
  if (n < N) {
    for (int m = m0 + ty; m < m1; m += 8) {
      const uint32_t u = *reinterpret_cast<const uint32_t*>(A + static_cast<long long>(m) * lda + n);
      const float2 v = is_bf16 ? rb::unpack_bf16(u) : rb::unpack_f16(u);
      s0 += v.x; s1 += v.y;
    }
  }
  red[ty][tx * 2] = s0; red[ty][tx * 2 + 1] = s1;
  __syncthreads();
  if (ty == 0) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { a += red[i][tx * 2]; b += red[i][tx * 2 + 1]; }
    if (n < N) atomicAdd(out + n, a);
    if (n + 1 < N) atomicAdd(out + n + 1, b);
  }
}

// hyper = {lr, 1-beta1^t, 1-beta2^t, t}: kept on the device so a captured CUDA graph sees the
// step count and learning rate of the replay, not of the capture.
__global__ void adam_tick_kernel(float* __restrict__ hyper, float beta1, float beta2) {
  const float t = hyper[3] + 1.f;
  hyper[3] = t;
  hyper[1] = 1.f - powf(beta1, t);
  hyper[2] = 1.f - powf(beta2, t);
}

__global__ void adam_flat_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                 float* __restrict__ v, uint16_t* __restrict__ shadow, int is_bf16, long long n,
                                 float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                                 float grad_scale, const float* __restrict__ hyper) {
  if (hyper) { lr = hyper[0]; bc1 = hyper[1]; bc2 = hyper[2]; }
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float gi = g[i] * grad_scale;
    float pi = p[i];
    gi += wd * pi;
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    m[i] = mi; v[i] = vi;
    pi -= (lr / bc1) * mi / (sqrtf(vi / bc2) + eps);
    p[i] = pi;
    if (shadow) shadow[i] = is_bf16 ? __bfloat16_as_ushort(__float2bfloat16(pi)) : __half_as_ushort(__float2half(pi));
  }
}

__global__ void sgd_flat_kernel(float* __restrict__ p, const float* __restrict__ g, uint16_t* __restrict__ shadow,
                                int is_bf16, long long n, float lr, float wd, float grad_scale) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float pi = p[i];
    pi -= lr * (g[i] * grad_scale + wd * pi);
    p[i] = pi;
    if (shadow) shadow[i] = is_bf16 ? __bfloat16_as_ushort(__float2bfloat16(pi)) : __half_as_ushort(__float2half(pi));
  }
}

__global__ void cast_pad_kernel(const float* __restrict__ src, long long lds, int rows, int cols,
                                uint16_t* __restrict__ dst, long long ldd, int cols_pad, int is_bf16) {
  const long long total = static_cast<long long>(rows) * cols_pad;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols_pad;
    const int c = static_cast<int>(i % cols_pad);
    const float v = (c < cols) ? src[r * lds + c] : 0.f;
    dst[r * ldd + c] = is_bf16 ? __bfloat16_as_ushort(__float2bfloat16(v)) : __half_as_ushort(__float2half(v));
  }
}

__global__ void scale_cast_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n,
                                  float scale) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __float2bfloat16(src[i] * scale);
}

inline int grid_for(long long n, int num_sms) {
  long long b = (n + 255) / 256;
  const long long cap = static_cast<long long>(num_sms > 0 ? num_sms : 148) * 8;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace

// H [B,K] bf16 (K even, <= 512).  Accumulates into loss_sum / dw / db (callers zero them).
// relu_mask != 0: H is the output of a ReLU, and dH is returned already multiplied by (H > 0).
RB_API int rb_bce_head(const void* H, long long ldh, int B, int K, const float* w, const float* bias,
                       const float* labels, float inv_batch, float* logits, float* loss_sum, void* dH,
                       long long lddh, float* dw, float* db, int relu_mask, int num_sms, cudaStream_t st) {
  if (B == 0) return 0;
  if (K > 512 || (K & 1)) return -1;
  if (num_sms <= 0) num_sms = 148;
  int blocks = (B + 7) / 8;
  if (blocks > num_sms * 4) blocks = num_sms * 4;
  const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(H);
  __nv_bfloat16* dh = reinterpret_cast<__nv_bfloat16*>(dH);
  if (K <= 128)
    bce_head_kernel<4><<<blocks, 256, 0, st>>>(h, ldh, B, K, w, bias, labels, inv_batch, logits, loss_sum, dh, lddh, dw, db, relu_mask);
  else if (K <= 256)
    bce_head_kernel<8><<<blocks, 256, 0, st>>>(h, ldh, B, K, w, bias, labels, inv_batch, logits, loss_sum, dh, lddh, dw, db, relu_mask);
  else
    bce_head_kernel<16><<<blocks, 256, 0, st>>>(h, ldh, B, K, w, bias, labels, inv_batch, logits, loss_sum, dh, lddh, dw, db, relu_mask);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_colsum16(const void* A, long long lda, int M, int N, int is_bf16, float* out, cudaStream_t st) {
  if (M == 0 || N == 0) return 0;
  if (lda & 1) return -1;
  const int rows_per_block = 1024;
  dim3 grid((N + 63) / 64, (M + rows_per_block - 1) / rows_per_block);
  colsum16_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint16_t*>(A), lda, M, N, rows_per_block, is_bf16, out);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_adam_flat(float* p, const float* g, float* m, float* v, void* shadow, int is_bf16, long long n,
                        float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                        float grad_scale, const float* hyper, int num_sms, cudaStream_t st) {
  if (n == 0) return 0;
  adam_flat_kernel<<<grid_for(n, num_sms), 256, 0, st>>>(p, g, m, v, reinterpret_cast<uint16_t*>(shadow), is_bf16,
                                                         n, lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale, hyper);
  return static_cast<int>(cudaGetLastError());
}

// hyper[3] += 1 and refresh the two bias corrections (one thread; ordered on the stream).
RB_API int rb_adam_tick(float* hyper, float beta1, float beta2, cudaStream_t st) {
  adam_tick_kernel<<<1, 1, 0, st>>>(hyper, beta1, beta2);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_sgd_flat(float* p, const float* g, void* shadow, int is_bf16, long long n, float lr, float wd,
                       float grad_scale, int num_sms, cudaStream_t st) {
  if (n == 0) return 0;
  sgd_flat_kernel<<<grid_for(n, num_sms), 256, 0, st>>>(p, g, reinterpret_cast<uint16_t*>(shadow), is_bf16, n, lr,
                                                        wd, grad_scale);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_cast_pad_f32_to_16(const float* src, long long lds, int rows, int cols, void* dst, long long ldd,
                                 int cols_pad, int is_bf16, int num_sms, cudaStream_t st) {
  if (rows == 0) return 0;
  cast_pad_kernel<<<grid_for(static_cast<long long>(rows) * cols_pad, num_sms), 256, 0, st>>>(
      src, lds, rows, cols, reinterpret_cast<uint16_t*>(dst), ldd, cols_pad, is_bf16);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_scale_cast_f32_to_bf16(const float* src, void* dst, long long n, float scale, int num_sms,
                                     cudaStream_t st) {
  if (n == 0) return 0;
  scale_cast_kernel<<<grid_for(n, num_sms), 256, 0, st>>>(src, reinterpret_cast<__nv_bfloat16*>(dst), n, scale);
  return static_cast<int>(cudaGetLastError());
}
