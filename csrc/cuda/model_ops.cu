// Model-level fused kernels around the tcgen05 GEMMs (HBM-bound row kernels, 16-byte vector accesses):
//
//   rb_sampled_softmax      sampled-softmax next-item loss of the HSTU trainer, forward and gradient in one pass over
//                           the logits: per row  pos = <h, e_pos>,  lse = logsumexp([pos, neg_logits]),  nll = lse - pos;
//                           writes d(neg_logits) in place of the logits (bf16), d h (direct part) and d e_pos, and adds
//                           the row losses into one fp32 cell.  The two GEMMs of the backward (d h += dL @ E_neg,
//                           d E_neg = dL^T @ h) then run on the stored gradient without any elementwise pass between.
//   rb_dcn_cross_fwd/bwd    DCN v2 cross layer combine  y = x0 * (W x_l + b) + x_l  and its three gradients in one pass
//                           each (the W x_l product itself is a GEMM with the bias in its epilogue).
//   rb_multislice_concat    out[:, concat of slices] = in[:, start_k : end_k] for a list of column slices (one launch
//                           instead of one copy per slice); reference op multislice_concat
//                           (cust_op/framework/torch_plugin/torch_library/multislice_concat).
//
// These have no counterpart kernel in the reference (its models leave them to framework ops); they exist so that no
// eager elementwise pass sits between the GEMMs of the two benchmark models.
#include "common.cuh"
#include "tbe_common.cuh"

using namespace rbtbe;

namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per row.  logits [M, N] (bf16, row stride ld_l) are overwritten by their gradient.
// MAXV = ceil(N / 256): 8-element vectors per lane held in registers.
template <int MAXV>
__global__ void __launch_bounds__(256) sampled_softmax_kernel(
    const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ e_pos, long long ld_h, long long ld_e, int d,
    __nv_bfloat16* __restrict__ logits, long long ld_l, int N, long long M, float grad_scale,
    __nv_bfloat16* __restrict__ dh, __nv_bfloat16* __restrict__ de_pos, long long ld_dh, long long ld_de,
    float* __restrict__ loss_sum, float* __restrict__ row_loss) {
  const int lane = threadIdx.x & 31;
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= M) return;
  // ---- positive logit
  const __nv_bfloat16* hr = h + row * ld_h;
  const __nv_bfloat16* er = e_pos + row * ld_e;
  float dot = 0.f;
  for (int c = lane * 8; c < d; c += 256) {
    float a[8], b[8];
    Vec8<__nv_bfloat16>::ld(hr + c, a);
    Vec8<__nv_bfloat16>::ld(er + c, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) dot = fmaf(a[i], b[i], dot);
  }
  const float pos = warp_sum_f(dot);
  // ---- negatives: max, sum of exponentials (values stay in registers)
  __nv_bfloat16* lr = logits + row * ld_l;
  float v[MAXV][8];
  float mx = pos;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int c = (k * 32 + lane) * 8;
    if (c < N) {
      Vec8<__nv_bfloat16>::ld(lr + c, v[k]);
#pragma unroll
      for (int i = 0; i < 8; ++i) mx = fmaxf(mx, v[k][i]);
    }
  }
  mx = warp_max(mx);
  float se = 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int c = (k * 32 + lane) * 8;
    if (c < N) {
#pragma unroll
      for (int i = 0; i < 8; ++i) { v[k][i] = __expf(v[k][i] - mx); se += v[k][i]; }
    }
  }
  se = warp_sum_f(se);
  const float ep = __expf(pos - mx);
  const float denom = se + ep;
  const float nll = __logf(denom) + mx - pos;
  const float inv = grad_scale / denom;
  // ---- gradients: d neg_logits = softmax * g (in place), d pos = (softmax_pos - 1) * g
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int c = (k * 32 + lane) * 8;
    if (c < N) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[k][i] *= inv;
      Vec8<__nv_bfloat16>::st(lr + c, v[k]);
    }
  }
  const float dpos = ep * inv - grad_scale;
  __nv_bfloat16* dhr = dh + row * ld_dh;
  __nv_bfloat16* der = de_pos + row * ld_de;
  for (int c = lane * 8; c < d; c += 256) {
    float a[8], b[8];
    Vec8<__nv_bfloat16>::ld(hr + c, a);
    Vec8<__nv_bfloat16>::ld(er + c, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) { const float t = a[i]; a[i] = dpos * b[i]; b[i] = dpos * t; }
    Vec8<__nv_bfloat16>::st(dhr + c, a);      // d h (direct part) = dpos * e_pos
    Vec8<__nv_bfloat16>::st(der + c, b);      // d e_pos           = dpos * h
  }
  if (lane == 0) {
    if (row_loss) row_loss[row] = nll;
    atomicAdd(loss_sum, nll * grad_scale);
  }
}

// y = x0 * xw + xl     (all [M, D], 16-bit; 8 elements per thread)
template <typename T>
__global__ void dcn_cross_fwd_kernel(const T* __restrict__ x0, const T* __restrict__ xw, const T* __restrict__ xl,
                                     T* __restrict__ y, long long n_vec) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  float a[8], b[8], c[8];
  Vec8<T>::ld(x0 + i * 8, a);
  Vec8<T>::ld(xw + i * 8, b);
  Vec8<T>::ld(xl + i * 8, c);
#pragma unroll
  for (int k = 0; k < 8; ++k) a[k] = fmaf(a[k], b[k], c[k]);
  Vec8<T>::st(y + i * 8, a);
}

// dxw = dy * x0 ;  dx0 (+)= dy * xw ;  dxl = dy (the caller aliases dxl to dy: nothing to write)
template <typename T>
__global__ void dcn_cross_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x0, const T* __restrict__ xw,
                                     T* __restrict__ dxw, float* __restrict__ dx0_acc, int accumulate, long long n_vec) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  float g[8], a[8], b[8], acc[8];
  Vec8<T>::ld(dy + i * 8, g);
  Vec8<T>::ld(x0 + i * 8, a);
  Vec8<T>::ld(xw + i * 8, b);
  if (accumulate) Vec8<float>::ld(dx0_acc + i * 8, acc);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    a[k] *= g[k];
    acc[k] = accumulate ? fmaf(g[k], b[k], acc[k]) : g[k] * b[k];
  }
  Vec8<T>::st(dxw + i * 8, a);
  Vec8<float>::st(dx0_acc + i * 8, acc);
}

struct SliceList {
  int start[32];
  int len[32];
  int out_off[32];
  int n;
};

// out[r, out_off[k] + c] = in[r, start[k] + c]; element size `es` bytes; one thread per (row, output byte quad)
__global__ void multislice_concat_kernel(const unsigned char* __restrict__ in, long long ld_in_bytes,
                                         unsigned char* __restrict__ out, long long ld_out_bytes, long long rows,
                                         int out_cols, int es, SliceList sl) {
  const long long total = rows * out_cols;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / out_cols;
    const int c = static_cast<int>(i - r * out_cols);
    int k = 0;
    while (k + 1 < sl.n && c >= sl.out_off[k + 1]) ++k;
    const int src_col = sl.start[k] + (c - sl.out_off[k]);
    const unsigned char* s = in + r * ld_in_bytes + static_cast<long long>(src_col) * es;
    unsigned char* d = out + r * ld_out_bytes + static_cast<long long>(c) * es;
    if (es == 2) *reinterpret_cast<unsigned short*>(d) = *reinterpret_cast<const unsigned short*>(s);
    else if (es == 4) *reinterpret_cast<unsigned int*>(d) = *reinterpret_cast<const unsigned int*>(s);
    else if (es == 8) *reinterpret_cast<unsigned long long*>(d) = *reinterpret_cast<const unsigned long long*>(s);
    else for (int b = 0; b < es; ++b) d[b] = s[b];
  }
}

}  // namespace

// h, e_pos [M, d] bf16 (d % 8 == 0), logits [M, N] bf16 (N % 8 == 0, N <= 2048): overwritten by d loss / d logits * grad_scale.
// dh, de_pos [M, d] bf16 outputs; loss_sum (fp32, pre-zeroed) += grad_scale * sum of row losses; row_loss [M] optional.
RB_API int rb_sampled_softmax(const void* h, const void* e_pos, long long ld_h, long long ld_e, int d, void* logits,
                              long long ld_l, int N, long long M, float grad_scale, void* dh, void* de_pos,
                              long long ld_dh, long long ld_de, float* loss_sum, float* row_loss, cudaStream_t st) {
  if (M == 0) return 0;
  if ((d % 8) || (N % 8) || N > 2048 || N <= 0 || (ld_h % 8) || (ld_e % 8) || (ld_l % 8) || (ld_dh % 8) || (ld_de % 8)) return -1;
  const long long blocks = (M * 32 + 255) / 256;
  auto H = reinterpret_cast<const __nv_bfloat16*>(h);
  auto E = reinterpret_cast<const __nv_bfloat16*>(e_pos);
  auto L = reinterpret_cast<__nv_bfloat16*>(logits);
  auto DH = reinterpret_cast<__nv_bfloat16*>(dh);
  auto DE = reinterpret_cast<__nv_bfloat16*>(de_pos);
#define RB_SSM(V) sampled_softmax_kernel<V><<<blocks, 256, 0, st>>>(H, E, ld_h, ld_e, d, L, ld_l, N, M, grad_scale, DH, DE, ld_dh, ld_de, loss_sum, row_loss)
  const int nv = (N + 255) / 256;
  if (nv <= 1) RB_SSM(1);
  else if (nv <= 2) RB_SSM(2);
  else if (nv <= 4) RB_SSM(4);
  else RB_SSM(8);
#undef RB_SSM
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_dcn_cross_fwd(const void* x0, const void* xw, const void* xl, void* y, long long n, int dtype, cudaStream_t st) {
  if (n == 0) return 0;
  if (n % 8) return -1;
  const long long nv = n / 8, blocks = (nv + 255) / 256;
  if (dtype == DT_BF16)
    dcn_cross_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x0), reinterpret_cast<const __nv_bfloat16*>(xw),
                                                               reinterpret_cast<const __nv_bfloat16*>(xl), reinterpret_cast<__nv_bfloat16*>(y), nv);
  else if (dtype == DT_F16)
    dcn_cross_fwd_kernel<__half><<<blocks, 256, 0, st>>>(reinterpret_cast<const __half*>(x0), reinterpret_cast<const __half*>(xw),
                                                        reinterpret_cast<const __half*>(xl), reinterpret_cast<__half*>(y), nv);
  else if (dtype == DT_F32)
    dcn_cross_fwd_kernel<float><<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(x0), reinterpret_cast<const float*>(xw),
                                                       reinterpret_cast<const float*>(xl), reinterpret_cast<float*>(y), nv);
  else return -1;
  return static_cast<int>(cudaGetLastError());
}

// dxw = dy * x0; dx0_acc (fp32) = dy * xw (accumulate = 0) or += (accumulate = 1).  The gradient of x_l is dy itself.
RB_API int rb_dcn_cross_bwd(const void* dy, const void* x0, const void* xw, void* dxw, float* dx0_acc, int accumulate,
                            long long n, int dtype, cudaStream_t st) {
  if (n == 0) return 0;
  if (n % 8) return -1;
  const long long nv = n / 8, blocks = (nv + 255) / 256;
  if (dtype == DT_BF16)
    dcn_cross_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x0),
                                                               reinterpret_cast<const __nv_bfloat16*>(xw), reinterpret_cast<__nv_bfloat16*>(dxw), dx0_acc, accumulate, nv);
  else if (dtype == DT_F16)
    dcn_cross_bwd_kernel<__half><<<blocks, 256, 0, st>>>(reinterpret_cast<const __half*>(dy), reinterpret_cast<const __half*>(x0),
                                                        reinterpret_cast<const __half*>(xw), reinterpret_cast<__half*>(dxw), dx0_acc, accumulate, nv);
  else if (dtype == DT_F32)
    dcn_cross_bwd_kernel<float><<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(dy), reinterpret_cast<const float*>(x0),
                                                       reinterpret_cast<const float*>(xw), reinterpret_cast<float*>(dxw), dx0_acc, accumulate, nv);
  else return -1;
  return static_cast<int>(cudaGetLastError());
}

// starts / lens: host arrays of n_slices (<= 32) column ranges of `in` (element units); out columns = sum(lens).
RB_API int rb_multislice_concat(const void* in, long long ld_in, void* out, long long ld_out, long long rows,
                                const int* starts, const int* lens, int n_slices, int elem_bytes, cudaStream_t st) {
  if (rows == 0 || n_slices == 0) return 0;
  if (n_slices > 32 || elem_bytes <= 0) return -1;
  SliceList sl;
  sl.n = n_slices;
  int off = 0;
  for (int k = 0; k < n_slices; ++k) {
    if (lens[k] < 0 || starts[k] < 0) return -1;
    sl.start[k] = starts[k]; sl.len[k] = lens[k]; sl.out_off[k] = off;
    off += lens[k];
  }
  for (int k = n_slices; k < 32; ++k) { sl.start[k] = 0; sl.len[k] = 0; sl.out_off[k] = off; }
  if (off == 0) return 0;
  const long long total = rows * off;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  multislice_concat_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
      reinterpret_cast<const unsigned char*>(in), ld_in * elem_bytes, reinterpret_cast<unsigned char*>(out),
      ld_out * elem_bytes, rows, off, elem_bytes, sl);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------------------
// Disentangled attention (DeBERTa): score[b,n,q,k] = (QK^T[q,k] + C2P[q, clamp(rel[q,k] + span)] + P2C[k, clamp(span - rel[k,q])]) * scale,
// masked softmax over k.  The three products come from plain GEMMs; this kernel fuses the two gathers, the scale, the
// mask, the softmax and both outputs (pre-softmax score and probabilities) into one pass over a row.
// One block per (b, n, q) row; the row lives in shared memory between the passes.
// Role in the reference: cust_op/framework/torch_plugin/torch_library/disentangle_attention/DisentangleAttenFusion.cpp.
// ---------------------------------------------------------------------------------------------------------------
namespace {

template <typename T>
__global__ void __launch_bounds__(256) disentangle_softmax_kernel(
    const T* __restrict__ qk, const T* __restrict__ c2p, const T* __restrict__ p2c, const long long* __restrict__ rel,
    const unsigned char* __restrict__ mask, long long mask_sb, int N, int S, int P, int span, float scale,
    T* __restrict__ probs, T* __restrict__ score) {
  extern __shared__ float row_sm[];
  __shared__ float red[8];
  const long long row = blockIdx.x;
  const int q = static_cast<int>(row % S);
  const long long bn = row / S;
  const long long b = bn / N;
  const T* qk_row = qk + row * S;
  const T* c2p_row = c2p ? c2p + row * P : nullptr;
  const T* p2c_bn = p2c ? p2c + bn * S * P : nullptr;
  const long long* rel_row = rel + static_cast<long long>(q) * S;
  const unsigned char* mask_row = mask + b * mask_sb + static_cast<long long>(q) * S;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float mx = -INFINITY;
  for (int k = threadIdx.x; k < S; k += blockDim.x) {
    const long long r = rel_row[k];
    float sc = static_cast<float>(qk_row[k]);
    if (c2p_row) {
      long long i = r + span;
      i = i < 0 ? 0 : (i > P - 1 ? P - 1 : i);
      sc += static_cast<float>(c2p_row[i]);
    }
    if (p2c_bn) {
      // the position-to-content term is gathered for (key, query) and transposed: its index uses rel[k][q]
      long long i = span - rel[static_cast<long long>(k) * S + q];
      i = i < 0 ? 0 : (i > P - 1 ? P - 1 : i);
      sc += static_cast<float>(p2c_bn[static_cast<long long>(k) * P + i]);
    }
    sc *= scale;
    score[row * S + k] = static_cast<T>(sc);
    const float m = mask_row[k] ? sc : -INFINITY;
    row_sm[k] = m;
    mx = fmaxf(mx, m);
  }
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < (blockDim.x >> 5); ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  float sum = 0.f;
  for (int k = threadIdx.x; k < S; k += blockDim.x) {
    const float v = row_sm[k];
    const float e = v == -INFINITY ? 0.f : __expf(v - mx);
    row_sm[k] = e;
    sum += e;
  }
  sum = warp_sum_f(sum);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) sum += red[w];
  const float inv = sum > 0.f ? 1.f / sum : 0.f;        // a fully masked row gives zeros
  for (int k = threadIdx.x; k < S; k += blockDim.x) probs[row * S + k] = static_cast<T>(row_sm[k] * inv);
}

}  // namespace

// qk [B,N,S,S], c2p / p2c [B,N,S,P] (either may be null), rel [S,S] int64, mask [B or 1][S][S] bytes (mask_stride_b = 0
// broadcasts one mask); probs / score [B,N,S,S]; all float tensors share `dtype` (0 fp32, 1 fp16, 2 bf16).
RB_API int rb_disentangle_softmax(const void* qk, const void* c2p, const void* p2c, const long long* rel, const void* mask,
                                  long long mask_stride_b, int B, int N, int S, int P, int span, float scale, int dtype,
                                  void* probs, void* score, cudaStream_t st) {
  const long long rows = static_cast<long long>(B) * N * S;
  if (rows == 0) return 0;
  if (rows > 0x7FFFFFFFll || S <= 0 || static_cast<size_t>(S) * 4 > 200 * 1024 || ((c2p || p2c) && P <= 0)) return -1;
  const size_t smem = static_cast<size_t>(S) * sizeof(float);
#define RB_DIS(T_)                                                                                                        \
  do {                                                                                                                    \
    if (smem > 48 * 1024)                                                                                                 \
      RB_CUDA_CHECK(cudaFuncSetAttribute(disentangle_softmax_kernel<T_>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                         static_cast<int>(smem)));                                                        \
    disentangle_softmax_kernel<T_><<<static_cast<unsigned>(rows), 256, smem, st>>>(                                       \
        reinterpret_cast<const T_*>(qk), reinterpret_cast<const T_*>(c2p), reinterpret_cast<const T_*>(p2c), rel,         \
        reinterpret_cast<const unsigned char*>(mask), mask_stride_b, N, S, P, span, scale, reinterpret_cast<T_*>(probs),  \
        reinterpret_cast<T_*>(score));                                                                                    \
  } while (0)
  if (dtype == DT_F32) RB_DIS(float);
  else if (dtype == DT_F16) RB_DIS(__half);
  else if (dtype == DT_BF16) RB_DIS(__nv_bfloat16);
  else return -1;
#undef RB_DIS
  return static_cast<int>(cudaGetLastError());
}
