// Row-wise and data-movement kernels around HSTU attention:
//   layer-norm * gate (ln_mul / norm_multiply_dropout) forward + backward, relative attention bias
//   (time buckets / positions) forward + backward, jagged <-> padded, 2-D jagged concat / split,
//   reverse_sequence, 1-D gather + scatter-add, paged KV-cache append and the positions of new tokens.
// Specs: cust_op/ascendc_op/ai_core_op/{ln_mul,norm_multiply_dropout,relative_attn_bias_time,
// relative_attn_bias_pos,relative_attn_bias_backward,concat_2d_jagged,reverse_sequence,gather_for_rank1}/
// */README.md and inference/kvcache_manager/src/kernels/*.
#include <algorithm>

#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p) { return static_cast<float>(*p); }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v) { *p = static_cast<T>(v); }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

__device__ __forceinline__ float hash_u01(unsigned long long seed, unsigned long long idx) {
  unsigned long long x = idx * 0x9E3779B97F4A7C15ull + seed;
  x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
  return (static_cast<float>(x >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

// ------------------------------------------------------------------ LayerNorm(x) * u (* dropout mask)
// one warp per row; C <= 2048.  keep = 1 - dropout_ratio; mask regenerated from (seed, element index).
template <typename T>
__global__ void ln_mul_fwd_kernel(const T* __restrict__ x, const T* __restrict__ u, const float* __restrict__ gamma,
                                  const float* __restrict__ beta, T* __restrict__ out, float* __restrict__ mean_out,
                                  float* __restrict__ rstd_out, long long rows, int C, float eps, float drop,
                                  unsigned long long seed) {
  const int lane = threadIdx.x & 31;
  const long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (r >= rows) return;
  const T* xr = x + r * C;
  float s = 0.f, s2 = 0.f;
  for (int c = lane; c < C; c += 32) { const float v = ldf(xr + c); s += v; s2 += v * v; }
  s = rb::warp_sum(s); s2 = rb::warp_sum(s2);
  const float mean = s / C;
  const float rstd = rsqrtf(fmaxf(s2 / C - mean * mean, 0.f) + eps);
  if (lane == 0) { if (mean_out) mean_out[r] = mean; if (rstd_out) rstd_out[r] = rstd; }
  const float inv_keep = drop > 0.f ? 1.f / (1.f - drop) : 1.f;
  for (int c = lane; c < C; c += 32) {
    float y = ((ldf(xr + c) - mean) * rstd * gamma[c] + beta[c]) * (u ? ldf(u + r * C + c) : 1.f);
    if (drop > 0.f) y = hash_u01(seed, static_cast<unsigned long long>(r) * C + c) < drop ? 0.f : y * inv_keep;
    stf(out + r * C + c, y);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
ln_mul_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ u,
                  const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ mean,
                  const float* __restrict__ rstd, T* __restrict__ dx, T* __restrict__ du, float* __restrict__ dgamma,
                  float* __restrict__ dbeta, long long rows, int C, float drop, unsigned long long seed) {
  extern __shared__ float sm_ln[];          // [2][C] partial dgamma / dbeta of this block
  float* sg = sm_ln;
  float* sb = sm_ln + C;
  for (int c = threadIdx.x; c < 2 * C; c += blockDim.x) sm_ln[c] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const float inv_keep = drop > 0.f ? 1.f / (1.f - drop) : 1.f;
  for (long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps_total) {
    const float m = mean[r], rs = rstd[r];
    float a = 0.f, b = 0.f;
    for (int c = lane; c < C; c += 32) {
      float g = ldf(dy + r * C + c);
      if (drop > 0.f) g = hash_u01(seed, static_cast<unsigned long long>(r) * C + c) < drop ? 0.f : g * inv_keep;
      const float xh = (ldf(x + r * C + c) - m) * rs;
      const float uu = u ? ldf(u + r * C + c) : 1.f;
      const float dn = g * uu * gamma[c];
      a += dn; b += dn * xh;
    }
    a = rb::warp_sum(a) / C; b = rb::warp_sum(b) / C;
    for (int c = lane; c < C; c += 32) {
      float g = ldf(dy + r * C + c);
      if (drop > 0.f) g = hash_u01(seed, static_cast<unsigned long long>(r) * C + c) < drop ? 0.f : g * inv_keep;
      const float xh = (ldf(x + r * C + c) - m) * rs;
      const float uu = u ? ldf(u + r * C + c) : 1.f;
      const float n = xh * gamma[c] + beta[c];
      const float dn = g * uu;
      stf(dx + r * C + c, rs * (dn * gamma[c] - a - xh * b));
      if (du) stf(du + r * C + c, g * n);
      atomicAdd(sg + c, dn * xh);
      atomicAdd(sb + c, dn);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) { atomicAdd(dgamma + c, sg[c]); atomicAdd(dbeta + c, sb[c]); }
}

// bf16, C = NCH * 256 (256 or 512): every lane keeps its 8 * NCH columns of the row packed in registers (one 16-byte load per
// tensor and chunk), so each input is read once; the per-column dgamma / dbeta partial sums live in a per-warp slice of shared
// memory (a lane owns its columns, so no atomics) and are combined once per block.
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

template <int NCH, bool DROP>
__global__ void __launch_bounds__(128, 4)
ln_mul_bwd_vec_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ u,
                      const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ mean,
                      const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ du,
                      float* __restrict__ dgamma, float* __restrict__ dbeta, long long rows, float drop, unsigned long long seed) {
  constexpr int C = NCH * 256;
  __shared__ __align__(16) float acc[4][2][C];      // per warp: dgamma / dbeta partial sums (a lane owns its columns)
  __shared__ __align__(16) float gb[2][C];          // gamma, beta
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const float inv_keep = DROP ? 1.f / (1.f - drop) : 1.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) { gb[0][c] = gamma[c]; gb[1][c] = beta[c]; }
  for (int c = threadIdx.x; c < 4 * 2 * C; c += blockDim.x) (&acc[0][0][0])[c] = 0.f;
  __syncthreads();
  for (long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps_total) {
    uint4 pg[NCH], px[NCH], pu[NCH];                // the row stays packed (bf16) in registers between the two passes
    const float m = mean[r], rs = rstd[r];
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const long long e0 = r * C + k * 256 + lane * 8;
      pg[k] = *reinterpret_cast<const uint4*>(dy + e0);
      px[k] = *reinterpret_cast<const uint4*>(x + e0);
      pu[k] = u ? *reinterpret_cast<const uint4*>(u + e0) : make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
    }
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      float g[8], xh[8], uu[8];
      unpack8(pg[k], g); unpack8(px[k], xh); unpack8(pu[k], uu);
      const float4 g0 = *reinterpret_cast<const float4*>(&gb[0][k * 256 + lane * 8]);
      const float4 g1 = *reinterpret_cast<const float4*>(&gb[0][k * 256 + lane * 8 + 4]);
      const float gm[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (DROP) {
          const unsigned long long e = static_cast<unsigned long long>(r) * C + k * 256 + lane * 8 + i;
          g[i] = hash_u01(seed, e) < drop ? 0.f : g[i] * inv_keep;
        }
        const float dng = g[i] * uu[i] * gm[i];
        a += dng;
        b += dng * (xh[i] - m) * rs;
      }
    }
    a = rb::warp_sum(a) * (1.f / C); b = rb::warp_sum(b) * (1.f / C);
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c0 = k * 256 + lane * 8;
      const long long e0 = r * C + c0;
      float g[8], xh[8], uu[8], o[8], q[8], sg[8], sb[8];
      unpack8(pg[k], g); unpack8(px[k], xh); unpack8(pu[k], uu);
      const float4 g0 = *reinterpret_cast<const float4*>(&gb[0][c0]), g1 = *reinterpret_cast<const float4*>(&gb[0][c0 + 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&gb[1][c0]), b1 = *reinterpret_cast<const float4*>(&gb[1][c0 + 4]);
      const float gm[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      const float bt[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      float4* ag = reinterpret_cast<float4*>(&acc[warp][0][c0]);
      float4* ab = reinterpret_cast<float4*>(&acc[warp][1][c0]);
      const float4 s0 = ag[0], s1 = ag[1], t0 = ab[0], t1 = ab[1];
      sg[0] = s0.x; sg[1] = s0.y; sg[2] = s0.z; sg[3] = s0.w; sg[4] = s1.x; sg[5] = s1.y; sg[6] = s1.z; sg[7] = s1.w;
      sb[0] = t0.x; sb[1] = t0.y; sb[2] = t0.z; sb[3] = t0.w; sb[4] = t1.x; sb[5] = t1.y; sb[6] = t1.z; sb[7] = t1.w;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (DROP) {
          const unsigned long long e = static_cast<unsigned long long>(r) * C + c0 + i;
          g[i] = hash_u01(seed, e) < drop ? 0.f : g[i] * inv_keep;
        }
        const float xn = (xh[i] - m) * rs;
        const float dn = g[i] * uu[i];
        o[i] = rs * (dn * gm[i] - a - xn * b);
        q[i] = g[i] * (xn * gm[i] + bt[i]);
        sg[i] += dn * xn;
        sb[i] += dn;
      }
      *reinterpret_cast<uint4*>(dx + e0) = pack8(o);
      if (du) *reinterpret_cast<uint4*>(du + e0) = pack8(q);
      ag[0] = make_float4(sg[0], sg[1], sg[2], sg[3]); ag[1] = make_float4(sg[4], sg[5], sg[6], sg[7]);
      ab[0] = make_float4(sb[0], sb[1], sb[2], sb[3]); ab[1] = make_float4(sb[4], sb[5], sb[6], sb[7]);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    atomicAdd(dgamma + c, acc[0][0][c] + acc[1][0][c] + acc[2][0][c] + acc[3][0][c]);
    atomicAdd(dbeta + c, acc[0][1][c] + acc[1][1][c] + acc[2][1][c] + acc[3][1][c]);
  }
}

// ------------------------------------------------------------------ relative attention bias
__device__ __forceinline__ int time_bucket(float dt, float divisor, int num_buckets) {
  const float a = fminf(fmaxf(fabsf(dt), 1.f), 7.0e16f);          // clamp(|dt|, 1, e^(129*0.301))
  int b = static_cast<int>(floorf(__logf(a) / divisor));
  return min(max(b, 0), num_buckets);
}
// out[l, b, i, j] = w[l, bucket(ts[b,i] - ts[b,j])]; optional bucket output [b, i, j]
__global__ void rab_time_fwd_kernel(const float* __restrict__ ts, const float* __restrict__ w, int L, int B, int S,
                                    int num_buckets, float divisor, float* __restrict__ out, int* __restrict__ bucket_out) {
  const long long total = static_cast<long long>(B) * S * S;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(e % S);
    const int i = static_cast<int>((e / S) % S);
    const int b = static_cast<int>(e / (static_cast<long long>(S) * S));
    const int bk = time_bucket(ts[b * S + i] - ts[b * S + j], divisor, num_buckets);
    if (bucket_out) bucket_out[e] = bk;
    for (int l = 0; l < L; ++l) out[l * total + e] = w[l * (num_buckets + 1) + bk];
  }
}
// dw[l, bucket] += grad[l, e]
__global__ void rab_time_bwd_kernel(const float* __restrict__ grad, const int* __restrict__ buckets, int L, long long per_layer,
                                    int num_buckets, float* __restrict__ dw) {
  extern __shared__ float sm_b[];           // [L][num_buckets+1]
  const int nb1 = num_buckets + 1;
  for (int c = threadIdx.x; c < L * nb1; c += blockDim.x) sm_b[c] = 0.f;
  __syncthreads();
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < per_layer;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int bk = buckets[e];
    for (int l = 0; l < L; ++l) atomicAdd(sm_b + l * nb1 + bk, grad[l * per_layer + e]);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < L * nb1; c += blockDim.x) atomicAdd(dw + c, sm_b[c]);
}
// out[b,i,j] = bias[min(i, v_b)][j] * (1 - id[i][j]) + id[i][j] * bias[0][0], cropped to [s, s]
__global__ void rab_pos_kernel(const float* __restrict__ bias, int S, const float* __restrict__ identity, int s,
                               const int* __restrict__ valid_lens, int B, float* __restrict__ out) {
  const long long total = static_cast<long long>(B) * s * s;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(e % s);
    const int i = static_cast<int>((e / s) % s);
    const int b = static_cast<int>(e / (static_cast<long long>(s) * s));
    const int v = valid_lens[b];
    const int ii = i >= v ? min(v, S - 1) : i;
    const float id = identity[i * s + j];
    out[e] = bias[ii * S + j] * (1.f - id) + id * bias[0];
  }
}

// ------------------------------------------------------------------ jagged data movement
// element-wise over [sum(len), D]; offsets [B+1]
template <typename T>
__global__ void jagged_to_padded_kernel(const T* __restrict__ values, const long long* __restrict__ offsets, int B, int max_len,
                                        int D, T* __restrict__ out, float pad) {
  const long long total = static_cast<long long>(B) * max_len * D;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int d = static_cast<int>(e % D);
    const int t = static_cast<int>((e / D) % max_len);
    const int b = static_cast<int>(e / (static_cast<long long>(D) * max_len));
    const long long len = offsets[b + 1] - offsets[b];
    if (t < len) out[e] = values[(offsets[b] + t) * D + d]; else stf(out + e, pad);
  }
}
template <typename T>
__global__ void padded_to_jagged_kernel(const T* __restrict__ padded, const long long* __restrict__ offsets, int B, int max_len,
                                        int D, T* __restrict__ values) {
  const long long total = static_cast<long long>(B) * max_len * D;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int d = static_cast<int>(e % D);
    const int t = static_cast<int>((e / D) % max_len);
    const int b = static_cast<int>(e / (static_cast<long long>(D) * max_len));
    if (t < offsets[b + 1] - offsets[b]) values[(offsets[b] + t) * D + d] = padded[e];
  }
}
// out rows of sample b = [A rows of b | B rows of b]; direction 0 = concat, 1 = split (out -> A, B)
template <typename T>
__global__ void concat_2d_jagged_kernel(T* __restrict__ a, T* __restrict__ bb, const long long* __restrict__ off_a,
                                        const long long* __restrict__ off_b, int B, int D, T* __restrict__ out, int split) {
  const int b = blockIdx.x;
  if (b >= B) return;
  const long long la = off_a[b + 1] - off_a[b], lb = off_b[b + 1] - off_b[b];
  const long long o0 = off_a[b] + off_b[b];
  const long long n = (la + lb) * D;
  for (long long e = threadIdx.x; e < n; e += blockDim.x) {
    const long long row = e / D;
    const int d = static_cast<int>(e % D);
    T* other = row < la ? a + (off_a[b] + row) * D + d : bb + (off_b[b] + row - la) * D + d;
    if (split) *other = out[(o0 + row) * D + d]; else out[(o0 + row) * D + d] = *other;
  }
}
// out[b, t, :] = in[b, len_b - 1 - t, :] for t < len_b, else copy
template <typename T>
__global__ void reverse_sequence_kernel(const T* __restrict__ in, const long long* __restrict__ lens, int B, int S, int D,
                                        T* __restrict__ out) {
  const long long total = static_cast<long long>(B) * S * D;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int d = static_cast<int>(e % D);
    const int t = static_cast<int>((e / D) % S);
    const int b = static_cast<int>(e / (static_cast<long long>(D) * S));
    const long long len = lens[b];
    const long long src = t < len ? len - 1 - t : t;
    out[e] = in[(static_cast<long long>(b) * S + src) * D + d];
  }
}
__global__ void gather1d_kernel(const float* __restrict__ x, const long long* __restrict__ idx, long long n, float* __restrict__ out) {
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < n;
       e += static_cast<long long>(gridDim.x) * blockDim.x) out[e] = x[idx[e]];
}
__global__ void scatter_add1d_kernel(const float* __restrict__ g, const long long* __restrict__ idx, long long n, float* __restrict__ dx) {
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < n;
       e += static_cast<long long>(gridDim.x) * blockDim.x) atomicAdd(dx + idx[e], g[e]);
}

// ------------------------------------------------------------------ paged KV cache
// cache layout [pages][2][page_size][H*D]; new K/V rows [nnz][H*D]; one 16-byte lane per thread
__global__ void kv_append_kernel(const uint4* __restrict__ k, const uint4* __restrict__ v, const int* __restrict__ batch_idx,
                                 const int* __restrict__ positions, const int* __restrict__ page_ids,
                                 const int* __restrict__ page_indptr, int nnz, int page_size, int vec_per_row,
                                 uint4* __restrict__ cache) {
  const long long total = static_cast<long long>(nnz) * vec_per_row;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(e / vec_per_row), c = static_cast<int>(e % vec_per_row);
    const int b = batch_idx[i], pos = positions[i];
    const long long page = page_ids[page_indptr[b] + pos / page_size];
    const int slot = pos % page_size;
    const long long base = (page * 2) * page_size * vec_per_row + static_cast<long long>(slot) * vec_per_row + c;
    cache[base] = k[e];
    cache[base + static_cast<long long>(page_size) * vec_per_row] = v[e];
  }
}
// batch index and absolute position of every new token: one block per sequence
__global__ void kv_positions_kernel(const int* __restrict__ new_offsets, const int* __restrict__ total_lens, int B,
                                    int* __restrict__ batch_idx, int* __restrict__ positions) {
  const int b = blockIdx.x;
  if (b >= B) return;
  const int beg = new_offsets[b], end = new_offsets[b + 1];
  const int first = total_lens[b] - (end - beg);
  for (int t = beg + threadIdx.x; t < end; t += blockDim.x) { batch_idx[t] = b; positions[t] = first + (t - beg); }
}

inline int grid1d(long long n, int num_sms) {
  long long b = (n + 255) / 256;
  const long long cap = static_cast<long long>(num_sms > 0 ? num_sms : 148) * 8;
  if (b > cap) b = cap;
  return static_cast<int>(b < 1 ? 1 : b);
}

}  // namespace

#define RB_T_DISPATCH(dt, ...)                                          \
  switch (dt) {                                                          \
    case 0: { using T = float; __VA_ARGS__; } break;                     \
    case 1: { using T = __half; __VA_ARGS__; } break;                    \
    case 2: { using T = __nv_bfloat16; __VA_ARGS__; } break;             \
    default: return -1;                                                  \
  }

RB_API int rb_ln_mul_fwd(const void* x, const void* u, const float* gamma, const float* beta, void* out, float* mean,
                         float* rstd, long long rows, int C, float eps, float drop, long long seed, int dtype,
                         cudaStream_t st) {
  if (rows == 0) return 0;
  const long long blocks = (rows * 32 + 255) / 256;
  if (dtype == 0)
    ln_mul_fwd_kernel<float><<<blocks, 256, 0, st>>>((const float*)x, (const float*)u, gamma, beta, (float*)out, mean, rstd, rows, C, eps, drop, (unsigned long long)seed);
  else if (dtype == 2)
    ln_mul_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)u, gamma, beta, (__nv_bfloat16*)out, mean, rstd, rows, C, eps, drop, (unsigned long long)seed);
  else return -1;
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_ln_mul_bwd(const void* dy, const void* x, const void* u, const float* gamma, const float* beta,
                         const float* mean, const float* rstd, void* dx, void* du, float* dgamma, float* dbeta,
                         long long rows, int C, float drop, long long seed, int dtype, int num_sms, cudaStream_t st) {
  if (rows == 0) return 0;
  const int blocks = (num_sms > 0 ? num_sms : 148) * 2;
  const size_t smem = sizeof(float) * 2 * C;
  auto al16 = [](const void* p) { return (reinterpret_cast<unsigned long long>(p) & 15ull) == 0; };
  if (dtype == 2 && (C == 256 || C == 512) && al16(dy) && al16(x) && al16(u) && al16(dx) && al16(du)) {
    const __nv_bfloat16 *pdy = (const __nv_bfloat16*)dy, *px = (const __nv_bfloat16*)x, *pu = (const __nv_bfloat16*)u;
    __nv_bfloat16 *pdx = (__nv_bfloat16*)dx, *pdu = (__nv_bfloat16*)du;
    const int vb = static_cast<int>(std::min<long long>((num_sms > 0 ? num_sms : 148) * 4LL, (rows + 3) / 4));
    const unsigned long long sd = (unsigned long long)seed;
#define RB_LN_BWD(NCH_, DROP_) ln_mul_bwd_vec_kernel<NCH_, DROP_><<<vb, 128, 0, st>>>(pdy, px, pu, gamma, beta, mean, rstd, pdx, pdu, dgamma, dbeta, rows, drop, sd)
    if (C == 256) { if (drop > 0.f) RB_LN_BWD(1, true); else RB_LN_BWD(1, false); }
    else { if (drop > 0.f) RB_LN_BWD(2, true); else RB_LN_BWD(2, false); }
#undef RB_LN_BWD
    return static_cast<int>(cudaGetLastError());
  }
  if (dtype == 0)
    ln_mul_bwd_kernel<float><<<blocks, 256, smem, st>>>((const float*)dy, (const float*)x, (const float*)u, gamma, beta, mean, rstd, (float*)dx, (float*)du, dgamma, dbeta, rows, C, drop, (unsigned long long)seed);
  else if (dtype == 2)
    ln_mul_bwd_kernel<__nv_bfloat16><<<blocks, 256, smem, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)u, gamma, beta, mean, rstd, (__nv_bfloat16*)dx, (__nv_bfloat16*)du, dgamma, dbeta, rows, C, drop, (unsigned long long)seed);
  else return -1;
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_rab_time_fwd(const float* ts, const float* w, int L, int B, int S, int num_buckets, float divisor,
                           float* out, int* bucket_out, int num_sms, cudaStream_t st) {
  const long long total = static_cast<long long>(B) * S * S;
  if (total == 0) return 0;
  rab_time_fwd_kernel<<<grid1d(total, num_sms), 256, 0, st>>>(ts, w, L, B, S, num_buckets, divisor, out, bucket_out);
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_rab_time_bwd(const float* grad, const int* buckets, int L, long long per_layer, int num_buckets, float* dw,
                           int num_sms, cudaStream_t st) {
  if (per_layer == 0) return 0;
  rab_time_bwd_kernel<<<grid1d(per_layer, num_sms), 256, sizeof(float) * L * (num_buckets + 1), st>>>(grad, buckets, L, per_layer, num_buckets, dw);
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_rab_pos(const float* bias, int S, const float* identity, int s, const int* valid_lens, int B, float* out,
                      int num_sms, cudaStream_t st) {
  const long long total = static_cast<long long>(B) * s * s;
  if (total == 0) return 0;
  rab_pos_kernel<<<grid1d(total, num_sms), 256, 0, st>>>(bias, S, identity, s, valid_lens, B, out);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_jagged_to_padded(const void* values, const long long* offsets, int B, int max_len, int D, void* out,
                               float pad, int dtype, int num_sms, cudaStream_t st) {
  const long long total = static_cast<long long>(B) * max_len * D;
  if (total == 0) return 0;
  RB_T_DISPATCH(dtype, jagged_to_padded_kernel<T><<<grid1d(total, num_sms), 256, 0, st>>>((const T*)values, offsets, B, max_len, D, (T*)out, pad))
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_padded_to_jagged(const void* padded, const long long* offsets, int B, int max_len, int D, void* values,
                               int dtype, int num_sms, cudaStream_t st) {
  const long long total = static_cast<long long>(B) * max_len * D;
  if (total == 0) return 0;
  RB_T_DISPATCH(dtype, padded_to_jagged_kernel<T><<<grid1d(total, num_sms), 256, 0, st>>>((const T*)padded, offsets, B, max_len, D, (T*)values))
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_concat_2d_jagged(void* a, void* b, const long long* off_a, const long long* off_b, int B, int D, void* out,
                               int split, int dtype, cudaStream_t st) {
  if (B == 0) return 0;
  RB_T_DISPATCH(dtype, concat_2d_jagged_kernel<T><<<B, 256, 0, st>>>((T*)a, (T*)b, off_a, off_b, B, D, (T*)out, split))
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_reverse_sequence(const void* in, const long long* lens, int B, int S, int D, void* out, int dtype,
                               int num_sms, cudaStream_t st) {
  const long long total = static_cast<long long>(B) * S * D;
  if (total == 0) return 0;
  RB_T_DISPATCH(dtype, reverse_sequence_kernel<T><<<grid1d(total, num_sms), 256, 0, st>>>((const T*)in, lens, B, S, D, (T*)out))
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_gather1d(const float* x, const long long* idx, long long n, float* out, int num_sms, cudaStream_t st) {
  if (n == 0) return 0;
  gather1d_kernel<<<grid1d(n, num_sms), 256, 0, st>>>(x, idx, n, out);
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_scatter_add1d(const float* g, const long long* idx, long long n, float* dx, int num_sms, cudaStream_t st) {
  if (n == 0) return 0;
  scatter_add1d_kernel<<<grid1d(n, num_sms), 256, 0, st>>>(g, idx, n, dx);
  return static_cast<int>(cudaGetLastError());
}

// k, v: [nnz][row_bytes] 16-bit rows (row_bytes % 16 == 0); cache: [pages][2][page_size][row_bytes]
RB_API int rb_kv_append_paged(const void* k, const void* v, const int* batch_idx, const int* positions,
                              const int* page_ids, const int* page_indptr, int nnz, int page_size, long long row_bytes,
                              void* cache, int num_sms, cudaStream_t st) {
  if (nnz == 0) return 0;
  if (row_bytes % 16) return -1;
  const int vpr = static_cast<int>(row_bytes / 16);
  kv_append_kernel<<<grid1d(static_cast<long long>(nnz) * vpr, num_sms), 256, 0, st>>>(
      (const uint4*)k, (const uint4*)v, batch_idx, positions, page_ids, page_indptr, nnz, page_size, vpr, (uint4*)cache);
  return static_cast<int>(cudaGetLastError());
}
RB_API int rb_kv_positions(const int* new_offsets, const int* total_lens, int B, int* batch_idx, int* positions,
                           cudaStream_t st) {
  if (B == 0) return 0;
  kv_positions_kernel<<<B, 256, 0, st>>>(new_offsets, total_lens, B, batch_idx, positions);
  return static_cast<int>(cudaGetLastError());
}
