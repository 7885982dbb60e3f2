// Pairwise dot-product feature interaction (DLRM) forward and backward.
//
// The interaction input is X = [X0 | XS] with X0 [B, D] the bottom-MLP output (feature 0) and
// XS [B, (F-1)*D] the pooled embeddings exactly as the embedding-lookup kernel wrote them; the
// two are read from their own buffers, so no concatenation pass exists.  The forward writes the top-MLP
// input row  R[b] = [ X[b,0,:] | <X_i, X_j> for 0 <= j < i < F | zero pad ]  and the backward
// turns dR into dX.  One warp owns one sample: the F x F Gram matrix is far too small for a
// tcgen05 tile (F = 27), so it is computed with per-warp mma.sync m16n8k16 tiles out of shared
// memory; the kernel is bound by the HBM traffic of X, not by math.
//
// The reference has no interaction operator (its models live outside the tree); the math is the
// standard DLRM dot interaction.
#include <mma.h>

#include "common.cuh"

namespace {

constexpr int FMAX = 32;  // features padded to two m16 tiles

// 16-byte asynchronous global -> shared copy (no register staging: a warp keeps its whole tile in flight)
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(rb::smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
               : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <int D>
struct Lay {
  static constexpr int XS = D + 8;               // padded row stride (elements) of X in smem
  static constexpr int X_ELEMS = FMAX * XS;
  static constexpr int ZS = 40;                  // padded row stride of the 32x32 dZ tile
};

// ------------------------------- forward -----------------------------------
template <int D, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
interaction_fwd_kernel(const __nv_bfloat16* __restrict__ X0, long long ld0, const __nv_bfloat16* __restrict__ XS,
                       long long lds, int B, int F, __nv_bfloat16* __restrict__ R, long long ldr, int out_cols) {
  using L = Lay<D>;
  extern __shared__ __align__(16) uint8_t smem_i[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_i) + warp * (L::X_ELEMS + 512);
  __nv_bfloat16* tri = xs + L::X_ELEMS;
  // rows F..31 stay zero for the whole kernel
  for (int i = lane; i < (FMAX - F) * L::XS / 2; i += 32)
    reinterpret_cast<uint32_t*>(xs + F * L::XS)[i] = 0u;
  const int n_tri = F * (F - 1) / 2;
  constexpr int VPR = D / 8;  // uint4 per row
  for (int b = blockIdx.x * WARPS + warp; b < B; b += gridDim.x * WARPS) {
    const uint4* src0 = reinterpret_cast<const uint4*>(X0 + static_cast<long long>(b) * ld0);
    const uint4* src = reinterpret_cast<const uint4*>(XS + static_cast<long long>(b) * lds);
    __syncwarp();
    for (int i = lane; i < F * VPR; i += 32) {
      const int r = i / VPR, c = i % VPR;
      cp_async16(xs + r * L::XS + c * 8, (r == 0) ? (src0 + c) : (src + i - VPR));
    }
    cp_async_wait_all();
    __syncwarp();
    float acc[2][4][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;
#pragma unroll 4
    for (int k = 0; k < D / 16; ++k) {
      uint32_t a[2][4], bf[4][2];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
        ldmatrix_x4(a[mt], rb::smem_u32(xs + (mt * 16 + (lane & 15)) * L::XS + k * 16 + (lane >> 4) * 8));
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
        ldmatrix_x2(bf[nt], rb::smem_u32(xs + (nt * 8 + (lane & 7)) * L::XS + k * 16 + ((lane >> 3) & 1) * 8));
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        if (nt < 2) mma_bf16(acc[0][nt], a[0], bf[nt]);
        mma_bf16(acc[1][nt], a[1], bf[nt]);
      }
    }
    // strictly-lower triangle -> packed order i*(i-1)/2 + j
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = mt * 16 + (lane >> 2) + (i >> 1) * 8;
          const int col = nt * 8 + (lane & 3) * 2 + (i & 1);
          if (row < F && col < row) tri[row * (row - 1) / 2 + col] = __float2bfloat16(acc[mt][nt][i]);
        }
    __syncwarp();
    __nv_bfloat16* o = R + static_cast<long long>(b) * ldr;
    for (int i = lane; i < VPR; i += 32)
      *reinterpret_cast<uint4*>(o + i * 8) = *reinterpret_cast<const uint4*>(xs + i * 8);
    for (int i = lane; i < out_cols - D; i += 32) o[D + i] = (i < n_tri) ? tri[i] : __float2bfloat16(0.f);
  }
}

// ------------------------------- backward ----------------------------------
// Per warp: X tile (also the output staging: the dX columns of an n-tile overwrite the X columns
// that only that n-tile reads), the packed dR row and the symmetric 32x32 dZ tile.
template <int D, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
interaction_bwd_kernel(const __nv_bfloat16* __restrict__ X0, long long ld0, const __nv_bfloat16* __restrict__ XS,
                       long long lds, const __nv_bfloat16* __restrict__ dR, long long ldr, int dr_cols, int B, int F,
                       __nv_bfloat16* __restrict__ dX0, long long ldd0, __nv_bfloat16* __restrict__ dXS,
                       long long ldds, int mask_x0) {
  using L = Lay<D>;
  extern __shared__ __align__(16) uint8_t smem_i[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int GS = D + 512;                       // dR row: D direct columns + up to 496 pair terms
  constexpr int PER_WARP = L::X_ELEMS + FMAX * L::ZS + GS;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_i) + warp * PER_WARP;
  __nv_bfloat16* zs = xs + L::X_ELEMS;
  __nv_bfloat16* gs = zs + FMAX * L::ZS;
  constexpr int VPR = D / 8;
  const int g_vec = (dr_cols + 7) / 8;
  for (int b = blockIdx.x * WARPS + warp; b < B; b += gridDim.x * WARPS) {
    const uint4* src0 = reinterpret_cast<const uint4*>(X0 + static_cast<long long>(b) * ld0);
    const uint4* src = reinterpret_cast<const uint4*>(XS + static_cast<long long>(b) * lds);
    const uint4* g4 = reinterpret_cast<const uint4*>(dR + static_cast<long long>(b) * ldr);
    __syncwarp();
    for (int i = lane; i < F * VPR; i += 32) {
      const int r = i / VPR, c = i % VPR;
      cp_async16(xs + r * L::XS + c * 8, (r == 0) ? (src0 + c) : (src + i - VPR));
    }
    for (int i = lane; i < g_vec; i += 32) cp_async16(reinterpret_cast<uint4*>(gs) + i, g4 + i);
    for (int i = lane; i < (FMAX - F) * L::XS / 2; i += 32)
      reinterpret_cast<uint32_t*>(xs + F * L::XS)[i] = 0u;       // padding rows (the tile is reused as output)
    cp_async_wait_all();
    __syncwarp();
    // symmetric dZ tile: zs[i][j] = dtri(max(i,j), min(i,j)), zero on the diagonal / padding
    for (int e = lane; e < FMAX * FMAX; e += 32) {
      const int i = e >> 5, j = e & 31;
      __nv_bfloat16 v = __float2bfloat16(0.f);
      if (i < F && j < F && i != j) {
        const int hi = i > j ? i : j, lo = i > j ? j : i;
        v = gs[D + hi * (hi - 1) / 2 + lo];
      }
      zs[i * L::ZS + j] = v;
    }
    __syncwarp();
    uint32_t a[2][2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int k = 0; k < 2; ++k)
        ldmatrix_x4(a[mt][k], rb::smem_u32(zs + (mt * 16 + (lane & 15)) * L::ZS + k * 16 + (lane >> 4) * 8));
#pragma unroll 2
    for (int nt = 0; nt < D / 8; ++nt) {
      float acc[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        uint32_t bf[2];
        ldmatrix_x2_trans(bf, rb::smem_u32(xs + (k * 16 + (lane & 15)) * L::XS + nt * 8));
        mma_bf16(acc[0], a[0][k], bf);
        mma_bf16(acc[1], a[1][k], bf);
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int row = mt * 16 + (lane >> 2) + h * 8;
          const int col = nt * 8 + (lane & 3) * 2;
          float v0 = acc[mt][2 * h], v1 = acc[mt][2 * h + 1];
          uint32_t* slot = reinterpret_cast<uint32_t*>(xs + row * L::XS + col);
          if (row == 0) {  // the dense feature also feeds the first D columns of R directly
            v0 += __bfloat162float(gs[col]);
            v1 += __bfloat162float(gs[col + 1]);
            if (mask_x0) {   // feature 0 is a ReLU output: hand back d(pre-activation)
              const float2 x = rb::unpack_bf16(*slot);
              v0 = x.x > 0.f ? v0 : 0.f;
              v1 = x.y > 0.f ? v1 : 0.f;
            }
          }
          *slot = rb::pack_bf16(v0, v1);
        }
    }
    __syncwarp();
    uint4* dst0 = reinterpret_cast<uint4*>(dX0 + static_cast<long long>(b) * ldd0);
    uint4* dst = reinterpret_cast<uint4*>(dXS + static_cast<long long>(b) * ldds);
    for (int i = lane; i < F * VPR; i += 32) {
      const int r = i / VPR, c = i % VPR;
      const uint4 v = *reinterpret_cast<const uint4*>(xs + r * L::XS + c * 8);
      if (r == 0) dst0[c] = v; else dst[i - VPR] = v;
    }
  }
}

template <int D>
int launch_fwd(const void* X0, long long ld0, const void* XS, long long lds, int B, int F, void* R, long long ldr,
               int out_cols, int num_sms, cudaStream_t st) {
  constexpr int WARPS = 8;
  const int smem = WARPS * (Lay<D>::X_ELEMS + 512) * 2;
  static bool set = false;
  if (!set) {
    RB_CUDA_CHECK(cudaFuncSetAttribute(interaction_fwd_kernel<D, WARPS>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    set = true;
  }
  int blocks = (B + WARPS - 1) / WARPS;
  if (blocks > num_sms * 3) blocks = num_sms * 3;
  interaction_fwd_kernel<D, WARPS><<<blocks, WARPS * 32, smem, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(X0), ld0, reinterpret_cast<const __nv_bfloat16*>(XS), lds, B, F,
      reinterpret_cast<__nv_bfloat16*>(R), ldr, out_cols);
  return static_cast<int>(cudaGetLastError());
}
template <int D>
int launch_bwd(const void* X0, long long ld0, const void* XS, long long lds, const void* dR, long long ldr,
               int dr_cols, int B, int F, void* dX0, long long ldd0, void* dXS, long long ldds, int mask_x0,
               int num_sms, cudaStream_t st) {
  constexpr int WARPS = 8;
  const int smem = WARPS * (Lay<D>::X_ELEMS + FMAX * Lay<D>::ZS + D + 512) * 2;
  if (dr_cols > D + 512 || (ldr % 8)) return -3;
  static bool set = false;
  if (!set) {
    RB_CUDA_CHECK(cudaFuncSetAttribute(interaction_bwd_kernel<D, WARPS>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    set = true;
  }
  int blocks = (B + WARPS - 1) / WARPS;
  if (blocks > num_sms * 2) blocks = num_sms * 2;
  interaction_bwd_kernel<D, WARPS><<<blocks, WARPS * 32, smem, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(X0), ld0, reinterpret_cast<const __nv_bfloat16*>(XS), lds,
      reinterpret_cast<const __nv_bfloat16*>(dR), ldr, dr_cols, B, F, reinterpret_cast<__nv_bfloat16*>(dX0), ldd0,
      reinterpret_cast<__nv_bfloat16*>(dXS), ldds, mask_x0);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// X0 [B,D] (row stride ld0) and XS [B,(F-1)*D] (row stride lds), bf16 -> R [B, ldr] bf16 with
// out_cols >= D + F(F-1)/2 columns written.  Row strides must keep rows 16-byte aligned.
RB_API int rb_dot_interaction_fwd(const void* X0, long long ld0, const void* XS, long long lds, int B, int F,
                                  int D, void* R, long long ldr, int out_cols, int num_sms, cudaStream_t st) {
  if (B == 0) return 0;
  if (F > FMAX || F < 2) return -1;
  if (num_sms <= 0) num_sms = 148;
  switch (D) {
    case 16: return launch_fwd<16>(X0, ld0, XS, lds, B, F, R, ldr, out_cols, num_sms, st);
    case 32: return launch_fwd<32>(X0, ld0, XS, lds, B, F, R, ldr, out_cols, num_sms, st);
    case 64: return launch_fwd<64>(X0, ld0, XS, lds, B, F, R, ldr, out_cols, num_sms, st);
    case 128: return launch_fwd<128>(X0, ld0, XS, lds, B, F, R, ldr, out_cols, num_sms, st);
    case 256: return launch_fwd<256>(X0, ld0, XS, lds, B, F, R, ldr, out_cols, num_sms, st);
    default: return -2;
  }
}

// dR [B, dr_cols] (row stride ldr, a multiple of 8).  mask_x0 != 0: X0 is a ReLU output and dX0 is
// returned multiplied by (X0 > 0).
RB_API int rb_dot_interaction_bwd(const void* X0, long long ld0, const void* XS, long long lds, const void* dR,
                                  long long ldr, int dr_cols, int B, int F, int D, void* dX0, long long ldd0,
                                  void* dXS, long long ldds, int mask_x0, int num_sms, cudaStream_t st) {
  if (B == 0) return 0;
  if (F > FMAX || F < 2) return -1;
  if (num_sms <= 0) num_sms = 148;
  switch (D) {
    case 16: return launch_bwd<16>(X0, ld0, XS, lds, dR, ldr, dr_cols, B, F, dX0, ldd0, dXS, ldds, mask_x0, num_sms, st);
    case 32: return launch_bwd<32>(X0, ld0, XS, lds, dR, ldr, dr_cols, B, F, dX0, ldd0, dXS, ldds, mask_x0, num_sms, st);
    case 64: return launch_bwd<64>(X0, ld0, XS, lds, dR, ldr, dr_cols, B, F, dX0, ldd0, dXS, ldds, mask_x0, num_sms, st);
    case 128: return launch_bwd<128>(X0, ld0, XS, lds, dR, ldr, dr_cols, B, F, dX0, ldd0, dXS, ldds, mask_x0, num_sms, st);
    case 256: return launch_bwd<256>(X0, ld0, XS, lds, dR, ldr, dr_cols, B, F, dX0, ldd0, dXS, ldds, mask_x0, num_sms, st);
    default: return -2;
  }
}
