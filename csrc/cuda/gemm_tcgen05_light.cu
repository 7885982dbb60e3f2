// The light variant of the tcgen05 GEMM (same tiles, pipeline and epilogue math as gemm_tcgen05.cu): 256 threads, four
// epilogue warps that store their rows directly, no shared-memory staging - about 194 KB of shared memory and 40 K
// registers per CTA instead of 226 KB and the whole register file.  That leaves room on every SM for a block of a
// concurrent kernel, which is what the multi-GPU step needs: the embedding exchange runs on its own stream beside the
// bottom-MLP GEMMs, and with the full-size variant its blocks could only start at GEMM kernel boundaries (measured on
// 4 GPUs: 1.276 ms per DLRM-large step with this variant against 1.332 ms with the other one, while a single GPU runs
// 2.3 % faster on the other one).  rb_gemm16 forwards here while rb_gemm_set_concurrent(1) is in force.
#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;

enum Epi : int {
  EPI_BF16 = 0,        // out16 = acc (+bias)
  EPI_BF16_RELU = 1,   // out16 = relu(acc + bias)
  EPI_BF16_MASK = 2,   // out16 = acc * (aux > 0)        (ReLU backward fused into dX)
  EPI_F32_ATOMIC = 3,  // out32 += acc                   (split-K)
  EPI_BF16_SILU = 4,   // out16 = silu(acc + bias)
  EPI_F32 = 5,         // out32 = acc (+bias)
  EPI_BF16_DSILU = 6,  // out16 = acc * silu'(aux)       (SiLU backward fused into dX)
};

struct GemmParams {
  int M, N, K;
  int splits, kb_per_split;
  void* out;
  long long ldc;
  const float* bias;
  const void* aux;
  long long ld_aux;
  int epi;
  int is_bf16;
  float alpha;
  float* colsum;          // optional [N] fp32: += column sums of the epilogue's output values (bias gradients)
  int* status;
};

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : ((BN == 128) ? 6 : 8);
  static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;
  static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
};

__device__ __forceinline__ float to_f32_16(uint16_t raw, int is_bf16) {
  if (is_bf16) return __bfloat162float(__ushort_as_bfloat16(raw));
  return __half2float(__ushort_as_half(raw));
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(256, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
            const GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* tfull = empty + C::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      rb::mbar_init(&full[s], 1);
      rb::mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      rb::mbar_init(&tfull[b], 1);
      rb::mbar_init(&tempty[b], 128);
    }
    *abort_flag = 0;
    rb::mbar_fence_init();
    rb::tma_prefetch_desc(&tma_a);
    rb::tma_prefetch_desc(&tma_b);
  }
  if (warp == 2) {
    rb::tmem_alloc(tmem_slot, C::TMEM_COLS);
    rb::tmem_relinquish();
  }
  rb::tc_fence_before();
  __syncthreads();
  rb::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int total = tiles_m * tiles_n * p.splits;
  const int kb_total = (p.K + BK - 1) / BK;

  if (warp == 0 && lane == 0) {
    // ------------------------------ TMA producer ------------------------------
    int stage = 0;
    uint32_t phase = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x) {
      const int ks = w % p.splits;
      const int t = w / p.splits;
      const int tn = t % tiles_n, tm = t / tiles_n;
      const int kb0 = ks * p.kb_per_split;
      const int kb1 = min(kb_total, kb0 + p.kb_per_split);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!rb::mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status)) goto done;
        uint8_t* sa = smem + stage * C::STAGE_BYTES;
        uint8_t* sb = sa + C::A_BYTES;
        rb::mbar_expect_tx(&full[stage], C::STAGE_BYTES);
        if (A_MN) {
#pragma unroll
          for (int c = 0; c < BM / 64; ++c)
            rb::tma_load_2d(sa + c * (BK * 128), &tma_a, &full[stage], tm * BM + c * 64, kb * BK);
        } else {
          rb::tma_load_2d(sa, &tma_a, &full[stage], kb * BK, tm * BM);
        }
        if (B_MN) {
#pragma unroll
          for (int c = 0; c < BN / 64; ++c)
            rb::tma_load_2d(sb + c * (BK * 128), &tma_b, &full[stage], tn * BN + c * 64, kb * BK);
        } else {
          rb::tma_load_2d(sb, &tma_b, &full[stage], kb * BK, tn * BN);
        }
        if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------- MMA issuer -------------------------------
    const uint32_t idesc = rb::umma_idesc(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0, p.is_bf16);
    int stage = 0;
    uint32_t phase = 0;
    int acc_it = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x, ++acc_it) {
      const int ks = w % p.splits;
      const int kb0 = ks * p.kb_per_split;
      const int kb1 = min(kb_total, kb0 + p.kb_per_split);
      const int buf = acc_it & 1;
      const uint32_t acc_phase = (acc_it >> 1) & 1;
      if (!rb::mbar_wait(&tempty[buf], acc_phase ^ 1, abort_flag, p.status)) goto done;
      rb::tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * BN;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!rb::mbar_wait(&full[stage], phase, abort_flag, p.status)) goto done;
        rb::tc_fence_after();
        const uint32_t sa = rb::smem_u32(smem + stage * C::STAGE_BYTES);
        const uint32_t sb = sa + C::A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint64_t da = A_MN ? rb::umma_smem_desc(sa + k * 2048, BK * 128, 1024)
                                   : rb::umma_smem_desc(sa + k * 32, 16, 1024);
          const uint64_t db = B_MN ? rb::umma_smem_desc(sb + k * 2048, BK * 128, 1024)
                                   : rb::umma_smem_desc(sb + k * 32, 16, 1024);
          rb::umma_f16_ss(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        }
        rb::umma_commit(&empty[stage]);
        if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
      }
      rb::umma_commit(&tfull[buf]);
    }
  } else if (warp >= 4) {
    // -------------------------------- epilogue --------------------------------
    const int ew = warp & 3;
    int acc_it = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x, ++acc_it) {
      const int t = w / p.splits;
      const int tn = t % tiles_n, tm = t / tiles_n;
      const int buf = acc_it & 1;
      const uint32_t acc_phase = (acc_it >> 1) & 1;
      bool ok = rb::mbar_wait(&tfull[buf], acc_phase, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) goto done;
      rb::tc_fence_after();
      const long long m = static_cast<long long>(tm) * BM + ew * 32 + lane;
      const bool row_ok = m < p.M;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        rb::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + buf * BN + c * 32, r);
        rb::tmem_ld_wait();
        const int n0 = tn * BN + c * 32;
        if (n0 >= p.N || (!row_ok && p.colsum == nullptr)) continue;
        const bool full_chunk = (n0 + 32 <= p.N);
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        if (p.bias != nullptr) {
          if (full_chunk) {
            const float4* b4 = reinterpret_cast<const float4*>(p.bias + n0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 b = __ldg(b4 + j);
              v[4 * j] += b.x; v[4 * j + 1] += b.y; v[4 * j + 2] += b.z; v[4 * j + 3] += b.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + j < p.N) v[j] += __ldg(p.bias + n0 + j);
          }
        }
        if (p.epi == EPI_F32_ATOMIC) {
          float* o = reinterpret_cast<float*>(p.out) + m * p.ldc + n0;
          if (full_chunk && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) rb::red_add_v4(o + j, v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + j < p.N) atomicAdd(o + j, v[j]);
          }
          continue;
        }
        if (p.epi == EPI_F32) {
          float* o = reinterpret_cast<float*>(p.out) + m * p.ldc + n0;
          if (full_chunk && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              reinterpret_cast<float4*>(o)[j] =
                  make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + j < p.N) o[j] = v[j];
          }
          continue;
        }
        if (p.epi == EPI_BF16_RELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
        } else if (p.epi == EPI_BF16_SILU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = rb::silu_f(v[j]);
        } else if (p.epi == EPI_BF16_MASK || p.epi == EPI_BF16_DSILU) {
          const uint16_t* a = reinterpret_cast<const uint16_t*>(p.aux) + m * p.ld_aux + n0;
          uint16_t araw[32];
          if (!row_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) araw[j] = 0;
          } else if (full_chunk && ((reinterpret_cast<uintptr_t>(a) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              reinterpret_cast<uint4*>(araw)[j] = __ldg(reinterpret_cast<const uint4*>(a) + j);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) araw[j] = (n0 + j < p.N) ? a[j] : 0;
          }
          if (p.epi == EPI_BF16_MASK) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = (to_f32_16(araw[j], p.is_bf16) > 0.f) ? v[j] : 0.f;
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float x = to_f32_16(araw[j], p.is_bf16);
              const float s = rb::sigmoid_f(x);
              v[j] *= s * (1.f + x * (1.f - s));
            }
          }
        }
        if (p.colsum != nullptr) {
          // column sums over the warp's 32 rows by recursive halving: after the step of width w a lane keeps the w
          // columns selected by its lane bit; at the end lane l holds column l summed over all rows
          float cs[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) cs[j] = row_ok ? v[j] : 0.f;
#pragma unroll
          for (int w = 16; w >= 1; w >>= 1) {
            const bool upper = (lane & w) != 0;
#pragma unroll
            for (int j = 0; j < w; ++j) {
              const float send = upper ? cs[j] : cs[j + w];
              const float keep = upper ? cs[j + w] : cs[j];
              cs[j] = keep + __shfl_xor_sync(0xffffffffu, send, w);
            }
          }
          if (n0 + lane < p.N && cs[0] != 0.f) atomicAdd(p.colsum + n0 + lane, cs[0]);
          if (!row_ok) continue;
        }
        uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + m * p.ldc + n0;
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j)
          pk[j] = p.is_bf16 ? rb::pack_bf16(v[2 * j], v[2 * j + 1]) : rb::pack_f16(v[2 * j], v[2 * j + 1]);
        if (full_chunk && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            reinterpret_cast<uint4*>(o)[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (n0 + j < p.N) o[j] = static_cast<uint16_t>((pk[j >> 1] >> ((j & 1) * 16)) & 0xffff);
        }
      }
      rb::tc_fence_before();
      rb::mbar_arrive(&tempty[buf]);
    }
  }
done:
  __syncwarp();
  rb::tc_fence_before();
  __syncthreads();
  if (warp == 2) rb::tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
// 2-D row-major tensor [rows][cols] of 16-bit elements, 128-byte swizzled boxes.
int make_map_2d(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld,
                int box_cols, int box_rows, int is_bf16) {
  return rb_host::make_map_2d(map, base, rows, cols, ld, box_cols, box_rows, is_bf16 != 0);
}

template <int BN, bool A_MN, bool B_MN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t st) {
  using C = Cfg<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    RB_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<BN, A_MN, B_MN>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    attr_set = true;
  }
  gemm_kernel<BN, A_MN, B_MN><<<grid, 256, C::SMEM_BYTES, st>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// out[M,N] = epi(alpha * A * B^T).
//   a_mn == 0: A is [M][K] with row stride lda;  a_mn == 1: A is stored [K][M] with row stride lda.
//   b_mn == 0: B is [N][K] with row stride ldb;  b_mn == 1: B is stored [K][N] with row stride ldb.
// Row strides are in elements and must be multiples of 8; bases 16-byte aligned.
// Returns 0, a cudaError_t, or a negative value for an argument / descriptor error.
RB_API int rb_gemm16_light(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn,
                     void* out, long long ldc, int M, int N, int K, const float* bias, const void* aux,
                     long long ld_aux, int epi, float alpha, int splits, int is_bf16, int num_sms,
                     float* colsum, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (colsum != nullptr && (epi == EPI_F32_ATOMIC || epi == EPI_F32)) return -5;   // column sums ride on the 16-bit epilogues
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -3;
  const int bn = (N > 128) ? 256 : ((N > 64) ? 128 : 64);
  const int kb_total = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > kb_total) splits = kb_total;
  int kbps = (kb_total + splits - 1) / splits;
  splits = (kb_total + kbps - 1) / kbps;  // every split owns at least one k-block
  if (splits > 1 && epi != EPI_F32_ATOMIC) return -4;

  CUtensorMap ta, tb;
  int rc;
  if (a_mn) rc = make_map_2d(&ta, A, K, M, lda, 64, BK, is_bf16);
  else      rc = make_map_2d(&ta, A, M, K, lda, BK, BM, is_bf16);
  if (rc) return rc;
  if (b_mn) rc = make_map_2d(&tb, B, K, N, ldb, 64, BK, is_bf16);
  else      rc = make_map_2d(&tb, B, N, K, ldb, BK, bn, is_bf16);
  if (rc) return rc;

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.splits = splits; p.kb_per_split = kbps;
  p.out = out; p.ldc = ldc; p.bias = bias; p.aux = aux; p.ld_aux = ld_aux;
  p.epi = epi; p.is_bf16 = is_bf16; p.alpha = alpha; p.colsum = colsum; p.status = status;

  const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn) * splits;
  if (num_sms <= 0) num_sms = 148;
  const int grid = tiles < num_sms ? tiles : num_sms;

#define RB_DISPATCH(BN_)                                                                     \
  if (a_mn && b_mn) return launch<BN_, true, true>(ta, tb, p, grid, stream);                 \
  if (a_mn && !b_mn) return launch<BN_, true, false>(ta, tb, p, grid, stream);               \
  if (!a_mn && b_mn) return launch<BN_, false, true>(ta, tb, p, grid, stream);               \
  return launch<BN_, false, false>(ta, tb, p, grid, stream);
  if (bn == 256) { RB_DISPATCH(256) }
  if (bn == 128) { RB_DISPATCH(128) }
  RB_DISPATCH(64)
#undef RB_DISPATCH
}
