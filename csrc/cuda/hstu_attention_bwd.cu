// HSTU jagged SiLU attention, backward, on tcgen05 / TMEM (sm_100a), head dim 64.
//
// One CTA owns one (sequence, head, 128-key block), keeps its K and V tiles in shared memory and the
// dK / dV accumulators in TMEM, and walks the query blocks that attend to those keys.  Everything is
// computed in the transposed orientation (rows = keys), so that each activation thread owns one key row:
//
//   S^T  = K Q^T            tcgen05.mma (A = K smem, B = Q smem)                 -> TMEM
//   dP^T = V dO^T           tcgen05.mma (A = V smem, B = dO smem)                -> TMEM
//   x = alpha (S + bias);  P^T = SiLU(x) scale mask;  dS^T = dP^T scale mask alpha sigma(x)(1 + x(1 - sigma(x)))
//        written as packed bf16 over the S^T / dP^T columns they came from (tcgen05.st), dS^T also into
//        shared memory as an MN-major operand
//   dV  += P^T  dO          tcgen05.mma (A = P^T in TMEM,  B = dO smem, MN-major)
//   dK  += dS^T Q           tcgen05.mma (A = dS^T in TMEM, B = Q smem,  MN-major)
//   dQ_partial = dS K       tcgen05.mma (A = dS^T smem MN-major, B = K smem MN-major) -> TMEM -> fp32
//                           vector atomics into the dQ accumulator
// The bias gradients (dBias = dS) are reduced per CTA in shared memory - run-length per key row for the
// monotone time buckets, conflict-free atomics for the Toeplitz position table - and flushed once.
// Every mbarrier wait is bounded.
//
// Math: build/presmoke/hstu/hstu_common.py:387-477 of the reference; kernel structure is this library's.
#include "common.cuh"

namespace {

constexpr int BQ = 128, BKV = 128, D = 64;
constexpr int TILE = 128 * 128;            // bytes of one [128][64] bf16 tile

struct HstuBwdParams {
  const int* q_offsets; const int* k_offsets;
  int B, H;
  float alpha, scale;
  int causal;
  const int* num_context; const int* num_target; int target_group_size;
  const float* ts; const float* ts_w; int num_buckets; float ts_divisor;
  const float* pos_w; int pos_len;
  float* dq32; long long ld_dq;            // fp32 accumulator [Tq][ld_dq]
  void* dk; void* dv; long long ld_dkv;    // bf16 [Tk][ld_dkv]
  float* d_ts_w; float* d_pos_w;
  int bucket_cap;                          // min(num_buckets, floor(log(7e16) / divisor))
  int* status;
};

__device__ __forceinline__ bool attends(int pi, int j, int len, int causal, int nctx, int ntgt, int gs) {
  if (j >= len) return false;
  if (!causal) return true;
  bool ok = j <= pi;
  if (nctx > 0 && pi < nctx && j < len - ntgt) ok = true;
  if (ntgt > 0 && gs > 0) {
    const int t0 = len - ntgt;
    if (pi >= t0 && j >= t0) ok = (j <= pi) && ((pi - t0) / gs == (j - t0) / gs);
  }
  return ok;
}
using rb::red_add_v4;
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

constexpr int POS_HIST = 4096;
// The CTA-level bias-gradient histograms are 64-bit fixed point (value * 2^36): integer atomics on shared memory are a
// single instruction, while a float add there is a compare-and-swap loop that serialises on equal addresses.
constexpr float FIX_SCALE = 68719476736.f;
__device__ __forceinline__ void hist_add(long long* h, float v) {
  atomicAdd(reinterpret_cast<unsigned long long*>(h), static_cast<unsigned long long>(__float2ll_rn(v * FIX_SCALE)));
}
__device__ __forceinline__ float hist_value(long long h) { return static_cast<float>(static_cast<double>(h) * (1.0 / 68719476736.0)); }
constexpr int SMEM_BYTES = TILE * 8 /*K,V,2x(Q,dO),dS(2 chunks)*/ + 16 * 2 * 32 * 4 /*ts*/ + 768 /*ts_w*/ + 768 /*d ts_w*/ +
                           POS_HIST * 8 + 768 /*64-bit d ts_w*/ + 256 /*barriers*/ + 16 * 64 * 4 /*distance-bias windows*/ + 1024;

// One warp's 32 (keys, one per thread) x 32 (queries, e) chunk: S^T, dP^T -> P^T, dS^T (packed bf16) and the bias
// gradient partial sums.  With h = alpha (S + bias) / 2 and th = tanh(h):
//   P  = scale SiLU(2h)                 = hs + hs th,                hs = h scale
//   dS = dP scale alpha SiLU'(2h)       = dP (sg + sg g),            sg = scale alpha (1 + th) / 2,  g = h - h th
// dts: run-length sums per thread (the bucket of |ts_i - ts_j| changes slowly along a key row), kept across tiles;
// dpos: the chunk's anti-diagonals (i - j constant) are summed across lanes with one shuffle per element: lane o owns
//       diagonals o and o + 32 of the 63, element (e, lane) lies on diagonal e - lane + 31.
template <bool BT, bool BP, bool WDT, bool WDP, bool MASKED>
__device__ __forceinline__ void bwd_chunk(const uint32_t (&rs)[16], const uint32_t (&rd)[16], uint32_t* pk, uint32_t* dk16, int e0,
                                          int& run_bucket, float& run_sum, float ts_j, const float* my_ts, const float* tsw_s, long long* dtsw_s, const float* my_pos,
                                          int lane, float k_log, int cap, float half_alpha, float scale, float half_sa, int pi0,
                                          int i0, int j, int len_q, int len_k, int causal, int nctx, int ntgt, int gs,
                                          float& acc_lo, float& acc_hi) {
  // phase A: straight-line math for 16 elements (no branches, so the loads and MUFU ops of different elements overlap)
  uint32_t bkp[4] = {0u, 0u, 0u, 0u};                              // time buckets, one byte each
#pragma unroll
  for (int e = 0; e < 16; e += 2) {
    float pv[2], dsv[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int ee = e0 + e + q;                                   // query column inside the 32-wide chunk
      float s = __uint_as_float(rs[e + q]);
      if (BT) {
        const float a = fmaxf(fabsf(my_ts[ee] - ts_j), 1.f);
        const int bk = min(static_cast<int>(__log2f(a) * k_log), cap);
        s += tsw_s[bk];
        if (WDT) bkp[(e + q) >> 2] |= static_cast<uint32_t>(bk) << (8 * ((e + q) & 3));
      }
      if (BP) s += my_pos[ee + 31 - lane];
      const float h = s * half_alpha;
      float th;
      asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(h));
      const float hs = h * scale;
      float pval = fmaf(hs, th, hs);
      const float g = fmaf(-h, th, h);
      const float sg = fmaf(half_sa, th, half_sa);
      float ds = __uint_as_float(rd[e + q]) * fmaf(sg, g, sg);
      if (MASKED) {
        const bool on = (i0 + ee < len_q) && attends(pi0 + ee, j, len_k, causal, nctx, ntgt, gs);
        pval = on ? pval : 0.f;
        ds = on ? ds : 0.f;
      }
      pv[q] = pval; dsv[q] = ds;
    }
    pk[e >> 1] = rb::pack_bf16(pv[0], pv[1]);
    dk16[e >> 1] = rb::pack_bf16(dsv[0], dsv[1]);
  }
  // phase B: bias gradients from the bf16 dS (the values the dK / dQ matmuls see)
  if (WDT || WDP) {
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const uint32_t w = dk16[e >> 1];
      const float ds = __uint_as_float((e & 1) ? (w & 0xffff0000u) : (w << 16));
      if (WDP) {
        const int ee = e0 + e;
        const int src = (ee + 31 - lane) & 31;
        const float got = __shfl_sync(0xffffffffu, ds, src);
        acc_hi += src < ee ? got : 0.f;
        acc_lo += src < ee ? 0.f : got;
      }
      if (WDT) {
        const int bk = static_cast<int>((bkp[e >> 2] >> (8 * (e & 3))) & 0xffu);
        if (bk != run_bucket) {
          if (run_bucket >= 0 && run_sum != 0.f) hist_add(dtsw_s + run_bucket, run_sum);
          run_bucket = bk; run_sum = 0.f;
        }
        run_sum += ds;
      }
    }
  }
}

template <bool BT, bool BP, bool WDT, bool WDP>
__global__ void __launch_bounds__(640, 1)
hstu_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                const HstuBwdParams p) {
  const int b = blockIdx.y / p.H, h = blockIdx.y % p.H;
  const int kb = blockIdx.x;
  const int q_start = p.q_offsets[b], len_q = p.q_offsets[b + 1] - q_start;
  const int k_start = p.k_offsets[b], len_k = p.k_offsets[b + 1] - k_start;
  if (kb * BKV >= len_k || len_q == 0) return;
  const int delta = len_k - len_q;
  const int nctx = p.num_context ? p.num_context[b] : 0;
  const int ntgt = p.num_target ? p.num_target[b] : 0;
  const int gs = p.target_group_size;
  const int qb_total = (len_q + BQ - 1) / BQ;
  int qb_first = 0;
  if (p.causal && nctx == 0) {
    const int first_row = kb * BKV - delta;                       // first query row whose position reaches this block
    qb_first = first_row <= 0 ? 0 : first_row / BQ;
  }
  const int n_iter = qb_total - qb_first;
  if (n_iter <= 0) {
    // keys that no query attends to still need zero gradients
    for (int e = threadIdx.x; e < BKV * D; e += blockDim.x) {
      const int r = e / D, c = e % D;
      if (kb * BKV + r < len_k) {
        const long long o = static_cast<long long>(k_start + kb * BKV + r) * p.ld_dkv + h * D + c;
        reinterpret_cast<__nv_bfloat16*>(p.dk)[o] = __float2bfloat16(0.f);
        reinterpret_cast<__nv_bfloat16*>(p.dv)[o] = __float2bfloat16(0.f);
      }
    }
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* k_s = smem;
  uint8_t* v_s = smem + TILE;
  uint8_t* qdo_s = smem + 2 * TILE;                                // stage s: Q at 2s, dO at 2s+1
  uint8_t* ds_s = smem + 6 * TILE;                                 // 2 chunks of [128 keys][64 q]
  float* ts_s = reinterpret_cast<float*>(smem + 8 * TILE);         // [4 warps][2][128]
  float* tsw_s = ts_s + 1024;                                      // [192]
  long long* dtsw_s = reinterpret_cast<long long*>(tsw_s + 192);   // [192] fixed point
  long long* dpos_s = dtsw_s + 192;                                // [POS_HIST] fixed point
  float* pos_s = reinterpret_cast<float*>(dpos_s + POS_HIST);      // [16 warps][64] distance-bias windows
  uint64_t* bars = reinterpret_cast<uint64_t*>(pos_s + 16 * 64);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;       // [2]
  uint64_t* qdo_empty = bars + 3;      // [2]
  uint64_t* sdp_full = bars + 5;
  uint64_t* act_done = bars + 6;
  uint64_t* dq_full = bars + 7;
  uint64_t* dq_empty = bars + 8;
  uint64_t* dkv_full = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* quarter_bar = bars + 11;   // [4] the four warps of one TMEM lane quarter meet here once per tile

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr bool want_dpos = WDP, want_dts = WDT;
  if (threadIdx.x == 0) {
    rb::mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) { rb::mbar_init(&qdo_full[s], 1); rb::mbar_init(&qdo_empty[s], 1); }
    rb::mbar_init(sdp_full, 1); rb::mbar_init(act_done, 512); rb::mbar_init(dq_full, 1); rb::mbar_init(dq_empty, 512);
    rb::mbar_init(dkv_full, 1);
    for (int i = 0; i < 4; ++i) rb::mbar_init(&quarter_bar[i], 128);
    *abort_flag = 0;
    rb::mbar_fence_init();
  }
  if (warp == 2) { rb::tmem_alloc(tmem_slot, 512); rb::tmem_relinquish(); }
  for (int i = threadIdx.x; i < 192; i += blockDim.x) {
    tsw_s[i] = (p.ts_w && i <= p.num_buckets) ? p.ts_w[i] : 0.f;
    dtsw_s[i] = 0;
  }
  for (int i = threadIdx.x; i < POS_HIST; i += blockDim.x) dpos_s[i] = 0;
  rb::tc_fence_before();
  __syncthreads();
  rb::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // columns: S^T / P^T [0,128), dP^T / dS^T [128,256), dV [256,320), dK [320,384), dQ [384,448)
  const uint32_t T_ST = tmem, T_DP = tmem + 128, T_DV = tmem + 256, T_DK = tmem + 320, T_DQ = tmem + 384;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------ TMA producer
    rb::mbar_expect_tx(kv_full, 2 * TILE);
    for (int half = 0; half < 2; ++half) {
      rb::tma_load_2d(k_s + half * 8192, &tm_k, kv_full, h * D, k_start + kb * BKV + half * 64);
      rb::tma_load_2d(v_s + half * 8192, &tm_v, kv_full, h * D, k_start + kb * BKV + half * 64);
    }
    for (int t = 0; t < n_iter; ++t) {
      const int st = t & 1, qb = qb_first + t;
      if (!rb::mbar_wait(&qdo_empty[st], ((t >> 1) & 1) ^ 1, abort_flag, p.status)) goto done;
      rb::mbar_expect_tx(&qdo_full[st], 2 * TILE);
      for (int half = 0; half < 2; ++half) {
        rb::tma_load_2d(qdo_s + (2 * st) * TILE + half * 8192, &tm_q, &qdo_full[st], h * D, q_start + qb * BQ + half * 64);
        rb::tma_load_2d(qdo_s + (2 * st + 1) * TILE + half * 8192, &tm_do, &qdo_full[st], h * D, q_start + qb * BQ + half * 64);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t id_kk = rb::umma_idesc(128, 128, 0, 0, 1);      // both operands contraction-major
    const uint32_t id_tn = rb::umma_idesc(128, D, 0, 1, 1);        // A in TMEM, B MN-major
    const uint32_t id_nn = rb::umma_idesc(128, D, 1, 1, 1);        // A and B MN-major
    const uint32_t k_addr = rb::smem_u32(k_s), v_addr = rb::smem_u32(v_s), ds_addr = rb::smem_u32(ds_s);
    if (!rb::mbar_wait(kv_full, 0, abort_flag, p.status)) goto done;
    for (int t = 0; t < n_iter; ++t) {
      const int st = t & 1;
      const uint32_t q_addr = rb::smem_u32(qdo_s + (2 * st) * TILE), do_addr = q_addr + TILE;
      if (!rb::mbar_wait(&qdo_full[st], (t >> 1) & 1, abort_flag, p.status)) goto done;
      rb::tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        rb::umma_f16_ss(T_ST, rb::umma_smem_desc(k_addr + kk * 32, 16, 1024), rb::umma_smem_desc(q_addr + kk * 32, 16, 1024),
                        id_kk, kk > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        rb::umma_f16_ss(T_DP, rb::umma_smem_desc(v_addr + kk * 32, 16, 1024), rb::umma_smem_desc(do_addr + kk * 32, 16, 1024),
                        id_kk, kk > 0 ? 1u : 0u);
      }
      rb::umma_commit(sdp_full);
      if (!rb::mbar_wait(act_done, t & 1, abort_flag, p.status)) goto done;
      if (t > 0 && !rb::mbar_wait(dq_empty, (t - 1) & 1, abort_flag, p.status)) goto done;   // dQ tile drained
      rb::tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < BQ / 16; ++kk) {
        rb::umma_f16_ts(T_DV, T_ST + kk * 8, rb::umma_smem_desc(do_addr + kk * 2048, 16384, 1024), id_tn,
                        (t > 0 || kk > 0) ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < BQ / 16; ++kk) {
        rb::umma_f16_ts(T_DK, T_DP + kk * 8, rb::umma_smem_desc(q_addr + kk * 2048, 16384, 1024), id_tn,
                        (t > 0 || kk > 0) ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < BKV / 16; ++kk) {
        rb::umma_f16_ss(T_DQ, rb::umma_smem_desc(ds_addr + kk * 2048, 16384, 1024),
                        rb::umma_smem_desc(k_addr + kk * 2048, 16384, 1024), id_nn, kk > 0 ? 1u : 0u);
      }
      rb::umma_commit(&qdo_empty[st]);
      rb::umma_commit(dq_full);
    }
    rb::umma_commit(dkv_full);
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ activation, dQ drain, dK / dV store
    // warp = 4 + 4*grp + ew: ew = TMEM lane quarter (32 key rows), grp = 32-query column chunk
    const int ew = warp & 3;
    const int grp = (warp - 4) >> 2;
    const int row = ew * 32 + lane;                                 // key row of this thread
    const int j = kb * BKV + row;
    const uint32_t lane_sel = static_cast<uint32_t>(ew * 32) << 16;
    const float ts_j = BT ? p.ts[k_start + min(j, len_k - 1)] : 0.f;
    const float k_log = 0.69314718f / p.ts_divisor;
    const float half_alpha = 0.5f * p.alpha;
    const float half_sa = 0.5f * p.scale * p.alpha;
    const int j0w = kb * BKV + ew * 32;                               // key of lane 0
    float* my_pos = pos_s + (warp - 4) * 64;
    auto load_ts = [&](int t) -> float {
      const int pi = (qb_first + t) * BQ + grp * 32 + lane + delta;
      return (t < n_iter && pi < len_k && pi >= 0) ? __ldg(p.ts + k_start + pi) : 0.f;
    };
    auto load_pos = [&](int t, int w) -> float {
      const int d = (qb_first + t) * BQ + grp * 32 + delta - j0w - 31 + w;
      return t < n_iter ? __ldg(p.pos_w + min(max(d, 0), p.pos_len - 1)) : 0.f;
    };
    float ts_nxt = BT ? load_ts(0) : 0.f;
    float pos_nxt0 = BP ? load_pos(0, lane) : 0.f, pos_nxt1 = BP ? load_pos(0, lane + 32) : 0.f;
    // time-bucket gradient: a key row meets its buckets in long runs (|ts_i - ts_j| grows with i), so the running sum
    // lives across tiles and reaches shared memory only when the bucket changes
    int run_bucket = -1;
    float run_sum = 0.f;
    for (int t = 0; t < n_iter; ++t) {
      const int qb = qb_first + t;
      float* my_ts = ts_s + ((warp - 4) * 2 + (t & 1)) * 32;
      if (BT || BP) {
        __syncwarp();
        if (BT) { my_ts[lane] = ts_nxt; ts_nxt = load_ts(t + 1); }
        if (BP) {
          my_pos[lane] = pos_nxt0; my_pos[lane + 32] = pos_nxt1;
          pos_nxt0 = load_pos(t + 1, lane); pos_nxt1 = load_pos(t + 1, lane + 32);
        }
        __syncwarp();
      }
      bool ok = rb::mbar_wait(sdp_full, t & 1, abort_flag, p.status);
      if (!__all_sync(0xffffffffu, ok)) goto done;
      rb::tc_fence_after();
      // a tile strictly below the diagonal with no ragged edge needs no mask
      const bool full = p.causal && ntgt == 0 && (kb * BKV + BKV - 1 <= qb * BQ + delta) && (kb * BKV + BKV <= len_k) &&
                        (qb * BQ + BQ <= len_q);
      {
        const int c = grp;
        uint32_t pk[16], dk16[16];
        const int i0 = qb * BQ + c * 32, pi0 = i0 + delta;
        float acc_lo = 0.f, acc_hi = 0.f;
        // two halves of 16 query columns keep the live registers under the 640-thread budget
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t rs[16], rd[16];
          rb::tmem_ld_32x16(T_ST + lane_sel + c * 32 + half * 16, rs);
          rb::tmem_ld_32x16(T_DP + lane_sel + c * 32 + half * 16, rd);
          rb::tmem_ld_wait();
          if (full)
            bwd_chunk<BT, BP, WDT, WDP, false>(rs, rd, pk + half * 8, dk16 + half * 8, half * 16, run_bucket, run_sum, ts_j, my_ts,
                                               tsw_s, dtsw_s, my_pos, lane, k_log, p.bucket_cap, half_alpha, p.scale, half_sa, pi0,
                                               i0, j, len_q, len_k, p.causal, nctx, ntgt, gs, acc_lo, acc_hi);
          else
            bwd_chunk<BT, BP, WDT, WDP, true>(rs, rd, pk + half * 8, dk16 + half * 8, half * 16, run_bucket, run_sum, ts_j, my_ts,
                                              tsw_s, dtsw_s, my_pos, lane, k_log, p.bucket_cap, half_alpha, p.scale, half_sa, pi0,
                                              i0, j, len_q, len_k, p.causal, nctx, ntgt, gs, acc_lo, acc_hi);
        }
        if (WDP) {
          const int hi_idx = min(p.pos_len, POS_HIST) - 1;
          const int base = pi0 - j0w - 31;
          if (acc_lo != 0.f) hist_add(dpos_s + min(max(base + lane, 0), hi_idx), acc_lo);
          if (acc_hi != 0.f) hist_add(dpos_s + min(max(base + lane + 32, 0), hi_idx), acc_hi);
        }
        // P^T / dS^T overwrite S^T / dP^T columns that OTHER warps of this lane quarter read: wait until all
        // four column groups of the quarter have their chunks in registers (bounded, like every wait here)
        rb::tc_fence_before();
        rb::mbar_arrive(&quarter_bar[ew]);
        ok = rb::mbar_wait(&quarter_bar[ew], t & 1, abort_flag, p.status);
        if (!__all_sync(0xffffffffu, ok)) goto done;
        rb::tc_fence_after();
        rb::tmem_st_32x16(T_ST + lane_sel + c * 16, pk);             // P^T over the S^T columns already consumed
        rb::tmem_st_32x16(T_DP + lane_sel + c * 16, dk16);           // dS^T over dP^T
        // dS^T row -> shared memory, MN-major operand layout (two 64-query chunks, 128-byte swizzle)
        uint8_t* dst = ds_s + (c >> 1) * TILE + row * 128;
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const int u = ((c & 1) * 4 + v4) ^ (row & 7);
          *reinterpret_cast<uint4*>(dst + u * 16) = make_uint4(dk16[4 * v4], dk16[4 * v4 + 1], dk16[4 * v4 + 2], dk16[4 * v4 + 3]);
        }
      }
      rb::tmem_st_wait();
      fence_async_smem();
      rb::tc_fence_before();
      rb::mbar_arrive(act_done);
      // ---- drain the dQ tile of this pair: rows = queries
      ok = rb::mbar_wait(dq_full, t & 1, abort_flag, p.status);
      if (!__all_sync(0xffffffffu, ok)) goto done;
      rb::tc_fence_after();
      const int iq = qb * BQ + row;
      float* dq_row = p.dq32 + static_cast<long long>(q_start + iq) * p.ld_dq + h * D;
      if (grp < D / 32) {
        const int c = grp;
        uint32_t r[32];
        rb::tmem_ld_32x32(T_DQ + lane_sel + c * 32, r);
        rb::tmem_ld_wait();
        if (iq < len_q) {
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            red_add_v4(dq_row + c * 32 + e, __uint_as_float(r[e]), __uint_as_float(r[e + 1]), __uint_as_float(r[e + 2]),
                       __uint_as_float(r[e + 3]));
        }
      }
      rb::tc_fence_before();
      rb::mbar_arrive(dq_empty);
    }
    if (WDT && run_bucket >= 0 && run_sum != 0.f) hist_add(dtsw_s + run_bucket, run_sum);
    {
      bool ok = rb::mbar_wait(dkv_full, 0, abort_flag, p.status);
      if (!__all_sync(0xffffffffu, ok)) goto done;
      rb::tc_fence_after();
      __nv_bfloat16* dk_row = reinterpret_cast<__nv_bfloat16*>(p.dk) + static_cast<long long>(k_start + j) * p.ld_dkv + h * D;
      __nv_bfloat16* dv_row = reinterpret_cast<__nv_bfloat16*>(p.dv) + static_cast<long long>(k_start + j) * p.ld_dkv + h * D;
      {
        const int which = grp >> 1;                                   // groups 0,1 store dV, groups 2,3 store dK
        {
          const int c = grp & 1;
          uint32_t r[32];
          rb::tmem_ld_32x32((which ? T_DK : T_DV) + lane_sel + c * 32, r);
          rb::tmem_ld_wait();
          if (j < len_k) {
            __nv_bfloat16* o = (which ? dk_row : dv_row) + c * 32;
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 w;
              w.x = rb::pack_bf16(__uint_as_float(r[e]), __uint_as_float(r[e + 1]));
              w.y = rb::pack_bf16(__uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
              w.z = rb::pack_bf16(__uint_as_float(r[e + 4]), __uint_as_float(r[e + 5]));
              w.w = rb::pack_bf16(__uint_as_float(r[e + 6]), __uint_as_float(r[e + 7]));
              *reinterpret_cast<uint4*>(o + e) = w;
            }
          }
        }
      }
    }
  }
done:
  __syncwarp();
  rb::tc_fence_before();
  __syncthreads();
  if (warp == 2) rb::tmem_dealloc(tmem, 512);
  // flush the bias-gradient histograms of this CTA
  if (want_dts) for (int i = threadIdx.x; i <= p.num_buckets && i < 192; i += blockDim.x) if (dtsw_s[i] != 0) atomicAdd(p.d_ts_w + i, hist_value(dtsw_s[i]));
  if (want_dpos) for (int i = threadIdx.x; i < p.pos_len && i < POS_HIST; i += blockDim.x) if (dpos_s[i] != 0) atomicAdd(p.d_pos_w + i, hist_value(dpos_s[i]));
}

int make_map(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld) {
  return rb_host::make_map_2d(m, base, rows, cols, ld, 64, 64, true);
}

template <bool BT, bool BP, bool WDT, bool WDP>
int launch_bwd(dim3 grid, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
               const HstuBwdParams& p, cudaStream_t st) {
  static bool set = false;
  if (!set) {
    RB_CUDA_CHECK(cudaFuncSetAttribute(hstu_bwd_kernel<BT, BP, WDT, WDP>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    set = true;
  }
  hstu_bwd_kernel<BT, BP, WDT, WDP><<<grid, 640, SMEM_BYTES, st>>>(tq, tk, tv, tdo, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// q, dO [Tq][ld_q / ld_do], k, v [Tk][ld_k] bf16 with head h at columns h*64.  dq32 is an fp32 accumulator the
// caller zeroed; dk, dv are bf16 [Tk][ld_dkv]; d_ts_w / d_pos_w fp32 accumulators (nullable).
RB_API int rb_hstu_attn_bwd(const void* q, long long ld_q, const void* dout, long long ld_do, long long Tq, const void* k,
                            const void* v, long long ld_k, long long Tk, const int* q_offsets, const int* k_offsets,
                            int B, int H, int D_, int max_len_k, float alpha, float scale, int causal,
                            const int* num_context, const int* num_target, int target_group_size, const float* ts,
                            const float* ts_w, int num_buckets, float ts_divisor, const float* pos_w, int pos_len,
                            float* dq32, long long ld_dq, void* dk, void* dv, long long ld_dkv, float* d_ts_w,
                            float* d_pos_w, int* status, cudaStream_t st) {
  if (B == 0 || H == 0 || max_len_k <= 0) return 0;
  if (D_ != D || (ld_q % 8) || (ld_k % 8) || (ld_do % 8) || (ld_dkv % 8) || (ld_dq % 4)) return -3;
  if (num_buckets >= 192 || pos_len > POS_HIST) return -4;
  HstuBwdParams p;
  p.q_offsets = q_offsets; p.k_offsets = k_offsets; p.B = B; p.H = H; p.alpha = alpha; p.scale = scale; p.causal = causal;
  p.num_context = num_context; p.num_target = num_target; p.target_group_size = target_group_size; p.ts = ts; p.ts_w = ts_w;
  p.num_buckets = num_buckets; p.ts_divisor = ts_divisor > 0.f ? ts_divisor : 1.f; p.pos_w = pos_w; p.pos_len = pos_len > 0 ? pos_len : 1;
  p.dq32 = dq32; p.ld_dq = ld_dq; p.dk = dk; p.dv = dv; p.ld_dkv = ld_dkv; p.d_ts_w = d_ts_w; p.d_pos_w = d_pos_w; p.status = status;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_map(&tq, q, Tq, static_cast<long long>(H) * D, ld_q))) return rc;
  if ((rc = make_map(&tdo, dout, Tq, static_cast<long long>(H) * D, ld_do))) return rc;
  if ((rc = make_map(&tk, k, Tk, static_cast<long long>(H) * D, ld_k))) return rc;
  if ((rc = make_map(&tv, v, Tk, static_cast<long long>(H) * D, ld_k))) return rc;
  {
    const int hi = static_cast<int>(38.787f / p.ts_divisor);         // log(7e16) / divisor
    p.bucket_cap = num_buckets < hi ? num_buckets : hi;
  }
  dim3 grid((max_len_k + BKV - 1) / BKV, B * H);
  const bool bt = ts != nullptr && ts_w != nullptr, bp = pos_w != nullptr;
  const int vt = !bt ? 0 : (d_ts_w ? 2 : 1), vp = !bp ? 0 : (d_pos_w ? 2 : 1);
#define RB_BWD(BT_, WDT_, BP_, WDP_) return launch_bwd<BT_, BP_, WDT_, WDP_>(grid, tq, tk, tv, tdo, p, st)
  switch (vt * 3 + vp) {
    case 0: RB_BWD(false, false, false, false);
    case 1: RB_BWD(false, false, true, false);
    case 2: RB_BWD(false, false, true, true);
    case 3: RB_BWD(true, false, false, false);
    case 4: RB_BWD(true, false, true, false);
    case 5: RB_BWD(true, false, true, true);
    case 6: RB_BWD(true, true, false, false);
    case 7: RB_BWD(true, true, true, false);
    default: RB_BWD(true, true, true, true);
  }
#undef RB_BWD
}
