// HSTU jagged SiLU attention, forward, on tcgen05 / TMEM (sm_100a).
//
//   O = ( SiLU(alpha * (Q K^T + bias)) * scale  (.)  mask ) V          (no softmax, no row statistics)
//
// One CTA owns one (sequence, head, 128-query block) and walks the key blocks it may attend to:
//   * TMA (64-row boxes, 128-byte swizzle) brings Q once and K/V blocks through a ring; K/V may come from
//     a jagged [T, H*D] tensor or from a paged KV cache [pages][2][page][H*D] through a page table,
//   * S = Q K^T is a 128x128xD tcgen05.mma into one of two TMEM S buffers,
//   * sixteen activation warps (four per TMEM lane quarter, one 32-column chunk each) read S with tcgen05.ld, add the relative position / time bias computed on the
//     fly from the bucket tables (never materialising a [B,H,S,S] bias), apply alpha, SiLU, scale and the
//     causal / contextual / target-group mask, and write P as packed bf16 back into TMEM (tcgen05.st),
//   * O += P V is a tcgen05.mma whose A operand is P in TMEM and whose B operand is the V tile in shared
//     memory (MN-major), accumulating across key blocks in TMEM; S(j+1) overlaps the activation of S(j).
// Query rows may be a suffix of the key positions (delta / incremental decoding).  Every mbarrier wait
// is bounded; on expiry the kernel records an error, frees TMEM and returns.
//
// Spec: cust_op/framework/torch_plugin/torch_library/hstu/README.md:18-44,96-145 (hstu_jagged, hstu_paged),
// golden build/presmoke/hstu/hstu_common.py:108-153 (mask), :286-345 (forward).
#include "common.cuh"

namespace {

constexpr int BQ = 128;   // query rows per CTA
constexpr int BKV = 128;  // keys per block

struct HstuFwdParams {
  const int* q_offsets;      // [B+1] rows of Q / O per sequence
  const int* k_offsets;      // [B+1] key positions per sequence (== q_offsets unless delta / paged)
  int B, H;
  void* out; long long ld_o; // O [Tq][ld_o], head h at columns h*D
  float alpha, scale;
  int causal;
  const int* num_context;    // [B] or null
  const int* num_target;     // [B] or null
  int target_group_size;
  // on-the-fly bias (all optional)
  const float* ts;           // [Tk] timestamp per key position (jagged, k_offsets space)
  const float* ts_w;         // [num_buckets + 1]
  int num_buckets; float ts_divisor;
  const float* pos_w;        // [pos_len]: bias of distance (i - j) clamped to [0, pos_len-1]
  int pos_len;
  // paged K/V
  const int* page_ids; const int* page_indptr; int page_size;
  int box_rows;              // rows per TMA box for K/V (64, or page_size when smaller)
  int bucket_cap;            // min(num_buckets, floor(log(7e16) / divisor)): replaces the clamp of |dt| from above
  int* status;
  // dense operands of the reference's calling convention (both optional): an additive bias [B][H][S][S] and a
  // multiplicative 0/1 mask of the same indexing; element (b, h, query position, key position) sits at
  // base + b * stride_b + h * stride_h + position_q * ld + position_k (strides in elements; stride_h may be 0)
  const void* dbias; int dbias_kind;      // 0 none, 1 bf16, 2 fp32
  long long db_sb, db_sh, db_ld;
  const void* dmask; int dmask_kind;      // 0 none, 1 uint8 / bool, 2 bf16, 3 fp32
  long long dm_sb, dm_sh, dm_ld;
  int dn_rows, dn_cols;                   // extent of the dense operands' last two dims: nothing is read outside it
};

// 8 consecutive elements of a dense operand row -> fp32 (vector load when the address is 16-byte aligned and all 8
// are inside the row, element loads with a fill value otherwise)
__device__ __forceinline__ void load_dense8(const void* base, int kind, long long off, int valid, float fill, float (&o)[8]) {
  if (kind == 1) {                                          // bf16 (bias kind 1)
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(base) + off;
    if (valid >= 8 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
      float2 a = rb::unpack_bf16(u.x), b = rb::unpack_bf16(u.y), c = rb::unpack_bf16(u.z), d = rb::unpack_bf16(u.w);
      o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y; o[4] = c.x; o[5] = c.y; o[6] = d.x; o[7] = d.y;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = i < valid ? __bfloat162float(p[i]) : fill;
    }
  } else if (kind == 2) {                                   // fp32
    const float* p = reinterpret_cast<const float*>(base) + off;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = i < valid ? __ldg(p + i) : fill;
  } else {                                                  // uint8
    const unsigned char* p = reinterpret_cast<const unsigned char*>(base) + off;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = i < valid ? (p[i] ? 1.f : 0.f) : fill;
  }
}

template <int D> struct FwdCfg {
  static constexpr int CH = D / 64;                       // 64-column swizzle chunks per row
  static constexpr int TILE_BYTES = BQ * 128 * CH;        // one Q, K or V tile
  static constexpr int STAGES = (D == 64) ? 3 : 2;
  static constexpr int SMEM_BYTES = TILE_BYTES * (1 + 2 * STAGES) + 6144 + 4096 + 1024;
};

// mask of (query position pi, key position j) inside a sequence of len keys
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


// One warp's 32 x 32 chunk of S -> P.  Thread = query row, e = key column of the chunk.
//   bias_t : tsw[min(int(log2(max(|ts_i - ts_j|, 1)) * k_log), cap)]      (k_log = ln 2 / divisor)
//   bias_p : window[lane + 31 - e], the warp's pre-clamped slice of pos_w (distance = pi - j)
//   silu(alpha x) * scale = hs + hs * tanh(h),  h = x * alpha / 2,  hs = h * scale
template <bool BT, bool BP, bool MASKED>
__device__ __forceinline__ void activate_chunk(const uint32_t (&r)[32], uint32_t (&pk)[16], float ts_i, const float* my_ts,
                                               const float* tsw_s, const float* my_pos, int lane, float k_log, int cap,
                                               float half_alpha, float scale, int pi, int j0, int len_k, int causal,
                                               int nctx, int ntgt, int gs) {
#pragma unroll
  for (int e = 0; e < 32; e += 2) {
    float v2[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      float x = __uint_as_float(r[e + q]);
      if (BT) {
        const float a = fmaxf(fabsf(ts_i - my_ts[e + q]), 1.f);
        x += tsw_s[min(static_cast<int>(__log2f(a) * k_log), cap)];
      }
      if (BP) x += my_pos[lane + 31 - (e + q)];
      const float h = x * half_alpha;
      float t;
      asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
      const float hs = h * scale;
      x = fmaf(hs, t, hs);
      if (MASKED && !attends(pi, j0 + e + q, len_k, causal, nctx, ntgt, gs)) x = 0.f;
      v2[q] = x;
    }
    pk[e >> 1] = rb::pack_bf16(v2[0], v2[1]);
  }
}

template <int D, bool BT, bool BP>
__global__ void __launch_bounds__(640, 1)
hstu_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const HstuFwdParams p) {
  using C = FwdCfg<D>;
  const int b = blockIdx.y / p.H, h = blockIdx.y % p.H;
  const int qblk = gridDim.x - 1 - blockIdx.x;                      // heavy (late) blocks first
  const int q_start = p.q_offsets[b], len_q = p.q_offsets[b + 1] - q_start;
  const int k_start = p.k_offsets[b], len_k = p.k_offsets[b + 1] - k_start;
  if (qblk * BQ >= len_q) return;
  const int delta = len_k - len_q;                                  // query row i sits at key position i + delta
  const int nctx = p.num_context ? p.num_context[b] : 0;
  const int ntgt = p.num_target ? p.num_target[b] : 0;
  const int gs = p.target_group_size;
  const int kb_total = (len_k + BKV - 1) / BKV;
  // key blocks this query block needs
  const int pi_lo = qblk * BQ + delta, pi_hi = min(qblk * BQ + BQ - 1, len_q - 1) + delta;
  int n_kb = kb_total, kb_skip_from = -1, kb_skip_to = -1;          // blocks [skip_from, skip_to) are skipped
  if (p.causal) {
    n_kb = min(kb_total, pi_hi / BKV + 1);
    if (nctx > 0 && pi_lo < nctx) n_kb = kb_total;
    if (ntgt > 0 && gs > 0) {
      const int t0 = len_k - ntgt;
      if (pi_lo >= t0 && !(nctx > 0 && pi_lo < nctx)) {
        // a block of target rows sees the history and only its own groups among the targets
        const int first_needed = (t0 + ((pi_lo - t0) / gs) * gs) / BKV;
        const int hist_end = (t0 + BKV - 1) / BKV;               // blocks holding non-target keys
        if (first_needed > hist_end) { kb_skip_from = hist_end; kb_skip_to = first_needed; }
      }
    }
  }
  const int n_iter = n_kb - (kb_skip_to > kb_skip_from ? kb_skip_to - kb_skip_from : 0);
  auto kb_of = [&](int t) { return (kb_skip_from >= 0 && t >= kb_skip_from) ? t + (kb_skip_to - kb_skip_from) : t; };

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_s = smem;
  uint8_t* kv_s = smem + C::TILE_BYTES;                             // stage s: K at 2*s, V at 2*s+1
  uint8_t* tail = kv_s + 2 * C::STAGES * C::TILE_BYTES;
  float* ts_s = reinterpret_cast<float*>(tail);                     // [4 warps][2][128] key timestamps
  float* tsw_s = ts_s + 1024;                                       // [<= 192] time-bucket weights
  float* pos_s = reinterpret_cast<float*>(tail + 6144);             // [16 warps][64] distance-bias windows
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail + 5120);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + C::STAGES;
  uint64_t* s_full = kv_empty + C::STAGES;
  uint64_t* p_full = s_full + 2;
  uint64_t* p_empty = p_full + 2;
  uint64_t* o_full = p_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    rb::mbar_init(q_full, 1);
    for (int s = 0; s < C::STAGES; ++s) { rb::mbar_init(&kv_full[s], 1); rb::mbar_init(&kv_empty[s], 1); }
    for (int i = 0; i < 2; ++i) { rb::mbar_init(&s_full[i], 1); rb::mbar_init(&p_full[i], 512); rb::mbar_init(&p_empty[i], 1); }
    rb::mbar_init(o_full, 1);
    *abort_flag = 0;
    rb::mbar_fence_init();
  }
  if (warp == 2) { rb::tmem_alloc(tmem_slot, 512); rb::tmem_relinquish(); }
  if (BT) for (int i = threadIdx.x; i <= p.num_buckets && i < 192; i += blockDim.x) tsw_s[i] = p.ts_w[i];
  rb::tc_fence_before();
  __syncthreads();
  rb::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t T_S = tmem, T_O = tmem + 256, T_P = tmem + 384;     // S: 2 x 128 cols, O: D cols, P: 2 x 64 cols

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------ TMA producer
    rb::mbar_expect_tx(q_full, C::TILE_BYTES);
#pragma unroll
    for (int c = 0; c < C::CH; ++c)
#pragma unroll
      for (int half = 0; half < 2; ++half)
        rb::tma_load_2d(q_s + c * (BQ * 128) + half * 8192, &tm_q, q_full, h * D + c * 64, q_start + qblk * BQ + half * 64);
    const int boxes = BKV / p.box_rows;
    for (int t = 0; t < n_iter; ++t) {
      const int st = t % C::STAGES;
      if (!rb::mbar_wait(&kv_empty[st], ((t / C::STAGES) & 1) ^ 1, abort_flag, p.status)) goto done;
      uint8_t* k_dst = kv_s + (2 * st) * C::TILE_BYTES;
      uint8_t* v_dst = k_dst + C::TILE_BYTES;
      rb::mbar_expect_tx(&kv_full[st], 2 * C::TILE_BYTES);
      const int kb = kb_of(t);
      for (int bx = 0; bx < boxes; ++bx) {
        const int tok = kb * BKV + bx * p.box_rows;
        int k_row, v_row;
        if (p.page_ids) {
          const int tk = min(tok, max(len_k - 1, 0));
          const int page = p.page_ids[p.page_indptr[b] + tk / p.page_size];
          const int slot = tok < len_k ? tok % p.page_size : 0;
          k_row = (page * 2) * p.page_size + slot;
          v_row = (page * 2 + 1) * p.page_size + slot;
        } else {
          k_row = v_row = k_start + tok;
        }
#pragma unroll
        for (int c = 0; c < C::CH; ++c) {
          rb::tma_load_2d(k_dst + c * (BKV * 128) + bx * p.box_rows * 128, &tm_k, &kv_full[st], h * D + c * 64, k_row);
          rb::tma_load_2d(v_dst + c * (BKV * 128) + bx * p.box_rows * 128, &tm_v, &kv_full[st], h * D + c * 64, v_row);
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc_s = rb::umma_idesc(BQ, BKV, 0, 0, 1);
    const uint32_t idesc_o = rb::umma_idesc(BQ, D, 0, 1, 1);
    const uint32_t q_addr = rb::smem_u32(q_s);
    auto issue_s = [&](int t) {
      const uint32_t k_addr = rb::smem_u32(kv_s + (2 * (t % C::STAGES)) * C::TILE_BYTES);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = (kk / 4) * (BQ * 128) + (kk % 4) * 32;
        rb::umma_f16_ss(T_S + (t & 1) * 128, rb::umma_smem_desc(q_addr + off, 16, 1024),
                        rb::umma_smem_desc(k_addr + off, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
      }
      rb::umma_commit(&s_full[t & 1]);
    };
    if (!rb::mbar_wait(q_full, 0, abort_flag, p.status)) goto done;
    if (!rb::mbar_wait(&kv_full[0], 0, abort_flag, p.status)) goto done;
    rb::tc_fence_after();
    issue_s(0);
    for (int t = 0; t < n_iter; ++t) {
      if (t + 1 < n_iter) {
        const int st1 = (t + 1) % C::STAGES;
        if (!rb::mbar_wait(&kv_full[st1], ((t + 1) / C::STAGES) & 1, abort_flag, p.status)) goto done;
        rb::tc_fence_after();
        issue_s(t + 1);
      }
      if (!rb::mbar_wait(&p_full[t & 1], (t >> 1) & 1, abort_flag, p.status)) goto done;
      rb::tc_fence_after();
      const uint32_t v_addr = rb::smem_u32(kv_s + (2 * (t % C::STAGES) + 1) * C::TILE_BYTES);
#pragma unroll
      for (int kk = 0; kk < BKV / 16; ++kk)
        rb::umma_f16_ts(T_O, T_P + (t & 1) * 64 + kk * 8, rb::umma_smem_desc(v_addr + kk * 2048, BKV * 128, 1024),
                        idesc_o, (t > 0 || kk > 0) ? 1u : 0u);
      rb::umma_commit(&kv_empty[t % C::STAGES]);
      rb::umma_commit(&p_empty[t & 1]);
    }
    rb::umma_commit(o_full);
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ activation + output
    // warp = 4 + 4*grp + ew: ew selects the TMEM lane quarter (32 query rows), grp the 32-key column chunk.
    // One CTA per SM (TMEM), so the elementwise work needs this many warps to keep the issue slots busy.
    const int ew = warp & 3;
    const int grp = (warp - 4) >> 2;
    const int row = ew * 32 + lane;
    const int i_local = qblk * BQ + row;
    const int pi = i_local + delta;
    const uint32_t lane_sel = static_cast<uint32_t>(ew * 32) << 16;
    const float ts_i = BT ? p.ts[k_start + min(pi, len_k - 1)] : 0.f;
    const float k_log = 0.69314718f / p.ts_divisor;
    const float half_alpha = 0.5f * p.alpha;
    const int pi0 = qblk * BQ + ew * 32 + delta;                      // key position of this warp's first row
    float* my_pos = pos_s + (warp - 4) * 64;
    // operands of the next iteration are fetched one iteration ahead so their latency hides behind the math
    auto load_ts = [&](int t) -> float {
      const int j = kb_of(t) * BKV + grp * 32 + lane;
      return (t < n_iter && j < len_k) ? __ldg(p.ts + k_start + j) : 0.f;
    };
    auto load_pos = [&](int t, int w) -> float {
      const int d = pi0 - (kb_of(t) * BKV + grp * 32) - 31 + w;
      return t < n_iter ? __ldg(p.pos_w + min(max(d, 0), p.pos_len - 1)) : 0.f;
    };
    float ts_nxt = BT ? load_ts(0) : 0.f;
    float pos_nxt0 = BP ? load_pos(0, lane) : 0.f, pos_nxt1 = BP ? load_pos(0, lane + 32) : 0.f;
    for (int t = 0; t < n_iter; ++t) {
      const int kb = kb_of(t), buf = t & 1;
      float* my_ts = ts_s + ((warp - 4) * 2 + buf) * 32;            // private to this warp: no CTA-level sync
      if (BT || BP) {
        __syncwarp();
        if (BT) { my_ts[lane] = ts_nxt; ts_nxt = load_ts(t + 1); }
        if (BP) {
          my_pos[lane] = pos_nxt0; my_pos[lane + 32] = pos_nxt1;
          pos_nxt0 = load_pos(t + 1, lane); pos_nxt1 = load_pos(t + 1, lane + 32);
        }
        __syncwarp();
      }
      bool ok = rb::mbar_wait(&s_full[buf], (t >> 1) & 1, abort_flag, p.status);
      ok = ok && rb::mbar_wait(&p_empty[buf], ((t >> 1) & 1) ^ 1, abort_flag, p.status);
      if (!__all_sync(0xffffffffu, ok)) goto done;
      rb::tc_fence_after();
      // fast path: a key block that lies wholly in the history (before the targets), strictly below the diagonal of this
      // row block, needs no mask - target rows see all of the history, ordinary rows everything up to themselves
      const bool full = p.causal && (kb * BKV + BKV - 1 <= pi_lo) && (kb * BKV + BKV <= len_k - ntgt);
      {
        const int c = grp;
        uint32_t r[32];
        rb::tmem_ld_32x32(T_S + buf * 128 + lane_sel + c * 32, r);
        rb::tmem_ld_wait();
        uint32_t pk[16];
        const int j0 = kb * BKV + c * 32;
        if (p.dbias_kind && i_local < len_q && pi < p.dn_rows) {              // dense additive bias: this thread's 32 keys of its query row
          const long long roff = static_cast<long long>(b) * p.db_sb + static_cast<long long>(h) * p.db_sh +
                                 static_cast<long long>(pi) * p.db_ld + j0;
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            float bv[8];
            load_dense8(p.dbias, p.dbias_kind, roff + e, min(len_k, p.dn_cols) - (j0 + e), 0.f, bv);
#pragma unroll
            for (int i = 0; i < 8; ++i) r[e + i] = __float_as_uint(__uint_as_float(r[e + i]) + bv[i]);
          }
        }
        if (full)
          activate_chunk<BT, BP, false>(r, pk, ts_i, my_ts, tsw_s, my_pos, lane, k_log, p.bucket_cap, half_alpha, p.scale, pi, j0,
                                        len_k, p.causal, nctx, ntgt, gs);
        else
          activate_chunk<BT, BP, true>(r, pk, ts_i, my_ts, tsw_s, my_pos, lane, k_log, p.bucket_cap, half_alpha, p.scale, pi, j0,
                                       len_k, p.causal, nctx, ntgt, gs);
        if (p.dmask_kind) {                                 // dense 0/1 mask on the activated values
          const long long roff = static_cast<long long>(b) * p.dm_sb + static_cast<long long>(h) * p.dm_sh +
                                 static_cast<long long>(pi) * p.dm_ld + j0;
          const int mk = p.dmask_kind == 1 ? 0 : (p.dmask_kind == 2 ? 1 : 2);    // load_dense8 kinds: 0 uint8, 1 bf16, 2 fp32
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            float mv[8];
            if (i_local < len_q && pi < p.dn_rows) load_dense8(p.dmask, mk, roff + e, min(len_k, p.dn_cols) - (j0 + e), 0.f, mv);
            else {
#pragma unroll
              for (int i = 0; i < 8; ++i) mv[i] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
              uint32_t w = pk[(e + i) >> 1];
              if (mv[i] == 0.f) w &= 0xFFFF0000u;
              if (mv[i + 1] == 0.f) w &= 0x0000FFFFu;
              pk[(e + i) >> 1] = w;
            }
          }
        }
        rb::tmem_st_32x16(T_P + buf * 64 + lane_sel + c * 16, pk);
      }
      rb::tmem_st_wait();
      rb::tc_fence_before();
      rb::mbar_arrive(&p_full[buf]);
    }
    {
      bool ok = rb::mbar_wait(o_full, 0, abort_flag, p.status);
      if (!__all_sync(0xffffffffu, ok)) goto done;
      rb::tc_fence_after();
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(q_start + i_local) * p.ld_o + h * D;
      if (grp < D / 32) {
        const int c = grp;
        uint32_t r[32];
        rb::tmem_ld_32x32(T_O + lane_sel + c * 32, r);
        rb::tmem_ld_wait();
        if (i_local < len_q) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 w;
            w.x = rb::pack_bf16(__uint_as_float(r[e]), __uint_as_float(r[e + 1]));
            w.y = rb::pack_bf16(__uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
            w.z = rb::pack_bf16(__uint_as_float(r[e + 4]), __uint_as_float(r[e + 5]));
            w.w = rb::pack_bf16(__uint_as_float(r[e + 6]), __uint_as_float(r[e + 7]));
            *reinterpret_cast<uint4*>(o + c * 32 + e) = w;
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
}

int make_map(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld, int box_rows) {
  return rb_host::make_map_2d(m, base, rows, cols, ld, 64, box_rows, true);
}

template <int D, bool BT, bool BP>
int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const HstuFwdParams& p,
               int max_qblocks, cudaStream_t st) {
  using C = FwdCfg<D>;
  static bool set = false;
  if (!set) {
    RB_CUDA_CHECK(cudaFuncSetAttribute(hstu_fwd_kernel<D, BT, BP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    set = true;
  }
  dim3 grid(max_qblocks, p.B * p.H);
  hstu_fwd_kernel<D, BT, BP><<<grid, 640, C::SMEM_BYTES, st>>>(tq, tk, tv, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// q [Tq][ld_q], k / v [Tk][ld_k] bf16 with head h at columns h*D (D = 64 or 128), or - when page_ids is given -
// kv_cache [pages][2][page_size][H*D] (k and v are then both the cache base).  Offsets are int32 device arrays.
// Row strides in elements, multiples of 8.  Returns 0 / cudaError_t / negative argument error.
static int hstu_attn_fwd_impl(const void* q, long long ld_q, long long Tq, const void* k, const void* v, long long ld_k,
                            long long Tk, const int* q_offsets, const int* k_offsets, int B, int H, int D,
                            int max_len_q, void* out, long long ld_o, float alpha, float scale, int causal,
                            const int* num_context, const int* num_target, int target_group_size, const float* ts,
                            const float* ts_w, int num_buckets, float ts_divisor, const float* pos_w, int pos_len,
                            const int* page_ids, const int* page_indptr, int page_size, long long num_pages,
                            int* status, cudaStream_t st, const void* dbias, int dbias_kind, long long db_sb, long long db_sh,
                            long long db_ld, const void* dmask, int dmask_kind, long long dm_sb, long long dm_sh,
                            long long dm_ld, int dn_rows, int dn_cols) {
  if (B == 0 || H == 0 || max_len_q <= 0) return 0;
  if ((ld_q % 8) || (ld_k % 8) || (ld_o % 8) || (D != 64 && D != 128)) return -3;
  if (num_buckets >= 192) return -4;
  HstuFwdParams p;
  p.q_offsets = q_offsets; p.k_offsets = k_offsets; p.B = B; p.H = H; p.out = out; p.ld_o = ld_o;
  p.alpha = alpha; p.scale = scale; p.causal = causal; p.num_context = num_context; p.num_target = num_target;
  p.target_group_size = target_group_size; p.ts = ts; p.ts_w = ts_w; p.num_buckets = num_buckets;
  p.ts_divisor = ts_divisor > 0.f ? ts_divisor : 1.f; p.pos_w = pos_w; p.pos_len = pos_len;
  {
    const int hi = static_cast<int>(38.787f / p.ts_divisor);         // log(7e16) / divisor
    p.bucket_cap = num_buckets < hi ? num_buckets : hi;
  }
  p.page_ids = page_ids; p.page_indptr = page_indptr; p.page_size = page_size; p.status = status;
  p.dbias = dbias; p.dbias_kind = dbias ? dbias_kind : 0; p.db_sb = db_sb; p.db_sh = db_sh; p.db_ld = db_ld;
  p.dmask = dmask; p.dmask_kind = dmask ? dmask_kind : 0; p.dm_sb = dm_sb; p.dm_sh = dm_sh; p.dm_ld = dm_ld;
  p.dn_rows = dn_rows; p.dn_cols = dn_cols;
  CUtensorMap tq, tk, tv;
  int rc = make_map(&tq, q, Tq, static_cast<long long>(H) * D, ld_q, 64);
  if (rc) return rc;
  if (page_ids) {
    if (page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128) return -5;
    p.box_rows = page_size < 64 ? page_size : 64;
    const long long rows = num_pages * 2 * page_size;
    rc = make_map(&tk, k, rows, static_cast<long long>(H) * D, ld_k, p.box_rows);
    if (rc) return rc;
    tv = tk;
  } else {
    p.box_rows = 64;
    rc = make_map(&tk, k, Tk, static_cast<long long>(H) * D, ld_k, 64);
    if (rc) return rc;
    rc = make_map(&tv, v, Tk, static_cast<long long>(H) * D, ld_k, 64);
    if (rc) return rc;
  }
  const int max_qblocks = (max_len_q + BQ - 1) / BQ;
  const bool bt = ts != nullptr && ts_w != nullptr, bp = pos_w != nullptr;
#define RB_FWD(DD)                                                                  \
  (bt ? (bp ? launch_fwd<DD, true, true>(tq, tk, tv, p, max_qblocks, st)            \
            : launch_fwd<DD, true, false>(tq, tk, tv, p, max_qblocks, st))          \
      : (bp ? launch_fwd<DD, false, true>(tq, tk, tv, p, max_qblocks, st)           \
            : launch_fwd<DD, false, false>(tq, tk, tv, p, max_qblocks, st)))
  if (D == 64) return RB_FWD(64);
  return RB_FWD(128);
#undef RB_FWD
}


RB_API int rb_hstu_attn_fwd(const void* q, long long ld_q, long long Tq, const void* k, const void* v, long long ld_k,
                            long long Tk, const int* q_offsets, const int* k_offsets, int B, int H, int D,
                            int max_len_q, void* out, long long ld_o, float alpha, float scale, int causal,
                            const int* num_context, const int* num_target, int target_group_size, const float* ts,
                            const float* ts_w, int num_buckets, float ts_divisor, const float* pos_w, int pos_len,
                            const int* page_ids, const int* page_indptr, int page_size, long long num_pages,
                            int* status, cudaStream_t st) {
  return hstu_attn_fwd_impl(q, ld_q, Tq, k, v, ld_k, Tk, q_offsets, k_offsets, B, H, D, max_len_q, out, ld_o, alpha, scale, causal,
                            num_context, num_target, target_group_size, ts, ts_w, num_buckets, ts_divisor, pos_w, pos_len,
                            page_ids, page_indptr, page_size, num_pages, status, st, nullptr, 0, 0, 0, 0, nullptr, 0, 0, 0, 0, 0, 0);
}

// Same forward with the dense operands of the reference's convention: attn_bias (bias_kind 1 bf16 / 2 fp32) added to
// Q K^T before the activation and a 0/1 mask (mask_kind 1 uint8 / 2 bf16 / 3 fp32) multiplied onto the result; both are
// indexed [batch][head][query position][key position] through element strides (a head stride of 0 broadcasts);
// positions at or beyond dense_rows / dense_cols read as bias 0, mask 0.
RB_API int rb_hstu_attn_fwd_dense(const void* q, long long ld_q, long long Tq, const void* k, const void* v, long long ld_k,
                                  long long Tk, const int* q_offsets, const int* k_offsets, int B, int H, int D,
                                  int max_len_q, void* out, long long ld_o, float alpha, float scale, int causal,
                                  const int* num_context, const int* num_target, int target_group_size,
                                  const void* attn_bias, int bias_kind, long long bias_stride_b, long long bias_stride_h,
                                  long long bias_ld, const void* mask, int mask_kind, long long mask_stride_b,
                                  long long mask_stride_h, long long mask_ld, int dense_rows, int dense_cols, int* status,
                                  cudaStream_t st) {
  return hstu_attn_fwd_impl(q, ld_q, Tq, k, v, ld_k, Tk, q_offsets, k_offsets, B, H, D, max_len_q, out, ld_o, alpha, scale, causal,
                            num_context, num_target, target_group_size, nullptr, nullptr, 0, 1.f, nullptr, 0, nullptr, nullptr, 0,
                            0, status, st, attn_bias, bias_kind, bias_stride_b, bias_stride_h, bias_ld, mask, mask_kind,
                            mask_stride_b, mask_stride_h, mask_ld, dense_rows, dense_cols);
}
