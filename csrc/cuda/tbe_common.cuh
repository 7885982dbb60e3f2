// Declarations shared by the table-batched embedding kernels (embedding.cu) and the push exchange (a2a_push.cu):
// shard records, row location, 4- and 8-element vector loads/stores with conversion to fp32.
#pragma once
#include "common.cuh"

namespace rbtbe {

enum ShardKind : int { SH_LOCAL = 0, SH_TABLE_WISE = 1, SH_ROW_MOD = 2, SH_ROW_BLOCK = 3 };
enum Pooling : int { POOL_SUM = 0, POOL_MEAN = 1, POOL_NONE = 2 };
enum WDtype : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };
enum OptType : int { OPT_SGD = 0, OPT_ROWWISE_ADAGRAD = 1, OPT_ADAGRAD = 2, OPT_ADAM = 3 };

// One record per feature (bag group); features that share a table carry the same table fields.
// `ptr_index` points into the flat pointer table
// ptrs[ptr_index + rank]; for SH_LOCAL / SH_TABLE_WISE only entry `owner` is used.
struct TableShard {
  int kind;
  int owner;
  int D;
  int D_offset;          // column offset of this table in the pooled output
  long long rows;        // logical row count (bounds check)
  long long block;       // rows per rank for SH_ROW_BLOCK
  long long ptr_index;
  long long key_base;    // first linear key of this table on its owner (backward)
};

template <typename T> struct Ld4;
template <> struct Ld4<float> {
  static __device__ __forceinline__ float4 ld(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void st(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Ld4<__half> {
  static __device__ __forceinline__ float4 ld(const __half* p) {
    uint2 u = *reinterpret_cast<const uint2*>(p);
    float2 a = rb::unpack_f16(u.x), b = rb::unpack_f16(u.y);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void st(__half* p, float4 v) {
    *reinterpret_cast<uint2*>(p) = make_uint2(rb::pack_f16(v.x, v.y), rb::pack_f16(v.z, v.w));
  }
};
template <> struct Ld4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 ld(const __nv_bfloat16* p) {
    uint2 u = *reinterpret_cast<const uint2*>(p);
    float2 a = rb::unpack_bf16(u.x), b = rb::unpack_bf16(u.y);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float4 v) {
    *reinterpret_cast<uint2*>(p) = make_uint2(rb::pack_bf16(v.x, v.y), rb::pack_bf16(v.z, v.w));
  }
};

__device__ __forceinline__ bool locate_row(const TableShard& ts, long long id, int world, int self,
                                           int& rank, long long& row) {
  if (id < 0 || id >= ts.rows) return false;
  switch (ts.kind) {
    case SH_ROW_MOD: rank = static_cast<int>(id % world); row = id / world; break;
    case SH_ROW_BLOCK: rank = static_cast<int>(id / ts.block); row = id % ts.block; break;
    case SH_TABLE_WISE: rank = ts.owner; row = id; break;
    default: rank = self; row = id; break;
  }
  return true;
}

template <typename T> struct Vec8;   // 8 consecutive elements <-> 8 floats
template <> struct Vec8<float> {
  static __device__ __forceinline__ void ld(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void st(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct Vec8<__half> {
  static __device__ __forceinline__ void ld(const __half* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    float2 a = rb::unpack_f16(u.x), b = rb::unpack_f16(u.y), c = rb::unpack_f16(u.z), d = rb::unpack_f16(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
  static __device__ __forceinline__ void st(__half* p, const float (&v)[8]) {
    *reinterpret_cast<uint4*>(p) = make_uint4(rb::pack_f16(v[0], v[1]), rb::pack_f16(v[2], v[3]),
                                              rb::pack_f16(v[4], v[5]), rb::pack_f16(v[6], v[7]));
  }
};
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    float2 a = rb::unpack_bf16(u.x), b = rb::unpack_bf16(u.y), c = rb::unpack_bf16(u.z), d = rb::unpack_bf16(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, const float (&v)[8]) {
    *reinterpret_cast<uint4*>(p) = make_uint4(rb::pack_bf16(v[0], v[1]), rb::pack_bf16(v[2], v[3]),
                                              rb::pack_bf16(v[4], v[5]), rb::pack_bf16(v[6], v[7]));
  }
};

}  // namespace rbtbe
