// Shared device helpers: tile-image addressing, number-format conversion, and the
// launch-geometry struct every phase kernel receives.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/akl.h"

namespace akl {

constexpr int kD = AKL_HEAD_DIM;          // 256 channels
constexpr int kTile = AKL_KV_TILE;        // 64-row quantisation tile
constexpr int kPair = 128;                // two tiles: one MMA-N block of keys
constexpr int kQTile = AKL_Q_TILE;        // 128 query rows per CTA
constexpr int kPlaneBytes = 128 * 128;    // one [128 rows][128 B] swizzled plane
constexpr int kImageBytes = 2 * kPlaneBytes;  // one 128-row x 256-byte operand tile
constexpr float kFp8Max = 448.0f;
constexpr float kInt8Max = 127.0f;
constexpr int kSlabTiles = AKL_STAT_SLAB / AKL_KV_TILE;

// Everything a phase kernel needs, resolved on the host from akl_call_t + layout.
struct Geom {
  const void* q;
  const void* k_pool;
  const void* v_pool;
  const void* idx;
  void* out;
  float* lse_out;
  uint8_t* q8;
  float* qscale;
  // batched entry only: Q rows of the q heads that share a kv head packed into common 128-row
  // tiles, row R = token * (Hq / Hkv) + (head inside the group); images [Hkv][group * mtiles_cap]
  uint8_t* q8p;
  float* qscalep;
  uint8_t* k8;
  uint8_t* v8t;
  float* kscale;
  float* vst;
  float* vlog2r;
  float* vinvr;
  float* vam;
  float* vscale;
  float* vsmax;
  float* kmean;
  float* vmean;
  float* ktsum;   // [ntiles_cap][Hkv][256], GLOBAL tile order
  float* vtsum;
  float* vtmax;   // [Hkv][ntiles_cap][256], local tile order
  float* vtmin;
  int* status;
  float* dbg_s;    // optional [Hq][mtiles][nt][128][64] raw QK^T accumulators (diagnostic entry only)
  uint8_t* dbg_p;  // optional, same shape: the E4M3 P bytes fed to the PV MMA
  int T, N, prefix, Hq, Hkv;
  int npairs_cap, ntiles_cap, mtiles_cap;
  int nt;          // local 64-row tiles = ceil(N / 64)
  int mtiles;      // ceil(T / 128)
  int ptiles;      // batched entry: packed Q tiles per kv head = ceil(T * (Hq / Hkv) / 128)
  int kv_pos0, n_total, tile0_global, ntiles_global;
  unsigned flags;
  float sm_scale;
};

// ---- request table of the batched entry ----------------------------------------------
// One buffer, written on the host by akl_batch_plan and read by the batch kernels:
//   BatchHeader | Geom[max_requests] | stat_off[max_requests + 1] | qcta_off[max_requests + 1]
//   | attention work items (int2 {request, q head << 16 | q tile}), longest first.
// stat_off / qcta_off are running totals of the statistics items (64-row tile x kv head) and
// of the packed Q tiles (128 (token, head) rows of one kv head's group) per request, so a flat
// item index is mapped back to its request by a binary search.
struct BatchHeader {
  int32_t magic;
  int32_t n_requests;
  int32_t n_stat_items;
  int32_t n_q_ctas;       // packed Q tiles over all requests (each is quantised as two 64-row items)
  int32_t n_attn_items;
  int32_t attn_counter;   // device side: next attention work item (reset by the means launch)
  int32_t reserved[10];
};
static_assert(sizeof(BatchHeader) == 64, "table header is 64 bytes");
constexpr int32_t kBatchMagic = 0x424c4b41;

struct BatchRef {
  uint8_t* table;
  uint32_t off_geoms, off_stat_off, off_qcta_off, off_items;
  int32_t max_requests;
};

__host__ __device__ __forceinline__ BatchHeader* batch_header(const BatchRef& b) {
  return reinterpret_cast<BatchHeader*>(b.table);
}

// Byte offset of (row r, byte column c) inside a [rows][128 B] plane stored with the
// 128-byte swizzle the tensor-core shared-memory descriptors expect: the 16-byte chunk
// index is XORed with the row index modulo 8.
__host__ __device__ __forceinline__ uint32_t swz128(uint32_t r, uint32_t c) {
  return r * 128u + ((((c >> 4) ^ (r & 7u)) << 4) | (c & 15u));
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t b) {
  return __uint_as_float(b << 16);
}

// 8 consecutive 16-bit values (one 16-byte load) -> 8 floats
template <int KV_DTYPE>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&x)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (KV_DTYPE == AKL_KV_BF16) {
      x[2 * i] = bf16_bits_to_float(w[i] & 0xFFFFu);
      x[2 * i + 1] = bf16_bits_to_float(w[i] >> 16);
    } else {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      float2 f = __half22float2(h);
      x[2 * i] = f.x;
      x[2 * i + 1] = f.y;
    }
  }
}

// float -> E4M3 byte, round-to-nearest-even, saturating (cvt.rn.satfinite.e4m3x2.f32).
// Returns two bytes: lo in bits 0-7, hi in bits 8-15.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
  return cvt_e4m3x2(a, b) | (cvt_e4m3x2(c, d) << 16);
}

// float -> INT8 byte, round half to even (the quotient is bounded by 127 (1 + 2 eps), so there
// is nothing to clamp).  Four bytes, first value in bits 0-7.
__device__ __forceinline__ uint32_t cvt_s8x4(float a, float b, float c, float d) {
  return (static_cast<uint32_t>(__float2int_rn(a)) & 0xFFu) | ((static_cast<uint32_t>(__float2int_rn(b)) & 0xFFu) << 8) |
         ((static_cast<uint32_t>(__float2int_rn(c)) & 0xFFu) << 16) | (static_cast<uint32_t>(__float2int_rn(d)) << 24);
}

// Q/K bytes in the call's QK operand type
__device__ __forceinline__ uint32_t cvt_qk_x4(bool i8, float a, float b, float c, float d) {
  return i8 ? cvt_s8x4(a, b, c, d) : cvt_e4m3x4(a, b, c, d);
}

// ---- packed fp32 pairs ------------------------------------------------------------------
// One issue slot for two IEEE round-to-nearest operations; bit-identical to the scalar forms.
// The preprocessing kernels are bound by instruction issue (a 256-point rotation and an exact
// division per element), so halving the arithmetic instruction count is what speeds them up.
struct f2 { unsigned long long v; };
__device__ __forceinline__ f2 pack2(float a, float b) {
  f2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r.v) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(f2 p, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(p.v));
}
__device__ __forceinline__ f2 add2p(f2 a, f2 b) {
  f2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
  return r;
}
__device__ __forceinline__ f2 sub2p(f2 a, f2 b) {
  f2 r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
  return r;
}
__device__ __forceinline__ f2 mul2p(f2 a, f2 b) {
  f2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
  return r;
}
__device__ __forceinline__ f2 fma2p(f2 a, f2 b, f2 c) {
  f2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.v) : "l"(a.v), "l"(b.v), "l"(c.v));
  return r;
}

// x[0..7] -= m[0..7]: four packed subtractions.
__device__ __forceinline__ void sub8(float (&x)[8], const float (&m)[8]) {
#pragma unroll
  for (int i = 0; i < 8; i += 2) unpack2(sub2p(pack2(x[i], x[i + 1]), pack2(m[i], m[i + 1])), x[i], x[i + 1]);
}

// Exact division by a divisor that many dividends share (a tile's or a row's scale):
// q = RN(x / s) with the bits of an IEEE division, in three packed operations per two dividends
// instead of one division routine per dividend.  With r = RN(1 / s):
//   q0 = RN(x r);  e = x - q0 s  (one fused operation, exact);  q = RN(q0 + e r).
// That is the final step of the textbook division by reciprocal (Markstein): a correctly rounded
// reciprocal and a quotient within one ulp give the correctly rounded quotient, provided nothing
// leaves the normal range on the way.  `exact` is false where that proviso could fail -- divisor
// or quotients too close to the ends of the exponent range, or a divisor whose significand is
// all ones (the one pattern the theorem excludes) -- and the caller divides the slow way there.
// The operator's divisors are amax/448 or amax/127 with amax >= 1e-8 and |x| <= amax, so the
// fast path is the one that runs; an exhaustive check over every dividend significand backs it
// (the division self-test of the library).
struct ExactDiv {
  float s, r, neg_s;
  bool exact;
};
__device__ __forceinline__ ExactDiv make_exact_div(float s) {
  ExactDiv d;
  d.s = s;
  d.neg_s = -s;
  d.r = __frcp_rn(s);
  const unsigned bits = __float_as_uint(s);
  const unsigned e = (bits >> 23) & 0xFFu;
  // |x| <= 512 |s| in this operator, so quotients stay far inside the range; the divisor's own
  // exponent must leave room for r and for the exact remainder x - q0 s (24 more bits below x)
  d.exact = (e >= 40u && e <= 200u) && ((bits & 0x7FFFFFu) != 0x7FFFFFu);
  return d;
}
// y[i] = x[i] / s for i = 0..7, to be rounded to an 8-bit code by the caller.  For |x| >= 2^-100
// (or zero) y is RN(x / s) bit for bit.  Below that the remainder may be inexact, but then
// |x / s| < 2^-13 (s >= 2^-87 on this path), and that quotient and the IEEE one both round to the
// same signed zero in E4M3 and in INT8.
__device__ __forceinline__ void div8(const ExactDiv& d, const float (&x)[8], float (&y)[8]) {
  if (d.exact) {
    const f2 r = pack2(d.r, d.r), ns = pack2(d.neg_s, d.neg_s);
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const f2 xv = pack2(x[i], x[i + 1]);
      const f2 q0 = mul2p(xv, r);
      const f2 e = fma2p(q0, ns, xv);
      unpack2(fma2p(e, r, q0), y[i], y[i + 1]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = __fdiv_rn(x[i], d.s);
  }
}

// 256-point fast Walsh-Hadamard transform over a warp: lane l holds elements
// 8l..8l+7.  Stage order h = 1, 2, 4 (in registers) then 8..128 (lane exchanges);
// pair (i, i+h) -> (a+b, a-b); final exact scale 1/16.  Additions only, so the
// result is a fixed tree of rounded fp32 adds (the CPU oracle's "butterfly" order).
// Stages h = 2, 4, the lane exchanges and the scale run as packed pairs.
__device__ __forceinline__ void fwht256(float (&x)[8], int lane) {
#pragma unroll
  for (int i = 0; i < 8; i += 2) {          // h = 1
    const float a = x[i], b = x[i + 1];
    x[i] = __fadd_rn(a, b);
    x[i + 1] = __fsub_rn(a, b);
  }
  f2 p[4] = {pack2(x[0], x[1]), pack2(x[2], x[3]), pack2(x[4], x[5]), pack2(x[6], x[7])};
  {                                         // h = 2: (0,1)+-(2,3), (4,5)+-(6,7)
    const f2 a0 = add2p(p[0], p[1]), a1 = sub2p(p[0], p[1]), a2 = add2p(p[2], p[3]), a3 = sub2p(p[2], p[3]);
    p[0] = a0; p[1] = a1; p[2] = a2; p[3] = a3;
  }
  {                                         // h = 4: (0,1)+-(4,5), (2,3)+-(6,7)
    const f2 a0 = add2p(p[0], p[2]), a2 = sub2p(p[0], p[2]), a1 = add2p(p[1], p[3]), a3 = sub2p(p[1], p[3]);
    p[0] = a0; p[1] = a1; p[2] = a2; p[3] = a3;
  }
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    // upper partner: o - x, lower partner: x + o; as one fused op, fma(+-1, x, o) rounds the
    // same exact sum once, so the bits are those of the add / subtract
    const float sign = (lane & m) ? -1.f : 1.f;
    const f2 sg = pack2(sign, sign);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f2 o;
      o.v = __shfl_xor_sync(0xffffffffu, p[i].v, m);
      p[i] = fma2p(sg, p[i], o);
    }
  }
  const f2 sixteenth = pack2(0.0625f, 0.0625f);
#pragma unroll
  for (int i = 0; i < 4; ++i) unpack2(mul2p(p[i], sixteenth), x[2 * i], x[2 * i + 1]);
}

// The same transform with a row spread over FOUR lanes: lane q (= lane & 3) holds the channels
// 32k + 8q + c, k = 0..7, c = 0..7, as x[k][c].  Stages h = 1, 2, 4 run inside x[k][.], h = 8, 16
// are the only lane exchanges (partners lane ^ 1, lane ^ 2), h = 32, 64, 128 run across k in
// registers: 128 shuffles per 64 elements instead of 320, and the same pairs, the same order of
// stages, the same rounded additions - so the same bits.
__device__ __forceinline__ void fwht256_quarter(float (&x)[8][8], int lane) {
  f2 p[8][4];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
#pragma unroll
    for (int i = 0; i < 8; i += 2) {          // h = 1
      const float a = x[k][i], b = x[k][i + 1];
      x[k][i] = __fadd_rn(a, b);
      x[k][i + 1] = __fsub_rn(a, b);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) p[k][i] = pack2(x[k][2 * i], x[k][2 * i + 1]);
    {                                         // h = 2
      const f2 a0 = add2p(p[k][0], p[k][1]), a1 = sub2p(p[k][0], p[k][1]), a2 = add2p(p[k][2], p[k][3]), a3 = sub2p(p[k][2], p[k][3]);
      p[k][0] = a0; p[k][1] = a1; p[k][2] = a2; p[k][3] = a3;
    }
    {                                         // h = 4
      const f2 a0 = add2p(p[k][0], p[k][2]), a2 = sub2p(p[k][0], p[k][2]), a1 = add2p(p[k][1], p[k][3]), a3 = sub2p(p[k][1], p[k][3]);
      p[k][0] = a0; p[k][1] = a1; p[k][2] = a2; p[k][3] = a3;
    }
  }
#pragma unroll
  for (int m = 1; m < 4; m <<= 1) {           // h = 8, 16: upper partner o - x, lower partner x + o
    const float sign = (lane & m) ? -1.f : 1.f;
    const f2 sg = pack2(sign, sign);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        f2 o;
        o.v = __shfl_xor_sync(0xffffffffu, p[k][i].v, m);
        p[k][i] = fma2p(sg, p[k][i], o);
      }
    }
  }
#pragma unroll
  for (int hk = 1; hk < 8; hk <<= 1) {        // h = 32, 64, 128: pairs (k, k + hk)
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (k & hk) continue;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const f2 a = p[k][i], b = p[k + hk][i];
        p[k][i] = add2p(a, b);
        p[k + hk][i] = sub2p(a, b);
      }
    }
  }
  const f2 sixteenth = pack2(0.0625f, 0.0625f);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
#pragma unroll
    for (int i = 0; i < 4; ++i) unpack2(mul2p(p[k][i], sixteenth), x[k][2 * i], x[k][2 * i + 1]);
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
  return v;
}

template <int IDX_DTYPE>
__device__ __forceinline__ long long load_idx(const void* idx, int i) {
  if (IDX_DTYPE == AKL_IDX_I64) return reinterpret_cast<const long long*>(idx)[i];
  return static_cast<long long>(reinterpret_cast<const int*>(idx)[i]);
}

// host-side launchers (one translation unit each)
int launch_kv_tile_stats(const Geom& g, int kv_dtype, int idx_dtype, cudaStream_t s, bool with_q = false);
int launch_kv_means(const Geom& g, cudaStream_t s, bool fuse_scales = false);
int launch_kv_scales(const Geom& g, cudaStream_t s);
int launch_kv_transform(const Geom& g, int kv_dtype, int idx_dtype, cudaStream_t s);
int launch_quantize_q(const Geom& g, cudaStream_t s);
int launch_attention(const Geom& g, cudaStream_t s, bool dump = false);
int launch_merge(const akl_merge_t& m, cudaStream_t s);
// batched forms: every kernel reads counts and per-request geometry from the request table
int launch_batch_stats(const BatchRef& b, int kv_dtype, int idx_dtype, int sm_count, cudaStream_t s);
int launch_batch_means(const BatchRef& b, int kv_heads, cudaStream_t s);
int launch_batch_transform(const BatchRef& b, int kv_dtype, int idx_dtype, int sm_count, cudaStream_t s);
int launch_batch_attention(const BatchRef& b, bool qk_i8, int sm_count, cudaStream_t s);
int launch_exact_division_selftest(const float* scales, int n, unsigned long long* mismatches, cudaStream_t s);
void note_cuda_error(cudaError_t e, const char* where);
int validate_prefill_call(const akl_call_t* c, Geom* g);

}  // namespace akl
