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
  int kv_pos0, n_total, tile0_global, ntiles_global;
  unsigned flags;
  float sm_scale;
};

// ---- request table of the batched entry ----------------------------------------------
// One buffer, written on the host by akl_batch_plan and read by the batch kernels:
//   BatchHeader | Geom[max_requests] | stat_off[max_requests + 1] | qcta_off[max_requests + 1]
//   | attention work items (int2 {request, q head << 16 | q tile}), longest first.
// stat_off / qcta_off are running totals of the statistics items (64-row tile x kv head) and
// of the Q-quantisation CTAs per request, so a flat item index is mapped back to its request
// by a binary search.
struct BatchHeader {
  int32_t magic;
  int32_t n_requests;
  int32_t n_stat_items;
  int32_t n_q_ctas;
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

// 256-point fast Walsh-Hadamard transform over a warp: lane l holds elements
// 8l..8l+7.  Stage order h = 1, 2, 4 (in registers) then 8..128 (lane exchanges);
// pair (i, i+h) -> (a+b, a-b); final exact scale 1/16.  Additions only, so the
// result is a fixed tree of rounded fp32 adds (the CPU oracle's "butterfly" order).
__device__ __forceinline__ void fwht256(float (&x)[8], int lane) {
#pragma unroll
  for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (!(i & h)) {
        float a = x[i], b = x[i + h];
        x[i] = __fadd_rn(a, b);
        x[i + h] = __fsub_rn(a, b);
      }
    }
  }
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    // upper partner: o - x, lower partner: x + o; as one fused op, fma(+-1, x, o) rounds the
    // same exact sum once, so the bits are those of the add / subtract
    const float sign = (lane & m) ? -1.f : 1.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float o = __shfl_xor_sync(0xffffffffu, x[i], m);
      x[i] = __fmaf_rn(sign, x[i], o);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(x[i], 0.0625f);
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
void note_cuda_error(cudaError_t e, const char* where);

}  // namespace akl
