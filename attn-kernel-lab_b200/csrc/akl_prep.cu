// Preprocessing kernels: paged gather, K/V statistics, K/V transform + quantisation, Q
// rotation + quantisation.  They replace the tensor-library pipeline of the reference's
// src/attn_kernel_lab/quant.py:433-695 (about 14 launches per call) with five launches.
//
// All arithmetic that decides a quantised byte is plain IEEE fp32 in a fixed order; this
// file is compiled with -fmad=false so no multiply-add is ever contracted.
//
// Work decomposition (HBM-bound byte work, so: 16-byte coalesced loads, one full 512-byte
// row per warp-load, 64 KiB in flight per CTA, grids of nt*Hkv CTAs):
//   CTA  = one 64-row tile of one kv head, 256 threads;
//   warp = 8 consecutive rows of the tile;
//   lane = 8 consecutive channels (one 16-byte load per row).
#include <atomic>

#include "akl_common.cuh"
#include "akl_sm100_ptx.cuh"

namespace akl {

namespace {

constexpr int kThreads = 256;

// ---------------------------------------------------------------------------
// 1. per-tile channel sums of K and V, per-tile channel min/max of V
//    (reference pass 1, quant.py:532-568)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void quantize_q_rows(const Geom& g, long long cta);

// Flat grid: CTAs [0, nt*Hkv) take one (tile, kv head) each; with kWithQ the CTAs after them
// quantise Q rows, so that the two independent passes share one launch and overlap.
// `item` = tile * Hkv + kv head.  Ends with every thread past its last shared-memory read of
// the tile, but not synchronised: a caller that runs several items per CTA synchronises between them.
template <int KV_DTYPE, int IDX_DTYPE>
__device__ __forceinline__ void kv_tile_stats_item(const Geom& g, int item) {
  __shared__ __align__(16) float sm_k[8][kD];
  __shared__ __align__(16) float sm_v[8][kD];
  __shared__ __align__(16) float sm_mx[8][kD];
  __shared__ __align__(16) float sm_mn[8][kD];
  const int t = item / g.Hkv, kvh = item % g.Hkv;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = t * kTile + w * 8;

  // pool rows of this warp's 8 positions
  long long pr = 0;
  if (lane < 8 && row0 + lane < g.N) pr = load_idx<IDX_DTYPE>(g.idx, row0 + lane);
  // the warp's 8 rows in four passes of 2 (4 x 16 bytes in flight per thread, four CTAs per SM);
  // the running sums see the rows in position order either way
  float ks[8], vs[8], mx[8], mn[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) { ks[c] = 0.f; vs[c] = 0.f; mx[c] = -INFINITY; mn[c] = INFINITY; }
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    uint4 kraw[2], vraw[2];
#pragma unroll
    for (int ii = 0; ii < 2; ++ii) {
      const int i = pass * 2 + ii;
      long long p = __shfl_sync(0xffffffffu, pr, i);
      if (row0 + i < g.N) {
        size_t off = (static_cast<size_t>(p) * g.Hkv + kvh) * kD + lane * 8;
        kraw[ii] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(g.k_pool) + off));
        vraw[ii] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(g.v_pool) + off));
      }
    }
#pragma unroll
    for (int ii = 0; ii < 2; ++ii) {
      const int i = pass * 2 + ii;
      if (row0 + i < g.N) {
        float kx[8], vx[8];
        unpack8<KV_DTYPE>(kraw[ii], kx);
        unpack8<KV_DTYPE>(vraw[ii], vx);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          ks[c] = __fadd_rn(ks[c], kx[c]);
          vs[c] = __fadd_rn(vs[c], vx[c]);
          mx[c] = fmaxf(mx[c], vx[c]);
          mn[c] = fminf(mn[c], vx[c]);
        }
      }
    }
  }
  // 16-byte stores: a quarter-warp's eight stores cover all 32 banks once (scalar stores of
  // lane * 8 + c would meet four banks eight deep)
  {
    float4* pk = reinterpret_cast<float4*>(&sm_k[w][lane * 8]);
    float4* pv = reinterpret_cast<float4*>(&sm_v[w][lane * 8]);
    float4* px = reinterpret_cast<float4*>(&sm_mx[w][lane * 8]);
    float4* pn = reinterpret_cast<float4*>(&sm_mn[w][lane * 8]);
    pk[0] = make_float4(ks[0], ks[1], ks[2], ks[3]); pk[1] = make_float4(ks[4], ks[5], ks[6], ks[7]);
    pv[0] = make_float4(vs[0], vs[1], vs[2], vs[3]); pv[1] = make_float4(vs[4], vs[5], vs[6], vs[7]);
    px[0] = make_float4(mx[0], mx[1], mx[2], mx[3]); px[1] = make_float4(mx[4], mx[5], mx[6], mx[7]);
    pn[0] = make_float4(mn[0], mn[1], mn[2], mn[3]); pn[1] = make_float4(mn[4], mn[5], mn[6], mn[7]);
  }
  __syncthreads();
  // the eight 8-row run sums are added in run order
  const int c = threadIdx.x;
  float sk = 0.f, sv = 0.f, vmx = -INFINITY, vmn = INFINITY;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    sk = __fadd_rn(sk, sm_k[r][c]);
    sv = __fadd_rn(sv, sm_v[r][c]);
    vmx = fmaxf(vmx, sm_mx[r][c]);
    vmn = fminf(vmn, sm_mn[r][c]);
  }
  const size_t gt = static_cast<size_t>(g.tile0_global + t);
  g.ktsum[(gt * g.Hkv + kvh) * kD + c] = sk;
  g.vtsum[(gt * g.Hkv + kvh) * kD + c] = sv;
  g.vtmax[(static_cast<size_t>(kvh) * g.ntiles_cap + t) * kD + c] = vmx;
  g.vtmin[(static_cast<size_t>(kvh) * g.ntiles_cap + t) * kD + c] = vmn;
}

template <int KV_DTYPE, int IDX_DTYPE, bool kWithQ>
__global__ void __launch_bounds__(kThreads, 4) kv_tile_stats_kernel(Geom g) {
  const int nstat = g.nt * g.Hkv;
  if (kWithQ && static_cast<int>(blockIdx.x) >= nstat) {
    quantize_q_rows(g, static_cast<long long>(blockIdx.x) - nstat);
    return;
  }
  kv_tile_stats_item<KV_DTYPE, IDX_DTYPE>(g, blockIdx.x);
}

// ---------------------------------------------------------------------------
// 2. channel means (ordered: tiles inside a 32768-row slab, then slabs) and the
//    centred per-tile V amax  (quant.py:566-581)
// ---------------------------------------------------------------------------
constexpr int kMeansThreads = 1024;

__device__ __forceinline__ void write_tile_scales(const Geom& g, int kvh, int t, float vsm, float floor_) {
  const int o = kvh * g.ntiles_cap + t;
  const float vst = __fdiv_rn(fmaxf(g.vam[o], floor_), kFp8Max);
  float r = __fdiv_rn(__fmul_rn(vst, kFp8Max), vsm);
  r = fminf(fmaxf(r, 0.0625f), 1.0f);
  g.vst[o] = vst;
  g.vlog2r[o] = log2f(r);
  g.vinvr[o] = __fdiv_rn(1.0f, r);
}

// One CTA per kv head.  Threads 0-255 add the K tile sums of their channel in tile order inside
// each 32768-row slab and the slab sums in slab order; threads 256-511 do the same for V (eight
// loads are kept in flight; the additions stay strictly ordered).  Then 32 warps form the
// centred per-tile V amax.  With `fuse_scales` (one GPU holds the whole request) the per-tile V
// scales and fold arrays follow in the same launch.
template <bool kFuseScales>
__device__ __forceinline__ void kv_means_head(const Geom& g, int kvh) {
  __shared__ float sm_vmean[kD];
  __shared__ float sm_wmax[32];
  __shared__ float sm_vsm;
  const int tid = threadIdx.x;
  const int ntg = g.ntiles_global;
  if (tid < 2 * kD) {
    const int c = tid & (kD - 1);
    const bool is_v = tid >= kD;
    const float* src = (is_v ? g.vtsum : g.ktsum) + static_cast<size_t>(kvh) * kD + c;
    const size_t stride = static_cast<size_t>(g.Hkv) * kD;
    float tot = 0.f;
    for (int s0 = 0; s0 < ntg; s0 += kSlabTiles) {
      const int s1 = min(s0 + kSlabTiles, ntg);
      float slab = 0.f;
      int t = s0;
      for (; t + 8 <= s1; t += 8) {
        float x[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = src[(t + i) * stride];
#pragma unroll
        for (int i = 0; i < 8; ++i) slab = __fadd_rn(slab, x[i]);
      }
      for (; t < s1; ++t) slab = __fadd_rn(slab, src[t * stride]);
      tot = __fadd_rn(tot, slab);
    }
    const float denom = static_cast<float>(max(g.n_total, 1));
    if (is_v) {
      const float vmean = __fdiv_rn(tot, denom);
      g.vmean[kvh * kD + c] = vmean;
      sm_vmean[c] = vmean;
    } else {
      g.kmean[kvh * kD + c] = (g.flags & AKL_FLAG_CENTER_K) ? __fdiv_rn(tot, denom) : 0.f;
    }
  }
  __syncthreads();
  // vam[t] = max_c max(fl(mx - mean), fl(mean - mn)); one warp per tile
  const int w = tid >> 5, lane = tid & 31;
  float wmax = 0.f;
  for (int t = w; t < g.nt; t += kMeansThreads / 32) {
    const float* pmx = g.vtmax + (static_cast<size_t>(kvh) * g.ntiles_cap + t) * kD;
    const float* pmn = g.vtmin + (static_cast<size_t>(kvh) * g.ntiles_cap + t) * kD;
    float a = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int ch = lane + 32 * j;
      const float m = sm_vmean[ch];
      a = fmaxf(a, fmaxf(__fsub_rn(pmx[ch], m), __fsub_rn(m, pmn[ch])));
    }
    a = warp_max(a);
    if (lane == 0) g.vam[kvh * g.ntiles_cap + t] = a;
    wmax = fmaxf(wmax, a);
  }
  if (lane == 0) sm_wmax[w] = wmax;
  __syncthreads();
  if (tid == 0) {
    float m = 0.f;
    for (int i = 0; i < kMeansThreads / 32; ++i) m = fmaxf(m, sm_wmax[i]);
    g.vsmax[kvh] = m;   // raw, unclamped: a MAX all-reduce may combine ranks here
    sm_vsm = fmaxf(m, 1e-8f);
    if (kFuseScales) g.vscale[kvh] = __fdiv_rn(sm_vsm, kFp8Max);
  }
  if (kFuseScales) {
    __syncthreads();       // also orders this CTA's vam stores before the loads below
    const float vsm = sm_vsm;
    const float floor_ = __fdiv_rn(vsm, 16.0f);
    for (int t = tid; t < g.nt; t += kMeansThreads) write_tile_scales(g, kvh, t, vsm, floor_);
  }
}

template <bool kFuseScales>
__global__ void __launch_bounds__(kMeansThreads) kv_means_kernel(Geom g) {
  kv_means_head<kFuseScales>(g, blockIdx.x);
}

// ---------------------------------------------------------------------------
// 3. per-tile V scales and the fold arrays  (quant.py:576-584, :673-679)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) kv_scales_kernel(Geom g) {
  const int kvh = blockIdx.x;
  const float vsm = fmaxf(g.vsmax[kvh], 1e-8f);
  const float floor_ = __fdiv_rn(vsm, 16.0f);
  for (int t = threadIdx.x; t < g.nt; t += blockDim.x) write_tile_scales(g, kvh, t, vsm, floor_);
  if (threadIdx.x == 0) g.vscale[kvh] = __fdiv_rn(vsm, kFp8Max);
}

// ---------------------------------------------------------------------------
// 4. K: gather, centre, rotate, per-tile amax, E4M3  -> swizzled [pair][2][128][128] image
//    V: gather, centre, per-tile scale, E4M3, transpose -> swizzled [pair][256][128] image
//    (quant.py:589-668).  blockIdx.z: 0 = K, 1 = V.
// ---------------------------------------------------------------------------
// The gather of one (64-row tile, kv head, K or V): this warp's eight rows, 16 bytes per lane each.
template <int IDX_DTYPE>
__device__ __forceinline__ void load_tile_rows(const Geom& g, int t, int kvh, bool is_v, uint4 (&raw)[8]) {
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = t * kTile + w * 8;
  const void* pool = is_v ? g.v_pool : g.k_pool;
  long long pr = 0;
  if (lane < 8 && row0 + lane < g.N) pr = load_idx<IDX_DTYPE>(g.idx, row0 + lane);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    long long p = __shfl_sync(0xffffffffu, pr, i);
    if (row0 + i < g.N) {
      size_t off = (static_cast<size_t>(p) * g.Hkv + kvh) * kD + lane * 8;
      raw[i] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(pool) + off));
    }
  }
}

// V transpose staging: row d (channel) holds its 64 key bytes as eight 8-byte slots; rows are
// 72 bytes apart and slot q of row d sits at position q ^ ((d >> 4) & 7).  A half-warp's stores
// (rows 8 apart, one slot each) and its loads (16 consecutive rows, one slot each) then touch
// sixteen different 8-byte bank pairs; an unswizzled 80-byte row met two of them sixteen deep.
constexpr int kVRow = 72;
constexpr int kVStagingBytes = kD * kVRow;

// `sm_vt`: kVStagingBytes of shared memory, 16-byte aligned, that no thread still reads for
// anything else (the V path writes it without a barrier of its own).  `mp`: this lane's eight
// channel means (global or shared memory, 16-byte aligned).  `v_scale`: the tile's V scale
// (ignored for K, whose scale is formed here).
template <int KV_DTYPE>
__device__ __forceinline__ void transform_tile_rows(const Geom& g, int t, int kvh, bool is_v, const uint4 (&raw)[8], uint8_t* sm_vt,
                                                    const float* mp, float v_scale) {
  __shared__ float sm_red[8];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = t * kTile + w * 8;
  float mean[8];
  {
    const float4 m0 = *reinterpret_cast<const float4*>(mp);
    const float4 m1 = *reinterpret_cast<const float4*>(mp + 4);
    mean[0] = m0.x; mean[1] = m0.y; mean[2] = m0.z; mean[3] = m0.w;
    mean[4] = m1.x; mean[5] = m1.y; mean[6] = m1.z; mean[7] = m1.w;
  }
  const bool center = is_v || (g.flags & AKL_FLAG_CENTER_K);
  const bool rotate = !is_v && (g.flags & AKL_FLAG_ROTATE);
  const bool qk_i8 = !is_v && (g.flags & AKL_FLAG_QK_I8);     // V is E4M3 in both modes

  float x[8][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (row0 + i < g.N) {          // warp-uniform
      unpack8<KV_DTYPE>(raw[i], x[i]);
      if (center) sub8(x[i], mean);
      if (rotate) fwht256(x[i], lane);
#pragma unroll
      for (int c = 0; c < 8; ++c) amax = fmaxf(amax, fabsf(x[i][c]));
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) x[i][c] = 0.f;   // padding rows are exact zeros
    }
  }

  float scale;
  if (!is_v) {
    amax = warp_max(amax);
    if (lane == 0) sm_red[w] = amax;
    __syncthreads();
    float a = sm_red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) a = fmaxf(a, sm_red[i]);
    a = fmaxf(a, 1e-8f);
    scale = __fdiv_rn(a, qk_i8 ? kInt8Max : kFp8Max);
    if (threadIdx.x == 0) g.kscale[kvh * g.ntiles_cap + t] = scale;
  } else {
    scale = v_scale;
  }

  const ExactDiv dv = make_exact_div(scale);
  uint32_t lo[8], hi[8];          // bytes of channels 0-3 / 4-7 of each row
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float y[8];
    div8(dv, x[i], y);
    lo[i] = cvt_qk_x4(qk_i8, y[0], y[1], y[2], y[3]);
    hi[i] = cvt_qk_x4(qk_i8, y[4], y[5], y[6], y[7]);
  }

  const int pair = t >> 1, half = t & 1;
  if (!is_v) {
    uint8_t* img = g.k8 + (static_cast<size_t>(kvh) * g.npairs_cap + pair) * kImageBytes;
    const int plane = lane >> 4;
    const uint32_t cbyte = (lane & 15) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t r = half * 64 + w * 8 + i;
      *reinterpret_cast<uint2*>(img + plane * kPlaneBytes + swz128(r, cbyte)) = make_uint2(lo[i], hi[i]);
    }
  } else {
    // transpose through shared memory: sm_vt[d][key]
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      // byte (c & 3) of rows 0-3 and of rows 4-7: three byte permutes per word
      const uint32_t* src = (c < 4) ? lo : hi;
      const uint32_t sel = (c & 3) | ((4 + (c & 3)) << 4);
      const uint32_t b0 = __byte_perm(__byte_perm(src[0], src[1], sel), __byte_perm(src[2], src[3], sel), 0x5410);
      const uint32_t b1 = __byte_perm(__byte_perm(src[4], src[5], sel), __byte_perm(src[6], src[7], sel), 0x5410);
      const int d = lane * 8 + c;
      *reinterpret_cast<uint2*>(sm_vt + d * kVRow + ((w ^ ((d >> 4) & 7)) * 8)) = make_uint2(b0, b1);
    }
    __syncthreads();
    const int d = threadIdx.x;
    uint8_t* img = g.v8t + (static_cast<size_t>(kvh) * g.npairs_cap + pair) * kImageBytes;
    const int sw = (d >> 4) & 7;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint2 lo2 = *reinterpret_cast<const uint2*>(sm_vt + d * kVRow + (((2 * j) ^ sw) * 8));
      const uint2 hi2 = *reinterpret_cast<const uint2*>(sm_vt + d * kVRow + (((2 * j + 1) ^ sw) * 8));
      *reinterpret_cast<uint4*>(img + swz128(d, half * 64 + j * 16)) = make_uint4(lo2.x, lo2.y, hi2.x, hi2.y);
    }
  }
}

// K out of a row stage in shared memory, a row spread over four lanes (fwht256_quarter): warp w
// transforms rows 8w .. 8w+7 of the tile, lane = 4 * (row in the warp) + quarter.  `rows`: the 64
// rows of 512 bytes; `mean`: the kv head's 256 channel means (shared memory).  Same bytes as the
// K path of transform_tile_rows.
template <int KV_DTYPE>
__device__ __forceinline__ void transform_k_tile_staged(const Geom& g, int t, int kvh, const uint8_t* rows, const float* mean) {
  __shared__ float sm_redk[8];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = lane & 3, lr = w * 8 + (lane >> 2);          // row inside the tile
  const bool live = t * kTile + lr < g.N;
  const bool center = (g.flags & AKL_FLAG_CENTER_K) != 0;
  const bool rotate = (g.flags & AKL_FLAG_ROTATE) != 0;
  const bool qk_i8 = (g.flags & AKL_FLAG_QK_I8) != 0;
  float x[8][8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (live) {
      const uint4 raw = *reinterpret_cast<const uint4*>(rows + lr * (kD * 2) + k * 64 + q * 16);
      unpack8<KV_DTYPE>(raw, x[k]);
      if (center) {
        const float4 m0 = *reinterpret_cast<const float4*>(mean + k * 32 + q * 8);
        const float4 m1 = *reinterpret_cast<const float4*>(mean + k * 32 + q * 8 + 4);
        const float m[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        sub8(x[k], m);
      }
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) x[k][c] = 0.f;             // padding rows are exact zeros
    }
  }
  if (rotate) fwht256_quarter(x, lane);                      // rows past the end rotate zeros: the exchanges stay warp-wide
  float amax = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
#pragma unroll
    for (int c = 0; c < 8; ++c) amax = fmaxf(amax, fabsf(x[k][c]));
  }
  amax = warp_max(amax);
  if (lane == 0) sm_redk[w] = amax;
  __syncthreads();
  float a = sm_redk[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) a = fmaxf(a, sm_redk[i]);
  a = fmaxf(a, 1e-8f);
  const float scale = __fdiv_rn(a, qk_i8 ? kInt8Max : kFp8Max);
  if (threadIdx.x == 0) g.kscale[kvh * g.ntiles_cap + t] = scale;

  const ExactDiv dv = make_exact_div(scale);
  const int pair = t >> 1, half = t & 1;
  uint8_t* img = g.k8 + (static_cast<size_t>(kvh) * g.npairs_cap + pair) * kImageBytes;
  const uint32_t r = half * 64 + lr;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float y[8];
    div8(dv, x[k], y);
    const uint32_t lo = cvt_qk_x4(qk_i8, y[0], y[1], y[2], y[3]);
    const uint32_t hi = cvt_qk_x4(qk_i8, y[4], y[5], y[6], y[7]);
    *reinterpret_cast<uint2*>(img + (k >> 2) * kPlaneBytes + swz128(r, (k & 3) * 32 + q * 8)) = make_uint2(lo, hi);
  }
}

template <int KV_DTYPE, int IDX_DTYPE>
__device__ __forceinline__ void kv_transform_item(const Geom& g, int t, int kvh, bool is_v) {
  __shared__ __align__(16) uint8_t sm_vt[kVStagingBytes];
  uint4 raw[8];
  load_tile_rows<IDX_DTYPE>(g, t, kvh, is_v, raw);
  transform_tile_rows<KV_DTYPE>(g, t, kvh, is_v, raw, sm_vt, (is_v ? g.vmean : g.kmean) + kvh * kD + (threadIdx.x & 31) * 8,
                                is_v ? g.vst[kvh * g.ntiles_cap + t] : 0.f);
}

template <int KV_DTYPE, int IDX_DTYPE>
__global__ void __launch_bounds__(kThreads, 3) kv_transform_kernel(Geom g) {
  kv_transform_item<KV_DTYPE, IDX_DTYPE>(g, blockIdx.x, blockIdx.y, blockIdx.z == 1);
}

// ---------------------------------------------------------------------------
// 5. Q: rotate, per-row amax, E4M3, scale*sm_scale  (quant.py:433-480)
//    one warp per (head, padded row); rows >= T are zero bytes with the clamp scale
// ---------------------------------------------------------------------------
constexpr int kQRowsPerWarp = 4;                 // rows a warp has in flight
constexpr int kQPasses = 4;                      // passes per warp
constexpr int kQRowsPerCta = 8 * kQRowsPerWarp * kQPasses;
static_assert(kQRowsPerCta == kQTile, "one Q item is one 128-row tile of one head");

// `cta` = head * mtiles + q tile.  Each warp owns 16 consecutive rows of the tile and transforms
// them four at a time (four independent loads, butterflies and divisions in flight); the loads of
// the next four rows are issued before the current four are transformed.
__device__ __forceinline__ void quantize_q_rows(const Geom& g, long long cta) {
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = static_cast<int>(cta / g.mtiles), tile = static_cast<int>(cta % g.mtiles);
  if (head >= g.Hq) return;
  const int row_base = tile * kQTile + w * (kQRowsPerWarp * kQPasses);
  const bool qk_i8 = (g.flags & AKL_FLAG_QK_I8) != 0;
  const bool rotate = (g.flags & AKL_FLAG_ROTATE) != 0;
  const uint16_t* qsrc = reinterpret_cast<const uint16_t*>(g.q) + static_cast<size_t>(head) * kD + lane * 8;
  uint8_t* img = g.q8 + (static_cast<size_t>(head) * g.mtiles_cap + tile) * kImageBytes + (lane >> 4) * kPlaneBytes;
  float* qscale = g.qscale + static_cast<size_t>(head) * g.mtiles_cap * kQTile;
  uint4 raw[kQRowsPerWarp], nxt[kQRowsPerWarp];
  auto load4 = [&](int pass, uint4 (&dst)[kQRowsPerWarp]) {
#pragma unroll
    for (int k = 0; k < kQRowsPerWarp; ++k) {
      const int r = row_base + pass * kQRowsPerWarp + k;
      if (r < g.T) dst[k] = __ldg(reinterpret_cast<const uint4*>(qsrc + static_cast<size_t>(r) * g.Hq * kD));
    }
  };
  load4(0, raw);
#pragma unroll
  for (int pass = 0; pass < kQPasses; ++pass) {
    if (pass + 1 < kQPasses) load4(pass + 1, nxt);
#pragma unroll
    for (int k = 0; k < kQRowsPerWarp; ++k) {
      const int r = row_base + pass * kQRowsPerWarp + k;
      float x[8];
      float amax = 0.f;
      if (r < g.T) {
        unpack8<AKL_KV_BF16>(raw[k], x);
        if (rotate) fwht256(x, lane);
#pragma unroll
        for (int c = 0; c < 8; ++c) amax = fmaxf(amax, fabsf(x[c]));
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) x[c] = 0.f;
      }
      amax = fmaxf(warp_max(amax), 1e-8f);
      const float scale = __fdiv_rn(amax, qk_i8 ? kInt8Max : kFp8Max);
      float y[8];
      div8(make_exact_div(scale), x, y);
      const uint32_t lo = cvt_qk_x4(qk_i8, y[0], y[1], y[2], y[3]);
      const uint32_t hi = cvt_qk_x4(qk_i8, y[4], y[5], y[6], y[7]);
      *reinterpret_cast<uint2*>(img + swz128(r & 127, (lane & 15) * 8)) = make_uint2(lo, hi);
      if (lane == 0) qscale[r] = __fmul_rn(scale, g.sm_scale);
    }
#pragma unroll
    for (int k = 0; k < kQRowsPerWarp; ++k) raw[k] = nxt[k];
  }
}

__global__ void __launch_bounds__(kThreads) quantize_q_kernel(Geom g) { quantize_q_rows(g, blockIdx.x); }

// ---------------------------------------------------------------------------
// Batched forms: the same per-item bodies, driven by the request table.  Grids are sized
// from the capacities only; each CTA walks the flat item range with a grid stride, finds an
// item's request by binary search in the running totals, and keeps that request's geometry
// in shared memory until the request changes.
// ---------------------------------------------------------------------------
__device__ __forceinline__ int find_request(const int* totals, int n, int item) {
  // largest r in [0, n) with totals[r] <= item   (totals[0] = 0, totals[n] > item)
  int lo = 0, hi = n;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(totals + mid) <= item) lo = mid; else hi = mid;
  }
  return lo;
}

// All threads of the CTA; `cur` is the request whose geometry `sg` holds (-1: none).
__device__ __forceinline__ void stage_geom(const BatchRef& b, int r, int& cur, Geom* sg) {
  if (r == cur) return;                              // CTA-uniform
  __syncthreads();                                   // nobody still reads the old geometry
  const uint32_t* src = reinterpret_cast<const uint32_t*>(b.table + b.off_geoms + static_cast<size_t>(r) * sizeof(Geom));
  uint32_t* dst = reinterpret_cast<uint32_t*>(sg);
  for (int i = threadIdx.x; i < static_cast<int>(sizeof(Geom) / 4); i += blockDim.x) dst[i] = src[i];
  __syncthreads();
  cur = r;
}

// The per-item body is called, not inlined, in the batch kernel: the loop state then lives
// across a call boundary instead of competing with the body for registers.
template <int KV_DTYPE, int IDX_DTYPE>
__device__ __noinline__ void stats_item(const Geom& g, int in_req) {
  kv_tile_stats_item<KV_DTYPE, IDX_DTYPE>(g, in_req);
}

// Tile statistics of the whole batch (the Q quantisation runs in the transform launch).
template <int KV_DTYPE, int IDX_DTYPE>
__global__ void __launch_bounds__(kThreads, 4) kv_tile_stats_batch_kernel(BatchRef b) {
  __shared__ Geom sg;
  const BatchHeader* hdr = batch_header(b);
  const int n_req = hdr->n_requests, n_stat = hdr->n_stat_items;
  const int* stat_off = reinterpret_cast<const int*>(b.table + b.off_stat_off);
  int cur = -1;
  for (int item = blockIdx.x; item < n_stat; item += gridDim.x) {
    const int r = find_request(stat_off, n_req, item);
    stage_geom(b, r, cur, &sg);
    stats_item<KV_DTYPE, IDX_DTYPE>(sg, item - __ldg(stat_off + r));
    __syncthreads();                                 // the item's shared-memory partials are dead
  }
}

// One CTA per (request, kv head) up to the request capacity; CTA 0 also rewinds the attention
// work counter for the attention launch that follows in stream order.
__global__ void __launch_bounds__(kMeansThreads) kv_means_batch_kernel(BatchRef b, int kv_heads) {
  __shared__ Geom sg;
  BatchHeader* hdr = batch_header(b);
  if (blockIdx.x == 0 && threadIdx.x == 0) hdr->attn_counter = 0;
  const int r = blockIdx.x / kv_heads, kvh = blockIdx.x % kv_heads;
  if (r >= hdr->n_requests) return;
  int cur = -1;
  stage_geom(b, r, cur, &sg);
  kv_means_head<true>(sg, kvh);
}

// Q out of a row stage: 64 consecutive PACKED rows of one kv head's group of q heads (half of a
// packed 128-row tile; row R stands for token R / group and head kvh * group + R % group), a row
// spread over four lanes as in transform_k_tile_staged; per-row amax over the four lanes, per-row
// divisor.  Same bytes and scales per row as quantize_q_rows.  Rows of tokens >= T are zero bytes
// with the clamp scale.  The batched attention launch reads 128 such rows per work item.
__device__ __forceinline__ void quantize_q_half_staged(const Geom& g, int kvh, int pt, int half, const uint8_t* rows) {
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = lane & 3, lr = w * 8 + (lane >> 2);              // row inside the 64-row stage
  const int group = g.Hq / g.Hkv;
  const int R = pt * kQTile + half * 64 + lr;
  const bool live = R / group < g.T;
  const bool qk_i8 = (g.flags & AKL_FLAG_QK_I8) != 0;
  const bool rotate = (g.flags & AKL_FLAG_ROTATE) != 0;
  float x[8][8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (live) {
      const uint4 raw = *reinterpret_cast<const uint4*>(rows + lr * (kD * 2) + k * 64 + q * 16);
      unpack8<AKL_KV_BF16>(raw, x[k]);
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) x[k][c] = 0.f;
    }
  }
  if (rotate) fwht256_quarter(x, lane);
  float amax = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
#pragma unroll
    for (int c = 0; c < 8; ++c) amax = fmaxf(amax, fabsf(x[k][c]));
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, 1e-8f);
  const float scale = __fdiv_rn(amax, qk_i8 ? kInt8Max : kFp8Max);
  const ExactDiv dv = make_exact_div(scale);
  const size_t stripe = static_cast<size_t>(group) * g.mtiles_cap;  // packed tiles in a kv head's stripe
  uint8_t* img = g.q8p + (static_cast<size_t>(kvh) * stripe + pt) * kImageBytes;
  const uint32_t prow = half * 64 + lr;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float y[8];
    div8(dv, x[k], y);
    const uint32_t lo = cvt_qk_x4(qk_i8, y[0], y[1], y[2], y[3]);
    const uint32_t hi = cvt_qk_x4(qk_i8, y[4], y[5], y[6], y[7]);
    *reinterpret_cast<uint2*>(img + (k >> 2) * kPlaneBytes + swz128(prow, (k & 3) * 32 + q * 8)) = make_uint2(lo, hi);
  }
  if (q == 0) g.qscalep[static_cast<size_t>(kvh) * stripe * kQTile + R] = __fmul_rn(scale, g.sm_scale);
}

// The transform as a two-stage pipeline.  A CTA owns a contiguous run of items: (64-row tile x kv
// head x {K, V}) and, after them, (64 packed Q rows of a kv head) - the Q quantisation needs nothing from the
// statistics and is the same arithmetic as K.  The 64 rows of an item are fetched by 64 bulk
// copies of 512 bytes (lanes 0-7 of each warp fetch eight rows each) into one of two 33 KB stages,
// completing on the stage's mbarrier; the kv head's channel means and the V tile's scale ride
// along.  While item i is transformed out of one stage, item i+1 is landing in the other, and the
// copies of item i+2 are issued into i's stage as soon as i is done with it, so every CTA keeps
// 32-64 KB of reads in flight through all of its arithmetic (three CTAs per SM).  The V transpose
// staging lives in the stage its rows came from.
struct ItemCursor {
  int space;          // 0: (tile, kv head) items, running totals stat_off; 1: Q CTAs, totals qcta_off
  int r, lo, hi;      // request r owns the local items [lo, hi) of that space
};

struct ItemSpace {
  const int* stat_off;
  const int* qcta_off;
  int n_req, n_kv, n_all;     // items [0, n_kv): K/V; [n_kv, n_all): Q halves
};

constexpr int kRowsBytes = kTile * kD * 2;           // 64 rows x 512 bytes
constexpr int kStageMeanOff = kRowsBytes;            // the kv head's 256 channel means (K or V)
constexpr int kStageScaleOff = kStageMeanOff + kD * 4;   // V: the tile's scale (one float in a 16-byte slot)
constexpr int kStageBytes = (kStageScaleOff + 16 + 127) / 128 * 128;
constexpr int kStageArrivals = kTile + 2;            // one per row, one for the means, one for the scale
constexpr int kXfStages = 2;
constexpr long long kXfWaitCycles = 4000000000ll;    // ~2 s: a copy that late is a defect
static_assert(kVStagingBytes <= kRowsBytes, "the V staging is carved out of a row stage");
// relative cost of an item, for the split of the item range over the CTAs
constexpr int kCostKV = 5;                           // a K item and its V neighbour together
constexpr int kCostQ = 3;

// kind: 0 K, 1 V, 2 Q.  Returns the index inside the request (tile * Hkv + kv head, or Q CTA) and,
// for Q, which half of the 128-row tile.
__device__ __forceinline__ int locate_item(const ItemSpace& sp, int item, ItemCursor& c, int& kind, int& half) {
  int space, local;
  if (item < sp.n_kv) {
    kind = item & 1;                                 // K and V of a (tile, kv head) are neighbours
    half = 0;
    space = 0;
    local = item >> 1;
  } else {
    kind = 2;
    half = (item - sp.n_kv) & 1;
    space = 1;
    local = (item - sp.n_kv) >> 1;
  }
  if (c.space != space || local < c.lo || local >= c.hi) {
    const int* totals = space ? sp.qcta_off : sp.stat_off;
    c.space = space;
    c.r = find_request(totals, sp.n_req, local);
    c.lo = __ldg(totals + c.r);
    c.hi = __ldg(totals + c.r + 1);
  }
  return local - c.lo;
}

template <int IDX_DTYPE>
__device__ __forceinline__ void fetch_item_rows(const BatchRef& b, const ItemSpace& sp, int item, ItemCursor& c, uint32_t stage, uint32_t bar) {
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane >= 8 && !(w == 0 && lane < 10)) return;
  int kind, half;
  const int in_req = locate_item(sp, item, c, kind, half);
  const Geom* gp = reinterpret_cast<const Geom*>(b.table + b.off_geoms + static_cast<size_t>(c.r) * sizeof(Geom));
  if (kind == 2) {
    if (lane >= 8) { ptx::mbar_arrive(bar); return; }          // no means, no scale: the arrivals still count
    // 64 consecutive PACKED rows of a kv head: row R is token R / group, head kvh * group + R % group;
    // the group's heads of a token are neighbours in memory
    const int pts = gp->ptiles, group = gp->Hq / gp->Hkv;
    const int kvh = in_req / pts, pt = in_req - kvh * pts;
    const int R = pt * kQTile + half * 64 + w * 8 + lane;
    const int token = R / group;
    if (token < gp->T) {
      const int head = kvh * group + (R - token * group);
      ptx::mbar_expect_tx(bar, kD * 2);
      ptx::bulk_g2s(stage + static_cast<uint32_t>(w * 8 + lane) * (kD * 2),
                    reinterpret_cast<const uint16_t*>(gp->q) + (static_cast<size_t>(token) * gp->Hq + head) * kD, kD * 2, bar);
    } else {
      ptx::mbar_arrive(bar);
    }
    return;
  }
  const bool is_v = kind == 1;
  const int hkv = gp->Hkv;
  const int t = in_req / hkv, kvh = in_req - t * hkv;
  if (lane == 8) {            // warp 0: the kv head's channel means ride along with the rows
    ptx::mbar_expect_tx(bar, kD * 4);
    ptx::bulk_g2s(stage + kStageMeanOff, (is_v ? gp->vmean : gp->kmean) + kvh * kD, kD * 4, bar);
    return;
  }
  if (lane == 9) {            // warp 0: and the V tile's scale (the arrival is counted in the barrier's total)
    if (is_v) {
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(stage + kStageScaleOff), "l"(gp->vst + kvh * gp->ntiles_cap + t) : "memory");
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
    } else {
      ptx::mbar_arrive(bar);
    }
    return;
  }
  const int row = t * kTile + w * 8 + lane;
  if (row < gp->N) {
    const long long p = load_idx<IDX_DTYPE>(gp->idx, row);
    const uint16_t* pool = reinterpret_cast<const uint16_t*>(is_v ? gp->v_pool : gp->k_pool);
    ptx::mbar_expect_tx(bar, kD * 2);
    ptx::bulk_g2s(stage + static_cast<uint32_t>(w * 8 + lane) * (kD * 2), pool + (static_cast<size_t>(p) * hkv + kvh) * kD, kD * 2, bar);
  } else {
    ptx::mbar_arrive(bar);          // a row past the end: nothing to copy, the arrival still counts
  }
}

// Item index at cost position x (costs: kCostKV per K/V pair, kCostQ per Q half).
__device__ __forceinline__ int item_at_cost(long long x, int n_kv, int n_all) {
  const long long kv_cost = static_cast<long long>(n_kv / 2) * kCostKV;
  if (x < kv_cost) return static_cast<int>(x / kCostKV) * 2;
  const long long i = n_kv + (x - kv_cost) / kCostQ;
  return static_cast<int>(i < n_all ? i : n_all);
}

template <int KV_DTYPE, int IDX_DTYPE>
__global__ void __launch_bounds__(kThreads, 3) kv_transform_batch_kernel(BatchRef b) {
  extern __shared__ __align__(128) uint8_t xf_stages[];      // kXfStages x kStageBytes
  __shared__ Geom sg;
  __shared__ __align__(8) unsigned long long sm_full[kXfStages];
  const BatchHeader* hdr = batch_header(b);
  ItemSpace sp;
  sp.stat_off = reinterpret_cast<const int*>(b.table + b.off_stat_off);
  sp.qcta_off = reinterpret_cast<const int*>(b.table + b.off_qcta_off);
  sp.n_req = hdr->n_requests;
  sp.n_kv = 2 * hdr->n_stat_items;
  sp.n_all = sp.n_kv + 2 * hdr->n_q_ctas;
  const long long total_cost = static_cast<long long>(hdr->n_stat_items) * kCostKV + static_cast<long long>(2 * hdr->n_q_ctas) * kCostQ;
  const long long g_ = gridDim.x, c_ = blockIdx.x;
  const int item_lo = item_at_cost(total_cost * c_ / g_, sp.n_kv, sp.n_all);
  const int item_hi = (c_ + 1 == g_) ? sp.n_all : item_at_cost(total_cost * (c_ + 1) / g_, sp.n_kv, sp.n_all);
  if (item_lo >= item_hi) return;                            // CTA-uniform
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t stage0 = ptx::smem_u32(xf_stages), bar0 = ptx::smem_u32(sm_full);
  if (threadIdx.x == 0) {
    for (int i = 0; i < kXfStages; ++i) ptx::mbar_init(bar0 + i * 8, kStageArrivals);
    ptx::mbar_init_fence();
  }
  __syncthreads();
  ItemCursor fc{-1, -1, 0, 0};
  for (int i = 0; i < kXfStages; ++i)
    if (item_lo + i < item_hi) fetch_item_rows<IDX_DTYPE>(b, sp, item_lo + i, fc, stage0 + i * kStageBytes, bar0 + i * 8);

  ItemCursor cc{-1, -1, 0, 0};
  int cur = -1;
  for (int item = item_lo; item < item_hi; ++item) {
    const int k = item - item_lo, st = k % kXfStages;
    const uint32_t parity = static_cast<uint32_t>(k / kXfStages) & 1u;
    int kind, half;
    const int in_req = locate_item(sp, item, cc, kind, half);
    stage_geom(b, cc.r, cur, &sg);

    // the rows have landed (bounded: a copy that never completes ends the CTA with a status code)
    bool ok = true;
    if (!ptx::mbar_try_wait(bar0 + st * 8, parity)) {
      const long long t0 = clock64();
      while (!ptx::mbar_try_wait(bar0 + st * 8, parity)) {
        if (clock64() - t0 > kXfWaitCycles) { ok = false; break; }
      }
    }
    const uint8_t* stage = xf_stages + st * kStageBytes;
    if (kind != 1) {
      if (!__syncthreads_and(ok)) {
        if (threadIdx.x == 0) atomicCAS(sg.status, 0, AKL_ERR_TIMEOUT);
        return;
      }
      if (kind == 0) {
        transform_k_tile_staged<KV_DTYPE>(sg, in_req / sg.Hkv, in_req % sg.Hkv, stage, reinterpret_cast<const float*>(stage + kStageMeanOff));
      } else {
        quantize_q_half_staged(sg, in_req / sg.ptiles, in_req % sg.ptiles, half, stage);
      }
    } else {
      uint4 raw[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) raw[i] = *reinterpret_cast<const uint4*>(stage + (w * 8 + i) * (kD * 2) + lane * 16);
      // every thread holds its rows: the stage may now serve as the V staging
      if (!__syncthreads_and(ok)) {
        if (threadIdx.x == 0) atomicCAS(sg.status, 0, AKL_ERR_TIMEOUT);
        return;
      }
      const float* st_mean = reinterpret_cast<const float*>(stage + kStageMeanOff) + lane * 8;
      const float v_scale = *reinterpret_cast<const float*>(stage + kStageScaleOff);
      transform_tile_rows<KV_DTYPE>(sg, in_req / sg.Hkv, in_req % sg.Hkv, true, raw, xf_stages + st * kStageBytes, st_mean, v_scale);
    }
    ptx::fence_async_smem();                             // generic accesses to the stage before the copies that overwrite it
    __syncthreads();                                     // the item is done with its stage
    if (item + kXfStages < item_hi)
      fetch_item_rows<IDX_DTYPE>(b, sp, item + kXfStages, fc, stage0 + st * kStageBytes, bar0 + st * 8);
  }
}

// ---------------------------------------------------------------------------
// Self-test of the shared-divisor division: every dividend significand (2^23 of them) in four
// quotient binades, both signs, against the IEEE division, for each divisor given.  Counts the
// quotients whose bits differ (expected: none).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) exact_division_selftest_kernel(const float* scales, unsigned long long* mismatches) {
  const float s = scales[blockIdx.y];
  const ExactDiv d = make_exact_div(s);
  const unsigned sexp = (__float_as_uint(s) >> 23) & 0xFFu;
  unsigned long long bad = 0;
  const int eoff[4] = {-3, 0, 5, 8};
  for (unsigned base = (blockIdx.x * 256u + threadIdx.x) * 8u; base < (1u << 23); base += gridDim.x * 256u * 8u) {
#pragma unroll 1
    for (int k = 0; k < 4; ++k) {
      const int e = static_cast<int>(sexp) + eoff[k];
      if (e < 1 || e > 254) continue;
#pragma unroll 1
      for (unsigned sign = 0; sign < 2; ++sign) {
        float x[8], y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = __uint_as_float((sign << 31) | (static_cast<unsigned>(e) << 23) | (base + i));
        div8(d, x, y);
#pragma unroll
        for (int i = 0; i < 8; ++i) bad += (__float_as_uint(y[i]) != __float_as_uint(__fdiv_rn(x[i], s))) ? 1ull : 0ull;
      }
    }
  }
  if (bad) atomicAdd(mismatches, bad);
}

}  // namespace

int launch_exact_division_selftest(const float* scales, int n, unsigned long long* mismatches, cudaStream_t s) {
  exact_division_selftest_kernel<<<dim3(64, static_cast<unsigned>(n)), 256, 0, s>>>(scales, mismatches);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { note_cuda_error(e, "exact_division_selftest"); return AKL_ERR_CUDA; }
  return AKL_OK;
}

#define AKL_LAUNCH_CHECK(where)                    \
  do {                                             \
    cudaError_t e_ = cudaGetLastError();           \
    if (e_ != cudaSuccess) {                       \
      note_cuda_error(e_, where);                  \
      return AKL_ERR_CUDA;                         \
    }                                              \
  } while (0)

static unsigned q_ctas(const Geom& g) { return static_cast<unsigned>(g.Hq) * static_cast<unsigned>(g.mtiles); }

template <bool kWithQ>
static void launch_stats_impl(const Geom& g, int kv_dtype, int idx_dtype, cudaStream_t s) {
  const unsigned grid = static_cast<unsigned>(g.nt) * g.Hkv + (kWithQ ? q_ctas(g) : 0u);
  if (kv_dtype == AKL_KV_BF16 && idx_dtype == AKL_IDX_I64)
    kv_tile_stats_kernel<AKL_KV_BF16, AKL_IDX_I64, kWithQ><<<grid, kThreads, 0, s>>>(g);
  else if (kv_dtype == AKL_KV_BF16)
    kv_tile_stats_kernel<AKL_KV_BF16, AKL_IDX_I32, kWithQ><<<grid, kThreads, 0, s>>>(g);
  else if (idx_dtype == AKL_IDX_I64)
    kv_tile_stats_kernel<AKL_KV_FP16, AKL_IDX_I64, kWithQ><<<grid, kThreads, 0, s>>>(g);
  else
    kv_tile_stats_kernel<AKL_KV_FP16, AKL_IDX_I32, kWithQ><<<grid, kThreads, 0, s>>>(g);
}

int launch_kv_tile_stats(const Geom& g, int kv_dtype, int idx_dtype, cudaStream_t s, bool with_q) {
  if (with_q)
    launch_stats_impl<true>(g, kv_dtype, idx_dtype, s);
  else
    launch_stats_impl<false>(g, kv_dtype, idx_dtype, s);
  AKL_LAUNCH_CHECK("kv_tile_stats");
  return AKL_OK;
}

int launch_kv_means(const Geom& g, cudaStream_t s, bool fuse_scales) {
  if (fuse_scales)
    kv_means_kernel<true><<<g.Hkv, kMeansThreads, 0, s>>>(g);
  else
    kv_means_kernel<false><<<g.Hkv, kMeansThreads, 0, s>>>(g);
  AKL_LAUNCH_CHECK("kv_means");
  return AKL_OK;
}

int launch_kv_scales(const Geom& g, cudaStream_t s) {
  kv_scales_kernel<<<g.Hkv, kThreads, 0, s>>>(g);
  AKL_LAUNCH_CHECK("kv_scales");
  return AKL_OK;
}

int launch_kv_transform(const Geom& g, int kv_dtype, int idx_dtype, cudaStream_t s) {
  dim3 grid(g.nt, g.Hkv, 2);
  if (kv_dtype == AKL_KV_BF16 && idx_dtype == AKL_IDX_I64)
    kv_transform_kernel<AKL_KV_BF16, AKL_IDX_I64><<<grid, kThreads, 0, s>>>(g);
  else if (kv_dtype == AKL_KV_BF16)
    kv_transform_kernel<AKL_KV_BF16, AKL_IDX_I32><<<grid, kThreads, 0, s>>>(g);
  else if (idx_dtype == AKL_IDX_I64)
    kv_transform_kernel<AKL_KV_FP16, AKL_IDX_I64><<<grid, kThreads, 0, s>>>(g);
  else
    kv_transform_kernel<AKL_KV_FP16, AKL_IDX_I32><<<grid, kThreads, 0, s>>>(g);
  AKL_LAUNCH_CHECK("kv_transform");
  return AKL_OK;
}

int launch_batch_stats(const BatchRef& b, int kv_dtype, int idx_dtype, int sm_count, cudaStream_t s) {
  const unsigned grid = static_cast<unsigned>(sm_count) * 4u;        // four resident CTAs per SM
  if (kv_dtype == AKL_KV_BF16 && idx_dtype == AKL_IDX_I64)
    kv_tile_stats_batch_kernel<AKL_KV_BF16, AKL_IDX_I64><<<grid, kThreads, 0, s>>>(b);
  else if (kv_dtype == AKL_KV_BF16)
    kv_tile_stats_batch_kernel<AKL_KV_BF16, AKL_IDX_I32><<<grid, kThreads, 0, s>>>(b);
  else if (idx_dtype == AKL_IDX_I64)
    kv_tile_stats_batch_kernel<AKL_KV_FP16, AKL_IDX_I64><<<grid, kThreads, 0, s>>>(b);
  else
    kv_tile_stats_batch_kernel<AKL_KV_FP16, AKL_IDX_I32><<<grid, kThreads, 0, s>>>(b);
  AKL_LAUNCH_CHECK("kv_tile_stats_batch");
  return AKL_OK;
}

int launch_batch_means(const BatchRef& b, int kv_heads, cudaStream_t s) {
  kv_means_batch_kernel<<<static_cast<unsigned>(b.max_requests) * kv_heads, kMeansThreads, 0, s>>>(b, kv_heads);
  AKL_LAUNCH_CHECK("kv_means_batch");
  return AKL_OK;
}

// Opts the four instantiations into their dynamic shared memory, once per device.
static int configure_transform_once() {
  static std::atomic<bool> configured[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { note_cuda_error(e, "cudaGetDevice"); return AKL_ERR_CUDA; }
  if (dev >= 0 && dev < 64 && configured[dev].load(std::memory_order_acquire)) return AKL_OK;
  const void* kernels[4] = {
      reinterpret_cast<const void*>(kv_transform_batch_kernel<AKL_KV_BF16, AKL_IDX_I64>), reinterpret_cast<const void*>(kv_transform_batch_kernel<AKL_KV_BF16, AKL_IDX_I32>),
      reinterpret_cast<const void*>(kv_transform_batch_kernel<AKL_KV_FP16, AKL_IDX_I64>), reinterpret_cast<const void*>(kv_transform_batch_kernel<AKL_KV_FP16, AKL_IDX_I32>)};
  for (const void* k : kernels) {
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kXfStages * kStageBytes);
    if (e != cudaSuccess) { note_cuda_error(e, "cudaFuncSetAttribute(transform)"); return AKL_ERR_CUDA; }
  }
  if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
  return AKL_OK;
}

int launch_batch_transform(const BatchRef& b, int kv_dtype, int idx_dtype, int sm_count, cudaStream_t s) {
  const int rc = configure_transform_once();
  if (rc != AKL_OK) return rc;
  const unsigned grid = static_cast<unsigned>(sm_count) * 3u;        // three resident CTAs per SM
  const size_t smem = kXfStages * kStageBytes;
  if (kv_dtype == AKL_KV_BF16 && idx_dtype == AKL_IDX_I64)
    kv_transform_batch_kernel<AKL_KV_BF16, AKL_IDX_I64><<<grid, kThreads, smem, s>>>(b);
  else if (kv_dtype == AKL_KV_BF16)
    kv_transform_batch_kernel<AKL_KV_BF16, AKL_IDX_I32><<<grid, kThreads, smem, s>>>(b);
  else if (idx_dtype == AKL_IDX_I64)
    kv_transform_batch_kernel<AKL_KV_FP16, AKL_IDX_I64><<<grid, kThreads, smem, s>>>(b);
  else
    kv_transform_batch_kernel<AKL_KV_FP16, AKL_IDX_I32><<<grid, kThreads, smem, s>>>(b);
  AKL_LAUNCH_CHECK("kv_transform_batch");
  return AKL_OK;
}

int launch_quantize_q(const Geom& g, cudaStream_t s) {
  quantize_q_kernel<<<q_ctas(g), kThreads, 0, s>>>(g);
  AKL_LAUNCH_CHECK("quantize_q");
  return AKL_OK;
}

}  // namespace akl
