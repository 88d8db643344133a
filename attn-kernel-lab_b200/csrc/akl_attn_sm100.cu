// Fused FP8 paged-prefill attention for sm_100a: tcgen05 kind::f8f6f4 MMAs with the S and O
// accumulators in tensor memory, operand tiles brought in by bulk asynchronous copies,
// exact online softmax (P x 448 fold, exact rescale skip) on two softmax warpgroups.
//
// It computes what the reference's mma.sync kernel computes
// (src/attn_kernel_lab/csrc/fp8_prefill_attn.cu:220-681): per (128-row Q tile, q head)
//   S  = Q8 K8^T                     e4m3 x e4m3 -> fp32            (:429-470)
//   s  = S * qscale[row] * kscale[t], bottom-right causal bound      (:471-521)
//   m' = max(m, rowmax);  alpha = ex2((m - m') log2e)                 (:528-541)
//   p' = ex2(fma(s, log2e, log2 448 + log2 r_t - m' log2e))           (:542-553)
//   l  = l alpha + sum(p') / r_t      (unrounded p')                  (:556-563)
//   O  = O alpha  (skipped, exactly, when no row of the warp moved)   (:564-584)
//   O += e4m3(p') V8                                                  (:591-611)
//   out = bf16(fma(O, vscale / l, vmean)),  lse2 = m log2e + log2 l - log2 448   (:636-680)
// per 64-key tile, in tile order -- the tile sequence is part of the operator because P is
// rounded against the running maximum.
//
// CTA = 20 warps, every role with its own loop over the CTA's work items:
//   warps 0-3   softmax warpgroup 0: even 64-key tiles  } thread i of a group owns query row i,
//   warps 4-7   softmax warpgroup 1: odd  64-key tiles  } which is TMEM lane i
//   warps 8-11  correction warpgroup A: O columns 0-127   } multiply O by alpha between two PV MMAs
//   warps 16-19 correction warpgroup B: O columns 128-255 } when a row's running maximum moved, so
//               that the softmax groups never wait for the tensor pipe,
//   warp  12    lane 0 issues the Q and K bulk copies; the warp owns TMEM allocation,
//   warp  14    lane 0 issues the V^T bulk copies (its own thread, so that a K tile whose stage
//               is free is never queued behind a wait for a V stage),
//   warp  13    lane 0 issues the PV MMAs (after P(j) is written and O carries alpha_j),
//   warp  15    lane 0 issues the QK^T MMAs (as soon as an S buffer has been read out).
// The two issuing threads sit on different warp schedulers and never wait for each other's
// inputs, so the tensor pipe always has the QK^T of a later pair to run while the correction of
// the next tile is in flight.  (One thread issuing both kinds was measured: an MMA costs its
// issuing thread about a hundred cycles, and eight QK^T issues in front of a PV lengthen the
// PV -> rescale -> PV chain that sets the tile period.)
// Registers are re-budgeted per role (setmaxnreg): the kernel starts at 96 per thread, the issuing
// warps drop to 40 and the softmax warpgroups take 120.
// The two softmax groups alternate tiles so that two warps share each scheduler and hide each
// other's latencies; the running row maximum is the only state that must travel from one tile
// to the next, and it is handed from group to group through a 64-bit (sequence, value) word per
// row in shared memory.  Each group keeps its own partial l against its own last maximum; the two
// are combined once, in the epilogue.
//
// Work items: one (q tile, q head) per CTA from the block index, or -- the batched entry -- a
// persistent CTA per SM that draws (request, q head, q tile) items from the request table
// through an atomic counter (the next item is drawn while the current one runs).
//
// Shared memory: Q tile 32 KiB; K and V^T 128-key pair tiles, two stages each (2 x 64 KiB);
// P 2 x 16 KiB.  Tensor memory (512 columns): O = columns 0-255, S ping-pong = 256-383 /
// 384-511.  QK^T runs at N = 128 keys per MMA group, softmax and PV at the operator's 64-key
// tile granularity (two K=32 MMAs of N = 256 per tile).
#include <atomic>
#include <cstring>

#include "akl_common.cuh"
#include "akl_sm100_ptx.cuh"

namespace akl {

namespace {

using namespace ptx;

// Timeline probe for kernel development: compiled in only with -DAKL_TRACE, never in the
// shipped library.  Thread 0 of each softmax group stamps clock64() at fixed points of a tile.
#ifdef AKL_TRACE
#define AKL_TRACE_POINT(k)                                                                       \
  do {                                                                                           \
    if (g.dbg_s != nullptr && row == 0 && blockIdx.x == 0 && blockIdx.y == 0 && j < 512)         \
      reinterpret_cast<long long*>(g.dbg_s)[(j * 8 + (k))] = clock64();                          \
  } while (0)
#define AKL_TRACE_AUX(cond, j_, k)                                                                \
  do {                                                                                           \
    if (g.dbg_s != nullptr && (cond) && blockIdx.x == 0 && blockIdx.y == 0 && (j_) < 512)        \
      reinterpret_cast<long long*>(g.dbg_s)[4096 + ((j_) * 8 + (k))] = clock64();                \
  } while (0)
#else
#define AKL_TRACE_POINT(k) do { } while (0)
#define AKL_TRACE_AUX(cond, j_, k) do { } while (0)
#endif

constexpr int kThreads = 640;
constexpr int kProducerWarp = 12, kVProducerWarp = 14, kQkWarp = 15;   // warp 13 issues the PV MMAs
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffK = 32768;
constexpr uint32_t kOffV = kOffK + 2 * 32768;
constexpr uint32_t kOffP = kOffV + 2 * 32768;
constexpr uint32_t kOffBar = kOffP + 2 * 16384;      // 196608
constexpr uint32_t kOffVmean = kOffBar + 512;        // 256 floats
constexpr uint32_t kOffChain = kOffVmean + 1024;     // 128 x u64 running-max hand-off words
constexpr uint32_t kOffFin = kOffChain + 1024;       // [2][128] (m, l) pairs for the epilogue
constexpr uint32_t kOffAlpha = kOffFin + 2048;       // [8][128] floats: alpha of tile j in slot j & 7
constexpr uint32_t kSmemBytes = kOffAlpha + 4096 + 1024;   // + alignment slack
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 0, kColS = 256;
constexpr uint32_t kIdescQK = idesc_e4m3(128, 128);
constexpr uint32_t kIdescQKi8 = idesc_s8(128, 128);
constexpr uint32_t kIdescPV = idesc_e4m3(128, 256);
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLog2_448 = 8.807354922057604f;
constexpr long long kWaitCycles = 4000000000ll;      // ~2 s: a wait that long is a defect

// barrier slots (8 bytes each)
enum {
  B_QFULL = 0,
  B_KFULL = 1,    // [2]
  B_KEMPTY = 3,   // [2]
  B_VFULL = 5,    // [2]
  B_VEMPTY = 7,   // [2]
  B_SFULL = 9,    // [2]
  B_SEMPTY = 11,  // [2]
  B_PFULL = 13,   // [2][2]
  B_PVDONE = 17,  // one phase per tile; only the correction group waits on it, every tile
  B_ALLDONE = 18,
  B_AREADY = 28,  // [8] alpha of tile j published (slot j & 7)
  B_OREADY = 23,  // O carries alpha_j: PV(j) may be issued
  B_PEMPTY = 24,  // [2][2] PV(j) has read P slot (j>>1)&1, j&1 (and the correction of tile j is over)
  B_COUNT = 36
};

struct Ctx {
  uint32_t bars;
  int* status;
  volatile int* abort_flag;   // shared memory
};

__device__ __forceinline__ bool give_up(const Ctx& c, long long& t0) {
  if (t0 == 0) {
    t0 = clock64();
    return false;
  }
  if (*c.abort_flag || clock64() - t0 > kWaitCycles) {
    *c.abort_flag = 1;
    atomicCAS(c.status, 0, AKL_ERR_TIMEOUT);
    return true;
  }
  return false;
}

// Bounded mbarrier wait.  Returns false after ~2 s (or as soon as another thread of the CTA
// gave up), having recorded AKL_ERR_TIMEOUT in the status word.
//
// A parity wait is only meaningful while the waiter is at most one phase behind the barrier,
// so every waiter in this kernel observes every phase of the barriers it waits on, in order.
__device__ __forceinline__ bool wait(const Ctx& c, int slot, uint32_t parity) {
  const uint32_t bar = c.bars + slot * 8;
  long long t0 = 0;
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 0xFFFu) == 0 && give_up(c, t0)) return false;
  }
}

// One arrival for the whole warp: every lane's earlier writes (and fences) are ordered before
// lane 0's releasing arrive by the warp barrier.  Barrier counts are in warps.
__device__ __forceinline__ void warp_arrive(uint32_t bar, int lane) {
  mbar_arrive(bar);
}

__device__ __forceinline__ void scale32(uint32_t (&v)[32], float alpha) {
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float x0 = __uint_as_float(v[i]), x1 = __uint_as_float(v[i + 1]);
    mul2(x0, x1, alpha);
    v[i] = __float_as_uint(x0);
    v[i + 1] = __float_as_uint(x1);
  }
}

// Running-maximum hand-off: word = (tiles finished << 32) | float bits of the maximum after
// them.  The consumer of tile j waits until `tiles finished` reaches j.
__device__ __forceinline__ void chain_post(uint32_t addr, uint32_t seq, float m) {
  asm volatile("st.volatile.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(__float_as_uint(m)), "r"(seq) : "memory");
}
__device__ __forceinline__ bool chain_wait(const Ctx& c, uint32_t addr, uint32_t seq, float& m) {
  long long t0 = 0;
  for (uint32_t spin = 1;; ++spin) {
    uint32_t lo, hi;
    asm volatile("ld.volatile.shared.v2.b32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(addr) : "memory");
    if (hi == seq) {
      m = __uint_as_float(lo);
      return true;
    }
    if ((spin & 0xFFFu) == 0 && give_up(c, t0)) return false;
  }
}

// Descriptor of a K-major SWIZZLE_128B operand: the high word is constant, the low word is the
// 16-byte-unit address (plus the unused leading-offset field); a byte offset adds offset/16.
constexpr uint32_t kDescHi = 64u | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint64_t desc_at(uint32_t lo, uint32_t byte_off) {
  return (static_cast<uint64_t>(kDescHi) << 32) | (lo + (byte_off >> 4));
}
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }

// QK^T of one 128-key pair: 8 MMAs of K = 32 (two 128-byte planes x four 32-byte steps);
// E4M3 operands with an fp32 accumulator, or INT8 operands with an exact s32 accumulator.
template <bool kI8>
__device__ __forceinline__ void issue_qk(uint32_t q_lo, uint32_t k_lo, uint32_t tmem_s) {
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t off = (k >> 2) * kPlaneBytes + (k & 3) * 32;
    if (kI8) mma_i8_ss(tmem_s, desc_at(q_lo, off), desc_at(k_lo, off), kIdescQKi8, k > 0 ? 1u : 0u);
    else mma_f8_ss(tmem_s, desc_at(q_lo, off), desc_at(k_lo, off), kIdescQK, k > 0 ? 1u : 0u);
  }
}

// PV of one 64-key tile: 2 MMAs of K = 32 inside one 128-byte row (offset half*64).
__device__ __forceinline__ void issue_pv(uint32_t p_lo, uint32_t v_lo, uint32_t tmem_o, uint32_t accumulate) {
  mma_f8_ss(tmem_o, desc_at(p_lo, 0), desc_at(v_lo, 0), kIdescPV, accumulate);
  mma_f8_ss(tmem_o, desc_at(p_lo, 32), desc_at(v_lo, 32), kIdescPV, 1u);
}

// One QK^T accumulator word as a float: the fp32 sum itself, or the s32 sum converted (exact:
// |sum| <= 256 * 127 * 127 < 2^24).
template <bool kI8>
__device__ __forceinline__ float acc_value(uint32_t word) {
  return kI8 ? __int2float_rn(static_cast<int>(word)) : __uint_as_float(word);
}

// Registers per thread after the per-role re-budgeting (setmaxnreg): the kernel starts with
// 96 per thread (640 threads x 96 = 61440); the four issuing warps give theirs up, the
// softmax warpgroups take them.  8*32*120 + 8*32*96 + 4*32*40 = 60416 <= 61440.
constexpr int kRegsStart = 96, kRegsSoftmax = 120, kRegsMisc = 40;    // the correction warps keep 96
static_assert(8 * 32 * kRegsSoftmax + 8 * 32 * kRegsStart + 4 * 32 * kRegsMisc <= kThreads * kRegsStart,
              "register budget: an increase waits for registers other warps never release");

// What one (q tile, q head) work item needs, derived by every thread for itself.
// kBatch = false: the 128 rows of an item are the tokens m0 .. m0+127 of q head h.  kBatch = true:
// they are 128 consecutive PACKED rows of kv head kvh, row R = qt * 128 + r standing for token
// R / group and q head kvh * group + R % group (group = Hq / Hkv), so that short requests do not
// pay a 128-row tile per q head.
struct Item {
  int qt, h, kvh, m0, ntile, npair, group;
};

// Token and q head of row `row` of the item.
template <bool kBatch>
__device__ __forceinline__ void item_row(const Item& it, int row, int& token, int& head) {
  if (kBatch) {
    const int R = it.qt * kQTile + row;
    token = R / it.group;
    head = it.kvh * it.group + (R - token * it.group);
  } else {
    token = it.m0 + row;
    head = it.h;
  }
}

struct Shared {
  uint32_t tmem_slot;
  int abort_flag;
  int item;       // batch mode: index of the current work item (or >= n_items: stop)
  int2 word;      // batch mode: {request, head << 16 | q tile} of the current item
  Geom geom;      // batch mode: geometry of the current request
};

// Top of every role's item loop; all 640 threads call it the same number of times.  Returns false
// when there is no further item.  kBatch = false: the single item comes from the block index.
// kBatch = true: thread 0 has drawn the item ahead of time (`drawn`), publishes it, and draws the
// next one so that the atomic's round trip is off the path; the request's geometry is copied to
// shared memory when the request changes; the mbarriers are invalidated and rebuilt (every async
// arrival of the previous item has landed: its last MMA was observed before the epilogue).
template <bool kBatch>
__device__ __forceinline__ bool begin_item(const Geom& g, const BatchRef& bref, Shared& sh, uint32_t smem, uint8_t* smem_gen,
                                           int iter, int& cur_request, int& drawn, Item& it) {
  const int tid = threadIdx.x;
  if (kBatch) {
    BatchHeader* hdr = batch_header(bref);
    if (tid == 0) {
      sh.item = drawn;
      if (drawn < hdr->n_attn_items) sh.word = __ldg(reinterpret_cast<const int2*>(bref.table + bref.off_items) + drawn);
    }
    __syncthreads();                    // every role is done with the previous item; the new one is published
    const int item = sh.item;
    if (item >= hdr->n_attn_items || sh.abort_flag != 0) return false;     // CTA-uniform
    const int2 w = sh.word;
    it.h = 0;
    it.kvh = w.y >> 16;
    it.qt = w.y & 0xFFFF;
    if (w.x != cur_request) {
      const uint32_t* src = reinterpret_cast<const uint32_t*>(bref.table + bref.off_geoms + static_cast<size_t>(w.x) * sizeof(Geom));
      uint32_t* dst = reinterpret_cast<uint32_t*>(&sh.geom);
      if (tid < static_cast<int>(sizeof(Geom) / 4)) dst[tid] = src[tid];
      cur_request = w.x;
    }
  } else {
    if (iter > 0) return false;
    it.qt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);   // deepest tiles first
    it.h = blockIdx.y;
  }
  if (tid == 0) {
    const uint32_t b = smem + kOffBar;
    if (iter > 0) {
      for (int i = 0; i < B_COUNT; ++i) mbar_inval(b + i * 8);
    }
    mbar_init(b + B_QFULL * 8, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(b + (B_KFULL + i) * 8, 1);
      mbar_init(b + (B_KEMPTY + i) * 8, 1);
      mbar_init(b + (B_VFULL + i) * 8, 1);
      mbar_init(b + (B_VEMPTY + i) * 8, 1);
      mbar_init(b + (B_SFULL + i) * 8, 1);
      mbar_init(b + (B_SEMPTY + i) * 8, 256);
    }
    for (int i = 0; i < 4; ++i) mbar_init(b + (B_PFULL + i) * 8, 128);
    for (int i = 0; i < 8; ++i) mbar_init(b + (B_AREADY + i) * 8, 128);
    for (int i = 0; i < 4; ++i) mbar_init(b + (B_PEMPTY + i) * 8, 1);
    mbar_init(b + B_PVDONE * 8, 1);
    mbar_init(b + B_OREADY * 8, 256);
    mbar_init(b + B_ALLDONE * 8, 1);
    mbar_init_fence();
    fence_async_smem();
  }
  if (kBatch) {
    __syncthreads();                    // the staged geometry is visible
    if (tid == 0) drawn = atomicAdd(&batch_header(bref)->attn_counter, 1);
  }
  it.group = g.Hq / g.Hkv;
  if (!kBatch) it.kvh = it.h / it.group;
  it.m0 = it.qt * kQTile;
  // keys this item visits, in local (this call's) positions: up to the last token of the item
  const int tok_end = kBatch ? (it.qt * kQTile + kQTile - 1) / it.group + 1 : it.m0 + kQTile;
  long long hi_ll = static_cast<long long>(g.prefix) + tok_end - g.kv_pos0;
  const int hi = static_cast<int>(hi_ll < 0 ? 0 : (hi_ll > g.N ? g.N : hi_ll));
  it.ntile = (hi + kTile - 1) / kTile;
  it.npair = (it.ntile + 1) / 2;
  if (tid < 128) {
    float* sm_vmean = reinterpret_cast<float*>(smem_gen + kOffVmean);
    sm_vmean[tid] = g.vmean[it.kvh * kD + tid];
    sm_vmean[tid + 128] = g.vmean[it.kvh * kD + tid + 128];
    chain_post(smem + kOffChain + tid * 8, 0u, -INFINITY);      // "zero tiles finished, max = -inf"
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  return true;
}

// kBatch = false: one work item per CTA, (q tile, head) from the block index, geometry in the
// kernel parameter.  kBatch = true: a persistent CTA draws (request, head, q tile) items from the
// request table's list through an atomic counter and keeps the current request's geometry in
// shared memory; tensor memory is allocated once, the mbarriers are rebuilt per item.
// Every role runs its own loop over the items, so that each loop is compiled for its own
// register budget.
template <bool kDump, bool kI8, bool kBatch>
__global__ void __launch_bounds__(kThreads, 1) attn_sm100_kernel(const __grid_constant__ Geom g_param, const __grid_constant__ BatchRef bref) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ Shared sh;
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem - smem_u32(smem_raw));
  float* sm_vmean = reinterpret_cast<float*>(smem_gen + kOffVmean);
  float2* sm_fin = reinterpret_cast<float2*>(smem_gen + kOffFin);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const Geom& g = kBatch ? sh.geom : g_param;

  if (tid == 0) sh.abort_flag = 0;
  if (warp == kProducerWarp) tmem_alloc(smem_u32(&sh.tmem_slot), kTmemCols);
  int drawn = 0;
  if (kBatch && tid == 0) drawn = atomicAdd(&batch_header(bref)->attn_counter, 1);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh.tmem_slot;
  int cur_request = -1;
  Ctx ctx{smem + kOffBar, nullptr, &sh.abort_flag};
  Item it;

  if (warp >= 12 && warp < 16) {
    // ================================================================ issuing warps
    reg_dealloc<kRegsMisc>();
    for (int iter = 0; begin_item<kBatch>(g, bref, sh, smem, smem_gen, iter, cur_request, drawn, it); ++iter) {
      ctx.status = g.status;
      const int ntile = it.ntile, npair = it.npair;
      if (lane != 0 || ntile == 0) continue;
      if (warp == kProducerWarp) {
        // ---------------------------------------------------------- Q and K copies
        const uint8_t* qsrc = kBatch
            ? g.q8p + (static_cast<size_t>(it.kvh) * it.group * g.mtiles_cap + it.qt) * kImageBytes
            : g.q8 + (static_cast<size_t>(it.h) * g.mtiles_cap + it.qt) * kImageBytes;
        const uint8_t* ksrc = g.k8 + static_cast<size_t>(it.kvh) * g.npairs_cap * kImageBytes;
        mbar_expect_tx(ctx.bars + B_QFULL * 8, kImageBytes);
        bulk_g2s(smem + kOffQ, qsrc, kImageBytes, ctx.bars + B_QFULL * 8);
        for (int u = 0; u < npair; ++u) {
          const int s = u & 1, n = u >> 1;
          if (n >= 1 && !wait(ctx, B_KEMPTY + s, (n - 1) & 1)) break;
          mbar_expect_tx(ctx.bars + (B_KFULL + s) * 8, kImageBytes);
          bulk_g2s(smem + kOffK + s * 32768, ksrc + static_cast<size_t>(u) * kImageBytes, kImageBytes,
                   ctx.bars + (B_KFULL + s) * 8);
        }
      } else if (warp == kVProducerWarp) {
        // ---------------------------------------------------------- V^T copies
        const uint8_t* vsrc = g.v8t + static_cast<size_t>(it.kvh) * g.npairs_cap * kImageBytes;
        for (int u = 0; u < npair; ++u) {
          const int s = u & 1, n = u >> 1;
          if (n >= 1 && !wait(ctx, B_VEMPTY + s, (n - 1) & 1)) break;
          mbar_expect_tx(ctx.bars + (B_VFULL + s) * 8, kImageBytes);
          bulk_g2s(smem + kOffV + s * 32768, vsrc + static_cast<size_t>(u) * kImageBytes, kImageBytes,
                   ctx.bars + (B_VFULL + s) * 8);
        }
      } else if (warp == kQkWarp) {
        // ---------------------------------------------------------- QK^T issuer
        const uint32_t q_lo = desc_lo(smem + kOffQ);
        bool ok = wait(ctx, B_QFULL, 0);
        for (int u = 0; ok && u < npair; ++u) {
          const int b = u & 1, n = u >> 1;
          ok = wait(ctx, B_KFULL + b, n & 1);
          if (ok && n >= 1) ok = wait(ctx, B_SEMPTY + b, (n - 1) & 1);   // both groups have read S(u-2)
          if (!ok) break;
          tc_fence_after();
          issue_qk<kI8>(q_lo, desc_lo(smem + kOffK + b * 32768), tmem + kColS + b * 128);
          tc_commit(ctx.bars + (B_SFULL + b) * 8);
          tc_commit(ctx.bars + (B_KEMPTY + b) * 8);
        }
      } else {
        // ---------------------------------------------------------- PV issuer
        bool ok = true;
        const uint32_t p_base = desc_lo(smem + kOffP), v_base = desc_lo(smem + kOffV);
        for (int j = 0; ok && j < ntile; ++j) {
          const int u = j >> 1, c = j & 1, b = u & 1, par = (u >> 1) & 1;
          const uint32_t p_lo = p_base + ((b * 16384 + c * 64) >> 4), v_lo = v_base + ((b * 32768 + c * 64) >> 4);
          const uint32_t acc = j > 0 ? 1u : 0u;
          if (c == 0) ok = wait(ctx, B_VFULL + b, par);
          ok = ok && wait(ctx, B_PFULL + b * 2 + c, par) && wait(ctx, B_OREADY, j & 1);
          if (!ok) break;
          tc_fence_after();
          AKL_TRACE_AUX(true, j, 3);
          issue_pv(p_lo, v_lo, tmem + kColO, acc);
          tc_commit(ctx.bars + B_PVDONE * 8);
          tc_commit(ctx.bars + (B_PEMPTY + b * 2 + c) * 8);
          AKL_TRACE_AUX(true, j, 4);
          if (c == 1 || j == ntile - 1) tc_commit(ctx.bars + (B_VEMPTY + b) * 8);
        }
        if (ok) tc_commit(ctx.bars + B_ALLDONE * 8);
      }
    }
  } else if (warp >= 8) {
    // ================================================================ correction warpgroups
    // warps 8-11 own O columns 0-127, warps 16-19 columns 128-255
    const int row = tid & 127;
    const uint32_t col0 = kColO + (warp >= 16 ? 128u : 0u);
    const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const float* sm_alpha = reinterpret_cast<const float*>(smem_gen + kOffAlpha);
    for (int iter = 0; begin_item<kBatch>(g, bref, sh, smem, smem_gen, iter, cur_request, drawn, it); ++iter) {
      ctx.status = g.status;
      const int ntile = it.ntile;
      for (int j = 0; j < ntile; ++j) {
        if (!wait(ctx, B_AREADY + (j & 7), (j >> 3) & 1)) break;
        AKL_TRACE_AUX(tid == 256, j, 0);
        const float alpha = sm_alpha[(j & 7) * 128 + row];
        if (j > 0) {
          // exact rescale skip: alpha == 1 for every row of the warp leaves O untouched (decided
          // before the wait, so that nothing but the fence stands between PV(j-1) and the loads)
          const bool rescale = __any_sync(0xffffffffu, alpha != 1.f);
          if (!wait(ctx, B_PVDONE, (j - 1) & 1)) break;          // every phase, in order
          AKL_TRACE_AUX(tid == 256, j, 1);
          if (rescale) {
            tc_fence_after();
            uint32_t oa[32], ob[32];
            tmem_ld32(lane_base + col0, oa);
            tmem_ld32(lane_base + col0 + 32, ob);
            tmem_wait_ld();
            scale32(oa, alpha);
            tmem_st32(lane_base + col0, oa);
            scale32(ob, alpha);
            tmem_st32(lane_base + col0 + 32, ob);
            tmem_ld32(lane_base + col0 + 64, oa);
            tmem_ld32(lane_base + col0 + 96, ob);
            tmem_wait_ld();
            scale32(oa, alpha);
            tmem_st32(lane_base + col0 + 64, oa);
            scale32(ob, alpha);
            tmem_st32(lane_base + col0 + 96, ob);
            tmem_wait_st();
            tc_fence_before();
          }
        }
        warp_arrive(ctx.bars + B_OREADY * 8, lane);
        AKL_TRACE_AUX(tid == 256, j, 2);
      }
    }
  } else {
    // ================================================================ softmax warpgroups
    reg_alloc<kRegsSoftmax>();
    const int wg = warp >> 2;                  // 0: even tiles, 1: odd tiles
    const int row = tid & 127;                 // query row inside the tile == TMEM lane
    const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t chain = smem + kOffChain + row * 8;
    float* sm_alpha = reinterpret_cast<float*>(smem_gen + kOffAlpha);
    for (int iter = 0; begin_item<kBatch>(g, bref, sh, smem, smem_gen, iter, cur_request, drawn, it); ++iter) {
    ctx.status = g.status;
    const int ntile = it.ntile, kvh = it.kvh, qt = it.qt;
    int grow, h;                                 // this row's token and q head
    item_row<kBatch>(it, row, grow, h);
    long long lim_ll = static_cast<long long>(g.prefix) + grow - g.kv_pos0;
    const int limit = static_cast<int>(lim_ll > g.N - 1 ? g.N - 1 : lim_ll);   // last visible local key (may be < 0)
    const float qs = kBatch
        ? g.qscalep[(static_cast<size_t>(kvh) * it.group * g.mtiles_cap + qt) * kQTile + row]
        : g.qscale[static_cast<size_t>(h) * g.mtiles_cap * kQTile + grow];
    const float* kscale = g.kscale + kvh * g.ntiles_cap;
    const float* vlog2r = g.vlog2r + kvh * g.ntiles_cap;
    const float* vinvr = g.vinvr + kvh * g.ntiles_cap;
    float m_own = -INFINITY, l_own = 0.f;      // this group's partial (m, l)
    bool ok = true;

    // per-tile constants are fetched one tile ahead so their latency is off the critical path
    float c_ks = 0.f, c_l2r = 0.f, c_inv = 0.f;
    if (wg < ntile) {
      c_ks = __ldg(kscale + wg);
      c_l2r = __ldg(vlog2r + wg);
      c_inv = __ldg(vinvr + wg);
    }

    for (int j = wg; j < ntile; j += 2) {
      const int u = j >> 1, b = u & 1, c = wg;
      const float t_ks = c_ks, t_l2r = c_l2r, t_inv = c_inv;
      if (j + 2 < ntile) {
        c_ks = __ldg(kscale + j + 2);
        c_l2r = __ldg(vlog2r + j + 2);
        c_inv = __ldg(vinvr + j + 2);
      }
      AKL_TRACE_POINT(7);
      // tile j reuses the P slot and the alpha slot of tile j-4: its PV must have completed
      // (which also means the correction group is done with alpha(j-4))
      if (j >= 4 && !wait(ctx, B_PEMPTY + b * 2 + c, ((u >> 1) - 1) & 1)) { ok = false; break; }
      if (!wait(ctx, B_SFULL + b, (u >> 1) & 1)) { ok = false; break; }
      tc_fence_after();
      __syncwarp();
      uint32_t sr[64];
      {
        uint32_t lo32[32], hi32[32];
        const uint32_t ta = lane_base + kColS + b * 128 + c * 64;
        tmem_ld32(ta, lo32);
        tmem_ld32(ta + 32, hi32);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) { sr[i] = lo32[i]; sr[32 + i] = hi32[i]; }
      }
      AKL_TRACE_POINT(0);
      tc_fence_before();
      warp_arrive(ctx.bars + (B_SEMPTY + b) * 8, lane);      // the eight softmax warps free the S buffer
      if (kDump) {
        float* dst = g.dbg_s + ((((static_cast<size_t>(h) * g.mtiles + qt) * g.nt + j) * kQTile + row) * kTile);
#pragma unroll
        for (int i = 0; i < 64; ++i) dst[i] = acc_value<kI8>(sr[i]);
      }
      const float sc = qs * t_ks;
      const int rem = limit - j * kTile;
      float s[64];
      float rowmax;
      float sc_late;      // factor still to be applied to s[] before the exponent
      if (rem >= kTile - 1) {
        // every key of the tile is visible: the row maximum of the scaled scores is the scaled
        // maximum of the raw ones (sc > 0 and rounding is monotonic, so the bits agree), and
        // the scaling itself moves into the exponent loop
        float rmax[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) rmax[i] = acc_value<kI8>(sr[i]);
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] = rmax[i];
#pragma unroll
        for (int i = 8; i < 64; i += 16) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            s[i + k] = acc_value<kI8>(sr[i + k]);
            s[i + 8 + k] = acc_value<kI8>(sr[i + 8 + k]);
            rmax[k] = fmax3(rmax[k], s[i + k], s[i + 8 + k]);
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) s[56 + k] = acc_value<kI8>(sr[56 + k]);
        rowmax = fmax3(fmax3(rmax[0], rmax[1], rmax[2]), fmax3(rmax[3], rmax[4], rmax[5]),
                       fmax3(rmax[6], rmax[7], fmax3(s[56], s[57], s[58])));
        rowmax = fmax3(rowmax, fmax3(s[59], s[60], s[61]), fmaxf(s[62], s[63]));
        rowmax *= sc;
        sc_late = sc;
      } else {
        float rmax[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) rmax[i] = -INFINITY;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float v = acc_value<kI8>(sr[i]) * sc;
          s[i] = (i <= rem) ? v : -INFINITY;
          rmax[i & 7] = fmaxf(rmax[i & 7], s[i]);
        }
        rowmax = fmaxf(fmaxf(fmaxf(rmax[0], rmax[1]), fmaxf(rmax[2], rmax[3])),
                       fmaxf(fmaxf(rmax[4], rmax[5]), fmaxf(rmax[6], rmax[7])));
        sc_late = 1.0f;     // already scaled; multiplying by one changes nothing (-inf stays -inf)
      }
      AKL_TRACE_POINT(1);
      // running maximum: take the value after tile j-1 from the other group, publish ours
      float m_prev;
      if (!chain_wait(ctx, chain, static_cast<uint32_t>(j), m_prev)) { ok = false; break; }
      const float m_new = fmaxf(m_prev, rowmax);
      chain_post(chain, static_cast<uint32_t>(j + 1), m_new);
      AKL_TRACE_POINT(2);
      // alpha of this tile goes to the correction group
      const float alpha_o = (m_prev == -INFINITY) ? 0.f : ex2((m_prev - m_new) * kLog2e);
      sm_alpha[(j & 7) * 128 + row] = alpha_o;
      warp_arrive(ctx.bars + (B_AREADY + (j & 7)) * 8, lane);
      const float alpha_l = (m_own == -INFINITY) ? 0.f : ex2((m_own - m_new) * kLog2e);
      const float pc = (m_new == -INFINITY) ? -INFINITY : (kLog2_448 + t_l2r) - m_new * kLog2e;
      m_own = m_new;
      float part[4] = {0.f, 0.f, 0.f, 0.f};
      // AKL_POLY_GROUPS of the 16 four-element groups send their second pair through the
      // polynomial on the FMA pipe instead of the MUFU (the two pipes run side by side)
#ifndef AKL_POLY_GROUPS
#define AKL_POLY_GROUPS 0
#endif
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        mul2(s[i], s[i + 1], sc_late);
        mul2(s[i + 2], s[i + 3], sc_late);
        fma2(s[i], s[i + 1], kLog2e, pc);
        fma2(s[i + 2], s[i + 3], kLog2e, pc);
        s[i] = ex2(s[i]);
        s[i + 1] = ex2(s[i + 1]);
        if (AKL_POLY_GROUPS > 0 && ((i >> 2) * AKL_POLY_GROUPS) % 16 < AKL_POLY_GROUPS) {
          s[i + 2] = fmaxf(s[i + 2], -125.f);
          s[i + 3] = fmaxf(s[i + 3], -125.f);
          exp2_poly2(s[i + 2], s[i + 3]);
        } else {
          s[i + 2] = ex2(s[i + 2]);
          s[i + 3] = ex2(s[i + 3]);
        }
        add2(part[0], part[1], s[i], s[i + 1]);
        add2(part[2], part[3], s[i + 2], s[i + 3]);
      }
      l_own = l_own * alpha_l + ((part[0] + part[1]) + (part[2] + part[3])) * t_inv;

      AKL_TRACE_POINT(3);
      // P -> E4M3 -> shared memory (128-byte-swizzled A operand of the PV MMA)
      const uint32_t prow = smem + kOffP + b * 16384;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const int i0 = q4 * 16;
        const uint32_t w0 = cvt_e4m3x4(s[i0 + 0], s[i0 + 1], s[i0 + 2], s[i0 + 3]);
        const uint32_t w1 = cvt_e4m3x4(s[i0 + 4], s[i0 + 5], s[i0 + 6], s[i0 + 7]);
        const uint32_t w2 = cvt_e4m3x4(s[i0 + 8], s[i0 + 9], s[i0 + 10], s[i0 + 11]);
        const uint32_t w3 = cvt_e4m3x4(s[i0 + 12], s[i0 + 13], s[i0 + 14], s[i0 + 15]);
        st_shared_v4(prow + swz128(row, c * 64 + i0), w0, w1, w2, w3);
        if (kDump) {
          uint8_t* dst = g.dbg_p + ((((static_cast<size_t>(h) * g.mtiles + qt) * g.nt + j) * kQTile + row) * kTile);
          *reinterpret_cast<uint4*>(dst + i0) = make_uint4(w0, w1, w2, w3);
        }
      }
      fence_async_smem();
      AKL_TRACE_POINT(4);

      warp_arrive(ctx.bars + (B_PFULL + b * 2 + c) * 8, lane);
      AKL_TRACE_POINT(6);
    }

    // ---------------------------------------------------------- epilogue
    // combine the two groups' partial (m, l); then each group writes half of the channels
    sm_fin[wg * 128 + row] = make_float2(m_own, l_own);
    if (ok && ntile > 0) ok = wait(ctx, B_ALLDONE, 0);
    asm volatile("bar.sync 1, 256;" ::: "memory");
    ok = __all_sync(0xffffffffu, ok) && (sh.abort_flag == 0);
    if (ok) {
      tc_fence_after();
      const float2 f0 = sm_fin[row], f1 = sm_fin[128 + row];
      const float m = fmaxf(f0.x, f1.x);
      const float l = ((f0.x == -INFINITY) ? 0.f : f0.y * ex2((f0.x - m) * kLog2e)) +
                      ((f1.x == -INFINITY) ? 0.f : f1.y * ex2((f1.x - m) * kLog2e));
      const float inv_l = (l > 0.f) ? g.vscale[kvh] / l : 0.f;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(g.out) + (static_cast<size_t>(grow) * g.Hq + h) * kD;
#pragma unroll 1
      for (int chh = 0; chh < 4; ++chh) {
        const int ch = wg * 4 + chh;
        uint32_t o[32];
        if (ntile > 0) {
          tmem_ld32(lane_base + kColO + ch * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (grow < g.T) {
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = v4 * 8 + e * 2;
              const float a = fmaf(__uint_as_float(o[i]), inv_l, sm_vmean[ch * 32 + i]);
              const float bb = fmaf(__uint_as_float(o[i + 1]), inv_l, sm_vmean[ch * 32 + i + 1]);
              __nv_bfloat162 t = __floats2bfloat162_rn(a, bb);
              pk[e] = *reinterpret_cast<uint32_t*>(&t);
            }
            *reinterpret_cast<uint4*>(orow + ch * 32 + v4 * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
      }
      if (wg == 0 && g.lse_out != nullptr && grow < g.T) {
        g.lse_out[static_cast<size_t>(grow) * g.Hq + h] =
            (l > 0.f) ? fmaf(m, kLog2e, log2f(l) - kLog2_448) : -INFINITY;
      }
      tc_fence_before();
    } else if (grow < g.T) {
      // a bounded wait ran out (the status word says so): leave no plausible-looking rows behind
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(g.out) + (static_cast<size_t>(grow) * g.Hq + h) * kD;
      const uint4 nan4 = make_uint4(0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u);
#pragma unroll 1
      for (int i = 0; i < 16; ++i) *reinterpret_cast<uint4*>(orow + wg * 128 + i * 8) = nan4;
      if (wg == 0 && g.lse_out != nullptr) g.lse_out[static_cast<size_t>(grow) * g.Hq + h] = INFINITY;
    }
    }   // items
  }

  __syncthreads();
  if (warp == kProducerWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

namespace {

// Opt the kernel instantiations into their dynamic shared memory once per device.
int configure_once() {
  static std::atomic<bool> configured[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { note_cuda_error(e, "cudaGetDevice"); return AKL_ERR_CUDA; }
  if (dev >= 0 && dev < 64 && configured[dev].load(std::memory_order_acquire)) return AKL_OK;
  // idempotent, so a race between host threads only repeats the calls
  const void* kernels[6] = {
      reinterpret_cast<const void*>(attn_sm100_kernel<false, false, false>), reinterpret_cast<const void*>(attn_sm100_kernel<false, true, false>),
      reinterpret_cast<const void*>(attn_sm100_kernel<true, false, false>), reinterpret_cast<const void*>(attn_sm100_kernel<true, true, false>),
      reinterpret_cast<const void*>(attn_sm100_kernel<false, false, true>), reinterpret_cast<const void*>(attn_sm100_kernel<false, true, true>)};
  for (const void* k : kernels) {
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) { note_cuda_error(e, "cudaFuncSetAttribute(attn)"); return AKL_ERR_CUDA; }
  }
  if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
  return AKL_OK;
}

}  // namespace

int launch_attention(const Geom& g, cudaStream_t s, bool dump) {
  int rc = configure_once();
  if (rc != AKL_OK) return rc;
  dim3 grid(g.mtiles, g.Hq);
  const bool i8 = (g.flags & AKL_FLAG_QK_I8) != 0;
  const BatchRef none{};
#ifdef AKL_TRACE
  dump = false;   // development build: the dump pointer receives the timeline, not the scores
#endif
  if (dump) {
    if (i8) attn_sm100_kernel<true, true, false><<<grid, kThreads, kSmemBytes, s>>>(g, none);
    else attn_sm100_kernel<true, false, false><<<grid, kThreads, kSmemBytes, s>>>(g, none);
  } else {
    if (i8) attn_sm100_kernel<false, true, false><<<grid, kThreads, kSmemBytes, s>>>(g, none);
    else attn_sm100_kernel<false, false, false><<<grid, kThreads, kSmemBytes, s>>>(g, none);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { note_cuda_error(e, "attn_sm100_kernel"); return AKL_ERR_CUDA; }
  return AKL_OK;
}

// Persistent form over the request table: one CTA per SM.
int launch_batch_attention(const BatchRef& b, bool qk_i8, int sm_count, cudaStream_t s) {
  int rc = configure_once();
  if (rc != AKL_OK) return rc;
  Geom unused;
  std::memset(&unused, 0, sizeof(unused));
  if (qk_i8) attn_sm100_kernel<false, true, true><<<sm_count, kThreads, kSmemBytes, s>>>(unused, b);
  else attn_sm100_kernel<false, false, true><<<sm_count, kThreads, kSmemBytes, s>>>(unused, b);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { note_cuda_error(e, "attn_sm100_kernel(batch)"); return AKL_ERR_CUDA; }
  return AKL_OK;
}

}  // namespace akl
