/*
 * akl.h -- C ABI of libakl_sm100a.so: fused FP8 paged EXTEND/prefill attention for
 * NVIDIA B200 (sm_100a).  Head dimension 256, page size 1, GQA n:4, E4M3 Q/K/V/P.
 *
 * This is the boundary a host binds instead of the reference's pybind11 torch
 * extension (one function taking 13 tensors, src/attn_kernel_lab/csrc/
 * fp8_prefill_attn.cu:689-696 and :812-824) and instead of the ~14 tensor-library
 * launches of its preprocessing (src/attn_kernel_lab/quant.py:433-695).
 *
 * Conventions (every entry point):
 *   - plain C types, raw device pointers, byte sizes; no tensor-library types;
 *   - returns 0 (AKL_OK) or a negative AKL_ERR_* code, never throws, never traps;
 *   - enqueues on the caller's stream and returns; never synchronises
 *     (docs/OPERATOR_CONTRACT.md:210-211 of the reference);
 *   - allocates no device memory: the caller owns inputs, outputs and the workspace
 *     (docs/OPERATOR_CONTRACT.md:204-221), whose addresses may be baked into a
 *     CUDA graph;
 *   - device-side waits are bounded; a wait that runs out stores a nonzero code in
 *     the workspace status word (akl_ws_layout_t.off_status) and the kernel returns.
 */
#ifndef AKL_H_
#define AKL_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AKL_ABI_VERSION 1
#define AKL_HEAD_DIM 256
#define AKL_KV_TILE 64   /* quantisation tile along the kv axis (reference BLK, quant.py:80) */
#define AKL_Q_TILE 128   /* query rows per CTA and padding granule (reference MPAD, quant.py:86) */
#define AKL_STAT_SLAB 32768 /* statistics slab in rows (reference SLAB, quant.py:87) */

enum {
  AKL_OK = 0,
  AKL_ERR_INVALID = -1,    /* null pointer, non-positive size, bad enum */
  AKL_ERR_UNSUPPORTED = -2,/* outside the surface: head_dim, heads, flags */
  AKL_ERR_CAPACITY = -3,   /* request does not fit the workspace it was given */
  AKL_ERR_CUDA = -4,       /* a CUDA runtime call failed; see akl_last_cuda_error() */
  AKL_ERR_ALIGN = -5,      /* pointer not aligned as required */
  AKL_ERR_TIMEOUT = -6     /* (status word only) a bounded device wait ran out */
};

enum { AKL_KV_BF16 = 0, AKL_KV_FP16 = 1 };
enum { AKL_IDX_I64 = 0, AKL_IDX_I32 = 1 };

/* akl_call_t.flags */
#define AKL_FLAG_ROTATE 1u    /* Hadamard-rotate Q and K (reference kwarg rotate, ops.py:497) */
#define AKL_FLAG_CENTER_K 2u  /* subtract the K channel mean (reference kwarg center_k, ops.py:498) */
#define AKL_FLAG_QK_I8 4u     /* Q and K as INT8 at amax/127 with an exact s32 QK^T (reference kwarg qk_i8,
                               * its default, ops.py:496; quant.py:416-430, 471-478); clear = FP8 E4M3 QK */

/* Capacity plan: the maxima a workspace is laid out for.
 * Replaces quant.FP8PrefillWorkspace.reserve / CapacityPlan (quant.py:175-196, :253-336). */
typedef struct akl_plan {
  int32_t max_kv_len;   /* largest idx length of any request */
  int32_t max_q_len;    /* largest extend length */
  int32_t q_heads;
  int32_t kv_heads;
} akl_plan_t;

/* Byte offsets of every named region inside ONE caller-owned allocation.
 * Replaces the named buffers of quant.py:303-321. */
typedef struct akl_ws_layout {
  uint64_t total_bytes;
  int32_t npairs;       /* ceil(max_kv_len / 128): 128-key tile pairs per kv head */
  int32_t ntiles;       /* 2 * npairs: capacity in 64-key tiles */
  int32_t mtiles;       /* ceil(max_q_len / 128) */
  int32_t reserved_;
  uint64_t off_q8;      /* [Hq][mtiles][2][128][128] u8, 128B-swizzled tile images */
  uint64_t off_qscale;  /* [Hq][mtiles*128] f32 */
  uint64_t off_k8;      /* [Hkv][npairs][2][128][128] u8, swizzled */
  uint64_t off_v8t;     /* [Hkv][npairs][256][128] u8, d-major, swizzled */
  uint64_t off_kscale;  /* [Hkv][ntiles] f32 */
  uint64_t off_vst;     /* [Hkv][ntiles] f32 */
  uint64_t off_vlog2r;  /* [Hkv][ntiles] f32 */
  uint64_t off_vinvr;   /* [Hkv][ntiles] f32 */
  uint64_t off_vam;     /* [Hkv][ntiles] f32 centred per-tile amax */
  uint64_t off_vscale;  /* [Hkv] f32 */
  uint64_t off_vsmax;   /* [Hkv] f32 raw max of vam (a MAX all-reduce may run on it) */
  uint64_t off_kmean;   /* [Hkv][256] f32 */
  uint64_t off_vmean;   /* [Hkv][256] f32 */
  uint64_t off_ktsum;   /* [Hkv][ntiles][256] f32 per-tile channel sums of K */
  uint64_t off_vtsum;   /* [Hkv][ntiles][256] f32 */
  uint64_t off_vtmax;   /* [Hkv][ntiles][256] f32 */
  uint64_t off_vtmin;   /* [Hkv][ntiles][256] f32 */
  uint64_t off_status;  /* [64] i32; word 0 = first device error code, 0 when clean */
} akl_ws_layout_t;

/* One rectangular request == one call of the reference operator
 * (ops.prefill_extend, src/attn_kernel_lab/ops.py:485-609). */
typedef struct akl_call {
  const void* q;        /* [T][Hq][256] bf16, contiguous */
  const void* k_pool;   /* [pool_rows][Hkv][256] bf16 | fp16 */
  const void* v_pool;
  const void* idx;      /* [N] i64 | i32 pool rows in position order (values unchecked) */
  void* out;            /* [T][Hq][256] bf16 */
  float* lse_out;       /* [T][Hq] f32 base-2 log-sum-exp, or NULL */
  void* workspace;      /* base of the allocation described by `plan` */
  uint64_t workspace_bytes;
  akl_plan_t plan;      /* what the workspace was laid out for */
  int32_t T;            /* extend length (q rows), >= 1 */
  int32_t N;            /* gathered kv length, >= 1 */
  int32_t prefix;       /* cached positions, 0 <= prefix <= N - T (+ kv_pos0 for a split) */
  int32_t q_heads;
  int32_t kv_heads;
  int32_t kv_dtype;     /* AKL_KV_* */
  int32_t idx_dtype;    /* AKL_IDX_* */
  uint32_t flags;       /* AKL_FLAG_* */
  float sm_scale;       /* folded into the Q scales (quant.py:479) */
  /* KV-axis split (multi-GPU long request): this call's idx covers global positions
   * [kv_pos0, kv_pos0 + N); `prefix` stays global; statistics are made global by the
   * caller between the phase calls below.  0 / N_total==N for an unsplit request. */
  int32_t kv_pos0;      /* multiple of 64 */
  int32_t n_total;      /* global kv length (the divisor of the channel means); 0 means N */
  int32_t tile0_global; /* index of this call's first 64-row tile in the global tile order */
  int32_t ntiles_global;/* number of global 64-row tiles present in the tile-sum arrays; 0 = local */
} akl_call_t;

/* (O, lse2) partial-state merge for a KV-axis split: out = sum_i 2^(lse_i - lse) O_i,
 * lse = log2 sum_i 2^lse_i.  New: the reference exposes base-2 LSE for this purpose
 * (docs/OPERATOR_CONTRACT.md:57,238-242) but ships no merge. */
typedef struct akl_merge {
  const void* const* parts_o;     /* device array of nparts pointers to [rows][256] bf16 */
  const float* const* parts_lse;  /* device array of nparts pointers to [rows] f32 */
  void* out;                      /* [rows][256] bf16 */
  float* lse_out;                 /* [rows] f32 or NULL */
  int32_t nparts;
  int32_t rows;                   /* T * Hq */
} akl_merge_t;

int akl_abi_version(void);
const char* akl_strerror(int code);
const char* akl_last_cuda_error(void);

/* Workspace geometry.  Pure host arithmetic; no CUDA call. */
int akl_workspace_layout(const akl_plan_t* plan, akl_ws_layout_t* out);

/* The whole operator for one request: statistics, transform, attention, output write.
 * Replaces gather_quantize_kv + quantize_q + ext.fp8_prefill_attn + the final
 * permute-copy (ops.py:563-609). */
int akl_prefill_extend(const akl_call_t* call, void* stream);

/* The same work as separate phases, for callers that must make the statistics global
 * between them (KV-axis split) or want the quantised artifacts alone:
 *   1 akl_kv_tile_stats      per-tile K/V channel sums + V min/max   (quant.py:532-568)
 *   2 akl_kv_means           ordered reduction -> kmean, vmean; vam, vsmax (quant.py:566-581)
 *   3 akl_kv_scales          vst, r_t, vlog2r, vinvr, vscale          (quant.py:582-584, :673-679)
 *   4 akl_kv_transform       centre, rotate, quantise K and V         (quant.py:589-668)
 *   5 akl_quantize_q         rotate + per-row quantise Q              (quant.py:433-480)
 *   6 akl_attention          the fused kernel                         (fp8_prefill_attn.cu:220-681)
 */
int akl_kv_tile_stats(const akl_call_t* call, void* stream);
int akl_kv_means(const akl_call_t* call, void* stream);
int akl_kv_scales(const akl_call_t* call, void* stream);
int akl_kv_transform(const akl_call_t* call, void* stream);
int akl_quantize_q(const akl_call_t* call, void* stream);
int akl_attention(const akl_call_t* call, void* stream);

/* Diagnostic twin of akl_attention: same launch, and additionally stores, for every
 * (q head, 128-row Q tile, 64-key tile, row), the 64 raw fp32 QK^T accumulators and the 64
 * E4M3 P bytes fed to the PV MMA.  s_dump / p_dump: [Hq][ceil(T/128)][ceil(N/64)][128][64].
 * Plays the role of the reference's score/probability probes (tests/kernel/
 * test_divergence_hunting.py); parity tests use it to check P byte-for-byte. */
int akl_attention_dump(const akl_call_t* call, float* s_dump, uint8_t* p_dump, void* stream);

int akl_merge_states(const akl_merge_t* m, void* stream);

/* ---- batched variable-length entry --------------------------------------------------
 * R independent requests in FOUR launches (statistics + Q quantisation, means + scales,
 * K/V transform, attention) instead of four per request.  Replaces the per-request Python
 * loop of the reference's engine backend
 * (engines/sglang/integration/fp8_prefill/backend.py:267-289); every request's result is
 * bit-equal to akl_prefill_extend on the same inputs.
 *
 * Lengths, pointers and offsets of the requests live in a REQUEST TABLE in device memory,
 * which the kernels read; the launch itself depends only on the capacities.  So a CUDA graph
 * that holds akl_prefill_extend_batch can be replayed after the table's contents changed
 * (other lengths, other request count, other tensors), as long as they fit the capacities.
 * The host fills a host copy of the table with akl_batch_plan and copies it to the device
 * (the copy may itself be a node of the graph).  The attention launch is persistent: one
 * CTA per SM draws (request, q head, 128-row tile) work items, longest first, from a list in
 * the table through an atomic counter. */
typedef struct akl_batch_caps {
  int32_t max_requests;
  int32_t max_total_kv_pairs;  /* capacity in 128-key tile pairs: >= sum_r ceil(N_r / 128) */
  int32_t max_total_q_tiles;   /* capacity in 128-row query tiles: >= sum_r ceil(T_r / 128) */
  int32_t q_heads;
  int32_t kv_heads;
  int32_t reserved_;
} akl_batch_caps_t;

typedef struct akl_batch_layout {
  uint64_t workspace_bytes;    /* device scratch shared by the batch (1024-byte aligned base) */
  uint64_t table_bytes;        /* size of the request table, host copy and device copy alike */
  uint64_t ws_off_status;      /* [64] i32 inside the workspace; word 0 = first device error code */
  /* inside the table: a 64-byte header of i32 words {magic, n_requests, n_stat_items, n_q_ctas,
   * n_attn_items, next work item, ...}; one geometry record per request; running totals of the
   * statistics items and of the Q-quantisation CTAs per request; the attention work list of
   * {request, q_head << 16 | q_tile} i32 pairs in execution order */
  uint32_t table_off_geoms;
  uint32_t table_geom_stride;
  uint32_t table_off_stat_totals;
  uint32_t table_off_qcta_totals;
  uint32_t table_off_items;
  uint32_t reserved_;
} akl_batch_layout_t;

typedef struct akl_batch_request {
  const void* q;        /* [T][Hq][256] bf16 */
  const void* k_pool;   /* [pool_rows][Hkv][256]; may differ between requests */
  const void* v_pool;
  const void* idx;      /* [N] */
  void* out;            /* [T][Hq][256] bf16 */
  float* lse_out;       /* [T][Hq] or NULL */
  int32_t T, N, prefix;
  int32_t reserved_;
} akl_batch_request_t;

typedef struct akl_batch {
  akl_batch_caps_t caps;
  void* workspace;             /* device, akl_batch_layout_t.workspace_bytes */
  uint64_t workspace_bytes;
  void* table;                 /* device copy of the request table (16-byte aligned) */
  uint64_t table_bytes;
  int32_t kv_dtype;            /* AKL_KV_*, one for the whole batch */
  int32_t idx_dtype;           /* AKL_IDX_* */
  uint32_t flags;              /* AKL_FLAG_* */
  float sm_scale;
} akl_batch_t;

/* Sizes for the given capacities.  Pure host arithmetic. */
int akl_batch_layout(const akl_batch_caps_t* caps, akl_batch_layout_t* out);

/* Validates the requests like akl_prefill_extend validates one, packs them into the batch
 * workspace, sorts the attention work items longest first and writes the request table into
 * `table_host` (b->table_bytes bytes of host memory; b->table is not touched).  Pure host
 * arithmetic: no CUDA call.  AKL_ERR_CAPACITY when the requests exceed b->caps. */
int akl_batch_plan(const akl_batch_t* b, const akl_batch_request_t* requests, int32_t n_requests,
                   void* table_host);

/* The four launches.  b->table must hold (in stream order) a table written by akl_batch_plan
 * for the same caps, workspace, dtypes and flags. */
int akl_prefill_extend_batch(const akl_batch_t* b, void* stream);

/* A subset of the batch's launches, in their fixed order, for callers that put their own work
 * between them and for per-phase timing: the batched counterpart of the phase entry points above. */
#define AKL_BATCH_STATS 1u      /* K/V tile statistics */
#define AKL_BATCH_MEANS 2u      /* channel means, V tile scales, fold arrays */
#define AKL_BATCH_TRANSFORM 4u  /* K/V centre, rotate, quantise; Q rotate, quantise */
#define AKL_BATCH_ATTENTION 8u
#define AKL_BATCH_ALL 15u
int akl_prefill_extend_batch_phases(const akl_batch_t* b, uint32_t phases, void* stream);

/* Self-test of the preprocessing kernels' division.  They divide 16 384 (a K/V tile) or 256 (a Q
 * row) values by one scale, and do it as a correctly rounded reciprocal plus one fused remainder
 * correction instead of one IEEE division per value; the bytes must be those of the reference's
 * true division (quant.py:416-430, 471-478).  For each of the n_scales device floats this launch
 * divides every dividend significand (2^23), both signs, in four quotient binades, both ways, and
 * adds the number of quotients whose bits differ to *mismatches (device, caller-zeroed).
 * No counterpart in the reference: a check of this build's own arithmetic. */
int akl_selftest_exact_division(const float* scales, int32_t n_scales, uint64_t* mismatches, void* stream);

/* The whole operator (same work and same results as akl_prefill_extend) for callers that cannot
 * allocate device memory -- an engine plugin that is handed no allocator, or a host whose memory
 * pool is frozen after start-up.  The workspace is a 16 MiB array built into the library (held by
 * every GPU that loads it, until the process exits), so `workspace`, `workspace_bytes` and `plan`
 * of the call are ignored.  Accepted while the workspace layout for the request's own sizes fits
 * 16 MiB (e.g. N = 4096, T = 512 at 32:4 heads needs 13.1 MiB); beyond that AKL_ERR_CAPACITY.
 * The first call on a device looks up the array's address: make it before any stream capture.
 * All calls share the array and it keeps the last call's contents (the status words are cleared
 * on every call); calls whose GPU work overlaps race.  Calls no cudaMalloc/cudaFree.
 * This entry point has no counterpart in the reference. */
int akl_prefill_extend_static_scratch(const akl_call_t* call, void* stream);

/* The status word of the last accepted static-scratch call on the current device, copied to
 * *host_out asynchronously on `stream` (synchronise, then read): 0 when clean, AKL_ERR_TIMEOUT when
 * a bounded device-side wait ran out.  The array's address is cached per device, so neither entry
 * point may be used on a device after cudaDeviceReset.  No counterpart in the reference. */
int akl_static_scratch_status(int32_t* host_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AKL_H_ */
