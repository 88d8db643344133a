// C ABI of libakl_sm100a.so (declared in include/akl.h): argument checking, workspace
// geometry, and the phase sequence of one request.  No device allocation, no stream
// synchronisation, no exceptions across the boundary.
#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <vector>

#include "akl_common.cuh"

namespace akl {

static thread_local char g_cuda_error[256] = "";

void note_cuda_error(cudaError_t e, const char* where) {
  std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", where, cudaGetErrorString(e));
}

namespace {

inline uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

int compute_layout(const akl_plan_t& p, akl_ws_layout_t* o) {
  if (p.max_kv_len < 1 || p.max_q_len < 1 || p.q_heads < 1 || p.kv_heads < 1) return AKL_ERR_INVALID;
  if (p.q_heads % p.kv_heads) return AKL_ERR_UNSUPPORTED;
  std::memset(o, 0, sizeof(*o));
  const uint64_t npairs = (static_cast<uint64_t>(p.max_kv_len) + kPair - 1) / kPair;
  const uint64_t ntiles = npairs * 2;
  const uint64_t mtiles = (static_cast<uint64_t>(p.max_q_len) + kQTile - 1) / kQTile;
  const uint64_t hq = p.q_heads, hkv = p.kv_heads;
  o->npairs = static_cast<int32_t>(npairs);
  o->ntiles = static_cast<int32_t>(ntiles);
  o->mtiles = static_cast<int32_t>(mtiles);
  uint64_t off = 0;
  auto take = [&](uint64_t bytes) {
    const uint64_t at = off;
    off = align_up(off + bytes, 1024);
    return at;
  };
  o->off_q8 = take(hq * mtiles * kImageBytes);
  o->off_qscale = take(hq * mtiles * kQTile * 4);
  o->off_k8 = take(hkv * npairs * kImageBytes);
  o->off_v8t = take(hkv * npairs * kImageBytes);
  o->off_kscale = take(hkv * ntiles * 4);
  o->off_vst = take(hkv * ntiles * 4);
  o->off_vlog2r = take(hkv * ntiles * 4);
  o->off_vinvr = take(hkv * ntiles * 4);
  o->off_vam = take(hkv * ntiles * 4);
  o->off_vscale = take(hkv * 4);
  o->off_vsmax = take(hkv * 4);
  o->off_kmean = take(hkv * kD * 4);
  o->off_vmean = take(hkv * kD * 4);
  o->off_ktsum = take(hkv * ntiles * kD * 4);
  o->off_vtsum = take(hkv * ntiles * kD * 4);
  o->off_vtmax = take(hkv * ntiles * kD * 4);
  o->off_vtmin = take(hkv * ntiles * kD * 4);
  o->off_status = take(256);
  o->total_bytes = off;
  return AKL_OK;
}

int build_geom(const akl_call_t* c, Geom* g) {
  if (c == nullptr) return AKL_ERR_INVALID;
  if (c->workspace == nullptr || c->k_pool == nullptr || c->v_pool == nullptr || c->idx == nullptr)
    return AKL_ERR_INVALID;
  if (c->T < 1 || c->N < 1 || c->prefix < 0) return AKL_ERR_INVALID;
  if (c->kv_dtype != AKL_KV_BF16 && c->kv_dtype != AKL_KV_FP16) return AKL_ERR_INVALID;
  if (c->idx_dtype != AKL_IDX_I64 && c->idx_dtype != AKL_IDX_I32) return AKL_ERR_INVALID;
  if (c->q_heads < 1 || c->kv_heads < 1 || c->q_heads % c->kv_heads) return AKL_ERR_UNSUPPORTED;
  if (c->kv_pos0 < 0 || c->kv_pos0 % kTile) return AKL_ERR_INVALID;
  if (!(c->sm_scale > 0.f)) return AKL_ERR_INVALID;
  if (c->flags & ~(AKL_FLAG_ROTATE | AKL_FLAG_CENTER_K | AKL_FLAG_QK_I8)) return AKL_ERR_INVALID;   // unknown mode bit
  akl_ws_layout_t L;
  int rc = compute_layout(c->plan, &L);
  if (rc != AKL_OK) return rc;
  if (c->workspace_bytes < L.total_bytes) return AKL_ERR_CAPACITY;
  if (c->q_heads != c->plan.q_heads || c->kv_heads != c->plan.kv_heads) return AKL_ERR_CAPACITY;
  const int nt = (c->N + kTile - 1) / kTile;
  const int mtiles = (c->T + kQTile - 1) / kQTile;
  // KV-axis split fields: the first local tile's global index must be the one kv_pos0 names,
  // the local tiles must lie inside the global tile range, and the global length must cover
  // this call's positions (all compared in 64 bits: the fields come from a foreign caller)
  if (c->tile0_global < 0 || c->ntiles_global < 0 || c->n_total < 0) return AKL_ERR_INVALID;
  if (static_cast<int64_t>(c->tile0_global) * kTile != static_cast<int64_t>(c->kv_pos0)) return AKL_ERR_INVALID;
  const int64_t last_tile = static_cast<int64_t>(c->tile0_global) + nt;
  const int64_t ntg64 = c->ntiles_global > 0 ? c->ntiles_global : last_tile;
  if (ntg64 < last_tile) return AKL_ERR_INVALID;
  if (c->n_total > 0 && static_cast<int64_t>(c->n_total) < static_cast<int64_t>(c->kv_pos0) + c->N) return AKL_ERR_INVALID;
  if (c->n_total == 0 && c->kv_pos0 != 0) return AKL_ERR_INVALID;   // a split must state the global length
  if (nt > L.ntiles || mtiles > L.mtiles || ntg64 > L.ntiles) return AKL_ERR_CAPACITY;
  const int ntg = static_cast<int>(ntg64);
  const uintptr_t mask = reinterpret_cast<uintptr_t>(c->workspace) | reinterpret_cast<uintptr_t>(c->k_pool) |
                         reinterpret_cast<uintptr_t>(c->v_pool) | reinterpret_cast<uintptr_t>(c->q) |
                         reinterpret_cast<uintptr_t>(c->out);
  if (mask & 15u) return AKL_ERR_ALIGN;
  if (reinterpret_cast<uintptr_t>(c->workspace) & 1023u) return AKL_ERR_ALIGN;
  uint8_t* ws = static_cast<uint8_t*>(c->workspace);
  std::memset(g, 0, sizeof(*g));
  g->q = c->q; g->k_pool = c->k_pool; g->v_pool = c->v_pool; g->idx = c->idx;
  g->out = c->out; g->lse_out = c->lse_out;
  g->q8 = ws + L.off_q8;
  g->qscale = reinterpret_cast<float*>(ws + L.off_qscale);
  g->k8 = ws + L.off_k8;
  g->v8t = ws + L.off_v8t;
  g->kscale = reinterpret_cast<float*>(ws + L.off_kscale);
  g->vst = reinterpret_cast<float*>(ws + L.off_vst);
  g->vlog2r = reinterpret_cast<float*>(ws + L.off_vlog2r);
  g->vinvr = reinterpret_cast<float*>(ws + L.off_vinvr);
  g->vam = reinterpret_cast<float*>(ws + L.off_vam);
  g->vscale = reinterpret_cast<float*>(ws + L.off_vscale);
  g->vsmax = reinterpret_cast<float*>(ws + L.off_vsmax);
  g->kmean = reinterpret_cast<float*>(ws + L.off_kmean);
  g->vmean = reinterpret_cast<float*>(ws + L.off_vmean);
  g->ktsum = reinterpret_cast<float*>(ws + L.off_ktsum);
  g->vtsum = reinterpret_cast<float*>(ws + L.off_vtsum);
  g->vtmax = reinterpret_cast<float*>(ws + L.off_vtmax);
  g->vtmin = reinterpret_cast<float*>(ws + L.off_vtmin);
  g->status = reinterpret_cast<int*>(ws + L.off_status);
  g->T = c->T; g->N = c->N; g->prefix = c->prefix; g->Hq = c->q_heads; g->Hkv = c->kv_heads;
  g->npairs_cap = L.npairs; g->ntiles_cap = L.ntiles; g->mtiles_cap = L.mtiles;
  g->nt = nt; g->mtiles = mtiles;
  g->kv_pos0 = c->kv_pos0;
  g->n_total = c->n_total > 0 ? c->n_total : c->N;
  g->tile0_global = c->tile0_global;
  g->ntiles_global = ntg;
  g->flags = c->flags;
  g->sm_scale = c->sm_scale;
  return AKL_OK;
}

// ---- batched entry: geometry of the shared workspace and of the request table ----------
struct BatchLayout {
  uint64_t ws_bytes, table_bytes;
  uint64_t off_q8, off_qscale, off_k8, off_v8t, off_kscale, off_vst, off_vlog2r, off_vinvr, off_vam,
      off_vscale, off_vsmax, off_kmean, off_vmean, off_ktsum, off_vtsum, off_vtmax, off_vtmin, off_status;
  uint32_t t_geoms, t_stat_off, t_qcta_off, t_items;
};

constexpr int kQRowsPerCtaHost = 128;  // rows one Q-quantisation item covers: one 128-row tile of one head

int compute_batch_layout(const akl_batch_caps_t& c, BatchLayout* o) {
  if (c.max_requests < 1 || c.max_total_kv_pairs < 1 || c.max_total_q_tiles < 1 || c.q_heads < 1 || c.kv_heads < 1)
    return AKL_ERR_INVALID;
  if (c.q_heads % c.kv_heads) return AKL_ERR_UNSUPPORTED;
  // flat item indices are 32-bit in the kernels
  const uint64_t R = c.max_requests, P = c.max_total_kv_pairs, NT = 2 * P, MT = c.max_total_q_tiles;
  const uint64_t hq = c.q_heads, hkv = c.kv_heads;
  if (R > (1u << 20) || 2 * NT * hkv >= (1ull << 31) || MT * hq * (kQTile / kQRowsPerCtaHost) >= (1ull << 31) ||
      hq >= (1u << 15))
    return AKL_ERR_UNSUPPORTED;
  std::memset(o, 0, sizeof(*o));
  uint64_t off = 0;
  auto take = [&](uint64_t bytes) {
    const uint64_t at = off;
    off = align_up(off + bytes, 1024);
    return at;
  };
  o->off_q8 = take(hq * MT * kImageBytes);
  o->off_qscale = take(hq * MT * kQTile * 4);
  o->off_k8 = take(hkv * P * kImageBytes);
  o->off_v8t = take(hkv * P * kImageBytes);
  o->off_kscale = take(hkv * NT * 4);
  o->off_vst = take(hkv * NT * 4);
  o->off_vlog2r = take(hkv * NT * 4);
  o->off_vinvr = take(hkv * NT * 4);
  o->off_vam = take(hkv * NT * 4);
  o->off_vscale = take(R * hkv * 4);
  o->off_vsmax = take(R * hkv * 4);
  o->off_kmean = take(R * hkv * kD * 4);
  o->off_vmean = take(R * hkv * kD * 4);
  o->off_ktsum = take(hkv * NT * kD * 4);
  o->off_vtsum = take(hkv * NT * kD * 4);
  o->off_vtmax = take(hkv * NT * kD * 4);
  o->off_vtmin = take(hkv * NT * kD * 4);
  o->off_status = take(256);
  o->ws_bytes = off;
  uint64_t t = sizeof(BatchHeader);
  o->t_geoms = static_cast<uint32_t>(t);
  t = align_up(t + R * sizeof(Geom), 16);
  o->t_stat_off = static_cast<uint32_t>(t);
  t = align_up(t + (R + 1) * 4, 16);
  o->t_qcta_off = static_cast<uint32_t>(t);
  t = align_up(t + (R + 1) * 4, 16);
  o->t_items = static_cast<uint32_t>(t);
  t = align_up(t + MT * hq * 8, 16);
  if (t >= (1ull << 32)) return AKL_ERR_UNSUPPORTED;
  o->table_bytes = t;
  return AKL_OK;
}

int check_batch(const akl_batch_t* b, BatchLayout* L) {
  if (b == nullptr || b->workspace == nullptr) return AKL_ERR_INVALID;
  if (b->kv_dtype != AKL_KV_BF16 && b->kv_dtype != AKL_KV_FP16) return AKL_ERR_INVALID;
  if (b->idx_dtype != AKL_IDX_I64 && b->idx_dtype != AKL_IDX_I32) return AKL_ERR_INVALID;
  if (!(b->sm_scale > 0.f)) return AKL_ERR_INVALID;
  if (b->flags & ~(AKL_FLAG_ROTATE | AKL_FLAG_CENTER_K | AKL_FLAG_QK_I8)) return AKL_ERR_INVALID;
  int rc = compute_batch_layout(b->caps, L);
  if (rc != AKL_OK) return rc;
  if (b->workspace_bytes < L->ws_bytes || b->table_bytes < L->table_bytes) return AKL_ERR_CAPACITY;
  if (reinterpret_cast<uintptr_t>(b->workspace) & 1023u) return AKL_ERR_ALIGN;
  return AKL_OK;
}

BatchRef make_ref(const akl_batch_t* b, const BatchLayout& L, void* table) {
  BatchRef r;
  r.table = static_cast<uint8_t*>(table);
  r.off_geoms = L.t_geoms;
  r.off_stat_off = L.t_stat_off;
  r.off_qcta_off = L.t_qcta_off;
  r.off_items = L.t_items;
  r.max_requests = b->caps.max_requests;
  return r;
}

int device_sm_count(int* out) {
  static std::atomic<int> cached[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { note_cuda_error(e, "cudaGetDevice"); return AKL_ERR_CUDA; }
  int n = (dev >= 0 && dev < 64) ? cached[dev].load(std::memory_order_relaxed) : 0;
  if (n == 0) {
    e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || n < 1) { note_cuda_error(e, "cudaDeviceGetAttribute(SM count)"); return AKL_ERR_CUDA; }
    if (dev >= 0 && dev < 64) cached[dev].store(n, std::memory_order_relaxed);
  }
  *out = n;
  return AKL_OK;
}

int need_q(const akl_call_t* c) { return (c->q == nullptr) ? AKL_ERR_INVALID : AKL_OK; }
int need_out(const akl_call_t* c) { return (c->out == nullptr) ? AKL_ERR_INVALID : AKL_OK; }

}  // namespace

// Every host-side check of the whole-operator entry, with no CUDA call: shared by
// akl_prefill_extend and the entry that works out of the library's own scratch.
int validate_prefill_call(const akl_call_t* c, Geom* g) {
  int rc = build_geom(c, g);
  if (rc != AKL_OK) return rc;
  if ((rc = need_q(c)) != AKL_OK) return rc;
  if ((rc = need_out(c)) != AKL_OK) return rc;
  if (c->kv_pos0 != 0 || (c->n_total != 0 && c->n_total != c->N) || c->tile0_global != 0)
    return AKL_ERR_INVALID;   // a split request must make its statistics global between the phases
  if (c->prefix > c->N - c->T) return AKL_ERR_INVALID;
  return AKL_OK;
}

}  // namespace akl

using namespace akl;

extern "C" {

int akl_abi_version(void) { return AKL_ABI_VERSION; }

const char* akl_strerror(int code) {
  switch (code) {
    case AKL_OK: return "ok";
    case AKL_ERR_INVALID: return "invalid argument (null pointer, non-positive size or unknown enum)";
    case AKL_ERR_UNSUPPORTED: return "outside the supported surface (head counts must divide; head_dim is 256)";
    case AKL_ERR_CAPACITY: return "request does not fit the workspace plan it was called with";
    case AKL_ERR_CUDA: return "a CUDA runtime call failed (see akl_last_cuda_error)";
    case AKL_ERR_ALIGN: return "pointer alignment: tensors need 16 bytes, the workspace 1024";
    case AKL_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    default: return "unknown error code";
  }
}

const char* akl_last_cuda_error(void) { return g_cuda_error; }

int akl_workspace_layout(const akl_plan_t* plan, akl_ws_layout_t* out) {
  if (plan == nullptr || out == nullptr) return AKL_ERR_INVALID;
  return compute_layout(*plan, out);
}

int akl_kv_tile_stats(const akl_call_t* c, void* stream) {
  Geom g;
  int rc = build_geom(c, &g);
  if (rc != AKL_OK) return rc;
  return launch_kv_tile_stats(g, c->kv_dtype, c->idx_dtype, static_cast<cudaStream_t>(stream));
}

int akl_kv_means(const akl_call_t* c, void* stream) {
  Geom g;
  int rc = build_geom(c, &g);
  if (rc != AKL_OK) return rc;
  return launch_kv_means(g, static_cast<cudaStream_t>(stream));
}

int akl_kv_scales(const akl_call_t* c, void* stream) {
  Geom g;
  int rc = build_geom(c, &g);
  if (rc != AKL_OK) return rc;
  return launch_kv_scales(g, static_cast<cudaStream_t>(stream));
}

int akl_kv_transform(const akl_call_t* c, void* stream) {
  Geom g;
  int rc = build_geom(c, &g);
  if (rc != AKL_OK) return rc;
  return launch_kv_transform(g, c->kv_dtype, c->idx_dtype, static_cast<cudaStream_t>(stream));
}

int akl_quantize_q(const akl_call_t* c, void* stream) {
  Geom g;
  int rc = build_geom(c, &g);
  if (rc != AKL_OK) return rc;
  if ((rc = need_q(c)) != AKL_OK) return rc;
  return launch_quantize_q(g, static_cast<cudaStream_t>(stream));
}

int akl_attention(const akl_call_t* c, void* stream) {
  Geom g;
  int rc = build_geom(c, &g);
  if (rc != AKL_OK) return rc;
  if ((rc = need_out(c)) != AKL_OK) return rc;
  return launch_attention(g, static_cast<cudaStream_t>(stream));
}

int akl_attention_dump(const akl_call_t* c, float* s_dump, uint8_t* p_dump, void* stream) {
  Geom g;
  int rc = build_geom(c, &g);
  if (rc != AKL_OK) return rc;
  if ((rc = need_out(c)) != AKL_OK) return rc;
  if (s_dump == nullptr || p_dump == nullptr) return AKL_ERR_INVALID;
  g.dbg_s = s_dump;
  g.dbg_p = p_dump;
  return launch_attention(g, static_cast<cudaStream_t>(stream), true);
}

int akl_prefill_extend(const akl_call_t* c, void* stream) {
  Geom g;
  int rc = validate_prefill_call(c, &g);
  if (rc != AKL_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if ((rc = launch_kv_tile_stats(g, c->kv_dtype, c->idx_dtype, s, /*with_q=*/true)) != AKL_OK) return rc;
  if ((rc = launch_kv_means(g, s, /*fuse_scales=*/true)) != AKL_OK) return rc;
  if ((rc = launch_kv_transform(g, c->kv_dtype, c->idx_dtype, s)) != AKL_OK) return rc;
  return launch_attention(g, s);
}

int akl_batch_layout(const akl_batch_caps_t* caps, akl_batch_layout_t* out) {
  if (caps == nullptr || out == nullptr) return AKL_ERR_INVALID;
  BatchLayout L;
  int rc = compute_batch_layout(*caps, &L);
  if (rc != AKL_OK) return rc;
  std::memset(out, 0, sizeof(*out));
  out->workspace_bytes = L.ws_bytes;
  out->table_bytes = L.table_bytes;
  out->ws_off_status = L.off_status;
  out->table_off_geoms = L.t_geoms;
  out->table_geom_stride = static_cast<uint32_t>(sizeof(Geom));
  out->table_off_stat_totals = L.t_stat_off;
  out->table_off_qcta_totals = L.t_qcta_off;
  out->table_off_items = L.t_items;
  return AKL_OK;
}

int akl_batch_plan(const akl_batch_t* b, const akl_batch_request_t* reqs, int32_t n, void* table_host) {
  BatchLayout L;
  int rc = check_batch(b, &L);
  if (rc != AKL_OK) return rc;
  if (table_host == nullptr || n < 0 || (n > 0 && reqs == nullptr)) return AKL_ERR_INVALID;
  if (n > b->caps.max_requests) return AKL_ERR_CAPACITY;
  const int hq = b->caps.q_heads, hkv = b->caps.kv_heads;
  const int64_t P = b->caps.max_total_kv_pairs, MT = b->caps.max_total_q_tiles;
  uint8_t* tab = static_cast<uint8_t*>(table_host);
  uint8_t* ws = static_cast<uint8_t*>(b->workspace);
  Geom* geoms = reinterpret_cast<Geom*>(tab + L.t_geoms);
  int32_t* stat_off = reinterpret_cast<int32_t*>(tab + L.t_stat_off);
  int32_t* qcta_off = reinterpret_cast<int32_t*>(tab + L.t_qcta_off);
  int32_t* items = reinterpret_cast<int32_t*>(tab + L.t_items);

  int64_t pair_off = 0, mtile_off = 0, stat_items = 0, q_ctas = 0;
  std::vector<double> req_cost(static_cast<size_t>(n), 0.0);
  for (int r = 0; r < n; ++r) {
    const akl_batch_request_t& q = reqs[r];
    if (q.q == nullptr || q.k_pool == nullptr || q.v_pool == nullptr || q.idx == nullptr || q.out == nullptr)
      return AKL_ERR_INVALID;
    if (q.T < 1 || q.N < 1 || q.prefix < 0 || q.prefix > q.N - q.T) return AKL_ERR_INVALID;
    const uintptr_t mask = reinterpret_cast<uintptr_t>(q.q) | reinterpret_cast<uintptr_t>(q.k_pool) |
                           reinterpret_cast<uintptr_t>(q.v_pool) | reinterpret_cast<uintptr_t>(q.out);
    if (mask & 15u) return AKL_ERR_ALIGN;
    const int64_t npairs = (static_cast<int64_t>(q.N) + kPair - 1) / kPair;
    const int64_t nt = (static_cast<int64_t>(q.N) + kTile - 1) / kTile;
    const int64_t mtiles = (static_cast<int64_t>(q.T) + kQTile - 1) / kQTile;
    if (pair_off + npairs > P || mtile_off + mtiles > MT || mtiles >= (1 << 16)) return AKL_ERR_CAPACITY;
    const int64_t tile_off = 2 * pair_off;
    Geom& g = geoms[r];
    std::memset(&g, 0, sizeof(g));
    g.q = q.q; g.k_pool = q.k_pool; g.v_pool = q.v_pool; g.idx = q.idx; g.out = q.out; g.lse_out = q.lse_out;
    g.q8 = ws + L.off_q8 + mtile_off * kImageBytes;
    g.qscale = reinterpret_cast<float*>(ws + L.off_qscale) + mtile_off * kQTile;
    // packed Q tiles: the same storage seen as [Hkv][group * MT] tiles; a request's packed tiles
    // (at most group * mtiles of them) start at group * mtile_off of every kv head's stripe
    const int group = hq / hkv;
    g.q8p = ws + L.off_q8 + static_cast<int64_t>(group) * mtile_off * kImageBytes;
    g.qscalep = reinterpret_cast<float*>(ws + L.off_qscale) + static_cast<int64_t>(group) * mtile_off * kQTile;
    const int64_t ptiles = (static_cast<int64_t>(q.T) * group + kQTile - 1) / kQTile;
    if (ptiles >= (1 << 16)) return AKL_ERR_CAPACITY;
    g.ptiles = static_cast<int>(ptiles);
    g.k8 = ws + L.off_k8 + pair_off * kImageBytes;
    g.v8t = ws + L.off_v8t + pair_off * kImageBytes;
    g.kscale = reinterpret_cast<float*>(ws + L.off_kscale) + tile_off;
    g.vst = reinterpret_cast<float*>(ws + L.off_vst) + tile_off;
    g.vlog2r = reinterpret_cast<float*>(ws + L.off_vlog2r) + tile_off;
    g.vinvr = reinterpret_cast<float*>(ws + L.off_vinvr) + tile_off;
    g.vam = reinterpret_cast<float*>(ws + L.off_vam) + tile_off;
    g.vscale = reinterpret_cast<float*>(ws + L.off_vscale) + static_cast<int64_t>(r) * hkv;
    g.vsmax = reinterpret_cast<float*>(ws + L.off_vsmax) + static_cast<int64_t>(r) * hkv;
    g.kmean = reinterpret_cast<float*>(ws + L.off_kmean) + static_cast<int64_t>(r) * hkv * kD;
    g.vmean = reinterpret_cast<float*>(ws + L.off_vmean) + static_cast<int64_t>(r) * hkv * kD;
    g.ktsum = reinterpret_cast<float*>(ws + L.off_ktsum) + tile_off * hkv * kD;
    g.vtsum = reinterpret_cast<float*>(ws + L.off_vtsum) + tile_off * hkv * kD;
    g.vtmax = reinterpret_cast<float*>(ws + L.off_vtmax) + tile_off * kD;
    g.vtmin = reinterpret_cast<float*>(ws + L.off_vtmin) + tile_off * kD;
    g.status = reinterpret_cast<int*>(ws + L.off_status);
    g.T = q.T; g.N = q.N; g.prefix = q.prefix; g.Hq = hq; g.Hkv = hkv;
    g.npairs_cap = static_cast<int>(P); g.ntiles_cap = static_cast<int>(2 * P); g.mtiles_cap = static_cast<int>(MT);
    g.nt = static_cast<int>(nt); g.mtiles = static_cast<int>(mtiles);
    g.kv_pos0 = 0; g.n_total = q.N; g.tile0_global = 0; g.ntiles_global = static_cast<int>(nt);
    g.flags = b->flags; g.sm_scale = b->sm_scale;
    stat_off[r] = static_cast<int32_t>(stat_items);
    qcta_off[r] = static_cast<int32_t>(q_ctas);
    stat_items += nt * hkv;
    q_ctas += static_cast<int64_t>(hkv) * ptiles;             // one per packed 128-row Q tile
    pair_off += npairs;
    mtile_off += mtiles;
    req_cost[r] = static_cast<double>(q.T) * (q.prefix + (q.T + 1) / 2.0);
  }
  stat_off[n] = static_cast<int32_t>(stat_items);
  qcta_off[n] = static_cast<int32_t>(q_ctas);
  for (int r = n + 1; r <= b->caps.max_requests; ++r) { stat_off[r] = stat_off[n]; qcta_off[r] = qcta_off[n]; }

  // attention work items: requests longest first (so the K/V tiles of one or two requests stay in
  // L2 while their items run), inside a request the deepest packed query tiles first, kv heads
  // together.  An item is (request, kv head, packed tile): 128 (token, head) rows of one kv head's
  // group, so a request of T tokens costs ceil(T * group / 128) tiles per kv head instead of
  // group * ceil(T / 128)
  std::vector<int> order(static_cast<size_t>(n));
  for (int r = 0; r < n; ++r) order[r] = r;
  std::stable_sort(order.begin(), order.end(), [&](int a, int c) { return req_cost[a] > req_cost[c]; });
  int64_t n_items = 0;
  for (int r : order) {
    const Geom& g = geoms[r];
    for (int pt = g.ptiles - 1; pt >= 0; --pt)
      for (int kvh = 0; kvh < hkv; ++kvh) {
        items[2 * n_items] = r;
        items[2 * n_items + 1] = (kvh << 16) | pt;
        ++n_items;
      }
  }
  BatchHeader* hdr = reinterpret_cast<BatchHeader*>(tab);
  std::memset(hdr, 0, sizeof(*hdr));
  hdr->magic = kBatchMagic;
  hdr->n_requests = n;
  hdr->n_stat_items = static_cast<int32_t>(stat_items);
  hdr->n_q_ctas = static_cast<int32_t>(q_ctas);
  hdr->n_attn_items = static_cast<int32_t>(n_items);
  hdr->attn_counter = 0;
  return AKL_OK;
}

int akl_prefill_extend_batch(const akl_batch_t* b, void* stream) {
  return akl_prefill_extend_batch_phases(b, AKL_BATCH_ALL, stream);
}

int akl_prefill_extend_batch_phases(const akl_batch_t* b, uint32_t phases, void* stream) {
  BatchLayout L;
  int rc = check_batch(b, &L);
  if (rc != AKL_OK) return rc;
  if (b->table == nullptr) return AKL_ERR_INVALID;
  if (reinterpret_cast<uintptr_t>(b->table) & 15u) return AKL_ERR_ALIGN;
  if (phases == 0 || (phases & ~AKL_BATCH_ALL)) return AKL_ERR_INVALID;
  int sms = 0;
  if ((rc = device_sm_count(&sms)) != AKL_OK) return rc;
  const BatchRef ref = make_ref(b, L, b->table);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if ((phases & AKL_BATCH_STATS) && (rc = launch_batch_stats(ref, b->kv_dtype, b->idx_dtype, sms, s)) != AKL_OK) return rc;
  if ((phases & AKL_BATCH_MEANS) && (rc = launch_batch_means(ref, b->caps.kv_heads, s)) != AKL_OK) return rc;
  if ((phases & AKL_BATCH_TRANSFORM) && (rc = launch_batch_transform(ref, b->kv_dtype, b->idx_dtype, sms, s)) != AKL_OK) return rc;
  if (phases & AKL_BATCH_ATTENTION) {
    if (!(phases & AKL_BATCH_MEANS)) {
      // the means launch rewinds the attention work counter; without it, do that here
      cudaError_t e = cudaMemsetAsync(&batch_header(ref)->attn_counter, 0, sizeof(int32_t), s);
      if (e != cudaSuccess) { note_cuda_error(e, "cudaMemsetAsync(work counter)"); return AKL_ERR_CUDA; }
    }
    return launch_batch_attention(ref, (b->flags & AKL_FLAG_QK_I8) != 0, sms, s);
  }
  return AKL_OK;
}

int akl_selftest_exact_division(const float* scales, int32_t n_scales, uint64_t* mismatches, void* stream) {
  if (scales == nullptr || mismatches == nullptr || n_scales < 1 || n_scales > 65535) return AKL_ERR_INVALID;
  return launch_exact_division_selftest(scales, n_scales, reinterpret_cast<unsigned long long*>(mismatches),
                                        static_cast<cudaStream_t>(stream));
}

int akl_merge_states(const akl_merge_t* m, void* stream) {
  if (m == nullptr || m->parts_o == nullptr || m->parts_lse == nullptr || m->out == nullptr) return AKL_ERR_INVALID;
  return launch_merge(*m, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
