// C ABI of libakl_sm100a.so (declared in include/akl.h): argument checking, workspace
// geometry, and the phase sequence of one request.  No device allocation, no stream
// synchronisation, no exceptions across the boundary.
#include <cstdio>
#include <cstring>

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

int need_q(const akl_call_t* c) { return (c->q == nullptr) ? AKL_ERR_INVALID : AKL_OK; }
int need_out(const akl_call_t* c) { return (c->out == nullptr) ? AKL_ERR_INVALID : AKL_OK; }

}  // namespace
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
  int rc = build_geom(c, &g);
  if (rc != AKL_OK) return rc;
  if ((rc = need_q(c)) != AKL_OK) return rc;
  if ((rc = need_out(c)) != AKL_OK) return rc;
  if (c->kv_pos0 != 0 || (c->n_total != 0 && c->n_total != c->N) || c->tile0_global != 0)
    return AKL_ERR_INVALID;   // a split request must make its statistics global between the phases
  if (c->prefix > c->N - c->T) return AKL_ERR_INVALID;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if ((rc = launch_kv_tile_stats(g, c->kv_dtype, c->idx_dtype, s, /*with_q=*/true)) != AKL_OK) return rc;
  if ((rc = launch_kv_means(g, s, /*fuse_scales=*/true)) != AKL_OK) return rc;
  if ((rc = launch_kv_transform(g, c->kv_dtype, c->idx_dtype, s)) != AKL_OK) return rc;
  return launch_attention(g, s);
}

int akl_merge_states(const akl_merge_t* m, void* stream) {
  if (m == nullptr || m->parts_o == nullptr || m->parts_lse == nullptr || m->out == nullptr) return AKL_ERR_INVALID;
  return launch_merge(*m, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
