// Merge of per-split partial attention states for a KV-axis split of one long request:
//   lse = log2 sum_i 2^lse_i,   O = sum_i 2^(lse_i - lse) O_i.
// Each O_i is a normalised BF16 output that already carries the V channel mean; the weights
// sum to one, so the mean is counted once.  The reference exposes the base-2 LSE for this
// composition (docs/OPERATOR_CONTRACT.md:57,238-242) but has no merge of its own.
//
// HBM-bound: one warp per (row, head) vector of 256 channels, one 16-byte load per lane per
// part, one 16-byte store.  The part pointers may address memory that a collective has
// already landed in this GPU's HBM; the kernel issues plain loads only.
#include "akl_common.cuh"

namespace akl {

namespace {

constexpr int kMaxParts = 64;

__global__ void __launch_bounds__(256) merge_states_kernel(akl_merge_t m) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * 8 + warp;
  if (row >= m.rows) return;
  float mx = -INFINITY;
  for (int i = 0; i < m.nparts; ++i) mx = fmaxf(mx, m.parts_lse[i][row]);
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = 0.f;
  float den = 0.f;
  if (mx == -INFINITY) {
    // no split saw a key for this row: every part holds the V mean; pass part 0 through
    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(m.parts_o[0]) + row * kD + lane * 8);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(m.out) + row * kD + lane * 8) = raw;
    if (m.lse_out != nullptr && lane == 0) m.lse_out[row] = -INFINITY;
    return;
  }
  for (int i = 0; i < m.nparts; ++i) {
    const float li = m.parts_lse[i][row];
    if (li == -INFINITY) continue;
    const float w = exp2f(li - mx);
    den += w;
    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(m.parts_o[i]) + row * kD + lane * 8);
    float x[8];
    unpack8<AKL_KV_BF16>(raw, x);
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = fmaf(w, x[c], acc[c]);
  }
  const float inv = 1.0f / den;
  uint32_t pk[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    __nv_bfloat162 t = __floats2bfloat162_rn(acc[2 * e] * inv, acc[2 * e + 1] * inv);
    pk[e] = *reinterpret_cast<uint32_t*>(&t);
  }
  *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(m.out) + row * kD + lane * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  if (m.lse_out != nullptr && lane == 0) m.lse_out[row] = mx + log2f(den);
}

}  // namespace

int launch_merge(const akl_merge_t& m, cudaStream_t s) {
  if (m.nparts < 1 || m.nparts > kMaxParts || m.rows < 1) return AKL_ERR_INVALID;
  const unsigned blocks = static_cast<unsigned>((static_cast<long long>(m.rows) + 7) / 8);
  merge_states_kernel<<<blocks, 256, 0, s>>>(m);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { note_cuda_error(e, "merge_states_kernel"); return AKL_ERR_CUDA; }
  return AKL_OK;
}

}  // namespace akl
