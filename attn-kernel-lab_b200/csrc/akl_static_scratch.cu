// akl_prefill_extend_static_scratch: the whole operator for hosts that cannot allocate.
//
// Some callers of this library have no way to obtain device memory for the workspace: a plugin
// loaded into an engine that owns every allocation and hands out none, a call site that runs
// after the engine has frozen its memory pool, a process whose allocator hooks forbid cudaMalloc
// outside start-up.  For them the scratch lives inside the library, in one file-scope
// `__device__` array that every GPU which loads the library holds until the process exits.
//
// The array is 16 MiB (+1 KiB so a 1024-byte-aligned window of 16 MiB always fits).  A request
// is accepted when the workspace layout for exactly its own sizes fits that window: for example
// 4096 gathered positions with a 512-token extend at 32:4 heads (13.1 MiB); 8192 positions do
// not fit.  Larger requests are refused with AKL_ERR_CAPACITY.
//
// Rules for the caller:
//   * the first call on each device resolves the array's device address; make that first call
//     outside any stream capture;
//   * every call uses the same array and overwrites what the previous call left there, so two
//     calls whose GPU work overlaps (different streams, no dependency) race; serialise them;
//   * nothing here calls cudaMalloc, cudaFree or any allocating library routine;
//   * the array's address is looked up once per device and kept: after a cudaDeviceReset the
//     process must not call this entry point again on that device.
#include <mutex>

#include "akl_common.cuh"

namespace {

constexpr unsigned long long kScratchWindow = 16ull << 20;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kScratchWindow + 1024];

std::mutex g_mutex;
unsigned char* g_window[kMaxDevices] = {};   // 1024-byte aligned device address, per device
unsigned long long g_status_off[kMaxDevices] = {};   // where the last accepted call put its status words

// In host code the array's name is only a handle for the runtime, not a device address: the
// address a kernel may use comes from cudaGetSymbolAddress, asked with the right device current.
int static_window(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { akl::note_cuda_error(e, "cudaGetDevice"); return AKL_ERR_CUDA; }
  if (dev < 0 || dev >= kMaxDevices) return AKL_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_window[dev] == nullptr) {
    void* raw = nullptr;
    e = cudaGetSymbolAddress(&raw, g_static_scratch);
    if (e != cudaSuccess || raw == nullptr) {
      akl::note_cuda_error(e, "cudaGetSymbolAddress(static scratch)");
      return AKL_ERR_CUDA;
    }
    const unsigned long long a = (reinterpret_cast<unsigned long long>(raw) + 1023ull) & ~1023ull;
    g_window[dev] = reinterpret_cast<unsigned char*>(a);
  }
  *out = g_window[dev];
  return AKL_OK;
}

}  // namespace

extern "C" int akl_prefill_extend_static_scratch(const akl_call_t* call, void* stream) {
  if (call == nullptr) return AKL_ERR_INVALID;
  if (call->T < 1 || call->N < 1 || call->q_heads < 1 || call->kv_heads < 1) return AKL_ERR_INVALID;
  akl_call_t c = *call;
  c.plan.max_kv_len = call->N;          // the layout is computed for this request's own sizes
  c.plan.max_q_len = call->T;
  c.plan.q_heads = call->q_heads;
  c.plan.kv_heads = call->kv_heads;
  akl_ws_layout_t layout;
  int rc = akl_workspace_layout(&c.plan, &layout);
  if (rc != AKL_OK) return rc;
  if (layout.total_bytes > kScratchWindow) {
    akl::note_cuda_error(cudaSuccess, "static scratch: request needs more than the 16 MiB built into the library");
    return AKL_ERR_CAPACITY;
  }
  unsigned char* window = nullptr;
  if ((rc = static_window(&window)) != AKL_OK) return rc;
  c.workspace = window;
  c.workspace_bytes = kScratchWindow;
  // every host-side refusal comes before anything is enqueued: a refused call leaves the array, and
  // the status an earlier call recorded there, alone
  akl::Geom unused;
  if ((rc = akl::validate_prefill_call(&c, &unused)) != AKL_OK) return rc;
  // the array keeps the previous call's bytes; only the status words must start at zero
  cudaError_t e = cudaMemsetAsync(window + layout.off_status, 0, 256, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) { akl::note_cuda_error(e, "cudaMemsetAsync(status)"); return AKL_ERR_CUDA; }
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_status_off[dev] = layout.off_status;
  }
  return akl_prefill_extend(&c, stream);
}

// Copies the status word of the last accepted static-scratch call on the current device to
// *host_out, asynchronously on `stream` (read it after synchronising the stream): 0 when clean,
// AKL_ERR_TIMEOUT when a bounded device-side wait ran out.
extern "C" int akl_static_scratch_status(int32_t* host_out, void* stream) {
  if (host_out == nullptr) return AKL_ERR_INVALID;
  unsigned char* window = nullptr;
  int rc = static_window(&window);
  if (rc != AKL_OK) return rc;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return AKL_ERR_CUDA;
  unsigned long long off;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    off = g_status_off[dev];
  }
  e = cudaMemcpyAsync(host_out, window + off, sizeof(int32_t), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) { akl::note_cuda_error(e, "cudaMemcpyAsync(status)"); return AKL_ERR_CUDA; }
  return AKL_OK;
}
