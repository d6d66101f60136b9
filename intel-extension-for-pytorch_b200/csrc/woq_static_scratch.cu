// woq_b200_linear_static_scratch: the decode-size linear for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run a linear:
// code running under a framework's memory planner that has already handed out every byte,
// inference servers that forbid allocation after start-up to rule out fragmentation and
// out-of-memory in steady state, and plug-in sandboxes whose allocator hooks are not
// re-entrant.  woq_b200_linear needs a caller-provided workspace (partial tiles of the
// split-K reduction, per-tile arrival counters, a status word); this entry point takes that
// workspace from a fixed array in the library's own device image instead, so the caller
// passes nothing but inputs and outputs.  woq_b200_static_scratch_status reads (and clears) the
// array's status word, the way woq_b200_workspace_status does for a caller's workspace.
//
// The array below exists once per GPU that loads the library and stays resident until the
// process exits.  In host code its name is only a handle for the runtime, not a device
// address, so the address is fetched with cudaGetSymbolAddress the first time the entry
// point runs on a device (with that device current) and cached per device.
#include <cstdarg>
#include <mutex>

#include "../../include/woq_b200.h"
#include "woq_internal.h"

namespace {

// 4 MiB covers the split-K scratch of a 16-token call on GPUs with up to 252 SMs
// (64 KiB header + 16 KiB of partial tiles per SM).
constexpr size_t kStaticScratchBytes = 4u << 20;
constexpr int kMaxTokens = 16;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// Address of the array on device `dev` (which must be current): looked up once per device.
int scratch_for_device(int dev, void** out) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p)
      return woq::set_error(WOQ_B200_ERR_CUDA, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    // the array starts zeroed (static storage); nothing to clear here
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return WOQ_B200_OK;
}

}  // namespace

extern "C" int woq_b200_linear_static_scratch(const woq_b200_ctx* ctx, const void* x, int64_t m,
                                              int64_t ldx, int32_t fusion,
                                              const void* const* others, int32_t n_others,
                                              void* y, int64_t ldy, void* stream) {
  if (m > kMaxTokens)
    return woq::set_error(WOQ_B200_ERR_INVALID_ARG,
                          "woq_b200_linear_static_scratch takes at most %d tokens per call, got %lld",
                          kMaxTokens, (long long)m);
  const size_t need = woq_b200_workspace_bytes(ctx, m);
  if (need == 0) return woq::set_error(WOQ_B200_ERR_BAD_HANDLE, "not a woq_b200 context");
  if (need > kStaticScratchBytes)
    return woq::set_error(WOQ_B200_ERR_WORKSPACE,
                          "this GPU needs %zu bytes of scratch, the built-in array holds %zu", need,
                          kStaticScratchBytes);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return woq::set_error(WOQ_B200_ERR_CUDA, "cudaGetDevice failed or device index out of range: %s",
                          cudaGetErrorString(e));
  // the array of the CURRENT device is used, so that must be the device the context lives on
  if (dev != woq::ctx_device(ctx))
    return woq::set_error(WOQ_B200_ERR_INVALID_ARG, "the context lives on device %d but device %d is current",
                          woq::ctx_device(ctx), dev);
  void* scratch = nullptr;
  if (int rc = scratch_for_device(dev, &scratch)) return rc;
  // The array keeps whatever the previous call left.  The per-tile arrival counters must start
  // at zero; the partial tiles are always written before they are read.  The status word is
  // left alone: a call whose kernel gave up a bounded wait stays visible to
  // woq_b200_static_scratch_status until that is called.
  e = cudaMemsetAsync(static_cast<unsigned char*>(scratch) + 256, 0, woq_b200_workspace_header_bytes() - 256,
                      static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess)
    return woq::set_error(WOQ_B200_ERR_CUDA, "cudaMemsetAsync failed: %s", cudaGetErrorString(e));
  return woq_b200_linear(ctx, x, m, ldx, fusion, others, n_others, y, ldy, scratch, kStaticScratchBytes,
                         stream);
}

extern "C" int woq_b200_static_scratch_status(void* stream) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return woq::set_error(WOQ_B200_ERR_CUDA, "cudaGetDevice failed or device index out of range: %s",
                          cudaGetErrorString(e));
  void* scratch = nullptr;
  if (int rc = scratch_for_device(dev, &scratch)) return rc;
  return woq_b200_workspace_status(scratch, stream);
}
