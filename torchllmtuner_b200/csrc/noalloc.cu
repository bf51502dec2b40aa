// RMSNorm backward for callers that cannot allocate: the per-block partial sums of the weight gradient go to a
// fixed array inside the library instead of a buffer obtained per call. See noalloc.h for who this is for, what
// it costs and how calls may be ordered. This file calls no cudaMalloc / cudaFree and no allocating library routine.
#include <mutex>
#include <stdio.h>

#include "kernels.h"
#include "noalloc.h"

namespace {

constexpr int kMaxPartialRows = 296;  // upper bound of llmt_rmsnorm_bwd_partials()
constexpr size_t kScratchFloats = (size_t)kMaxPartialRows * kLlmtNoallocMaxHidden;

// The scratch itself. Device code could name it directly; host code below must translate it first.
static __device__ __align__(256) float g_noalloc_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;
thread_local char g_err[256] = "";

int fail(int code, const char* fmt, long a = 0, long b = 0) {
  snprintf(g_err, sizeof(g_err), fmt, a, b);
  return code;
}

// Once per device, with that device current: resolve the array's device address.
int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(-20, "llmt_rmsnorm_bwd_noalloc: cannot identify the current device (cudaGetDevice -> %ld, device %ld)", (long)e, dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(-20, "llmt_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed on device %ld with error %ld", dev, (long)e);
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" size_t llmt_noalloc_scratch_bytes(void) { return kScratchFloats * sizeof(float); }
extern "C" const char* llmt_noalloc_last_error(void) { return g_err; }

extern "C" int llmt_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                        void* dx, float* dw, int T, int D, cudaStream_t stream) {
  if (T < 0 || D <= 0 || (D % 8) != 0)
    return fail(-10, "llmt_rmsnorm_bwd_noalloc: bad shape T=%ld D=%ld (D must be a positive multiple of 8)", T, D);
  if (D > kLlmtNoallocMaxHidden)
    return fail(-10, "llmt_rmsnorm_bwd_noalloc: D=%ld exceeds the built-in scratch, which covers at most %ld columns", D,
                (long)kLlmtNoallocMaxHidden);
  if (T == 0) return 0;
  if (llmt_rmsnorm_bwd_partials(T) > kMaxPartialRows)
    return fail(-10, "llmt_rmsnorm_bwd_noalloc: kernel wants %ld partial rows, scratch holds %ld", llmt_rmsnorm_bwd_partials(T),
                (long)kMaxPartialRows);
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  // Every partial element read by the column reduction is written first by the row kernel of this same call, so
  // stale contents of the shared array are harmless and nothing is cleared here.
  const int lrc = llmt_rmsnorm_bwd(dy, x, w, rstd, dres, dx, scratch, dw, nullptr, /*accumulate=*/0, T, D, stream);
  if (lrc != 0) return fail(lrc, "llmt_rmsnorm_bwd_noalloc: kernel launch failed with code %ld", lrc);
  return 0;
}
