// Allocation-free entry point of the kernel library. It has no counterpart in the reference project, which never
// launches device code of its own.
//
// Who needs it: code that must not, or cannot, call cudaMalloc at the moment it wants the kernel. Examples are a
// host that hands this library a fixed memory budget up front and forbids later growth, a caller running inside
// someone else's allocator or memory pool where a stray cudaMalloc would fragment or exceed that pool, and
// plugin-style callers that receive only raw device pointers and a stream and own no allocator at all. The
// regular RMSNorm backward needs a scratch matrix of per-block partial sums for the weight gradient; normally
// the bindings allocate it per call through torch. Here that scratch lives in a file-scope `static __device__`
// array inside the library instead, so the call needs nothing but the caller's own input and output buffers.
//
// Cost and limit: the array is sized for the largest supported row width, kLlmtNoallocMaxHidden = 8192 columns,
// times the 296 partial rows the kernel can produce: 296 * 8192 * 4 bytes = 9,699,328 bytes (about 9.25 MiB).
// Every GPU on which a process loads this library holds that memory from load until the process exits.
// Rows wider than the maximum are rejected (see the return codes); nothing is truncated.
//
// First call on a device: the host cannot use the array's name as a device address (in host code the name is
// only a stand-in symbol), so the first call made while a given device is current asks the runtime for the real
// address with cudaGetSymbolAddress and caches it for that device. Make that first call outside of any stream
// capture. The caller must have the target device current (cudaSetDevice) when calling.
//
// Sharing: all calls on one device use the same array, and it keeps whatever the previous call left in it. This
// kernel overwrites every element it later reads, so nothing needs clearing between calls. Two calls that may
// overlap on the GPU (different streams without an ordering between them) race on the array and must not be
// issued; calls on one stream, or on streams ordered by events, are safe.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { kLlmtNoallocMaxHidden = 8192 };

// RMSNorm backward without any allocation.
//   dy, x : bf16 [T, D] contiguous (x is the tensor that was normalised)     w : bf16 [D]
//   rstd  : fp32 [T] from the forward pass                                    dres : bf16 [T, D] or NULL, added to dx
//   dx    : bf16 [T, D] out                                                   dw : fp32 [D] out (overwritten)
// Returns 0 on success, -10 for a bad shape (D not a multiple of 8, D > kLlmtNoallocMaxHidden, T < 0),
// -20 when the scratch address could not be obtained on the current device, -3 when a launch failed.
// llmt_noalloc_last_error() returns a human-readable description of the last non-zero return on this thread.
int llmt_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                             float* dw, int T, int D, cudaStream_t stream);

// Bytes of device memory the library reserves per GPU for this entry point.
size_t llmt_noalloc_scratch_bytes(void);
const char* llmt_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
