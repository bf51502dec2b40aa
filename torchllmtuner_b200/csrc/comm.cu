// Standalone communication kernels over NVLink peer memory (reference call sites being replaced: torch FSDP2's
// all_gather_into_tensor / reduce_scatter_tensor inside fully_shard,
// llmt reference llmtuner/parallel/fully_shard_parallel/fully_shard_parallel.py:198-604):
//   llmt_side_job      run one SideJob without a GEMM (first unit of a pass, or the tail a GEMM could not carry)
//   llmt_signal_peers  publish an epoch into one flag slot of every peer (release, system scope)
//   llmt_wait_flags    bounded wait until `n` consecutive local flags reach a value (acquire, system scope)
#include "comm.cuh"
#include "kernels.h"

namespace llmt {

__global__ void __launch_bounds__(256) side_job_kernel(SideJob job, int* status) {
  run_side_job(job, (long long)blockIdx.x * blockDim.x + threadIdx.x, (long long)gridDim.x * blockDim.x, status);
}

struct PeerFlagPtrs {
  uint32_t* p[kMaxPeers];
};

__global__ void signal_peers_kernel(PeerFlagPtrs flags, int npeers, int slot, uint32_t value) {
  const int i = threadIdx.x;
  if (i < npeers) {
    __threadfence_system();
    st_release_sys(flags.p[i] + slot, value);
  }
}

__global__ void wait_flags_kernel(const uint32_t* flags, int n, uint32_t value, int* status, int site, uint32_t max_polls) {
  const int i = threadIdx.x;
  if (i < n) flag_wait_bounded(flags + i, value, status, site + i, max_polls);
}

}  // namespace llmt

using namespace llmt;

static SideJob make_job(int kind, int nsrc, const void* const* src, void* dst, long long n, int accumulate,
                        const uint32_t* wait_flags, int n_wait, uint32_t wait_value) {
  SideJob j{};
  j.kind = kind;
  j.nsrc = nsrc;
  for (int i = 0; i < kMaxPeers; ++i) j.src[i] = (i < nsrc) ? src[i] : nullptr;
  j.dst = dst;
  j.n = n;
  j.accumulate = accumulate;
  j.wait_flags = wait_flags;
  j.n_wait = n_wait;
  j.wait_value = wait_value;
  return j;
}

extern "C" int llmt_side_job(int kind, int nsrc, const void* const* src, void* dst, long long n, int accumulate,
                             const uint32_t* wait_flags, int n_wait, uint32_t wait_value, int ctas, int* status,
                             cudaStream_t st) {
  if (kind == kSideNone || n <= 0) return 0;
  if (nsrc < 1 || nsrc > kMaxPeers || (kind == kSideCopy && (n & 15)) || (kind == kSideReduce && (n & 7))) return -10;
  if (ctas < 1) ctas = 32;
  side_job_kernel<<<ctas, 256, 0, st>>>(make_job(kind, nsrc, src, dst, n, accumulate, wait_flags, n_wait, wait_value), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int llmt_signal_peers(uint32_t* const* peer_flags, int npeers, int slot, uint32_t value, cudaStream_t st) {
  if (npeers < 1 || npeers > kMaxPeers) return -10;
  PeerFlagPtrs f{};
  for (int i = 0; i < npeers; ++i) f.p[i] = peer_flags[i];
  signal_peers_kernel<<<1, 32, 0, st>>>(f, npeers, slot, value);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int llmt_wait_flags(const uint32_t* flags, int n, uint32_t value, int site, uint32_t max_polls, int* status,
                               cudaStream_t st) {
  if (n < 1 || n > 32) return -10;
  wait_flags_kernel<<<1, 32, 0, st>>>(flags, n, value, status, site, max_polls ? max_polls : kMaxFlagPolls);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
