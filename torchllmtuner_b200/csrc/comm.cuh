// Peer-memory side jobs: the communication half of a fused compute + collective kernel.
//
// A SideJob describes a slice of a collective over NVLink peer memory (plain P2P loads and local stores, never a
// multicast load): either a copy of a byte range out of one peer's shard into this GPU's gather buffer (all-gather),
// or the reduction of one element range over every rank's bf16 gradient buffer into this GPU's fp32 shard
// (reduce-scatter with the cast and the accumulation folded in). The GEMM kernel runs the job on extra "comm" warps
// of every CTA while its MMA warps work through the tiles, so the transfer overlaps the math inside one kernel;
// the standalone kernel in comm.cu runs a job on its own when no GEMM is left to carry it.
// Cross-rank ordering uses epoch flags in symmetric memory: writers publish with st.release.sys into each reader's
// flag array, readers poll their own array with ld.acquire.sys under a poll limit (common.cuh).
#pragma once
#include "common.cuh"

namespace llmt {

constexpr int kMaxPeers = 8;
constexpr int kCommWarps = 4;
constexpr int kCommThreads = kCommWarps * 32;

enum SideJobKind : int { kSideNone = 0, kSideCopy = 1, kSideReduce = 2 };

struct SideJob {
  int kind;                     // SideJobKind
  int nsrc;                     // reduce: number of ranks summed (in rank order); copy: 1
  const void* src[kMaxPeers];   // copy: src[0]; reduce: bf16 base of the element range on every rank
  void* dst;                    // copy: local destination; reduce: fp32 shard range
  long long n;                  // copy: bytes (multiple of 16); reduce: elements (multiple of 8)
  int accumulate;               // reduce: dst += sum instead of dst = sum
  const uint32_t* wait_flags;   // optional: local flag array to poll before touching src
  int n_wait;                   // number of consecutive flags that must reach wait_value
  uint32_t wait_value;
};

__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Runs `job` cooperatively on `nthreads` threads (this thread is `tid`). Returns false when a flag wait expired.
__device__ __forceinline__ bool run_side_job(const SideJob& job, long long tid, long long nthreads, int* status) {
  if (job.kind == kSideNone) return true;
  if (job.wait_flags != nullptr) {
    // every lane polls (loads of one address coalesce); bounded
    for (int f = 0; f < job.n_wait; ++f)
      if (!flag_wait_bounded(job.wait_flags + f, job.wait_value, status, 5000 + f)) return false;
  }
  if (job.kind == kSideCopy) {
    const long long n16 = job.n >> 4;
    const uint4* s = reinterpret_cast<const uint4*>(job.src[0]);
    uint4* d = reinterpret_cast<uint4*>(job.dst);
    long long i = tid;
    for (; i + 3 * nthreads < n16; i += 4 * nthreads) {   // four loads in flight per thread
      const uint4 a = ld_peer16(s + i), b = ld_peer16(s + i + nthreads), c = ld_peer16(s + i + 2 * nthreads),
                  e = ld_peer16(s + i + 3 * nthreads);
      d[i] = a; d[i + nthreads] = b; d[i + 2 * nthreads] = c; d[i + 3 * nthreads] = e;
    }
    for (; i < n16; i += nthreads) d[i] = ld_peer16(s + i);
  } else {
    const long long n8 = job.n >> 3;
    float* d = reinterpret_cast<float*>(job.dst);
    for (long long i = tid; i < n8; i += nthreads) {
      uint4 v[kMaxPeers];
#pragma unroll
      for (int p = 0; p < kMaxPeers; ++p)
        if (p < job.nsrc) v[p] = ld_peer16(reinterpret_cast<const uint4*>(job.src[p]) + i);
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int p = 0; p < kMaxPeers; ++p) {
        if (p < job.nsrc) {
          const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v[p]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(b[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
      }
      float4* o = reinterpret_cast<float4*>(d + i * 8);
      float4 o0 = make_float4(acc[0], acc[1], acc[2], acc[3]), o1 = make_float4(acc[4], acc[5], acc[6], acc[7]);
      if (job.accumulate) {
        const float4 p0 = o[0], p1 = o[1];
        o0.x += p0.x; o0.y += p0.y; o0.z += p0.z; o0.w += p0.w;
        o1.x += p1.x; o1.y += p1.y; o1.z += p1.z; o1.w += p1.w;
      }
      o[0] = o0;
      o[1] = o1;
    }
  }
  return true;
}

}  // namespace llmt
