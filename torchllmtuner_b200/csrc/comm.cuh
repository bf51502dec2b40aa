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
constexpr int kCommWarps = 8;
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

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Streaming copy out of (possibly peer) memory with `kCopyUnroll` 16-byte loads in flight per thread: over NVLink the
// round trip is a few microseconds, so the bytes in flight across the comm warps must cover bandwidth x latency (~2 MB).
constexpr int kCopyUnroll = 8;
__device__ __forceinline__ void copy_stream16(const uint4* __restrict__ s, uint4* __restrict__ d, long long n16, long long tid,
                                              long long nthreads) {
  long long i = tid;
  for (; i + (kCopyUnroll - 1) * nthreads < n16; i += kCopyUnroll * nthreads) {
    uint4 v[kCopyUnroll];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) v[u] = ld_stream16(s + i + u * nthreads);
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) d[i + u * nthreads] = v[u];
  }
  for (; i < n16; i += nthreads) d[i] = ld_stream16(s + i);
}

// Runs `job` cooperatively on `nthreads` threads (this thread is `tid`). Returns false when a flag wait expired.
__device__ __forceinline__ bool run_side_job(const SideJob& job, long long tid, long long nthreads, int* status) {
  if (job.kind == kSideNone) return true;
#ifdef LLMT_DEBUG
  {  // debug build: argument contracts are checked on the device and reported through the status word, never by a trap
    bool bad = (reinterpret_cast<uintptr_t>(job.dst) & 15) != 0 || job.n <= 0 || job.nsrc < 1 || job.nsrc > kMaxPeers;
    bad = bad || (job.kind == kSideCopy && (job.n & 15)) || (job.kind == kSideReduce && (job.n & 7));
    for (int p = 0; p < kMaxPeers; ++p)
      if (p < job.nsrc && (job.src[p] == nullptr || (reinterpret_cast<uintptr_t>(job.src[p]) & 15))) bad = true;
    if (bad) {
      if (tid == 0) report_status(status, kStatusBadArgument, 5900, job.kind);
      return false;
    }
  }
#endif
  if (job.wait_flags != nullptr) {
    // every lane polls (loads of one address coalesce); bounded
    for (int f = 0; f < job.n_wait; ++f)
      if (!flag_wait_bounded(job.wait_flags + f, job.wait_value, status, 5000 + f)) return false;
  }
  if (job.kind == kSideCopy) {
    copy_stream16(reinterpret_cast<const uint4*>(job.src[0]), reinterpret_cast<uint4*>(job.dst), job.n >> 4, tid, nthreads);
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

// ---------------------------------------------------------------------------------------------------------------
// Tensor-parallel row collectives fused with the GEMM that consumes / produces them (sequence parallelism: M rows are
// cut into `world` chunks of `chunk_rows`, chunk p belongs to rank p).
//
//   kTPAllGather      C = gather(A) * B. Every rank keeps its chunk of A in a symmetric slot. The comm warps pull the
//                     chunks out of peer memory into the local gathered matrix in ring order (own chunk first) and
//                     publish a per-chunk `landed` flag; the TMA producer walks the tiles in the same chunk order and
//                     polls the flag once per chunk, so the math on chunk i overlaps the transfer of chunk i+1.
//   kTPReduceScatter  out = sum over ranks of (A * B) restricted to this rank's chunk. Tiles are computed in the order
//                     rank+1, rank+2, ..., rank, written as bf16 partials into this rank's symmetric buffer; the warp
//                     that completes a chunk tells the chunk's owner. The comm warps pull this rank's chunk out of each
//                     peer's buffer as it becomes ready (nearest finisher first), accumulate in fp32 in a fixed order
//                     and finally add the local partial (and an optional residual) and store bf16.
//
// Flags live in symmetric memory, `ready[world] | done[world]` per slot, and carry the slot's epoch; counters are local,
// reset by the last arriver. Every wait is bounded.
enum TPMode : int { kTPNone = 0, kTPAllGather = 1, kTPReduceScatter = 2 };

struct TPFuse {
  int mode, world, rank;
  int chunk_rows;                       // multiple of 128; M == world * chunk_rows
  uint32_t epoch;                       // value the flags of this launch carry (monotonic per slot, from 1)
  const void* peer_src[kMaxPeers];      // AG: rank p's chunk [chunk_rows, K]; RS: rank p's partial matrix [M, N], both bf16
  void* local_dst;                      // AG: gathered A [M, K] (what the A tensor map covers)
  long long chunk_bytes;                // AG: bytes of one chunk
  const uint32_t* flags;                // local flag block of the slot: ready[world] | done[world]
  uint32_t* peer_flags[kMaxPeers];      // the same block on every rank
  uint32_t* counters;                   // local, zero between launches: arrive_a[world] | arrive_b[world] | landed[world]
  float* acc;                           // RS: fp32 scratch [chunk_rows, N]
  __nv_bfloat16* out;                   // RS: result [chunk_rows, N]
  const __nv_bfloat16* residual;        // RS: optional addend [chunk_rows, N]
  int n_cols;                           // RS: N (row length of partial / acc / out)
};

__device__ __forceinline__ void comm_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCommThreads) : "memory"); }

// All comm-warp groups of the grid arrive once; the last one resets the counter and returns true.
__device__ __forceinline__ bool grid_arrive_last(uint32_t* counter, uint32_t expected) {
  __threadfence();
  const uint32_t old = atomicAdd(counter, 1u);
  if (old + 1 == expected) {
    atomicExch(counter, 0u);
    __threadfence();
    return true;
  }
  return false;
}

// One comm thread polls, all comm threads of the CTA get the same verdict (so they reach the same barriers).
__device__ __forceinline__ bool comm_flag_wait(const uint32_t* flag, uint32_t expected, int* status, int site,
                                               volatile int* word, int ctid) {
  if (ctid == 0) *word = flag_wait_bounded(flag, expected, status, site) ? 1 : 0;
  comm_bar_sync();
  const int ok = *word;
  comm_bar_sync();
  return ok != 0;
}

// Comm warps of the all-gather form. `ctid` is the thread's index among the CTA's comm threads; `word` is a shared
// memory scratch word owned by the comm warps.
__device__ __forceinline__ void tp_allgather_comm(const TPFuse& tp, int ctid, volatile int* word, int* status) {
  const long long tid = (long long)blockIdx.x * kCommThreads + ctid, nthreads = (long long)gridDim.x * kCommThreads;
  const long long n16 = tp.chunk_bytes >> 4;
  uint32_t* arrive = tp.counters;
  uint32_t* landed = tp.counters + 2 * tp.world;
  for (int ci = 0; ci < tp.world; ++ci) {
    const int p = (tp.rank + ci) % tp.world;
    if (p != tp.rank && !comm_flag_wait(tp.flags + p, tp.epoch, status, 7000 + p, word, ctid)) return;
    const uint4* s = reinterpret_cast<const uint4*>(tp.peer_src[p]);
    uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(tp.local_dst) + (long long)p * tp.chunk_bytes);
    copy_stream16(s, d, n16, tid, nthreads);
    __threadfence();
    comm_bar_sync();
    if (ctid == 0 && grid_arrive_last(arrive + p, gridDim.x)) {
      st_release_gpu(landed + p, tp.epoch);                                   // the TMA producers may read chunk p now
      __threadfence_system();
      st_release_sys(tp.peer_flags[p] + tp.world + tp.rank, tp.epoch);        // rank p (or this rank) may reuse its slot
    }
  }
}

// TMA-producer side of the all-gather form: chunk p of the gathered matrix is complete.
__device__ __forceinline__ bool tp_wait_landed(const TPFuse& tp, int p, volatile int* abort_flag, int* status) {
  const uint32_t* f = tp.counters + 2 * tp.world + p;
  for (uint32_t i = 0; i < kMaxFlagPolls; ++i) {
    if ((int32_t)(ld_acquire_gpu(f) - tp.epoch) >= 0) {
      asm volatile("fence.proxy.async;" ::: "memory");   // generic-proxy writes of the comm warps -> async-proxy (TMA) reads
      return true;
    }
    if (*abort_flag) return false;
    __nanosleep(64);
  }
  report_status(status, kStatusFlagTimeout, 7100 + p, (int)tp.epoch);
  *abort_flag = 1;
  return false;
}

// Epilogue side of the reduce-scatter form: one warp finished its quarter of a tile of chunk `c`.
__device__ __forceinline__ void tp_tile_done(const TPFuse& tp, int c, uint32_t arrivals_per_chunk, int lane) {
  __threadfence();
  __syncwarp();
  if (lane == 0 && grid_arrive_last(tp.counters + c, arrivals_per_chunk)) {
    __threadfence_system();
    st_release_sys(tp.peer_flags[c] + tp.rank, tp.epoch);   // owner of chunk c (possibly this rank): my partial is complete
  }
}

// Comm warps of the reduce-scatter form.
__device__ __forceinline__ void tp_reducescatter_comm(const TPFuse& tp, int ctid, volatile int* word, int* status) {
  const long long tid = (long long)blockIdx.x * kCommThreads + ctid, nthreads = (long long)gridDim.x * kCommThreads;
  const long long n8 = ((long long)tp.chunk_rows * tp.n_cols) >> 3;
  const long long chunk_off16 = ((long long)tp.rank * tp.chunk_rows * tp.n_cols) >> 3;   // in uint4 (8 bf16)
  uint32_t* arrive_b = tp.counters + tp.world;
  for (int s = 1; s <= tp.world; ++s) {
    const int p = (tp.rank - s + 2 * tp.world) % tp.world;      // s == world: this rank's own partial, last
    if (!comm_flag_wait(tp.flags + p, tp.epoch, status, 7200 + p, word, ctid)) return;
    const uint4* src = reinterpret_cast<const uint4*>(tp.peer_src[p]) + chunk_off16;
    const bool first = (s == 1), last = (s == tp.world);
    constexpr int U = 4;   // peer loads and accumulator loads of U groups are all issued before the first use
    for (long long i0 = tid; i0 < n8; i0 += U * nthreads) {
      uint4 pv[U];
      float4 a0[U], a1[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * nthreads;
        if (i < n8) pv[u] = ld_stream16(src + i);
      }
      if (!first) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * nthreads;
          if (i < n8) {
            const float4* a = reinterpret_cast<const float4*>(tp.acc + i * 8);
            a0[u] = __ldcs(a);
            a1[u] = __ldcs(a + 1);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * nthreads;
        if (i < n8) {
          const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&pv[u]);
          float f[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 x = __bfloat1622float2(b[j]);
            f[2 * j] = x.x;
            f[2 * j + 1] = x.y;
          }
          if (!first) {
            f[0] += a0[u].x; f[1] += a0[u].y; f[2] += a0[u].z; f[3] += a0[u].w;
            f[4] += a1[u].x; f[5] += a1[u].y; f[6] += a1[u].z; f[7] += a1[u].w;
          }
          if (!last) {
            float4* a = reinterpret_cast<float4*>(tp.acc + i * 8);
            __stcs(a, make_float4(f[0], f[1], f[2], f[3]));
            __stcs(a + 1, make_float4(f[4], f[5], f[6], f[7]));
          } else {
            if (tp.residual != nullptr) {
              const uint4 r = reinterpret_cast<const uint4*>(tp.residual)[i];
              const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 x = __bfloat1622float2(rb[j]);
                f[2 * j] += x.x;
                f[2 * j + 1] += x.y;
              }
            }
            uint4 o;
            o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]); o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
            reinterpret_cast<uint4*>(tp.out)[i] = o;
          }
        }
      }
    }
    comm_bar_sync();
    if (ctid == 0 && grid_arrive_last(arrive_b + p, gridDim.x)) {
      __threadfence_system();
      st_release_sys(tp.peer_flags[p] + tp.world + tp.rank, tp.epoch);       // rank p (or this rank) may overwrite its partial
    }
  }
}

}  // namespace llmt
