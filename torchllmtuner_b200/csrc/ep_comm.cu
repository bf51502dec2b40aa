// Expert-parallel token exchange over NVLink peer memory, without NCCL and without a host synchronisation
// (replaces the count all-to-all + D2H sync + token all-to-all + permute of
// llmtuner/parallel/expert_parallel/token_dispatch.py:327-395,579-636 and its combine :396-408,234-275).
//
//   ep_exchange   every rank histograms its token copies per global expert, stores the row into every peer's count
//                 table (P2P stores + an epoch flag), waits (bounded) for all rows and derives, on the device:
//                 the 128-aligned segment offsets of its own experts, the live rows per expert, and for every global
//                 expert the row at which this rank's run starts inside the owner's padded buffer.
//   ep_push_rows  one warp per token copy writes the (optionally scaled) source row straight into the owner's receive
//                 buffer at its final expert-major position; can also emit <source row, other row> dot products
//                 (the router-weight gradient of the combine backward).
//   ep_pull_rows  one warp per token reads its k rows out of the owners' buffers, accumulates them score-weighted in
//                 fp32 and stores bf16; optionally keeps the raw rows for the backward pass.
//   ep_clone_rows copies the live rows of a receive buffer and zero-fills the alignment padding of every segment.
// Receive buffers have a fixed capacity; a run that would not fit sets the CapacityOverflow status and is dropped.
#include "comm.cuh"
#include "kernels.h"

namespace llmt {

int sm_count();   // gemm.cu: SMs of the current device

constexpr int kEpMaxExperts = 1024;

struct EpPeers {
  void* p[kMaxPeers];
};

__global__ void __launch_bounds__(1024) ep_exchange_kernel(const int64_t* __restrict__ flat, int64_t ncopies, int E, int R, int me,
                                                           EpPeers tables, EpPeers flags, uint32_t epoch, int cap,
                                                           int* __restrict__ seg_offsets, int* __restrict__ totals,
                                                           int* __restrict__ send_off, int* status) {
  __shared__ int hist[kEpMaxExperts];
  __shared__ int ok;
  const int El = E / R;
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  for (int64_t c = threadIdx.x; c < ncopies; c += blockDim.x) {
    const int64_t g = flat[c];
    if (g >= 0 && g < E) atomicAdd(&hist[(int)g], 1);
  }
  __syncthreads();
  // my row into every rank's table: table[slot][src = me][E]
  const int slot = epoch & 1u;
  for (int i = threadIdx.x; i < R * E; i += blockDim.x) {
    const int p = i / E, e = i - p * E;
    reinterpret_cast<int*>(tables.p[p])[((size_t)slot * R + me) * E + e] = hist[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < R) st_release_sys(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + me, epoch);
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < R) {
    if (!flag_wait_bounded(reinterpret_cast<const uint32_t*>(flags.p[me]) + threadIdx.x, epoch, status, 8000 + threadIdx.x)) ok = 0;
  }
  __syncthreads();
  if (!ok) return;
  const int* tab = reinterpret_cast<const int*>(tables.p[me]) + (size_t)slot * R * E;   // [src][E], complete
  // Per destination rank d (thread d): padded segment starts of d's experts, and where my run for each expert begins.
  if (threadIdx.x < R) {
    const int d = threadIdx.x;
    int seg = 0;
    for (int e = 0; e < El; ++e) {
      const int g = d * El + e;
      int tot = 0, before = 0;
      for (int s = 0; s < R; ++s) {
        const int c = __ldcv(tab + (size_t)s * E + g);
        if (s < me) before += c;
        tot += c;
      }
      send_off[g] = seg + before;
      if (d == me) {
        seg_offsets[e] = seg;
        totals[e] = tot;
      }
      seg += (tot + 127) / 128 * 128;
    }
    if (d == me) {
      seg_offsets[El] = seg < cap ? seg : (cap / 128 * 128);
      if (seg > cap) report_status(status, kStatusCapacityOverflow, 8100, seg);
    }
  }
}

// Destination of every token copy, in one pass: pos = stable rank of copy c among this rank's copies of the same expert
// (copies are numbered token-major, so the order is the one a stable sort by expert would give), then
// drank[c] = expert / El and drow[c] = send_off[expert] + pos. One CTA of 1024 threads walks the copies in chunks of
// 1024: lanes rank themselves inside their warp with match_any, a per-warp histogram and a scan over the 32 warps give
// the offset of each warp inside the chunk, a running per-expert count carries over between chunks. E <= 256.
constexpr int kEpPlanMaxExperts = 256;
__global__ void __launch_bounds__(1024) ep_plan_kernel(const int64_t* __restrict__ flat, int64_t ncopies, int E, int El,
                                                       const int* __restrict__ send_off, int* __restrict__ drank,
                                                       int* __restrict__ drow) {
  __shared__ int run[kEpPlanMaxExperts];             // copies of each expert in earlier chunks
  __shared__ int hist[32][kEpPlanMaxExperts];        // per warp: copies of each expert in this chunk, then exclusive scan over warps
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int e = threadIdx.x; e < E; e += blockDim.x) run[e] = 0;
  for (int64_t base = 0; base < ncopies; base += blockDim.x) {
    for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) hist[i / E][i % E] = 0;
    __syncthreads();
    const int64_t c = base + threadIdx.x;
    const bool live = c < ncopies;
    int g = live ? (int)flat[c] : -1;
    if (g < 0 || g >= E) g = -1;
    const unsigned peers = __match_any_sync(0xffffffffu, g);
    const int in_warp = __popc(peers & ((1u << lane) - 1u));
    if (g >= 0 && in_warp == 0) hist[warp][g] = __popc(peers);
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {   // exclusive scan over the warps, seeded with the running count
      int acc = run[e];
      for (int w = 0; w < 32; ++w) {
        const int n = hist[w][e];
        hist[w][e] = acc;
        acc += n;
      }
      run[e] = acc;
    }
    __syncthreads();
    if (g >= 0) {
      drank[c] = g / El;
      drow[c] = send_off[g] + hist[warp][g] + in_warp;
    } else if (live) {
      drank[c] = 0;
      drow[c] = -1;                                      // dropped by the push / pull kernels
    }
    __syncthreads();
  }
}

// dst_peer[drank[c]][drow[c]] = scale[c] * src[c / k]; optional dot_out[c] = <src[c / k], other[c]>
__global__ void __launch_bounds__(256) ep_push_rows_kernel(const __nv_bfloat16* __restrict__ src, const float* __restrict__ scale,
                                                           const int* __restrict__ drank, const int* __restrict__ drow,
                                                           EpPeers bufs, int cap, int64_t ncopies, int k, int D,
                                                           const __nv_bfloat16* __restrict__ other, float* __restrict__ dot_out,
                                                           int* status) {
  const int lane = threadIdx.x & 31;
  const int64_t c = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (c >= ncopies) return;
  const int r = drank[c], row = drow[c];
  const bool fits = row >= 0 && row < cap && r >= 0 && r < kMaxPeers && bufs.p[r] != nullptr;
  if (!fits && lane == 0) report_status(status, kStatusCapacityOverflow, 8200, row);
  const uint4* s = reinterpret_cast<const uint4*>(src + (c / k) * D);
  uint4* d = fits ? reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(bufs.p[r]) + (int64_t)row * D) : nullptr;
  const uint4* o = (other != nullptr) ? reinterpret_cast<const uint4*>(other + c * D) : nullptr;
  const float w = (scale != nullptr) ? scale[c] : 1.f;
  float dot = 0.f;
  for (int i = lane; i < D / 8; i += 32) {
    uint4 v = s[i];
    if (o != nullptr || scale != nullptr) {
      const __nv_bfloat162* vb = reinterpret_cast<const __nv_bfloat162*>(&v);
      float f[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 x = __bfloat1622float2(vb[q]);
        f[2 * q] = x.x;
        f[2 * q + 1] = x.y;
      }
      if (o != nullptr) {
        const uint4 ov = o[i];
        const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&ov);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 y = __bfloat1622float2(ob[q]);
          dot += f[2 * q] * y.x + f[2 * q + 1] * y.y;
        }
      }
      v.x = pack_bf16x2(w * f[0], w * f[1]); v.y = pack_bf16x2(w * f[2], w * f[3]);
      v.z = pack_bf16x2(w * f[4], w * f[5]); v.w = pack_bf16x2(w * f[6], w * f[7]);
    }
    if (d != nullptr) d[i] = v;
  }
  if (dot_out != nullptr) {
    dot = warp_sum(dot);
    if (lane == 0) dot_out[c] = dot;
  }
  __threadfence_system();   // this thread's peer stores are performed before the kernel (and so the ready flag) completes
}

// out[t] = sum_j w[t*k+j] * peer[drank][drow] (w == nullptr: plain sum); keep[t*k+j] = the raw row (optional)
__global__ void __launch_bounds__(256) ep_pull_rows_kernel(EpPeers bufs, const int* __restrict__ drank, const int* __restrict__ drow,
                                                           const float* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                                           __nv_bfloat16* __restrict__ keep, int cap, int T, int k, int D) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  for (int i = lane; i < D / 8; i += 32) {
    float acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = 0.f;
    for (int j0 = 0; j0 < k; j0 += 4) {           // four peer loads in flight per lane
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j0 + u;
        v[u] = make_uint4(0u, 0u, 0u, 0u);
        if (j < k) {
          const int64_t c = (int64_t)t * k + j;
          const int r = drank[c], row = drow[c];
          if (row >= 0 && row < cap) v[u] = ld_stream16(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(bufs.p[r]) + (int64_t)row * D) + i);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j0 + u;
        if (j < k) {
          const int64_t c = (int64_t)t * k + j;
          if (keep != nullptr) reinterpret_cast<uint4*>(keep + c * D)[i] = v[u];
          const float wj = (w != nullptr) ? w[c] : 1.f;
          const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = __bfloat1622float2(b[q]);
            acc[2 * q] += wj * f.x;
            acc[2 * q + 1] += wj * f.y;
          }
        }
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + (int64_t)t * D)[i] = o;
  }
}

// dst[r] = live(r) ? src[r] : 0 for r < seg_offsets[G]; one warp per row (grid-stride)
__global__ void __launch_bounds__(256) ep_clone_rows_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                            const int* __restrict__ seg_offsets, const int* __restrict__ totals,
                                                            int G, int D, int zero_pad) {
  const int lane = threadIdx.x & 31;
  const int used = seg_offsets[G];
  const int warps = gridDim.x * (blockDim.x >> 5);
  for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < used; r += warps) {
    int lo = 0, hi = G - 1;                      // last segment whose start is <= r
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (seg_offsets[mid] <= r) lo = mid; else hi = mid - 1;
    }
    const bool live = !zero_pad || (r - seg_offsets[lo] < totals[lo]);
    const uint4* s = reinterpret_cast<const uint4*>(src + (int64_t)r * D);
    uint4* d = reinterpret_cast<uint4*>(dst + (int64_t)r * D);
    for (int i = lane; i < D / 8; i += 32) d[i] = live ? s[i] : make_uint4(0u, 0u, 0u, 0u);
  }
}

}  // namespace llmt

using namespace llmt;
#define LLMT_CHECK_LAUNCH() return (cudaGetLastError() == cudaSuccess) ? 0 : -3

static EpPeers make_peers(void* const* p, int n) {
  EpPeers e{};
  for (int i = 0; i < kMaxPeers; ++i) e.p[i] = (i < n) ? p[i] : nullptr;
  return e;
}

extern "C" int llmt_ep_exchange(const int64_t* flat, int64_t ncopies, int E, int R, int me, void* const* tables,
                                void* const* flags, uint32_t epoch, int cap, int* seg_offsets, int* totals, int* send_off,
                                int* status, cudaStream_t st) {
  if (R < 1 || R > kMaxPeers || E < R || E % R || E > kEpMaxExperts || me < 0 || me >= R || cap % 128) return -10;
  ep_exchange_kernel<<<1, 1024, 0, st>>>(flat, ncopies, E, R, me, make_peers(tables, R), make_peers(flags, R), epoch, cap,
                                         seg_offsets, totals, send_off, status);
  LLMT_CHECK_LAUNCH();
}

extern "C" int llmt_ep_plan(const int64_t* flat, int64_t ncopies, int E, int R, const int* send_off, int* drank, int* drow,
                            cudaStream_t st) {
  if (ncopies <= 0) return 0;
  if (R < 1 || E % R || E > kEpPlanMaxExperts) return -10;
  ep_plan_kernel<<<1, 1024, 0, st>>>(flat, ncopies, E, E / R, send_off, drank, drow);
  LLMT_CHECK_LAUNCH();
}

extern "C" int llmt_ep_push_rows(const void* src, const float* scale, const int* drank, const int* drow, void* const* bufs, int R,
                                 int cap, int64_t ncopies, int k, int D, const void* other, float* dot_out, int* status,
                                 cudaStream_t st) {
  if (ncopies <= 0) return 0;
  if (D % 8 || R < 1 || R > kMaxPeers) return -10;
  ep_push_rows_kernel<<<(unsigned)((ncopies + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)src, scale, drank, drow, make_peers(bufs, R),
                                                                    cap, ncopies, k, D, (const __nv_bfloat16*)other, dot_out, status);
  LLMT_CHECK_LAUNCH();
}

extern "C" int llmt_ep_pull_rows(void* const* bufs, int R, const int* drank, const int* drow, const float* w, void* out, void* keep,
                                 int cap, int T, int k, int D, cudaStream_t st) {
  if (T <= 0) return 0;
  if (D % 8 || R < 1 || R > kMaxPeers) return -10;
  ep_pull_rows_kernel<<<(T + 7) / 8, 256, 0, st>>>(make_peers(bufs, R), drank, drow, w, (__nv_bfloat16*)out, (__nv_bfloat16*)keep, cap,
                                                  T, k, D);
  LLMT_CHECK_LAUNCH();
}

extern "C" int llmt_ep_clone_rows(const void* src, void* dst, const int* seg_offsets, const int* totals, int G, int D, int zero_pad,
                                  cudaStream_t st) {
  if (G <= 0) return 0;
  if (D % 8) return -10;
  ep_clone_rows_kernel<<<sm_count() * 4, 256, 0, st>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, seg_offsets, totals, G, D, zero_pad);
  LLMT_CHECK_LAUNCH();
}
