// MoE routing and token movement kernels for sm_100a (reference call sites: llmtuner/models/common/moe/routing.py:31-345,
// llmtuner/models/qwen/routing.py:20-78, llmtuner/parallel/expert_parallel/token_dispatch.py:146-275,579-636):
//   router_topk      fp32 logits -> softmax / sigmoid scores -> (+bias for the selection only) -> top-k -> renormalise ->
//                    weights, indices and a per-expert histogram, one warp per token
//   router_topk_bwd  gradient of the combine weights back to the logits
//   permute_rows     token copies to their rows of the zero-padded expert-major layout
//   combine_rows     out[t] = sum_j w[t, j] * y[dest(t, j)] in fp32 (also the backward of permute with w = 1)
//   combine_bwd      dy rows and dw from d(out)
#include "common.cuh"
#include "kernels.h"

namespace llmt {

constexpr int kMaxEPerLane = 16;   // up to 512 experts
constexpr int kMaxTopK = 16;

// score_fn: 0 softmax, 1 sigmoid
__global__ void __launch_bounds__(256) router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                          float* __restrict__ weights, int64_t* __restrict__ indices,
                                                          float* __restrict__ counts, float* __restrict__ denom_out, int T, int E,
                                                          int k, int score_fn, int renorm, float route_scale) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int per = (E + 31) / 32;
  float sc[kMaxEPerLane], sel[kMaxEPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxEPerLane; ++i) {
    const int e = i * 32 + lane;
    sc[i] = (i < per && e < E) ? logits[(int64_t)t * E + e] : -INFINITY;
    mx = fmaxf(mx, sc[i]);
  }
  if (score_fn == 0) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i) {
      sc[i] = (sc[i] == -INFINITY) ? 0.f : __expf(sc[i] - mx);
      sum += sc[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i) sc[i] *= inv;
  } else {
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i) sc[i] = (sc[i] == -INFINITY) ? 0.f : 1.f / (1.f + __expf(-sc[i]));
  }
#pragma unroll
  for (int i = 0; i < kMaxEPerLane; ++i) {
    const int e = i * 32 + lane;
    sel[i] = (i < per && e < E) ? sc[i] + (bias != nullptr ? bias[e] : 0.f) : -INFINITY;
  }
  float wsel[kMaxTopK];
  int isel[kMaxTopK];
  float wsum = 0.f;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int bi = 0;
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i)
      if (sel[i] > best) { best = sel[i]; bi = i; }
    int be = bi * 32 + lane;
    // warp argmax, ties to the lower expert id (matches a stable top-k)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    const int owner = be & 31, slot = be >> 5;
    float w = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i)
      if (i == slot && lane == owner) { w = sc[i]; sel[i] = -INFINITY; }
    w = __shfl_sync(0xffffffffu, w, owner);
    wsel[j] = w;
    isel[j] = be;
    wsum += w;
  }
  const float d = renorm ? (wsum + 1e-20f) : 1.f;
  if (lane == 0) {
    for (int j = 0; j < k; ++j) {
      weights[(int64_t)t * k + j] = wsel[j] / d * route_scale;
      indices[(int64_t)t * k + j] = isel[j];
      atomicAdd(&counts[isel[j]], 1.f);
    }
    if (denom_out != nullptr) denom_out[t] = d;
  }
}

// dlogits from dweights. softmax: s = softmax(l), w_j = scale * s_j / S (S = sum_sel s + 1e-20 when renorm, else 1).
__global__ void __launch_bounds__(256) router_topk_bwd_kernel(const float* __restrict__ logits, const float* __restrict__ dweights,
                                                              const int64_t* __restrict__ indices, const float* __restrict__ denom,
                                                              float* __restrict__ dlogits, int T, int E, int k, int score_fn,
                                                              int renorm, float route_scale) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int per = (E + 31) / 32;
  float sc[kMaxEPerLane], ds[kMaxEPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxEPerLane; ++i) {
    const int e = i * 32 + lane;
    sc[i] = (i < per && e < E) ? logits[(int64_t)t * E + e] : -INFINITY;
    ds[i] = 0.f;
    mx = fmaxf(mx, sc[i]);
  }
  if (score_fn == 0) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i) { sc[i] = (sc[i] == -INFINITY) ? 0.f : __expf(sc[i] - mx); sum += sc[i]; }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i) sc[i] *= inv;
  } else {
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i) sc[i] = (sc[i] == -INFINITY) ? 0.f : 1.f / (1.f + __expf(-sc[i]));
  }
  const float S = renorm ? denom[t] : 1.f;
  // sum_j dW_j * w_j / scale, with w_j / scale = s_j / S
  float dot = 0.f;
  if (renorm) {
    for (int j = 0; j < k; ++j) {
      const int e = (int)indices[(int64_t)t * k + j];
      float sj = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxEPerLane; ++i)
        if (i == (e >> 5) && lane == (e & 31)) sj = sc[i];
      sj = __shfl_sync(0xffffffffu, sj, e & 31);
      dot += dweights[(int64_t)t * k + j] * sj / S;
    }
  }
  for (int j = 0; j < k; ++j) {
    const int e = (int)indices[(int64_t)t * k + j];
    const float g = (dweights[(int64_t)t * k + j] - dot) * route_scale / S;
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i)
      if (i == (e >> 5) && lane == (e & 31)) ds[i] = g;
  }
  if (score_fn == 0) {
    float inner = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i) inner += ds[i] * sc[i];
    inner = warp_sum(inner);
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i) {
      const int e = i * 32 + lane;
      if (i < per && e < E) dlogits[(int64_t)t * E + e] = sc[i] * (ds[i] - inner);
    }
  } else {
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i) {
      const int e = i * 32 + lane;
      if (i < per && e < E) dlogits[(int64_t)t * E + e] = ds[i] * sc[i] * (1.f - sc[i]);
    }
  }
}

// rows[dest[c]] = x[c / k] ; one warp per copy, 16-byte accesses (D % 8 == 0)
__global__ void __launch_bounds__(256) permute_rows_kernel(const __nv_bfloat16* __restrict__ x, const int64_t* __restrict__ dest,
                                                           __nv_bfloat16* __restrict__ rows, int64_t ncopies, int k, int D) {
  const int lane = threadIdx.x & 31;
  const int64_t c = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (c >= ncopies) return;
  const uint4* s = reinterpret_cast<const uint4*>(x + (c / k) * D);
  uint4* d = reinterpret_cast<uint4*>(rows + dest[c] * D);
  for (int i = lane; i < D / 8; i += 32) d[i] = s[i];
}

// out[t] = sum_j w[t, j] * y[dest[t * k + j]] (w == nullptr: plain sum), fp32 accumulate; one warp per token
__global__ void __launch_bounds__(256) combine_rows_kernel(const __nv_bfloat16* __restrict__ y, const int64_t* __restrict__ dest,
                                                           const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int T,
                                                           int k, int D) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  for (int i = lane; i < D / 8; i += 32) {
    float acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = 0.f;
    for (int j = 0; j < k; ++j) {
      const uint4 v = reinterpret_cast<const uint4*>(y + dest[(int64_t)t * k + j] * D)[i];
      const float wj = (w != nullptr) ? w[(int64_t)t * k + j] : 1.f;
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(b[q]);
        acc[2 * q] += wj * f.x;
        acc[2 * q + 1] += wj * f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + (int64_t)t * D)[i] = o;
  }
}

// dy[dest[c]] = w[c] * dout[c / k] ; dw[c] = <dout[c / k], y[dest[c]]> ; one warp per copy
__global__ void __launch_bounds__(256) combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                                                          const int64_t* __restrict__ dest, const float* __restrict__ w,
                                                          __nv_bfloat16* __restrict__ dy, float* __restrict__ dw, int64_t ncopies,
                                                          int k, int D) {
  const int lane = threadIdx.x & 31;
  const int64_t c = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (c >= ncopies) return;
  const uint4* g = reinterpret_cast<const uint4*>(dout + (c / k) * D);
  const uint4* yy = reinterpret_cast<const uint4*>(y + dest[c] * D);
  uint4* d = reinterpret_cast<uint4*>(dy + dest[c] * D);
  const float wc = w[c];
  float dot = 0.f;
  for (int i = lane; i < D / 8; i += 32) {
    const uint4 gv = g[i], yv = yy[i];
    const __nv_bfloat162 *gb = reinterpret_cast<const __nv_bfloat162*>(&gv), *yb = reinterpret_cast<const __nv_bfloat162*>(&yv);
    float o[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 gf = __bfloat1622float2(gb[q]), yf = __bfloat1622float2(yb[q]);
      dot += gf.x * yf.x + gf.y * yf.y;
      o[2 * q] = wc * gf.x;
      o[2 * q + 1] = wc * gf.y;
    }
    uint4 ov;
    ov.x = pack_bf16x2(o[0], o[1]); ov.y = pack_bf16x2(o[2], o[3]); ov.z = pack_bf16x2(o[4], o[5]); ov.w = pack_bf16x2(o[6], o[7]);
    d[i] = ov;
  }
  dot = warp_sum(dot);
  if (lane == 0 && dw != nullptr) dw[c] = dot;
}

}  // namespace llmt

using namespace llmt;
#define LLMT_CHECK_LAUNCH() return (cudaGetLastError() == cudaSuccess) ? 0 : -3

extern "C" int llmt_router_topk(const float* logits, const float* bias, float* weights, int64_t* indices, float* counts,
                                float* denom, int T, int E, int k, int score_fn, int renorm, float route_scale, cudaStream_t st) {
  if (T <= 0) return 0;
  if (E > 32 * kMaxEPerLane || k > kMaxTopK || k > E) return -10;
  router_topk_kernel<<<(T + 7) / 8, 256, 0, st>>>(logits, bias, weights, indices, counts, denom, T, E, k, score_fn, renorm, route_scale);
  LLMT_CHECK_LAUNCH();
}
extern "C" int llmt_router_topk_bwd(const float* logits, const float* dweights, const int64_t* indices, const float* denom,
                                    float* dlogits, int T, int E, int k, int score_fn, int renorm, float route_scale, cudaStream_t st) {
  if (T <= 0) return 0;
  if (E > 32 * kMaxEPerLane || k > kMaxTopK) return -10;
  router_topk_bwd_kernel<<<(T + 7) / 8, 256, 0, st>>>(logits, dweights, indices, denom, dlogits, T, E, k, score_fn, renorm, route_scale);
  LLMT_CHECK_LAUNCH();
}
extern "C" int llmt_permute_rows(const void* x, const int64_t* dest, void* rows, int64_t ncopies, int k, int D, cudaStream_t st) {
  if (ncopies <= 0) return 0;
  if (D % 8) return -10;
  permute_rows_kernel<<<(unsigned)((ncopies + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)x, dest, (__nv_bfloat16*)rows, ncopies, k, D);
  LLMT_CHECK_LAUNCH();
}
extern "C" int llmt_combine_rows(const void* y, const int64_t* dest, const float* w, void* out, int T, int k, int D, cudaStream_t st) {
  if (T <= 0) return 0;
  if (D % 8) return -10;
  combine_rows_kernel<<<(T + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)y, dest, w, (__nv_bfloat16*)out, T, k, D);
  LLMT_CHECK_LAUNCH();
}
extern "C" int llmt_combine_bwd(const void* dout, const void* y, const int64_t* dest, const float* w, void* dy, float* dw,
                                int64_t ncopies, int k, int D, cudaStream_t st) {
  if (ncopies <= 0) return 0;
  if (D % 8) return -10;
  combine_bwd_kernel<<<(unsigned)((ncopies + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)y, dest, w,
                                                                   (__nv_bfloat16*)dy, dw, ncopies, k, D);
  LLMT_CHECK_LAUNCH();
}
