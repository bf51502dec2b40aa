// Memory-bound training kernels for sm_100a: RMSNorm (with residual add) fwd/bwd, per-head QK-norm + RoPE
// fwd/bwd, SwiGLU fwd/bwd, row-wise cross-entropy with in-place gradient, fused AdamW on flat shards,
// deterministic squared-norm. bf16 storage, fp32 math, 16-byte vector accesses.
// (reference call sites: llmtuner/models/qwen/ops.py:80-131,503; llmtuner/components/loss.py:35-70;
//  llmtuner/components/optimizer/optimizer.py:62-106; llmtuner/accelerator/collectives.py:290-558)
#include "common.cuh"
#include "kernels.h"

namespace llmt {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < nw) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < nw) ? red[l] : -INFINITY;
  t = warp_max(t);
  return t;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = __bfloat1622float2(b[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ------------------------------------------------------------------------------------------ RMSNorm
// y = (x [+ res]) * rsqrt(mean((x+res)^2) + eps) * w ; optionally writes s = x + res (the new residual stream).
template <int NV>  // each thread owns NV groups of 8 columns: col = (v * kRowThreads + tid) * 8
__global__ void __launch_bounds__(kRowThreads) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                                  const __nv_bfloat16* __restrict__ res,
                                                                  const __nv_bfloat16* __restrict__ w,
                                                                  __nv_bfloat16* __restrict__ y,
                                                                  __nv_bfloat16* __restrict__ sum_out,
                                                                  float* __restrict__ rstd, int T, int D, float eps) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    float v[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (i * kRowThreads + threadIdx.x) * 8;
      if (col < D) {
        load8(x + (int64_t)row * D + col, v[i]);
        if (res != nullptr) {
          float r[8];
          load8(res + (int64_t)row * D + col, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j] + r[j]));
          if (sum_out != nullptr) store8(sum_out + (int64_t)row * D + col, v[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    ss = block_sum(ss, red);
    const float r = rsqrtf(ss / (float)D + eps);
    if (threadIdx.x == 0 && rstd != nullptr) rstd[row] = r;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (i * kRowThreads + threadIdx.x) * 8;
      if (col < D) {
        float wv[8], o[8];
        load8(w + col, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i][j] * r * wv[j];
        store8(y + (int64_t)row * D + col, o);
      }
    }
  }
}

// dx = r * (g - x * r^2 * mean(g * x)) [+ dres], g = dy * w ; dw partial per block = sum_rows dy * x * r.
template <int NV>
__global__ void __launch_bounds__(kRowThreads) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                                  const __nv_bfloat16* __restrict__ x,
                                                                  const __nv_bfloat16* __restrict__ w,
                                                                  const float* __restrict__ rstd,
                                                                  const __nv_bfloat16* __restrict__ dres,
                                                                  __nv_bfloat16* __restrict__ dx,
                                                                  float* __restrict__ dw_partial, int T, int D) {
  __shared__ float red[32];
  float dw[NV][8];
  float wv[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (i * kRowThreads + threadIdx.x) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) { dw[i][j] = 0.f; wv[i][j] = 0.f; }
    if (col < D) load8(w + col, wv[i]);
  }
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    float xv[NV][8], g[NV][8];
    const float r = rstd[row];
    float c = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (i * kRowThreads + threadIdx.x) * 8;
      if (col < D) {
        float d[8];
        load8(x + (int64_t)row * D + col, xv[i]);
        load8(dy + (int64_t)row * D + col, d);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          g[i][j] = d[j] * wv[i][j];
          c += g[i][j] * xv[i][j];
          dw[i][j] += d[j] * xv[i][j] * r;
        }
      }
    }
    c = block_sum(c, red);
    const float k = r * r * r * c / (float)D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (i * kRowThreads + threadIdx.x) * 8;
      if (col < D) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * g[i][j] - xv[i][j] * k;
        if (dres != nullptr) {
          float e[8];
          load8(dres + (int64_t)row * D + col, e);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += e[j];
        }
        store8(dx + (int64_t)row * D + col, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (i * kRowThreads + threadIdx.x) * 8;
    if (col < D) {
      float* p = dw_partial + (int64_t)blockIdx.x * D + col;
#pragma unroll
      for (int j = 0; j < 8; ++j) p[j] = dw[i][j];
    }
  }
}

// out[c] (+)= sum_p partial[p][c]
__global__ void colsum_kernel(const float* __restrict__ partial, float* __restrict__ out_f32,
                              __nv_bfloat16* __restrict__ out_bf16, int P, int D, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += partial[(int64_t)p * D + c];
  if (out_f32 != nullptr) out_f32[c] = accumulate ? out_f32[c] + s : s;
  if (out_bf16 != nullptr) out_bf16[c] = __float2bfloat16_rn(accumulate ? __bfloat162float(out_bf16[c]) + s : s);
}

// ------------------------------------------------------------------------------------------ QK-norm + RoPE
// A group of G = 8 * P lanes per (token, head); HD = 64 * P, so a warp holds 32 / G items (HD 128: two items per warp).
// Lane g of the group owns columns [4g, 4g + 4) of the first half and their rotation partners [HD/2 + 4g, ...): every
// access is an 8-byte vector (bf16 x 4) or a 16-byte vector (cos / sin fp32 x 4). Token rows are `tok_stride` elements
// apart, heads are packed (HD apart), all strides multiples of 4 elements.
// Forward: n = x * rsqrt(mean x^2 + eps) * w (skipped when w == nullptr), then half rotation with cos/sin [T, HD/2]:
//   y1 = n1 cos - n2 sin ; y2 = n2 cos + n1 sin.
__device__ __forceinline__ void ld_bf16x4(const __nv_bfloat16* p, float* f) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void st_bf16x4(__nv_bfloat16* p, const float* f) {
  uint2 v;
  v.x = pack_bf16x2(f[0], f[1]);
  v.y = pack_bf16x2(f[2], f[3]);
  *reinterpret_cast<uint2*>(p) = v;
}
template <int G>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int P>
__global__ void __launch_bounds__(256) qk_norm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ x, int64_t tok_stride,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               const float* __restrict__ cosb,
                                                               const float* __restrict__ sinb,
                                                               __nv_bfloat16* __restrict__ y, int64_t y_tok_stride,
                                                               float* __restrict__ rstd, int T, int H, float eps) {
  constexpr int HD = 64 * P, HALF = HD / 2, G = 8 * P, IPW = 32 / G;
  const int lane = threadIdx.x & 31, g = lane % G;
  const int64_t total = (int64_t)T * H;
  int64_t item = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * IPW + lane / G;
  const bool live = item < total;
  if (!live) item = total - 1;                       // keep the whole warp in the shuffles
  const int t = (int)(item / H), h = (int)(item % H);
  const __nv_bfloat16* px = x + (int64_t)t * tok_stride + (int64_t)h * HD + 4 * g;
  float a[4], b[4];
  ld_bf16x4(px, a);
  ld_bf16x4(px + HALF, b);
  float r = 1.f;
  float wa[4] = {1.f, 1.f, 1.f, 1.f}, wb[4] = {1.f, 1.f, 1.f, 1.f};
  if (w != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) ss += a[j] * a[j] + b[j] * b[j];
    ss = group_sum<G>(ss);
    r = rsqrtf(ss / (float)HD + eps);
    if (g == 0 && live && rstd != nullptr) rstd[item] = r;
    ld_bf16x4(w + 4 * g, wa);
    ld_bf16x4(w + HALF + 4 * g, wb);
  }
  const float4 cs = *reinterpret_cast<const float4*>(cosb + (int64_t)t * HALF + 4 * g);
  const float4 sn = *reinterpret_cast<const float4*>(sinb + (int64_t)t * HALF + 4 * g);
  const float c4[4] = {cs.x, cs.y, cs.z, cs.w}, s4[4] = {sn.x, sn.y, sn.z, sn.w};
  float o1[4], o2[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float n1 = a[j] * r * wa[j], n2 = b[j] * r * wb[j];
    o1[j] = n1 * c4[j] - n2 * s4[j];
    o2[j] = n2 * c4[j] + n1 * s4[j];
  }
  if (live) {
    __nv_bfloat16* py = y + (int64_t)t * y_tok_stride + (int64_t)h * HD + 4 * g;
    st_bf16x4(py, o1);
    st_bf16x4(py + HALF, o2);
  }
}

// Backward: un-rotate dy (dn1 = d1 cos + d2 sin ; dn2 = d2 cos - d1 sin), then RMSNorm backward per head.
// The weight gradient is accumulated per lane over its items, then per block in shared memory and written to
// dw_partial[blockIdx.x][HD].
template <int P>
__global__ void __launch_bounds__(256) qk_norm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dy, int64_t dy_tok_stride,
                                                               const __nv_bfloat16* __restrict__ x, int64_t tok_stride,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               const float* __restrict__ cosb,
                                                               const float* __restrict__ sinb,
                                                               const float* __restrict__ rstd,
                                                               __nv_bfloat16* __restrict__ dx, int64_t dx_tok_stride,
                                                               float* __restrict__ dw_partial, int T, int H) {
  constexpr int HD = 64 * P, HALF = HD / 2, G = 8 * P, IPW = 32 / G;
  // weight-gradient partials of the block's 256 / G thread groups, summed in a fixed order at the end (an atomic add into
  // one row would make the last bit depend on the order in which the groups arrive)
  constexpr int kGroups = 256 / G;
  __shared__ float sparts[kGroups * HD];
  const int lane = threadIdx.x & 31, g = lane % G;
  const int wpb = blockDim.x >> 5;
  const int64_t total = (int64_t)T * H;
  float dwa[4] = {0.f, 0.f, 0.f, 0.f}, dwb[4] = {0.f, 0.f, 0.f, 0.f};
  float wa[4] = {1.f, 1.f, 1.f, 1.f}, wb[4] = {1.f, 1.f, 1.f, 1.f};
  if (w != nullptr) {
    ld_bf16x4(w + 4 * g, wa);
    ld_bf16x4(w + HALF + 4 * g, wb);
  }
  // every warp runs the same number of rounds so that the group shuffles stay converged
  const int64_t warp_items = (int64_t)gridDim.x * wpb * IPW;
  const int64_t rounds = (total + warp_items - 1) / warp_items;
  for (int64_t rd = 0; rd < rounds; ++rd) {
    int64_t item = rd * warp_items + ((int64_t)blockIdx.x * wpb + (threadIdx.x >> 5)) * IPW + lane / G;
    const bool live = item < total;
    if (!live) item = total - 1;
    const int t = (int)(item / H), h = (int)(item % H);
    const int64_t off = (int64_t)h * HD + 4 * g;
    float d1[4], d2[4], xa[4] = {0.f, 0.f, 0.f, 0.f}, xb[4] = {0.f, 0.f, 0.f, 0.f};
    ld_bf16x4(dy + (int64_t)t * dy_tok_stride + off, d1);
    ld_bf16x4(dy + (int64_t)t * dy_tok_stride + off + HALF, d2);
    const float4 cs = *reinterpret_cast<const float4*>(cosb + (int64_t)t * HALF + 4 * g);
    const float4 sn = *reinterpret_cast<const float4*>(sinb + (int64_t)t * HALF + 4 * g);
    const float c4[4] = {cs.x, cs.y, cs.z, cs.w}, s4[4] = {sn.x, sn.y, sn.z, sn.w};
    const float r = (w != nullptr) ? rstd[item] : 1.f;
    if (w != nullptr) {
      ld_bf16x4(x + (int64_t)t * tok_stride + off, xa);
      ld_bf16x4(x + (int64_t)t * tok_stride + off + HALF, xb);
    }
    float ga[4], gb[4], c_acc = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float dn1 = d1[j] * c4[j] + d2[j] * s4[j];
      float dn2 = d2[j] * c4[j] - d1[j] * s4[j];
      if (w != nullptr) {
        if (live) {
          dwa[j] += dn1 * xa[j] * r;
          dwb[j] += dn2 * xb[j] * r;
        }
        dn1 *= wa[j];
        dn2 *= wb[j];
        c_acc += dn1 * xa[j] + dn2 * xb[j];
      }
      ga[j] = dn1;
      gb[j] = dn2;
    }
    float k = 0.f;
    if (w != nullptr) {
      c_acc = group_sum<G>(c_acc);
      k = r * r * r * c_acc / (float)HD;
    }
    float o1[4], o2[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o1[j] = (w != nullptr) ? r * ga[j] - xa[j] * k : ga[j];
      o2[j] = (w != nullptr) ? r * gb[j] - xb[j] * k : gb[j];
    }
    if (live) {
      st_bf16x4(dx + (int64_t)t * dx_tok_stride + off, o1);
      st_bf16x4(dx + (int64_t)t * dx_tok_stride + off + HALF, o2);
    }
  }
  if (w != nullptr && dw_partial != nullptr) {
    float* mine = sparts + (threadIdx.x / G) * HD;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mine[4 * g + j] = dwa[j];
      mine[HALF + 4 * g + j] = dwb[j];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < HD; i += blockDim.x) {
      float acc = 0.f;
#pragma unroll 4
      for (int c = 0; c < kGroups; ++c) acc += sparts[c * HD + i];
      dw_partial[(int64_t)blockIdx.x * HD + i] = acc;
    }
  }
}

// ------------------------------------------------------------------------------------------ attention backward by rows
// The two elementwise steps of the attention backward that rebuilds probabilities per block of query rows (head sizes with
// a forward kernel only): S [rows, C] fp32 from a batched product -> P = exp(S * scale - lse[row]) in bf16 with the causal
// limit applied, and dS = (dP - delta[row]) * P in bf16. One read of the fp32 block and one bf16 write each, where the
// same algebra as tensor expressions takes eight passes. Row r of the block is query (r % n) of the chunk; it sees columns
// [0, (r % n) + diag + 1).
__global__ void attn_rows_probs_kernel(const float* __restrict__ s, const float* __restrict__ lse, __nv_bfloat16* __restrict__ p,
                                       int64_t rows, int C, int n, int diag, float scale_log2, int causal) {
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float l = lse[row];
    const float l2 = isinf(l) ? 0.f : l * 1.4426950408889634f;    // a row that sees no key: every column is beyond its limit
    const int i = (int)(row % n);
    const int lim = causal ? min(C, i + diag + 1) : C;
    const float* sr = s + row * (int64_t)C;
    __nv_bfloat16* pr = p + row * (int64_t)C;
    for (int c = threadIdx.x; c < C; c += blockDim.x)
      pr[c] = __float2bfloat16_rn(c < lim ? exp2f(sr[c] * scale_log2 - l2) : 0.f);
  }
}
__global__ void attn_rows_ds_kernel(const float* __restrict__ dp, const __nv_bfloat16* __restrict__ p, const float* __restrict__ delta,
                                    __nv_bfloat16* __restrict__ ds, int64_t rows, int C) {
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float dl = delta[row];
    const float* dr = dp + row * (int64_t)C;
    const __nv_bfloat16* pr = p + row * (int64_t)C;
    __nv_bfloat16* or_ = ds + row * (int64_t)C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) or_[c] = __float2bfloat16_rn((dr[c] - dl) * __bfloat162float(pr[c]));
  }
}

// ------------------------------------------------------------------------------------------ SwiGLU
// Rows of `gate` and `up` may be strided (views into one [T, 2F] buffer); out/dgate/dup likewise.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                  __nv_bfloat16* __restrict__ out, int64_t T, int F, int64_t ld_in, int64_t ld_out,
                                  const int* __restrict__ row_limit) {
  // row_limit (optional, device memory): rows at or beyond *row_limit of a statically sized buffer hold nothing
  if (row_limit != nullptr && *row_limit < T) T = *row_limit;
  const int64_t nvec = T * (F / 8);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / (F / 8);
    const int col = (int)(i % (F / 8)) * 8;
    float g[8], u[8], o[8];
    load8(gate + row * ld_in + col, g);
    load8(up + row * ld_in + col, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    store8(out + row * ld_out + col, o);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gate,
                                  const __nv_bfloat16* __restrict__ up, __nv_bfloat16* __restrict__ dgate,
                                  __nv_bfloat16* __restrict__ dup, int64_t T, int F, int64_t ld_in, int64_t ld_dout,
                                  int64_t ld_dg, const int* __restrict__ row_limit) {
  if (row_limit != nullptr && *row_limit < T) T = *row_limit;
  const int64_t nvec = T * (F / 8);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / (F / 8);
    const int col = (int)(i % (F / 8)) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gate + row * ld_in + col, g);
    load8(up + row * ld_in + col, u);
    load8(dout + row * ld_dout + col, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * s;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (s + silu * (1.f - s));
    }
    store8(dgate + row * ld_dg + col, dg);
    store8(dup + row * ld_dg + col, du);
  }
}

// ------------------------------------------------------------------------------------------ cross-entropy
// One CTA per row of bf16 logits [rows, V] (row stride ld). Pass 1: online max / sum-exp. Pass 2: overwrite the
// logits with d(loss_sum)/d(logit) * grad_scale = (softmax - onehot) * grad_scale. Rows whose label is
// ignore_index get zero gradient and no loss. Row losses go to `row_loss` (fp32); the caller sums them
// (deterministic), lse goes to `row_lse` when given.
__global__ void __launch_bounds__(512) ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ labels,
                                                         float* __restrict__ row_loss, float* __restrict__ row_lse,
                                                         int V, int64_t ld, const float* __restrict__ grad_scale_ptr,
                                                         float grad_scale, int ignore_index, int write_grad) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  __nv_bfloat16* p = logits + row * ld;
  const int64_t label = labels[row];
  const bool valid = (label != ignore_index) && label >= 0 && label < V;
  float m = -INFINITY, s = 0.f;
  const int nvec = V / 8;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    load8(p + i * 8, f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {
    const float f = __bfloat162float(p[i]);
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  const float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum(s, red);
  const float lse = gm + logf(gs);
  if (threadIdx.x == 0) {
    if (row_lse != nullptr) row_lse[row] = lse;
    row_loss[row] = valid ? (lse - __bfloat162float(p[label])) : 0.f;
  }
  if (!write_grad) return;
  __syncthreads();  // the label logit was read above before anyone overwrites it
  const float gsc = valid ? grad_scale * (grad_scale_ptr != nullptr ? *grad_scale_ptr : 1.f) : 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    load8(p + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float g = __expf(f[j] - lse);
      if (i * 8 + j == label) g -= 1.f;
      f[j] = g * gsc;
    }
    store8(p + i * 8, f);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {
    float g = __expf(__bfloat162float(p[i]) - lse);
    if (i == label) g -= 1.f;
    p[i] = __float2bfloat16_rn(g * gsc);
  }
}

// ------------------------------------------------------------------------------------------ AdamW on a flat shard
// p32: fp32 master, m/v: fp32 moments, g: bf16 or fp32 gradient, p16: bf16 working copy (optional).
// clip_coef (device, optional) multiplies the gradient: it is min(1, max_norm / (norm + 1e-6)) computed on the device.
template <typename GT>
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p32, __nv_bfloat16* __restrict__ p16, const GT* __restrict__ g,
                                                    float* __restrict__ m, float* __restrict__ v, int64_t n, float lr, float b1,
                                                    float b2, float eps, float wd, float bc1, float bc2,
                                                    const float* __restrict__ clip_coef, float grad_scale, int decoupled) {
  const float gs = grad_scale * (clip_coef != nullptr ? *clip_coef : 1.f);
  if (!isfinite(gs)) return;  // non-finite gradient norm: leave parameters and moments untouched
  const float inv_bc1 = 1.f / bc1, inv_bc2 = 1.f / bc2, decay = decoupled ? (1.f - lr * wd) : 1.f;
  auto update = [&](float& p, float& mi, float& vi, float gr) {
    gr *= gs;
    if (!decoupled) gr += wd * p;
    mi = b1 * mi + (1.f - b1) * gr;
    vi = b2 * vi + (1.f - b2) * gr * gr;
    p = p * decay - lr * (mi * inv_bc1) / (sqrtf(vi * inv_bc2) + eps);
  };
  // 4 elements per thread per iteration, 16-byte accesses when every base pointer allows it
  const bool vec = ((reinterpret_cast<uintptr_t>(p32) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(g) & (sizeof(GT) * 4 - 1)) == 0 &&
                   (p16 == nullptr || (reinterpret_cast<uintptr_t>(p16) & 7) == 0);
  const int64_t n4 = vec ? n / 4 : 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(p32)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float gr[4];
    if constexpr (sizeof(GT) == 2) {
      const uint2 u = reinterpret_cast<const uint2*>(g)[i];
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
      gr[0] = a.x; gr[1] = a.y; gr[2] = b.x; gr[3] = b.y;
    } else {
      const float4 u = reinterpret_cast<const float4*>(g)[i];
      gr[0] = u.x; gr[1] = u.y; gr[2] = u.z; gr[3] = u.w;
    }
    update(p.x, mm.x, vv.x, gr[0]);
    update(p.y, mm.y, vv.y, gr[1]);
    update(p.z, mm.z, vv.z, gr[2]);
    update(p.w, mm.w, vv.w, gr[3]);
    reinterpret_cast<float4*>(p32)[i] = p;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (p16 != nullptr) {
      uint2 o;
      o.x = pack_bf16x2(p.x, p.y);
      o.y = pack_bf16x2(p.z, p.w);
      reinterpret_cast<uint2*>(p16)[i] = o;
    }
  }
  for (int64_t i = n4 * 4 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float gr;
    if constexpr (sizeof(GT) == 2) gr = __bfloat162float(g[i]);
    else gr = g[i];
    float p = p32[i], mi = m[i], vi = v[i];
    update(p, mi, vi, gr);
    p32[i] = p; m[i] = mi; v[i] = vi;
    if (p16 != nullptr) p16[i] = __float2bfloat16_rn(p);
  }
}

// ------------------------------------------------------------------------------------------ squared norm
// Deterministic two-stage sum of squares: stage 1 writes one partial per block into `scratch`, stage 2 (one
// block) adds them in index order into out[0] (accumulating when `accumulate`).
template <typename T>
__global__ void __launch_bounds__(256) sqnorm_partial_kernel(const T* __restrict__ x, int64_t n, float* __restrict__ scratch) {
  __shared__ float red[32];
  float s = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float f;
    if constexpr (sizeof(T) == 2) f = __bfloat162float(x[i]);
    else f = x[i];
    s += f * f;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) scratch[blockIdx.x] = s;
}
__global__ void __launch_bounds__(256) sqnorm_final_kernel(const float* __restrict__ scratch, int nparts,
                                                           float* __restrict__ out, int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += scratch[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}
// clip_coef[0] = min(1, max_norm / (sqrt(total_sq[0]) + 1e-6)); norm_out[0] = sqrt(total_sq[0]); finite[0] = isfinite
__global__ void clip_coef_kernel(const float* __restrict__ total_sq, float max_norm, float* __restrict__ clip_coef,
                                 float* __restrict__ norm_out, int* __restrict__ finite) {
  const float n = sqrtf(total_sq[0]);
  norm_out[0] = n;
  clip_coef[0] = isfinite(n) ? fminf(1.f, max_norm / (n + 1e-6f)) : NAN;
  if (finite != nullptr) finite[0] = isfinite(n) ? 1 : 0;
}

int sm_count();   // gemm.cu: SMs of the current device

static inline int grid_for(int64_t n, int threads, int per_sm = 8) {
  int64_t b = (n + threads - 1) / threads;
  const int64_t cap = (int64_t)sm_count() * per_sm;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace llmt

using namespace llmt;

#define LLMT_CHECK_LAUNCH() return (cudaGetLastError() == cudaSuccess) ? 0 : -3

extern "C" int llmt_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* sum_out, float* rstd, int T,
                                int D, float eps, cudaStream_t st) {
  if (T <= 0) return 0;
  if (D % 8 || D > 8 * kRowThreads * 4) return -10;
  const int nv = (D + 8 * kRowThreads - 1) / (8 * kRowThreads);
  const int grid = T < sm_count() * 8 ? T : sm_count() * 8;
  auto X = (const __nv_bfloat16*)x; auto R = (const __nv_bfloat16*)res; auto W = (const __nv_bfloat16*)w;
  auto Y = (__nv_bfloat16*)y; auto S = (__nv_bfloat16*)sum_out;
  if (nv == 1) rmsnorm_fwd_kernel<1><<<grid, kRowThreads, 0, st>>>(X, R, W, Y, S, rstd, T, D, eps);
  else if (nv == 2) rmsnorm_fwd_kernel<2><<<grid, kRowThreads, 0, st>>>(X, R, W, Y, S, rstd, T, D, eps);
  else rmsnorm_fwd_kernel<4><<<grid, kRowThreads, 0, st>>>(X, R, W, Y, S, rstd, T, D, eps);
  LLMT_CHECK_LAUNCH();
}

// dw_partial: fp32 scratch of llmt_rmsnorm_bwd_partials(T) * D floats.
// Two row blocks per SM, at most 296 (the allocation-free entry point in noalloc.cu sizes its scratch for that bound).
extern "C" int llmt_rmsnorm_bwd_partials(int T) {
  const int cap = sm_count() * 2 < 296 ? sm_count() * 2 : 296;
  return T < cap ? (T < 1 ? 1 : T) : cap;
}
extern "C" int llmt_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                                float* dw_partial, float* dw_f32, void* dw_bf16, int accumulate, int T, int D,
                                cudaStream_t st) {
  if (T <= 0) return 0;
  if (D % 8 || D > 8 * kRowThreads * 4) return -10;
  const int nv = (D + 8 * kRowThreads - 1) / (8 * kRowThreads);
  const int grid = llmt_rmsnorm_bwd_partials(T);
  auto DY = (const __nv_bfloat16*)dy; auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w;
  auto DR = (const __nv_bfloat16*)dres; auto DX = (__nv_bfloat16*)dx;
  if (nv == 1) rmsnorm_bwd_kernel<1><<<grid, kRowThreads, 0, st>>>(DY, X, W, rstd, DR, DX, dw_partial, T, D);
  else if (nv == 2) rmsnorm_bwd_kernel<2><<<grid, kRowThreads, 0, st>>>(DY, X, W, rstd, DR, DX, dw_partial, T, D);
  else rmsnorm_bwd_kernel<4><<<grid, kRowThreads, 0, st>>>(DY, X, W, rstd, DR, DX, dw_partial, T, D);
  colsum_kernel<<<(D + 255) / 256, 256, 0, st>>>(dw_partial, dw_f32, (__nv_bfloat16*)dw_bf16, grid, D, accumulate);
  LLMT_CHECK_LAUNCH();
}

extern "C" int llmt_qk_norm_rope_fwd(const void* x, int64_t tok_stride, const void* w, const float* cosb, const float* sinb,
                                     void* y, int64_t y_tok_stride, float* rstd, int T, int H, int HD, float eps,
                                     cudaStream_t st) {
  if (T <= 0 || H <= 0) return 0;
  if ((tok_stride & 3) || (y_tok_stride & 3) || (reinterpret_cast<uintptr_t>(x) & 7) || (reinterpret_cast<uintptr_t>(y) & 7)) return -10;
  const int64_t items = (int64_t)T * H;
  const int ipw = HD == 64 ? 4 : (HD == 128 ? 2 : 1);          // items per warp
  const int grid = (int)((items + 8 * ipw - 1) / (8 * ipw));
  auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w; auto Y = (__nv_bfloat16*)y;
  if (HD == 64) qk_norm_rope_fwd_kernel<1><<<grid, 256, 0, st>>>(X, tok_stride, W, cosb, sinb, Y, y_tok_stride, rstd, T, H, eps);
  else if (HD == 128) qk_norm_rope_fwd_kernel<2><<<grid, 256, 0, st>>>(X, tok_stride, W, cosb, sinb, Y, y_tok_stride, rstd, T, H, eps);
  else if (HD == 256) qk_norm_rope_fwd_kernel<4><<<grid, 256, 0, st>>>(X, tok_stride, W, cosb, sinb, Y, y_tok_stride, rstd, T, H, eps);
  else return -10;
  LLMT_CHECK_LAUNCH();
}

extern "C" int llmt_qk_norm_rope_bwd_partials(int T, int H) {
  const int64_t items = (int64_t)T * H;
  const int64_t b = (items + 7) / 8;
  const int64_t cap = (int64_t)sm_count() * 4;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}
extern "C" int llmt_qk_norm_rope_bwd(const void* dy, int64_t dy_tok_stride, const void* x, int64_t tok_stride, const void* w,
                                     const float* cosb, const float* sinb, const float* rstd, void* dx,
                                     int64_t dx_tok_stride, float* dw_partial, float* dw_f32, void* dw_bf16,
                                     int accumulate, int T, int H, int HD, cudaStream_t st) {
  if (T <= 0 || H <= 0) return 0;
  if ((tok_stride & 3) || (dy_tok_stride & 3) || (dx_tok_stride & 3) || (reinterpret_cast<uintptr_t>(x) & 7) ||
      (reinterpret_cast<uintptr_t>(dy) & 7) || (reinterpret_cast<uintptr_t>(dx) & 7))
    return -10;
  const int grid = llmt_qk_norm_rope_bwd_partials(T, H);
  auto DY = (const __nv_bfloat16*)dy; auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w;
  auto DX = (__nv_bfloat16*)dx;
  if (HD == 64) qk_norm_rope_bwd_kernel<1><<<grid, 256, 0, st>>>(DY, dy_tok_stride, X, tok_stride, W, cosb, sinb, rstd, DX, dx_tok_stride, dw_partial, T, H);
  else if (HD == 128) qk_norm_rope_bwd_kernel<2><<<grid, 256, 0, st>>>(DY, dy_tok_stride, X, tok_stride, W, cosb, sinb, rstd, DX, dx_tok_stride, dw_partial, T, H);
  else if (HD == 256) qk_norm_rope_bwd_kernel<4><<<grid, 256, 0, st>>>(DY, dy_tok_stride, X, tok_stride, W, cosb, sinb, rstd, DX, dx_tok_stride, dw_partial, T, H);
  else return -10;
  if (w != nullptr && dw_partial != nullptr)
    colsum_kernel<<<(HD + 255) / 256, 256, 0, st>>>(dw_partial, dw_f32, (__nv_bfloat16*)dw_bf16, grid, HD, accumulate);
  LLMT_CHECK_LAUNCH();
}

extern "C" int llmt_attn_rows_probs(const float* s, const float* lse, void* p, int64_t rows, int C, int n, int diag, float scale,
                                    int causal, cudaStream_t st) {
  if (rows <= 0 || C <= 0) return 0;
  if (n <= 0) return -10;
  const int64_t cap = (int64_t)sm_count() * 8;
  attn_rows_probs_kernel<<<(int)(rows < cap ? rows : cap), 256, 0, st>>>(s, lse, (__nv_bfloat16*)p, rows, C, n, diag,
                                                                          scale * 1.4426950408889634f, causal);
  LLMT_CHECK_LAUNCH();
}
extern "C" int llmt_attn_rows_ds(const float* dp, const void* p, const float* delta, void* ds, int64_t rows, int C, cudaStream_t st) {
  if (rows <= 0 || C <= 0) return 0;
  const int64_t cap = (int64_t)sm_count() * 8;
  attn_rows_ds_kernel<<<(int)(rows < cap ? rows : cap), 256, 0, st>>>(dp, (const __nv_bfloat16*)p, delta, (__nv_bfloat16*)ds, rows, C);
  LLMT_CHECK_LAUNCH();
}

extern "C" int llmt_swiglu_fwd(const void* gate, const void* up, void* out, int64_t T, int F, int64_t ld_in, int64_t ld_out,
                               const int* row_limit, cudaStream_t st) {
  if (T <= 0) return 0;
  if (F % 8 || ld_in % 8 || ld_out % 8) return -10;
  swiglu_fwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, st>>>((const __nv_bfloat16*)gate, (const __nv_bfloat16*)up,
                                                                 (__nv_bfloat16*)out, T, F, ld_in, ld_out, row_limit);
  LLMT_CHECK_LAUNCH();
}
extern "C" int llmt_swiglu_bwd(const void* dout, const void* gate, const void* up, void* dgate, void* dup, int64_t T, int F,
                               int64_t ld_in, int64_t ld_dout, int64_t ld_dg, const int* row_limit, cudaStream_t st) {
  if (T <= 0) return 0;
  if (F % 8 || ld_in % 8 || ld_dout % 8 || ld_dg % 8) return -10;
  swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)gate,
                                                                 (const __nv_bfloat16*)up, (__nv_bfloat16*)dgate,
                                                                 (__nv_bfloat16*)dup, T, F, ld_in, ld_dout, ld_dg, row_limit);
  LLMT_CHECK_LAUNCH();
}

extern "C" int llmt_ce_fwd_bwd(void* logits, const int64_t* labels, float* row_loss, float* row_lse, int rows, int V,
                               int64_t ld, const float* grad_scale_ptr, float grad_scale, int ignore_index, int write_grad,
                               cudaStream_t st) {
  if (rows <= 0) return 0;
  if (ld % 8) return -10;
  ce_fwd_bwd_kernel<<<rows, 512, 0, st>>>((__nv_bfloat16*)logits, labels, row_loss, row_lse, V, ld, grad_scale_ptr,
                                          grad_scale, ignore_index, write_grad);
  LLMT_CHECK_LAUNCH();
}

extern "C" int llmt_adamw(float* p32, void* p16, const void* g, int g_is_bf16, float* m, float* v, int64_t n, float lr,
                          float b1, float b2, float eps, float wd, int step, const float* clip_coef, float grad_scale,
                          int decoupled, cudaStream_t st) {
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  const int grid = grid_for((n + 3) / 4, 256, 16);
  if (g_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p32, (__nv_bfloat16*)p16, (const __nv_bfloat16*)g, m, v, n, lr, b1, b2,
                                                       eps, wd, bc1, bc2, clip_coef, grad_scale, decoupled);
  else
    adamw_kernel<float><<<grid, 256, 0, st>>>(p32, (__nv_bfloat16*)p16, (const float*)g, m, v, n, lr, b1, b2, eps, wd, bc1,
                                               bc2, clip_coef, grad_scale, decoupled);
  LLMT_CHECK_LAUNCH();
}

// scratch must hold llmt_sqnorm_scratch_floats() floats.
extern "C" int llmt_sqnorm_scratch_floats() { return sm_count() * 8; }
extern "C" int llmt_sqnorm(const void* x, int is_bf16, int64_t n, float* scratch, float* out, int accumulate,
                           cudaStream_t st) {
  if (n <= 0) {
    if (!accumulate) cudaMemsetAsync(out, 0, sizeof(float), st);
    return 0;
  }
  const int grid = grid_for(n, 256);
  if (is_bf16) sqnorm_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, n, scratch);
  else sqnorm_partial_kernel<float><<<grid, 256, 0, st>>>((const float*)x, n, scratch);
  sqnorm_final_kernel<<<1, 256, 0, st>>>(scratch, grid, out, accumulate);
  LLMT_CHECK_LAUNCH();
}
extern "C" int llmt_clip_coef(const float* total_sq, float max_norm, float* clip_coef, float* norm_out, int* finite,
                              cudaStream_t st) {
  clip_coef_kernel<<<1, 1, 0, st>>>(total_sq, max_norm, clip_coef, norm_out, finite);
  LLMT_CHECK_LAUNCH();
}
