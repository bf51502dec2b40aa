// Vocabulary-parallel cross-entropy and embedding over NVLink peer memory
// (reference: llmtuner/components/loss.py:92-238, three all-reduces per loss chunk; llmtuner/parallel/vocab_parallel/
//  vocab_parallel.py:16-96, all-gather of ids + masked lookup + all-reduce).
//
//   ce_vocab_parallel   one CTA per token row of this rank's logits shard [rows, V/R]. The CTA reduces its shard to
//                       (max, sum of exponentials, target logit), stores the triple into EVERY rank's statistics table
//                       with plain peer stores followed by a release store of the row's epoch flag, polls (bounded) its
//                       own table until all R triples of the row have arrived, combines them and overwrites the shard
//                       with d(loss)/d(logits) = softmax - onehot. One kernel, one exchange of three scalars per token,
//                       no collective library call; backward needs no communication at all.
//   vp_embed_scatter    every rank walks all T token ids of the tensor-parallel group; a token whose id falls into this
//                       rank's rows of the table is copied straight into the token owner's output shard (peer stores).
//                       Exactly one rank owns each id, so the sequence-sharded embedding output needs no reduction.
// A CTA publishes its own triple before it waits for the others, and rows are taken in the same order on every rank, so
// the waits cannot form a cycle; they are bounded and report through the status word like every wait of this library.
#include "comm.cuh"
#include "kernels.h"

namespace llmt {

struct VpPeers {
  void* p[kMaxPeers];
};

// Block-wide reductions: every thread receives the result (through red[0]).
__device__ __forceinline__ float vp_block_max(float v, float* red) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : -INFINITY;
    r = warp_max(r);
    if (threadIdx.x == 0) red[0] = r;
  }
  __syncthreads();
  const float out = red[0];
  __syncthreads();
  return out;
}
__device__ __forceinline__ float vp_block_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0) red[0] = r;
  }
  __syncthreads();
  const float out = red[0];
  __syncthreads();
  return out;
}

__device__ __forceinline__ void vp_load8(const __nv_bfloat16* p, float* f) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = __bfloat1622float2(h[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ void vp_store8(__nv_bfloat16* p, const float* f) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]); v.y = pack_bf16x2(f[2], f[3]); v.z = pack_bf16x2(f[4], f[5]); v.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = v;
}

// stats table of a rank: float4 [R sources][cap rows] = {max, sumexp (relative to max), target logit, unused};
// flags table: uint32 [R sources][cap rows], holds the epoch of the last complete triple.
__global__ void __launch_bounds__(512) ce_vocab_parallel_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ labels,
                                                                float* __restrict__ row_loss, int rows, int Vr, int64_t ld,
                                                                int64_t vocab_start, int R, int me, VpPeers stats, VpPeers flags,
                                                                int cap, uint32_t epoch, float grad_scale, int ignore_index,
                                                                int write_grad, int* status) {
  __shared__ float red[32];
  __shared__ float4 got[kMaxPeers];
  __shared__ int ok;
  const int row = blockIdx.x;
  __nv_bfloat16* p = logits + (int64_t)row * ld;
  const int64_t label = labels[row];
  const bool valid = label != ignore_index && label >= 0;
  const int64_t local = label - vocab_start;
  const bool owned = valid && local >= 0 && local < Vr;
  float m = -INFINITY, s = 0.f;
  const int nvec = Vr / 8;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    vp_load8(p + i * 8, f);
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
  for (int i = nvec * 8 + threadIdx.x; i < Vr; i += blockDim.x) {
    const float f = __bfloat162float(p[i]);
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  const float lmax = vp_block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - lmax);
  const float lsum = vp_block_sum(s, red);
  const float tl = owned ? __bfloat162float(p[local]) : 0.f;
  // publish this rank's triple to every rank (itself included), then the row's flag
  if (threadIdx.x < R) {
    float4* dst = reinterpret_cast<float4*>(stats.p[threadIdx.x]) + (size_t)me * cap + row;
    *dst = make_float4(lmax, lsum, tl, 0.f);
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + (size_t)me * cap + row, epoch);
  }
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < R) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(flags.p[me]) + (size_t)threadIdx.x * cap + row;
    if (!flag_wait_bounded(f, epoch, status, 8500 + threadIdx.x)) ok = 0;
    else got[threadIdx.x] = __ldcv(reinterpret_cast<const float4*>(stats.p[me]) + (size_t)threadIdx.x * cap + row);
  }
  __syncthreads();
  if (!ok) return;
  float gmax = -INFINITY;
  for (int r = 0; r < R; ++r) gmax = fmaxf(gmax, got[r].x);
  float gsum = 0.f, gt = 0.f;
  for (int r = 0; r < R; ++r) {
    gsum += (got[r].x == -INFINITY) ? 0.f : got[r].y * __expf(got[r].x - gmax);
    gt += got[r].z;
  }
  const float lse = gmax + logf(gsum);
  if (threadIdx.x == 0) row_loss[row] = valid ? (lse - gt) : 0.f;
  if (!write_grad) return;
  const float gsc = valid ? grad_scale : 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    vp_load8(p + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float g = __expf(f[j] - lse);
      if (owned && i * 8 + j == local) g -= 1.f;
      f[j] = g * gsc;
    }
    vp_store8(p + i * 8, f);
  }
  for (int i = nvec * 8 + threadIdx.x; i < Vr; i += blockDim.x) {
    float g = __expf(__bfloat162float(p[i]) - lse);
    if (owned && i == local) g -= 1.f;
    p[i] = __float2bfloat16_rn(g * gsc);
  }
}

// One warp per token of the whole tensor-parallel group: ids [T] (all ranks hold the same gathered ids), table shard
// `w` [.., D] holds vocabulary rows [vstart, vend). Token t belongs to rank t / chunk, row t % chunk of that rank's
// output shard `out.p[rank]` ([chunk, D] bf16 in symmetric memory).
__global__ void __launch_bounds__(256) vp_embed_scatter_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                                                               int64_t vstart, int64_t vend, VpPeers out, int T, int chunk, int D) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int64_t id = ids[t];
  if (id < vstart || id >= vend) return;
  const uint4* src = reinterpret_cast<const uint4*>(w + (id - vstart) * D);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out.p[t / chunk]) + (t % chunk) * (int64_t)D);
  for (int i = lane; i < D / 8; i += 32) dst[i] = src[i];
}

}  // namespace llmt

using namespace llmt;

#define VP_CHECK_LAUNCH() return cudaGetLastError() == cudaSuccess ? 0 : -3

extern "C" int llmt_ce_vocab_parallel(void* logits, const int64_t* labels, float* row_loss, int rows, int Vr, int64_t ld,
                                      int64_t vocab_start, int R, int me, void* const* stats, void* const* flags, int cap,
                                      uint32_t epoch, float grad_scale, int ignore_index, int write_grad, int* status,
                                      cudaStream_t st) {
  if (rows <= 0) return 0;
  if ((ld % 8) || R < 1 || R > kMaxPeers || rows > cap || me < 0 || me >= R) return -10;
  VpPeers s{}, f{};
  for (int i = 0; i < R; ++i) { s.p[i] = stats[i]; f.p[i] = flags[i]; }
  ce_vocab_parallel_kernel<<<rows, 512, 0, st>>>((__nv_bfloat16*)logits, labels, row_loss, rows, Vr, ld, vocab_start, R, me, s, f, cap,
                                                 epoch, grad_scale, ignore_index, write_grad, status);
  VP_CHECK_LAUNCH();
}

extern "C" int llmt_vp_embed_scatter(const int64_t* ids, const void* w, int64_t vstart, int64_t vend, void* const* out, int R, int T,
                                     int chunk, int D, cudaStream_t st) {
  if (T <= 0) return 0;
  if ((D % 8) || R < 1 || R > kMaxPeers || chunk <= 0 || (int64_t)chunk * R < T) return -10;
  VpPeers o{};
  for (int i = 0; i < R; ++i) o.p[i] = out[i];
  vp_embed_scatter_kernel<<<(T + 7) / 8, 256, 0, st>>>(ids, (const __nv_bfloat16*)w, vstart, vend, o, T, chunk, D);
  VP_CHECK_LAUNCH();
}
