// Helpers shared by the attention kernels (attention.cu: forward and the two-kernel backward; attention_bwd.cu: the
// single-kernel backward): exp2, shared-memory descriptor offsets of the swizzled tiles, swizzled row stores and the
// [T, H, HD] tensor maps.
#pragma once
#include <type_traits>
#include "common.cuh"
#include "kernels.h"

namespace llmt {

constexpr int kAttnThreads = 192;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 16-column slice `ks` of a K-major tile stored as 64-column halves of [128 rows][128 B].
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int ks) {
  return umma_desc_sw128(base + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);
}
// 16-row slice `ks` of the same physical tile read as an MN-major operand (rows = reduction index).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int ks) {
  return umma_desc_sw128(base + ks * 2048, 16384, 1024);
}
// Store 32 consecutive bf16 (packed in 16 words) of row `row`, columns [col0, col0+32) into a swizzled K-major tile.
__device__ __forceinline__ void store_row32_swz(uint8_t* tile, int row, int col0, const uint32_t* w) {
  uint8_t* base = tile + (col0 >> 6) * 16384 + row * 128;
  const int chunk0 = (col0 & 63) >> 3;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 v = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
    *reinterpret_cast<uint4*>(base + (((chunk0 + c) ^ (row & 7)) << 4)) = v;
  }
}

template <int HD>
struct AttnSmem {
  static constexpr int kTile = 128 * HD * 2;   // Q / K / V / dO tile, 128 rows
  static constexpr int kP = 128 * 128 * 2;     // P / dS tile
};

// 16-column slice `ks` of a K-major tile with `rows` rows stored as 64-column halves of [rows][128 B].
__device__ __forceinline__ uint64_t desc_kmajor_rows(uint32_t base, int ks, int rows) {
  return umma_desc_sw128(base + (ks >> 2) * (rows * 128) + (ks & 3) * 32, 16, 1024);
}
// 16-row slice `ks` of a tile with `rows` rows read as an MN-major operand (64-column blocks `rows * 128` B apart).
__device__ __forceinline__ uint64_t desc_mnmajor_rows(uint32_t base, int ks, int rows) {
  return umma_desc_sw128(base + ks * 2048, rows * 128, 1024);
}

// offset (in 16-byte units) of 16-column slice `ks` of a K-major tile with `rows` rows / of 16-row slice `ks` read MN-major
__host__ __device__ constexpr uint32_t koff(int ks, int rows) { return (uint32_t)(((ks >> 2) * (rows * 128) + (ks & 3) * 32) >> 4); }
__host__ __device__ constexpr uint32_t mnoff(int ks) { return (uint32_t)((ks * 2048) >> 4); }

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h).
static __global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, int64_t o_stride, const __nv_bfloat16* __restrict__ d_o,
                                         int64_t do_stride, float* __restrict__ delta, int T, int H, int HD) {
  const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (int64_t)T * H) return;
  const int t = (int)(item / H), h = (int)(item % H), lane = threadIdx.x & 31;
  const __nv_bfloat16* po = o + (int64_t)t * o_stride + (int64_t)h * HD;
  const __nv_bfloat16* pd = d_o + (int64_t)t * do_stride + (int64_t)h * HD;
  float s = 0.f;
  for (int c = lane * 2; c < HD; c += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(po + c));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pd + c));
    s += a.x * b.x + a.y * b.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[(int64_t)h * T + t] = s;
}

// ------------------------------------------------------------------------------------------- host
int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                   const uint32_t* box);

// [T, H, HD] tensor with token stride `tok_stride` elements -> 3-D map {HD, H, T}, box {64, 1, rows}.
static inline int make_thd_map(CUtensorMap* m, const void* p, int T, int H, int HD, int64_t tok_stride, uint32_t rows = 128) {
  uint64_t dims[3] = {(uint64_t)HD, (uint64_t)H, (uint64_t)T};
  uint64_t str[2] = {(uint64_t)HD * 2, (uint64_t)tok_stride * 2};
  uint32_t box[3] = {64, 1, rows};
  return make_tmap_bf16(m, p, 3, dims, str, box);
}

template <typename K>
static inline int set_smem(K kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? 0 : -2;
}


}  // namespace llmt
