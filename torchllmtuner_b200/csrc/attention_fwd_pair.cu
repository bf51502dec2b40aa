// Flash-attention forward for sm_100a with two query heads of one key/value group per CTA (tcgen05 / TMEM).
// (reference call sites: llmtuner/models/qwen/qwen3/model.py:270-283, llmtuner/kernel/ops/varlen_attention.py:60-85.)
//
// A 128x128x16 product with both operands in shared memory reads 8 KB per 64 clocks, the whole shared-memory bandwidth of
// the SM, so the kernel is laid out to read as little shared memory per product as possible:
//   * one CTA owns a 128-row query tile of TWO query heads that share a key/value head; every 128-key K and V tile is
//     loaded once and multiplied by both heads;
//   * S = Q K^T is one N = 128 product per head into tensor memory (two S buffers, one per head);
//   * P = exp2(S * c - m) is written back over S as packed bf16 and fed to O += P V from tensor memory, so P never
//     touches shared memory.
// Tensor memory: S0 | S1 | O0 | O1, 128 columns each (HD = 128). Warps: 0 TMA producer, 1 MMA issuer (+ TMEM
// allocation), 2-5 softmax of head 0, 6-9 softmax of head 1 (one thread per query row). While the softmax warps of one
// head work, the tensor pipe runs the products of the other head. Masks come from the q-tile table (documents, causal
// diagonal) exactly as in the single-head kernel of attention.cu, which remains the path for groups of one query head.
#include "attn_common.cuh"

namespace llmt {

constexpr int kPairThreads = 64 + 256;
constexpr int kPairKV = 128;

template <int HD>
__global__ void __launch_bounds__(kPairThreads, 1)
attn_fwd_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ O, float* __restrict__ lse,
                     const int* __restrict__ tiles, int Hq, int Hkv, int Tq, int64_t o_stride, float scale_log2, int causal,
                     int* status) {
  constexpr int NH = HD / 64;
  constexpr int kTile = 128 * HD * 2;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) report_status(status, kStatusBadArgument, 1501, (int)(smem_u32(smem_raw) & 1023u));
    return;
  }
  uint8_t* sQ = smem_raw;             // [2 heads]
  uint8_t* sK = sQ + 2 * kTile;       // [2 stages]
  uint8_t* sV = sK + 2 * kTile;       // [2 stages]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * kTile);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2 heads]
  uint64_t* p_full = bars + 11;   // [2 heads]
  uint64_t* pv_done = bars + 13;  // [2 heads]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pairs = Hq >> 1;
  const int tile_idx = blockIdx.x / pairs;
  const int h0 = (blockIdx.x % pairs) * 2;            // heads h0, h0 + 1 share a key/value head (group size is even)
  const int hk = h0 / (Hq / Hkv);
  const int* tl = tiles + tile_idx * 8;
  const int q0 = tl[0], nq = tl[1], kbeg = tl[2], klen = tl[3], diag0 = tl[4];
  const int kmax = causal ? min(klen, diag0 + nq - 1) : klen;
  const int n_kv = (kmax + kPairKV - 1) / kPairKV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 128); mbar_init(&pv_done[s], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // S of head g at columns g * 128, O of head g at columns 256 + g * HD
  const uint32_t tS = tmem_base, tO = tmem_base + 256;

  if (warp == 0) {
    // ------------------------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_kv > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_arrive_expect_tx(q_full, 2 * kTile);
#pragma unroll
      for (int g = 0; g < 2; ++g)
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) tma_load_3d(sQ + g * kTile + hf * 16384, &tmQ, q_full, hf * 64, h0 + g, q0);
      int armed_k[2] = {-1, -1}, armed_v[2] = {-1, -1};
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait_bounded(&k_empty[s], ph ^ 1, abort_flag, status, 1510 + s)) break;
        mbar_arrive_expect_tx(&k_full[s], kTile);
        armed_k[s] = (int)ph;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) tma_load_3d(sK + s * kTile + hf * 16384, &tmK, &k_full[s], hf * 64, hk, kbeg + j * kPairKV);
        if (!mbar_wait_bounded(&v_empty[s], ph ^ 1, abort_flag, status, 1520 + s)) break;
        mbar_arrive_expect_tx(&v_full[s], kTile);
        armed_v[s] = (int)ph;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) tma_load_3d(sV + s * kTile + hf * 16384, &tmV, &v_full[s], hf * 64, hk, kbeg + j * kPairKV);
      }
      if (*abort_flag) {
        // wait (bounded) for copies in flight before shared memory is released
        for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try_wait(q_full, 0)) break;
        for (int x = 0; x < 2; ++x) {
          if (armed_k[x] >= 0)
            for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try_wait(&k_full[x], (uint32_t)armed_k[x])) break;
          if (armed_v[x] >= 0)
            for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try_wait(&v_full[x], (uint32_t)armed_v[x])) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idS = umma_idesc_bf16(128, kPairKV, false, false);
      constexpr uint32_t idPV = umma_idesc_bf16(128, HD, false, true);
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag, status, 1600);
      auto issue_S = [&](int j, int g) -> bool {            // S_g = Q_g K(j)^T
        const int s = j & 1;
        if (g == 0) {
          if (!mbar_wait_bounded(&k_full[s], (j >> 1) & 1, abort_flag, status, 1610 + s)) return false;
          tc_fence_after();
        }
        const uint32_t loQ = desc_lo(aQ + g * kTile, 16), loK = desc_lo(aK + s * kTile, 16);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma_bf16_ss(tS + g * 128, desc_pack(loQ + koff(ks, 128)), desc_pack(loK + koff(ks, 128)), idS, ks ? 1u : 0u);
        umma_commit(&s_full[g]);
        if (g == 1) umma_commit(&k_empty[s]);
        return true;
      };
      if (ok) ok = issue_S(0, 0) && issue_S(0, 1);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        const bool next = j + 1 < n_kv;
        bool fail = false;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          if (!mbar_wait_bounded(&p_full[g], j & 1, abort_flag, status, 1620 + g)) { fail = true; break; }
          if (g == 0 && !mbar_wait_bounded(&v_full[s], (j >> 1) & 1, abort_flag, status, 1630 + s)) { fail = true; break; }
          tc_fence_after();
          const uint32_t loVm = desc_lo(aV + s * kTile, 16384);
#pragma unroll
          for (int ks = 0; ks < kPairKV / 16; ++ks)           // O_g += P_g V(j), P_g from tensor memory
            umma_bf16_ts(tO + g * HD, tS + g * 128 + ks * 8, desc_pack(loVm + mnoff(ks)), idPV, (j | ks) ? 1u : 0u);
          umma_commit(&pv_done[g]);
          if (g == 1) umma_commit(&v_empty[s]);
          if (next && !issue_S(j + 1, g)) { fail = true; break; }   // refill the S buffer just consumed
        }
        if (fail) break;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------------------------ softmax, one row per thread
    const int g = (warp - 2) >> 2;            // which of the two heads
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tSg = tS + g * 128 + lane_off, tOg = tO + g * HD + lane_off;
    float m_used = -INFINITY, l = 0.f;
    const int row_limit = causal ? min(klen, diag0 + row) : klen;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      if (!mbar_wait_bounded(&s_full[g], j & 1, abort_flag, status, 1700 + g)) { ok = false; break; }
      tc_fence_after();
      const int kbase = j * kPairKV;
      const bool need_mask = kbase + kPairKV > (causal ? min(klen, diag0) : klen);
      // pass 1: running maximum of the row (four 32-column reads; eight independent maxima keep the chains short)
      float mxs[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) mxs[q] = -INFINITY;
#pragma unroll
      for (int c = 0; c < kPairKV / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tSg + c * 32, r);
        tmem_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) if (kbase + c * 32 + i < row_limit) mxs[i & 7] = fmaxf(mxs[i & 7], __uint_as_float(r[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mxs[i & 7] = fmaxf(mxs[i & 7], __uint_as_float(r[i]));
        }
      }
      float mx = fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])), fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
      mx *= scale_log2;
      const float m_new = fmaxf(m_used, mx);
      const bool need = m_new > m_used + 8.f;  // lazy rescale: only when the running maximum moved by more than 2^8
      if (__any_sync(0xffffffffu, need)) {
        const float alpha = need ? ((m_used == -INFINITY) ? 0.f : ex2(m_used - m_new)) : 1.f;
        if (need) { l *= alpha; m_used = m_new; }
        if (j > 0) {
          if (!mbar_wait_bounded(&pv_done[g], (j - 1) & 1, abort_flag, status, 1710 + g)) { ok = false; break; }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tOg + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tOg + c * 32, o);
          }
          tmem_wait_st();
        }
      }
      // pass 2: P = exp2(S * c - m), packed bf16 over the columns already read; row sum in fp32
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
      float rsum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < kPairKV / 32; ++c) {
        uint32_t r[32], w[16];
        tmem_ld_32x32(tSg + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2(__uint_as_float(r[i]) * scale_log2 - m_safe);
          float p1 = ex2(__uint_as_float(r[i + 1]) * scale_log2 - m_safe);
          if (need_mask) {
            if (kbase + c * 32 + i >= row_limit) p0 = 0.f;
            if (kbase + c * 32 + i + 1 >= row_limit) p1 = 0.f;
          }
          rsum[(i >> 1) & 3] += p0 + p1;
          w[i >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x16(tSg + c * 16, w);       // columns [16c, 16c + 16) lie behind the read position 32c
      }
      l += (rsum[0] + rsum[1]) + (rsum[2] + rsum[3]);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&p_full[g]);
    }
    // ---- finalize
    if (ok && n_kv > 0) ok = mbar_wait_bounded(&pv_done[g], (n_kv - 1) & 1, abort_flag, status, 1720 + g);
    if (ok) {
      tc_fence_after();
      const int h = h0 + g;
      const float inv = (l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow = O + (int64_t)(q0 + row) * o_stride + (int64_t)h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        if (n_kv > 0) {
          tmem_ld_32x32(tOg + c * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (row < nq) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[8 * v]) * inv, __uint_as_float(r[8 * v + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]) * inv, __uint_as_float(r[8 * v + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]) * inv, __uint_as_float(r[8 * v + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]) * inv, __uint_as_float(r[8 * v + 7]) * inv);
            reinterpret_cast<uint4*>(orow + c * 32)[v] = o;
          }
        }
      }
      if (row < nq) lse[(int64_t)h * Tq + q0 + row] = (l > 0.f) ? (m_used + log2f(l)) * kLn2 : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace llmt

using namespace llmt;

// Same contract as llmt_attn_fwd; needs an even number of query heads per key/value head.
extern "C" int llmt_attn_fwd_pair(const void* q, const void* k, const void* v, void* o, float* lse, const int* tiles, int num_tiles,
                                  int Tq, int Tk, int Hq, int Hkv, int HD, int64_t q_stride, int64_t k_stride, int64_t v_stride,
                                  int64_t o_stride, float scale, int causal, int* status, cudaStream_t st) {
  if (num_tiles <= 0 || Hq <= 0) return 0;
  if ((HD != 64 && HD != 128) || Hq % Hkv || ((Hq / Hkv) & 1) || (q_stride & 7) || (k_stride & 7) || (v_stride & 7) || (o_stride & 7))
    return -10;
  CUtensorMap tq, tk, tv;
  if (make_thd_map(&tq, q, Tq, Hq, HD, q_stride) || make_thd_map(&tk, k, Tk, Hkv, HD, k_stride) || make_thd_map(&tv, v, Tk, Hkv, HD, v_stride))
    return -11;
  const int smem = 6 * 128 * HD * 2 + 256;   // exact: no alignment slack, see the kernel
  const float sl2 = scale * kLog2e;
  if (HD == 128) {
    static bool cfg = false;
    if (!cfg) { if (set_smem(attn_fwd_pair_kernel<128>, smem)) return -2; cfg = true; }
    attn_fwd_pair_kernel<128><<<num_tiles * (Hq / 2), kPairThreads, smem, st>>>(tq, tk, tv, (__nv_bfloat16*)o, lse, tiles, Hq, Hkv, Tq,
                                                                                 o_stride, sl2, causal, status);
  } else {
    static bool cfg = false;
    if (!cfg) { if (set_smem(attn_fwd_pair_kernel<64>, smem)) return -2; cfg = true; }
    attn_fwd_pair_kernel<64><<<num_tiles * (Hq / 2), kPairThreads, smem, st>>>(tq, tk, tv, (__nv_bfloat16*)o, lse, tiles, Hq, Hkv, Tq,
                                                                                o_stride, sl2, causal, status);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
