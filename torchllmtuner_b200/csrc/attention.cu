// Variable-length causal GQA flash attention for sm_100a on tcgen05 / TMEM, forward and backward.
// (reference call sites: llmtuner/models/qwen/qwen3/model.py:270-283 through the HF attention interface, and
//  llmtuner/kernel/ops/varlen_attention.py:60-85; the reference builds a dense [B,1,T,T] mask for packed rows
//  (llmtuner/models/common/attention.py:14-62) where this kernel masks from per-tile document bounds.)
//
// Layout: q [Tq, Hq, HD], k/v [Tk, Hkv, HD], bf16, heads packed (head stride HD), arbitrary token stride.
// Work is described by tile tables built on the host from cu_seqlens (int32 [n][8]):
//   q tile : {q0, nq, kbeg, klen, diag0}        rows q0..q0+nq of one document; its keys are rows kbeg..kbeg+klen;
//                                               row i of the tile sees keys [0, min(klen, diag0 + i)) when causal.
//   k tile : {k0, nk, kk0, qbeg, qlen, off, klen} keys k0..k0+nk (index kk0.. inside the document); the document's
//                                               queries are rows qbeg..qbeg+qlen; query r sees key x iff x <= r + off.
// Forward: one CTA per (q tile, head): S = Q K^T into TMEM, softmax in registers (row per thread, lazy rescale of
// the TMEM-resident O), P through shared memory, O += P V.  Backward: a dK/dV kernel per (k tile, kv head) that
// loops over the query heads of the group and the q tiles, and a dQ kernel per (q tile, head); both recompute
// S and dP so that no atomics are needed.
#include <type_traits>
#include "attn_common.cuh"

namespace llmt {

// =========================================================================================== forward
// Forward tiles: 128 query rows x 64 keys. K is double buffered, V single buffered, P goes through shared memory:
// 96 KB of shared memory and 256 TMEM columns per CTA at head size 128, so two CTAs share an SM and the softmax of one
// overlaps the MMAs of the other. Head size 256 (a K loop of 16 slices for S, one N=256 product for P V) takes 192 KB and
// 128 + 256 = 384 columns, allocated as 512: one CTA per SM, which shared memory already enforces, so the allocation
// never waits on a co-resident CTA of this kernel.
constexpr int kFwdKV = 64;


template <int HD>
__global__ void __launch_bounds__(kAttnThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ O, float* __restrict__ lse,
                const int* __restrict__ tiles, int Hq, int Hkv, int Tq, int64_t o_stride, float scale_log2, int causal,
                int* status) {
  constexpr int NH = HD / 64;
  constexpr int kQBytes = 128 * HD * 2;
  constexpr int kKVBytes = kFwdKV * HD * 2;
  constexpr int kPBytes = 128 * kFwdKV * 2;
  constexpr uint32_t kTmemCols = HD > 128 ? 512u : 256u;
  // The launch asks for exactly the bytes used (two CTAs must fit in one SM), so the dynamic shared memory base has to be
  // 1024-byte aligned already; the kernel refuses to run otherwise instead of overrunning its allocation.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) report_status(status, kStatusBadArgument, 1001, (int)(smem_u32(smem_raw) & 1023u));
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kQBytes;        // 2 stages
  uint8_t* sV = sK + 2 * kKVBytes;   // 1 stage
  uint8_t* sP = sV + kKVBytes;       // 2 buffers
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kPBytes);
  uint64_t* q_full = bars;
  uint64_t* kfull = bars + 1;
  uint64_t* kempty = bars + 3;
  uint64_t* vfull = bars + 5;
  uint64_t* vempty = bars + 6;
  uint64_t* sfull = bars + 7;
  uint64_t* sempty = bars + 9;
  uint64_t* pfull = bars + 11;    // [2]
  uint64_t* pvdone = bars + 13;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_idx = blockIdx.x / Hq;
  const int h = blockIdx.x % Hq;
  const int hk = h / (Hq / Hkv);
  const int* tl = tiles + tile_idx * 8;
  const int q0 = tl[0], nq = tl[1], kbeg = tl[2], klen = tl[3], diag0 = tl[4];
  const int kmax = causal ? min(klen, diag0 + nq - 1) : klen;
  const int n_kv = (kmax + kFwdKV - 1) / kFwdKV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kfull[s], 1); mbar_init(&kempty[s], 1);
      mbar_init(&sfull[s], 1); mbar_init(&sempty[s], 128);
      mbar_init(&pfull[s], 128); mbar_init(&pvdone[s], 1);
    }
    mbar_init(vfull, 1); mbar_init(vempty, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tO = tmem_base + 128;   // S: 2 buffers x 64 columns; O: HD columns

  if (warp == 0) {
    if (lane == 0 && n_kv > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_arrive_expect_tx(q_full, kQBytes);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) tma_load_3d(sQ + hf * 16384, &tmQ, q_full, hf * 64, h, q0);
      int armed_k[2] = {-1, -1}, armed_v = -1;
      auto load_k = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait_bounded(&kempty[s], ph ^ 1, abort_flag, status, 1100 + s)) return false;
        mbar_arrive_expect_tx(&kfull[s], kKVBytes);
        armed_k[s] = (int)ph;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf)
          tma_load_3d(sK + s * kKVBytes + hf * (kFwdKV * 128), &tmK, &kfull[s], hf * 64, hk, kbeg + j * kFwdKV);
        return true;
      };
      bool pok = load_k(0);
      for (int j = 0; j < n_kv && pok; ++j) {
        if (j + 1 < n_kv && !load_k(j + 1)) break;     // K runs one tile ahead of V: S(j+1) is issued before PV(j)
        if (!mbar_wait_bounded(vempty, (j & 1) ^ 1, abort_flag, status, 1110)) break;
        mbar_arrive_expect_tx(vfull, kKVBytes);
        armed_v = j & 1;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) tma_load_3d(sV + hf * (kFwdKV * 128), &tmV, vfull, hf * 64, hk, kbeg + j * kFwdKV);
      }
      if (*abort_flag) {
        // wait (bounded) for copies in flight before shared memory is released
        for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try_wait(q_full, 0)) break;
        for (int x = 0; x < 2; ++x)
          if (armed_k[x] >= 0)
            for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try_wait(&kfull[x], (uint32_t)armed_k[x])) break;
        if (armed_v >= 0)
          for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try_wait(vfull, (uint32_t)armed_v)) break;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idS = umma_idesc_bf16(128, kFwdKV, false, false);
      constexpr uint32_t idPV = umma_idesc_bf16(128, HD, false, true);
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP);
      const uint32_t loVm = desc_lo(aV, kFwdKV * 128);
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag, status, 1200);
      auto issue_S = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait_bounded(&kfull[s], ph, abort_flag, status, 1210 + s)) return false;
        if (!mbar_wait_bounded(&sempty[s], ph ^ 1, abort_flag, status, 1220 + s)) return false;
        tc_fence_after();
        {
          // descriptors differ only in the start address field: build the two bases once and step the low word
          const uint64_t dq0 = desc_kmajor_rows(aQ, 0, 128), dk0 = desc_kmajor_rows(aK + s * kKVBytes, 0, kFwdKV);
          const uint32_t d_s = tS + s * kFwdKV;
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint64_t offq = (uint64_t)(((ks >> 2) * (128 * 128) + (ks & 3) * 32) >> 4);
            const uint64_t offk = (uint64_t)(((ks >> 2) * (kFwdKV * 128) + (ks & 3) * 32) >> 4);
            umma_bf16_ss(d_s, dq0 + offq, dk0 + offk, idS, ks ? 1u : 0u);
          }
        }
        umma_commit(&sfull[s]);
        umma_commit(&kempty[s]);
        return true;
      };
      if (ok) ok = issue_S(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) { if (!issue_S(j + 1)) break; }
        const int pb = j & 1;
        if (!mbar_wait_bounded(&pfull[pb], (j >> 1) & 1, abort_flag, status, 1230 + pb)) break;
        if (!mbar_wait_bounded(vfull, j & 1, abort_flag, status, 1240)) break;
        tc_fence_after();
        const uint32_t loP = desc_lo(aP + pb * kPBytes, 16), acc0 = j ? 1u : 0u;
#pragma unroll
        for (int ks = 0; ks < kFwdKV / 16; ++ks)
          umma_bf16_ss(tO, desc_pack(loP + koff(ks, 128)), desc_pack(loVm + mnoff(ks)), idPV, ks ? 1u : acc0);
        umma_commit(vempty);
        umma_commit(&pvdone[pb]);
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    const int row_limit = causal ? min(klen, diag0 + row) : klen;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int s = j & 1;
      if (!mbar_wait_bounded(&sfull[s], (j >> 1) & 1, abort_flag, status, 1300 + s)) { ok = false; break; }
      tc_fence_after();
      const uint32_t ts = tS + lane_off + s * kFwdKV;
      const int kbase = j * kFwdKV;
      const bool need_mask = kbase + kFwdKV > (causal ? min(klen, diag0) : klen);
      // the whole S row of this tile (64 values) stays in registers between the max pass and the exp pass
      uint32_t r[kFwdKV];
      tmem_ld_32x32(ts, r);
      tmem_ld_32x32(ts + 32, r + 32);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&sempty[s]);      // S buffer s may be overwritten by the MMA of tile j + 2
      // eight independent running maxima keep the dependency chains short
      float mxs[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) mxs[q] = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < kFwdKV; ++i) if (kbase + i < row_limit) mxs[i & 7] = fmaxf(mxs[i & 7], __uint_as_float(r[i]));
      } else {
#pragma unroll
        for (int i = 0; i < kFwdKV; ++i) mxs[i & 7] = fmaxf(mxs[i & 7], __uint_as_float(r[i]));
      }
      float mx = fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])), fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
      mx *= scale_log2;
      const float m_new = fmaxf(m_used, mx);
      const bool need = m_new > m_used + 8.f;  // lazy rescale: only when the running max moved by more than 2^8
      if (__any_sync(0xffffffffu, need)) {
        const float alpha = need ? ((m_used == -INFINITY) ? 0.f : ex2(m_used - m_new)) : 1.f;
        if (need) { l *= alpha; m_used = m_new; }
        if (j > 0) {
          if (!mbar_wait_bounded(&pvdone[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, status, 1310)) { ok = false; break; }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tO + lane_off + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tO + lane_off + c * 32, o);
          }
          tmem_wait_st();
        }
      }
      if (j > 1) {   // P buffer j & 1 was last read by the PV product of tile j - 2
        if (!mbar_wait_bounded(&pvdone[j & 1], (((j >> 1) & 1) ^ 1), abort_flag, status, 1320)) { ok = false; break; }
      }
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
      float rsum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < kFwdKV / 32; ++c) {
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2(__uint_as_float(r[c * 32 + i]) * scale_log2 - m_safe);
          float p1 = ex2(__uint_as_float(r[c * 32 + i + 1]) * scale_log2 - m_safe);
          if (need_mask) {
            if (kbase + c * 32 + i >= row_limit) p0 = 0.f;
            if (kbase + c * 32 + i + 1 >= row_limit) p1 = 0.f;
          }
          rsum[(i >> 1) & 3] += p0 + p1;
          w[i >> 1] = pack_bf16x2(p0, p1);
        }
        store_row32_swz(sP + (j & 1) * kPBytes, row, c * 32, w);
      }
      l += (rsum[0] + rsum[1]) + (rsum[2] + rsum[3]);
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&pfull[j & 1]);
    }
    // ---- finalize
    if (ok && n_kv > 0) ok = mbar_wait_bounded(&pvdone[(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, abort_flag, status, 1330);
    if (ok) {
      tc_fence_after();
      const float inv = (l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow = O + (int64_t)(q0 + row) * o_stride + (int64_t)h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        if (n_kv > 0) {
          tmem_ld_32x32(tO + lane_off + c * 32, r);
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// =========================================================================================== backward: dK, dV
// One CTA per (128-key tile, kv head). It walks the query heads of the group and their 64-row q tiles. S^T and dP^T are
// double buffered in TMEM, Q / dO and P^T / dS^T are double buffered in shared memory, so the MMAs of q tile i+1 run
// while the 128 compute threads turn S^T, dP^T of tile i into P^T, dS^T; dV and dK accumulate in TMEM over the whole walk.
constexpr int kBwdQ = 64;
constexpr int kBwdQStages = 3;   // Q / dO stages of the dK/dV kernel
constexpr int kBwdThreads = 64 + 256;   // TMA warp, MMA warp, 8 compute warps (two per TMEM lane quarter, one per column half)

template <int HD>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const float* __restrict__ lse, const float* __restrict__ delta, __nv_bfloat16* __restrict__ dK,
                    __nv_bfloat16* __restrict__ dV, const int* __restrict__ tiles, int Hq, int Hkv, int Tq, int64_t dk_stride,
                    int64_t dv_stride, float scale, int causal, int accumulate, int* status) {
  constexpr int NH = HD / 64;
  constexpr int kKVBytes = 128 * HD * 2;
  constexpr int kQBytes = kBwdQ * HD * 2;
  constexpr int kPBytes = 128 * kBwdQ * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + kKVBytes;
  // Q / dO tiles have three stages: a stage is free again only when the dV / dK products that read it have completed,
  // and with two stages the reload (a full TMA round trip) sat on the critical path of every iteration.
  uint8_t* sQ = sV + kKVBytes;              // kBwdQStages stages
  uint8_t* sdO = sQ + kBwdQStages * kQBytes;
  uint8_t* sPT = sdO + kBwdQStages * kQBytes;   // 2 buffers
  uint8_t* sdST = sPT + 2 * kPBytes;    // 2 buffers
  float* s_lse = reinterpret_cast<float*>(sdST + 2 * kPBytes);   // [2][64]
  float* s_delta = s_lse + 2 * kBwdQ;                            // [2][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_delta + 2 * kBwdQ);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;     // [kBwdQStages]
  uint64_t* qdo_empty = bars + 4;    // [kBwdQStages]
  uint64_t* s_full = bars + 7;       // [2]
  uint64_t* s_empty = bars + 9;      // [2]
  uint64_t* p_full = bars + 11;      // [2]
  uint64_t* p_empty = bars + 13;     // [2]
  uint64_t* acc_done = bars + 15;
  uint64_t* stat_ready = bars + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_idx = blockIdx.x / Hkv;
  const int hk = blockIdx.x % Hkv;
  const int g = Hq / Hkv;
  const int* tl = tiles + tile_idx * 8;
  const int k0 = tl[0], nk = tl[1], kk0 = tl[2], qbeg = tl[3], qlen = tl[4], off = tl[5], klen = tl[6];
  int qs = 0;
  if (causal) { qs = kk0 - off; if (qs < 0) qs = 0; qs &= ~(kBwdQ - 1); }
  const int n_qt = (qlen > qs) ? (qlen - qs + kBwdQ - 1) / kBwdQ : 0;
  const int n_it = n_qt * g;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int b = 0; b < kBwdQStages; ++b) { mbar_init(&qdo_full[b], 1); mbar_init(&qdo_empty[b], 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1); mbar_init(&s_empty[b], 256);
      mbar_init(&p_full[b], 256); mbar_init(&p_empty[b], 1);
    }
    mbar_init(acc_done, 1); mbar_init(stat_ready, 256);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tST = tmem_base, tDPT = tmem_base + 2 * kBwdQ, tDV = tmem_base + 256, tDK = tmem_base + 256 + HD;

  if (warp == 0) {
    if (lane == 0 && n_it > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
      mbar_arrive_expect_tx(kv_full, 2 * kKVBytes);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
        tma_load_3d(sK + hf * 16384, &tmK, kv_full, hf * 64, hk, k0);
        tma_load_3d(sV + hf * 16384, &tmV, kv_full, hf * 64, hk, k0);
      }
      int armed[kBwdQStages] = {-1, -1, -1};
      for (int it = 0; it < n_it; ++it) {
        const int b = it % kBwdQStages;
        const uint32_t ph = (it / kBwdQStages) & 1;
        const int h = hk * g + it / n_qt;
        const int qrow = qbeg + qs + (it % n_qt) * kBwdQ;
        if (!mbar_wait_bounded(&qdo_empty[b], ph ^ 1, abort_flag, status, 2100 + b)) break;
        mbar_arrive_expect_tx(&qdo_full[b], 2 * kQBytes);
        armed[b] = (int)ph;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) {
          tma_load_3d(sQ + b * kQBytes + hf * (kBwdQ * 128), &tmQ, &qdo_full[b], hf * 64, h, qrow);
          tma_load_3d(sdO + b * kQBytes + hf * (kBwdQ * 128), &tmdO, &qdo_full[b], hf * 64, h, qrow);
        }
      }
      if (*abort_flag) {
        for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try_wait(kv_full, 0)) break;
        for (int b = 0; b < kBwdQStages; ++b)
          if (armed[b] >= 0)
            for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try_wait(&qdo_full[b], (uint32_t)armed[b])) break;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idS = umma_idesc_bf16(128, kBwdQ, false, false);
      constexpr uint32_t idAcc = umma_idesc_bf16(128, HD, false, true);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), adO = smem_u32(sdO), aPT = smem_u32(sPT),
                     adST = smem_u32(sdST);
      bool ok = mbar_wait_bounded(kv_full, 0, abort_flag, status, 2200);
      const uint32_t loK = desc_lo(aK, 16), loV = desc_lo(aV, 16);
      auto issue_S = [&](int it) -> bool {
        const int b = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int qb = it % kBwdQStages;                       // Q / dO stage
        if (!mbar_wait_bounded(&qdo_full[qb], (it / kBwdQStages) & 1, abort_flag, status, 2210 + qb)) return false;
        if (!mbar_wait_bounded(&s_empty[b], ph ^ 1, abort_flag, status, 2215 + b)) return false;
        tc_fence_after();
        const uint32_t loQ = desc_lo(aQ + qb * kQBytes, 16), lodO = desc_lo(adO + qb * kQBytes, 16);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma_bf16_ss(tST + b * kBwdQ, desc_pack(loK + koff(ks, 128)), desc_pack(loQ + koff(ks, kBwdQ)), idS, ks ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma_bf16_ss(tDPT + b * kBwdQ, desc_pack(loV + koff(ks, 128)), desc_pack(lodO + koff(ks, kBwdQ)), idS, ks ? 1u : 0u);
        umma_commit(&s_full[b]);
        return true;
      };
      if (ok) ok = issue_S(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const int b = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int qb = it % kBwdQStages;
        if (it + 1 < n_it) { if (!issue_S(it + 1)) break; }
        if (!mbar_wait_bounded(&p_full[b], ph, abort_flag, status, 2220 + b)) break;
        tc_fence_after();
        const uint32_t loPT = desc_lo(aPT + b * kPBytes, 16), lodST = desc_lo(adST + b * kPBytes, 16);
        const uint32_t lodOm = desc_lo(adO + qb * kQBytes, kBwdQ * 128), loQm = desc_lo(aQ + qb * kQBytes, kBwdQ * 128);
        const uint32_t acc0 = it ? 1u : 0u;
#pragma unroll
        for (int ks = 0; ks < kBwdQ / 16; ++ks)
          umma_bf16_ss(tDV, desc_pack(loPT + koff(ks, 128)), desc_pack(lodOm + mnoff(ks)), idAcc, ks ? 1u : acc0);
#pragma unroll
        for (int ks = 0; ks < kBwdQ / 16; ++ks)
          umma_bf16_ss(tDK, desc_pack(lodST + koff(ks, 128)), desc_pack(loQm + mnoff(ks)), idAcc, ks ? 1u : acc0);
        umma_commit(&qdo_empty[qb]);
        umma_commit(&p_empty[b]);
        if (it == n_it - 1) umma_commit(acc_done);
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // key row inside the tile
    const int tid = threadIdx.x - 64;     // 0..255
    const int half = tid >> 7;            // which 32 of the 64 query columns this thread handles
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const int key_idx = kk0 + row;
    const bool key_ok = (row < nk) && (key_idx < klen);
    const float scale_log2 = scale * kLog2e;
    bool ok = true;
    // Row statistics (log-sum-exp, delta) of a query tile are fetched one iteration ahead: the global loads are issued
    // at the top of iteration it-1, parked in registers while that iteration computes, and published at its end.
    auto load_stats = [&](int it, float& l, float& d) {
      const int h = hk * g + it / n_qt;
      const int qi = qs + (it % n_qt) * kBwdQ + tid;
      const bool v = qi < qlen;
      l = v ? lse[(int64_t)h * Tq + qbeg + qi] * kLog2e : INFINITY;
      d = v ? delta[(int64_t)h * Tq + qbeg + qi] : 0.f;
    };
    if (n_it > 0) {
      if (tid < kBwdQ) {
        float l, d;
        load_stats(0, l, d);
        s_lse[tid] = l;
        s_delta[tid] = d;
      }
      mbar_arrive(stat_ready);
    }
    for (int it = 0; it < n_it && ok; ++it) {
      const int b = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      const int qi0 = qs + (it % n_qt) * kBwdQ;  // first query index (inside the document) of this q tile
      float next_l = INFINITY, next_d = 0.f;
      const bool have_next = it + 1 < n_it;
      if (have_next && tid < kBwdQ) load_stats(it + 1, next_l, next_d);
      if (!mbar_wait_bounded(stat_ready, it & 1, abort_flag, status, 2330)) { ok = false; break; }
      if (!mbar_wait_bounded(&s_full[b], ph, abort_flag, status, 2300 + b)) { ok = false; break; }
      tc_fence_after();
      uint32_t rs[32], rd[32];
      tmem_ld_32x32(tST + lane_off + b * kBwdQ + half * 32, rs);
      tmem_ld_32x32(tDPT + lane_off + b * kBwdQ + half * 32, rd);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&s_empty[b]);
      if (!mbar_wait_bounded(&p_empty[b], ph ^ 1, abort_flag, status, 2310 + b)) { ok = false; break; }
      // Most tiles lie wholly below the causal diagonal and inside the document: they skip the per-element visibility
      // test (the branch is uniform over the CTA). Row statistics come from shared memory four at a time.
      const bool tile_full = (nk == 128) && (kk0 + 128 <= klen) && (qi0 + kBwdQ <= qlen) && (!causal || kk0 + 127 <= qi0 + off);
      const float4* pl4 = reinterpret_cast<const float4*>(s_lse + b * kBwdQ + half * 32);
      const float4* pd4 = reinterpret_cast<const float4*>(s_delta + b * kBwdQ + half * 32);
      uint32_t wp[16], wd[16];
      auto softmax_cols = [&](auto masked) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 l4 = pl4[i >> 2], d4 = pd4[i >> 2];
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dv[4] = {d4.x, d4.y, d4.z, d4.w};
          float p[4], ds[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float pv = ex2(__uint_as_float(rs[i + e]) * scale_log2 - lv[e]);
            if constexpr (decltype(masked)::value) {
              const int qi = qi0 + half * 32 + i + e;
              const bool vis = key_ok && (qi < qlen) && (!causal || key_idx <= qi + off);
              pv = vis ? pv : 0.f;
            }
            p[e] = pv;
            ds[e] = pv * (__uint_as_float(rd[i + e]) - dv[e]);
          }
          wp[i >> 1] = pack_bf16x2(p[0], p[1]);
          wp[(i >> 1) + 1] = pack_bf16x2(p[2], p[3]);
          wd[i >> 1] = pack_bf16x2(ds[0], ds[1]);
          wd[(i >> 1) + 1] = pack_bf16x2(ds[2], ds[3]);
        }
      };
      if (tile_full) softmax_cols(std::false_type{}); else softmax_cols(std::true_type{});
      store_row32_swz(sPT + b * kPBytes, row, half * 32, wp);
      store_row32_swz(sdST + b * kPBytes, row, half * 32, wd);
      fence_proxy_async_smem();
      mbar_arrive(&p_full[b]);
      if (have_next) {
        // every thread has passed this iteration's stat_ready wait, so nobody still reads the other buffer
        if (tid < kBwdQ) {
          s_lse[(b ^ 1) * kBwdQ + tid] = next_l;
          s_delta[(b ^ 1) * kBwdQ + tid] = next_d;
        }
        mbar_arrive(stat_ready);
      }
    }
    if (ok && n_it > 0) ok = mbar_wait_bounded(acc_done, 0, abort_flag, status, 2320);
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* kr = dK + (int64_t)(k0 + row) * dk_stride + (int64_t)hk * HD;
      __nv_bfloat16* vr = dV + (int64_t)(k0 + row) * dv_stride + (int64_t)hk * HD;
#pragma unroll 1
      for (int c = half * (HD / 64); c < (half + 1) * (HD / 64); ++c) {
        uint32_t rk[32], rv[32];
        if (n_it > 0) {
          tmem_ld_32x32(tDK + lane_off + c * 32, rk);
          tmem_ld_32x32(tDV + lane_off + c * 32, rv);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { rk[i] = 0u; rv[i] = 0u; }
        }
        if (row < nk) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 a, bq;
            a.x = pack_bf16x2(__uint_as_float(rk[8 * v]) * scale, __uint_as_float(rk[8 * v + 1]) * scale);
            a.y = pack_bf16x2(__uint_as_float(rk[8 * v + 2]) * scale, __uint_as_float(rk[8 * v + 3]) * scale);
            a.z = pack_bf16x2(__uint_as_float(rk[8 * v + 4]) * scale, __uint_as_float(rk[8 * v + 5]) * scale);
            a.w = pack_bf16x2(__uint_as_float(rk[8 * v + 6]) * scale, __uint_as_float(rk[8 * v + 7]) * scale);
            bq.x = pack_bf16x2(__uint_as_float(rv[8 * v]), __uint_as_float(rv[8 * v + 1]));
            bq.y = pack_bf16x2(__uint_as_float(rv[8 * v + 2]), __uint_as_float(rv[8 * v + 3]));
            bq.z = pack_bf16x2(__uint_as_float(rv[8 * v + 4]), __uint_as_float(rv[8 * v + 5]));
            bq.w = pack_bf16x2(__uint_as_float(rv[8 * v + 6]), __uint_as_float(rv[8 * v + 7]));
            if (accumulate) {
              const uint4 pa = reinterpret_cast<const uint4*>(kr + c * 32)[v], pb = reinterpret_cast<const uint4*>(vr + c * 32)[v];
              const __nv_bfloat162 *ha = reinterpret_cast<const __nv_bfloat162*>(&pa), *hb = reinterpret_cast<const __nv_bfloat162*>(&pb);
              __nv_bfloat162 *na = reinterpret_cast<__nv_bfloat162*>(&a), *nb = reinterpret_cast<__nv_bfloat162*>(&bq);
#pragma unroll
              for (int jj = 0; jj < 4; ++jj) {
                na[jj] = __hadd2(na[jj], ha[jj]);
                nb[jj] = __hadd2(nb[jj], hb[jj]);
              }
            }
            reinterpret_cast<uint4*>(kr + c * 32)[v] = a;
            reinterpret_cast<uint4*>(vr + c * 32)[v] = bq;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// =========================================================================================== backward: dQ
template <int HD>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const float* __restrict__ lse, const float* __restrict__ delta, __nv_bfloat16* __restrict__ dQ,
                   const int* __restrict__ tiles, int Hq, int Hkv, int Tq, int64_t dq_stride, float scale, int causal,
                   int* status) {
  using SM = AttnSmem<HD>;
  constexpr int NH = HD / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + SM::kTile;
  uint8_t* sK = sdO + SM::kTile;      // 2 stages
  uint8_t* sV = sK + 2 * SM::kTile;   // 2 stages
  uint8_t* sdS = sV + 2 * SM::kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + SM::kP);
  uint64_t* qdo_full = bars;
  uint64_t* kfull = bars + 1;
  uint64_t* kempty = bars + 3;
  uint64_t* vfull = bars + 5;
  uint64_t* vempty = bars + 7;
  uint64_t* s_full = bars + 9;       // [2]: S of key tile j lands in TMEM buffer j & 1
  uint64_t* dp_full = bars + 11;
  uint64_t* ds_full = bars + 12;
  uint64_t* dq_done = bars + 13;
  uint64_t* dp_empty = bars + 14;    // the softmax warps hold dP of the current tile in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_idx = blockIdx.x / Hq;
  const int h = blockIdx.x % Hq;
  const int hk = h / (Hq / Hkv);
  const int* tl = tiles + tile_idx * 8;
  const int q0 = tl[0], nq = tl[1], kbeg = tl[2], klen = tl[3], diag0 = tl[4];
  const int kmax = causal ? min(klen, diag0 + nq - 1) : klen;
  const int n_kv = (kmax + 127) / 128;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kfull[s], 1); mbar_init(&kempty[s], 1); mbar_init(&vfull[s], 1); mbar_init(&vempty[s], 1);
    }
    mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1); mbar_init(dp_full, 1); mbar_init(ds_full, 256); mbar_init(dq_done, 1);
    mbar_init(dp_empty, 256);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // S is double buffered (columns 0..127 and 384..511) so that Q K^T of the next key tile is issued while the softmax
  // warps still work on the current one; dP (128..255) and dQ (256..) are single.
  const uint32_t tS0 = tmem_base, tS1 = tmem_base + 384, tDP = tmem_base + 128, tDQ = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0 && n_kv > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
      mbar_arrive_expect_tx(qdo_full, 2 * SM::kTile);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
        tma_load_3d(sQ + hf * 16384, &tmQ, qdo_full, hf * 64, h, q0);
        tma_load_3d(sdO + hf * 16384, &tmdO, qdo_full, hf * 64, h, q0);
      }
      int armed[4] = {-1, -1, -1, -1};
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait_bounded(&kempty[s], ph ^ 1, abort_flag, status, 3100 + s)) break;
        mbar_arrive_expect_tx(&kfull[s], SM::kTile);
        armed[s] = (int)ph;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) tma_load_3d(sK + s * SM::kTile + hf * 16384, &tmK, &kfull[s], hf * 64, hk, kbeg + j * 128);
        if (!mbar_wait_bounded(&vempty[s], ph ^ 1, abort_flag, status, 3110 + s)) break;
        mbar_arrive_expect_tx(&vfull[s], SM::kTile);
        armed[2 + s] = (int)ph;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) tma_load_3d(sV + s * SM::kTile + hf * 16384, &tmV, &vfull[s], hf * 64, hk, kbeg + j * 128);
      }
      if (*abort_flag) {
        for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try_wait(qdo_full, 0)) break;
        for (int x = 0; x < 4; ++x) {
          if (armed[x] < 0) continue;
          uint64_t* b = (x < 2) ? &kfull[x] : &vfull[x - 2];
          for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try_wait(b, (uint32_t)armed[x])) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idS = umma_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idDQ = umma_idesc_bf16(128, HD, false, true);
      const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO), aK = smem_u32(sK), aV = smem_u32(sV), adS = smem_u32(sdS);
      bool ok = mbar_wait_bounded(qdo_full, 0, abort_flag, status, 3200);
      const uint32_t loQ = desc_lo(aQ, 16), lodO = desc_lo(adO, 16), lodS = desc_lo(adS, 16);
      auto issue_S = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait_bounded(&kfull[s], (j >> 1) & 1, abort_flag, status, 3210 + s)) return false;
        tc_fence_after();
        const uint32_t loKs = desc_lo(aK + s * SM::kTile, 16);
        const uint32_t tSj = s ? tS1 : tS0;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma_bf16_ss(tSj, desc_pack(loQ + koff(ks, 128)), desc_pack(loKs + koff(ks, 128)), idS, ks ? 1u : 0u);
        umma_commit(&s_full[s]);
        return true;
      };
      auto issue_dP = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait_bounded(&vfull[s], (j >> 1) & 1, abort_flag, status, 3220 + s)) return false;
        tc_fence_after();
        const uint32_t loVs = desc_lo(aV + s * SM::kTile, 16);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma_bf16_ss(tDP, desc_pack(lodO + koff(ks, 128)), desc_pack(loVs + koff(ks, 128)), idS, ks ? 1u : 0u);
        umma_commit(dp_full);
        umma_commit(&vempty[s]);
        return true;
      };
      if (ok) ok = issue_S(0) && issue_dP(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        // S of the next tile goes into the other TMEM buffer while the softmax warps are busy with tile j
        if (j + 1 < n_kv) {
          if (!issue_S(j + 1)) break;
          // dP has one TMEM buffer: the next product starts as soon as the softmax warps have copied this tile's dP
          // into registers, not when they have finished its math, so it runs under that math
          if (!mbar_wait_bounded(dp_empty, j & 1, abort_flag, status, 3225)) break;
          if (!issue_dP(j + 1)) break;
        }
        if (!mbar_wait_bounded(ds_full, j & 1, abort_flag, status, 3230)) break;
        tc_fence_after();
        const uint32_t loKm = desc_lo(aK + s * SM::kTile, 16384);
        const uint32_t acc0 = j ? 1u : 0u;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_bf16_ss(tDQ, desc_pack(lodS + koff(ks, 128)), desc_pack(loKm + mnoff(ks)), idDQ, ks ? 1u : acc0);
        umma_commit(&kempty[s]);
        umma_commit(dq_done);
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int half = (threadIdx.x - 64) >> 7;   // which 64 of the 128 key columns this thread handles
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const bool row_ok = row < nq;
    const float scale_log2 = scale * kLog2e;
    const float lse2 = row_ok ? lse[(int64_t)h * Tq + q0 + row] * kLog2e : INFINITY;
    const float dl = row_ok ? delta[(int64_t)h * Tq + q0 + row] : 0.f;
    const int row_limit = row_ok ? (causal ? min(klen, diag0 + row) : klen) : 0;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      if (!mbar_wait_bounded(&s_full[j & 1], (j >> 1) & 1, abort_flag, status, 3300)) { ok = false; break; }
      if (!mbar_wait_bounded(dp_full, j & 1, abort_flag, status, 3305)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tS = (j & 1) ? tS1 : tS0;
      const int kbase = j * 128;
      uint32_t rs[2][32], rd[2][32];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        tmem_ld_32x32(tS + lane_off + (half * 2 + cc) * 32, rs[cc]);
        tmem_ld_32x32(tDP + lane_off + (half * 2 + cc) * 32, rd[cc]);
      }
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(dp_empty);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        uint32_t wd[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float ds[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const bool vis = kbase + c * 32 + i + e < row_limit;
            const float p = vis ? ex2(__uint_as_float(rs[cc][i + e]) * scale_log2 - lse2) : 0.f;
            ds[e] = p * (__uint_as_float(rd[cc][i + e]) - dl);
          }
          wd[i >> 1] = pack_bf16x2(ds[0], ds[1]);
        }
        if (j > 0 && cc == 0) {   // dQ of the previous tile still reads the dS buffer until its MMAs complete
          if (!mbar_wait_bounded(dq_done, (j - 1) & 1, abort_flag, status, 3310)) { ok = false; break; }
        }
        store_row32_swz(sdS, row, c * 32, wd);
      }
      if (!ok) break;
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(ds_full);
    }
    if (ok && n_kv > 0) ok = mbar_wait_bounded(dq_done, (n_kv - 1) & 1, abort_flag, status, 3320);
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* qr = dQ + (int64_t)(q0 + row) * dq_stride + (int64_t)h * HD;
#pragma unroll 1
      for (int c = half * (HD / 64); c < (half + 1) * (HD / 64); ++c) {
        uint32_t r[32];
        if (n_kv > 0) {
          tmem_ld_32x32(tDQ + lane_off + c * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[8 * v]) * scale, __uint_as_float(r[8 * v + 1]) * scale);
            o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]) * scale, __uint_as_float(r[8 * v + 3]) * scale);
            o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]) * scale, __uint_as_float(r[8 * v + 5]) * scale);
            o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]) * scale, __uint_as_float(r[8 * v + 7]) * scale);
            reinterpret_cast<uint4*>(qr + c * 32)[v] = o;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace llmt

using namespace llmt;

extern "C" int llmt_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* tiles, int num_tiles,
                             int Tq, int Tk, int Hq, int Hkv, int HD, int64_t q_stride, int64_t k_stride, int64_t v_stride,
                             int64_t o_stride, float scale, int causal, int* status, cudaStream_t st) {
  if (num_tiles <= 0 || Hq <= 0) return 0;
  if ((HD != 64 && HD != 128 && HD != 256) || Hq % Hkv || (q_stride & 7) || (k_stride & 7) || (v_stride & 7) || (o_stride & 7)) return -10;
  CUtensorMap tq, tk, tv;
  if (make_thd_map(&tq, q, Tq, Hq, HD, q_stride) || make_thd_map(&tk, k, Tk, Hkv, HD, k_stride, kFwdKV) ||
      make_thd_map(&tv, v, Tk, Hkv, HD, v_stride, kFwdKV))
    return -11;
  const int smem = 128 * HD * 2 + 3 * kFwdKV * HD * 2 + 2 * 128 * kFwdKV * 2 + 256;   // exact: no alignment slack, see the kernel
  const float sl2 = scale * kLog2e;
  if (HD == 256) {
    static bool cfg = false;
    if (!cfg) { if (set_smem(attn_fwd_kernel<256>, smem)) return -2; cfg = true; }
    attn_fwd_kernel<256><<<num_tiles * Hq, kAttnThreads, smem, st>>>(tq, tk, tv, (__nv_bfloat16*)o, lse, tiles, Hq, Hkv, Tq,
                                                                     o_stride, sl2, causal, status);
  } else if (HD == 128) {
    static bool cfg = false;
    if (!cfg) { if (set_smem(attn_fwd_kernel<128>, smem)) return -2; cfg = true; }
    attn_fwd_kernel<128><<<num_tiles * Hq, kAttnThreads, smem, st>>>(tq, tk, tv, (__nv_bfloat16*)o, lse, tiles, Hq, Hkv, Tq,
                                                                     o_stride, sl2, causal, status);
  } else {
    static bool cfg = false;
    if (!cfg) { if (set_smem(attn_fwd_kernel<64>, smem)) return -2; cfg = true; }
    attn_fwd_kernel<64><<<num_tiles * Hq, kAttnThreads, smem, st>>>(tq, tk, tv, (__nv_bfloat16*)o, lse, tiles, Hq, Hkv, Tq,
                                                                    o_stride, sl2, causal, status);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int llmt_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                             float* delta, void* dq, void* dk, void* dv, const int* q_tiles, int num_q_tiles,
                             const int* k_tiles, int num_k_tiles, int Tq, int Tk, int Hq, int Hkv, int HD, int64_t q_stride,
                             int64_t k_stride, int64_t v_stride, int64_t o_stride, int64_t do_stride, int64_t dq_stride,
                             int64_t dk_stride, int64_t dv_stride, float scale, int causal, int pass, int* status, cudaStream_t st) {
  // pass 0: delta, dK/dV (overwrite), dQ. pass > 0: only dK/dV over another k-tile table, accumulating into dK/dV.
  if (Hq <= 0 || Tq <= 0) return 0;
  if ((HD != 64 && HD != 128) || Hq % Hkv || (q_stride & 7) || (k_stride & 7) || (v_stride & 7) || (do_stride & 7) ||
      (dq_stride & 7) || (dk_stride & 7) || (dv_stride & 7))
    return -10;
  if (pass == 0) {
    const int64_t items = (int64_t)Tq * Hq;
    attn_delta_kernel<<<(int)((items + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)o, o_stride, (const __nv_bfloat16*)dout,
                                                              do_stride, delta, Tq, Hq, HD);
  }
  CUtensorMap tq, tk, tv, tdo;
  if (make_thd_map(&tq, q, Tq, Hq, HD, q_stride) || make_thd_map(&tk, k, Tk, Hkv, HD, k_stride) ||
      make_thd_map(&tv, v, Tk, Hkv, HD, v_stride) || make_thd_map(&tdo, dout, Tq, Hq, HD, do_stride))
    return -11;
  CUtensorMap tq64, tdo64;   // 64-row boxes for the dK/dV kernel's q tiles
  if (make_thd_map(&tq64, q, Tq, Hq, HD, q_stride, kBwdQ) || make_thd_map(&tdo64, dout, Tq, Hq, HD, do_stride, kBwdQ)) return -11;
  const int smem_kv = 2 * 128 * HD * 2 + 2 * kBwdQStages * kBwdQ * HD * 2 + 4 * 128 * kBwdQ * 2 + 4 * kBwdQ * 4 + 1024 + 256;
  const int smem_q = 6 * 128 * HD * 2 + 128 * 128 * 2 + 1024 + 256;
  if (HD == 128) {
    static bool cfg = false;
    if (!cfg) {
      if (set_smem(attn_bwd_dkv_kernel<128>, smem_kv) || set_smem(attn_bwd_dq_kernel<128>, smem_q)) return -2;
      cfg = true;
    }
    if (num_k_tiles > 0)
      attn_bwd_dkv_kernel<128><<<num_k_tiles * Hkv, kBwdThreads, smem_kv, st>>>(
          tq64, tk, tv, tdo64, lse, delta, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, k_tiles, Hq, Hkv, Tq, dk_stride, dv_stride, scale,
          causal, pass > 0, status);
    if (num_q_tiles > 0 && pass == 0)
      attn_bwd_dq_kernel<128><<<num_q_tiles * Hq, kBwdThreads, smem_q, st>>>(tq, tk, tv, tdo, lse, delta, (__nv_bfloat16*)dq,
                                                                              q_tiles, Hq, Hkv, Tq, dq_stride, scale, causal,
                                                                              status);
  } else {
    static bool cfg = false;
    if (!cfg) {
      if (set_smem(attn_bwd_dkv_kernel<64>, smem_kv) || set_smem(attn_bwd_dq_kernel<64>, smem_q)) return -2;
      cfg = true;
    }
    if (num_k_tiles > 0)
      attn_bwd_dkv_kernel<64><<<num_k_tiles * Hkv, kBwdThreads, smem_kv, st>>>(
          tq64, tk, tv, tdo64, lse, delta, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, k_tiles, Hq, Hkv, Tq, dk_stride, dv_stride, scale,
          causal, pass > 0, status);
    if (num_q_tiles > 0 && pass == 0)
      attn_bwd_dq_kernel<64><<<num_q_tiles * Hq, kBwdThreads, smem_q, st>>>(tq, tk, tv, tdo, lse, delta, (__nv_bfloat16*)dq,
                                                                             q_tiles, Hq, Hkv, Tq, dq_stride, scale, causal,
                                                                             status);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
