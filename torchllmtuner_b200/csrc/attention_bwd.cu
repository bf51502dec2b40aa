// Single-kernel flash-attention backward for sm_100a (tcgen05 / TMEM): dK, dV and dQ from five products per tile pair.
// (reference call sites: the backward of llmtuner/models/qwen/qwen3/model.py:270-283 and of
//  llmtuner/kernel/ops/varlen_attention.py:60-85, which the reference leaves to the attention library.)
//
// One CTA per (128-key tile, kv head). It walks the query heads of the group and their 128-row query tiles:
//   S^T  = K Q^T          (keys in TMEM lanes, queries in columns), issued as two 64-query halves a, b
//   dP^T = V dO^T
//   P^T  = exp2(S^T * c - lse)            written back over S^T as packed bf16: the A operand of the next product
//   dV  += P^T dO                         A from tensor memory, per half
//   dS^T = P^T o (dP^T - delta)           bf16, through shared memory
//   dQ   = dS K                           the shared tile read MN-major; lands in the columns dP^T occupied
//   dK  += dS^T Q
// dV and dK stay in TMEM for the whole walk. Each dQ tile is scaled, staged through swizzled shared memory in 32-column
// slices and added into an fp32 [Tq, Hq, HD] accumulator with bulk tensor reduce-adds; `attn_dq_cast_kernel` turns the
// accumulator into bf16 afterwards. The order in which key tiles reach the accumulator is not fixed, so dQ is
// reproducible only up to fp32 summation order; the two-kernel backward in attention.cu is the bitwise-reproducible one.
//
// Tensor memory holds S^T, dP^T, dV and dK (512 columns), so S^T has one buffer. The half split keeps both sides busy:
// while the softmax warps turn half b of tile i into P^T, the tensor pipe consumes half a (dV += P_a^T dO_a) and already
// refills it with S_a^T of tile i+1. The softmax warps keep P as packed bf16 between the two passes and use the packed
// two-lane fp32 instructions for the scale / subtract / multiply steps.
//
// Warps: 0 TMA producer, 1 MMA issuer (+ TMEM allocation), 2-9 softmax / dS math (two per TMEM lane quarter, each takes
// 32 of the 64 query columns of a half), 10-13 dQ read-out and reduce. Every wait is bounded and reports through the
// status word.
#include "attn_common.cuh"

namespace llmt {

constexpr int kFusedThreads = 64 + 256 + 128;

// Packed two-lane fp32 arithmetic (one issue slot for two elements).
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  uint64_t ra, rb, rc, rd;
  float2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.ftz.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  uint64_t ra, rb, rd;
  float2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("add.rn.ftz.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  uint64_t ra, rb, rd;
  float2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mul.rn.ftz.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
constexpr int kStageBytes = 128 * 32 * 4;   // one 32-column fp32 slice of a dQ tile

template <int HD>
__global__ void __launch_bounds__(kFusedThreads, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                      const __grid_constant__ CUtensorMap tmdQ, const float* __restrict__ lse,
                      const float* __restrict__ delta, __nv_bfloat16* __restrict__ dK, __nv_bfloat16* __restrict__ dV,
                      const int* __restrict__ tiles, int Hq, int Hkv, int Tq, int64_t dk_stride, int64_t dv_stride,
                      float scale, int causal, int accumulate, int* status) {
  constexpr int NH = HD / 64;
  constexpr int kTile = 128 * HD * 2;
  constexpr int kDS = 128 * 128 * 2;
  // The launch asks for exactly the bytes used, so the dynamic shared memory base has to be 1024-byte aligned already;
  // the kernel refuses to run otherwise instead of overrunning its allocation.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) report_status(status, kStatusBadArgument, 4001, (int)(smem_u32(smem_raw) & 1023u));
    return;
  }
  uint8_t* sK = smem_raw;
  uint8_t* sV = sK + kTile;
  uint8_t* sQ = sV + kTile;          // 2 stages
  uint8_t* sdO = sQ + 2 * kTile;     // 1 stage
  uint8_t* sdS = sdO + kTile;        // [128 keys][128 queries] bf16, two 64-query halves
  uint8_t* sStage = sdS + kDS;       // 2 x 16 KB
  float* s_lse = reinterpret_cast<float*>(sStage + 2 * kStageBytes);   // [2][128]
  float* s_delta = s_lse + 2 * 128;                                     // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_delta + 2 * 128);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;      // [2]
  uint64_t* q_empty = bars + 3;     // [2]
  uint64_t* do_full = bars + 5;
  uint64_t* do_empty = bars + 6;
  uint64_t* s_full = bars + 7;      // [2]: halves a, b of S^T
  uint64_t* p_full = bars + 9;      // [2]
  uint64_t* dp_full = bars + 11;
  uint64_t* ds_full = bars + 12;
  uint64_t* ds_empty = bars + 13;
  uint64_t* dq_full = bars + 14;
  uint64_t* dq_empty = bars + 15;
  uint64_t* acc_done = bars + 16;
  uint64_t* stat_ready = bars + 17;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_idx = blockIdx.x / Hkv;
  const int hk = blockIdx.x % Hkv;
  const int g = Hq / Hkv;
  const int* tl = tiles + tile_idx * 8;
  const int k0 = tl[0], nk = tl[1], kk0 = tl[2], qbeg = tl[3], qlen = tl[4], off = tl[5], klen = tl[6];
  int qs = 0;
  if (causal) { qs = kk0 - off; if (qs < 0) qs = 0; qs &= ~127; }
  const int n_qt = (qlen > qs) ? (qlen - qs + 127) / 128 : 0;
  const int n_it = n_qt * g;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int b = 0; b < 2; ++b) { mbar_init(&q_full[b], 1); mbar_init(&q_empty[b], 1); }
    mbar_init(do_full, 1); mbar_init(do_empty, 1);
    for (int b = 0; b < 2; ++b) { mbar_init(&s_full[b], 1); mbar_init(&p_full[b], 256); }
    mbar_init(dp_full, 1); mbar_init(ds_full, 256); mbar_init(ds_empty, 1);
    mbar_init(dq_full, 1); mbar_init(dq_empty, 128); mbar_init(acc_done, 1); mbar_init(stat_ready, 256);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDV = tmem_base + 256, tDK = tmem_base + 256 + HD;

  if (warp == 0) {
    // ------------------------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_it > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
      mbar_arrive_expect_tx(kv_full, 2 * kTile);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
        tma_load_3d(sK + hf * 16384, &tmK, kv_full, hf * 64, hk, k0);
        tma_load_3d(sV + hf * 16384, &tmV, kv_full, hf * 64, hk, k0);
      }
      int armed_q[2] = {-1, -1}, armed_do = -1;
      for (int it = 0; it < n_it; ++it) {
        const int b = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int h = hk * g + it / n_qt;
        const int qrow = qbeg + qs + (it % n_qt) * 128;
        if (!mbar_wait_bounded(&q_empty[b], ph ^ 1, abort_flag, status, 4100 + b)) break;
        mbar_arrive_expect_tx(&q_full[b], kTile);
        armed_q[b] = (int)ph;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) tma_load_3d(sQ + b * kTile + hf * 16384, &tmQ, &q_full[b], hf * 64, h, qrow);
        if (!mbar_wait_bounded(do_empty, (it & 1) ^ 1, abort_flag, status, 4110)) break;
        mbar_arrive_expect_tx(do_full, kTile);
        armed_do = it & 1;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) tma_load_3d(sdO + hf * 16384, &tmdO, do_full, hf * 64, h, qrow);
      }
      if (*abort_flag) {
        // wait (bounded) for copies in flight before shared memory is released
        for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try_wait(kv_full, 0)) break;
        for (int b = 0; b < 2; ++b)
          if (armed_q[b] >= 0)
            for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try_wait(&q_full[b], (uint32_t)armed_q[b])) break;
        if (armed_do >= 0)
          for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try_wait(do_full, (uint32_t)armed_do)) break;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idS = umma_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idSh = umma_idesc_bf16(128, 64, false, false);
      constexpr uint32_t idAcc = umma_idesc_bf16(128, HD, false, true);
      constexpr uint32_t idDQ = umma_idesc_bf16(128, HD, true, true);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), adO = smem_u32(sdO), adS = smem_u32(sdS);
      const uint32_t loK = desc_lo(aK, 16), loV = desc_lo(aV, 16), loKm = desc_lo(aK, 16384);
      const uint32_t lodO = desc_lo(adO, 16), lodOm = desc_lo(adO, 16384);
      const uint32_t lodS = desc_lo(adS, 16), lodSm = desc_lo(adS, 16384);
      bool ok = mbar_wait_bounded(kv_full, 0, abort_flag, status, 4200);
      // S^T half hb (queries hb*64 .. +64) = K Q_hb^T; the half's 64 query rows sit 8192 B into each 64-column block of Q
      auto issue_S = [&](int it, int hb) -> bool {
        const int b = it & 1;
        if (hb == 0) {
          if (!mbar_wait_bounded(&q_full[b], (it >> 1) & 1, abort_flag, status, 4210 + b)) return false;
          tc_fence_after();
        }
        const uint32_t loQ = desc_lo(aQ + b * kTile + hb * 8192, 16);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma_bf16_ss(tS + hb * 64, desc_pack(loK + koff(ks, 128)), desc_pack(loQ + koff(ks, 128)), idSh, ks ? 1u : 0u);
        umma_commit(&s_full[hb]);
        return true;
      };
      auto issue_dP = [&](int it) -> bool {          // dP^T = V dO^T, into the columns the previous dQ tile has left
        if (!mbar_wait_bounded(do_full, it & 1, abort_flag, status, 4220)) return false;
        if (it > 0 && !mbar_wait_bounded(dq_empty, (it - 1) & 1, abort_flag, status, 4225)) return false;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma_bf16_ss(tDP, desc_pack(loV + koff(ks, 128)), desc_pack(lodO + koff(ks, 128)), idS, ks ? 1u : 0u);
        umma_commit(dp_full);
        return true;
      };
      if (ok) ok = issue_S(0, 0) && issue_S(0, 1) && issue_dP(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const int b = it & 1;
        const uint32_t acc0 = it ? 1u : 0u;
        const bool next = it + 1 < n_it;
        bool fail = false;
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          if (!mbar_wait_bounded(&p_full[hb], it & 1, abort_flag, status, 4230 + hb)) { fail = true; break; }
          tc_fence_after();
          // dV += P_hb^T dO_hb: 16-query slice ks of the half sits at column (ks >> 1) * 32 + (ks & 1) * 8 of the half
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_bf16_ts(tDV, tS + (uint32_t)(hb * 64 + (ks >> 1) * 32 + (ks & 1) * 8), desc_pack(lodOm + mnoff(hb * 4 + ks)), idAcc,
                         (hb | ks) ? 1u : acc0);
          if (hb == 1) umma_commit(do_empty);
          if (next && !issue_S(it + 1, hb)) { fail = true; break; }     // refill the half just consumed
        }
        if (fail) break;
        if (!mbar_wait_bounded(ds_full, it & 1, abort_flag, status, 4240)) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)                // dQ = dS K, first: its read-out gates the next dP^T product
          umma_bf16_ss(tDP, desc_pack(lodSm + mnoff(ks)), desc_pack(loKm + mnoff(ks)), idDQ, ks ? 1u : 0u);
        umma_commit(dq_full);
        const uint32_t loQm = desc_lo(aQ + b * kTile, 16384);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)                // dK += dS^T Q
          umma_bf16_ss(tDK, desc_pack(lodS + koff(ks, 128)), desc_pack(loQm + mnoff(ks)), idAcc, ks ? 1u : acc0);
        umma_commit(&q_empty[b]);
        umma_commit(ds_empty);
        if (it == n_it - 1) umma_commit(acc_done);
        if (next && !issue_dP(it + 1)) break;
      }
    }
    __syncwarp();
  } else if (warp < 10) {
    // ------------------------------------------------------------------------------------ softmax / dS math
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;   // key row inside the tile
    const int tid = threadIdx.x - 64;      // 0..255
    const int w2 = tid >> 7;               // which 32 of the 64 query columns of a half this thread handles
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const int key_idx = kk0 + row;
    const bool key_ok = (row < nk) && (key_idx < klen);
    const float2 c2 = make_float2(scale * kLog2e, scale * kLog2e);
    bool ok = true;
    // Row statistics of a query tile are fetched one iteration ahead: threads 0..127 carry minus the log-sum-exp (base 2)
    // of query tid, threads 128..255 minus the delta of query tid - 128.
    auto load_stat = [&](int it) -> float {
      const int h = hk * g + it / n_qt;
      const int qi = qs + (it % n_qt) * 128 + (tid & 127);
      const bool v = qi < qlen;
      if (tid < 128) return v ? -lse[(int64_t)h * Tq + qbeg + qi] * kLog2e : -INFINITY;
      return v ? -delta[(int64_t)h * Tq + qbeg + qi] : 0.f;
    };
    float* my_stat = (tid < 128) ? (s_lse + tid) : (s_delta + (tid - 128));
    if (n_it > 0) {
      my_stat[0] = load_stat(0);
      mbar_arrive(stat_ready);
    }
    for (int it = 0; it < n_it && ok; ++it) {
      const int sb = it & 1;
      const int qi0 = qs + (it % n_qt) * 128;
      const bool have_next = it + 1 < n_it;
      float next_stat = 0.f;
      if (have_next) next_stat = load_stat(it + 1);
      if (!mbar_wait_bounded(stat_ready, it & 1, abort_flag, status, 4330)) { ok = false; break; }
      // Most tiles lie wholly below the causal diagonal and inside the document: they skip the per-element visibility test.
      const bool tile_full = (nk == 128) && (kk0 + 128 <= klen) && (qi0 + 128 <= qlen) && (!causal || kk0 + 127 <= qi0 + off);
      uint32_t pk[32];   // P of this thread's 2 x 32 columns, packed bf16 pairs
      auto p_pass = [&](int hb, auto masked) {
        const int col0 = hb * 64 + w2 * 32;
        uint32_t rs[32];
        tmem_ld_32x32(tS + lane_off + col0, rs);
        tmem_wait_ld();
        const float4* pl4 = reinterpret_cast<const float4*>(s_lse + sb * 128 + col0);
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 l4 = pl4[i >> 2];
          const float2 x0 = ffma2(make_float2(__uint_as_float(rs[i]), __uint_as_float(rs[i + 1])), c2, make_float2(l4.x, l4.y));
          const float2 x1 = ffma2(make_float2(__uint_as_float(rs[i + 2]), __uint_as_float(rs[i + 3])), c2, make_float2(l4.z, l4.w));
          float p[4] = {ex2(x0.x), ex2(x0.y), ex2(x1.x), ex2(x1.y)};
          if constexpr (decltype(masked)::value) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int qi = qi0 + col0 + i + e;
              const bool vis = key_ok && (qi < qlen) && (!causal || key_idx <= qi + off);
              p[e] = vis ? p[e] : 0.f;
            }
          }
          pk[hb * 16 + (i >> 1)] = pack_bf16x2(p[0], p[1]);
          pk[hb * 16 + (i >> 1) + 1] = pack_bf16x2(p[2], p[3]);
        }
        // P^T of these 32 queries goes over the first 16 of the columns this thread has just read
        tmem_st_32x16(tS + lane_off + col0, pk + hb * 16);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&p_full[hb]);
      };
#pragma unroll
      for (int hb = 0; hb < 2; ++hb) {
        if (!mbar_wait_bounded(&s_full[hb], it & 1, abort_flag, status, 4300 + hb)) { ok = false; break; }
        tc_fence_after();
        if (tile_full) p_pass(hb, std::false_type{}); else p_pass(hb, std::true_type{});
      }
      if (!ok) break;
      if (!mbar_wait_bounded(dp_full, it & 1, abort_flag, status, 4310)) { ok = false; break; }
      if (it > 0 && !mbar_wait_bounded(ds_empty, (it - 1) & 1, abort_flag, status, 4315)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int hb = 0; hb < 2; ++hb) {
        const int col0 = hb * 64 + w2 * 32;
        uint32_t rd[32];
        tmem_ld_32x32(tDP + lane_off + col0, rd);
        tmem_wait_ld();
        const float4* pd4 = reinterpret_cast<const float4*>(s_delta + sb * 128 + col0);
        uint32_t wd[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 d4 = pd4[i >> 2];
          const uint32_t pa = pk[hb * 16 + (i >> 1)], pb = pk[hb * 16 + (i >> 1) + 1];
          const float2 p0 = make_float2(__uint_as_float(pa << 16), __uint_as_float(pa & 0xffff0000u));
          const float2 p1 = make_float2(__uint_as_float(pb << 16), __uint_as_float(pb & 0xffff0000u));
          const float2 e0 = fmul2(p0, fadd2(make_float2(__uint_as_float(rd[i]), __uint_as_float(rd[i + 1])), make_float2(d4.x, d4.y)));
          const float2 e1 = fmul2(p1, fadd2(make_float2(__uint_as_float(rd[i + 2]), __uint_as_float(rd[i + 3])), make_float2(d4.z, d4.w)));
          wd[i >> 1] = pack_bf16x2(e0.x, e0.y);
          wd[(i >> 1) + 1] = pack_bf16x2(e1.x, e1.y);
        }
        store_row32_swz(sdS, row, col0, wd);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(ds_full);
      if (have_next) {
        // every thread has passed this iteration's stat_ready wait, so nobody still reads the other buffer
        my_stat[(sb ^ 1) * 128] = next_stat;
        mbar_arrive(stat_ready);
      }
    }
    if (ok && n_it > 0) ok = mbar_wait_bounded(acc_done, 0, abort_flag, status, 4320);
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* kr = dK + (int64_t)(k0 + row) * dk_stride + (int64_t)hk * HD;
      __nv_bfloat16* vr = dV + (int64_t)(k0 + row) * dv_stride + (int64_t)hk * HD;
#pragma unroll 1
      for (int c = w2 * (HD / 64); c < (w2 + 1) * (HD / 64); ++c) {
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
  } else {
    // ------------------------------------------------------------------------------------ dQ read-out and reduce
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;   // query row inside the tile
    const int rt = threadIdx.x - 320;      // 0..127
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    bool ok = true;
    // Two 32-column slices (both staging buffers) are in flight at a time. The columns go back to the MMA warp as soon as
    // the last slice of the tile sits in registers, before its staging and reduce.
    auto wait_staging = [&]() {
      if (rt == 0) bulk_wait_read<0>();   // the reduces that last read the staging buffers have drained them
      named_bar_sync(1, 128);
    };
    auto stage_pair = [&](const uint32_t* r, int c0, int h, int qrow) {
#pragma unroll
      for (int s2 = 0; s2 < 2; ++s2) {
        uint8_t* st = sStage + s2 * kStageBytes;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 v = make_float4(__uint_as_float(r[s2 * 32 + 4 * j]) * scale, __uint_as_float(r[s2 * 32 + 4 * j + 1]) * scale,
                                 __uint_as_float(r[s2 * 32 + 4 * j + 2]) * scale, __uint_as_float(r[s2 * 32 + 4 * j + 3]) * scale);
          *reinterpret_cast<float4*>(st + row * 128 + ((j ^ (row & 7)) << 4)) = v;
        }
      }
      fence_proxy_async_smem();
      named_bar_sync(1, 128);
      if (rt == 0) {
        tma_reduce_add_3d(&tmdQ, sStage, c0 * 32, h, qrow);
        tma_reduce_add_3d(&tmdQ, sStage + kStageBytes, (c0 + 1) * 32, h, qrow);
        bulk_commit();
      }
    };
    for (int it = 0; it < n_it && ok; ++it) {
      const int h = hk * g + it / n_qt;
      const int qrow = qbeg + qs + (it % n_qt) * 128;
      wait_staging();
      if (!mbar_wait_bounded(dq_full, it & 1, abort_flag, status, 4400)) { ok = false; break; }
      tc_fence_after();
      uint32_t r[64];
      tmem_ld_32x32(tDP + lane_off, r);
      tmem_ld_32x32(tDP + lane_off + 32, r + 32);
      tmem_wait_ld();
      if (HD == 64) {
        tc_fence_before();
        mbar_arrive(dq_empty);       // the next dP^T product may overwrite these columns
      }
      stage_pair(r, 0, h, qrow);
      if (HD == 128) {
        tmem_ld_32x32(tDP + lane_off + 64, r);
        tmem_ld_32x32(tDP + lane_off + 96, r + 32);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(dq_empty);
        wait_staging();
        stage_pair(r, 2, h, qrow);
      }
    }
    if (rt == 0) bulk_wait<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// dq[t, h, :] (bf16, token stride dq_stride) = acc[t, h, :] (fp32, packed)
__global__ void attn_dq_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int64_t rows, int row_elems,
                                    int64_t dq_stride) {
  const int64_t n8 = rows * (row_elems / 8);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / (row_elems / 8);
    const int c = (int)(i % (row_elems / 8)) * 8;
    const float4 a = *reinterpret_cast<const float4*>(acc + t * row_elems + c);
    const float4 b = *reinterpret_cast<const float4*>(acc + t * row_elems + c + 4);
    uint4 o;
    o.x = pack_bf16x2(a.x, a.y); o.y = pack_bf16x2(a.z, a.w); o.z = pack_bf16x2(b.x, b.y); o.w = pack_bf16x2(b.z, b.w);
    *reinterpret_cast<uint4*>(dq + t * dq_stride + c) = o;
  }
}

int make_tmap_typed(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box, int is_f32);
int sm_count();

}  // namespace llmt

using namespace llmt;

// Single-kernel backward over one k-tile table. `first` runs the delta pre-pass and clears the fp32 dQ accumulator
// `dq_acc` [Tq, Hq, HD]; `last` casts the accumulator into `dq`. Passes after the first add into dK / dV.
extern "C" int llmt_attn_bwd_fused(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                                   float* delta, float* dq_acc, void* dq, void* dk, void* dv, const int* k_tiles,
                                   int num_k_tiles, int Tq, int Tk, int Hq, int Hkv, int HD, int64_t q_stride, int64_t k_stride,
                                   int64_t v_stride, int64_t o_stride, int64_t do_stride, int64_t dq_stride, int64_t dk_stride,
                                   int64_t dv_stride, float scale, int causal, int first, int last, int* status,
                                   cudaStream_t st) {
  if (Hq <= 0 || Tq <= 0) return 0;
  if ((HD != 64 && HD != 128) || Hq % Hkv || (q_stride & 7) || (k_stride & 7) || (v_stride & 7) || (do_stride & 7) ||
      (dq_stride & 7) || (dk_stride & 7) || (dv_stride & 7))
    return -10;
  if (first) {
    const int64_t items = (int64_t)Tq * Hq;
    attn_delta_kernel<<<(int)((items + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)o, o_stride, (const __nv_bfloat16*)dout,
                                                              do_stride, delta, Tq, Hq, HD);
    if (cudaMemsetAsync(dq_acc, 0, sizeof(float) * (size_t)Tq * Hq * HD, st) != cudaSuccess) return -3;
  }
  if (num_k_tiles > 0) {
    CUtensorMap tq, tk, tv, tdo, tdq;
    if (make_thd_map(&tq, q, Tq, Hq, HD, q_stride) || make_thd_map(&tk, k, Tk, Hkv, HD, k_stride) ||
        make_thd_map(&tv, v, Tk, Hkv, HD, v_stride) || make_thd_map(&tdo, dout, Tq, Hq, HD, do_stride))
      return -11;
    {
      uint64_t dims[3] = {(uint64_t)HD, (uint64_t)Hq, (uint64_t)Tq};
      uint64_t str[2] = {(uint64_t)HD * 4, (uint64_t)Hq * HD * 4};
      uint32_t box[3] = {32, 1, 128};
      if (make_tmap_typed(&tdq, dq_acc, 3, dims, str, box, 1)) return -11;
    }
    const int smem = 5 * 128 * HD * 2 + 128 * 128 * 2 + 2 * kStageBytes + 4 * 128 * 4 + 256;   // exact, see the kernel
    if (HD == 128) {
      static bool cfg = false;
      if (!cfg) { if (set_smem(attn_bwd_fused_kernel<128>, smem)) return -2; cfg = true; }
      attn_bwd_fused_kernel<128><<<num_k_tiles * Hkv, kFusedThreads, smem, st>>>(
          tq, tk, tv, tdo, tdq, lse, delta, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, k_tiles, Hq, Hkv, Tq, dk_stride, dv_stride,
          scale, causal, !first, status);
    } else {
      static bool cfg = false;
      if (!cfg) { if (set_smem(attn_bwd_fused_kernel<64>, smem)) return -2; cfg = true; }
      attn_bwd_fused_kernel<64><<<num_k_tiles * Hkv, kFusedThreads, smem, st>>>(
          tq, tk, tv, tdo, tdq, lse, delta, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, k_tiles, Hq, Hkv, Tq, dk_stride, dv_stride,
          scale, causal, !first, status);
    }
  }
  if (last) {
    const int64_t n8 = (int64_t)Tq * (Hq * HD / 8);
    const int blocks = (int)((n8 + 255) / 256 < (int64_t)sm_count() * 16 ? (n8 + 255) / 256 : (int64_t)sm_count() * 16);
    attn_dq_cast_kernel<<<blocks > 0 ? blocks : 1, 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dq, Tq, Hq * HD, dq_stride);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
