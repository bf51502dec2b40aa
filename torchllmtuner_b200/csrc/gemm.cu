// Persistent bf16 GEMM for sm_100a: TMA -> shared memory (128B swizzle) -> tcgen05.mma with the fp32
// accumulator in TMEM -> tcgen05.ld epilogue. One kernel covers the three products of a linear layer
// (reference call sites: llmtuner/models/qwen/qwen3/model.py:255-268 via nn.Linear, and the packed
// expert products of llmtuner/models/common/moe/experts.py:206-209,268 via torch._grouped_mm):
//   forward  y  = x  * W^T   A K-major,  B K-major
//   dgrad    dx = dy * W     A K-major,  B MN-major
//   wgrad    dW = dy^T * x   A MN-major, B MN-major
// so no operand is ever transposed in memory. The grouped form runs the same tiles over row segments
// of A (one per expert, 128-row aligned) against a stack of B matrices.
//
// CTA = 6 warps: warp 0 issues TMA, warp 1 owns TMEM and issues MMAs, warps 2-5 drain the accumulator.
// The accumulator is double buffered in TMEM so the epilogue of tile i overlaps the MMAs of tile i+1.
#include "comm.cuh"
#include "kernels.h"

namespace llmt {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int kGemmThreads = 192;                       // TMA warp, MMA warp, 4 epilogue warps
constexpr int kGemmThreadsComm = 192 + kCommThreads;   // plus the comm warps that carry a SideJob

template <int BN>
struct GemmCfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;  // two accumulators
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align slack*/ + 256 /*barriers*/;
};

struct GroupedArgs {
  const int* seg_offsets;  // [G+1] row offsets into A / C, each a multiple of BM; nullptr = plain GEMM
  int num_groups;
};

template <int BN, bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM, int MODE>
__global__ void __launch_bounds__(kGemmThreadsComm, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    void* __restrict__ Cptr, int M, int N, int K, int64_t ldc, GroupedArgs grp, SideJob side, TPFuse tp, int* status) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + Cfg::kStages;
  uint64_t* tfull = bars + 2 * Cfg::kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* comm_word = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Tile enumeration. Plain: tile -> (m = t % num_m, n = t / num_m). Grouped: m tiles walk the 128-row
  // aligned segments; the segment index selects the B matrix (third TMA coordinate).
  // MODE 0: plain. MODE 1: rows of A/C are 128-aligned segments, segment g uses B[g] (third TMA coordinate).
  // MODE 2: one M x N product per segment, reduced over that segment's rows (the K dimension); C[g] is M x N.
  constexpr bool GROUPED = (MODE == 1);
  const int num_n = (N + BN - 1) / BN;
  // MODE 1: M is the capacity of the padded row buffer (a multiple of BM); only the tiles below the last segment's end
  // hold rows, the rest of a statically sized buffer is skipped.
  int num_m = (M + BM - 1) / BM;
  if constexpr (MODE == 1) {
    const int used = grp.seg_offsets[grp.num_groups] / BM;
    num_m = used < num_m ? used : num_m;
  }
  const int tiles_per_group = num_m * num_n;
  const int num_tiles = (MODE == 2) ? tiles_per_group * grp.num_groups : tiles_per_group;
  const int num_kb_plain = (K + BK - 1) / BK;
  auto kb_range = [&](int t, int& k_begin) -> int {
    if constexpr (MODE == 2) {
      const int g = t / tiles_per_group;
      k_begin = grp.seg_offsets[g];
      return (grp.seg_offsets[g + 1] - k_begin + BK - 1) / BK;
    } else {
      k_begin = 0;
      return num_kb_plain;
    }
  };

  // Tile order inside one M x N problem: super-rows of kGroupM m-tiles are swept column by column, so the CTAs that
  // run concurrently cover a near-square patch (A and B tiles are both reused out of L2).
  constexpr int kGroupM = 16;
  // With a fused tensor-parallel collective (MODE 0 only) the rows are walked chunk by chunk instead: the all-gather
  // form starts with this rank's own chunk, the reduce-scatter form ends with it.
  const bool tp_on = (MODE == 0) && tp.mode != kTPNone;
  const int tp_mpc = tp_on ? tp.chunk_rows / BM : 1;
  const int tp_tpc = tp_mpc * num_n;
  auto tp_chunk_of = [&](int tt) -> int { return (tp.rank + tt / tp_tpc + (tp.mode == kTPReduceScatter ? 1 : 0)) % tp.world; };
  auto tile_mn = [&](int tt, int& m0, int& n0) {
    if (tp_on) {   // the same super-row sweep, inside one chunk
      const int w = tt % tp_tpc;
      const int per_group = kGroupM * num_n;
      const int grp_i = w / per_group;
      const int first_m = grp_i * kGroupM;
      const int gm = (tp_mpc - first_m < kGroupM) ? (tp_mpc - first_m) : kGroupM;
      const int r = w - grp_i * per_group;
      m0 = (tp_chunk_of(tt) * tp_mpc + first_m + r % gm) * BM;
      n0 = (r / gm) * BN;
      return;
    }
    const int per_group = kGroupM * num_n;
    const int grp_i = tt / per_group;
    const int first_m = grp_i * kGroupM;
    const int gm = (num_m - first_m < kGroupM) ? (num_m - first_m) : kGroupM;
    const int r = tt - grp_i * per_group;
    m0 = (first_m + r % gm) * BM;
    n0 = (r / gm) * BN;
  };

  auto group_of_row = [&](int row) -> int {
    // segments are few (<= a few hundred); linear scan by one thread per tile is negligible
    int g = 0;
    while (g + 1 < grp.num_groups && row >= grp.seg_offsets[g + 1]) ++g;
    return g;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed = 0, armed_parity = 0;  // per-stage bookkeeping for the abort drain
      bool ok = true;
      int landed_chunk = -1;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m0, n0;
        tile_mn(t % tiles_per_group, m0, n0);
        if (tp_on && tp.mode == kTPAllGather) {
          const int c = tp_chunk_of(t);
          if (c != landed_chunk) {
            if (!tp_wait_landed(tp, c, abort_flag, status)) break;
            landed_chunk = c;
          }
        }
        int g = 0;
        if constexpr (GROUPED) g = group_of_row(m0);
        int k_begin;
        const int num_kb = kb_range(t, k_begin);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty[stage], phase ^ 1, abort_flag, status, 100 + stage)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_arrive_expect_tx(&full[stage], Cfg::kStageBytes);
          armed |= 1u << stage;
          armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
          const int k0 = k_begin + kb * BK;
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmA, &full[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (BK * 128), &tmA, &full[stage], m0 + 64 * j, k0);
          }
          if constexpr (!B_MN) {
            if constexpr (GROUPED) tma_load_3d(sb, &tmB, &full[stage], k0, n0, g);
            else tma_load_2d(sb, &tmB, &full[stage], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) {
              if constexpr (GROUPED) tma_load_3d(sb + j * (BK * 128), &tmB, &full[stage], n0 + 64 * j, k0, g);
              else tma_load_2d(sb + j * (BK * 128), &tmB, &full[stage], n0 + 64 * j, k0);
            }
          }
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (*abort_flag) {
        // Let copies that are still in flight land before this CTA's shared memory is released.
        for (int s = 0; s < Cfg::kStages; ++s) {
          if (!(armed & (1u << s))) continue;
          const uint32_t par = (armed_parity >> s) & 1u;
          for (uint32_t i = 0; i < (1u << 16); ++i)
            if (mbar_try_wait(&full[s], par)) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait_bounded(&tempty[acc], acc_phase ^ 1, abort_flag, status, 200 + acc)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        int k_begin;
        const int num_kb = kb_range(t, k_begin);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full[stage], phase, abort_flag, status, 300 + stage)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kABytes;
          const uint32_t la = desc_lo(sa, A_MN ? BK * 128 : 16), lb = desc_lo(sb, B_MN ? BK * 128 : 16);
          const uint32_t acc0 = kb ? 1u : 0u;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = desc_pack(la + (A_MN ? k * 128 : k * 2));
            const uint64_t db = desc_pack(lb + (B_MN ? k * 128 : k * 2));
            umma_bf16_ss(d_tmem, da, db, idesc, k ? 1u : acc0);
          }
          umma_commit(&empty[stage]);  // frees the stage once these MMAs have read it
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ comm warps (only launched with a SideJob)
    if (tp_on) {
      if (tp.mode == kTPAllGather) tp_allgather_comm(tp, threadIdx.x - 192, comm_word, status);
      else tp_reducescatter_comm(tp, threadIdx.x - 192, comm_word, status);
    } else {
      run_side_job(side, (long long)blockIdx.x * kCommThreads + (threadIdx.x - 192), (long long)gridDim.x * kCommThreads, status);
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int m0, n0;
      tile_mn(t % tiles_per_group, m0, n0);
      const int row_limit = M;  // MODE 1: padded rows are written too (their inputs are zero)
      int k_begin;
      const bool empty_k = kb_range(t, k_begin) == 0;  // MODE 2 segment without rows: the product is zero
      const int64_t c_base = (MODE == 2) ? (int64_t)(t / tiles_per_group) * M * ldc : 0;
      if (!mbar_wait_bounded(&tfull[acc], acc_phase, abort_flag, status, 400 + acc)) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_wait_ld();
        if (empty_k) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        const int col0 = n0 + c * 32;
        if (row < row_limit && col0 < N) {
          if constexpr (OUT_F32) {
            float* dst = reinterpret_cast<float*>(Cptr) + c_base + (int64_t)row * ldc + col0;
            if (col0 + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                       __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                if constexpr (ACCUM) {
                  const float4 p = reinterpret_cast<float4*>(dst)[v];
                  o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                }
                reinterpret_cast<float4*>(dst)[v] = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j) {
                float o = __uint_as_float(r[j]);
                if constexpr (ACCUM) o += dst[j];
                dst[j] = o;
              }
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cptr) + c_base + (int64_t)row * ldc + col0;
            if (col0 + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[8 * v + j]);
                if constexpr (ACCUM) {
                  const uint4 p = reinterpret_cast<const uint4*>(dst)[v];
                  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&p);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 pf = __bfloat1622float2(pb[j]);
                    f[2 * j] += pf.x;
                    f[2 * j + 1] += pf.y;
                  }
                }
                uint4 o;
                o.x = pack_bf16x2(f[0], f[1]);
                o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]);
                o.w = pack_bf16x2(f[6], f[7]);
                reinterpret_cast<uint4*>(dst)[v] = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j) {
                float o = __uint_as_float(r[j]);
                if constexpr (ACCUM) o += __bfloat162float(dst[j]);
                dst[j] = __float2bfloat16_rn(o);
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tempty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      if (tp_on && tp.mode == kTPReduceScatter) tp_tile_done(tp, tp_chunk_of(t), (uint32_t)tp_tpc * 4u, lane);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return (EncodeTiledFn) nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// bf16 tensor map with a 128-byte swizzle. dims/strides are innermost-first; strides in bytes for dims 1..rank-1.
int make_tmap_typed(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box, int is_f32);
int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                   const uint32_t* box) {
  return make_tmap_typed(out, base, rank, dims, strides_bytes, box, 0);
}
// Same for fp32 elements when `is_f32` (inner box of at most 32 elements = one 128-byte swizzle row).
int make_tmap_typed(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box, int is_f32) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  // The encoder is a driver call and needs the primary context bound to the calling thread; a fresh thread (the
  // autograd engine's) has none until its first runtime call.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = enc(out, is_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (r == CUDA_SUCCESS) ? 0 : (int)r;
}

int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

template <int BN, bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM, int MODE>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, int64_t ldc, GroupedArgs grp,
                  int* status, int max_ctas, cudaStream_t stream, const SideJob* side = nullptr, const TPFuse* tpf = nullptr) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_tcgen05_kernel<BN, A_MN, B_MN, OUT_F32, ACCUM, MODE>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) return -2;
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * (MODE == 2 ? grp.num_groups : 1);
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid < 1) return 0;
  SideJob none{};
  TPFuse no_tp{};
  const bool with_tp = tpf != nullptr && tpf->mode != kTPNone;
  const bool with_side = (side != nullptr && side->kind != kSideNone) || with_tp;
  if (with_side && max_ctas <= 0) grid = sm_count();   // every SM carries comm warps, even past the last tile
  kern<<<grid, with_side ? kGemmThreadsComm : kGemmThreads, Cfg::kSmemBytes, stream>>>(
      ta, tb, C, M, N, K, ldc, grp, (side != nullptr && !with_tp) ? *side : none, with_tp ? *tpf : no_tp, status);
  return (cudaGetLastError() == cudaSuccess) ? 0 : -3;
}

template <int BN>
static int dispatch_plain(bool a_mn, bool b_mn, bool out_f32, bool accum, const CUtensorMap& ta, const CUtensorMap& tb,
                          void* C, int M, int N, int K, int64_t ldc, int* status, int max_ctas, cudaStream_t s,
                          const SideJob* side, const TPFuse* tpf = nullptr) {
  GroupedArgs grp{nullptr, 0};
#define LLMT_CASE(AM, BMN, F32, ACC)                                                            \
  if (a_mn == AM && b_mn == BMN && out_f32 == F32 && accum == ACC)                              \
    return launch<BN, AM, BMN, F32, ACC, 0>(ta, tb, C, M, N, K, ldc, grp, status, max_ctas, s, side, tpf);
  LLMT_CASE(false, false, false, false)
  LLMT_CASE(false, false, true, false)
  LLMT_CASE(false, true, false, false)
  LLMT_CASE(false, true, true, false)
  LLMT_CASE(false, true, false, true)
  LLMT_CASE(true, true, false, false)
  LLMT_CASE(true, true, true, false)
  LLMT_CASE(true, true, false, true)
  LLMT_CASE(true, true, true, true)
#undef LLMT_CASE
  return -4;  // combination not instantiated
}

}  // namespace llmt

using namespace llmt;

// C[M,N] (+)= A * B with bf16 inputs and fp32 accumulation.
//   a_mn == 0: A stored [M][K] (row stride lda elements); a_mn == 1: A stored [K][M].
//   b_mn == 0: B stored [N][K] (row stride ldb);          b_mn == 1: B stored [K][N].
// Requirements: base pointers 16-byte aligned, lda/ldb multiples of 8 elements.
static int gemm_impl(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int a_mn,
                     int b_mn, int out_f32, int accumulate, int* status, int max_ctas, cudaStream_t stream, const SideJob* side,
                     const TPFuse* tpf = nullptr) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -10;
  const bool bn256 = N > 128;
  const uint32_t bn = bn256 ? 256 : 128;
  CUtensorMap ta, tb;
  {
    uint64_t dims[2], str[1];
    uint32_t box[2];
    if (!a_mn) { dims[0] = K; dims[1] = M; box[0] = 64; box[1] = BM; }
    else       { dims[0] = M; dims[1] = K; box[0] = 64; box[1] = BK; }
    str[0] = (uint64_t)lda * 2;
    if (int rc = make_tmap_bf16(&ta, A, 2, dims, str, box)) return -1100 - rc;
    if (!b_mn) { dims[0] = K; dims[1] = N; box[0] = 64; box[1] = bn; }
    else       { dims[0] = N; dims[1] = K; box[0] = 64; box[1] = BK; }
    str[0] = (uint64_t)ldb * 2;
    if (make_tmap_bf16(&tb, B, 2, dims, str, box)) return -12;
  }
  if (bn256) return dispatch_plain<256>(a_mn, b_mn, out_f32, accumulate, ta, tb, C, M, N, K, ldc, status, max_ctas, stream, side, tpf);
  return dispatch_plain<128>(a_mn, b_mn, out_f32, accumulate, ta, tb, C, M, N, K, ldc, status, max_ctas, stream, side, tpf);
}

extern "C" int llmt_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                              int64_t ldc, int a_mn, int b_mn, int out_f32, int accumulate, int* status, int max_ctas,
                              cudaStream_t stream) {
  return gemm_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_f32, accumulate, status, max_ctas, stream, nullptr);
}

// Same product, with a slice of a peer-memory collective carried by the comm warps of every CTA (see comm.cuh).
extern "C" int llmt_gemm_bf16_fused(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                                    int64_t ldc, int a_mn, int b_mn, int out_f32, int accumulate, int job_kind, int job_nsrc,
                                    const void* const* job_src, void* job_dst, long long job_n, int job_accumulate,
                                    const uint32_t* wait_flags, int n_wait, uint32_t wait_value, int* status,
                                    cudaStream_t stream) {
  SideJob j{};
  j.kind = job_kind;
  j.nsrc = job_nsrc;
  for (int i = 0; i < kMaxPeers; ++i) j.src[i] = (i < job_nsrc) ? job_src[i] : nullptr;
  j.dst = job_dst;
  j.n = job_n;
  j.accumulate = job_accumulate;
  j.wait_flags = wait_flags;
  j.n_wait = n_wait;
  j.wait_value = wait_value;
  if (job_kind != kSideNone && (job_nsrc < 1 || job_nsrc > kMaxPeers)) return -10;
  return gemm_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_f32, accumulate, status, 0, stream, &j);
}

// Tensor-parallel fused forms (see comm.cuh). mode 1: C[M,N] = gather(A) * B where `A` is the local gathered matrix
// [M,K] that the comm warps fill from `peer_src` (every rank's chunk); mode 2: `C` is this rank's symmetric bf16 partial
// matrix [M,N] (ldc == N), `out` [M/world, N] receives the reduced chunk (+ residual). A is row-major in both.
// `accumulate` (only with b_mn) adds the product to what C already holds before the partial is published.
extern "C" int llmt_gemm_bf16_tp(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                                 int64_t ldc, int b_mn, int accumulate, int mode, int world, int rank, uint32_t epoch,
                                 const void* const* peer_src, const uint32_t* flags, uint32_t* const* peer_flags,
                                 uint32_t* counters, float* acc, void* out, const void* residual, int* status,
                                 cudaStream_t stream) {
  if (world < 2 || world > kMaxPeers || rank < 0 || rank >= world || M % world) return -10;
  const int chunk_rows = M / world;
  if (chunk_rows % BM || (mode != kTPAllGather && mode != kTPReduceScatter)) return -10;
  if (mode == kTPReduceScatter && (ldc != N || (N & 7))) return -10;
  if (mode == kTPAllGather && lda != K) return -10;
  TPFuse t{};
  t.mode = mode; t.world = world; t.rank = rank; t.chunk_rows = chunk_rows; t.epoch = epoch;
  for (int i = 0; i < world; ++i) { t.peer_src[i] = peer_src[i]; t.peer_flags[i] = peer_flags[i]; }
  t.local_dst = const_cast<void*>(A);
  t.chunk_bytes = (long long)chunk_rows * K * 2;
  t.flags = flags; t.counters = counters;
  t.acc = acc; t.out = reinterpret_cast<__nv_bfloat16*>(out); t.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  t.n_cols = N;
  return gemm_impl(A, B, C, M, N, K, lda, ldb, ldc, 0, b_mn, 0, accumulate, status, 0, stream, nullptr, &t);
}

// Grouped forward/dgrad: rows of A (and C) are cut into `num_groups` segments at seg_offsets (device int32,
// [G+1], multiples of 128, seg_offsets[G] == M_padded); segment g multiplies B[g].
//   b_mn == 0: B stored [G][N][K];  b_mn == 1: B stored [G][K][N].
extern "C" int llmt_grouped_gemm_bf16(const void* A, const void* B, void* C, const int* seg_offsets, int num_groups,
                                      int M_padded, int N, int K, int64_t lda, int64_t ldc, int b_mn, int out_f32,
                                      int* status, cudaStream_t stream) {
  if (M_padded <= 0 || N <= 0 || num_groups <= 0) return 0;
  if (K <= 0 || (lda & 7) || (M_padded % BM)) return -10;
  const bool bn256 = N > 128;
  const uint32_t bn = bn256 ? 256 : 128;
  CUtensorMap ta, tb;
  {
    uint64_t dims[3], str[2];
    uint32_t box[3];
    dims[0] = K; dims[1] = M_padded; box[0] = 64; box[1] = BM;
    str[0] = (uint64_t)lda * 2;
    if (int rc = make_tmap_bf16(&ta, A, 2, dims, str, box)) return -1100 - rc;
    if (!b_mn) { dims[0] = K; dims[1] = N; box[0] = 64; box[1] = bn; str[0] = (uint64_t)K * 2; }
    else       { dims[0] = N; dims[1] = K; box[0] = 64; box[1] = BK; str[0] = (uint64_t)N * 2; }
    dims[2] = num_groups; box[2] = 1;
    str[1] = (uint64_t)N * K * 2;
    if (make_tmap_bf16(&tb, B, 3, dims, str, box)) return -12;
  }
  GroupedArgs grp{seg_offsets, num_groups};
  if (out_f32) return -4;
  if (bn256) {
    if (b_mn) return launch<256, false, true, false, false, 1>(ta, tb, C, M_padded, N, K, ldc, grp, status, 0, stream);
    return launch<256, false, false, false, false, 1>(ta, tb, C, M_padded, N, K, ldc, grp, status, 0, stream);
  }
  if (b_mn) return launch<128, false, true, false, false, 1>(ta, tb, C, M_padded, N, K, ldc, grp, status, 0, stream);
  return launch<128, false, false, false, false, 1>(ta, tb, C, M_padded, N, K, ldc, grp, status, 0, stream);
}

// Grouped wgrad: C[g] (M x N, row stride N) (+)= A_g^T * B_g where A is stored [rows][M], B is stored [rows][N] and
// segment g covers rows [seg_offsets[g], seg_offsets[g+1]) (multiples of 128; padded rows must hold zeros).
extern "C" int llmt_grouped_wgrad_bf16(const void* A, const void* B, void* C, const int* seg_offsets, int num_groups,
                                       int rows_padded, int M, int N, int64_t lda, int64_t ldb, int out_f32,
                                       int accumulate, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || num_groups <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (rows_padded % BM) || rows_padded <= 0) return -10;
  const bool bn256 = N > 128;
  CUtensorMap ta, tb;
  {
    uint64_t dims[2], str[1];
    uint32_t box[2];
    dims[0] = M; dims[1] = rows_padded; box[0] = 64; box[1] = BK; str[0] = (uint64_t)lda * 2;
    if (int rc = make_tmap_bf16(&ta, A, 2, dims, str, box)) return -1100 - rc;
    dims[0] = N; dims[1] = rows_padded; box[0] = 64; box[1] = BK; str[0] = (uint64_t)ldb * 2;
    if (make_tmap_bf16(&tb, B, 2, dims, str, box)) return -12;
  }
  GroupedArgs grp{seg_offsets, num_groups};
  const int K = rows_padded;
#define LLMT_W(BNV, F32, ACC) \
  if (bn256 == (BNV == 256) && (bool)out_f32 == F32 && (bool)accumulate == ACC) \
    return launch<BNV, true, true, F32, ACC, 2>(ta, tb, C, M, N, K, (int64_t)N, grp, status, 0, stream);
  LLMT_W(256, false, false) LLMT_W(256, true, false) LLMT_W(256, false, true) LLMT_W(256, true, true)
  LLMT_W(128, false, false) LLMT_W(128, true, false) LLMT_W(128, false, true) LLMT_W(128, true, true)
#undef LLMT_W
  return -4;
}
