// Python bindings: thin tensor -> pointer adapters over the C entry points in kernels.h. All checks that can be
// done on the host (dtype, device, contiguity, alignment) are done here so the kernels can assume them.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "kernels.h"

namespace {

using torch::Tensor;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
}
// Number of kernels of this library launched so far (the caller-side count; each binding adds what it enqueues).
static int64_t g_launches = 0;
inline void check_rc(int rc, const char* what, int launches = 1) {
  TORCH_CHECK(rc == 0, what, " failed with code ", rc);
  g_launches += launches;
}

Tensor& status_word() {
  static Tensor s;
  if (!s.defined()) s = torch::zeros({8}, torch::dtype(torch::kInt32).device(torch::kCUDA));
  return s;
}
inline int* status_ptr() { return status_word().data_ptr<int>(); }

// Row-major 2-D view description of a tensor whose last dim is contiguous.
struct Mat {
  const void* ptr;
  int64_t rows, cols, ld;
};
inline Mat as_mat(const Tensor& t, const char* name) {
  check_bf16(t, name);
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, name, " must be 2-D with a contiguous last dim");
  return Mat{t.data_ptr(), t.size(0), t.size(1), t.stride(0)};
}

// A slice of a peer-memory collective handed to a kernel's comm warps (see csrc/comm.cuh). Pointers are raw device
// addresses (peers' symmetric buffers are not torch tensors on this rank).
struct PySideJob {
  int64_t kind = 0;                 // 0 none, 1 copy, 2 reduce
  std::vector<int64_t> src;         // device addresses
  int64_t dst = 0;
  int64_t n = 0;                    // copy: bytes; reduce: elements
  bool accumulate = false;
  int64_t wait_flags = 0;           // device address of the local flag array, 0 = no wait
  int64_t n_wait = 0;
  int64_t wait_value = 0;
};

// out[M,N] (+)= op(a) * op(b); layouts as in llmt_gemm_bf16. a_mn / b_mn say that the stored matrix is [K][M] / [K][N].
void gemm(const Tensor& a, const Tensor& b, Tensor& out, bool a_mn, bool b_mn, bool accumulate, int64_t max_ctas,
          const c10::optional<PySideJob>& side) {
  c10::cuda::CUDAGuard guard(a.device());
  const Mat A = as_mat(a, "a"), B = as_mat(b, "b");
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.stride(1) == 1, "out must be 2-D CUDA with contiguous last dim");
  const bool f32 = out.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || out.scalar_type() == at::kBFloat16, "out must be float32 or bfloat16");
  const int64_t M = a_mn ? A.cols : A.rows, K = a_mn ? A.rows : A.cols;
  const int64_t N = b_mn ? B.cols : B.rows, Kb = b_mn ? B.rows : B.cols;
  TORCH_CHECK(K == Kb, "inner dimensions differ: ", K, " vs ", Kb);
  TORCH_CHECK(out.size(0) == M && out.size(1) == N, "out has the wrong shape");
  if (side.has_value() && side->kind != 0) {
    const void* src[8] = {nullptr};
    TORCH_CHECK(side->src.size() >= 1 && side->src.size() <= 8, "side job needs 1..8 sources");
    for (size_t i = 0; i < side->src.size(); ++i) src[i] = reinterpret_cast<const void*>(side->src[i]);
    check_rc(llmt_gemm_bf16_fused(A.ptr, B.ptr, out.data_ptr(), (int)M, (int)N, (int)K, A.ld, B.ld, out.stride(0), a_mn, b_mn, f32,
                                  accumulate, (int)side->kind, (int)side->src.size(), src, reinterpret_cast<void*>(side->dst),
                                  (long long)side->n, side->accumulate, reinterpret_cast<const uint32_t*>(side->wait_flags),
                                  (int)side->n_wait, (uint32_t)side->wait_value, status_ptr(), cur_stream()),
             "llmt_gemm_bf16_fused");
    return;
  }
  const int rc = llmt_gemm_bf16(A.ptr, B.ptr, out.data_ptr(), (int)M, (int)N, (int)K, A.ld, B.ld, out.stride(0), a_mn, b_mn, f32,
                                accumulate, status_ptr(), (int)max_ctas, cur_stream());
  TORCH_CHECK(rc == 0, "llmt_gemm_bf16 failed with code ", rc, " (M=", M, " N=", N, " K=", K, " lda=", A.ld, " ldb=", B.ld,
              " ldc=", out.stride(0), " a_mn=", a_mn, " b_mn=", b_mn, " a%16=", reinterpret_cast<uintptr_t>(A.ptr) % 16,
              " b%16=", reinterpret_cast<uintptr_t>(B.ptr) % 16, ")");
  g_launches += 1;
}

// GEMM fused with a tensor-parallel row collective over peer memory (csrc/comm.cuh). mode 1: `a` is the local gathered
// matrix [M,K] that the kernel fills from `peer_src` (each rank's [M/world, K] chunk) while it multiplies; mode 2: `c` is
// this rank's symmetric partial matrix [M,N], `out` [M/world, N] receives the reduced rows (+ residual).
void gemm_tp(const Tensor& a, const Tensor& b, Tensor& c, bool b_mn, bool accumulate, int64_t mode, int64_t world, int64_t rank, int64_t epoch,
             const std::vector<int64_t>& peer_src, int64_t flags, const std::vector<int64_t>& peer_flags, Tensor& counters,
             const c10::optional<Tensor>& acc, const c10::optional<Tensor>& out, const c10::optional<Tensor>& residual) {
  c10::cuda::CUDAGuard guard(a.device());
  const Mat A = as_mat(a, "a"), B = as_mat(b, "b");
  check_bf16(c, "c");
  TORCH_CHECK(c.dim() == 2 && c.stride(1) == 1);
  const int64_t M = A.rows, K = A.cols, N = b_mn ? B.cols : B.rows, Kb = b_mn ? B.rows : B.cols;
  TORCH_CHECK(K == Kb && c.size(0) == M && c.size(1) == N, "gemm_tp: shapes do not match");
  TORCH_CHECK(!accumulate || b_mn, "gemm_tp: accumulate is only built for the [K][N] layout of b");
  TORCH_CHECK((int64_t)peer_src.size() == world && (int64_t)peer_flags.size() == world && world <= 8);
  TORCH_CHECK(counters.is_cuda() && counters.scalar_type() == at::kInt && counters.numel() >= 3 * world);
  const void* ps[8] = {nullptr};
  uint32_t* pf[8] = {nullptr};
  for (int64_t i = 0; i < world; ++i) {
    ps[i] = reinterpret_cast<const void*>(peer_src[i]);
    pf[i] = reinterpret_cast<uint32_t*>(peer_flags[i]);
  }
  float* accp = nullptr;
  void* outp = nullptr;
  const void* resp = nullptr;
  if (mode == 2) {
    TORCH_CHECK(acc.has_value() && out.has_value(), "reduce-scatter form needs acc and out");
    TORCH_CHECK(acc->scalar_type() == at::kFloat && acc->is_contiguous() && acc->numel() >= M / world * N);
    check_bf16(*out, "out");
    TORCH_CHECK(out->is_contiguous() && out->numel() == M / world * N);
    accp = acc->data_ptr<float>();
    outp = out->data_ptr();
    if (residual.has_value()) {
      check_bf16(*residual, "residual");
      TORCH_CHECK(residual->is_contiguous() && residual->numel() == out->numel());
      resp = residual->data_ptr();
    }
  }
  check_rc(llmt_gemm_bf16_tp(A.ptr, B.ptr, c.data_ptr(), (int)M, (int)N, (int)K, A.ld, B.ld, c.stride(0), b_mn, accumulate, (int)mode, (int)world,
                             (int)rank, (uint32_t)epoch, ps, reinterpret_cast<const uint32_t*>(flags), pf,
                             reinterpret_cast<uint32_t*>(counters.data_ptr<int>()), accp, outp, resp, status_ptr(), cur_stream()),
           "llmt_gemm_bf16_tp");
}

// ---- expert-parallel exchange over peer memory (csrc/ep_comm.cu). Peer buffers are raw device addresses.
static void fill_ptrs(const std::vector<int64_t>& v, void** out) {
  TORCH_CHECK(v.size() >= 1 && v.size() <= 8, "1..8 peers");
  for (size_t i = 0; i < 8; ++i) out[i] = i < v.size() ? reinterpret_cast<void*>(v[i]) : nullptr;
}
inline void check_i32(const Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), n, " must be a contiguous CUDA int32 tensor");
}

// Returns (seg_offsets [E/R + 1], totals [E/R], send_off [E]) as int32 device tensors.
std::vector<Tensor> ep_exchange(const Tensor& flat, int64_t E, int64_t me, const std::vector<int64_t>& tables,
                                const std::vector<int64_t>& flags, int64_t epoch, int64_t cap) {
  c10::cuda::CUDAGuard guard(flat.device());
  TORCH_CHECK(flat.is_cuda() && flat.scalar_type() == at::kLong && flat.is_contiguous());
  const int64_t R = (int64_t)tables.size();
  void *tp[8], *fp[8];
  fill_ptrs(tables, tp);
  fill_ptrs(flags, fp);
  auto o = torch::dtype(torch::kInt32).device(flat.device());
  Tensor seg = torch::empty({E / R + 1}, o), tot = torch::empty({E / R}, o), off = torch::empty({E}, o);
  check_rc(llmt_ep_exchange(flat.data_ptr<int64_t>(), flat.numel(), (int)E, (int)R, (int)me, tp, fp, (uint32_t)epoch, (int)cap,
                            seg.data_ptr<int>(), tot.data_ptr<int>(), off.data_ptr<int>(), status_ptr(), cur_stream()),
           "llmt_ep_exchange");
  return {seg, tot, off};
}

// (drank, drow) int32 [ncopies]: owner rank and row of every token copy (stable order inside each expert's run).
std::vector<Tensor> ep_plan(const Tensor& flat, int64_t E, int64_t R, const Tensor& send_off) {
  c10::cuda::CUDAGuard guard(flat.device());
  TORCH_CHECK(flat.is_cuda() && flat.scalar_type() == at::kLong && flat.is_contiguous());
  check_i32(send_off, "send_off");
  auto o = torch::dtype(torch::kInt32).device(flat.device());
  Tensor drank = torch::empty({flat.numel()}, o), drow = torch::empty({flat.numel()}, o);
  check_rc(llmt_ep_plan(flat.data_ptr<int64_t>(), flat.numel(), (int)E, (int)R, send_off.data_ptr<int>(), drank.data_ptr<int>(),
                        drow.data_ptr<int>(), cur_stream()),
           "llmt_ep_plan");
  return {drank, drow};
}

// peers[drank[c]][drow[c]] = scale[c] * src[c / k]; returns dot[c] = <src[c / k], other[c]> when `other` is given.
c10::optional<Tensor> ep_push_rows(const Tensor& src, const c10::optional<Tensor>& scale, const Tensor& drank, const Tensor& drow,
                                   const std::vector<int64_t>& bufs, int64_t cap, int64_t k, const c10::optional<Tensor>& other) {
  c10::cuda::CUDAGuard guard(src.device());
  check_bf16(src, "src");
  TORCH_CHECK(src.dim() == 2 && src.is_contiguous());
  check_i32(drank, "drank");
  check_i32(drow, "drow");
  const int64_t n = drank.numel(), D = src.size(1);
  TORCH_CHECK(drow.numel() == n && n == src.size(0) * k, "one destination per token copy");
  void* bp[8];
  fill_ptrs(bufs, bp);
  const float* sp = nullptr;
  if (scale.has_value()) {
    TORCH_CHECK(scale->scalar_type() == at::kFloat && scale->is_contiguous() && scale->numel() == n);
    sp = scale->data_ptr<float>();
  }
  c10::optional<Tensor> dot;
  const void* op = nullptr;
  float* dp = nullptr;
  if (other.has_value()) {
    check_bf16(*other, "other");
    TORCH_CHECK(other->is_contiguous() && other->numel() == n * D);
    dot = torch::empty({n}, torch::dtype(torch::kFloat32).device(src.device()));
    op = other->data_ptr();
    dp = dot->data_ptr<float>();
  }
  check_rc(llmt_ep_push_rows(src.data_ptr(), sp, drank.data_ptr<int>(), drow.data_ptr<int>(), bp, (int)bufs.size(), (int)cap, n, (int)k,
                             (int)D, op, dp, status_ptr(), cur_stream()),
           "llmt_ep_push_rows");
  return dot;
}

// out[t] = sum_j w[t, j] * peers[drank][drow]; returns (out, raw rows [T*k, D] when keep).
std::vector<Tensor> ep_pull_rows(const std::vector<int64_t>& bufs, const Tensor& drank, const Tensor& drow,
                                 const c10::optional<Tensor>& w, int64_t cap, int64_t T, int64_t k, int64_t D, bool keep) {
  c10::cuda::CUDAGuard guard(drank.device());
  check_i32(drank, "drank");
  check_i32(drow, "drow");
  TORCH_CHECK(drank.numel() == T * k && drow.numel() == T * k);
  void* bp[8];
  fill_ptrs(bufs, bp);
  auto o = torch::dtype(torch::kBFloat16).device(drank.device());
  Tensor out = torch::empty({T, D}, o);
  Tensor kp = keep ? torch::empty({T * k, D}, o) : Tensor();
  const float* wp = nullptr;
  if (w.has_value()) {
    TORCH_CHECK(w->scalar_type() == at::kFloat && w->is_contiguous() && w->numel() == T * k);
    wp = w->data_ptr<float>();
  }
  check_rc(llmt_ep_pull_rows(bp, (int)bufs.size(), drank.data_ptr<int>(), drow.data_ptr<int>(), wp, out.data_ptr(),
                             keep ? kp.data_ptr() : nullptr, (int)cap, (int)T, (int)k, (int)D, cur_stream()),
           "llmt_ep_pull_rows");
  if (keep) return {out, kp};
  return {out};
}

// dst rows below seg_offsets[-1] = live rows of src (address), alignment padding zeroed when zero_pad.
void ep_clone_rows(int64_t src, Tensor& dst, const Tensor& seg_offsets, const Tensor& totals, bool zero_pad) {
  c10::cuda::CUDAGuard guard(dst.device());
  check_bf16(dst, "dst");
  TORCH_CHECK(dst.dim() == 2 && dst.is_contiguous());
  check_i32(seg_offsets, "seg_offsets");
  check_i32(totals, "totals");
  check_rc(llmt_ep_clone_rows(reinterpret_cast<const void*>(src), dst.data_ptr(), seg_offsets.data_ptr<int>(), totals.data_ptr<int>(),
                              (int)totals.numel(), (int)dst.size(1), zero_pad, cur_stream()),
           "llmt_ep_clone_rows");
}

void side_job(const PySideJob& j, int64_t ctas) {
  const void* src[8] = {nullptr};
  TORCH_CHECK(j.src.size() >= 1 && j.src.size() <= 8, "side job needs 1..8 sources");
  for (size_t i = 0; i < j.src.size(); ++i) src[i] = reinterpret_cast<const void*>(j.src[i]);
  check_rc(llmt_side_job((int)j.kind, (int)j.src.size(), src, reinterpret_cast<void*>(j.dst), (long long)j.n, j.accumulate,
                         reinterpret_cast<const uint32_t*>(j.wait_flags), (int)j.n_wait, (uint32_t)j.wait_value, (int)ctas,
                         status_ptr(), cur_stream()),
           "llmt_side_job");
}

void signal_peers(const std::vector<int64_t>& peer_flag_ptrs, int64_t slot, int64_t value) {
  uint32_t* p[8] = {nullptr};
  TORCH_CHECK(peer_flag_ptrs.size() >= 1 && peer_flag_ptrs.size() <= 8);
  for (size_t i = 0; i < peer_flag_ptrs.size(); ++i) p[i] = reinterpret_cast<uint32_t*>(peer_flag_ptrs[i]);
  check_rc(llmt_signal_peers(p, (int)peer_flag_ptrs.size(), (int)slot, (uint32_t)value, cur_stream()), "llmt_signal_peers");
}

// max_polls == 0: the library's default limit (seconds); tests pass a small limit to see a wait expire quickly.
void wait_flags(int64_t flags_ptr, int64_t n, int64_t value, int64_t site, int64_t max_polls) {
  check_rc(llmt_wait_flags(reinterpret_cast<const uint32_t*>(flags_ptr), (int)n, (uint32_t)value, (int)site, (uint32_t)max_polls,
                           status_ptr(), cur_stream()),
           "llmt_wait_flags");
}

void grouped_gemm(const Tensor& a, const Tensor& b, Tensor& out, const Tensor& seg_offsets, bool b_mn) {
  c10::cuda::CUDAGuard guard(a.device());
  const Mat A = as_mat(a, "a");
  check_bf16(b, "b");
  check_bf16(out, "out");
  TORCH_CHECK(b.dim() == 3 && b.is_contiguous(), "b must be contiguous [G, N, K] or [G, K, N]");
  TORCH_CHECK(seg_offsets.is_cuda() && seg_offsets.scalar_type() == at::kInt && seg_offsets.is_contiguous());
  const int G = (int)b.size(0);
  TORCH_CHECK(seg_offsets.numel() == G + 1);
  const int64_t N = b_mn ? b.size(2) : b.size(1), K = b_mn ? b.size(1) : b.size(2);
  TORCH_CHECK(A.cols == K && out.size(0) == A.rows && out.size(1) == N && out.stride(1) == 1);
  check_rc(llmt_grouped_gemm_bf16(A.ptr, b.data_ptr(), out.data_ptr(), seg_offsets.data_ptr<int>(), G, (int)A.rows, (int)N,
                                  (int)K, A.ld, out.stride(0), b_mn, 0, status_ptr(), cur_stream()),
           "llmt_grouped_gemm_bf16");
}

// out[G, M, N] (+)= a_g^T b_g ; a [rows, M], b [rows, N]
void grouped_wgrad(const Tensor& a, const Tensor& b, Tensor& out, const Tensor& seg_offsets, bool accumulate) {
  c10::cuda::CUDAGuard guard(a.device());
  const Mat A = as_mat(a, "a"), B = as_mat(b, "b");
  TORCH_CHECK(out.dim() == 3 && out.is_contiguous() && out.is_cuda());
  const bool f32 = out.scalar_type() == at::kFloat;
  const int G = (int)out.size(0);
  TORCH_CHECK(seg_offsets.numel() == G + 1 && A.rows == B.rows && out.size(1) == A.cols && out.size(2) == B.cols);
  check_rc(llmt_grouped_wgrad_bf16(A.ptr, B.ptr, out.data_ptr(), seg_offsets.data_ptr<int>(), G, (int)A.rows, (int)A.cols,
                                   (int)B.cols, A.ld, B.ld, f32, accumulate, status_ptr(), cur_stream()),
           "llmt_grouped_wgrad_bf16");
}

std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const c10::optional<Tensor>& res, const Tensor& w, double eps) {
  c10::cuda::CUDAGuard guard(x.device());
  check_bf16(x, "x");
  check_bf16(w, "w");
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous());
  const int64_t D = x.size(-1), T = x.numel() / D;
  Tensor y = torch::empty_like(x);
  Tensor rstd = torch::empty({T}, x.options().dtype(torch::kFloat));
  Tensor s;
  const void* rp = nullptr;
  void* sp = nullptr;
  if (res.has_value()) {
    check_bf16(*res, "res");
    TORCH_CHECK(res->is_contiguous() && res->numel() == x.numel());
    s = torch::empty_like(x);
    rp = res->data_ptr();
    sp = s.data_ptr();
  }
  check_rc(llmt_rmsnorm_fwd(x.data_ptr(), rp, w.data_ptr(), y.data_ptr(), sp, rstd.data_ptr<float>(), (int)T, (int)D,
                            (float)eps, cur_stream()),
           "llmt_rmsnorm_fwd");
  if (res.has_value()) return {y, rstd, s};
  return {y, rstd};
}

// Returns (dx, dw fp32 [D]). `x` is the tensor that was normalised (the sum when a residual was added).
std::vector<Tensor> rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd,
                                const c10::optional<Tensor>& dres) {
  c10::cuda::CUDAGuard guard(x.device());
  check_bf16(dy, "dy");
  check_bf16(x, "x");
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous());
  const int64_t D = x.size(-1), T = x.numel() / D;
  Tensor dx = torch::empty_like(x);
  Tensor dw = torch::empty({D}, x.options().dtype(torch::kFloat));
  Tensor part = torch::empty({llmt_rmsnorm_bwd_partials((int)T), D}, x.options().dtype(torch::kFloat));
  const void* dr = nullptr;
  if (dres.has_value()) {
    check_bf16(*dres, "dres");
    TORCH_CHECK(dres->is_contiguous());
    dr = dres->data_ptr();
  }
  check_rc(llmt_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dr, dx.data_ptr(),
                            part.data_ptr<float>(), dw.data_ptr<float>(), nullptr, 0, (int)T, (int)D, cur_stream()),
           "llmt_rmsnorm_bwd", 2);
  return {dx, dw};
}

// x [T, H, HD] with arbitrary token stride (stride(1) == HD, stride(2) == 1). w may be undefined (no norm).
std::vector<Tensor> qk_norm_rope_fwd(const Tensor& x, const c10::optional<Tensor>& w, const Tensor& cosb, const Tensor& sinb,
                                     double eps) {
  c10::cuda::CUDAGuard guard(x.device());
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 3 && x.stride(2) == 1 && x.stride(1) == x.size(2), "x must be [T, H, HD] with packed heads");
  TORCH_CHECK(cosb.scalar_type() == at::kFloat && sinb.scalar_type() == at::kFloat && cosb.is_contiguous() && sinb.is_contiguous());
  const int T = (int)x.size(0), H = (int)x.size(1), HD = (int)x.size(2);
  TORCH_CHECK(cosb.size(0) == T && cosb.size(1) == HD / 2);
  Tensor y = torch::empty({T, H, HD}, x.options());
  Tensor rstd = torch::empty({(int64_t)T * H}, x.options().dtype(torch::kFloat));
  const void* wp = w.has_value() ? w->data_ptr() : nullptr;
  check_rc(llmt_qk_norm_rope_fwd(x.data_ptr(), x.stride(0), wp, cosb.data_ptr<float>(), sinb.data_ptr<float>(), y.data_ptr(),
                                 y.stride(0), rstd.data_ptr<float>(), T, H, HD, (float)eps, cur_stream()),
           "llmt_qk_norm_rope_fwd");
  return {y, rstd};
}

std::vector<Tensor> qk_norm_rope_bwd(const Tensor& dy, const Tensor& x, const c10::optional<Tensor>& w, const Tensor& cosb,
                                     const Tensor& sinb, const Tensor& rstd) {
  c10::cuda::CUDAGuard guard(x.device());
  check_bf16(dy, "dy");
  TORCH_CHECK(dy.dim() == 3 && dy.stride(2) == 1 && dy.stride(1) == dy.size(2));
  TORCH_CHECK(x.dim() == 3 && x.stride(2) == 1 && x.stride(1) == x.size(2));
  const int T = (int)x.size(0), H = (int)x.size(1), HD = (int)x.size(2);
  Tensor dx = torch::empty({T, H, HD}, x.options());
  Tensor dw, part;
  const void* wp = nullptr;
  float *pp = nullptr, *dwp = nullptr;
  if (w.has_value()) {
    wp = w->data_ptr();
    dw = torch::empty({HD}, x.options().dtype(torch::kFloat));
    part = torch::empty({llmt_qk_norm_rope_bwd_partials(T, H), HD}, x.options().dtype(torch::kFloat));
    pp = part.data_ptr<float>();
    dwp = dw.data_ptr<float>();
  }
  check_rc(llmt_qk_norm_rope_bwd(dy.data_ptr(), dy.stride(0), x.data_ptr(), x.stride(0), wp, cosb.data_ptr<float>(),
                                 sinb.data_ptr<float>(), rstd.data_ptr<float>(), dx.data_ptr(), dx.stride(0), pp, dwp, nullptr,
                                 0, T, H, HD, cur_stream()),
           "llmt_qk_norm_rope_bwd", w.has_value() ? 2 : 1);
  if (w.has_value()) return {dx, dw};
  return {dx};
}

inline int64_t row_stride_2d(const Tensor& t) {
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, "expected a 2-D tensor with a contiguous last dim");
  return t.stride(0);
}

static const int* limit_ptr(const c10::optional<Tensor>& row_limit) {
  if (!row_limit.has_value()) return nullptr;
  TORCH_CHECK(row_limit->is_cuda() && row_limit->scalar_type() == at::kInt && row_limit->numel() >= 1, "row_limit must be a CUDA int32 tensor");
  return row_limit->data_ptr<int>();
}

// s fp32 [B, R, C] contiguous, lse fp32 with B * R elements -> P bf16 [B, R, C]; row r is query (r % n) of its chunk.
Tensor attn_rows_probs(const Tensor& s, const Tensor& lse, int64_t n, int64_t diag, double scale, bool causal) {
  c10::cuda::CUDAGuard guard(s.device());
  TORCH_CHECK(s.is_cuda() && s.scalar_type() == at::kFloat && s.is_contiguous() && s.dim() == 3, "s must be a contiguous fp32 [B, R, C]");
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == s.size(0) * s.size(1));
  TORCH_CHECK(n > 0 && s.size(1) % n == 0, "rows per batch must be a multiple of the chunk length");
  Tensor p = torch::empty(s.sizes(), s.options().dtype(at::kBFloat16));
  check_rc(llmt_attn_rows_probs(s.data_ptr<float>(), lse.data_ptr<float>(), p.data_ptr(), s.size(0) * s.size(1), (int)s.size(2), (int)n,
                                (int)diag, (float)scale, causal ? 1 : 0, cur_stream()),
           "llmt_attn_rows_probs");
  return p;
}
Tensor attn_rows_ds(const Tensor& dp, const Tensor& p, const Tensor& delta) {
  c10::cuda::CUDAGuard guard(dp.device());
  TORCH_CHECK(dp.is_cuda() && dp.scalar_type() == at::kFloat && dp.is_contiguous() && dp.dim() == 3);
  TORCH_CHECK(p.is_cuda() && p.scalar_type() == at::kBFloat16 && p.is_contiguous() && p.sizes() == dp.sizes());
  TORCH_CHECK(delta.is_cuda() && delta.scalar_type() == at::kFloat && delta.is_contiguous() && delta.numel() == dp.size(0) * dp.size(1));
  Tensor ds = torch::empty(dp.sizes(), p.options());
  check_rc(llmt_attn_rows_ds(dp.data_ptr<float>(), p.data_ptr(), delta.data_ptr<float>(), ds.data_ptr(), dp.size(0) * dp.size(1),
                             (int)dp.size(2), cur_stream()),
           "llmt_attn_rows_ds");
  return ds;
}

// row_limit (optional int32 device scalar): rows at or beyond it are neither read nor written.
Tensor swiglu_fwd(const Tensor& gate, const Tensor& up, const c10::optional<Tensor>& row_limit) {
  c10::cuda::CUDAGuard guard(gate.device());
  check_bf16(gate, "gate");
  check_bf16(up, "up");
  TORCH_CHECK(row_stride_2d(gate) == row_stride_2d(up) && gate.sizes() == up.sizes());
  Tensor out = torch::empty({gate.size(0), gate.size(1)}, gate.options());
  check_rc(llmt_swiglu_fwd(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.size(0), (int)gate.size(1), gate.stride(0),
                           out.stride(0), limit_ptr(row_limit), cur_stream()),
           "llmt_swiglu_fwd");
  return out;
}

// dgate/dup are written into `dgate_out` / `dup_out` (same row stride), which lets them be the two halves of one buffer.
void swiglu_bwd(const Tensor& dout, const Tensor& gate, const Tensor& up, Tensor& dgate_out, Tensor& dup_out,
                const c10::optional<Tensor>& row_limit) {
  c10::cuda::CUDAGuard guard(gate.device());
  check_bf16(dout, "dout");
  TORCH_CHECK(row_stride_2d(gate) == row_stride_2d(up) && row_stride_2d(dgate_out) == row_stride_2d(dup_out));
  check_rc(llmt_swiglu_bwd(dout.data_ptr(), gate.data_ptr(), up.data_ptr(), dgate_out.data_ptr(), dup_out.data_ptr(),
                           gate.size(0), (int)gate.size(1), gate.stride(0), row_stride_2d(dout), dgate_out.stride(0),
                           limit_ptr(row_limit), cur_stream()),
           "llmt_swiglu_bwd");
}

// In place: logits become d(sum CE)/d(logits) * grad_scale. Returns (row_loss fp32 [rows], row_lse fp32 [rows]).
std::vector<Tensor> ce_fwd_bwd(Tensor& logits, const Tensor& labels, double grad_scale, const c10::optional<Tensor>& scale_t,
                               int64_t ignore_index, bool write_grad) {
  c10::cuda::CUDAGuard guard(logits.device());
  check_bf16(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1);
  TORCH_CHECK(labels.is_cuda() && labels.scalar_type() == at::kLong && labels.is_contiguous() && labels.numel() == logits.size(0));
  const int rows = (int)logits.size(0), V = (int)logits.size(1);
  Tensor loss = torch::empty({rows}, logits.options().dtype(torch::kFloat));
  Tensor lse = torch::empty({rows}, logits.options().dtype(torch::kFloat));
  const float* sp = scale_t.has_value() ? scale_t->data_ptr<float>() : nullptr;
  check_rc(llmt_ce_fwd_bwd(logits.data_ptr(), labels.data_ptr<int64_t>(), loss.data_ptr<float>(), lse.data_ptr<float>(), rows,
                           V, logits.stride(0), sp, (float)grad_scale, (int)ignore_index, write_grad, cur_stream()),
           "llmt_ce_fwd_bwd");
  return {loss, lse};
}

// Vocabulary-parallel cross-entropy over one shard of the logits [rows, V/R] (in place: the shard becomes its gradient);
// `stats` / `flags` are every rank's statistics and flag tables in symmetric memory (device addresses).
Tensor ce_vocab_parallel(Tensor& logits, const Tensor& labels, int64_t vocab_start, int64_t me, const std::vector<int64_t>& stats,
                         const std::vector<int64_t>& flags, int64_t cap, int64_t epoch, double grad_scale, int64_t ignore_index,
                         bool write_grad) {
  c10::cuda::CUDAGuard guard(logits.device());
  check_bf16(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1);
  TORCH_CHECK(labels.is_cuda() && labels.scalar_type() == at::kLong && labels.is_contiguous() && labels.numel() == logits.size(0));
  TORCH_CHECK(stats.size() == flags.size() && stats.size() >= 1 && stats.size() <= 8);
  const int rows = (int)logits.size(0), V = (int)logits.size(1), R = (int)stats.size();
  void* sp[8] = {nullptr};
  void* fp[8] = {nullptr};
  for (int i = 0; i < R; ++i) { sp[i] = reinterpret_cast<void*>(stats[i]); fp[i] = reinterpret_cast<void*>(flags[i]); }
  Tensor loss = torch::empty({rows}, logits.options().dtype(torch::kFloat));
  check_rc(llmt_ce_vocab_parallel(logits.data_ptr(), labels.data_ptr<int64_t>(), loss.data_ptr<float>(), rows, V, logits.stride(0),
                                  vocab_start, R, (int)me, sp, fp, (int)cap, (uint32_t)epoch, (float)grad_scale, (int)ignore_index,
                                  write_grad, status_ptr(), cur_stream()),
           "llmt_ce_vocab_parallel");
  return loss;
}

// Table rows of the ids this rank owns, stored into the output shard of the rank that owns each token.
void vp_embed_scatter(const Tensor& ids, const Tensor& w, int64_t vstart, int64_t vend, const std::vector<int64_t>& out, int64_t chunk) {
  c10::cuda::CUDAGuard guard(w.device());
  check_bf16(w, "weight");
  TORCH_CHECK(w.dim() == 2 && w.is_contiguous() && ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous());
  TORCH_CHECK(out.size() >= 1 && out.size() <= 8);
  void* op[8] = {nullptr};
  for (size_t i = 0; i < out.size(); ++i) op[i] = reinterpret_cast<void*>(out[i]);
  check_rc(llmt_vp_embed_scatter(ids.data_ptr<int64_t>(), w.data_ptr(), vstart, vend, op, (int)out.size(), (int)ids.numel(), (int)chunk,
                                 (int)w.size(1), cur_stream()),
           "llmt_vp_embed_scatter");
}

void adamw(Tensor& p32, const c10::optional<Tensor>& p16, const Tensor& g, Tensor& m, Tensor& v, double lr, double b1,
           double b2, double eps, double wd, int64_t step, const c10::optional<Tensor>& clip_coef, double grad_scale,
           bool decoupled) {
  c10::cuda::CUDAGuard guard(p32.device());
  TORCH_CHECK(p32.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat);
  TORCH_CHECK(p32.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous());
  const int64_t n = p32.numel();
  TORCH_CHECK(g.numel() == n && m.numel() == n && v.numel() == n);
  const bool gb = g.scalar_type() == at::kBFloat16;
  TORCH_CHECK(gb || g.scalar_type() == at::kFloat, "grad must be bf16 or fp32");
  void* p16p = nullptr;
  if (p16.has_value()) {
    check_bf16(*p16, "p16");
    TORCH_CHECK(p16->is_contiguous() && p16->numel() == n);
    p16p = p16->data_ptr();
  }
  const float* cc = clip_coef.has_value() ? clip_coef->data_ptr<float>() : nullptr;
  check_rc(llmt_adamw(p32.data_ptr<float>(), p16p, g.data_ptr(), gb, m.data_ptr<float>(), v.data_ptr<float>(), n, (float)lr,
                      (float)b1, (float)b2, (float)eps, (float)wd, (int)step, cc, (float)grad_scale, decoupled, cur_stream()),
           "llmt_adamw");
}

// out[0] (+)= sum(x^2), deterministic. scratch: fp32 >= sqnorm_scratch_floats().
void sqnorm(const Tensor& x, Tensor& scratch, Tensor& out, bool accumulate) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && scratch.scalar_type() == at::kFloat && out.scalar_type() == at::kFloat);
  TORCH_CHECK(scratch.numel() >= llmt_sqnorm_scratch_floats());
  const bool b = x.scalar_type() == at::kBFloat16;
  TORCH_CHECK(b || x.scalar_type() == at::kFloat);
  check_rc(llmt_sqnorm(x.data_ptr(), b, x.numel(), scratch.data_ptr<float>(), out.data_ptr<float>(), accumulate, cur_stream()),
           "llmt_sqnorm", 2);
}
int64_t sqnorm_scratch_floats() { return llmt_sqnorm_scratch_floats(); }

void clip_coef(const Tensor& total_sq, double max_norm, Tensor& coef, Tensor& norm_out, Tensor& finite) {
  c10::cuda::CUDAGuard guard(total_sq.device());
  check_rc(llmt_clip_coef(total_sq.data_ptr<float>(), (float)max_norm, coef.data_ptr<float>(), norm_out.data_ptr<float>(),
                          finite.data_ptr<int>(), cur_stream()),
           "llmt_clip_coef");
}

// pair: two query heads of a key/value group per CTA (attention_fwd_pair.cu); needs an even group size.
std::vector<Tensor> attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& tiles, double scale, bool causal,
                             bool pair) {
  c10::cuda::CUDAGuard guard(q.device());
  check_bf16(q, "q"); check_bf16(k, "k"); check_bf16(v, "v");
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3);
  TORCH_CHECK(q.stride(2) == 1 && q.stride(1) == q.size(2) && k.stride(2) == 1 && k.stride(1) == k.size(2) &&
              v.stride(2) == 1 && v.stride(1) == v.size(2), "q/k/v need packed heads [T, H, HD]");
  TORCH_CHECK(tiles.is_cuda() && tiles.scalar_type() == at::kInt && tiles.is_contiguous() && tiles.size(1) == 8);
  const int Tq = (int)q.size(0), Hq = (int)q.size(1), HD = (int)q.size(2), Tk = (int)k.size(0), Hkv = (int)k.size(1);
  Tensor o = torch::empty({Tq, Hq, HD}, q.options());
  Tensor lse = torch::empty({Hq, Tq}, q.options().dtype(torch::kFloat));
  if (pair && HD <= 128 && Hkv > 0 && Hq % Hkv == 0 && ((Hq / Hkv) % 2) == 0) {
    check_rc(llmt_attn_fwd_pair(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), tiles.data_ptr<int>(),
                                (int)tiles.size(0), Tq, Tk, Hq, Hkv, HD, q.stride(0), k.stride(0), v.stride(0), o.stride(0),
                                (float)scale, causal, status_ptr(), cur_stream()),
             "llmt_attn_fwd_pair");
    return {o, lse};
  }
  check_rc(llmt_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), tiles.data_ptr<int>(),
                         (int)tiles.size(0), Tq, Tk, Hq, Hkv, HD, q.stride(0), k.stride(0), v.stride(0), o.stride(0),
                         (float)scale, causal, status_ptr(), cur_stream()),
           "llmt_attn_fwd");
  return {o, lse};
}

// k_tile_passes: the dK/dV kernel runs once per pass; passes after the first accumulate (pieces that share keys).
std::vector<Tensor> attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& dout,
                             const Tensor& lse, const Tensor& q_tiles, const std::vector<Tensor>& k_tile_passes, double scale,
                             bool causal, bool zero_init, bool fused) {
  c10::cuda::CUDAGuard guard(q.device());
  check_bf16(dout, "dout");
  TORCH_CHECK(dout.dim() == 3 && dout.stride(2) == 1 && dout.stride(1) == dout.size(2) && o.is_contiguous());
  const int Tq = (int)q.size(0), Hq = (int)q.size(1), HD = (int)q.size(2), Tk = (int)k.size(0), Hkv = (int)k.size(1);
  Tensor dq = (zero_init && !fused) ? torch::zeros({Tq, Hq, HD}, q.options()) : torch::empty({Tq, Hq, HD}, q.options());
  Tensor dk = zero_init ? torch::zeros({Tk, Hkv, HD}, k.options()) : torch::empty({Tk, Hkv, HD}, k.options());
  Tensor dv = zero_init ? torch::zeros({Tk, Hkv, HD}, v.options()) : torch::empty({Tk, Hkv, HD}, v.options());
  Tensor delta = torch::empty({Hq, Tq}, q.options().dtype(torch::kFloat));
  const int npass = (int)k_tile_passes.size();
  if (fused) {
    // one walk per key tile yields dK, dV and that tile's share of dQ, which is summed in an fp32 accumulator
    Tensor acc = torch::empty({Tq, Hq, HD}, q.options().dtype(torch::kFloat));
    const int n = npass > 0 ? npass : 1;
    for (int p = 0; p < n; ++p) {
      const int* kt = npass > 0 ? k_tile_passes[p].data_ptr<int>() : nullptr;
      const int nkt = npass > 0 ? (int)k_tile_passes[p].size(0) : 0;
      check_rc(llmt_attn_bwd_fused(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dout.data_ptr(), lse.data_ptr<float>(),
                                   delta.data_ptr<float>(), acc.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), kt,
                                   nkt, Tq, Tk, Hq, Hkv, HD, q.stride(0), k.stride(0), v.stride(0), o.stride(0), dout.stride(0),
                                   dq.stride(0), dk.stride(0), dv.stride(0), (float)scale, causal, p == 0, p == n - 1,
                                   status_ptr(), cur_stream()),
               "llmt_attn_bwd_fused", (p == 0 ? 1 : 0) + (nkt > 0 ? 1 : 0) + (p == n - 1 ? 1 : 0));
    }
    return {dq, dk, dv};
  }
  for (int p = 0; p < (npass > 0 ? npass : 1); ++p) {
    const int* kt = npass > 0 ? k_tile_passes[p].data_ptr<int>() : nullptr;
    const int nkt = npass > 0 ? (int)k_tile_passes[p].size(0) : 0;
    check_rc(llmt_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dout.data_ptr(), lse.data_ptr<float>(),
                           delta.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), q_tiles.data_ptr<int>(),
                           p == 0 ? (int)q_tiles.size(0) : 0, kt, nkt, Tq, Tk, Hq, Hkv, HD, q.stride(0), k.stride(0), v.stride(0),
                           o.stride(0), dout.stride(0), dq.stride(0), dk.stride(0), dv.stride(0), (float)scale, causal,
                           /*pass=*/p, status_ptr(), cur_stream()),
             "llmt_attn_bwd", p == 0 ? 3 : 1);
  }
  return {dq, dk, dv};
}

// ---- MoE
std::vector<Tensor> router_topk(const Tensor& logits, const c10::optional<Tensor>& bias, int64_t k, int64_t score_fn, bool renorm,
                                double route_scale) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.is_contiguous());
  const int T = (int)logits.size(0), E = (int)logits.size(1);
  Tensor w = torch::empty({T, k}, logits.options());
  Tensor idx = torch::empty({T, k}, logits.options().dtype(torch::kLong));
  Tensor counts = torch::zeros({E}, logits.options());
  Tensor denom = torch::empty({T}, logits.options());
  const float* bp = bias.has_value() ? bias->data_ptr<float>() : nullptr;
  check_rc(llmt_router_topk(logits.data_ptr<float>(), bp, w.data_ptr<float>(), idx.data_ptr<int64_t>(), counts.data_ptr<float>(),
                            denom.data_ptr<float>(), T, E, (int)k, (int)score_fn, renorm, (float)route_scale, cur_stream()),
           "llmt_router_topk");
  return {w, idx, counts, denom};
}
Tensor router_topk_bwd(const Tensor& logits, const Tensor& dw, const Tensor& idx, const Tensor& denom, int64_t score_fn, bool renorm,
                       double route_scale) {
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor dl = torch::zeros_like(logits);
  Tensor dwc = dw.contiguous();
  check_rc(llmt_router_topk_bwd(logits.data_ptr<float>(), dwc.data_ptr<float>(), idx.data_ptr<int64_t>(), denom.data_ptr<float>(),
                                dl.data_ptr<float>(), (int)logits.size(0), (int)logits.size(1), (int)idx.size(1), (int)score_fn, renorm,
                                (float)route_scale, cur_stream()),
           "llmt_router_topk_bwd");
  return dl;
}
// rows must be zero-initialised by the caller (padding rows stay zero)
void permute_rows(const Tensor& x, const Tensor& dest, Tensor& rows, int64_t k) {
  c10::cuda::CUDAGuard guard(x.device());
  check_bf16(x, "x"); check_bf16(rows, "rows");
  TORCH_CHECK(x.is_contiguous() && rows.is_contiguous() && dest.scalar_type() == at::kLong && dest.is_contiguous());
  check_rc(llmt_permute_rows(x.data_ptr(), dest.data_ptr<int64_t>(), rows.data_ptr(), dest.numel(), (int)k, (int)x.size(1), cur_stream()),
           "llmt_permute_rows");
}
Tensor combine_rows(const Tensor& y, const Tensor& dest, const c10::optional<Tensor>& w, int64_t T, int64_t k) {
  c10::cuda::CUDAGuard guard(y.device());
  check_bf16(y, "y");
  TORCH_CHECK(y.is_contiguous() && dest.is_contiguous());
  Tensor out = torch::empty({T, y.size(1)}, y.options());
  const float* wp = w.has_value() ? w->data_ptr<float>() : nullptr;
  check_rc(llmt_combine_rows(y.data_ptr(), dest.data_ptr<int64_t>(), wp, out.data_ptr(), (int)T, (int)k, (int)y.size(1), cur_stream()),
           "llmt_combine_rows");
  return out;
}
std::vector<Tensor> combine_bwd(const Tensor& dout, const Tensor& y, const Tensor& dest, const Tensor& w, int64_t k) {
  c10::cuda::CUDAGuard guard(y.device());
  Tensor dy = torch::zeros_like(y);
  Tensor dw = torch::empty({dest.numel()}, y.options().dtype(torch::kFloat));
  Tensor d = dout.contiguous();
  check_rc(llmt_combine_bwd(d.data_ptr(), y.data_ptr(), dest.data_ptr<int64_t>(), w.data_ptr<float>(), dy.data_ptr(), dw.data_ptr<float>(),
                            dest.numel(), (int)k, (int)y.size(1), cur_stream()),
           "llmt_combine_bwd");
  return {dy, dw};
}

// Reads the status word (synchronises the current stream) and clears it. Returns {code, site, block, extra}.
std::vector<int64_t> read_status(bool clear) {
  Tensor h = status_word().cpu();
  std::vector<int64_t> r{h[0].item<int64_t>(), h[1].item<int64_t>(), h[2].item<int64_t>(), h[3].item<int64_t>()};
  if (clear && r[0] != 0) status_word().zero_();
  return r;
}
Tensor status_tensor() { return status_word(); }
int64_t launch_count() { return g_launches; }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  py::class_<PySideJob>(m, "SideJob")
      .def(py::init<>())
      .def_readwrite("kind", &PySideJob::kind)
      .def_readwrite("src", &PySideJob::src)
      .def_readwrite("dst", &PySideJob::dst)
      .def_readwrite("n", &PySideJob::n)
      .def_readwrite("accumulate", &PySideJob::accumulate)
      .def_readwrite("wait_flags", &PySideJob::wait_flags)
      .def_readwrite("n_wait", &PySideJob::n_wait)
      .def_readwrite("wait_value", &PySideJob::wait_value);
  m.def("gemm", &gemm, "bf16 tcgen05 GEMM", py::arg("a"), py::arg("b"), py::arg("out"), py::arg("a_mn"), py::arg("b_mn"),
        py::arg("accumulate") = false, py::arg("max_ctas") = 0, py::arg("side") = py::none());
  m.def("router_topk", &router_topk);
  m.def("router_topk_bwd", &router_topk_bwd);
  m.def("permute_rows", &permute_rows);
  m.def("combine_rows", &combine_rows);
  m.def("combine_bwd", &combine_bwd);
  m.def("gemm_tp", &gemm_tp, py::arg("a"), py::arg("b"), py::arg("c"), py::arg("b_mn"), py::arg("accumulate"), py::arg("mode"), py::arg("world"),
        py::arg("rank"), py::arg("epoch"), py::arg("peer_src"), py::arg("flags"), py::arg("peer_flags"), py::arg("counters"),
        py::arg("acc") = py::none(), py::arg("out") = py::none(), py::arg("residual") = py::none());
  m.def("ep_exchange", &ep_exchange);
  m.def("ep_plan", &ep_plan);
  m.def("ep_push_rows", &ep_push_rows);
  m.def("ep_pull_rows", &ep_pull_rows);
  m.def("ep_clone_rows", &ep_clone_rows);
  m.def("side_job", &side_job);
  m.def("signal_peers", &signal_peers);
  m.def("wait_flags", &wait_flags, py::arg("flags_ptr"), py::arg("n"), py::arg("value"), py::arg("site"), py::arg("max_polls") = 0);
  m.def("grouped_gemm", &grouped_gemm);
  m.def("grouped_wgrad", &grouped_wgrad);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("qk_norm_rope_fwd", &qk_norm_rope_fwd);
  m.def("qk_norm_rope_bwd", &qk_norm_rope_bwd);
  m.def("attn_rows_probs", &attn_rows_probs);
  m.def("attn_rows_ds", &attn_rows_ds);
  m.def("swiglu_fwd", &swiglu_fwd, py::arg("gate"), py::arg("up"), py::arg("row_limit") = py::none());
  m.def("swiglu_bwd", &swiglu_bwd, py::arg("dout"), py::arg("gate"), py::arg("up"), py::arg("dgate_out"), py::arg("dup_out"),
        py::arg("row_limit") = py::none());
  m.def("ce_fwd_bwd", &ce_fwd_bwd);
  m.def("ce_vocab_parallel", &ce_vocab_parallel);
  m.def("vp_embed_scatter", &vp_embed_scatter);
  m.def("adamw", &adamw);
  m.def("sqnorm", &sqnorm);
  m.def("sqnorm_scratch_floats", &sqnorm_scratch_floats);
  m.def("clip_coef", &clip_coef);
  m.def("attn_fwd", &attn_fwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("tiles"), py::arg("scale"), py::arg("causal"),
        py::arg("pair") = false);
  m.def("attn_bwd", &attn_bwd);
  m.def("read_status", &read_status, py::arg("clear") = true);
  m.def("status_tensor", &status_tensor);
  m.def("launch_count", &launch_count);
}
