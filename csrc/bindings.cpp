// torch glue for the sm_100a kernel library: registers torch.ops.cosmos_b200.* and validates
// shapes/dtypes/strides before handing raw pointers to the launchers in kernels.h.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <optional>

#include "kernels.h"
#include "runtime.h"

namespace {
constexpr int kDefaultAttnExpEmu = 0;

using at::Tensor;
using OptT = std::optional<Tensor>;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_bf16_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
}
const void* opt_ptr(const OptT& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

// One int32 status word per device; kernels CAS their first failure code into it.
Tensor status_tensor(int device) {
  static std::mutex mu;
  static std::map<int, Tensor> words;
  std::lock_guard<std::mutex> g(mu);
  auto it = words.find(device);
  if (it == words.end()) {
    Tensor t = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
    it = words.emplace(device, t).first;
  }
  return it->second;
}

Tensor status_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  return status_tensor(dev);
}

Tensor as_2d(const Tensor& x) { return x.dim() == 2 ? x : x.reshape({-1, x.size(-1)}); }

// C = A @ W^T with fused epilogue. A [.., K]; W [N, K]; returns [.., N] (or [.., N/2] for SwiGLU).
Tensor gemm(const Tensor& A_, const Tensor& W, const OptT& bias, int64_t epi, const OptT& resid,
            const OptT& gate, int64_t rows_per_batch, const OptT& out) {
  check_bf16_cuda(A_, "A");
  check_bf16_cuda(W, "W");
  c10::cuda::CUDAGuard guard(A_.device());
  Tensor A = as_2d(A_);
  TORCH_CHECK(A.stride(1) == 1 && W.dim() == 2 && W.stride(1) == 1, "A and W must be row-major");
  TORCH_CHECK(A.size(1) == W.size(1), "K mismatch: A ", A.sizes(), " W ", W.sizes());
  const int64_t M = A.size(0), N = W.size(0), K = A.size(1);
  const int64_t n_out = (epi == EPI_SWIGLU) ? N / 2 : N;
  Tensor C;
  if (out.has_value() && out->defined()) {
    C = as_2d(*out);
    check_bf16_cuda(C, "out");
    TORCH_CHECK(C.size(0) == M && C.size(1) == n_out && C.stride(1) == 1, "bad out shape");
  } else {
    C = at::empty({M, n_out}, A.options());
  }
  cosmos::GemmArgs g;
  g.A = A.data_ptr(); g.B = W.data_ptr(); g.C = C.data_ptr();
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.lda = A.stride(0); g.ldb = W.stride(0); g.ldc = C.stride(0);
  g.epi = (int)epi;
  if (bias.has_value() && bias->defined()) {
    check_bf16_cuda(*bias, "bias");
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "bias must be [N]");
    TORCH_CHECK(epi != EPI_SWIGLU, "bias is not supported with the SwiGLU epilogue");
    g.bias = bias->data_ptr();
  }
  Tensor R;
  if (epi == EPI_GATED_RESID) {
    TORCH_CHECK(resid.has_value() && resid->defined(), "gated-residual epilogue needs a residual");
    R = as_2d(*resid);
    check_bf16_cuda(R, "resid");
    TORCH_CHECK(R.size(0) == M && R.size(1) == N && R.stride(1) == 1 && R.stride(0) % 8 == 0,
                "bad residual shape");
    g.R = R.data_ptr(); g.ldr = R.stride(0);
    if (gate.has_value() && gate->defined()) {
      check_bf16_cuda(*gate, "gate");
      TORCH_CHECK(gate->is_contiguous() && gate->size(-1) == N && N % 8 == 0, "gate must be [B, N]");
      TORCH_CHECK(rows_per_batch > 0 && gate->numel() / N * rows_per_batch >= M,
                  "gate rows do not cover M");
      g.gate = gate->data_ptr();
    }
    g.rows_per_batch = (int)rows_per_batch;
  }
  g.status = status_tensor(A.get_device()).data_ptr<int>();
  Tensor partial;
  const int ks = cosmos::gemm_pick_k_splits(g.M, g.N, g.K, g.epi);
  if (ks > 1 && C.stride(0) % 4 == 0) {  // skinny problem (decode): split K across CTAs, fp32 partials as scratch
    partial = at::empty({ks, M, N}, A.options().dtype(at::kFloat));
    g.k_splits = ks;
    g.partial = partial.data_ptr<float>();
  }
  cosmos::gemm_bf16(g, cur_stream());
  auto shape = A_.sizes().vec();
  shape.back() = n_out;
  return C.reshape(shape);
}

std::tuple<Tensor, Tensor> rmsnorm(const Tensor& x, const OptT& gamma, double eps, const OptT& residual);

// Output projection of a decode step with the residual add and the RMS-norm that follow it:
//   x_new = residual + a w^T,  h = rmsnorm(x_new) * gamma   ->  (h, x_new)
// For skinny problems (split-K) the reduction pass does all three; otherwise the GEMM and the norm kernel run
// one after the other.
std::tuple<Tensor, Tensor> gemm_reduce_rmsnorm(const Tensor& A_, const Tensor& W, const Tensor& residual,
                                               const OptT& gamma, double eps) {
  check_bf16_cuda(A_, "a"); check_bf16_cuda(W, "w"); check_bf16_cuda(residual, "residual");
  c10::cuda::CUDAGuard guard(A_.device());
  Tensor A = as_2d(A_);
  const int64_t M = A.size(0), K = A.size(1), N = W.size(0);
  TORCH_CHECK(W.dim() == 2 && W.size(1) == K && A.stride(1) == 1 && W.stride(1) == 1, "a [.., K] and w [N, K] expected");
  TORCH_CHECK(A.stride(0) % 8 == 0 && W.stride(0) % 8 == 0 && N % 8 == 0, "rows must be 16-byte aligned");
  Tensor R = as_2d(residual);
  TORCH_CHECK(R.size(0) == M && R.size(1) == N && R.stride(1) == 1 && R.stride(0) % 8 == 0, "bad residual shape");
  if (gamma.has_value() && gamma->defined()) { check_bf16_cuda(*gamma, "gamma"); TORCH_CHECK(gamma->numel() == N && gamma->is_contiguous()); }
  const int ks = cosmos::gemm_pick_k_splits((int)M, (int)N, (int)K, EPI_PLAIN);
  Tensor x_new = at::empty({M, N}, A.options());
  if (ks > 1 && N <= 8192) {
    Tensor h = at::empty({M, N}, A.options());
    Tensor partial = at::empty({ks, M, N}, A.options().dtype(at::kFloat));
    cosmos::GemmArgs g;
    g.A = A.data_ptr(); g.B = W.data_ptr(); g.C = x_new.data_ptr();
    g.M = (int)M; g.N = (int)N; g.K = (int)K;
    g.lda = A.stride(0); g.ldb = W.stride(0); g.ldc = N;
    g.epi = EPI_PLAIN;
    g.R = R.data_ptr(); g.ldr = R.stride(0);
    g.k_splits = ks; g.partial = partial.data_ptr<float>();
    g.norm_gamma = opt_ptr(gamma); g.norm_out = h.data_ptr(); g.norm_eps = (float)eps;
    g.status = status_tensor(A.get_device()).data_ptr<int>();
    cosmos::gemm_bf16(g, cur_stream());
    return {h.reshape(residual.sizes()), x_new.reshape(residual.sizes())};
  }
  Tensor y = gemm(A, W, {}, EPI_PLAIN, {}, {}, 0, {});
  auto hr = rmsnorm(y, gamma, eps, R.contiguous());
  return {std::get<0>(hr).reshape(residual.sizes()), std::get<1>(hr).reshape(residual.sizes())};
}

// General-major GEMM C[M, N] = op(A) op(B)^T for the backward passes:
//   a_mn = false: A is [M, K];  a_mn = true: A is stored as [K, M] (read transposed in place)
//   b_mn = false: B is [N, K];  b_mn = true: B is stored as [K, N]
// dX = dY W      -> gemm_ex(dY [M, N], W [N, K], false, true)   (contraction over N)
// dW = dY^T X    -> gemm_ex(dY [M, N], X [M, K], true, true)    (contraction over M)
Tensor gemm_ex(const Tensor& A, const Tensor& B, bool a_mn, bool b_mn, const OptT& out) {
  check_bf16_cuda(A, "A"); check_bf16_cuda(B, "B");
  c10::cuda::CUDAGuard guard(A.device());
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && A.stride(1) == 1 && B.stride(1) == 1, "A and B must be 2-D row-major");
  const int64_t M = a_mn ? A.size(1) : A.size(0), K = a_mn ? A.size(0) : A.size(1);
  const int64_t N = b_mn ? B.size(1) : B.size(0), Kb = b_mn ? B.size(0) : B.size(1);
  TORCH_CHECK(K == Kb, "contraction sizes differ: ", K, " vs ", Kb);
  TORCH_CHECK(A.stride(0) % 8 == 0 && B.stride(0) % 8 == 0, "row strides must be multiples of 8");
  Tensor C;
  if (out.has_value() && out->defined()) {
    C = *out;
    check_bf16_cuda(C, "out");
    TORCH_CHECK(C.dim() == 2 && C.size(0) == M && C.size(1) == N && C.stride(1) == 1 && C.stride(0) % 8 == 0);
  } else {
    C = at::empty({M, (N + 7) / 8 * 8}, A.options()).narrow(1, 0, N);
  }
  cosmos::GemmArgs g;
  g.A = A.data_ptr(); g.B = B.data_ptr(); g.C = C.data_ptr();
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.lda = A.stride(0); g.ldb = B.stride(0); g.ldc = C.stride(0);
  g.a_mn = a_mn; g.b_mn = b_mn;
  g.epi = EPI_PLAIN;
  g.status = status_tensor(A.get_device()).data_ptr<int>();
  cosmos::gemm_bf16(g, cur_stream());
  return C;
}

// Attention-backward score GEMMs for one head (scores materialised as bf16 [Sq, Skv]):
//   mode 0: P  = exp(q k^T * scale - lse[:, None]) under the forward mask
//   mode 1: dS = P * (dO v^T - D[:, None]) * scale        (P passed in `p_in`)
// a [Sq, 128] (q or dO), b [Skv, 128] (k or v), rowvec fp32 [Sq].
Tensor attn_bwd_scores(const Tensor& a, const Tensor& b, const Tensor& rowvec, double scale, int64_t mask,
                       int64_t n_ar, int64_t mode, const OptT& p_in, const OptT& out) {
  check_bf16_cuda(a, "a"); check_bf16_cuda(b, "b");
  c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && a.size(1) == b.size(1));
  TORCH_CHECK(rowvec.is_cuda() && rowvec.scalar_type() == at::kFloat && rowvec.is_contiguous() && rowvec.numel() == a.size(0));
  const int64_t M = a.size(0), N = b.size(0), K = a.size(1);
  const int64_t ld = (N + 7) / 8 * 8;
  Tensor C = out.has_value() && out->defined() ? *out : at::empty({M, ld}, a.options()).narrow(1, 0, N);
  TORCH_CHECK(C.size(0) == M && C.size(1) == N && C.stride(1) == 1 && C.stride(0) % 8 == 0);
  cosmos::GemmArgs g;
  g.A = a.data_ptr(); g.B = b.data_ptr(); g.C = C.data_ptr();
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.lda = a.stride(0); g.ldb = b.stride(0); g.ldc = C.stride(0);
  g.rowvec = rowvec.data_ptr<float>(); g.attn_scale = (float)scale; g.attn_mask = (int)mask; g.attn_n_ar = (int)n_ar;
  if (mode == 0) {
    g.epi = EPI_ATTN_P;
  } else {
    g.epi = EPI_ATTN_DS;
    TORCH_CHECK(p_in.has_value() && p_in->defined() && p_in->size(0) == M && p_in->size(1) == N && p_in->stride(1) == 1);
    check_bf16_cuda(*p_in, "p_in");
    g.R = p_in->data_ptr(); g.ldr = p_in->stride(0);
  }
  g.status = status_tensor(a.get_device()).data_ptr<int>();
  cosmos::gemm_bf16(g, cur_stream());
  return C;
}

// Grouped GEMM over two token segments with their own weights (MoT per-modality routing), one launch.
// epi in {PLAIN, SWIGLU, GATED_RESID}; returns (C0, C1).
std::tuple<Tensor, Tensor> gemm_grouped2(const Tensor& A0_, const Tensor& W0, const Tensor& A1_, const Tensor& W1,
                                         int64_t epi, const OptT& resid0, const OptT& resid1, const OptT& gate0,
                                         const OptT& gate1, int64_t rpb0, int64_t rpb1) {
  TORCH_CHECK(epi == EPI_PLAIN || epi == EPI_SWIGLU || epi == EPI_GATED_RESID, "unsupported epilogue for grouped GEMM");
  c10::cuda::CUDAGuard guard(A0_.device());
  const Tensor* As[2] = {&A0_, &A1_};
  const Tensor* Ws[2] = {&W0, &W1};
  const OptT* Rs[2] = {&resid0, &resid1};
  const OptT* Gs[2] = {&gate0, &gate1};
  const int64_t rpbs[2] = {rpb0, rpb1};
  cosmos::GemmArgs args[2];
  Tensor A2[2], C[2], R2[2];
  for (int i = 0; i < 2; ++i) {
    check_bf16_cuda(*As[i], "A"); check_bf16_cuda(*Ws[i], "W");
    A2[i] = as_2d(*As[i]);
    TORCH_CHECK(A2[i].stride(1) == 1 && Ws[i]->dim() == 2 && Ws[i]->stride(1) == 1 && A2[i].size(1) == Ws[i]->size(1),
                "bad A/W in problem ", i);
    const int64_t M = A2[i].size(0), N = Ws[i]->size(0), K = A2[i].size(1);
    const int64_t n_out = (epi == EPI_SWIGLU) ? N / 2 : N;
    C[i] = at::empty({M, n_out}, A2[i].options());
    cosmos::GemmArgs& g = args[i];
    g.A = A2[i].data_ptr(); g.B = Ws[i]->data_ptr(); g.C = C[i].data_ptr();
    g.M = (int)M; g.N = (int)N; g.K = (int)K;
    g.lda = A2[i].stride(0); g.ldb = Ws[i]->stride(0); g.ldc = C[i].stride(0);
    g.epi = (int)epi;
    if (epi == EPI_GATED_RESID) {
      TORCH_CHECK(Rs[i]->has_value() && (*Rs[i])->defined(), "gated-residual epilogue needs residuals");
      R2[i] = as_2d(**Rs[i]);
      check_bf16_cuda(R2[i], "resid");
      TORCH_CHECK(R2[i].size(0) == M && R2[i].size(1) == N && R2[i].stride(1) == 1 && R2[i].stride(0) % 8 == 0);
      g.R = R2[i].data_ptr(); g.ldr = R2[i].stride(0);
      if (Gs[i]->has_value() && (*Gs[i])->defined()) {
        check_bf16_cuda(**Gs[i], "gate");
        TORCH_CHECK((*Gs[i])->is_contiguous() && (*Gs[i])->size(-1) == N && rpbs[i] > 0 &&
                    (*Gs[i])->numel() / N * rpbs[i] >= M, "bad gate in problem ", i);
        g.gate = (*Gs[i])->data_ptr();
      }
      g.rows_per_batch = (int)rpbs[i];
    }
    g.status = status_tensor(A0_.get_device()).data_ptr<int>();
  }
  if (args[0].M == 0) {
    if (args[1].M > 0) cosmos::gemm_bf16(args[1], cur_stream());
  } else {
    cosmos::gemm_bf16_grouped(args, 2, cur_stream());
  }
  auto shape_of = [&](int i) {
    auto sh = As[i]->sizes().vec();
    sh.back() = C[i].size(1);
    return sh;
  };
  return {C[0].reshape(shape_of(0)), C[1].reshape(shape_of(1))};
}

// QKV projection with per-head RMSNorm + rotary embedding in the epilogue and optional
// routing of each 128-column head chunk (route_ptr / route_ld are int64 device tensors).
Tensor gemm_qkv_rope(const Tensor& A_, const Tensor& W, const OptT& bias, const OptT& cos_t,
                     const OptT& sin_t, const OptT& gamma_q, const OptT& gamma_k, int64_t n_q_heads,
                     int64_t n_k_heads, double eps, const OptT& route_ptr, const OptT& route_ld,
                     const OptT& out) {
  check_bf16_cuda(A_, "A");
  check_bf16_cuda(W, "W");
  c10::cuda::CUDAGuard guard(A_.device());
  Tensor A = as_2d(A_);
  TORCH_CHECK(A.stride(1) == 1 && W.stride(1) == 1 && A.size(1) == W.size(1), "bad A/W");
  const int64_t M = A.size(0), N = W.size(0), K = A.size(1);
  TORCH_CHECK(N % 128 == 0, "N must be a multiple of the head size 128");
  cosmos::GemmArgs g;
  Tensor C;
  const bool routed = route_ptr.has_value() && route_ptr->defined();
  if (routed) {
    TORCH_CHECK(route_ld.has_value() && route_ptr->scalar_type() == at::kLong &&
                    route_ld->scalar_type() == at::kLong && route_ptr->is_cuda() &&
                    route_ptr->numel() == N / 128 && route_ld->numel() == N / 128,
                "route tables must be int64 CUDA tensors with one entry per head");
    g.route_ptr = reinterpret_cast<const long long*>(route_ptr->data_ptr<int64_t>());
    g.route_ld = reinterpret_cast<const long long*>(route_ld->data_ptr<int64_t>());
    C = out.has_value() && out->defined() ? *out : at::empty({0}, A.options());
  } else {
    if (out.has_value() && out->defined()) {
      C = as_2d(*out);
      TORCH_CHECK(C.size(0) == M && C.size(1) == N && C.stride(1) == 1 && C.stride(0) % 8 == 0);
    } else {
      C = at::empty({M, N}, A.options());
    }
    g.C = C.data_ptr(); g.ldc = C.stride(0);
  }
  g.A = A.data_ptr(); g.B = W.data_ptr();
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.lda = A.stride(0); g.ldb = W.stride(0);
  g.epi = EPI_QKV_ROPE;
  if (bias.has_value() && bias->defined()) {
    check_bf16_cuda(*bias, "bias");
    g.bias = bias->data_ptr();
  }
  if (cos_t.has_value() && cos_t->defined()) {
    TORCH_CHECK(sin_t.has_value() && cos_t->scalar_type() == at::kFloat && cos_t->is_contiguous() &&
                    sin_t->is_contiguous() && cos_t->size(-1) == 64 && sin_t->sizes() == cos_t->sizes(),
                "cos/sin tables must be contiguous fp32 [rows, 64]");
    g.cos_tab = cos_t->data_ptr<float>(); g.sin_tab = sin_t->data_ptr<float>();
    g.rope_rows = (int)(cos_t->numel() / 64);
  }
  if (gamma_q.has_value() && gamma_q->defined()) { check_bf16_cuda(*gamma_q, "gamma_q"); g.gamma_q = gamma_q->data_ptr(); }
  if (gamma_k.has_value() && gamma_k->defined()) { check_bf16_cuda(*gamma_k, "gamma_k"); g.gamma_k = gamma_k->data_ptr(); }
  g.n_q_heads = (int)n_q_heads; g.n_k_heads = (int)n_k_heads; g.eps = (float)eps;
  g.status = status_tensor(A.get_device()).data_ptr<int>();
  cosmos::gemm_bf16(g, cur_stream());
  if (routed) return C;
  auto shape = A_.sizes().vec();
  shape.back() = N;
  return C.reshape(shape);
}

// Forward-attention switches: share of exponentials on the FMA pipe (AttnArgs::exp_emulation, initial value from
// COSMOS_ATTN_EXP_EMU) and the timing-experiment bits (AttnArgs::debug, COSMOS_ATTN_DEBUG).
static int& attn_exp_emu() {
  static int v = [] { const char* e = std::getenv("COSMOS_ATTN_EXP_EMU"); return e ? std::atoi(e) : kDefaultAttnExpEmu; }();
  return v;
}
static int& attn_debug() {
  static int v = [] { const char* e = std::getenv("COSMOS_ATTN_DEBUG"); return e ? std::atoi(e) : 0; }();
  return v;
}

// q [B, Sq, Hq, 128], k/v [B, Skv, Hkv, 128] (any strides with unit inner stride) -> (o, lse)
std::tuple<Tensor, Tensor> attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, double scale,
                                    int64_t mask, int64_t n_ar, bool return_lse, const OptT& dest_ptr,
                                    int64_t rows_per_dest, const OptT& out) {
  check_bf16_cuda(q, "q"); check_bf16_cuda(k, "k"); check_bf16_cuda(v, "v");
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "q/k/v must be [B, S, H, 128]");
  TORCH_CHECK(q.size(3) == 128 && k.size(3) == 128 && v.size(3) == 128, "head_dim must be 128");
  TORCH_CHECK(q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1, "inner stride must be 1");
  TORCH_CHECK(k.sizes() == v.sizes() && q.size(0) == k.size(0), "shape mismatch");
  for (const Tensor* t : {&q, &k, &v})
    for (int d = 0; d < 3; ++d) TORCH_CHECK(t->stride(d) % 8 == 0, "strides must be multiples of 8");
  const int64_t B = q.size(0), Sq = q.size(1), Hq = q.size(2), Skv = k.size(1), Hkv = k.size(2);
  Tensor o;
  const bool routed = dest_ptr.has_value() && dest_ptr->defined();
  if (out.has_value() && out->defined()) {
    o = *out;
    check_bf16_cuda(o, "out");
    TORCH_CHECK(o.dim() == 4 && o.stride(3) == 1 && o.size(2) == Hq && o.size(3) == 128, "bad out");
  } else {
    TORCH_CHECK(!routed, "routed output needs an explicit `out` describing the destination strides");
    o = at::empty({B, Sq, Hq, 128}, q.options());
  }
  Tensor lse;
  cosmos::AttnArgs a;
  if (return_lse) {
    lse = at::empty({B, Hq, Sq}, q.options().dtype(at::kFloat));
    a.lse = lse.data_ptr<float>();
  } else {
    lse = at::empty({0}, q.options().dtype(at::kFloat));
  }
  a.Q = q.data_ptr(); a.K = k.data_ptr(); a.V = v.data_ptr(); a.O = o.data_ptr();
  a.B = (int)B; a.Sq = (int)Sq; a.Skv = (int)Skv; a.Hq = (int)Hq; a.Hkv = (int)Hkv;
  a.q_stride_b = q.stride(0); a.q_stride_s = q.stride(1); a.q_stride_h = q.stride(2);
  a.k_stride_b = k.stride(0); a.k_stride_s = k.stride(1); a.k_stride_h = k.stride(2);
  a.v_stride_b = v.stride(0); a.v_stride_s = v.stride(1); a.v_stride_h = v.stride(2);
  a.o_stride_b = o.stride(0); a.o_stride_s = o.stride(1); a.o_stride_h = o.stride(2);
  a.scale = (float)scale; a.mask = (int)mask; a.n_ar = (int)n_ar;
  if (routed) {
    TORCH_CHECK(dest_ptr->scalar_type() == at::kLong && dest_ptr->is_cuda() && rows_per_dest > 0 &&
                    dest_ptr->numel() * rows_per_dest >= Sq,
                "dest_ptr must be an int64 CUDA tensor covering all query rows");
    a.dest_ptr = reinterpret_cast<const long long*>(dest_ptr->data_ptr<int64_t>());
    a.rows_per_dest = (int)rows_per_dest;
  }
  a.status = status_tensor(q.get_device()).data_ptr<int>();
  {
    a.exp_emulation = attn_exp_emu();
    a.debug = attn_debug();
  }
  cosmos::flash_attn_fwd(a, cur_stream());
  return {o, lse};
}

// Attention of q [B, Sq, Hq, 128] over several K/V sources in ONE launch (full mask): source s is a contiguous
// [B, lens[s], Hkv, 128] bf16 buffer at device address k_ptrs[s] / v_ptrs[s] (own memory or a peer GPU's symmetric
// buffer), visited in the given order. This is ring-KV context parallelism with the peers' K/V tiles pulled over
// NVLink by the attention kernel's own TMA loads.
Tensor attn_fwd_sources(const Tensor& q, std::vector<int64_t> k_ptrs, std::vector<int64_t> v_ptrs,
                        std::vector<int64_t> lens, int64_t Hkv, double scale, const OptT& out) {
  check_bf16_cuda(q, "q");
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.dim() == 4 && q.size(3) == 128 && q.stride(3) == 1, "q must be [B, Sq, Hq, 128]");
  const size_t n = k_ptrs.size();
  TORCH_CHECK(n >= 1 && n <= 9 && v_ptrs.size() == n && lens.size() == n, "1 to 9 K/V sources with one length each");
  const int64_t B = q.size(0), Sq = q.size(1), Hq = q.size(2);
  Tensor o = (out.has_value() && out->defined()) ? *out : at::empty({B, Sq, Hq, 128}, q.options());
  TORCH_CHECK(o.dim() == 4 && o.stride(3) == 1 && o.size(1) == Sq && o.size(2) == Hq, "bad out");
  cosmos::AttnArgs a;
  a.Q = q.data_ptr(); a.O = o.data_ptr();
  a.B = (int)B; a.Sq = (int)Sq; a.Hq = (int)Hq; a.Hkv = (int)Hkv;
  a.q_stride_b = q.stride(0); a.q_stride_s = q.stride(1); a.q_stride_h = q.stride(2);
  a.o_stride_b = o.stride(0); a.o_stride_s = o.stride(1); a.o_stride_h = o.stride(2);
  a.scale = (float)scale; a.mask = MASK_FULL;
  int64_t total = 0;
  a.n_src = (int)n;
  for (size_t s = 0; s < n; ++s) {
    TORCH_CHECK(lens[s] > 0 && k_ptrs[s] % 16 == 0 && v_ptrs[s] % 16 == 0, "sources need a positive length and 16-byte aligned addresses");
    a.src_k[s] = reinterpret_cast<const void*>(k_ptrs[s]);
    a.src_v[s] = reinterpret_cast<const void*>(v_ptrs[s]);
    a.src_len[s] = (int)lens[s];
    total += lens[s];
  }
  a.Skv = (int)total;
  if (n == 1) {   // the ordinary single-buffer call
    a.n_src = 0;
    a.K = a.src_k[0]; a.V = a.src_v[0];
    a.k_stride_h = a.v_stride_h = 128; a.k_stride_s = a.v_stride_s = Hkv * 128;
    a.k_stride_b = a.v_stride_b = Hkv * 128 * lens[0];
  }
  a.status = status_tensor(q.get_device()).data_ptr<int>();
  cosmos::flash_attn_fwd(a, cur_stream());
  return o;
}

// Flash attention backward: q/k/v/do [B, S, H, 128] (unit inner stride), lse/delta [B, Hq, Sq] fp32
// -> (dq, dk, dv) contiguous bf16.
std::tuple<Tensor, Tensor, Tensor> attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& dout,
                                            const Tensor& lse, const Tensor& delta, double scale, int64_t mask,
                                            int64_t n_ar) {
  check_bf16_cuda(q, "q"); check_bf16_cuda(k, "k"); check_bf16_cuda(v, "v"); check_bf16_cuda(dout, "do");
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4 && dout.dim() == 4, "q/k/v/do must be [B, S, H, 128]");
  TORCH_CHECK(q.size(3) == 128 && k.size(3) == 128 && v.size(3) == 128, "head_dim must be 128");
  TORCH_CHECK(k.sizes() == v.sizes() && q.size(0) == k.size(0) && dout.sizes() == q.sizes(), "shape mismatch");
  for (const Tensor* t : {&q, &k, &v, &dout}) {
    TORCH_CHECK(t->stride(3) == 1, "inner stride must be 1");
    for (int d = 0; d < 3; ++d) TORCH_CHECK(t->stride(d) % 8 == 0, "strides must be multiples of 8");
  }
  const int64_t B = q.size(0), Sq = q.size(1), Hq = q.size(2), Skv = k.size(1), Hkv = k.size(2);
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == B * Hq * Sq,
              "lse must be contiguous fp32 [B, Hq, Sq]");
  TORCH_CHECK(delta.is_cuda() && delta.scalar_type() == at::kFloat && delta.is_contiguous() &&
                  delta.numel() == B * Hq * Sq, "delta must be contiguous fp32 [B, Hq, Sq]");
  Tensor dq = at::empty({B, Sq, Hq, 128}, q.options());
  Tensor dk = at::empty({B, Skv, Hkv, 128}, q.options());
  Tensor dv = at::empty({B, Skv, Hkv, 128}, q.options());
  cosmos::AttnBwdArgs a;
  a.Q = q.data_ptr(); a.K = k.data_ptr(); a.V = v.data_ptr(); a.dO = dout.data_ptr();
  a.lse = lse.data_ptr<float>(); a.delta = delta.data_ptr<float>();
  a.dQ = dq.data_ptr(); a.dK = dk.data_ptr(); a.dV = dv.data_ptr();
  a.B = (int)B; a.Sq = (int)Sq; a.Skv = (int)Skv; a.Hq = (int)Hq; a.Hkv = (int)Hkv;
  a.q_stride_b = q.stride(0); a.q_stride_s = q.stride(1); a.q_stride_h = q.stride(2);
  a.k_stride_b = k.stride(0); a.k_stride_s = k.stride(1); a.k_stride_h = k.stride(2);
  a.v_stride_b = v.stride(0); a.v_stride_s = v.stride(1); a.v_stride_h = v.stride(2);
  a.do_stride_b = dout.stride(0); a.do_stride_s = dout.stride(1); a.do_stride_h = dout.stride(2);
  a.scale = (float)scale; a.mask = (int)mask; a.n_ar = (int)n_ar;
  a.status = status_tensor(q.get_device()).data_ptr<int>();
  cosmos::flash_attn_bwd(a, cur_stream());
  return {dq, dk, dv};
}

std::tuple<Tensor, Tensor> rmsnorm(const Tensor& x, const OptT& gamma, double eps, const OptT& residual) {
  check_bf16_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous(), "x must be contiguous");
  const int64_t d = x.size(-1), rows = x.numel() / d;
  Tensor y = at::empty_like(x);
  Tensor res_out;
  const void* rin = nullptr;
  void* rout = nullptr;
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->is_contiguous() && residual->sizes() == x.sizes(), "bad residual");
    res_out = at::empty_like(x);
    rin = residual->data_ptr();
    rout = res_out.data_ptr();
  } else {
    res_out = at::empty({0}, x.options());
  }
  if (gamma.has_value() && gamma->defined()) TORCH_CHECK(gamma->numel() == d && gamma->is_contiguous());
  cosmos::rmsnorm(x.data_ptr(), opt_ptr(gamma), y.data_ptr(), rows, (int)d, (float)eps, rin, rout,
                  cur_stream());
  return {y, res_out};
}

Tensor adaln_rmsnorm(const Tensor& x, const OptT& gamma, const Tensor& shift, const Tensor& scale,
                     int64_t rows_per_batch, double eps) {
  check_bf16_cuda(x, "x"); check_bf16_cuda(shift, "shift"); check_bf16_cuda(scale, "scale");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous(), "x must be contiguous");
  const int64_t d = x.size(-1), rows = x.numel() / d;
  TORCH_CHECK(shift.size(-1) == d && scale.size(-1) == d && shift.stride(-1) == 1 && scale.stride(-1) == 1);
  Tensor sh = shift.dim() == 1 ? shift.unsqueeze(0) : shift.reshape({-1, d});
  Tensor sc = scale.dim() == 1 ? scale.unsqueeze(0) : scale.reshape({-1, d});
  TORCH_CHECK(sh.stride(0) == sc.stride(0) || sh.size(0) == 1, "shift/scale need equal row strides");
  TORCH_CHECK(sh.size(0) * rows_per_batch >= rows, "modulation rows do not cover x");
  Tensor y = at::empty_like(x);
  cosmos::adaln_rmsnorm(x.data_ptr(), opt_ptr(gamma), sh.data_ptr(), sc.data_ptr(), y.data_ptr(), rows,
                        (int)d, (int)rows_per_batch, sh.size(0) == 1 ? 0 : sh.stride(0), (float)eps,
                        cur_stream());
  return y;
}

// In place on x [rows.., heads, 128]
void mrope_(Tensor x, const OptT& cos_t, const OptT& sin_t, const OptT& gamma, double eps) {
  check_bf16_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() >= 3 && x.size(-1) == 128 && x.stride(-1) == 1 && x.stride(-2) == 128,
              "x must be [..., heads, 128] with packed heads");
  const int64_t heads = x.size(-2);
  const int64_t row_stride = x.stride(-3);
  const int64_t rows = x.numel() / (heads * 128);
  if (x.dim() > 3)
    for (int d = 0; d < x.dim() - 3; ++d)
      TORCH_CHECK(x.stride(d) == x.stride(d + 1) * x.size(d + 1), "leading dims must be collapsible");
  const float* c = nullptr;
  const float* s = nullptr;
  int rr = 0;
  if (cos_t.has_value() && cos_t->defined()) {
    TORCH_CHECK(cos_t->scalar_type() == at::kFloat && cos_t->is_contiguous() && sin_t.has_value() &&
                sin_t->is_contiguous() && cos_t->size(-1) == 64);
    c = cos_t->data_ptr<float>(); s = sin_t->data_ptr<float>(); rr = (int)(cos_t->numel() / 64);
  }
  cosmos::mrope_apply(x.data_ptr(), rows, (int)heads, row_stride, c, s, rr, opt_ptr(gamma), (float)eps,
                      cur_stream());
}

Tensor gated_residual(const Tensor& x, const Tensor& f, const OptT& gate, int64_t rows_per_batch) {
  check_bf16_cuda(x, "x"); check_bf16_cuda(f, "f");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && f.is_contiguous() && x.sizes() == f.sizes());
  const int64_t d = x.size(-1), rows = x.numel() / d;
  Tensor y = at::empty_like(x);
  long long gs = 0;
  if (gate.has_value() && gate->defined()) {
    check_bf16_cuda(*gate, "gate");
    TORCH_CHECK(gate->size(-1) == d && gate->stride(-1) == 1);
    Tensor g2 = gate->dim() == 1 ? gate->unsqueeze(0) : gate->reshape({-1, d});
    gs = g2.size(0) == 1 ? 0 : g2.stride(0);
    TORCH_CHECK(gs % 8 == 0 && g2.size(0) * rows_per_batch >= rows);
  }
  cosmos::gated_residual(x.data_ptr(), f.data_ptr(), opt_ptr(gate), y.data_ptr(), rows, (int)d,
                         (int)rows_per_batch, gs, cur_stream());
  return y;
}

Tensor swiglu(const Tensor& gate_up) {
  check_bf16_cuda(gate_up, "gate_up");
  c10::cuda::CUDAGuard guard(gate_up.device());
  TORCH_CHECK(gate_up.is_contiguous() && gate_up.size(-1) % 16 == 0);
  const int64_t dff = gate_up.size(-1) / 2, rows = gate_up.numel() / (2 * dff);
  auto shape = gate_up.sizes().vec();
  shape.back() = dff;
  Tensor y = at::empty(shape, gate_up.options());
  cosmos::swiglu(gate_up.data_ptr(), y.data_ptr(), rows, (int)dff, cur_stream());
  return y;
}

// ---- backward of the bandwidth kernels
// Returns (dx, part): part [B, blocks, 3, d] fp32 per-block column sums (d shift, d scale, d gamma) when
// `want_cols`, else an empty tensor. gamma / scale optional; scale [B or 1, d] (unit inner stride).
std::tuple<Tensor, Tensor> rmsnorm_bwd(const Tensor& x, const Tensor& dy, const OptT& gamma, const OptT& scale,
                                       int64_t rows_per_batch, double eps, bool want_cols) {
  check_bf16_cuda(x, "x"); check_bf16_cuda(dy, "dy");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous() && x.sizes() == dy.sizes(), "x / dy must be contiguous and alike");
  const int64_t d = x.size(-1), rows = x.numel() / d;
  if (rows_per_batch <= 0) rows_per_batch = rows;
  TORCH_CHECK(rows % rows_per_batch == 0, "rows must be a multiple of rows_per_batch");
  const int64_t B = rows / rows_per_batch;
  long long ms = 0;
  if (gamma.has_value() && gamma->defined()) { check_bf16_cuda(*gamma, "gamma"); TORCH_CHECK(gamma->numel() == d && gamma->is_contiguous()); }
  const void* scp = nullptr;
  if (scale.has_value() && scale->defined()) {
    check_bf16_cuda(*scale, "scale");
    TORCH_CHECK(scale->size(-1) == d && scale->stride(-1) == 1);
    Tensor s2 = scale->dim() == 1 ? scale->unsqueeze(0) : scale->reshape({-1, d});
    TORCH_CHECK(s2.size(0) == 1 || s2.size(0) == B, "scale must have one row or one row per batch");
    ms = s2.size(0) == 1 ? 0 : s2.stride(0);
    TORCH_CHECK(ms % 8 == 0);
    scp = s2.data_ptr();
  }
  Tensor dx = at::empty_like(x);
  Tensor rinv = at::empty({rows}, x.options().dtype(at::kFloat));
  Tensor part = want_cols ? at::empty({B, (int64_t)cosmos::rmsnorm_bwd_blocks((int)rows_per_batch), 3, d},
                                      x.options().dtype(at::kFloat))
                          : at::empty({0}, x.options().dtype(at::kFloat));
  cosmos::rmsnorm_bwd(x.data_ptr(), dy.data_ptr(), opt_ptr(gamma), scp, rows, (int)d, (int)rows_per_batch, ms,
                      (float)eps, dx.data_ptr(), rinv.data_ptr<float>(), want_cols ? part.data_ptr<float>() : nullptr,
                      cur_stream());
  return {dx, part};
}

// y = resid + gate[b] * f  ->  (df, part [B, blocks, d] per-block sums of dy * f)
std::tuple<Tensor, Tensor> gated_residual_bwd(const Tensor& dy, const Tensor& f, const Tensor& gate,
                                              int64_t rows_per_batch) {
  check_bf16_cuda(dy, "dy"); check_bf16_cuda(f, "f"); check_bf16_cuda(gate, "gate");
  c10::cuda::CUDAGuard guard(dy.device());
  TORCH_CHECK(dy.is_contiguous() && f.is_contiguous() && dy.sizes() == f.sizes());
  const int64_t d = dy.size(-1), rows = dy.numel() / d;
  if (rows_per_batch <= 0) rows_per_batch = rows;
  TORCH_CHECK(rows % rows_per_batch == 0, "rows must be a multiple of rows_per_batch");
  const int64_t B = rows / rows_per_batch;
  TORCH_CHECK(gate.size(-1) == d && gate.stride(-1) == 1);
  Tensor g2 = gate.dim() == 1 ? gate.unsqueeze(0) : gate.reshape({-1, d});
  TORCH_CHECK(g2.size(0) == 1 || g2.size(0) == B, "gate must have one row or one row per batch");
  const long long gs = g2.size(0) == 1 ? 0 : g2.stride(0);
  TORCH_CHECK(gs % 8 == 0);
  Tensor df = at::empty_like(dy);
  Tensor part = at::empty({B, (int64_t)cosmos::rmsnorm_bwd_blocks((int)rows_per_batch), d}, dy.options().dtype(at::kFloat));
  cosmos::gated_residual_bwd(dy.data_ptr(), f.data_ptr(), g2.data_ptr(), rows, (int)d, (int)rows_per_batch, gs,
                             df.data_ptr(), part.data_ptr<float>(), cur_stream());
  return {df, part};
}

Tensor swiglu_bwd(const Tensor& gate_up, const Tensor& dy) {
  check_bf16_cuda(gate_up, "gate_up"); check_bf16_cuda(dy, "dy");
  c10::cuda::CUDAGuard guard(gate_up.device());
  TORCH_CHECK(gate_up.is_contiguous() && dy.is_contiguous() && gate_up.size(-1) % 16 == 0 &&
              dy.size(-1) * 2 == gate_up.size(-1) && dy.numel() * 2 == gate_up.numel());
  const int64_t dff = dy.size(-1), rows = dy.numel() / dff;
  Tensor out = at::empty_like(gate_up);
  cosmos::swiglu_bwd(gate_up.data_ptr(), dy.data_ptr(), out.data_ptr(), rows, (int)dff, cur_stream());
  return out;
}

static void rope_tables(const OptT& cos_t, const OptT& sin_t, const float*& c, const float*& s, int& rr) {
  c = s = nullptr;
  rr = 1;
  if (cos_t.has_value() && cos_t->defined()) {
    TORCH_CHECK(sin_t.has_value() && sin_t->defined(), "cos without sin");
    TORCH_CHECK(cos_t->is_cuda() && cos_t->scalar_type() == at::kFloat && cos_t->is_contiguous() && cos_t->size(-1) == 64 &&
                sin_t->is_cuda() && sin_t->scalar_type() == at::kFloat && sin_t->is_contiguous() && sin_t->sizes() == cos_t->sizes(),
                "cos/sin must be contiguous fp32 [rope_rows, 64]");
    c = cos_t->data_ptr<float>();
    s = sin_t->data_ptr<float>();
    rr = (int)(cos_t->numel() / 64);
  }
}

// qkv [rows.., Hq + 2 Hkv, 128] -> (q [rows, Hq, 128], k [rows, Hkv, 128], v [rows, Hkv, 128])
std::tuple<Tensor, Tensor, Tensor> qkv_post_fwd(const Tensor& qkv, int64_t n_q_heads, const OptT& cos_t,
                                                const OptT& sin_t, const OptT& gamma_q, const OptT& gamma_k,
                                                double eps) {
  check_bf16_cuda(qkv, "qkv");
  c10::cuda::CUDAGuard guard(qkv.device());
  TORCH_CHECK(qkv.dim() >= 3 && qkv.size(-1) == 128 && qkv.is_contiguous(), "qkv must be contiguous [.., heads, 128]");
  const int64_t heads = qkv.size(-2), rows = qkv.numel() / (heads * 128), Hq = n_q_heads;
  TORCH_CHECK(Hq > 0 && heads > Hq && (heads - Hq) % 2 == 0, "bad head split");
  const int64_t Hkv = (heads - Hq) / 2;
  const float *c, *s;
  int rr;
  rope_tables(cos_t, sin_t, c, s, rr);
  Tensor q = at::empty({rows, Hq, 128}, qkv.options()), k = at::empty({rows, Hkv, 128}, qkv.options()),
         v = at::empty({rows, Hkv, 128}, qkv.options());
  cosmos::qkv_post_fwd(qkv.data_ptr(), rows, (int)Hq, (int)Hkv, c, s, rr, opt_ptr(gamma_q), opt_ptr(gamma_k),
                       (float)eps, q.data_ptr(), k.data_ptr(), v.data_ptr(), cur_stream());
  return {q, k, v};
}

// -> (d_qkv like qkv, part [blocks, 2, 128] per-block sums of d gamma_q / d gamma_k)
std::tuple<Tensor, Tensor> qkv_post_bwd(const Tensor& qkv, const Tensor& dq, const Tensor& dk, const Tensor& dv,
                                        const OptT& cos_t, const OptT& sin_t, const OptT& gamma_q,
                                        const OptT& gamma_k, double eps) {
  check_bf16_cuda(qkv, "qkv"); check_bf16_cuda(dq, "dq"); check_bf16_cuda(dk, "dk"); check_bf16_cuda(dv, "dv");
  c10::cuda::CUDAGuard guard(qkv.device());
  TORCH_CHECK(qkv.is_contiguous() && dq.is_contiguous() && dk.is_contiguous() && dv.is_contiguous());
  const int64_t heads = qkv.size(-2), rows = qkv.numel() / (heads * 128);
  const int64_t Hq = dq.numel() / (rows * 128), Hkv = dk.numel() / (rows * 128);
  TORCH_CHECK(Hq + 2 * Hkv == heads && dv.numel() == dk.numel(), "gradient shapes do not match qkv");
  const float *c, *s;
  int rr;
  rope_tables(cos_t, sin_t, c, s, rr);
  Tensor d_qkv = at::empty_like(qkv);
  const int blocks = cosmos::qkv_post_bwd_blocks(rows, (int)Hq, (int)Hkv);
  Tensor part = at::empty({blocks, 2, 128}, qkv.options().dtype(at::kFloat));
  cosmos::qkv_post_bwd(qkv.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), rows, (int)Hq, (int)Hkv, c, s, rr,
                       opt_ptr(gamma_q), opt_ptr(gamma_k), (float)eps, d_qkv.data_ptr(), part.data_ptr<float>(),
                       cur_stream());
  return {d_qkv, part};
}

// x fp32 [rows, d] updated in place: x += dt * cfg(vc, vu)
void cfg_unipc_step_(Tensor x, const Tensor& vc, const OptT& vu, Tensor L, const Tensor& P, Tensor P2, double guidance,
                     bool normalize, std::vector<double> coef, bool correct, bool final_step, bool has_p, bool has_p2) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.is_contiguous() && x.dim() == 2, "x must be fp32 [rows, d]");
  check_bf16_cuda(vc, "vc");
  TORCH_CHECK(vc.is_contiguous() && vc.numel() == x.numel(), "vc must match x");
  if (vu.has_value() && vu->defined()) TORCH_CHECK(vu->is_contiguous() && vu->numel() == x.numel(), "vu must match x");
  for (const Tensor* t : {static_cast<const Tensor*>(&L), &P, static_cast<const Tensor*>(&P2)})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == x.numel(),
                "L, P, P2 must be fp32 tensors of x's size");
  TORCH_CHECK(coef.size() == 8, "eight coefficients expected");
  float c8[8];
  for (int i = 0; i < 8; ++i) c8[i] = (float)coef[i];
  cosmos::cfg_unipc_step(x.data_ptr<float>(), vc.data_ptr(), opt_ptr(vu), L.data_ptr<float>(), P.data_ptr<float>(),
                         P2.data_ptr<float>(), (float)guidance, normalize ? 1 : 0, c8, correct, final_step, has_p, has_p2,
                         x.size(0), (int)x.size(1), cur_stream());
}

void cfg_euler_step_(Tensor x, const Tensor& vc, const OptT& vu, double guidance, double dt, bool normalize) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.is_contiguous(), "x must be fp32 contiguous");
  check_bf16_cuda(vc, "vc");
  TORCH_CHECK(vc.is_contiguous() && vc.numel() == x.numel());
  if (vu.has_value() && vu->defined()) { check_bf16_cuda(*vu, "vu"); TORCH_CHECK(vu->is_contiguous() && vu->numel() == x.numel()); }
  const int64_t d = x.size(-1), rows = x.numel() / d;
  cosmos::cfg_euler_step(x.data_ptr<float>(), vc.data_ptr(), opt_ptr(vu), (float)guidance, (float)dt,
                         normalize ? 1 : 0, rows, (int)d, cur_stream());
}

void l2_flush_(Tensor buf) {
  c10::cuda::CUDAGuard guard(buf.device());
  TORCH_CHECK(buf.is_cuda() && buf.is_contiguous());
  cosmos::l2_flush(buf.data_ptr(), buf.nbytes(), cur_stream());
}

// Decode attention over a paged KV cache; `scratch` (fp32) holds the split-KV partials.
// impl: 0 = tensor-core kernel (TMA + tcgen05) when page size and GQA group allow it, 1 = CUDA-core kernel
Tensor paged_decode(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& block_table,
                    const Tensor& seq_lens, double scale, int64_t n_splits, const OptT& scratch, int64_t impl) {
  check_bf16_cuda(q, "q"); check_bf16_cuda(k_cache, "k_cache"); check_bf16_cuda(v_cache, "v_cache");
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.dim() == 3 && q.size(2) == 128 && q.is_contiguous(), "q must be contiguous [B, Hq, 128]");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.size(3) == 128 && k_cache.is_contiguous() &&
                  v_cache.is_contiguous() && v_cache.sizes() == k_cache.sizes(),
              "caches must be contiguous [pages, Hkv, page_size, 128]");
  TORCH_CHECK(block_table.scalar_type() == at::kInt && block_table.is_cuda() && block_table.is_contiguous() &&
                  block_table.dim() == 2 && block_table.size(0) == q.size(0), "block_table must be int32 [B, max_pages]");
  TORCH_CHECK(seq_lens.scalar_type() == at::kInt && seq_lens.is_cuda() && seq_lens.numel() == q.size(0));
  cosmos::PagedDecodeArgs a;
  a.q = q.data_ptr(); a.k_cache = k_cache.data_ptr(); a.v_cache = v_cache.data_ptr();
  a.block_table = block_table.data_ptr<int>(); a.seq_lens = seq_lens.data_ptr<int>();
  a.B = (int)q.size(0); a.Hq = (int)q.size(1); a.Hkv = (int)k_cache.size(1);
  a.page_size = (int)k_cache.size(2); a.max_pages = (int)block_table.size(1);
  a.scale = (float)scale; a.n_splits = (int)n_splits;
  a.num_pages = (int)k_cache.size(0); a.impl = (int)impl;
  a.status = status_tensor(q.get_device()).data_ptr<int>();
  Tensor out = at::empty_like(q);
  a.out = out.data_ptr();
  Tensor ws;
  if (n_splits > 1) {
    const size_t need = cosmos::paged_decode_scratch_bytes(a.B, a.Hq, a.n_splits);
    if (scratch.has_value() && scratch->defined()) {
      TORCH_CHECK(scratch->is_cuda() && scratch->is_contiguous() && scratch->nbytes() >= need, "scratch too small");
      ws = *scratch;
    } else {
      ws = at::empty({(int64_t)(need / 4)}, q.options().dtype(at::kFloat));
    }
    a.scratch = ws.data_ptr(); a.scratch_bytes = ws.nbytes();
  }
  cosmos::paged_decode(a, cur_stream());
  return out;
}

int64_t paged_decode_pick_splits(int64_t B, int64_t Hkv, int64_t max_len, int64_t impl) {
  return impl == 1 ? cosmos::paged_decode_pick_splits((int)B, (int)Hkv, (int)max_len)
                   : cosmos::paged_decode_tc_pick_splits((int)B, (int)Hkv, (int)max_len);
}

// Causal 3x3x3 convolution as an implicit GEMM. x: padded channels-last volume [F, Hp, Wp, C]
// (C % 64 == 0; F includes `tpad` = 2 leading context frames); w: [Cout, 27 * C]; out: a padded
// volume [F, Hp, Wp, Cout] whose interior rows are written (border rows are left untouched);
// resid (optional) has the layout of out and is added.
void conv3d_cl(const Tensor& x, const Tensor& w, const OptT& bias, const OptT& resid, Tensor out, int64_t tpad) {
  check_bf16_cuda(x, "x"); check_bf16_cuda(w, "w"); check_bf16_cuda(out, "out");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 4 && x.is_contiguous() && out.dim() == 4 && out.is_contiguous(), "volumes must be contiguous [F, Hp, Wp, C]");
  const int64_t F = x.size(0), Hp = x.size(1), Wp = x.size(2), C = x.size(3), Cout = out.size(3);
  TORCH_CHECK(out.size(0) == F && out.size(1) == Hp && out.size(2) == Wp, "out must have the padded shape of x");
  TORCH_CHECK(w.dim() == 2 && w.is_contiguous() && w.size(0) == Cout && w.size(1) == 27 * C, "w must be [Cout, 27 * C]");
  TORCH_CHECK(F * Hp * Wp < (1ll << 31), "volume too large for 32-bit row indices; decode in temporal chunks");
  cosmos::GemmArgs g;
  g.A = x.data_ptr(); g.B = w.data_ptr(); g.C = out.data_ptr();
  g.M = (int)(F * Hp * Wp); g.N = (int)Cout; g.K = (int)(27 * C);
  g.lda = C; g.ldb = 27 * C; g.ldc = Cout;
  g.epi = EPI_CONV;
  g.conv_c = (int)C; g.conv_hp = (int)Hp; g.conv_wp = (int)Wp; g.conv_tpad = (int)tpad;
  if (bias.has_value() && bias->defined()) {
    check_bf16_cuda(*bias, "bias");
    TORCH_CHECK(bias->numel() == Cout && bias->is_contiguous());
    g.bias = bias->data_ptr();
  }
  if (resid.has_value() && resid->defined()) {
    check_bf16_cuda(*resid, "resid");
    TORCH_CHECK(resid->is_contiguous() && resid->sizes() == out.sizes());
    g.R = resid->data_ptr(); g.ldr = Cout;
  }
  g.status = status_tensor(x.get_device()).data_ptr<int>();
  cosmos::gemm_bf16(g, cur_stream());
}

Tensor rmsnorm_silu(const Tensor& x, const Tensor& gamma, double eps) {
  check_bf16_cuda(x, "x"); check_bf16_cuda(gamma, "gamma");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && gamma.is_contiguous() && gamma.numel() == x.size(-1));
  Tensor y = at::empty_like(x);
  cosmos::rmsnorm_silu(x.data_ptr(), gamma.data_ptr(), y.data_ptr(), x.numel() / x.size(-1), (int)x.size(-1),
                       (float)eps, cur_stream());
  return y;
}

void upsample_cl(const Tensor& src, Tensor dst, int64_t tpad, bool temporal, bool first_chunk) {
  check_bf16_cuda(src, "src"); check_bf16_cuda(dst, "dst");
  c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.dim() == 4 && dst.dim() == 4 && src.is_contiguous() && dst.is_contiguous() && src.size(3) == dst.size(3));
  const int64_t hs = src.size(1) - 2, ws = src.size(2) - 2;
  TORCH_CHECK(dst.size(1) == 2 * hs + 2 && dst.size(2) == 2 * ws + 2, "dst must be the x2 padded volume");
  const int64_t t_src = src.size(0) - tpad, t_dst = dst.size(0) - tpad;
  const int64_t want = temporal ? (first_chunk ? 2 * t_src - 1 : 2 * t_src) : t_src;
  TORCH_CHECK(t_dst == want, "dst frame count mismatch");
  cosmos::upsample_cl(src.data_ptr(), dst.data_ptr(), (int)t_dst, (int)hs, (int)ws, (int)src.size(3), (int)tpad,
                      temporal ? 1 : 0, first_chunk ? 1 : 0, cur_stream());
}

// x: padded CL volume [T + 2, H + 2, W + 2, 64]; w [3, 27, 64] fp32; bias [3] fp32 -> uint8 [T, H, W, 3]
Tensor conv_out_rgb(const Tensor& x, const Tensor& w, const Tensor& bias) {
  check_bf16_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 4 && x.is_contiguous() && x.size(3) == 64, "x must be [T+2, H+2, W+2, 64]");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kFloat && w.is_contiguous() && w.numel() == 3 * 27 * 64);
  TORCH_CHECK(bias.is_cuda() && bias.scalar_type() == at::kFloat && bias.numel() == 3);
  const int64_t T = x.size(0) - 2, H = x.size(1) - 2, W = x.size(2) - 2;
  Tensor out = at::empty({T, H, W, 3}, x.options().dtype(at::kByte));
  cosmos::conv_out_rgb(x.data_ptr(), w.data_ptr<float>(), bias.data_ptr<float>(), out.data_ptr(), (int)T, (int)H,
                       (int)W, cur_stream());
  return out;
}

const long long* ptr_table(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kLong && t.is_contiguous(), name,
              " must be a contiguous int64 CUDA tensor of addresses");
  return reinterpret_cast<const long long*>(t.data_ptr<int64_t>());
}

void comm_barrier(const Tensor& pads, int64_t rank, int64_t world, int64_t slot, int64_t epoch) {
  c10::cuda::CUDAGuard guard(pads.device());
  TORCH_CHECK(pads.numel() >= world, "one signal pad address per rank is needed");
  cosmos::comm_barrier(ptr_table(pads, "pads"), (int)rank, (int)world, (int)slot, (int)epoch,
                       status_tensor(pads.get_device()).data_ptr<int>(), cur_stream());
}

void comm_barrier_counted(const Tensor& pads, int64_t rank, int64_t world, int64_t slot, Tensor counters) {
  c10::cuda::CUDAGuard guard(pads.device());
  TORCH_CHECK(pads.numel() >= world, "one signal pad address per rank is needed");
  TORCH_CHECK(counters.is_cuda() && counters.scalar_type() == at::kInt && counters.numel() > slot, "counters: int32 per slot");
  cosmos::comm_barrier_counted(ptr_table(pads, "pads"), (int)rank, (int)world, (int)slot, counters.data_ptr<int>(),
                               status_tensor(pads.get_device()).data_ptr<int>(), cur_stream());
}

void allreduce_oneshot(const Tensor& bufs, const Tensor& pads, Tensor out, int64_t rank, int64_t world,
                       int64_t slot, int64_t epoch, const OptT& counters) {
  check_bf16_cuda(out, "out");
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_contiguous() && bufs.numel() >= world && pads.numel() >= world);
  int* cnt = nullptr;
  if (counters.has_value() && counters->defined()) {
    TORCH_CHECK(counters->is_cuda() && counters->scalar_type() == at::kInt && counters->numel() >= slot + 8);
    cnt = counters->data_ptr<int>();
  }
  cosmos::allreduce_oneshot(ptr_table(bufs, "bufs"), ptr_table(pads, "pads"), out.data_ptr(), out.numel(),
                            (int)rank, (int)world, (int)slot, (int)epoch, cnt,
                            status_tensor(out.get_device()).data_ptr<int>(), cur_stream());
}

void kv_cache_write(const Tensor& k, const Tensor& v, const Tensor& slots, Tensor k_cache, Tensor v_cache) {
  check_bf16_cuda(k, "k"); check_bf16_cuda(v, "v"); check_bf16_cuda(k_cache, "k_cache"); check_bf16_cuda(v_cache, "v_cache");
  c10::cuda::CUDAGuard guard(k.device());
  TORCH_CHECK(k.is_contiguous() && v.is_contiguous() && k.sizes() == v.sizes() && k.dim() == 3 && k.size(2) == 128);
  TORCH_CHECK(k_cache.is_contiguous() && v_cache.is_contiguous() && k_cache.dim() == 4 && k_cache.size(1) == k.size(1) &&
              k_cache.size(3) == 128 && v_cache.sizes() == k_cache.sizes());
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == at::kLong && slots.is_contiguous() && slots.numel() == k.size(0));
  cosmos::kv_cache_write(k.data_ptr(), v.data_ptr(), reinterpret_cast<const long long*>(slots.data_ptr<int64_t>()),
                         k_cache.data_ptr(), v_cache.data_ptr(), k.size(0), (int)k.size(1), (int)k_cache.size(2),
                         k_cache.size(0) * k_cache.size(2), status_tensor(k.get_device()).data_ptr<int>(), cur_stream());
}

Tensor decode_qkv_post(const Tensor& qkv, int64_t n_q_heads, const Tensor& cos_t, const Tensor& sin_t,
                       const Tensor& gamma_q, const Tensor& gamma_k, double eps, const Tensor& slots,
                       Tensor k_cache, Tensor v_cache) {
  check_bf16_cuda(qkv, "qkv"); check_bf16_cuda(gamma_q, "gamma_q"); check_bf16_cuda(gamma_k, "gamma_k");
  check_bf16_cuda(k_cache, "k_cache"); check_bf16_cuda(v_cache, "v_cache");
  c10::cuda::CUDAGuard guard(qkv.device());
  TORCH_CHECK(qkv.dim() == 3 && qkv.size(2) == 128 && qkv.is_contiguous(), "qkv must be contiguous [B, Hq + 2 Hkv, 128]");
  const int64_t B = qkv.size(0), Hq = n_q_heads;
  TORCH_CHECK(Hq > 0 && (qkv.size(1) - Hq) > 0 && (qkv.size(1) - Hq) % 2 == 0, "bad head split");
  const int64_t Hkv = (qkv.size(1) - Hq) / 2;
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous() && k_cache.size(1) == Hkv &&
              k_cache.size(3) == 128 && v_cache.sizes() == k_cache.sizes(), "caches must be contiguous [pages, Hkv, page_size, 128]");
  TORCH_CHECK(cos_t.is_cuda() && cos_t.scalar_type() == at::kFloat && cos_t.is_contiguous() && cos_t.numel() == B * 64 &&
              sin_t.is_cuda() && sin_t.scalar_type() == at::kFloat && sin_t.is_contiguous() && sin_t.numel() == B * 64,
              "cos/sin must be contiguous fp32 [B, 64]");
  TORCH_CHECK(gamma_q.numel() == 128 && gamma_k.numel() == 128 && gamma_q.is_contiguous() && gamma_k.is_contiguous());
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == at::kLong && slots.is_contiguous() && slots.numel() == B);
  Tensor q = at::empty({B, Hq, 128}, qkv.options());
  cosmos::decode_qkv_post(qkv.data_ptr(), (int)B, (int)Hq, (int)Hkv, cos_t.data_ptr<float>(), sin_t.data_ptr<float>(),
                          gamma_q.data_ptr(), gamma_k.data_ptr(), (float)eps,
                          reinterpret_cast<const long long*>(slots.data_ptr<int64_t>()), q.data_ptr(),
                          k_cache.data_ptr(), v_cache.data_ptr(), (int)k_cache.size(2), k_cache.size(0) * k_cache.size(2),
                          status_tensor(qkv.get_device()).data_ptr<int>(), cur_stream());
  return q;
}

// QKV projection of a decode step and its post-processing without the bf16 round trip: the skinny GEMM leaves its
// split-K partial sums, and the q/k norm + rotary + cache-write kernel reduces them while it reads (one launch fewer
// per layer than gemm + decode_qkv_post). h [B, K]; w [(Hq + 2 Hkv) * 128, K]. Returns q [B, Hq, 128].
Tensor gemm_decode_qkv_post(const Tensor& h, const Tensor& w, int64_t n_q_heads, const Tensor& cos_t, const Tensor& sin_t,
                            const Tensor& gamma_q, const Tensor& gamma_k, double eps, const Tensor& slots,
                            Tensor k_cache, Tensor v_cache) {
  check_bf16_cuda(h, "h"); check_bf16_cuda(w, "w");
  c10::cuda::CUDAGuard guard(h.device());
  Tensor A = as_2d(h);
  const int64_t M = A.size(0), K = A.size(1), N = w.size(0);
  TORCH_CHECK(w.dim() == 2 && w.size(1) == K && A.stride(1) == 1 && w.stride(1) == 1 && N % 128 == 0, "h [B, K], w [heads * 128, K]");
  const int ks = cosmos::gemm_pick_k_splits((int)M, (int)N, (int)K, EPI_PLAIN);
  const int64_t heads = N / 128, Hq = n_q_heads, Hkv = (heads - Hq) / 2;
  if (ks <= 1 || A.stride(0) % 8 != 0 || w.stride(0) % 8 != 0) {
    Tensor qkv = gemm(A, w, {}, EPI_PLAIN, {}, {}, 0, {});
    return decode_qkv_post(qkv.view({M, heads, 128}), n_q_heads, cos_t, sin_t, gamma_q, gamma_k, eps, slots, k_cache, v_cache);
  }
  check_bf16_cuda(gamma_q, "gamma_q"); check_bf16_cuda(gamma_k, "gamma_k");
  check_bf16_cuda(k_cache, "k_cache"); check_bf16_cuda(v_cache, "v_cache");
  TORCH_CHECK(Hq > 0 && Hkv > 0 && Hq + 2 * Hkv == heads, "bad head split");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous() && k_cache.size(1) == Hkv &&
              k_cache.size(3) == 128 && v_cache.sizes() == k_cache.sizes(), "caches must be contiguous [pages, Hkv, page_size, 128]");
  TORCH_CHECK(cos_t.is_cuda() && cos_t.scalar_type() == at::kFloat && cos_t.is_contiguous() && cos_t.numel() == M * 64 &&
              sin_t.is_cuda() && sin_t.scalar_type() == at::kFloat && sin_t.is_contiguous() && sin_t.numel() == M * 64,
              "cos/sin must be contiguous fp32 [B, 64]");
  TORCH_CHECK(gamma_q.numel() == 128 && gamma_k.numel() == 128 && gamma_q.is_contiguous() && gamma_k.is_contiguous());
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == at::kLong && slots.is_contiguous() && slots.numel() == M);
  Tensor partial = at::empty({ks, M, N}, A.options().dtype(at::kFloat));
  cosmos::GemmArgs g;
  g.A = A.data_ptr(); g.B = w.data_ptr(); g.C = nullptr;
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.lda = A.stride(0); g.ldb = w.stride(0); g.ldc = N;
  g.epi = EPI_PLAIN;
  g.k_splits = ks; g.partial = partial.data_ptr<float>(); g.partial_only = true;
  g.status = status_tensor(A.get_device()).data_ptr<int>();
  cosmos::gemm_bf16(g, cur_stream());
  Tensor q = at::empty({M, Hq, 128}, A.options());
  cosmos::decode_qkv_post(nullptr, (int)M, (int)Hq, (int)Hkv, cos_t.data_ptr<float>(), sin_t.data_ptr<float>(),
                          gamma_q.data_ptr(), gamma_k.data_ptr(), (float)eps,
                          reinterpret_cast<const long long*>(slots.data_ptr<int64_t>()), q.data_ptr(),
                          k_cache.data_ptr(), v_cache.data_ptr(), (int)k_cache.size(2), k_cache.size(0) * k_cache.size(2),
                          status_tensor(A.get_device()).data_ptr<int>(), cur_stream(), partial.data_ptr<float>(), ks);
  return q;
}

bool bounds_check_enabled() { return cosmos::bounds_check_enabled(); }
void gemm_set_grid_limit(int64_t max_ctas) { cosmos::gemm_set_grid_limit((int)max_ctas); }
// A/B switches for timing and tests: CTA-pair GEMM tiles on/off, attention forward variant bits.
void gemm_set_cta_pair(bool on) { cosmos::gemm_set_cta_pair(on); }
// Decode-step sampling: the 64 best penalised logits of this rank's vocabulary shard per sequence ...
Tensor sample_topk(const Tensor& logits, const OptT& seen_any, const OptT& seen_out, const OptT& tokens,
                   const OptT& presence, const OptT& repetition, int64_t vocab_offset) {
  check_bf16_cuda(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "logits must be [B, V] with unit column stride");
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t B = logits.size(0), V = logits.size(1);
  auto flags = [&](const OptT& t, const char* name) -> void* {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->element_size() == 1 && t->numel() == B * V, name,
                " must be a contiguous [B, V] tensor of 1-byte flags");
    return t->data_ptr();
  };
  auto vecf = [&](const OptT& t, const char* name) -> const float* {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == B, name,
                " must be a float tensor [B]");
    return t->data_ptr<float>();
  };
  const long long* tok = nullptr;
  if (tokens.has_value() && tokens->defined()) {
    TORCH_CHECK(tokens->is_cuda() && tokens->scalar_type() == at::kLong && tokens->is_contiguous() && tokens->numel() == B,
                "tokens must be an int64 tensor [B]");
    tok = reinterpret_cast<const long long*>(tokens->data_ptr<int64_t>());
  }
  Tensor cand = at::empty({B, 64, 2}, logits.options().dtype(at::kFloat));
  cosmos::sample_topk(logits.data_ptr(), logits.stride(0), (int)B, (int)V, flags(seen_any, "seen_any"),
                      flags(seen_out, "seen_out"), tok, vecf(presence, "presence"), vecf(repetition, "repetition"),
                      (int)vocab_offset, cand.data_ptr(), cur_stream());
  return cand;
}

// ... and the draw among the candidates of all shards (cand [n_src * B, 64, 2], source-major) into tokens_out.
void sample_pick_(const Tensor& cand, int64_t n_src, const Tensor& temperature, const Tensor& top_k, const Tensor& top_p,
                  const Tensor& noise, int64_t vocab_size, Tensor tokens_out) {
  TORCH_CHECK(cand.is_cuda() && cand.scalar_type() == at::kFloat && cand.is_contiguous() && cand.dim() == 3 &&
              cand.size(1) == 64 && cand.size(2) == 2 && cand.size(0) % n_src == 0, "cand must be [n_src * B, 64, 2] float");
  c10::cuda::CUDAGuard guard(cand.device());
  const int64_t B = cand.size(0) / n_src;
  TORCH_CHECK(temperature.scalar_type() == at::kFloat && temperature.numel() == B && temperature.is_contiguous() &&
              top_p.scalar_type() == at::kFloat && top_p.numel() == B && top_p.is_contiguous() &&
              top_k.scalar_type() == at::kLong && top_k.numel() == B && top_k.is_contiguous(),
              "temperature / top_p float [B], top_k int64 [B]");
  TORCH_CHECK(noise.scalar_type() == at::kFloat && noise.dim() == 2 && noise.size(0) == B && noise.size(1) >= 64 &&
              noise.stride(1) == 1, "noise must be float [B, >= 64]");
  TORCH_CHECK(tokens_out.scalar_type() == at::kLong && tokens_out.numel() == B && tokens_out.is_contiguous(),
              "tokens_out must be int64 [B]");
  cosmos::sample_pick(cand.data_ptr(), (int)n_src, (int)B, temperature.data_ptr<float>(),
                      reinterpret_cast<const long long*>(top_k.data_ptr<int64_t>()), top_p.data_ptr<float>(),
                      noise.data_ptr<float>(), noise.stride(0), (int)vocab_size,
                      reinterpret_cast<long long*>(tokens_out.data_ptr<int64_t>()), cur_stream());
}

void gemm_set_debug(int64_t bits) { cosmos::gemm_set_debug((int)bits); }
// Split count that the skinny-GEMM path would use for this problem (1 = no split); host-side, needs no device.
int64_t gemm_pick_k_splits(int64_t M, int64_t N, int64_t K, int64_t epi) {
  return cosmos::gemm_pick_k_splits((int)M, (int)N, (int)K, (int)epi);
}
void set_pdl(bool on) { cosmos::set_pdl(on); }
void attn_set_cta_pair(bool on) { cosmos::attn_set_cta_pair(on); }
void attn_set_exp_emulation(int64_t v) { attn_exp_emu() = (int)v; }
void attn_set_debug(int64_t v) { attn_debug() = (int)v; }

// ok[i] = 1 if 0 <= idx[i] < limit[i] (always 1 in a build without the checks); a failed check also
// records its status code, exactly as inside the kernels. No memory is addressed through idx.
Tensor bounds_check_selftest(const Tensor& idx, const Tensor& limit) {
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kLong && idx.is_contiguous() && limit.is_cuda() &&
              limit.scalar_type() == at::kLong && limit.is_contiguous() && limit.numel() == idx.numel());
  c10::cuda::CUDAGuard guard(idx.device());
  Tensor ok = at::empty({idx.numel()}, idx.options().dtype(at::kInt));
  cosmos::bounds_check_selftest(reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()),
                                reinterpret_cast<const long long*>(limit.data_ptr<int64_t>()), ok.data_ptr<int>(),
                                (int)idx.numel(), status_tensor(idx.get_device()).data_ptr<int>(), cur_stream());
  return ok;
}

// mode 0: reduce + update; mode 1: reduce into `reduced` and add sum(g^2) to sq; mode 2: update from `reduced`
void rs_adamw(const Tensor& grads, int64_t world, int64_t shard_off, Tensor master, Tensor m, Tensor v,
              Tensor param_shard, double grad_scale, double lr, double b1, double b2, double eps, double wd,
              int64_t step, int64_t mode, const OptT& sq, const OptT& reduced) {
  c10::cuda::CUDAGuard guard(master.device());
  TORCH_CHECK(master.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat);
  check_bf16_cuda(param_shard, "param_shard");
  const int64_t n = master.numel();
  TORCH_CHECK(m.numel() == n && v.numel() == n && param_shard.numel() == n, "shard size mismatch");
  TORCH_CHECK(master.is_contiguous() && m.is_contiguous() && v.is_contiguous() && param_shard.is_contiguous());
  float* sqp = nullptr;
  float* redp = nullptr;
  if (mode == 1) {
    // sum of squares of the reduced gradient; the reduced values are kept only when `reduced` is given
    TORCH_CHECK(sq.has_value() && sq->defined(), "mode 1 needs the sum-of-squares accumulator");
    sqp = sq->data_ptr<float>();
    if (reduced.has_value() && reduced->defined()) {
      TORCH_CHECK(reduced->numel() == n && reduced->scalar_type() == at::kFloat);
      redp = reduced->data_ptr<float>();
    }
  } else if (mode == 2) {
    TORCH_CHECK(reduced.has_value() && reduced->numel() == n && reduced->scalar_type() == at::kFloat);
    redp = reduced->data_ptr<float>();
  }
  cosmos::rs_adamw(ptr_table(grads, "grads"), (int)world, shard_off, n, master.data_ptr<float>(),
                   m.data_ptr<float>(), v.data_ptr<float>(), param_shard.data_ptr(), (float)grad_scale, (float)lr,
                   (float)b1, (float)b2, (float)eps, (float)wd, (int)step, sqp, redp, cur_stream());
}

// ---- fused communication ops (comm.cu) ----
// grads / bufs: int64 CUDA tensors with one device address per rank; mc_ptr: NVLink multicast address of the same
// symmetric buffer (0 = none: plain peer loads).
void reduce_scatter_pull(const Tensor& grads, int64_t mc_ptr, int64_t world, int64_t shard_off, Tensor out,
                         bool accumulate, double scale, const OptT& sq) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.is_contiguous(), "out must be contiguous fp32");
  float* sqp = nullptr;
  if (sq.has_value() && sq->defined()) {
    TORCH_CHECK(sq->is_cuda() && sq->scalar_type() == at::kFloat && sq->numel() >= 1);
    sqp = sq->data_ptr<float>();
  }
  cosmos::reduce_scatter_pull(ptr_table(grads, "grads"), reinterpret_cast<const void*>(mc_ptr), (int)world, shard_off,
                              out.numel(), out.data_ptr<float>(), accumulate, (float)scale, sqp, cur_stream());
}

void adamw_shard(const Tensor& grad, Tensor master, Tensor m, Tensor v, Tensor param, double grad_scale, double lr,
                 double b1, double b2, double eps, double wd, int64_t step) {
  c10::cuda::CUDAGuard guard(grad.device());
  const int64_t n = grad.numel();
  TORCH_CHECK(grad.scalar_type() == at::kFloat && grad.is_contiguous() && master.numel() == n && m.numel() == n &&
                  v.numel() == n && param.numel() == n && param.scalar_type() == at::kBFloat16 &&
                  master.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat &&
                  master.is_contiguous() && m.is_contiguous() && v.is_contiguous() && param.is_contiguous(),
              "adamw_shard: fp32 grad / master / moments and a bf16 parameter shard of one length");
  cosmos::adamw_shard(grad.data_ptr<float>(), n, master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                      param.data_ptr(), (float)grad_scale, (float)lr, (float)b1, (float)b2, (float)eps, (float)wd,
                      (int)step, cur_stream());
}

// x_new = residual + sum over ranks of (a w^T), h = rmsnorm(x_new) * gamma -> (h, x_new). `own` is this rank's
// symmetric buffer ([M, N] bf16) that the peers read (`bufs` = its addresses on every rank). A skinny problem runs
// split-K and the all-reduce kernel sums the fp32 partials itself; otherwise the GEMM epilogue writes `own`.
// With `a` undefined-size-0 semantics are not supported: a is always given.
std::tuple<Tensor, Tensor> gemm_allreduce_norm(const Tensor& A_, const Tensor& W, const OptT& residual,
                                               const OptT& gamma, double eps, const Tensor& bufs, int64_t mc_ptr,
                                               Tensor own, const Tensor& pads, int64_t rank, int64_t world,
                                               int64_t slot, Tensor counters, bool want_norm) {
  check_bf16_cuda(A_, "a"); check_bf16_cuda(W, "w"); check_bf16_cuda(own, "own");
  c10::cuda::CUDAGuard guard(A_.device());
  Tensor A = as_2d(A_);
  const int64_t M = A.size(0), K = A.size(1), N = W.size(0);
  TORCH_CHECK(W.dim() == 2 && W.size(1) == K && A.stride(1) == 1 && W.stride(1) == 1, "a [.., K] and w [N, K] expected");
  TORCH_CHECK(A.stride(0) % 8 == 0 && W.stride(0) % 8 == 0 && N % 8 == 0 && N <= 8192, "rows must be 16-byte aligned, N <= 8192");
  TORCH_CHECK(own.is_contiguous() && own.numel() >= M * N, "own buffer too small");
  TORCH_CHECK(counters.is_cuda() && counters.scalar_type() == at::kInt && counters.numel() >= 64, "counters: int32[64]");
  const void* Rp = nullptr;
  Tensor R;
  if (residual.has_value() && residual->defined()) {
    check_bf16_cuda(*residual, "residual");
    R = as_2d(*residual).contiguous();
    TORCH_CHECK(R.size(0) == M && R.size(1) == N, "bad residual shape");
    Rp = R.data_ptr();
  }
  if (gamma.has_value() && gamma->defined()) { check_bf16_cuda(*gamma, "gamma"); TORCH_CHECK(gamma->numel() == N && gamma->is_contiguous()); }
  const int ks = cosmos::gemm_pick_k_splits((int)M, (int)N, (int)K, EPI_PLAIN);
  cosmos::GemmArgs g;
  g.A = A.data_ptr(); g.B = W.data_ptr(); g.C = own.data_ptr();
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.lda = A.stride(0); g.ldb = W.stride(0); g.ldc = N;
  g.epi = EPI_PLAIN;
  g.status = status_tensor(A.get_device()).data_ptr<int>();
  Tensor partial;
  if (ks > 1) {
    partial = at::empty({ks, M, N}, A.options().dtype(at::kFloat));
    g.k_splits = ks; g.partial = partial.data_ptr<float>(); g.partial_only = true;
  }
  cosmos::gemm_bf16(g, cur_stream());
  Tensor x_new = at::empty({M, N}, A.options());
  Tensor h = want_norm ? at::empty({M, N}, A.options()) : Tensor();
  cosmos::allreduce_norm(ptr_table(bufs, "bufs"), reinterpret_cast<const void*>(mc_ptr), own.data_ptr(),
                         ptr_table(pads, "pads"), (int)rank, (int)world, (int)slot, counters.data_ptr<int>(),
                         ks > 1 ? partial.data_ptr<float>() : nullptr, ks, (int)M, (int)N, Rp, opt_ptr(gamma), (float)eps,
                         x_new.data_ptr(), want_norm ? h.data_ptr() : nullptr, g.status, cur_stream());
  return {want_norm ? h : x_new, x_new};
}

// The all-reduce (+ residual + RMS-norm) kernel on values that are already in `own`.
std::tuple<Tensor, Tensor> allreduce_norm(const Tensor& bufs, int64_t mc_ptr, Tensor own, const Tensor& pads,
                                          int64_t rank, int64_t world, int64_t slot, Tensor counters, int64_t M,
                                          int64_t N, const OptT& residual, const OptT& gamma, double eps, bool want_norm) {
  check_bf16_cuda(own, "own");
  c10::cuda::CUDAGuard guard(own.device());
  TORCH_CHECK(own.is_contiguous() && own.numel() >= M * N && N % 8 == 0 && N <= 8192, "own: [M, N] bf16, N % 8 == 0, N <= 8192");
  TORCH_CHECK(counters.is_cuda() && counters.scalar_type() == at::kInt && counters.numel() >= 64, "counters: int32[64]");
  const void* Rp = nullptr;
  Tensor R;
  if (residual.has_value() && residual->defined()) {
    check_bf16_cuda(*residual, "residual");
    R = residual->reshape({M, N}).contiguous();
    Rp = R.data_ptr();
  }
  if (gamma.has_value() && gamma->defined()) { check_bf16_cuda(*gamma, "gamma"); TORCH_CHECK(gamma->numel() == N && gamma->is_contiguous()); }
  Tensor x_new = at::empty({M, N}, own.options());
  Tensor h = want_norm ? at::empty({M, N}, own.options()) : Tensor();
  cosmos::allreduce_norm(ptr_table(bufs, "bufs"), reinterpret_cast<const void*>(mc_ptr), own.data_ptr(),
                         ptr_table(pads, "pads"), (int)rank, (int)world, (int)slot, counters.data_ptr<int>(), nullptr, 1,
                         (int)M, (int)N, Rp, opt_ptr(gamma), (float)eps, x_new.data_ptr(),
                         want_norm ? h.data_ptr() : nullptr, status_tensor(own.get_device()).data_ptr<int>(), cur_stream());
  return {want_norm ? h : x_new, x_new};
}

// out = resid + gate[row / rows_per_batch] * sum_p part[p]; part [P, rows, d] bf16 contiguous.
Tensor sum_partials_gated_residual(const Tensor& part, const OptT& resid, const OptT& gate, int64_t rows_per_batch) {
  check_bf16_cuda(part, "part");
  c10::cuda::CUDAGuard guard(part.device());
  TORCH_CHECK(part.dim() >= 3 && part.is_contiguous(), "part must be contiguous [P, rows.., d]");
  const int64_t P = part.size(0), d = part.size(-1), rows = part.numel() / (P * d);
  const void* Rp = nullptr; const void* Gp = nullptr;
  Tensor R, G;
  if (resid.has_value() && resid->defined()) { check_bf16_cuda(*resid, "resid"); R = resid->contiguous(); TORCH_CHECK(R.numel() == rows * d); Rp = R.data_ptr(); }
  if (gate.has_value() && gate->defined()) {
    check_bf16_cuda(*gate, "gate"); G = gate->contiguous();
    TORCH_CHECK(rows_per_batch > 0 && G.numel() == ((rows + rows_per_batch - 1) / rows_per_batch) * d, "gate: [rows / rows_per_batch, d]");
    Gp = G.data_ptr();
  }
  std::vector<int64_t> shp(part.sizes().begin() + 1, part.sizes().end());
  Tensor out = at::empty(shp, part.options());
  cosmos::sum_partials_gated_residual(part.data_ptr(), (int)P, rows, (int)d, Rp, Gp, (int)rows_per_batch, out.data_ptr(),
                                      cur_stream());
  return out;
}

void allgather_pull(const Tensor& srcs, int64_t world, Tensor dst, int64_t bytes_per_rank) {
  c10::cuda::CUDAGuard guard(dst.device());
  TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && dst.nbytes() >= (size_t)(bytes_per_rank * world));
  cosmos::allgather_pull(ptr_table(srcs, "srcs"), (int)world, dst.data_ptr(), bytes_per_rank, cur_stream());
}

}  // namespace

TORCH_LIBRARY(cosmos_b200, m) {
  m.def("status_word", &status_word);
  m.def("gemm", &gemm);
  m.def("gemm_qkv_rope", &gemm_qkv_rope);
  m.def("gemm_grouped2", &gemm_grouped2);
  m.def("gemm_ex", &gemm_ex);
  m.def("gemm_reduce_rmsnorm", &gemm_reduce_rmsnorm);
  m.def("attn_bwd_scores", &attn_bwd_scores);
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
  m.def("attn_fwd_sources", &attn_fwd_sources);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("gated_residual_bwd", &gated_residual_bwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("qkv_post_fwd", &qkv_post_fwd);
  m.def("qkv_post_bwd", &qkv_post_bwd);
  m.def("rmsnorm", &rmsnorm);
  m.def("adaln_rmsnorm", &adaln_rmsnorm);
  m.def("mrope_", &mrope_);
  m.def("gated_residual", &gated_residual);
  m.def("swiglu", &swiglu);
  m.def("cfg_euler_step_", &cfg_euler_step_);
  m.def("cfg_unipc_step_", &cfg_unipc_step_);
  m.def("l2_flush_", &l2_flush_);
  m.def("conv3d_cl", &conv3d_cl);
  m.def("rmsnorm_silu", &rmsnorm_silu);
  m.def("upsample_cl", &upsample_cl);
  m.def("conv_out_rgb", &conv_out_rgb);
  m.def("paged_decode", &paged_decode);
  m.def("paged_decode_pick_splits", &paged_decode_pick_splits);
  m.def("comm_barrier", &comm_barrier);
  m.def("comm_barrier_counted", &comm_barrier_counted);
  m.def("allreduce_oneshot", &allreduce_oneshot);
  m.def("kv_cache_write", &kv_cache_write);
  m.def("decode_qkv_post", &decode_qkv_post);
  m.def("gemm_decode_qkv_post", &gemm_decode_qkv_post);
  m.def("bounds_check_enabled", &bounds_check_enabled);
  m.def("gemm_set_grid_limit", &gemm_set_grid_limit);
  m.def("gemm_set_cta_pair", &gemm_set_cta_pair);
  m.def("gemm_set_debug", &gemm_set_debug);
  m.def("gemm_pick_k_splits", &gemm_pick_k_splits);
  m.def("set_pdl", &set_pdl);
  m.def("sample_topk", &sample_topk);
  m.def("sample_pick_", &sample_pick_);
  m.def("attn_set_cta_pair", &attn_set_cta_pair);
  m.def("attn_set_exp_emulation", &attn_set_exp_emulation);
  m.def("attn_set_debug", &attn_set_debug);
  m.def("bounds_check_selftest", &bounds_check_selftest);
  m.def("rs_adamw", &rs_adamw);
  m.def("allgather_pull", &allgather_pull);
  m.def("reduce_scatter_pull", &reduce_scatter_pull);
  m.def("adamw_shard", &adamw_shard);
  m.def("gemm_allreduce_norm", &gemm_allreduce_norm);
  m.def("allreduce_norm", &allreduce_norm);
  m.def("sum_partials_gated_residual", &sum_partials_gated_residual);
  cosmos::register_runtime_ops(m);
  cosmos::register_safetensors(m);
}
