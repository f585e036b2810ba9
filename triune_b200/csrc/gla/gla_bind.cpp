// Python bindings of the GLA kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "gla.cuh"

namespace {
using torch::Tensor;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// view of columns [col0, col0 + H*64) of a 2-D bf16 matrix with contiguous rows
tb::GlaMat mat(const Tensor& t, int64_t col0) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.stride(1) == 1,
              "expected a 2-D CUDA bf16 matrix with contiguous rows");
  TORCH_CHECK(t.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, "rows must be 16-byte aligned");
  return tb::GlaMat{t.data_ptr(), t.stride(0), (int)col0};
}

// Forward: returns (states bf16 [BH*NT,64,64], decay fp32 [BH*NT,64], final_state fp32 [BH,64,64]); writes out.
std::vector<Tensor> gla_fwd(const Tensor& q, int64_t qcol, const Tensor& k, int64_t kcol, const Tensor& v, int64_t vcol,
                            const Tensor& g, int64_t gcol, Tensor& out, int64_t ocol, const c10::optional<Tensor>& init,
                            int64_t B, int64_t T, int64_t H, bool gate_logits) {
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t NT = T / 64, BH = B * H;
  auto f32 = q.options().dtype(at::kFloat);
  Tensor kv = torch::empty({BH * NT, 64, 64}, f32);
  Tensor decay = torch::empty({BH * NT, 64}, f32);
  Tensor states = torch::empty({BH * NT, 64, 64}, q.options());
  Tensor fin = torch::empty({BH, 64, 64}, f32);
  Tensor status = torch::zeros({1}, q.options().dtype(at::kInt));
  tb::GlaDims d{(int)B, (int)T, (int)H, gate_logits};
  auto s = cur_stream();
  tb::launch_gla_chunk_outer(0, mat(k, kcol), mat(v, vcol), mat(g, gcol), kv.data_ptr<float>(), decay.data_ptr<float>(), d,
                             status.data_ptr<int>(), s);
  const float* ip = nullptr;
  Tensor initc;
  if (init.has_value() && init->defined()) {
    initc = init->to(at::kFloat).contiguous();
    ip = initc.data_ptr<float>();
  }
  tb::launch_gla_scan(kv.data_ptr<float>(), decay.data_ptr<float>(), ip,
                      reinterpret_cast<__nv_bfloat16*>(states.data_ptr()), fin.data_ptr<float>(), (int)BH, (int)NT, false, s);
  tb::launch_gla_fwd_out(mat(q, qcol), mat(k, kcol), mat(v, vcol), mat(g, gcol),
                         reinterpret_cast<const __nv_bfloat16*>(states.data_ptr()), mat(out, ocol), d,
                         status.data_ptr<int>(), s);
  return {states, decay, fin, status};
}

// Backward: writes dq, dk, dv, dg into the given matrices. With `dfin` (gradient of the final state, fp32
// [BH,64,64]) and `fin` (the final state itself) the reverse scan starts from dfin instead of zero and the gate
// gradient receives rowsum(dfin * fin). Returns (status, gradient of the initial state [BH,64,64] fp32).
std::vector<Tensor> gla_bwd(const Tensor& q, int64_t qcol, const Tensor& k, int64_t kcol, const Tensor& v, int64_t vcol, const Tensor& g,
               int64_t gcol, const Tensor& dout, int64_t docol, const Tensor& states, const Tensor& decay, Tensor& dq,
               int64_t dqcol, Tensor& dk, int64_t dkcol, Tensor& dv, int64_t dvcol, Tensor& dg, int64_t dgcol, int64_t B,
               int64_t T, int64_t H, bool gate_logits, const c10::optional<Tensor>& dfin,
               const c10::optional<Tensor>& fin) {
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t NT = T / 64, BH = B * H;
  auto f32 = q.options().dtype(at::kFloat);
  Tensor dfinc, end_term;
  Tensor dinit = torch::empty({BH, 64, 64}, f32);
  if (dfin.has_value() && dfin->defined()) {
    TORCH_CHECK(fin.has_value() && fin->defined(), "the final state is needed with its gradient");
    dfinc = dfin->to(at::kFloat).reshape({BH, 64, 64}).contiguous();
    end_term = (dfinc * fin->to(at::kFloat).reshape({BH, 64, 64})).sum(-1).contiguous();
  }
  Tensor m = torch::empty({BH * NT, 64, 64}, f32);
  Tensor dstates = torch::empty({BH * NT, 64, 64}, q.options());
  Tensor dgl = torch::empty({B * T, H * 64}, f32);
  Tensor tot = torch::empty({BH * NT, 64}, f32);
  Tensor status = torch::zeros({1}, q.options().dtype(at::kInt));
  tb::GlaDims d{(int)B, (int)T, (int)H, gate_logits};
  auto s = cur_stream();
  tb::launch_gla_chunk_outer(1, mat(q, qcol), mat(dout, docol), mat(g, gcol), m.data_ptr<float>(), nullptr, d,
                             status.data_ptr<int>(), s);
  tb::launch_gla_scan(m.data_ptr<float>(), decay.data_ptr<float>(), dfinc.defined() ? dfinc.data_ptr<float>() : nullptr,
                      reinterpret_cast<__nv_bfloat16*>(dstates.data_ptr()), dinit.data_ptr<float>(), (int)BH, (int)NT,
                      true, s);
  tb::launch_gla_bwd_main(mat(q, qcol), mat(k, kcol), mat(v, vcol), mat(g, gcol), mat(dout, docol),
                          reinterpret_cast<const __nv_bfloat16*>(states.data_ptr()),
                          reinterpret_cast<const __nv_bfloat16*>(dstates.data_ptr()), mat(dq, dqcol), mat(dk, dkcol),
                          mat(dv, dvcol), dgl.data_ptr<float>(), tot.data_ptr<float>(), d, status.data_ptr<int>(), s);
  tb::launch_gla_dg_finalize(dgl.data_ptr<float>(), tot.data_ptr<float>(), mat(g, gcol), mat(dg, dgcol), d, s,
                             end_term.defined() ? end_term.data_ptr<float>() : nullptr);
  return {status, dinit};
}

void gla_decode(const Tensor& q, int64_t qcol, const Tensor& k, int64_t kcol, const Tensor& v, int64_t vcol, const Tensor& g,
                int64_t gcol, Tensor& state, Tensor& out, int64_t ocol, int64_t B, int64_t H, bool gate_logits) {
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(state.scalar_type() == at::kFloat && state.is_contiguous(), "state must be fp32 contiguous [B,H,64,64]");
  tb::launch_gla_decode_step(mat(q, qcol), mat(k, kcol), mat(v, vcol), mat(g, gcol), state.data_ptr<float>(), mat(out, ocol),
                             (int)B, (int)H, gate_logits, cur_stream());
}

// Gated DeltaNet recurrence (no gradient): q,k,v,g as [B*T, ld] matrices whose columns col0 + h*D.. hold head h.
void gdn_recurrent(const Tensor& q, int64_t qcol, const Tensor& k, int64_t kcol, const Tensor& v, int64_t vcol,
                   const Tensor& g, int64_t gcol, const c10::optional<Tensor>& beta, Tensor& state, Tensor& out,
                   int64_t ocol, int64_t B, int64_t T, int64_t H, int64_t D, bool gate_logits, double scale) {
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(state.scalar_type() == at::kFloat && state.is_contiguous() && state.numel() == B * H * D * D,
              "state must be fp32 contiguous [B,H,D,D]");
  const float* bp = nullptr;
  int mode = 0;
  if (beta.has_value() && beta->defined()) {
    TORCH_CHECK(beta->scalar_type() == at::kFloat && beta->is_contiguous(), "beta must be fp32 contiguous");
    if (beta->numel() == B * T * H) mode = 1;
    else if (beta->numel() == B * T * H * D) mode = 2;
    else TORCH_CHECK(false, "beta must be [B,T,H] or [B,T,H,D]");
    bp = beta->data_ptr<float>();
  }
  tb::launch_gdn_recurrent(mat(q, qcol), mat(k, kcol), mat(v, vcol), mat(g, gcol), bp, mode, state.data_ptr<float>(),
                           mat(out, ocol), (int)B, (int)T, (int)H, (int)D, gate_logits, (float)scale, cur_stream());
}
inline __nv_bfloat16* bfp(Tensor& t) { return reinterpret_cast<__nv_bfloat16*>(t.data_ptr()); }

// Chunk-parallel Gated DeltaNet forward. q, k, v, g: [B*T, ld] bf16 matrices with head h at columns col + h*D;
// beta fp32 [B*T, H] or None; init fp32 [B*H, D, D] or None. Writes `out`; returns
// [U0, W, Tm, Kend, decay, Lraw (empty when not kept), U, states, fin, status].
std::vector<Tensor> gdn_chunk_fwd(const Tensor& q, int64_t qcol, const Tensor& k, int64_t kcol, const Tensor& v,
                                  int64_t vcol, const Tensor& g, int64_t gcol, const c10::optional<Tensor>& beta,
                                  const c10::optional<Tensor>& init, Tensor& out, int64_t ocol, int64_t B, int64_t T,
                                  int64_t H, int64_t D, bool gate_logits, double scale, bool keep_scores) {
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(T % 64 == 0 && (D == 64 || D == 128), "gdn_chunk_fwd: T % 64 == 0 and D in {64, 128}");
  const int64_t NT = T / 64, BH = B * H, n = BH * NT;
  auto bf = q.options();
  auto f32 = q.options().dtype(at::kFloat);
  Tensor U0 = torch::empty({n, 64, D}, bf), W = torch::empty({n, 64, D}, bf), Tm = torch::empty({n, 64, 64}, bf),
         Kend = torch::empty({n, 64, D}, bf), decay = torch::empty({n, D}, f32), U = torch::empty({n, 64, D}, bf),
         states = torch::empty({n, D, D}, bf), fin = torch::empty({BH, D, D}, f32);
  Tensor Lraw = keep_scores ? torch::empty({n, 64, 64}, f32) : torch::empty({0}, f32);
  Tensor status = torch::zeros({1}, q.options().dtype(at::kInt));
  const float* bp = nullptr;
  Tensor betac, initc;
  if (beta.has_value() && beta->defined()) {
    betac = beta->to(at::kFloat).contiguous();
    TORCH_CHECK(betac.numel() == B * T * H, "beta must be [B*T, H]");
    bp = betac.data_ptr<float>();
  }
  const float* ip = nullptr;
  if (init.has_value() && init->defined()) {
    initc = init->to(at::kFloat).contiguous();
    TORCH_CHECK(initc.numel() == BH * D * D, "init must be [B*H, D, D]");
    ip = initc.data_ptr<float>();
  }
  tb::GdnScratch w{bfp(U0), bfp(W), bfp(Tm), bfp(Kend), decay.data_ptr<float>(),
                   keep_scores ? Lraw.data_ptr<float>() : nullptr, bfp(U), bfp(states), fin.data_ptr<float>()};
  tb::GdnDims d{(int)B, (int)T, (int)H, (int)D, gate_logits};
  tb::launch_gdn_chunk_fwd(mat(q, qcol), mat(k, kcol), mat(v, vcol), mat(g, gcol), bp, ip, mat(out, ocol), w, d,
                           (float)scale, status.data_ptr<int>(), cur_stream());
  return {U0, W, Tm, Kend, decay, Lraw, U, states, fin, status};
}

// Backward. `saved` is the list returned by gdn_chunk_fwd. Writes dq, dk, dv, dg into the given matrices; returns
// [dbeta (fp32 [B*T, H], empty without beta), dS0 (fp32 [B*H, D, D]), status, then the per-chunk intermediates].
std::vector<Tensor> gdn_chunk_bwd(const Tensor& q, int64_t qcol, const Tensor& k, int64_t kcol, const Tensor& v,
                                  int64_t vcol, const Tensor& g, int64_t gcol, const Tensor& dout, int64_t docol,
                                  const c10::optional<Tensor>& beta, const c10::optional<Tensor>& dfin,
                                  std::vector<Tensor> saved, Tensor& dq, int64_t dqcol, Tensor& dk, int64_t dkcol,
                                  Tensor& dv, int64_t dvcol, Tensor& dg, int64_t dgcol, int64_t B, int64_t T, int64_t H,
                                  int64_t D, bool gate_logits, double scale) {
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(saved.size() >= 9, "gdn_chunk_bwd: the forward's saved tensors are missing");
  const int64_t NT = T / 64, BH = B * H, n = BH * NT, NH = D / 64;
  auto bf = q.options();
  auto f32 = q.options().dtype(at::kFloat);
  Tensor G1 = torch::empty({n, 64, D}, f32), H1 = torch::empty({n, D, D}, f32), dU = torch::empty({n, 64, D}, bf),
         dSend = torch::empty({n, D, D}, bf), dS0 = torch::empty({BH, D, D}, f32), dq1 = torch::empty({n, 64, D}, f32),
         dkw1 = torch::empty({n, 64, D}, f32), dkr1 = torch::empty({n, 64, D}, f32), dW = torch::empty({n, 64, D}, bf),
         dLraw = torch::empty({n, 64, 64}, bf), dgl = torch::empty({B * T, H * D}, f32),
         tot = torch::empty({BH * NH * NT, 64}, f32);
  Tensor status = torch::zeros({1}, q.options().dtype(at::kInt));
  const float* bp = nullptr;
  Tensor betac, dfinc, dbeta = torch::empty({0}, f32);
  if (beta.has_value() && beta->defined()) {
    betac = beta->to(at::kFloat).contiguous();
    bp = betac.data_ptr<float>();
    dbeta = torch::empty({B * T, H}, f32);
    TORCH_CHECK(saved[5].numel() == n * 64 * 64, "gdn_chunk_bwd: the key-key scores were not kept by the forward pass");
  }
  const float* dfp = nullptr;
  if (dfin.has_value() && dfin->defined()) {
    dfinc = dfin->to(at::kFloat).contiguous();
    dfp = dfinc.data_ptr<float>();
  }
  tb::GdnScratch w{bfp(saved[0]), bfp(saved[1]), bfp(saved[2]), bfp(saved[3]), saved[4].data_ptr<float>(),
                   saved[5].numel() > 0 ? saved[5].data_ptr<float>() : nullptr, bfp(saved[6]), bfp(saved[7]),
                   saved[8].data_ptr<float>()};
  tb::GdnBwdScratch x{G1.data_ptr<float>(), H1.data_ptr<float>(), bfp(dU), bfp(dSend), dS0.data_ptr<float>(),
                      dq1.data_ptr<float>(), dkw1.data_ptr<float>(), dkr1.data_ptr<float>(), bfp(dW), bfp(dLraw),
                      bp != nullptr ? dbeta.data_ptr<float>() : nullptr, dgl.data_ptr<float>(), tot.data_ptr<float>()};
  tb::GdnDims d{(int)B, (int)T, (int)H, (int)D, gate_logits};
  auto s = cur_stream();
  tb::launch_gdn_chunk_bwd(mat(q, qcol), mat(k, kcol), mat(v, vcol), mat(g, gcol), mat(dout, docol), bp, dfp, mat(dq, dqcol),
                           mat(dk, dkcol), mat(dv, dvcol), w, x, d, (float)scale, status.data_ptr<int>(), s);
  // the suffix sums over the chunks and the derivative of the clamped log decay: the GLA finalize kernel with every
  // 64-wide slice of a head counted as a head of its own
  Tensor end_term;
  if (dfp != nullptr) end_term = (dfinc.reshape({BH, D, D}) * saved[8].reshape({BH, D, D})).sum(-1).reshape({BH * NH, 64}).contiguous();
  tb::GlaDims gd{(int)B, (int)T, (int)(H * NH), gate_logits};
  tb::launch_gla_dg_finalize(dgl.data_ptr<float>(), tot.data_ptr<float>(), mat(g, gcol), mat(dg, dgcol), gd, s,
                             end_term.defined() ? end_term.data_ptr<float>() : nullptr);
  // the per-chunk intermediates follow for inspection (stage-by-stage comparison against the PyTorch oracle)
  return {dbeta, dS0, status, G1, H1, dU, dSend, dq1, dkw1, dkr1, dW, dLraw, dgl, tot};
}
}  // namespace

void register_gla(pybind11::module& m) {
  m.def("gla_fwd", &gla_fwd);
  m.def("gla_bwd", &gla_bwd);
  m.def("gla_decode", &gla_decode);
  m.def("gla_debug_buffer", [](const c10::optional<Tensor>& t) {
    TORCH_CHECK(!t.has_value() || !t->defined() || (t->scalar_type() == at::kLong && t->numel() >= 8), "int64[8] expected");
    tb::gla_set_debug_buffer(t.has_value() && t->defined() ? (long long*)t->data_ptr<int64_t>() : nullptr);
  });
  m.def("gdn_recurrent", &gdn_recurrent);
  m.def("gdn_chunk_fwd", &gdn_chunk_fwd);
  m.def("gdn_chunk_bwd", &gdn_chunk_bwd);
}
