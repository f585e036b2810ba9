// Python bindings (torch extension `triune_b200._C`). Thin argument checking + stream plumbing; all
// device work is in the .cu translation units.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "elementwise/elementwise.cuh"
#include "gemm/tc_gemm.cuh"
#include "gla/gla.cuh"
#include "quant/quant.cuh"

namespace {

using torch::Tensor;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline const __nv_bfloat16* bf(const Tensor& t) { return reinterpret_cast<const __nv_bfloat16*>(t.data_ptr()); }
inline __nv_bfloat16* bfm(Tensor& t) { return reinterpret_cast<__nv_bfloat16*>(t.data_ptr()); }
inline const __nv_bfloat16* bf_opt(const c10::optional<Tensor>& t) {
  return t.has_value() && t->defined() ? reinterpret_cast<const __nv_bfloat16*>(t->data_ptr()) : nullptr;
}

void check_bf16_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
  // every kernel reads and writes bf16 data in 16-byte vectors: a misaligned base would fault on the device
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name, " must start on a 16-byte boundary");
}

// C[b] = alpha * op(A[b]) * op(B[b])^T with the fused epilogue. a: [batch?, M, K] (or [batch?, K, M] when
// a_mn_major), b: [batch?, N, K] (or [batch?, K, N] when b_mn_major). Inner dims must be contiguous.
void tc_gemm(const Tensor& a, const Tensor& b, Tensor& c, bool a_mn_major, bool b_mn_major, int64_t mode, int64_t flags,
             double alpha, const c10::optional<Tensor>& bias, const c10::optional<Tensor>& aux_in,
             const c10::optional<Tensor>& aux_out, const c10::optional<Tensor>& row_scale,
             const c10::optional<Tensor>& tile_group, const c10::optional<Tensor>& group_offsets,
             const c10::optional<Tensor>& status, double beta, const c10::optional<Tensor>& k_runs) {
  check_bf16_cuda(a, "a");
  check_bf16_cuda(b, "b");
  TORCH_CHECK(c.is_cuda(), "c must be CUDA");
  TORCH_CHECK(a.stride(-1) == 1 && b.stride(-1) == 1 && c.stride(-1) == 1, "inner dims must be contiguous");
  c10::cuda::CUDAGuard guard(a.device());
  tb::GemmArgs g{};
  g.A = bf(a);
  g.B = bf(b);
  g.C = c.data_ptr();
  g.a_mn_major = a_mn_major;
  g.b_mn_major = b_mn_major;
  g.mode = (int)mode;
  g.flags = (int)flags;
  if (c.scalar_type() == at::kFloat) g.flags |= tb::GF_OUT_F32;
  else TORCH_CHECK(c.scalar_type() == at::kBFloat16, "c must be bf16 or fp32");
  g.alpha = (float)alpha;
  g.beta = (float)beta;
  const int ad = a.dim(), bd = b.dim(), cd = c.dim();
  TORCH_CHECK(ad >= 2 && bd >= 2 && cd >= 2, "operands must be at least 2-D");
  g.lda = a.stride(-2);
  g.ldb = b.stride(-2);
  g.ldc = c.stride(-2);
  g.strideA = ad == 3 ? a.stride(0) : 0;
  g.strideB = bd == 3 ? b.stride(0) : 0;
  g.strideC = cd == 3 ? c.stride(0) : 0;
  g.batch = cd == 3 ? (int)c.size(0) : 1;
  g.M = (int)c.size(-2);
  g.N = (int)c.size(-1);
  if (mode == tb::GEMM_GROUPED_K) {
    g.K = (int)a.size(-2);  // total rows being reduced over
    TORCH_CHECK(a.size(-2) == b.size(-2), "grouped-K operands must share the row dimension");
    TORCH_CHECK(a.size(-1) == g.M && b.size(-1) == g.N, "grouped-K: c[g] is [a.cols, b.cols]");
  } else {
    g.K = (int)(a_mn_major ? a.size(-2) : a.size(-1));
    const int64_t kb = b_mn_major ? b.size(-2) : b.size(-1);
    TORCH_CHECK(kb == g.K, "reduction dims differ: ", g.K, " vs ", kb);
    const int64_t am = a_mn_major ? a.size(-1) : a.size(-2);
    const int64_t bn = b_mn_major ? b.size(-1) : b.size(-2);
    TORCH_CHECK(am == g.M, "a rows (", am, ") != c rows (", g.M, ")");
    TORCH_CHECK(bn == g.N, "b rows (", bn, ") != c cols (", g.N, ")");
  }
  if (mode == tb::GEMM_GROUPED_M) {
    TORCH_CHECK(bd == 3, "grouped-M: b must be [groups, N, K]");
    g.batch = (int)b.size(0);
    g.strideB = b.stride(0);
  }
  if (bias.has_value() && bias->defined()) {
    check_bf16_cuda(*bias, "bias");
    g.bias = bf(*bias);
    g.bias_stride = bias->dim() == 2 ? bias->stride(0) : 0;
  }
  if (aux_in.has_value() && aux_in->defined()) {
    check_bf16_cuda(*aux_in, "aux_in");
    TORCH_CHECK(aux_in->stride(-2) == g.ldc, "aux_in must share c's layout");
    g.aux_in = bf(*aux_in);
  }
  if (aux_out.has_value() && aux_out->defined()) {
    check_bf16_cuda(*aux_out, "aux_out");
    TORCH_CHECK(aux_out->stride(-2) == g.ldc, "aux_out must share c's layout");
    g.aux_out = reinterpret_cast<__nv_bfloat16*>(aux_out->data_ptr());
  }
  if (row_scale.has_value() && row_scale->defined()) {
    TORCH_CHECK(row_scale->scalar_type() == at::kFloat && row_scale->is_contiguous(), "row_scale must be fp32");
    g.row_scale = row_scale->data_ptr<float>();
  }
  if (tile_group.has_value() && tile_group->defined()) {
    TORCH_CHECK(tile_group->scalar_type() == at::kInt, "tile_group must be int32");
    g.tile_group = tile_group->data_ptr<int>();
  }
  if (group_offsets.has_value() && group_offsets->defined()) {
    TORCH_CHECK(group_offsets->scalar_type() == at::kInt, "group_offsets must be int32");
    g.group_offsets = group_offsets->data_ptr<int>();
  }
  if (status.has_value() && status->defined()) {
    TORCH_CHECK(status->scalar_type() == at::kInt, "status must be int32");
    g.status = status->data_ptr<int>();
  }
  if (k_runs.has_value() && k_runs->defined()) {
    TORCH_CHECK(mode == tb::GEMM_GROUPED_K && g.group_offsets != nullptr, "k_runs belongs to the grouped-K mode");
    TORCH_CHECK(k_runs->is_cuda() && k_runs->scalar_type() == at::kInt && k_runs->is_contiguous() && k_runs->dim() == 2 &&
                    k_runs->size(1) == 2,
                "k_runs must be a contiguous CUDA int32 tensor [runs, 2]");
    g.k_runs = k_runs->data_ptr<int>();
  }
  tb::launch_tc_gemm(g, cur_stream());
}

std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const c10::optional<Tensor>& res, const Tensor& w, double eps) {
  check_bf16_cuda(x, "x");
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous(), "rmsnorm: contiguous inputs required");
  check_bf16_cuda(w, "w");
  if (res.has_value() && res->defined()) check_bf16_cuda(*res, "residual");
  const int d = (int)x.size(-1);
  TORCH_CHECK(d % 8 == 0 && d <= 2048, "rmsnorm kernel supports d % 8 == 0, d <= 2048");
  c10::cuda::CUDAGuard guard(x.device());
  const int rows = (int)(x.numel() / d);
  Tensor y = torch::empty_like(x);
  Tensor rstd = torch::empty({rows}, x.options().dtype(at::kFloat));
  Tensor sum_out;
  const bool has_res = res.has_value() && res->defined();
  if (has_res) {
    TORCH_CHECK(res->is_contiguous() && res->sizes() == x.sizes(), "residual shape mismatch");
    sum_out = torch::empty_like(x);
  }
  tb::launch_rmsnorm_fwd(bf(x), has_res ? bf(*res) : nullptr, bf(w), bfm(y), has_res ? bfm(sum_out) : nullptr,
                         rstd.data_ptr<float>(), rows, d, (float)eps, cur_stream());
  return {y, rstd, has_res ? sum_out : Tensor()};
}

std::vector<Tensor> rmsnorm_bwd(const Tensor& x, const Tensor& w, const Tensor& dy, const Tensor& rstd,
                                const c10::optional<Tensor>& dres) {
  check_bf16_cuda(x, "x");
  check_bf16_cuda(w, "w");
  const int d = (int)x.size(-1);
  const int rows = (int)(x.numel() / d);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = torch::empty_like(x);
  Tensor dw = torch::zeros({d}, x.options().dtype(at::kFloat));
  Tensor dyc = dy.contiguous();
  const bool has = dres.has_value() && dres->defined();
  Tensor drc = has ? dres->contiguous() : Tensor();
  tb::launch_rmsnorm_bwd(bf(x), bf(w), bf(dyc), rstd.data_ptr<float>(), has ? bf(drc) : nullptr, bfm(dx),
                         dw.data_ptr<float>(), rows, d, cur_stream());
  return {dx, dw};
}

// in: [tokens, ld] with q at col 0 and k at col k_off; returns [tokens, 2, H, D].
Tensor qk_prep_fwd(const Tensor& in, int64_t k_off, const c10::optional<Tensor>& cs, const c10::optional<Tensor>& sn,
                   int64_t T, int64_t H, int64_t D) {
  check_bf16_cuda(in, "in");
  TORCH_CHECK(in.dim() == 2 && in.stride(1) == 1, "in must be [tokens, ld]");
  TORCH_CHECK(D == 64 || D == 128, "head_dim must be 64 or 128");
  c10::cuda::CUDAGuard guard(in.device());
  const int64_t tokens = in.size(0);
  Tensor out = torch::empty({tokens, 2, H, D}, in.options());
  const bool rope = cs.has_value() && cs->defined();
  tb::launch_qk_prep_fwd(bf(in), in.stride(0), (int)k_off, bfm(out), rope ? cs->data_ptr<float>() : nullptr,
                         rope ? sn->data_ptr<float>() : nullptr, tokens, (int)T, (int)H, (int)D, cur_stream());
  return out;
}

void qk_prep_bwd(const Tensor& in, int64_t k_off, const Tensor& dout, Tensor& d_in, const c10::optional<Tensor>& cs,
                 const c10::optional<Tensor>& sn, int64_t T, int64_t H, int64_t D) {
  check_bf16_cuda(in, "in");
  check_bf16_cuda(dout, "dout");
  TORCH_CHECK(dout.is_contiguous(), "dout must be contiguous");
  c10::cuda::CUDAGuard guard(in.device());
  const bool rope = cs.has_value() && cs->defined();
  tb::launch_qk_prep_bwd(bf(in), in.stride(0), (int)k_off, bf(dout), bfm(d_in), d_in.stride(0),
                         rope ? cs->data_ptr<float>() : nullptr, rope ? sn->data_ptr<float>() : nullptr, in.size(0),
                         (int)T, (int)H, (int)D, cur_stream());
}

// Cross entropy that leaves the logits intact: returns (per-row loss, grad_scale * (softmax - onehot) as a new tensor).
std::vector<Tensor> ce_loss_grad(const Tensor& logits, const Tensor& targets, int64_t ignore_index, double grad_scale) {
  check_bf16_cuda(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && logits.stride(0) % 8 == 0, "logits must be [rows, V] with 16-byte rows");
  TORCH_CHECK(targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.numel() == logits.size(0),
              "targets must be int64 [rows]");
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor loss = torch::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  Tensor grad;
  __nv_bfloat16* gp = nullptr;
  if (grad_scale != 0.0) {
    grad = torch::empty_strided(logits.sizes(), logits.strides(), logits.options());
    gp = reinterpret_cast<__nv_bfloat16*>(grad.data_ptr());
  }
  tb::launch_ce_fwd_bwd(const_cast<__nv_bfloat16*>(bf(logits)), logits.stride(0),
                        reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()), loss.data_ptr<float>(),
                        (int)logits.size(0), (int)logits.size(1), ignore_index, (float)grad_scale, cur_stream(), gp);
  return {loss, grad};
}

// SwiGLU over the fused gate/up weight inside the GEMM: h [M, H] = silu(x Wg^T) * (x Wu^T) with w13 = [Wg ; Wu]
// ([2H, K]); gu (optional, [M, 2H]) receives both pre-activations for the backward pass.
void tc_gemm_swiglu(const Tensor& x, const Tensor& w13, Tensor& h, const c10::optional<Tensor>& gu) {
  check_bf16_cuda(x, "x");
  check_bf16_cuda(w13, "w13");
  check_bf16_cuda(h, "h");
  TORCH_CHECK(x.dim() == 2 && w13.dim() == 2 && h.dim() == 2 && x.stride(1) == 1 && w13.stride(1) == 1 && h.stride(1) == 1,
              "tc_gemm_swiglu: 2-D operands with contiguous rows");
  const int64_t M = x.size(0), K = x.size(1), H = h.size(1);
  TORCH_CHECK(w13.size(0) == 2 * H && w13.size(1) == K && h.size(0) == M, "tc_gemm_swiglu: shapes");
  c10::cuda::CUDAGuard guard(x.device());
  tb::GemmArgs g{};
  g.A = bf(x); g.B = bf(w13); g.C = h.data_ptr();
  g.M = (int)M; g.N = (int)H; g.K = (int)K;
  g.lda = x.stride(0); g.ldb = w13.stride(0); g.ldc = h.stride(0);
  g.batch = 1; g.mode = tb::GEMM_DENSE; g.flags = tb::GF_SWIGLU; g.alpha = 1.0f; g.n_split = (int)H;
  if (gu.has_value() && gu->defined()) {
    check_bf16_cuda(*gu, "gu");
    TORCH_CHECK(gu->dim() == 2 && gu->is_contiguous() && gu->size(0) == M && gu->size(1) == 2 * H, "gu must be [M, 2H] contiguous");
    g.aux_out = reinterpret_cast<__nv_bfloat16*>(gu->data_ptr());
  }
  tb::launch_tc_gemm(g, cur_stream());
}

// Backward of the SwiGLU epilogue inside the GEMM that forms d(hidden): dgu [M, 2H] = (d gate | d up) from
// dh = dy op(w) ([M, H], never written) and the saved pre-activations gu [M, 2H]. w is [H, K] (K-major) or, with
// w_mn_major, stored [K, H] (the FFN's down projection as it is stored).
void tc_gemm_dswiglu(const Tensor& dy, const Tensor& w, bool w_mn_major, const Tensor& gu, Tensor& dgu) {
  check_bf16_cuda(dy, "dy");
  check_bf16_cuda(w, "w");
  check_bf16_cuda(gu, "gu");
  check_bf16_cuda(dgu, "dgu");
  TORCH_CHECK(dy.dim() == 2 && w.dim() == 2 && dy.stride(1) == 1 && w.stride(1) == 1, "tc_gemm_dswiglu: 2-D operands");
  const int64_t M = dy.size(0), K = dy.size(1);
  const int64_t H = w_mn_major ? w.size(1) : w.size(0);
  TORCH_CHECK((w_mn_major ? w.size(0) : w.size(1)) == K, "tc_gemm_dswiglu: reduction dims differ");
  TORCH_CHECK(gu.is_contiguous() && dgu.is_contiguous() && gu.size(0) == M && gu.size(1) == 2 * H && dgu.sizes() == gu.sizes(),
              "gu and dgu must be [M, 2H] contiguous");
  c10::cuda::CUDAGuard guard(dy.device());
  tb::GemmArgs g{};
  g.A = bf(dy); g.B = bf(w); g.C = dgu.data_ptr();
  g.M = (int)M; g.N = (int)H; g.K = (int)K;
  g.lda = dy.stride(0); g.ldb = w.stride(0); g.ldc = dgu.stride(0);
  g.b_mn_major = w_mn_major;
  g.batch = 1; g.mode = tb::GEMM_DENSE; g.flags = tb::GF_DSWIGLU; g.alpha = 1.0f; g.n_split = (int)H;
  g.aux_in = bf(gu);
  tb::launch_tc_gemm(g, cur_stream());
}

struct RowMat {
  const __nv_bfloat16* p;
  long long ld;
};
RowMat rows_of(const Tensor& t, int64_t width, const char* name) {
  check_bf16_cuda(t, name);
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1 && t.size(1) == width && t.stride(0) % 8 == 0, name,
              ": [rows, width] with contiguous, 16-byte aligned rows expected");
  return RowMat{bf(t), t.stride(0)};
}

Tensor swiglu_fwd(const Tensor& gate, const Tensor& up) {
  const int64_t rows = gate.size(0), width = gate.size(1);
  TORCH_CHECK(width % 8 == 0 && up.size(0) == rows, "swiglu: width must be a multiple of 8");
  RowMat g = rows_of(gate, width, "gate"), u = rows_of(up, width, "up");
  c10::cuda::CUDAGuard guard(gate.device());
  Tensor out = torch::empty({rows, width}, gate.options());
  tb::launch_swiglu_fwd(g.p, g.ld, u.p, u.ld, bfm(out), width, rows, (int)width, cur_stream());
  return out;
}

std::vector<Tensor> swiglu_bwd(const Tensor& gate, const Tensor& up, const Tensor& dh) {
  const int64_t rows = gate.size(0), width = gate.size(1);
  TORCH_CHECK(width % 8 == 0, "swiglu: width must be a multiple of 8");
  RowMat g = rows_of(gate, width, "gate"), u = rows_of(up, width, "up"), d = rows_of(dh, width, "dh");
  c10::cuda::CUDAGuard guard(gate.device());
  // the two gradients are the halves of one [rows, 2 * width] tensor, so a fused gate/up projection gets its
  // output gradient without a concatenation
  Tensor dgu = torch::empty({rows, 2 * width}, gate.options());
  __nv_bfloat16* base = bfm(dgu);
  tb::launch_swiglu_bwd(g.p, g.ld, u.p, u.ld, d.p, d.ld, base, 2 * width, base + width, 2 * width, rows, (int)width,
                        cur_stream());
  return {dgu.slice(1, 0, width), dgu.slice(1, width, 2 * width), dgu};
}

// x: [rows = B*T, H*D] bf16 (row pitch free); cos/sin: fp32 [T, D/2] contiguous.
Tensor rope_apply(const Tensor& x, const Tensor& cs, const Tensor& sn, int64_t T, int64_t H, int64_t D, bool transpose) {
  RowMat xm = rows_of(x, H * D, "x");
  TORCH_CHECK(D % 16 == 0 && cs.scalar_type() == at::kFloat && sn.scalar_type() == at::kFloat && cs.is_contiguous() &&
                  sn.is_contiguous() && cs.numel() == T * (D / 2) && sn.numel() == T * (D / 2),
              "rope: cos/sin must be fp32 [T, D/2] and D a multiple of 16");
  TORCH_CHECK(x.size(0) % T == 0, "rope: rows must be a multiple of T");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty({x.size(0), H * D}, x.options());
  tb::launch_rope(xm.p, xm.ld, bfm(y), H * D, cs.data_ptr<float>(), sn.data_ptr<float>(), x.size(0), (int)T, (int)H, (int)D,
                  transpose, cur_stream());
  return y;
}

// grad [V, d] fp32 += scatter of dy [tokens, d] bf16 by ids [tokens] int64.
void embedding_bwd(const Tensor& dy, const Tensor& ids, Tensor& grad) {
  check_bf16_cuda(dy, "dy");
  TORCH_CHECK(dy.dim() == 2 && dy.stride(1) == 1 && dy.stride(0) % 4 == 0 && dy.size(1) % 4 == 0, "dy must be [tokens, d], d % 4 == 0");
  TORCH_CHECK(ids.scalar_type() == at::kLong && ids.is_contiguous() && ids.numel() == dy.size(0), "ids must be int64 [tokens]");
  TORCH_CHECK(grad.is_cuda() && grad.scalar_type() == at::kFloat && grad.is_contiguous() && grad.dim() == 2 &&
                  grad.size(1) == dy.size(1) && (reinterpret_cast<uintptr_t>(grad.data_ptr()) & 15) == 0,
              "grad must be a contiguous, 16-byte aligned fp32 [V, d]");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(dy.data_ptr()) & 7) == 0, "dy must be 8-byte aligned");
  c10::cuda::CUDAGuard guard(dy.device());
  tb::launch_embedding_bwd(bf(dy), dy.stride(0), reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()),
                           grad.data_ptr<float>(), dy.size(0), (int)dy.size(1), grad.size(0), cur_stream());
}

Tensor ce_fwd_bwd(Tensor& logits, const Tensor& targets, int64_t ignore_index, double grad_scale) {
  check_bf16_cuda(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "logits must be [rows, V]");
  TORCH_CHECK(targets.scalar_type() == at::kLong && targets.is_contiguous(), "targets must be int64");
  TORCH_CHECK(logits.stride(0) % 8 == 0, "logits row stride must be a multiple of 8");
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor loss = torch::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  tb::launch_ce_fwd_bwd(bfm(logits), logits.stride(0), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()), loss.data_ptr<float>(),
                        (int)logits.size(0), (int)logits.size(1), ignore_index, (float)grad_scale, cur_stream());
  return loss;
}

// Column sums of a bf16 [M, N] matrix in fp32: returns a new [N] tensor, or adds into `out` when given.
Tensor colsum(const Tensor& x, const c10::optional<Tensor>& out) {
  check_bf16_cuda(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.size(1) % 8 == 0 && x.stride(0) % 8 == 0,
              "x must be [M, N] with N and the row pitch multiples of 8");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "x must be 16-byte aligned");
  c10::cuda::CUDAGuard guard(x.device());
  const int M = (int)x.size(0), N = (int)x.size(1);
  const bool acc = out.has_value() && out->defined();
  if (acc)
    TORCH_CHECK(out->scalar_type() == at::kFloat && out->is_contiguous() && out->numel() == N, "out must be fp32 [N]");
  Tensor res = acc ? *out : torch::empty({N}, x.options().dtype(at::kFloat));
  const int parts = tb::colsum_parts(M, N);
  Tensor partial = torch::empty({parts, N}, x.options().dtype(at::kFloat));
  tb::launch_colsum(bf(x), x.stride(0), M, N, partial.data_ptr<float>(), parts, res.data_ptr<float>(), acc, cur_stream());
  return res;
}

Tensor gather_rows(const Tensor& src, const Tensor& row_src, const c10::optional<Tensor>& row_scale) {
  check_bf16_cuda(src, "src");
  TORCH_CHECK(src.dim() == 2 && src.is_contiguous() && src.size(1) % 8 == 0, "src must be [rows, width%8==0]");
  TORCH_CHECK(row_src.scalar_type() == at::kInt, "row_src must be int32");
  c10::cuda::CUDAGuard guard(src.device());
  Tensor dst = torch::empty({row_src.size(0), src.size(1)}, src.options());
  const bool has = row_scale.has_value() && row_scale->defined();
  tb::launch_gather_rows(bfm(dst), bf(src), row_src.data_ptr<int>(), has ? row_scale->data_ptr<float>() : nullptr,
                         (int)row_src.size(0), (int)src.size(1), (int)src.size(0), cur_stream());
  return dst;
}

Tensor combine_rows(const Tensor& src, const Tensor& pos, const c10::optional<Tensor>& w,
                    const c10::optional<Tensor>& add, double add_scale) {
  check_bf16_cuda(src, "src");
  TORCH_CHECK(pos.scalar_type() == at::kInt && pos.dim() == 2 && pos.is_contiguous(), "pos must be int32 [tokens,k]");
  c10::cuda::CUDAGuard guard(src.device());
  const int tokens = (int)pos.size(0), k = (int)pos.size(1), width = (int)src.size(1);
  Tensor out = torch::empty({tokens, width}, src.options());
  const bool hw = w.has_value() && w->defined();
  const bool ha = add.has_value() && add->defined();
  if (hw) TORCH_CHECK(w->scalar_type() == at::kFloat && w->is_contiguous(), "w must be fp32 contiguous");
  if (ha) TORCH_CHECK(add->is_contiguous(), "add must be contiguous");
  tb::launch_combine_rows(bfm(out), bf(src), pos.data_ptr<int>(), hw ? w->data_ptr<float>() : nullptr,
                          ha ? bf(*add) : nullptr, (float)add_scale, tokens, k, width, (int)src.size(0), cur_stream());
  return out;
}

std::vector<int64_t> index_error_word(bool clear) {
  int w[4];
  tb::index_error_word(w, clear);
  return {w[0], w[1], w[2], w[3]};
}

Tensor row_dots(const Tensor& a, const Tensor& b, const Tensor& pos) {
  check_bf16_cuda(a, "a");
  check_bf16_cuda(b, "b");
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && pos.is_contiguous(), "contiguous inputs required");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor dots = torch::empty({pos.size(0), pos.size(1)}, a.options().dtype(at::kFloat));
  tb::launch_row_dots(dots.data_ptr<float>(), bf(a), bf(b), pos.data_ptr<int>(), (int)pos.size(0), (int)pos.size(1),
                      (int)a.size(1), cur_stream());
  return dots;
}

std::vector<Tensor> moe_route_topk(const Tensor& logits, const Tensor& bias, const c10::optional<Tensor>& temperature,
                                   double temp_value, int64_t K) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous() && logits.scalar_type() == at::kFloat, "logits: contiguous fp32 [N, E]");
  TORCH_CHECK(bias.scalar_type() == at::kFloat && bias.is_contiguous() && bias.numel() == logits.size(1), "bias: fp32 [E]");
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t N = logits.size(0), E = logits.size(1);
  Tensor idx = torch::empty({N, K}, logits.options().dtype(at::kLong));
  Tensor w = torch::empty({N, K}, logits.options());
  const bool keys32 = E <= 32;  // 31-bit sort keys: half the radix passes of the plan's one sort
  Tensor keys = torch::empty({N * K}, logits.options().dtype(keys32 ? at::kInt : at::kLong));
  Tensor counts = torch::empty({E, K}, logits.options().dtype(at::kInt));
  const bool ht = temperature.has_value() && temperature->defined();
  if (ht) TORCH_CHECK(temperature->scalar_type() == at::kFloat && temperature->is_cuda(), "temperature: fp32 device scalar");
  tb::launch_moe_route_topk(logits.data_ptr<float>(), bias.data_ptr<float>(), ht ? temperature->data_ptr<float>() : nullptr,
                            (float)temp_value, (int)N, (int)E, (int)K, (long long*)idx.data_ptr<int64_t>(), w.data_ptr<float>(),
                            keys.data_ptr(), keys32, counts.data_ptr<int>(), cur_stream());
  return {idx, w, keys, counts};
}

Tensor moe_route_bwd(const Tensor& logits, const c10::optional<Tensor>& temperature, double temp_value, const Tensor& idx,
                     const Tensor& w, const Tensor& dw) {
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t N = logits.size(0), E = logits.size(1), K = idx.size(1);
  Tensor dl = torch::empty_like(logits);
  const bool ht = temperature.has_value() && temperature->defined();
  tb::launch_moe_route_bwd(logits.data_ptr<float>(), ht ? temperature->data_ptr<float>() : nullptr, (float)temp_value,
                           (const long long*)idx.data_ptr<int64_t>(), w.data_ptr<float>(), dw.contiguous().data_ptr<float>(), (int)N,
                           (int)E, (int)K, dl.data_ptr<float>(), cur_stream());
  return dl;
}

std::vector<Tensor> moe_plan_sorted(const Tensor& sorted_keys, const Tensor& order, const Tensor& counts, int64_t N, int64_t K,
                                    int64_t cap) {
  const bool keys32 = sorted_keys.scalar_type() == at::kInt;
  TORCH_CHECK((keys32 || sorted_keys.scalar_type() == at::kLong) && order.scalar_type() == at::kLong && counts.scalar_type() == at::kInt,
              "dtypes");
  c10::cuda::CUDAGuard guard(sorted_keys.device());
  const int64_t A = N * K, E = counts.size(0);
  const int64_t R = (A + 255) / 256 * 256 + E * 256;  // every expert's rows are padded to a multiple of 256
  auto oi = sorted_keys.options().dtype(at::kInt);
  Tensor pos = torch::empty({N, K}, oi), keep = torch::empty({N, K}, sorted_keys.options().dtype(at::kBool));
  Tensor row_src = torch::empty({R}, oi), tile_group = torch::empty({R / 128}, oi), offsets = torch::empty({E + 1}, oi);
  Tensor accepted = torch::empty({E}, sorted_keys.options().dtype(at::kLong));
  tb::launch_moe_plan_sorted(sorted_keys.data_ptr(), keys32, (const long long*)order.data_ptr<int64_t>(),
                             counts.data_ptr<int>(), (int)A, (int)E, (int)K, (int)cap, (int)R, pos.data_ptr<int>(),
                             (unsigned char*)keep.data_ptr<bool>(), row_src.data_ptr<int>(), tile_group.data_ptr<int>(),
                             offsets.data_ptr<int>(), (long long*)accepted.data_ptr<int64_t>(), cur_stream());
  return {pos, keep, row_src, tile_group, offsets, accepted};
}

void adamw_flat(Tensor& master, Tensor& m, Tensor& v, const Tensor& grad, const c10::optional<Tensor>& param_bf16,
                double lr, double beta1, double beta2, double eps, double wd, int64_t step,
                const c10::optional<Tensor>& grad_scale_ptr, double grad_scale, const c10::optional<Tensor>& hyper) {
  TORCH_CHECK(master.scalar_type() == at::kFloat && master.is_contiguous(), "master must be fp32 contiguous");
  TORCH_CHECK(grad.is_contiguous() && grad.numel() == master.numel(), "grad shape mismatch");
  c10::cuda::CUDAGuard guard(master.device());
  const bool gf32 = grad.scalar_type() == at::kFloat;
  TORCH_CHECK(gf32 || grad.scalar_type() == at::kBFloat16, "grad must be fp32 or bf16");
  const float bc1 = 1.0f - (float)std::pow(beta1, (double)step);
  const float bc2 = 1.0f - (float)std::pow(beta2, (double)step);
  const bool hp = param_bf16.has_value() && param_bf16->defined();
  const bool hs = grad_scale_ptr.has_value() && grad_scale_ptr->defined();
  tb::launch_adamw_flat(master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), grad.data_ptr(), gf32,
                        hp ? reinterpret_cast<__nv_bfloat16*>(param_bf16->data_ptr()) : nullptr, master.numel(),
                        (float)lr, (float)beta1, (float)beta2, (float)eps, (float)wd, bc1, bc2,
                        hs ? grad_scale_ptr->data_ptr<float>() : nullptr, (float)grad_scale,
                        hyper.has_value() && hyper->defined() ? hyper->data_ptr<float>() : nullptr, cur_stream());
}

void sumsq(const Tensor& x, Tensor& out) {
  TORCH_CHECK(x.is_contiguous() && out.scalar_type() == at::kFloat, "sumsq: contiguous x, fp32 out");
  c10::cuda::CUDAGuard guard(x.device());
  tb::launch_sumsq(x.data_ptr(), x.scalar_type() == at::kFloat, x.numel(), out.data_ptr<float>(), cur_stream());
}

void muon_momentum(Tensor& mom, const Tensor& grad, Tensor& u_out, double beta, bool nesterov,
                   const c10::optional<Tensor>& grad_scale_ptr) {
  c10::cuda::CUDAGuard guard(mom.device());
  const bool hs = grad_scale_ptr.has_value() && grad_scale_ptr->defined();
  tb::launch_muon_momentum(mom.data_ptr<float>(), grad.data_ptr(), grad.scalar_type() == at::kFloat, bfm(u_out),
                           mom.numel(), (float)beta, nesterov, hs ? grad_scale_ptr->data_ptr<float>() : nullptr,
                           cur_stream());
}

void muon_apply(Tensor& master, const Tensor& o, const c10::optional<Tensor>& param_bf16, double lr, double wd,
                double scale, const c10::optional<Tensor>& hyper) {
  c10::cuda::CUDAGuard guard(master.device());
  const bool hp = param_bf16.has_value() && param_bf16->defined();
  tb::launch_muon_apply(master.data_ptr<float>(), bf(o),
                        hp ? reinterpret_cast<__nv_bfloat16*>(param_bf16->data_ptr()) : nullptr, master.numel(),
                        (float)lr, (float)wd, (float)scale,
                        hyper.has_value() && hyper->defined() ? hyper->data_ptr<float>() : nullptr, cur_stream());
}

// X [batch, m, n] bf16 contiguous (m <= n) -> X / safe spectral bound, bf16 (see launch_ns_prepare)
Tensor ns_prepare(const Tensor& x, double eps) {
  check_bf16_cuda(x, "x");
  TORCH_CHECK(x.dim() == 3 && x.is_contiguous() && x.size(2) % 8 == 0 && x.size(1) <= x.size(2),
              "ns_prepare: contiguous [batch, m, n] with m <= n and n % 8 == 0");
  TORCH_CHECK(x.size(2) <= 11568, "ns_prepare: n <= 11568 (the iterate and an 8-row tile live in one CTA's shared memory)");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  const int64_t K = x.size(0), n = x.size(2);
  Tensor scratch = torch::empty({2 * K * n + 2 * K}, x.options().dtype(at::kFloat));
  tb::launch_ns_prepare(bf(x), bfm(y), (int)K, (int)x.size(1), (int)n, (float)eps, scratch.data_ptr<float>(), cur_stream());
  return y;
}

void axpby_bf16(Tensor& x, const Tensor& y, double a, double b) {
  c10::cuda::CUDAGuard guard(x.device());
  tb::launch_axpby_bf16(bfm(x), bf(y), (float)a, (float)b, x.numel(), cur_stream());
}

Tensor triangular_adamw(const Tensor& S, Tensor& m, Tensor& v, double beta1, double beta2, double eps, int64_t step,
                        bool triu, const c10::optional<Tensor>& hyper) {
  TORCH_CHECK(S.scalar_type() == at::kFloat && S.is_contiguous() && S.dim() == 3 && S.size(1) == S.size(2),
              "S must be fp32 [n, r, r]");
  c10::cuda::CUDAGuard guard(S.device());
  Tensor delta = torch::empty_like(S);
  tb::launch_triangular_adamw(S.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), delta.data_ptr<float>(),
                              (int)S.size(0), (int)S.size(1), (float)beta1, (float)beta2, (float)eps,
                              1.0f - (float)std::pow(beta1, (double)step), 1.0f - (float)std::pow(beta2, (double)step),
                              triu, hyper.has_value() && hyper->defined() ? hyper->data_ptr<float>() : nullptr, cur_stream());
  return delta;
}

void steer_update(Tensor& P, const Tensor& G, double momentum, double steer) {
  c10::cuda::CUDAGuard guard(P.device());
  tb::launch_steer_update(P.data_ptr<float>(), G.data_ptr<float>(), P.numel(), (float)momentum, (float)steer,
                          cur_stream());
}

std::vector<Tensor> route_tiers(const Tensor& logits, double threshold) {
  TORCH_CHECK(logits.scalar_type() == at::kFloat && logits.is_contiguous() && logits.size(-1) == 3, "logits [rows,3]");
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor tiers = torch::empty({logits.size(0)}, logits.options().dtype(at::kInt));
  Tensor flag = torch::ones({1}, logits.options().dtype(at::kInt));
  tb::launch_route_tiers(logits.data_ptr<float>(), tiers.data_ptr<int>(), flag.data_ptr<int>(), (int)logits.size(0),
                         (float)threshold, cur_stream());
  return {tiers, flag};
}

Tensor neuron_heatmap(const Tensor& act, int64_t num_bins) {
  TORCH_CHECK(act.scalar_type() == at::kFloat && act.is_contiguous(), "act must be fp32 contiguous");
  c10::cuda::CUDAGuard guard(act.device());
  Tensor scratch = torch::empty({num_bins}, act.options());
  Tensor rgba = torch::empty({num_bins}, act.options().dtype(at::kInt));
  tb::launch_neuron_heatmap(act.data_ptr<float>(), act.numel(), (int)num_bins, scratch.data_ptr<float>(),
                            reinterpret_cast<uint32_t*>(rgba.data_ptr<int>()), cur_stream());
  return rgba;
}

Tensor tier_render(const Tensor& act, const Tensor& tiers) {
  TORCH_CHECK(act.scalar_type() == at::kFloat && act.is_contiguous() && act.dim() == 2, "act must be fp32 [rows,w]");
  c10::cuda::CUDAGuard guard(act.device());
  Tensor rgba = torch::empty({act.size(0), act.size(1)}, act.options().dtype(at::kInt));
  tb::launch_tier_render(act.data_ptr<float>(), tiers.data_ptr<int>(), reinterpret_cast<uint32_t*>(rgba.data_ptr<int>()),
                         (int)act.size(0), (int)act.size(1), cur_stream());
  return rgba;
}

}  // namespace

void register_gla(pybind11::module& m);
void register_quant(pybind11::module& m);
void register_comm(pybind11::module& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("tc_gemm", &tc_gemm);
  m.def("tc_gemm_debug_buffer", [](const c10::optional<Tensor>& t) {
    const bool on = t.has_value() && t->defined();
    TORCH_CHECK(!on || (t->is_cuda() && t->scalar_type() == at::kLong && t->is_contiguous() && t->numel() >= 16),
                "tc_gemm_debug_buffer: a contiguous CUDA int64 tensor with at least 16 entries, or None");
    tb::tc_gemm_set_debug_buffer(on ? (long long*)t->data_ptr<int64_t>() : nullptr);
  });
  m.def("tc_gemm_pair_launches", []() { return (int64_t)tb::tc_gemm_pair_launch_count(); });
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("qk_prep_fwd", &qk_prep_fwd);
  m.def("qk_prep_bwd", &qk_prep_bwd);
  m.def("ce_fwd_bwd", &ce_fwd_bwd);
  m.def("ce_loss_grad", &ce_loss_grad);
  m.def("tc_gemm_swiglu", &tc_gemm_swiglu);
  m.def("tc_gemm_dswiglu", &tc_gemm_dswiglu);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("rope_apply", &rope_apply);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("colsum", &colsum);
  m.def("gather_rows", &gather_rows);
  m.def("combine_rows", &combine_rows);
  m.def("index_error_word", &index_error_word, "first out-of-table index seen by the row-movement kernels: [kernel, row, index, limit]");
  m.def("row_dots", &row_dots);
  m.def("moe_route_topk", &moe_route_topk);
  m.def("moe_route_bwd", &moe_route_bwd);
  m.def("moe_plan_sorted", &moe_plan_sorted);
  m.def("adamw_flat", &adamw_flat);
  m.def("sumsq", &sumsq);
  m.def("muon_momentum", &muon_momentum);
  m.def("muon_apply", &muon_apply);
  m.def("axpby_bf16", &axpby_bf16);
  m.def("ns_prepare", &ns_prepare);
  m.def("triangular_adamw", &triangular_adamw);
  m.def("steer_update", &steer_update);
  m.def("route_tiers", &route_tiers);
  m.def("neuron_heatmap", &neuron_heatmap);
  m.def("tier_render", &tier_render);
  register_gla(m);
  register_quant(m);
  register_comm(m);
}
