// Python bindings of the quantisation kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "quant.cuh"

namespace {

void need(bool c, const char* msg) { TORCH_CHECK(c, msg); }
cudaStream_t cur() { return at::cuda::getCurrentCUDAStream().stream(); }
const __nv_bfloat16* bf(const at::Tensor& t) { return reinterpret_cast<const __nv_bfloat16*>(t.data_ptr()); }
__nv_bfloat16* bfm(at::Tensor& t) { return reinterpret_cast<__nv_bfloat16*>(t.data_ptr()); }

std::vector<at::Tensor> fp8_quantize_act(const at::Tensor& x) {
  need(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "fp8_quantize_act: bf16 [M,K] CUDA");
  c10::cuda::CUDAGuard g(x.device());
  const int64_t M = x.size(0), K = x.size(1);
  auto q = at::empty({M, K}, x.options().dtype(at::kFloat8_e4m3fn));
  auto s = at::empty({M, (K + 127) / 128}, x.options().dtype(at::kFloat));
  tb::launch_fp8_quantize_act(bf(x), (uint8_t*)q.data_ptr(), s.data_ptr<float>(), (int)M, (int)K, cur());
  return {q, s};
}

at::Tensor fp8_block_gemm(const at::Tensor& xq, const at::Tensor& xs, const at::Tensor& wq, const at::Tensor& ws) {
  need(xq.is_cuda() && wq.is_cuda() && xq.dim() == 2 && wq.dim() == 2 && xq.is_contiguous() && wq.is_contiguous(), "fp8_block_gemm: contiguous 2-D CUDA operands");
  need(xq.element_size() == 1 && wq.element_size() == 1, "fp8_block_gemm: E4M3 operands");
  need(xs.scalar_type() == at::kFloat && ws.scalar_type() == at::kFloat && xs.is_contiguous() && ws.is_contiguous(), "fp8_block_gemm: fp32 scales");
  const int64_t M = xq.size(0), K = xq.size(1), N = wq.size(0);
  need(wq.size(1) == K, "fp8_block_gemm: K mismatch");
  const int64_t KB = (K + 127) / 128;
  need(xs.numel() == M * KB && ws.numel() == ((N + 127) / 128) * KB, "fp8_block_gemm: scale shapes");
  c10::cuda::CUDAGuard g(xq.device());
  auto out = at::empty({M, N}, xq.options().dtype(at::kBFloat16));
  auto status = at::zeros({1}, xq.options().dtype(at::kInt));
  tb::launch_fp8_block_gemm((const uint8_t*)xq.data_ptr(), xs.data_ptr<float>(), (const uint8_t*)wq.data_ptr(),
                            ws.data_ptr<float>(), bfm(out), (int)M, (int)N, (int)K, status.data_ptr<int>(), cur());
  return out;
}

std::vector<at::Tensor> nvfp4_quantize(const at::Tensor& w, bool hadamard) {
  need(w.is_cuda() && w.dim() == 2 && w.is_contiguous(), "nvfp4_quantize: contiguous [N,K] CUDA");
  need(w.scalar_type() == at::kBFloat16 || w.scalar_type() == at::kFloat, "nvfp4_quantize: bf16 or fp32");
  need(w.size(1) % 16 == 0, "nvfp4_quantize: K % 16");
  c10::cuda::CUDAGuard g(w.device());
  const int64_t N = w.size(0), K = w.size(1);
  auto packed = at::empty({N, K / 2}, w.options().dtype(at::kByte));
  auto scales = at::empty({N, K / 16}, w.options().dtype(at::kFloat8_e4m3fn));
  auto tscale = at::empty({}, w.options().dtype(at::kFloat));
  auto scratch = at::empty({1}, w.options().dtype(at::kInt));
  tb::launch_nvfp4_quantize(w.data_ptr(), w.scalar_type() == at::kBFloat16, N, K, hadamard, packed.data_ptr<uint8_t>(),
                            (uint8_t*)scales.data_ptr(), tscale.data_ptr<float>(), (unsigned int*)scratch.data_ptr(), cur());
  return {packed, scales, tscale};
}

// x bf16 [M, K] -> (packed E2M1 uint8 [M, K/2], block scales uint8 [ceil(M/128), sf_kblocks, 512] in the GEMM's layout)
std::vector<at::Tensor> nvfp4_quantize_act(const at::Tensor& x, bool hadamard) {
  need(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == at::kBFloat16, "nvfp4_quantize_act: bf16 [M,K] CUDA");
  need(x.size(1) % 32 == 0 && x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0,
       "nvfp4_quantize_act: K % 32 == 0 and 16-byte aligned rows");
  c10::cuda::CUDAGuard g(x.device());
  const int64_t M = x.size(0), K = x.size(1);
  auto packed = at::empty({M, K / 2}, x.options().dtype(at::kByte));
  auto sf = at::zeros({(M + 127) / 128, (int64_t)tb::nvfp4_sf_kblocks((int)K), 512}, x.options().dtype(at::kByte));
  tb::launch_nvfp4_quantize_act(bf(x), x.stride(0), (int)M, (int)K, hadamard, packed.data_ptr<uint8_t>(), sf.data_ptr<uint8_t>(), cur());
  return {packed, sf};
}

// E4M3 scales [R, K/16] (row-major, as the weight quantiser writes them) -> the GEMM's blocked layout
at::Tensor nvfp4_block_scales(const at::Tensor& scales, int64_t K) {
  need(scales.is_cuda() && scales.dim() == 2 && scales.is_contiguous() && scales.element_size() == 1 && scales.size(1) == K / 16,
       "nvfp4_block_scales: contiguous E4M3 [R, K/16] CUDA");
  c10::cuda::CUDAGuard g(scales.device());
  const int64_t R = scales.size(0);
  auto out = at::zeros({(R + 127) / 128, (int64_t)tb::nvfp4_sf_kblocks((int)K), 512}, scales.options().dtype(at::kByte));
  tb::launch_nvfp4_block_scales((const uint8_t*)scales.data_ptr(), (int)R, (int)K, out.data_ptr<uint8_t>(), cur());
  return out;
}

// y [M, N] bf16 = alpha * (a .* sfa) (b .* sfb)^T, both operands packed E2M1 with blocked unsigned-E4M3 scales
const __nv_bfloat16* opt_bias(const c10::optional<at::Tensor>& bias, int64_t N) {
  if (!bias.has_value() || !bias->defined()) return nullptr;
  need(bias->is_cuda() && bias->scalar_type() == at::kBFloat16 && bias->is_contiguous() && bias->numel() == N &&
           (reinterpret_cast<uintptr_t>(bias->data_ptr()) & 15) == 0,
       "block-scaled GEMM: bias must be a contiguous, 16-byte aligned bf16 [N] CUDA tensor");
  return bf(*bias);
}

std::vector<at::Tensor> nvfp4_gemm(const at::Tensor& a, const at::Tensor& sfa, const at::Tensor& b, const at::Tensor& sfb, double alpha,
                                   int64_t tile_n, const c10::optional<at::Tensor>& bias, bool gelu) {
  need(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2 && a.is_contiguous() && b.is_contiguous() &&
           a.element_size() == 1 && b.element_size() == 1 && a.size(1) == b.size(1),
       "nvfp4_gemm: contiguous packed [M, K/2] and [N, K/2]");
  const int64_t M = a.size(0), N = b.size(0), K = a.size(1) * 2;
  const int64_t kb = tb::nvfp4_sf_kblocks((int)K);
  need(sfa.is_contiguous() && sfb.is_contiguous() && sfa.numel() == ((M + 127) / 128) * kb * 512 &&
           sfb.numel() == ((N + 127) / 128) * kb * 512,
       "nvfp4_gemm: scale tensors must be in the blocked layout of nvfp4_quantize_act / nvfp4_block_scales");
  need((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(b.data_ptr()) & 15) == 0,
       "nvfp4_gemm: operands must be 16-byte aligned");
  c10::cuda::CUDAGuard g(a.device());
  auto out = at::empty({M, N}, a.options().dtype(at::kBFloat16));
  auto status = at::zeros({1}, a.options().dtype(at::kInt));
  tb::launch_nvfp4_gemm(a.data_ptr<uint8_t>(), sfa.data_ptr<uint8_t>(), b.data_ptr<uint8_t>(), sfb.data_ptr<uint8_t>(), bfm(out),
                        (int)M, (int)N, (int)K, (float)alpha, opt_bias(bias, N), gelu, status.data_ptr<int>(), (int)tile_n, cur());
  return {out, status};
}

// bf16 [R, K] -> (E4M3 [R, K], blocked power-of-two scales per 32 elements)
std::vector<at::Tensor> mxfp8_quantize(const at::Tensor& x) {
  need(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == at::kBFloat16, "mxfp8_quantize: bf16 [R,K] CUDA");
  need(x.size(1) % 32 == 0 && x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0,
       "mxfp8_quantize: K % 32 == 0 and 16-byte aligned rows");
  c10::cuda::CUDAGuard g(x.device());
  const int64_t R = x.size(0), K = x.size(1);
  auto q = at::empty({R, K}, x.options().dtype(at::kFloat8_e4m3fn));
  auto sf = at::zeros({(R + 127) / 128, (int64_t)tb::mxfp8_sf_kblocks((int)K), 512}, x.options().dtype(at::kByte));
  tb::launch_mxfp8_quantize(bf(x), x.stride(0), (int)R, (int)K, (uint8_t*)q.data_ptr(), sf.data_ptr<uint8_t>(), cur());
  return {q, sf};
}

// y [M, N] bf16 = alpha * (a .* sfa) (b .* sfb)^T, E4M3 operands with blocked power-of-two scales per 32 elements
std::vector<at::Tensor> mxfp8_gemm(const at::Tensor& a, const at::Tensor& sfa, const at::Tensor& b, const at::Tensor& sfb, double alpha,
                                   int64_t tile_n, const c10::optional<at::Tensor>& bias, bool gelu) {
  need(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2 && a.is_contiguous() && b.is_contiguous() &&
           a.element_size() == 1 && b.element_size() == 1 && a.size(1) == b.size(1),
       "mxfp8_gemm: contiguous E4M3 [M, K] and [N, K]");
  const int64_t M = a.size(0), N = b.size(0), K = a.size(1);
  const int64_t kb = tb::mxfp8_sf_kblocks((int)K);
  need(sfa.is_contiguous() && sfb.is_contiguous() && sfa.numel() == ((M + 127) / 128) * kb * 512 &&
           sfb.numel() == ((N + 127) / 128) * kb * 512,
       "mxfp8_gemm: scale tensors must be in the blocked layout of mxfp8_quantize");
  need((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(b.data_ptr()) & 15) == 0,
       "mxfp8_gemm: operands must be 16-byte aligned");
  c10::cuda::CUDAGuard g(a.device());
  auto out = at::empty({M, N}, a.options().dtype(at::kBFloat16));
  auto status = at::zeros({1}, a.options().dtype(at::kInt));
  tb::launch_mxfp8_gemm((const uint8_t*)a.data_ptr(), sfa.data_ptr<uint8_t>(), (const uint8_t*)b.data_ptr(), sfb.data_ptr<uint8_t>(),
                        bfm(out), (int)M, (int)N, (int)K, (float)alpha, opt_bias(bias, N), gelu, status.data_ptr<int>(), (int)tile_n, cur());
  return {out, status};
}

bool scale_is_bf16(const at::Tensor& scales) {
  need(scales.scalar_type() == at::kBFloat16 || scales.element_size() == 1, "nvfp4: scales must be E4M3 or bf16");
  return scales.scalar_type() == at::kBFloat16;
}

at::Tensor nvfp4_dequant(const at::Tensor& packed, const at::Tensor& scales, const at::Tensor& tscale) {
  need(packed.is_cuda() && packed.dim() == 2 && packed.is_contiguous() && packed.scalar_type() == at::kByte, "nvfp4_dequant: packed uint8 [N,K/2]");
  need(scales.is_contiguous() && scales.numel() * 8 == packed.numel(), "nvfp4_dequant: one scale per 16 elements");
  need(tscale.is_cuda() && tscale.scalar_type() == at::kFloat && tscale.numel() == 1, "nvfp4_dequant: fp32 device tensor scale");
  c10::cuda::CUDAGuard g(packed.device());
  const int64_t N = packed.size(0), K = packed.size(1) * 2;
  auto out = at::empty({N, K}, packed.options().dtype(at::kBFloat16));
  tb::launch_nvfp4_dequant(packed.data_ptr<uint8_t>(), scales.data_ptr(), scale_is_bf16(scales), tscale.data_ptr<float>(), N, K, bfm(out), cur());
  return out;
}

at::Tensor nvfp4_gemv(const at::Tensor& x, const at::Tensor& packed, const at::Tensor& scales, const at::Tensor& tscale) {
  need(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "nvfp4_gemv: bf16 [M,K]");
  need(packed.is_contiguous() && packed.scalar_type() == at::kByte && packed.size(1) * 2 == x.size(1), "nvfp4_gemv: K mismatch");
  need(scales.is_contiguous() && scales.numel() * 8 == packed.numel(), "nvfp4_gemv: one scale per 16 elements");
  need(tscale.is_cuda() && tscale.scalar_type() == at::kFloat && tscale.numel() == 1, "nvfp4_gemv: fp32 device tensor scale");
  c10::cuda::CUDAGuard g(x.device());
  const int64_t M = x.size(0), K = x.size(1), N = packed.size(0);
  auto y = at::empty({M, N}, x.options());
  tb::launch_nvfp4_gemv(bf(x), packed.data_ptr<uint8_t>(), scales.data_ptr(), scale_is_bf16(scales), tscale.data_ptr<float>(), bfm(y), (int)M, (int)N, (int)K, cur());
  return y;
}

at::Tensor fwht16(const at::Tensor& x) {
  need(x.is_cuda() && x.is_contiguous() && x.scalar_type() == at::kBFloat16 && x.numel() % 16 == 0, "fwht16: contiguous bf16, numel % 16");
  c10::cuda::CUDAGuard g(x.device());
  auto out = at::empty_like(x);
  tb::launch_fwht16(bf(x), bfm(out), x.numel(), cur());
  return out;
}


at::Tensor ggml_dequant(const at::Tensor& raw, int64_t type, int64_t numel) {
  need(raw.is_cuda() && raw.scalar_type() == at::kByte && raw.is_contiguous(), "ggml_dequant: contiguous uint8 CUDA buffer");
  c10::cuda::CUDAGuard g(raw.device());
  auto out = at::empty({numel}, raw.options().dtype(at::kBFloat16));
  tb::launch_ggml_dequant(raw.data_ptr<uint8_t>(), (int)type, numel, bfm(out), cur());
  return out;
}

std::vector<at::Tensor> ggml_to_nvfp4(const at::Tensor& raw, int64_t type, int64_t rows, int64_t K, bool hadamard) {
  need(raw.is_cuda() && raw.scalar_type() == at::kByte && raw.is_contiguous(), "ggml_to_nvfp4: contiguous uint8 CUDA buffer");
  c10::cuda::CUDAGuard g(raw.device());
  auto packed = at::empty({rows, K / 2}, raw.options());
  auto scales = at::empty({rows, K / 16}, raw.options().dtype(at::kFloat8_e4m3fn));
  auto tscale = at::empty({}, raw.options().dtype(at::kFloat));
  auto scratch = at::empty({1}, raw.options().dtype(at::kInt));
  tb::launch_ggml_to_nvfp4(raw.data_ptr<uint8_t>(), (int)type, rows, K, hadamard, packed.data_ptr<uint8_t>(),
                           (uint8_t*)scales.data_ptr(), tscale.data_ptr<float>(), (unsigned int*)scratch.data_ptr(), cur());
  return {packed, scales, tscale};
}
}  // namespace

void register_quant(pybind11::module& m) {
  namespace py = pybind11;
  m.def("fp8_quantize_act", &fp8_quantize_act, "bf16 [M,K] -> (E4M3 [M,K], fp32 scales [M,K/128])");
  m.def("fp8_block_gemm", &fp8_block_gemm, "block-scaled E4M3 GEMM (tcgen05 kind::f8f6f4), bf16 out");
  m.def("nvfp4_quantize", &nvfp4_quantize, "[N,K] -> (packed E2M1, E4M3 block scales, fp32 tensor scale)");
  m.def("nvfp4_dequant", &nvfp4_dequant, "packed NVFP4 -> bf16 [N,K]");
  m.def("nvfp4_quantize_act", &nvfp4_quantize_act, "bf16 [M,K] -> (packed E2M1, blocked E4M3 scales) for the block-scaled GEMM");
  m.def("nvfp4_block_scales", &nvfp4_block_scales, "row-major E4M3 scales -> the block-scaled GEMM's layout");
  m.def("nvfp4_gemm", &nvfp4_gemm, "block-scaled E2M1 x E2M1 GEMM (tcgen05 kind::mxf4nvf4), bf16 out", py::arg("a"), py::arg("sfa"),
        py::arg("b"), py::arg("sfb"), py::arg("alpha"), py::arg("tile_n") = 0, py::arg("bias") = py::none(), py::arg("gelu") = false);
  m.def("mxfp8_quantize", &mxfp8_quantize, "bf16 [R,K] -> (E4M3, blocked power-of-two scales per 32 elements)");
  m.def("mxfp8_gemm", &mxfp8_gemm, "block-scaled E4M3 x E4M3 GEMM (tcgen05 kind::mxf8f6f4.block_scale), bf16 out", py::arg("a"),
        py::arg("sfa"), py::arg("b"), py::arg("sfb"), py::arg("alpha"), py::arg("tile_n") = 0, py::arg("bias") = py::none(),
        py::arg("gelu") = false);
  m.def("nvfp4_gemv", &nvfp4_gemv, "y = x @ W^T for M <= 8 straight from packed NVFP4 weights");
  m.def("ggml_dequant", &ggml_dequant, "GGML block formats -> bf16");
  m.def("ggml_to_nvfp4", &ggml_to_nvfp4, "GGML block formats -> NVFP4 (packed, scales, tensor scale) without a bf16 copy");
  m.def("fwht16", &fwht16, "orthonormal 16-point Walsh-Hadamard transform over consecutive groups of 16");
}
