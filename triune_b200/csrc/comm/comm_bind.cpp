// Python bindings of the in-kernel NVLink collectives.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "comm.cuh"
#include "fused_gemm.cuh"

namespace {
using torch::Tensor;
inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

tb::PeerTable table(int64_t rank, int64_t world, int64_t bufs_dev, int64_t signals_dev, int64_t multicast) {
  tb::PeerTable pt;
  pt.rank = (int)rank;
  pt.world = (int)world;
  pt.bufs = reinterpret_cast<const uint64_t*>(bufs_dev);
  pt.signals = reinterpret_cast<const uint64_t*>(signals_dev);
  pt.multicast = (uint64_t)multicast;
  return pt;
}

tb::RangeList ranges(const std::vector<int64_t>& flat) {
  TORCH_CHECK(flat.size() % 2 == 0 && flat.size() / 2 <= 64, "at most 64 (begin, end) ranges");
  tb::RangeList r;
  r.count = (int)(flat.size() / 2);
  for (int i = 0; i < r.count; ++i) {
    TORCH_CHECK(flat[2 * i] % 8 == 0 && flat[2 * i + 1] % 8 == 0, "range bounds must be multiples of 8 elements");
    r.r[i].begin = flat[2 * i];
    r.r[i].end = flat[2 * i + 1];
  }
  return r;
}

const uint32_t* epoch_ptr(const c10::optional<Tensor>& t) {
  return t.has_value() && t->defined() ? reinterpret_cast<const uint32_t*>(t->data_ptr<int>()) : nullptr;
}
const float* hyper_ptr(const c10::optional<Tensor>& t) {
  return t.has_value() && t->defined() ? t->data_ptr<float>() : nullptr;
}

int* status_ptr(const c10::optional<Tensor>& st) {
  return st.has_value() && st->defined() ? st->data_ptr<int>() : nullptr;
}

void dp_reduce_scatter(int64_t rank, int64_t world, int64_t bufs, int64_t sigs, int64_t mc, int64_t grad_off, int64_t norm_off,
                       std::vector<int64_t> owned, int64_t epoch, bool use_multimem, Tensor& counter,
                       const c10::optional<Tensor>& status, const c10::optional<Tensor>& epoch_dev) {
  tb::launch_dp_reduce_scatter(table(rank, world, bufs, sigs, mc), grad_off, norm_off, ranges(owned), (uint32_t)epoch,
                               epoch_ptr(epoch_dev), use_multimem, reinterpret_cast<unsigned int*>(counter.data_ptr<int>()), status_ptr(status),
                               cur_stream());
}

void dp_adamw_allgather(int64_t rank, int64_t world, int64_t bufs, int64_t sigs, int64_t mc, int64_t grad_off, int64_t norm_off,
                        int64_t param_off, int64_t begin, int64_t end, int64_t state_base, Tensor& master, Tensor& m, Tensor& v,
                        double lr, double beta1, double beta2, double eps, double wd, int64_t step, double max_norm,
                        Tensor& clip_out, Tensor& norm_out, int64_t epoch, bool use_multimem,
                        const c10::optional<Tensor>& status, const c10::optional<Tensor>& epoch_dev,
                        const c10::optional<Tensor>& hyper) {
  TORCH_CHECK(begin % 8 == 0 && end % 8 == 0, "owned AdamW range must be a multiple of 8 elements");
  tb::ElemRange owned{begin, end};
  tb::launch_dp_adamw_allgather(table(rank, world, bufs, sigs, mc), grad_off, norm_off, param_off, owned, state_base,
                                master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), (float)lr, (float)beta1,
                                (float)beta2, (float)eps, (float)wd, 1.0f - (float)std::pow(beta1, (double)step),
                                1.0f - (float)std::pow(beta2, (double)step), (float)max_norm, clip_out.data_ptr<float>(),
                                norm_out.data_ptr<float>(), (uint32_t)epoch, epoch_ptr(epoch_dev), hyper_ptr(hyper), use_multimem,
                                status_ptr(status), cur_stream());
}

void dp_broadcast_ranges(int64_t rank, int64_t world, int64_t bufs, int64_t sigs, int64_t mc, int64_t param_off,
                         std::vector<int64_t> owned, bool use_multimem) {
  tb::launch_dp_broadcast_ranges(table(rank, world, bufs, sigs, mc), param_off, ranges(owned), use_multimem, cur_stream());
}

void comm_barrier(int64_t rank, int64_t world, int64_t bufs, int64_t sigs, int64_t channel, int64_t epoch,
                  const c10::optional<Tensor>& status, const c10::optional<Tensor>& epoch_dev) {
  tb::launch_comm_barrier(table(rank, world, bufs, sigs, 0), (int)channel, (uint32_t)epoch, epoch_ptr(epoch_dev),
                          status_ptr(status), cur_stream());
}

void comm_wait_only(int64_t rank, int64_t world, int64_t bufs, int64_t sigs, int64_t channel, int64_t epoch, int64_t limit_ns,
                    const c10::optional<Tensor>& status) {
  tb::launch_comm_wait_only(table(rank, world, bufs, sigs, 0), (int)channel, (uint32_t)epoch, (unsigned long long)limit_ns,
                            status_ptr(status), cur_stream());
}

void metric_allreduce(int64_t rank, int64_t world, int64_t bufs, int64_t sigs, int64_t metric_off, const Tensor& local,
                      Tensor& out, int64_t channel, int64_t epoch, const c10::optional<Tensor>& status,
                      const c10::optional<Tensor>& epoch_dev) {
  TORCH_CHECK(local.scalar_type() == at::kFloat && local.is_contiguous() && out.scalar_type() == at::kFloat &&
                  out.is_contiguous() && out.numel() >= local.numel(),
              "metric_allreduce: fp32 contiguous vectors");
  const uint32_t* ed = epoch_ptr(epoch_dev);
  tb::launch_metric_allreduce(table(rank, world, bufs, sigs, 0), metric_off, local.data_ptr<float>(), out.data_ptr<float>(),
                              (int)local.numel(), (int)channel, (uint32_t)epoch, ed, status_ptr(status), cur_stream());
}

// ---------------------------------------------------------------- GEMMs fused with collectives
const __nv_bfloat16* bfp(const Tensor& t) { return reinterpret_cast<const __nv_bfloat16*>(t.data_ptr()); }

Tensor peer_c_maps(std::vector<int64_t> peer_ptrs, int64_t byte_offset, int64_t rows, int64_t N, int64_t ldc, bool f32,
                   const Tensor& like) {
  std::vector<uint64_t> ptrs(peer_ptrs.begin(), peer_ptrs.end());
  auto host = at::empty({(int64_t)ptrs.size() * 128}, at::TensorOptions().dtype(at::kByte).pinned_memory(true));
  tb::build_peer_c_maps(ptrs.data(), (int)ptrs.size(), byte_offset, (int)rows, (int)N, ldc, f32, host.data_ptr());
  auto dev = at::empty({(int64_t)ptrs.size() * 128 + 128}, like.options().dtype(at::kByte));
  // tensor maps must sit on a 64-byte boundary; the caching allocator hands out 512-byte aligned blocks
  dev.narrow(0, 0, host.numel()).copy_(host, /*non_blocking=*/false);
  return dev;
}

void gemm_reduce_scatter(const Tensor& a, const Tensor& b, bool b_mn, int64_t rank, int64_t world, int64_t bufs_dev,
                         const Tensor& c_maps, int64_t rows_per_dest, bool out_f32, const c10::optional<Tensor>& status) {
  TORCH_CHECK(a.is_cuda() && a.dim() == 2 && a.scalar_type() == at::kBFloat16 && a.stride(1) == 1, "A: bf16 [M,K] row-major");
  TORCH_CHECK(b.dim() == 2 && b.scalar_type() == at::kBFloat16 && b.stride(1) == 1, "B: bf16 2-D row-major");
  c10::cuda::CUDAGuard g(a.device());
  tb::FusedGemmArgs f{};
  f.mode = tb::FG_REDUCE_SCATTER;
  f.A = bfp(a); f.B = bfp(b);
  f.M = (int)a.size(0); f.K = (int)a.size(1); f.N = (int)(b_mn ? b.size(1) : b.size(0));
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == f.K, "K mismatch");
  f.lda = a.stride(0); f.ldb = b.stride(0); f.strideB = b.stride(0) * b.size(0);
  f.b_mn_major = b_mn; f.out_f32 = out_f32; f.groups = 1;
  f.rank = (int)rank; f.world = (int)world; f.peer_bufs = reinterpret_cast<const uint64_t*>(bufs_dev);
  f.c_maps = c_maps.data_ptr(); f.rows_per_dest = (int)rows_per_dest;
  f.status = status_ptr(status);
  tb::launch_fused_gemm(f, cur_stream());
}

void allgather_gemm(const Tensor& a_full, const Tensor& b, bool b_mn, Tensor& c, int64_t rank, int64_t world, int64_t bufs_dev,
                    int64_t a_off, int64_t rows_per_src, Tensor& chunk_flags, int64_t epoch, const c10::optional<Tensor>& status) {
  TORCH_CHECK(a_full.is_cuda() && a_full.dim() == 2 && a_full.scalar_type() == at::kBFloat16 && a_full.is_contiguous(), "A: contiguous bf16 [M,K]");
  TORCH_CHECK(c.dim() == 2 && c.stride(1) == 1, "C: 2-D row-major");
  c10::cuda::CUDAGuard g(a_full.device());
  tb::FusedGemmArgs f{};
  f.mode = tb::FG_ALL_GATHER;
  f.A = bfp(a_full); f.B = bfp(b);
  f.M = (int)a_full.size(0); f.K = (int)a_full.size(1); f.N = (int)(b_mn ? b.size(1) : b.size(0));
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == f.K, "K mismatch");
  f.lda = a_full.stride(0); f.ldb = b.stride(0); f.strideB = b.stride(0) * b.size(0);
  f.b_mn_major = b_mn; f.out_f32 = c.scalar_type() == at::kFloat; f.groups = 1;
  f.rank = (int)rank; f.world = (int)world; f.peer_bufs = reinterpret_cast<const uint64_t*>(bufs_dev);
  f.C = c.data_ptr(); f.ldc = c.stride(0); f.a_off = a_off; f.rows_per_src = (int)rows_per_src;
  TORCH_CHECK(chunk_flags.numel() >= 4 * ((f.M + 127) / 128), "chunk_flags too small (4 per 128 rows)");
  f.chunk_flags = reinterpret_cast<uint32_t*>(chunk_flags.data_ptr<int>()); f.epoch = (uint32_t)epoch;
  f.status = status_ptr(status);
  tb::launch_fused_gemm(f, cur_stream());
}

void gemm_scatter_rows(const Tensor& a, const Tensor& b, bool b_mn, const c10::optional<Tensor>& bias, const c10::optional<Tensor>& row_scale,
                       const Tensor& tile_group, const Tensor& row_dst, int64_t slots_per_rank, int64_t rank, int64_t world,
                       int64_t bufs_dev, int64_t out_off, int64_t out_ld, const c10::optional<Tensor>& status) {
  TORCH_CHECK(a.is_cuda() && a.dim() == 2 && a.scalar_type() == at::kBFloat16 && a.stride(1) == 1, "A: bf16 [M,K] row-major");
  TORCH_CHECK(b.dim() == 3 && b.is_contiguous() && b.scalar_type() == at::kBFloat16, "B: contiguous bf16 [groups, N, K] ([groups, K, N] when b_mn)");
  c10::cuda::CUDAGuard g(a.device());
  tb::FusedGemmArgs f{};
  f.mode = tb::FG_SCATTER_ROWS;
  f.A = bfp(a); f.B = bfp(b);
  f.M = (int)a.size(0); f.K = (int)a.size(1); f.N = (int)(b_mn ? b.size(2) : b.size(1));
  TORCH_CHECK((b_mn ? b.size(1) : b.size(2)) == f.K, "K mismatch");
  f.lda = a.stride(0); f.ldb = b.stride(1); f.strideB = b.stride(0); f.groups = (int)b.size(0);
  f.b_mn_major = b_mn; f.out_f32 = false;
  f.rank = (int)rank; f.world = (int)world; f.peer_bufs = reinterpret_cast<const uint64_t*>(bufs_dev);
  f.tile_group = tile_group.data_ptr<int>(); f.row_dst = row_dst.data_ptr<int>(); f.slots_per_rank = (int)slots_per_rank;
  f.out_off = out_off; f.out_ld = out_ld;
  if (bias.has_value() && bias->defined()) { f.bias = bfp(*bias); f.bias_stride = bias->stride(0); }
  if (row_scale.has_value() && row_scale->defined()) f.row_scale = row_scale->data_ptr<float>();
  f.status = status_ptr(status);
  tb::launch_fused_gemm(f, cur_stream());
}

void ep_dispatch(const Tensor& x, const Tensor& idx, const Tensor& pos, int64_t top_k, int64_t experts_per_rank, int64_t cap,
                 int64_t rank, int64_t world, int64_t bufs_dev, int64_t in_off, int64_t dst_off, int64_t cnt_off,
                 const Tensor& counts, int64_t slots_per_rank) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "x: contiguous bf16 [T, d]");
  TORCH_CHECK(idx.scalar_type() == at::kInt && pos.scalar_type() == at::kInt && counts.scalar_type() == at::kInt, "int32 routing tensors");
  c10::cuda::CUDAGuard g(x.device());
  tb::launch_ep_dispatch(bfp(x), (int)x.size(1), idx.data_ptr<int>(), pos.data_ptr<int>(), (int)idx.numel(), (int)top_k,
                         (int)experts_per_rank, (int)cap, (int)rank, (int)world, reinterpret_cast<const uint64_t*>(bufs_dev), in_off,
                         dst_off, cnt_off, counts.data_ptr<int>(), (int)counts.numel(), (int)slots_per_rank, cur_stream());
}

void ep_build_tiles(const Tensor& counts_all, int64_t experts_per_rank, int64_t world, int64_t cap, Tensor& tile_group, Tensor& row_dst) {
  c10::cuda::CUDAGuard g(counts_all.device());
  tb::launch_ep_build_tiles(counts_all.data_ptr<int>(), (int)experts_per_rank, (int)world, (int)cap, tile_group.data_ptr<int>(),
                            row_dst.data_ptr<int>(), cur_stream());
}

void ep_zero_invalid_rows(Tensor& buf, const Tensor& counts_all, int64_t experts_per_rank, int64_t world, int64_t cap) {
  TORCH_CHECK(buf.is_cuda() && buf.dim() == 2 && buf.is_contiguous() && buf.scalar_type() == at::kBFloat16, "buf: contiguous bf16 [rows, d]");
  TORCH_CHECK(buf.size(0) == experts_per_rank * world * cap, "buf rows must be experts_per_rank * world * cap");
  c10::cuda::CUDAGuard g(buf.device());
  tb::launch_ep_zero_invalid_rows(reinterpret_cast<__nv_bfloat16*>(buf.data_ptr()), (int)buf.size(1), counts_all.data_ptr<int>(),
                                  (int)experts_per_rank, (int)world, (int)cap, cur_stream());
}
}  // namespace

void register_comm(pybind11::module& m) {
  namespace py = pybind11;
  m.def("dp_reduce_scatter", &dp_reduce_scatter, py::arg("rank"), py::arg("world"), py::arg("bufs"), py::arg("sigs"),
        py::arg("mc"), py::arg("grad_off"), py::arg("norm_off"), py::arg("owned"), py::arg("epoch"),
        py::arg("use_multimem"), py::arg("counter"), py::arg("status") = py::none(), py::arg("epoch_dev") = py::none());
  m.def("dp_adamw_allgather", &dp_adamw_allgather, py::arg("rank"), py::arg("world"), py::arg("bufs"), py::arg("sigs"),
        py::arg("mc"), py::arg("grad_off"), py::arg("norm_off"), py::arg("param_off"), py::arg("begin"), py::arg("end"),
        py::arg("state_base"), py::arg("master"), py::arg("m"), py::arg("v"), py::arg("lr"), py::arg("beta1"),
        py::arg("beta2"), py::arg("eps"), py::arg("wd"), py::arg("step"), py::arg("max_norm"), py::arg("clip_out"),
        py::arg("norm_out"), py::arg("epoch"), py::arg("use_multimem"), py::arg("status") = py::none(),
        py::arg("epoch_dev") = py::none(), py::arg("hyper") = py::none());
  m.def("dp_broadcast_ranges", &dp_broadcast_ranges);
  m.def("comm_barrier", &comm_barrier, py::arg("rank"), py::arg("world"), py::arg("bufs"), py::arg("sigs"),
        py::arg("channel"), py::arg("epoch"), py::arg("status") = py::none(), py::arg("epoch_dev") = py::none());
  m.def("comm_wait_only", &comm_wait_only);
  m.def("peer_c_maps", &peer_c_maps, "device table of tensor maps over every peer's reduce-scatter output buffer");
  m.def("gemm_reduce_scatter", &gemm_reduce_scatter, "GEMM whose output tiles are TMA reduce-added into the owning rank");
  m.def("allgather_gemm", &allgather_gemm, "GEMM over row-sharded A; remote shards are fetched by in-kernel copy warps");
  m.def("gemm_scatter_rows", &gemm_scatter_rows, "grouped expert GEMM storing each output row into its token owner's buffer");
  m.def("ep_dispatch", &ep_dispatch, "token rows -> expert-major buffers on the expert owners (peer stores)");
  m.def("ep_zero_invalid_rows", &ep_zero_invalid_rows, "zero the rows of an expert-major buffer beyond each segment's count");
  m.def("ep_build_tiles", &ep_build_tiles, "tile list and row validity of the expert owner from the received counts");
  m.def("metric_allreduce", &metric_allreduce, py::arg("rank"), py::arg("world"), py::arg("bufs"), py::arg("sigs"),
        py::arg("metric_off"), py::arg("local"), py::arg("out"), py::arg("channel"), py::arg("epoch"),
        py::arg("status") = py::none(), py::arg("epoch_dev") = py::none());
}
