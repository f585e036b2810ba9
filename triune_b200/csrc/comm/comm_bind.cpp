// Python bindings of the in-kernel NVLink collectives.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "comm.cuh"

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
                      Tensor& out, int64_t channel, int64_t epoch, const c10::optional<Tensor>& status) {
  tb::launch_metric_allreduce(table(rank, world, bufs, sigs, 0), metric_off, local.data_ptr<float>(), out.data_ptr<float>(),
                              (int)local.numel(), (int)channel, (uint32_t)epoch, status_ptr(status), cur_stream());
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
  m.def("metric_allreduce", &metric_allreduce);
}
