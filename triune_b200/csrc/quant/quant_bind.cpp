// Python bindings of the quantisation kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "quant.cuh"

void register_quant(pybind11::module& m) { (void)m; }
