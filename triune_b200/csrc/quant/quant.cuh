// Launchers of the quantisation kernels (NVFP4 / FP8 block-scaled quantise, dequantise, GEMM).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {
}  // namespace tb
