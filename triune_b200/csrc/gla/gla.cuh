// Launchers of the gated-linear-attention kernels (chunked scan forward/backward, decode step).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {
}  // namespace tb
