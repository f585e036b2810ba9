// One-time-per-device bookkeeping for launchers. Function attributes such as the dynamic shared-memory limit
// (cudaFuncSetAttribute) belong to one device: a process that drives several GPUs has to set them once on each, so a
// single per-process flag is wrong for every device after the first.
#pragma once
#include <cuda_runtime.h>

namespace tb {

struct PerDeviceOnce {
  static constexpr int kMaxDevices = 64;
  bool done[kMaxDevices] = {};
  // True exactly once per device (the current one); always true for device ordinals past the table.
  bool first_use() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return true;
    if (done[dev]) return false;
    done[dev] = true;
    return true;
  }
};

}  // namespace tb
