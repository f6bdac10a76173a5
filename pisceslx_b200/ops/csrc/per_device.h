// A flag per CUDA device for one-time, per-device set-up (cudaFuncSetAttribute opt-ins and the like).  Function
// attributes belong to the device's context, so a process that drives several GPUs has to repeat the opt-in on each.
#pragma once
#include <cuda_runtime.h>

namespace yv {

struct PerDeviceInt {
  static constexpr int kMaxDevices = 64;
  int v[kMaxDevices] = {0};
  // Value slot of the calling thread's current device.
  int& cur() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) d = 0;
    return v[d];
  }
};

}  // namespace yv
