// Host helpers shared by the launchers: cached device properties and launch error codes.
#pragma once
#include <cuda_runtime.h>

#include <algorithm>

namespace zc {

// Number of SMs of the current device (cached per device index).
inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

// 0 on success, else the cudaError_t of the launch (configuration errors are reported here;
// execution errors surface at the next synchronisation).
inline int launch_status() {
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

constexpr int ERR_BAD_ARG = -1;
constexpr int ERR_UNSUPPORTED = -2;

}  // namespace zc
