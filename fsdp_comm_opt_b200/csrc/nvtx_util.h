// NVTX ranges around the C launchers, so that a timeline (Nsight Systems, torch.profiler with NVTX
// capture) shows the collective / codec / GEMM calls of this library by name on the host row next to
// the kernels they launch.  NVTX v3 is header-only and does nothing until a tool attaches.
#pragma once
#include <nvtx3/nvToolsExt.h>

namespace zc {

struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

}  // namespace zc

#define ZC_NVTX_RANGE(name) ::zc::NvtxRange zc_nvtx_range_(name)
