// NVTX ranges around the host API calls, for timelines in Nsight Systems.
// Compiled out unless the library is built with -DYALI_NVTX (YALI_BUILD_NVTX=1 for
// `python -m yali_b200._build`): the default build contains no NVTX symbol at all.
// NVTX v3 is header-only and does nothing until a tool attaches, so an NVTX build
// costs a few nanoseconds per call when no profiler runs.
//
// Parity: the reference profiles through the sweep script's nsys wrapper only
// (scripts/sweep.py:1198-1496) and has no ranges in the library.
#pragma once

#ifdef YALI_NVTX
#include <nvtx3/nvToolsExt.h>

namespace yali {
class NvtxRange {
   public:
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};
}  // namespace yali
#define YALI_NVTX_RANGE(name) ::yali::NvtxRange yali_nvtx_range_(name)
#else
#define YALI_NVTX_RANGE(name) \
    do {                      \
    } while (0)
#endif
