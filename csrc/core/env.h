// Environment knobs.  The reference documents YALI_* variables in README.md:284-303
// but reads only YALI_DTYPE and YALI_PROFILE_KERNELS (bench/benchmark_yali.cu:87,
// src/ops/allreduce.cuh:55); here every documented knob is live.
#pragma once

#include <cstdint>
#include <string>

#include "status.h"

namespace yali {
namespace env {

// Integer / string lookups with defaults.  Empty values count as unset.
long long GetInt(const char* name, long long dflt);
std::string GetStr(const char* name, const char* dflt);
bool GetBool(const char* name, bool dflt);

KernelMode ForcedKernelMode();  // YALI_KERNEL_MODE=auto|flash|stream|nvls
int DebugLevel();               // YALI_DEBUG=0|1|2
int DevLanes();                 // YALI_DEV_LANES (stream lanes override, 0 = auto)
int DevCtas();                  // YALI_DEV_CTAS  (flash CTA count override, 0 = auto)
long long DevSlotBytes();       // YALI_DEV_SLOT_BYTES (stream slot size override, 0 = auto)
long long TimeoutMs();          // YALI_TIMEOUT_MS (device wait limit; default 2000)
long long HeapBytes();          // YALI_HEAP_BYTES (symmetric heap size; 0 = default for the world size)
bool NvlsDisabled();            // YALI_NVLS_DISABLE=1
bool ProfileKernels();          // YALI_PROFILE_KERNELS=1
std::string TuningFile();       // YALI_TUNING_FILE (json written by the sweep tool)

}  // namespace env
}  // namespace yali
