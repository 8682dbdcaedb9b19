// Parsing helpers and environment knobs (see env.h, status.h).
#include <strings.h>

#include <cstdlib>
#include <cstring>

#include "env.h"
#include "status.h"

namespace yali {

bool ParseDtype(const char* s, Dtype* out) {
    if (!s) return false;
    if (!strcasecmp(s, "fp32") || !strcasecmp(s, "f32") || !strcasecmp(s, "float") || !strcasecmp(s, "float32")) {
        *out = Dtype::FP32;
        return true;
    }
    if (!strcasecmp(s, "fp16") || !strcasecmp(s, "f16") || !strcasecmp(s, "half") || !strcasecmp(s, "float16")) {
        *out = Dtype::FP16;
        return true;
    }
    if (!strcasecmp(s, "bf16") || !strcasecmp(s, "bfloat16")) {
        *out = Dtype::BF16;
        return true;
    }
    return false;
}

bool ParseKernelMode(const char* s, KernelMode* out) {
    if (!s) return false;
    if (!strcasecmp(s, "auto")) *out = KernelMode::Auto;
    else if (!strcasecmp(s, "flash")) *out = KernelMode::Flash;
    else if (!strcasecmp(s, "stream")) *out = KernelMode::Stream;
    else if (!strcasecmp(s, "nvls")) *out = KernelMode::NVLS;
    else if (!strcasecmp(s, "flash_pull")) *out = KernelMode::FlashPull;
    else if (!strcasecmp(s, "stream_direct")) *out = KernelMode::StreamDirect;
    else if (!strcasecmp(s, "copy_engine") || !strcasecmp(s, "ce")) *out = KernelMode::CopyEngine;
    else return false;
    return true;
}

namespace env {

long long GetInt(const char* name, long long dflt) {
    const char* v = std::getenv(name);
    if (!v || !*v) return dflt;
    char* end = nullptr;
    long long x = std::strtoll(v, &end, 0);
    if (end == v) return dflt;
    // Size suffixes: K, M, G (binary).
    if (*end == 'k' || *end == 'K') x <<= 10;
    else if (*end == 'm' || *end == 'M') x <<= 20;
    else if (*end == 'g' || *end == 'G') x <<= 30;
    return x;
}

std::string GetStr(const char* name, const char* dflt) {
    const char* v = std::getenv(name);
    return (v && *v) ? std::string(v) : std::string(dflt ? dflt : "");
}

bool GetBool(const char* name, bool dflt) {
    const char* v = std::getenv(name);
    if (!v || !*v) return dflt;
    return !(v[0] == '0' || v[0] == 'n' || v[0] == 'N' || v[0] == 'f' || v[0] == 'F');
}

KernelMode ForcedKernelMode() {
    KernelMode m = KernelMode::Auto;
    std::string s = GetStr("YALI_KERNEL_MODE", "auto");
    ParseKernelMode(s.c_str(), &m);
    return m;
}
int DebugLevel() { return static_cast<int>(GetInt("YALI_DEBUG", 0)); }
int DevLanes() { return static_cast<int>(GetInt("YALI_DEV_LANES", 0)); }
int DevCtas() { return static_cast<int>(GetInt("YALI_DEV_CTAS", 0)); }
long long DevSlotBytes() { return GetInt("YALI_DEV_SLOT_BYTES", 0); }
long long TimeoutMs() { return GetInt("YALI_TIMEOUT_MS", 2000); }
long long HeapBytes() { return GetInt("YALI_HEAP_BYTES", 0); }
bool NvlsDisabled() { return GetBool("YALI_NVLS_DISABLE", false); }
bool ProfileKernels() { return GetBool("YALI_PROFILE_KERNELS", false); }
std::string TuningFile() { return GetStr("YALI_TUNING_FILE", ""); }

}  // namespace env
}  // namespace yali
