#include "cuda_driver.h"

#include <mutex>

namespace yali {

namespace {
DriverApi g_api;
bool g_ok = false;
std::string g_err;
std::once_flag g_once;

template <typename F>
bool Resolve(const char* name, F* out) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
        (void)cudaGetLastError();
        g_err = std::string("driver entry point not available: ") + name;
        return false;
    }
    *out = reinterpret_cast<F>(fn);
    return true;
}

void Init() {
    g_ok = Resolve("cuGetErrorString", &g_api.GetErrorString) && Resolve("cuDeviceGet", &g_api.DeviceGet) &&
           Resolve("cuDeviceGetAttribute", &g_api.DeviceGetAttribute) &&
           Resolve("cuMemGetAllocationGranularity", &g_api.MemGetAllocationGranularity) &&
           Resolve("cuMemCreate", &g_api.MemCreate) && Resolve("cuMemRelease", &g_api.MemRelease) &&
           Resolve("cuMemAddressReserve", &g_api.MemAddressReserve) &&
           Resolve("cuMemAddressFree", &g_api.MemAddressFree) && Resolve("cuMemMap", &g_api.MemMap) &&
           Resolve("cuMemUnmap", &g_api.MemUnmap) && Resolve("cuMemSetAccess", &g_api.MemSetAccess) &&
           Resolve("cuMemGetAddressRange", &g_api.MemGetAddressRange) &&
           Resolve("cuMemExportToShareableHandle", &g_api.MemExportToShareableHandle) &&
           Resolve("cuMemImportFromShareableHandle", &g_api.MemImportFromShareableHandle) &&
           Resolve("cuMulticastCreate", &g_api.MulticastCreate) &&
           Resolve("cuMulticastAddDevice", &g_api.MulticastAddDevice) &&
           Resolve("cuMulticastBindMem", &g_api.MulticastBindMem) &&
           Resolve("cuMulticastUnbind", &g_api.MulticastUnbind) &&
           Resolve("cuMulticastGetGranularity", &g_api.MulticastGetGranularity) &&
           Resolve("cuTensorMapEncodeTiled", &g_api.TensorMapEncodeTiled);
}
}  // namespace

const DriverApi* DriverApi::Get(std::string* err) {
    std::call_once(g_once, Init);
    if (!g_ok) {
        if (err) *err = g_err;
        return nullptr;
    }
    return &g_api;
}

std::string DriverApi::ErrorText(CUresult r) const {
    const char* s = nullptr;
    if (GetErrorString && GetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
    return "CUresult " + std::to_string(static_cast<int>(r));
}

}  // namespace yali
