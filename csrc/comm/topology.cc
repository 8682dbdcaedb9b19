#include "topology.h"

#include <cstdio>
#include <cstdlib>

#include "cuda_driver.h"

namespace yali {

P2PCapability CheckP2PAccess(int dev0, int dev1) {
    P2PCapability cap;
    int a = 0, b = 0;
    if (cudaDeviceCanAccessPeer(&a, dev0, dev1) != cudaSuccess) (void)cudaGetLastError();
    if (cudaDeviceCanAccessPeer(&b, dev1, dev0) != cudaSuccess) (void)cudaGetLastError();
    cap.can_access_0_to_1 = a != 0;
    cap.can_access_1_to_0 = b != 0;
    cap.bidirectional = a && b;
    int v = 0;
    if (cudaDeviceGetP2PAttribute(&v, cudaDevP2PAttrPerformanceRank, dev0, dev1) == cudaSuccess) cap.perf_rank = v;
    else (void)cudaGetLastError();
    if (cudaDeviceGetP2PAttribute(&v, cudaDevP2PAttrNativeAtomicSupported, dev0, dev1) == cudaSuccess)
        cap.native_atomics = v != 0;
    else (void)cudaGetLastError();
    return cap;
}

cudaError_t EnableP2PAccess(int dev, int peer) {
    if (dev == peer) return cudaSuccess;
    int can = 0;
    cudaError_t e = cudaDeviceCanAccessPeer(&can, dev, peer);
    if (e != cudaSuccess) return e;
    if (!can) return cudaErrorPeerAccessUnsupported;
    int prev = 0;
    cudaGetDevice(&prev);
    e = cudaSetDevice(dev);
    if (e != cudaSuccess) return e;
    e = cudaDeviceEnablePeerAccess(peer, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();
        e = cudaSuccess;
    }
    cudaSetDevice(prev);
    return e;
}

bool EnableBidirectionalP2P(int dev0, int dev1) {
    return EnableP2PAccess(dev0, dev1) == cudaSuccess && EnableP2PAccess(dev1, dev0) == cudaSuccess;
}

bool EnableAllPairsP2P(const std::vector<int>& devices) {
    for (size_t i = 0; i < devices.size(); ++i)
        for (size_t j = i + 1; j < devices.size(); ++j)
            if (devices[i] != devices[j] && !EnableBidirectionalP2P(devices[i], devices[j])) return false;
    return true;
}

void EnablePeerAccessOrDie(int dev, int peer) {
    cudaError_t e = EnableP2PAccess(dev, peer);
    if (e != cudaSuccess) {
        std::fprintf(stderr, "Peer access %d -> %d failed: %s\n", dev, peer, cudaGetErrorString(e));
        std::exit(EXIT_FAILURE);
    }
}

bool TopologyInfo::AllPairsConnected() const {
    for (int i = 0; i < device_count; ++i)
        for (int j = 0; j < device_count; ++j)
            if (i != j && !can_access[i][j]) return false;
    return true;
}

int TopologyInfo::ConnectedPairs() const {
    int n = 0;
    for (int i = 0; i < device_count; ++i)
        for (int j = i + 1; j < device_count; ++j)
            if (can_access[i][j] && can_access[j][i]) ++n;
    return n;
}

TopologyInfo QueryTopology() {
    TopologyInfo t;
    if (cudaGetDeviceCount(&t.device_count) != cudaSuccess) {
        (void)cudaGetLastError();
        t.device_count = 0;
    }
    const int n = t.device_count;
    t.can_access.assign(n, std::vector<bool>(n, false));
    t.multicast_supported.assign(n, false);
    t.fabric_handle_supported.assign(n, false);
    t.names.assign(n, "");
    std::string err;
    const DriverApi* d = n ? DriverApi::Get(&err) : nullptr;
    for (int i = 0; i < n; ++i) {
        cudaDeviceProp p;
        if (cudaGetDeviceProperties(&p, i) == cudaSuccess) t.names[i] = p.name;
        for (int j = 0; j < n; ++j) {
            if (i == j) {
                t.can_access[i][j] = true;
                continue;
            }
            int can = 0;
            if (cudaDeviceCanAccessPeer(&can, i, j) != cudaSuccess) (void)cudaGetLastError();
            t.can_access[i][j] = can != 0;
        }
        if (d) {
            CUdevice cd;
            int v = 0;
            if (d->DeviceGet(&cd, i) == CUDA_SUCCESS) {
                if (d->DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd) == CUDA_SUCCESS)
                    t.multicast_supported[i] = v != 0;
                if (d->DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_FABRIC_SUPPORTED, cd) == CUDA_SUCCESS)
                    t.fabric_handle_supported[i] = v != 0;
            }
        }
    }
    return t;
}

void PrintTopology(const TopologyInfo& t) {
    std::printf("GPUs: %d, peer-connected pairs: %d of %d\n", t.device_count, t.ConnectedPairs(),
                t.device_count * (t.device_count - 1) / 2);
    for (int i = 0; i < t.device_count; ++i) {
        std::printf("  GPU %d %-24s multicast=%d fabric=%d  peers:", i, t.names[i].c_str(),
                    static_cast<int>(t.multicast_supported[i]), static_cast<int>(t.fabric_handle_supported[i]));
        for (int j = 0; j < t.device_count; ++j)
            if (i != j) std::printf(" %d%s", j, t.can_access[i][j] ? "" : "(x)");
        std::printf("\n");
    }
}

NVLinkInfo NVLinkConfigForComputeCapability(int major, int /*minor*/) {
    NVLinkInfo info;
    if (major >= 10) {
        info.linkCount = 18;
        info.bwPerLinkGBs = 50.0;
        info.viaSwitch = true;
    } else if (major == 9) {
        info.linkCount = 18;
        info.bwPerLinkGBs = 25.0;
        info.viaSwitch = true;
    } else if (major == 8) {
        info.linkCount = 12;
        info.bwPerLinkGBs = 25.0;
    } else if (major == 7) {
        info.linkCount = 6;
        info.bwPerLinkGBs = 25.0;
    } else {
        return info;
    }
    info.unidirectionalGBs = info.linkCount * info.bwPerLinkGBs;
    info.bidirectionalGBs = 2.0 * info.unidirectionalGBs;
    info.valid = true;
    return info;
}

NVLinkInfo DetectNVLinkConfig(int device) {
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, device) != cudaSuccess) {
        (void)cudaGetLastError();
        return NVLinkInfo();
    }
    NVLinkInfo info = NVLinkConfigForComputeCapability(p.major, p.minor);
    // A measured peer-copy rate, when the operator provides one, is the honest denominator.
    if (const char* m = std::getenv("YALI_MEASURED_P2P_GBS")) info.measuredUnidirectionalGBs = std::atof(m);
    return info;
}

const char* GetGpuName(int device) {
    static thread_local char name[256];
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, device) != cudaSuccess) {
        (void)cudaGetLastError();
        std::snprintf(name, sizeof(name), "unknown");
    } else {
        std::snprintf(name, sizeof(name), "%s", p.name);
    }
    return name;
}

SoLMetrics CalculateSoL(size_t bytes, double avgSec, int numGpus, const NVLinkInfo& nv) {
    SoLMetrics m;
    if (avgSec <= 0.0) return m;
    m.algBwGBs = static_cast<double>(bytes) / avgSec / 1e9;
    m.busBwGBs = m.algBwGBs * BusBwFactor(numGpus);
    m.unidirectionalPeakGBs = nv.unidirectionalGBs;
    m.bidirectionalPeakGBs = nv.bidirectionalGBs;
    m.nvlinkCount = nv.linkCount;
    if (nv.unidirectionalGBs > 0.0) {
        m.theoreticalMinUs = static_cast<double>(bytes) * BusBwFactor(numGpus) / (nv.unidirectionalGBs * 1e9) * 1e6;
        m.solPercent = 100.0 * m.busBwGBs / nv.unidirectionalGBs;
    }
    return m;
}

}  // namespace yali
