// Peer-access helpers, topology query and NVLink speed-of-light arithmetic.
//
// Parity: P2PCapability / CheckP2PAccess / EnableP2PAccess /
// EnableBidirectionalP2P / EnablePeerAccessOrDie / TopologyInfo / QueryTopology /
// PrintTopology (src/common/peer_access.cuh:14-134); NVLinkInfo /
// DetectNVLinkConfig / GetGpuName / SoLMetrics / CalculateSoL
// (src/common/hw_info.cuh:40-205).  The reference shells out to `nvidia-smi
// nvlink -s`; here the link configuration comes from the device's compute
// capability plus an optional measured-peaks file, and the topology also reports
// multicast (NVLS) and fabric-handle support.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <string>
#include <vector>

namespace yali {

struct P2PCapability {
    bool can_access_0_to_1 = false;
    bool can_access_1_to_0 = false;
    bool bidirectional = false;
    int perf_rank = -1;        // cudaDevP2PAttrPerformanceRank (lower is better), -1 unknown
    bool native_atomics = false;
};

P2PCapability CheckP2PAccess(int dev0, int dev1);
// Enables dev -> peer access; "already enabled" counts as success.
cudaError_t EnableP2PAccess(int dev, int peer);
bool EnableBidirectionalP2P(int dev0, int dev1);
// All pairs among `devices`.
bool EnableAllPairsP2P(const std::vector<int>& devices);
// Prints the CUDA error and exits the process when access cannot be enabled (harness use only).
void EnablePeerAccessOrDie(int dev, int peer);

struct TopologyInfo {
    int device_count = 0;
    std::vector<std::vector<bool>> can_access;  // [from][to]
    std::vector<bool> multicast_supported;      // per device
    std::vector<bool> fabric_handle_supported;  // per device
    std::vector<std::string> names;
    bool AllPairsConnected() const;
    // Number of unordered pairs with access both ways.
    int ConnectedPairs() const;
};
TopologyInfo QueryTopology();
void PrintTopology(const TopologyInfo& info);

struct NVLinkInfo {
    int linkCount = 0;
    double bwPerLinkGBs = 0.0;       // per direction
    double unidirectionalGBs = 0.0;  // linkCount * bwPerLinkGBs
    double bidirectionalGBs = 0.0;
    double measuredUnidirectionalGBs = 0.0;  // from a measured-peaks file when available, else 0
    bool viaSwitch = false;                  // every peer at full rate (NVSwitch)
    bool valid = false;
};
// Compute capability 10.x: NVLink 5, 18 links x 50 GB/s per direction through NVSwitch.
// 9.x: NVLink 4, 18 x 25.  8.x: NVLink 3, 12 x 25.
NVLinkInfo DetectNVLinkConfig(int device = 0);
NVLinkInfo NVLinkConfigForComputeCapability(int major, int minor);
const char* GetGpuName(int device = 0);

struct SoLMetrics {
    double algBwGBs = 0.0;
    double busBwGBs = 0.0;               // algBw * 2(n-1)/n
    double unidirectionalPeakGBs = 0.0;
    double bidirectionalPeakGBs = 0.0;
    double theoreticalMinUs = 0.0;       // bus bytes at the unidirectional rate
    double solPercent = 0.0;             // busBw / unidirectional peak
    int nvlinkCount = 0;
};
SoLMetrics CalculateSoL(size_t bytes, double avgSec, int numGpus, const NVLinkInfo& nvlink);
// NCCL's all-reduce bus-bandwidth factor 2(n-1)/n.
inline double BusBwFactor(int n) { return n > 1 ? 2.0 * (n - 1) / n : 1.0; }

}  // namespace yali
