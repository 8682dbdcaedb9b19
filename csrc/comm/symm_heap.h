// The symmetric heap: one device allocation per rank, mapped into every rank's
// address space, optionally also bound to one NVSwitch multicast object.
//
// Parity: the reference makes peer memory reachable with
// cudaDeviceEnablePeerAccess inside one process (src/common/peer_access.cuh:41-71)
// and with legacy CUDA IPC across processes, one handle per buffer and three per
// ring lane (src/comm/ipc.cu:27-148, 166-379).  Here a communicator exports ONE
// cuMem allocation per rank as a POSIX file descriptor (passed over the
// bootstrap's Unix sockets), with cudaMalloc + cudaIpc as the fallback, and
// cuMulticast* for the NVLS path.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "../core/status.h"
#include "bootstrap.h"

namespace yali {

class SymmHeapSet {
   public:
    // One process drives all ranks.  devices[r] is the GPU of rank r; the same
    // device may appear several times (ranks emulated on one GPU: no multicast).
    static Result CreateLocal(const std::vector<int>& devices, uint64_t bytes, bool want_multicast,
                              std::unique_ptr<SymmHeapSet>* out, std::string* err);
    // One rank per process.  Collective over `bs`.
    static Result CreateShared(Bootstrap& bs, int device, uint64_t bytes, bool want_multicast,
                               std::unique_ptr<SymmHeapSet>* out, std::string* err);
    ~SymmHeapSet();

    int world() const { return static_cast<int>(base_.size()); }
    uint64_t bytes() const { return bytes_; }
    char* base(int rank) const { return base_[rank]; }
    char* mc_base() const { return mc_base_; }
    const char* kind() const { return kind_; }  // "cumem-local" | "cumem-fd" | "cuda-ipc"

    // Size/alignment that both the allocation and (if supported) the multicast object accept.
    static uint64_t RoundUpBytes(uint64_t bytes, int device, int world, bool want_multicast);

   private:
    SymmHeapSet() = default;
    void Destroy();
    bool SetupMulticastLocal(const std::vector<int>& devices, std::string* why);
    bool SetupMulticastShared(Bootstrap& bs, int device, std::string* why);

    std::vector<char*> base_;
    std::vector<unsigned long long> handles_;  // CUmemGenericAllocationHandle per mapped heap (0 for cudaIpc)
    std::vector<int> own_devices_;             // devices whose memory this process allocated
    std::vector<int> owned_;                   // 1 when this process allocated heap r
    uint64_t bytes_ = 0;
    char* mc_base_ = nullptr;
    unsigned long long mc_handle_ = 0;
    std::vector<int> mc_devices_;  // devices this process added/bound (for unbind)
    const char* kind_ = "none";
    bool ipc_ = false;
};

}  // namespace yali
