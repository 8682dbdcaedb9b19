#include "symm_heap.h"

#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstring>

#include "../core/env.h"
#include "cuda_driver.h"
#include "layout.h"

namespace yali {

namespace {

constexpr uint64_t kFallbackGranularity = 2ull << 20;

CUmemAllocationProp AllocProp(int device) {
    CUmemAllocationProp prop;
    std::memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

bool EnsureContext(int device) {
    if (cudaSetDevice(device) != cudaSuccess) return false;
    return cudaFree(nullptr) == cudaSuccess;
}

bool DeviceSupportsMulticast(const DriverApi* d, int device) {
    CUdevice dev;
    if (d->DeviceGet(&dev, device) != CUDA_SUCCESS) return false;
    int v = 0;
    if (d->DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return false;
    return v != 0;
}

void Debug(const char* fmt, const std::string& s) {
    if (env::DebugLevel() > 0) std::fprintf(stderr, fmt, s.c_str());
}

uint64_t RoundUp(uint64_t x, uint64_t g) { return (x + g - 1) / g * g; }

// Reserves VA, maps `handle` and grants read/write to `devices`.
CUresult MapHandle(const DriverApi* d, CUmemGenericAllocationHandle handle, uint64_t bytes, uint64_t align,
                   const std::vector<int>& devices, char** out) {
    CUdeviceptr va = 0;
    CUresult r = d->MemAddressReserve(&va, bytes, align, 0, 0);
    if (r != CUDA_SUCCESS) return r;
    r = d->MemMap(va, bytes, 0, handle, 0);
    if (r != CUDA_SUCCESS) {
        d->MemAddressFree(va, bytes);
        return r;
    }
    std::vector<CUmemAccessDesc> acc(devices.size());
    for (size_t i = 0; i < devices.size(); ++i) {
        std::memset(&acc[i], 0, sizeof(CUmemAccessDesc));
        acc[i].location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        acc[i].location.id = devices[i];
        acc[i].flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    }
    r = d->MemSetAccess(va, bytes, acc.data(), acc.size());
    if (r != CUDA_SUCCESS) {
        d->MemUnmap(va, bytes);
        d->MemAddressFree(va, bytes);
        return r;
    }
    *out = reinterpret_cast<char*>(va);
    return CUDA_SUCCESS;
}

std::vector<int> Unique(const std::vector<int>& v) {
    std::vector<int> u(v);
    std::sort(u.begin(), u.end());
    u.erase(std::unique(u.begin(), u.end()), u.end());
    return u;
}

}  // namespace

uint64_t SymmHeapSet::RoundUpBytes(uint64_t bytes, int device, int world, bool want_multicast) {
    std::string err;
    const DriverApi* d = DriverApi::Get(&err);
    uint64_t g = kFallbackGranularity;
    if (d && EnsureContext(device)) {
        CUmemAllocationProp prop = AllocProp(device);
        size_t ag = 0;
        if (d->MemGetAllocationGranularity(&ag, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && ag)
            g = std::max<uint64_t>(g, ag);
        if (want_multicast && world > 1 && DeviceSupportsMulticast(d, device)) {
            CUmulticastObjectProp mp;
            std::memset(&mp, 0, sizeof(mp));
            mp.numDevices = world;
            mp.size = RoundUp(bytes, g);
            mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
            size_t mg = 0;
            if (d->MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg)
                g = std::max<uint64_t>(g, mg);
        }
    }
    return RoundUp(bytes, g);
}

Result SymmHeapSet::CreateLocal(const std::vector<int>& devices, uint64_t bytes, bool want_multicast,
                                std::unique_ptr<SymmHeapSet>* out, std::string* err) {
    const int world = static_cast<int>(devices.size());
    if (world < 1 || world > kMaxRanks) {
        if (err) *err = "world size out of range";
        return Result::InvalidArg;
    }
    std::string derr;
    const DriverApi* d = DriverApi::Get(&derr);
    if (!d) {
        if (err) *err = derr;
        return Result::CudaError;
    }
    const std::vector<int> uniq = Unique(devices);
    for (int a : uniq) {
        for (int b : uniq) {
            if (a == b) continue;
            int can = 0;
            if (cudaDeviceCanAccessPeer(&can, a, b) != cudaSuccess || !can) {
                if (err) *err = "GPU " + std::to_string(a) + " cannot access GPU " + std::to_string(b);
                return Result::PeerAccessFailed;
            }
        }
    }
    std::unique_ptr<SymmHeapSet> h(new SymmHeapSet());
    const bool mc_possible = want_multicast && static_cast<int>(uniq.size()) == world && world > 1;
    h->bytes_ = RoundUpBytes(bytes, devices[0], world, mc_possible);
    h->kind_ = "cumem-local";
    h->base_.assign(world, nullptr);
    h->handles_.assign(world, 0);
    h->owned_.assign(world, 1);
    h->own_devices_ = devices;
    for (int r = 0; r < world; ++r) {
        if (!EnsureContext(devices[r])) {
            if (err) *err = "cannot initialise GPU " + std::to_string(devices[r]);
            return Result::CudaError;
        }
        CUmemAllocationProp prop = AllocProp(devices[r]);
        CUmemGenericAllocationHandle handle = 0;
        CUresult cr = d->MemCreate(&handle, h->bytes_, &prop, 0);
        if (cr != CUDA_SUCCESS) {
            if (err) *err = "cuMemCreate failed: " + d->ErrorText(cr);
            return Result::CudaError;
        }
        h->handles_[r] = handle;
        cr = MapHandle(d, handle, h->bytes_, kFallbackGranularity, uniq, &h->base_[r]);
        if (cr != CUDA_SUCCESS) {
            if (err) *err = "mapping a heap failed: " + d->ErrorText(cr);
            return cr == CUDA_ERROR_INVALID_DEVICE ? Result::PeerAccessFailed : Result::CudaError;
        }
        if (cudaMemset(h->base_[r], 0, kFlagRegionBytes) != cudaSuccess) {
            if (err) *err = "cudaMemset of the flag region failed";
            return Result::CudaError;
        }
    }
    for (int dev : uniq) {
        cudaSetDevice(dev);
        cudaDeviceSynchronize();
    }
    if (mc_possible && !env::NvlsDisabled()) {
        std::string why;
        if (!h->SetupMulticastLocal(devices, &why)) Debug("[yali] multicast not used: %s\n", why);
    }
    *out = std::move(h);
    return Result::Success;
}

bool SymmHeapSet::SetupMulticastLocal(const std::vector<int>& devices, std::string* why) {
    const DriverApi* d = DriverApi::Get(why);
    if (!d) return false;
    for (int dev : devices) {
        if (!DeviceSupportsMulticast(d, dev)) {
            *why = "GPU " + std::to_string(dev) + " does not support multicast";
            return false;
        }
    }
    CUmulticastObjectProp mp;
    std::memset(&mp, 0, sizeof(mp));
    mp.numDevices = static_cast<unsigned>(devices.size());
    mp.size = bytes_;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUmemGenericAllocationHandle mc = 0;
    CUresult r = d->MulticastCreate(&mc, &mp);
    if (r != CUDA_SUCCESS) {
        *why = "cuMulticastCreate: " + d->ErrorText(r);
        return false;
    }
    mc_handle_ = mc;
    for (int dev : devices) {
        CUdevice cd;
        d->DeviceGet(&cd, dev);
        r = d->MulticastAddDevice(mc, cd);
        if (r != CUDA_SUCCESS) {
            *why = "cuMulticastAddDevice: " + d->ErrorText(r);
            d->MemRelease(mc);
            mc_handle_ = 0;
            return false;
        }
    }
    for (size_t i = 0; i < devices.size(); ++i) {
        r = d->MulticastBindMem(mc, 0, handles_[i], 0, bytes_, 0);
        if (r != CUDA_SUCCESS) {
            *why = "cuMulticastBindMem: " + d->ErrorText(r);
            for (int dev : mc_devices_) {
                CUdevice cd;
                d->DeviceGet(&cd, dev);
                d->MulticastUnbind(mc, cd, 0, bytes_);
            }
            mc_devices_.clear();
            d->MemRelease(mc);
            mc_handle_ = 0;
            return false;
        }
        mc_devices_.push_back(devices[i]);
    }
    r = MapHandle(d, mc, bytes_, kFallbackGranularity, Unique(devices), &mc_base_);
    if (r != CUDA_SUCCESS) {
        *why = "mapping the multicast object: " + d->ErrorText(r);
        for (int dev : mc_devices_) {
            CUdevice cd;
            d->DeviceGet(&cd, dev);
            d->MulticastUnbind(mc, cd, 0, bytes_);
        }
        mc_devices_.clear();
        d->MemRelease(mc);
        mc_handle_ = 0;
        mc_base_ = nullptr;
        return false;
    }
    return true;
}

Result SymmHeapSet::CreateShared(Bootstrap& bs, int device, uint64_t bytes, bool want_multicast,
                                 std::unique_ptr<SymmHeapSet>* out, std::string* err) {
    const int world = bs.world(), rank = bs.rank();
    if (world == 1) return CreateLocal({device}, bytes, false, out, err);
    if (!EnsureContext(device)) {
        if (err) *err = "cannot initialise GPU " + std::to_string(device);
        return Result::CudaError;
    }
    std::string derr;
    const DriverApi* d = DriverApi::Get(&derr);
    std::unique_ptr<SymmHeapSet> h(new SymmHeapSet());
    h->base_.assign(world, nullptr);
    h->handles_.assign(world, 0);
    h->owned_.assign(world, 0);
    h->owned_[rank] = 1;
    h->own_devices_.assign(1, device);

    // All ranks must use the same size: rank 0 decides.
    uint64_t rounded = RoundUpBytes(bytes, device, world, want_multicast);
    if (bs.broadcast(&rounded, sizeof(rounded), 0) != Result::Success) {
        if (err) *err = bs.last_error();
        return Result::BootstrapError;
    }
    h->bytes_ = rounded;

    // --- preferred: cuMem allocation shared as a POSIX file descriptor
    int my_fd = -1;
    char ok = 0;
    CUmemGenericAllocationHandle own = 0;
    if (d && !env::GetBool("YALI_FORCE_CUDA_IPC", false)) {
        CUmemAllocationProp prop = AllocProp(device);
        if (d->MemCreate(&own, h->bytes_, &prop, 0) == CUDA_SUCCESS) {
            if (d->MemExportToShareableHandle(&my_fd, own, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) ==
                CUDA_SUCCESS)
                ok = 1;
            else
                d->MemRelease(own), own = 0;
        }
    }
    std::vector<char> oks(world);
    if (bs.allgather(&ok, oks.data(), 1) != Result::Success) {
        if (err) *err = bs.last_error();
        return Result::BootstrapError;
    }
    const bool all_fd = std::all_of(oks.begin(), oks.end(), [](char c) { return c != 0; });
    if (all_fd) {
        h->kind_ = "cumem-fd";
        std::vector<int> fds;
        Result br = bs.allgather_fd(my_fd, &fds);
        ::close(my_fd);
        if (br != Result::Success) {
            if (err) *err = bs.last_error();
            d->MemRelease(own);
            return br;
        }
        char map_ok = 1;
        std::string map_err;
        for (int r = 0; r < world; ++r) {
            CUmemGenericAllocationHandle handle = own;
            if (r != rank) {
                CUresult cr = d->MemImportFromShareableHandle(&handle, reinterpret_cast<void*>(static_cast<intptr_t>(fds[r])),
                                                              CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
                if (cr != CUDA_SUCCESS) {
                    map_ok = 0;
                    map_err = "cuMemImportFromShareableHandle: " + d->ErrorText(cr);
                    break;
                }
            }
            h->handles_[r] = handle;
            CUresult cr = MapHandle(d, handle, h->bytes_, kFallbackGranularity, {device}, &h->base_[r]);
            if (cr != CUDA_SUCCESS) {
                map_ok = 0;
                map_err = "mapping the heap of rank " + std::to_string(r) + ": " + d->ErrorText(cr);
                break;
            }
        }
        for (int fd : fds)
            if (fd >= 0) ::close(fd);
        if (!map_ok && own && h->handles_[rank] == 0) d->MemRelease(own);
        std::vector<char> maps(world);
        if (bs.allgather(&map_ok, maps.data(), 1) != Result::Success) {
            if (err) *err = bs.last_error();
            return Result::BootstrapError;
        }
        if (!std::all_of(maps.begin(), maps.end(), [](char c) { return c != 0; })) {
            if (err) *err = map_ok ? "another rank could not map the heaps" : map_err;
            return Result::PeerAccessFailed;
        }
    } else {
        // --- fallback: cudaMalloc + legacy CUDA IPC handles (what the reference always does)
        if (own) d->MemRelease(own);
        if (my_fd >= 0) ::close(my_fd);
        h->kind_ = "cuda-ipc";
        h->ipc_ = true;
        void* p = nullptr;
        cudaIpcMemHandle_t mine;
        std::memset(&mine, 0, sizeof(mine));
        char a_ok = cudaMalloc(&p, h->bytes_) == cudaSuccess && cudaIpcGetMemHandle(&mine, p) == cudaSuccess;
        h->base_[rank] = static_cast<char*>(p);
        std::vector<cudaIpcMemHandle_t> all(world);
        std::vector<char> aoks(world);
        if (bs.allgather(&a_ok, aoks.data(), 1) != Result::Success ||
            bs.allgather(&mine, all.data(), sizeof(mine)) != Result::Success) {
            if (err) *err = bs.last_error();
            return Result::BootstrapError;
        }
        char o_ok = std::all_of(aoks.begin(), aoks.end(), [](char c) { return c != 0; });
        for (int r = 0; r < world && o_ok; ++r) {
            if (r == rank) continue;
            void* q = nullptr;
            if (cudaIpcOpenMemHandle(&q, all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                (void)cudaGetLastError();
                o_ok = 0;
                break;
            }
            h->base_[r] = static_cast<char*>(q);
        }
        std::vector<char> ooks(world);
        if (bs.allgather(&o_ok, ooks.data(), 1) != Result::Success) {
            if (err) *err = bs.last_error();
            return Result::BootstrapError;
        }
        if (!std::all_of(ooks.begin(), ooks.end(), [](char c) { return c != 0; })) {
            if (err) *err = "neither cuMem file descriptors nor CUDA IPC could share the heaps";
            return Result::PeerAccessFailed;
        }
        want_multicast = false;
    }
    if (cudaMemset(h->base_[rank], 0, kFlagRegionBytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        if (err) *err = "clearing the flag region failed";
        return Result::CudaError;
    }
    if (bs.barrier() != Result::Success) {
        if (err) *err = bs.last_error();
        return Result::BootstrapError;
    }
    if (want_multicast && !env::NvlsDisabled()) {
        std::string why;
        if (!h->SetupMulticastShared(bs, device, &why) && rank == 0) Debug("[yali] multicast not used: %s\n", why);
    }
    *out = std::move(h);
    return Result::Success;
}

// Collective.  Every step that can fail on one rank is followed by an agreement
// round, so either all ranks end up with a mapped multicast object or none.
bool SymmHeapSet::SetupMulticastShared(Bootstrap& bs, int device, std::string* why) {
    const int world = bs.world(), rank = bs.rank();
    const DriverApi* d = DriverApi::Get(why);
    auto agree = [&](bool mine) {
        char c = mine ? 1 : 0;
        std::vector<char> all(world);
        if (bs.allgather(&c, all.data(), 1) != Result::Success) return false;
        return std::all_of(all.begin(), all.end(), [](char x) { return x != 0; });
    };
    if (!agree(d && DeviceSupportsMulticast(d, device))) {
        *why = "a GPU of the communicator does not support multicast";
        return false;
    }
    CUdevice cd;
    d->DeviceGet(&cd, device);
    CUmemGenericAllocationHandle mc = 0;
    int fd = -1;
    bool ok = true;
    if (rank == 0) {
        CUmulticastObjectProp mp;
        std::memset(&mp, 0, sizeof(mp));
        mp.numDevices = world;
        mp.size = bytes_;
        mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        CUresult r = d->MulticastCreate(&mc, &mp);
        if (r != CUDA_SUCCESS) {
            *why = "cuMulticastCreate: " + d->ErrorText(r);
            ok = false;
        } else if ((r = d->MemExportToShareableHandle(&fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0)) !=
                   CUDA_SUCCESS) {
            *why = "exporting the multicast object: " + d->ErrorText(r);
            d->MemRelease(mc);
            mc = 0;
            ok = false;
        }
    }
    char root_ok = ok ? 1 : 0;
    if (bs.broadcast(&root_ok, 1, 0) != Result::Success || !root_ok) {
        if (why->empty()) *why = "rank 0 could not create the multicast object";
        return false;
    }
    int got = fd;
    if (bs.broadcast_fd(&got, 0) != Result::Success) {
        if (rank == 0) {
            ::close(fd);
            d->MemRelease(mc);
        }
        *why = bs.last_error();
        return false;
    }
    if (rank == 0) {
        ::close(fd);
    } else {
        CUresult r = d->MemImportFromShareableHandle(&mc, reinterpret_cast<void*>(static_cast<intptr_t>(got)),
                                                     CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
        if (r != CUDA_SUCCESS) {
            *why = "importing the multicast object: " + d->ErrorText(r);
            ok = false;
            mc = 0;
        }
    }
    if (got >= 0) ::close(got);
    if (ok) {
        CUresult r = d->MulticastAddDevice(mc, cd);
        if (r != CUDA_SUCCESS) {
            *why = "cuMulticastAddDevice: " + d->ErrorText(r);
            ok = false;
        }
    }
    if (!agree(ok)) {  // doubles as the barrier "all devices added" that binding requires
        if (mc) d->MemRelease(mc);
        if (why->empty()) *why = "another rank could not join the multicast object";
        return false;
    }
    CUresult r = d->MulticastBindMem(mc, 0, handles_[rank], 0, bytes_, 0);
    bool bound = (r == CUDA_SUCCESS);
    if (!bound) *why = "cuMulticastBindMem: " + d->ErrorText(r);
    char* va = nullptr;
    bool mapped = false;
    if (bound) {
        r = MapHandle(d, mc, bytes_, kFallbackGranularity, {device}, &va);
        mapped = (r == CUDA_SUCCESS);
        if (!mapped) *why = "mapping the multicast object: " + d->ErrorText(r);
    }
    if (!agree(bound && mapped)) {
        if (mapped) {
            d->MemUnmap(reinterpret_cast<CUdeviceptr>(va), bytes_);
            d->MemAddressFree(reinterpret_cast<CUdeviceptr>(va), bytes_);
        }
        if (bound) d->MulticastUnbind(mc, cd, 0, bytes_);
        d->MemRelease(mc);
        if (why->empty()) *why = "another rank could not bind or map the multicast object";
        return false;
    }
    mc_handle_ = mc;
    mc_base_ = va;
    mc_devices_.assign(1, device);
    return true;
}

void SymmHeapSet::Destroy() {
    std::string err;
    const DriverApi* d = DriverApi::Get(&err);
    if (mc_handle_ && d) {
        if (mc_base_) {
            d->MemUnmap(reinterpret_cast<CUdeviceptr>(mc_base_), bytes_);
            d->MemAddressFree(reinterpret_cast<CUdeviceptr>(mc_base_), bytes_);
        }
        for (int dev : mc_devices_) {
            CUdevice cd;
            if (d->DeviceGet(&cd, dev) == CUDA_SUCCESS) d->MulticastUnbind(mc_handle_, cd, 0, bytes_);
        }
        d->MemRelease(mc_handle_);
        mc_handle_ = 0;
        mc_base_ = nullptr;
    }
    for (size_t r = 0; r < base_.size(); ++r) {
        if (!base_[r]) continue;
        if (ipc_) {
            if (owned_[r]) cudaFree(base_[r]);
            else cudaIpcCloseMemHandle(base_[r]);
        } else if (d) {
            d->MemUnmap(reinterpret_cast<CUdeviceptr>(base_[r]), bytes_);
            d->MemAddressFree(reinterpret_cast<CUdeviceptr>(base_[r]), bytes_);
            if (handles_[r]) d->MemRelease(handles_[r]);
        }
        base_[r] = nullptr;
    }
    (void)cudaGetLastError();
}

SymmHeapSet::~SymmHeapSet() { Destroy(); }

}  // namespace yali
