// yaliAllReduceLocalNoAlloc: the one-shot all-reduce kernel run with its staging and
// flags in a link-time __device__ array instead of a communicator's heap.  See
// capi/yali_no_alloc.h for the contract.  This file has no counterpart in the
// reference library.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../capi/yali_no_alloc.h"
#include "../comm/layout.h"
#include "../ops/tuning.h"
#include "launch.h"

namespace {

// The working memory.  One copy per GPU that loads this library, for the life of the process.
// Zero-initialised by the loader; the flag words are cleared again at set-up.
static __device__ __align__(256) unsigned char g_no_alloc_scratch[YALI_NO_ALLOC_SCRATCH_BYTES];

// The one-shot kernel only touches its own flag rows (the status words are skipped when no status
// block is given), so those rows are all that must fit the per-rank flag area.
static_assert((yali::kFlashFlagOff + yali::kMaxFlashCtas * yali::kMaxRanks) * 4ull <= 128u * 1024u,
              "one-shot flag rows must fit the per-rank flag area");

constexpr int kMaxDevices = 64;
struct PerDevice {
    unsigned char* base = nullptr;  // device address of g_no_alloc_scratch on this device
    int world = 0;                  // group size of the last call (the ranks' call counters must agree)
    int sms = 0;
};
PerDevice g_dev[kMaxDevices];
std::mutex g_mu;
thread_local char g_err[256] = "";

cudaError_t Refuse(cudaError_t e, const char* what) {
    std::snprintf(g_err, sizeof(g_err), "%s", what);
    return e;
}

}  // namespace

extern "C" const char* yaliNoAllocLastError(void) { return g_err; }

extern "C" cudaError_t yaliAllReduceLocalNoAlloc(const void* const* send, void* const* recv, int world, size_t count,
                                                 int dtype, cudaStream_t stream) {
    using namespace yali;
    g_err[0] = 0;
    if (!send || !recv) return Refuse(cudaErrorInvalidValue, "send / recv table is null");
    if (world < 2 || world > YALI_NO_ALLOC_MAX_WORLD)
        return Refuse(cudaErrorInvalidValue, "world must be between 2 and YALI_NO_ALLOC_MAX_WORLD (4)");
    if (dtype < 0 || dtype > 2) return Refuse(cudaErrorInvalidValue, "dtype must be 0 (fp32), 1 (fp16) or 2 (bf16)");
    const Dtype dt = static_cast<Dtype>(dtype);
    // Compare in elements first: count * element size could wrap around for absurd counts.
    if (count > YALI_NO_ALLOC_MAX_BYTES / DtypeSize(dt))
        return Refuse(cudaErrorInvalidValue,
                      "message larger than YALI_NO_ALLOC_MAX_BYTES (262144 bytes per rank): the scratch array is fixed");
    const size_t bytes = count * DtypeSize(dt);
    if (bytes > YALI_NO_ALLOC_MAX_BYTES)
        return Refuse(cudaErrorInvalidValue,
                      "message larger than YALI_NO_ALLOC_MAX_BYTES (262144 bytes per rank): the scratch array is fixed");
    for (int r = 0; r < world; ++r)
        if (!send[r] || !recv[r]) return Refuse(cudaErrorInvalidValue, "a send / recv pointer is null");
    if (count == 0) return cudaSuccess;

    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return Refuse(e, "cudaGetDevice failed");
    if (dev < 0 || dev >= kMaxDevices) return Refuse(cudaErrorInvalidDevice, "device index out of range");

    std::lock_guard<std::mutex> lock(g_mu);
    PerDevice& pd = g_dev[dev];
    if (!pd.base) {
        // Set-up, once per device, with that device current: in host code the array's name is
        // only a handle; the kernel needs the device address.
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_no_alloc_scratch);
        if (e != cudaSuccess) return Refuse(e, "cudaGetSymbolAddress of the scratch array failed");
        e = cudaDeviceGetAttribute(&pd.sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return Refuse(e, "cudaDeviceGetAttribute failed");
        pd.base = static_cast<unsigned char*>(p);
        pd.world = 0;
    }
    if (pd.world != world) {
        // Flags and the ranks' call counters must start at zero, and all ranks of a group must
        // have seen the same calls: clear them on first use and whenever the group size changes
        // (stream-ordered, like the kernel).  Staging needs no clearing: it is written before it
        // is read.
        for (int r = 0; r < YALI_NO_ALLOC_MAX_WORLD; ++r) {
            e = cudaMemsetAsync(pd.base + static_cast<size_t>(r) * YALI_NO_ALLOC_RANK_BYTES, 0, 128u * 1024u, stream);
            if (e != cudaSuccess) return Refuse(e, "clearing the flag words failed");
        }
        pd.world = world;
    }

    const void* fn = FlashKernelFor(dt, dt, kEpiIdentity, world, /*emu=*/true);
    if (!fn) return Refuse(cudaErrorNotSupported, "no kernel for this dtype");

    // CTAs per rank: all ranks' CTAs must be resident together (two 512-thread CTAs fit every SM).
    uint32_t ctas = static_cast<uint32_t>(FlashLanePreset(bytes, dt, world));
    const uint32_t max_ctas = static_cast<uint32_t>(pd.sms > 0 ? pd.sms * 2 / world : 1);
    if (ctas > max_ctas) ctas = max_ctas;
    if (ctas < 1) ctas = 1;

    EmuArgs args;
    std::memset(&args, 0, sizeof(args));
    for (int r = 0; r < world; ++r) {
        CollArgs& a = args.r[r];
        for (int q = 0; q < world; ++q)
            a.cv.heap[q] = reinterpret_cast<char*>(pd.base) + static_cast<size_t>(q) * YALI_NO_ALLOC_RANK_BYTES;
        a.cv.mc_heap = nullptr;
        a.cv.lay.total_bytes = YALI_NO_ALLOC_RANK_BYTES;
        a.cv.lay.flags_off = 0;
        a.cv.lay.flash_off = 128u * 1024u;
        a.cv.lay.flash_cap = YALI_NO_ALLOC_MAX_BYTES;
        a.cv.status = nullptr;
        a.cv.timeout_ns = 2000000000ull;
        a.cv.rank = r;
        a.cv.world = world;
        a.send = send[r];
        a.recv = recv[r];
        a.count = count;
        a.ctas = ctas;
        // The kernel cuts the message into CTA slices from `count` and the CTA count alone, so a
        // rank whose own buffers are not 16-byte aligned may fall back to scalar accesses without
        // its peers noticing.
        const bool aligned = ((reinterpret_cast<uintptr_t>(send[r]) | reinterpret_cast<uintptr_t>(recv[r])) & 15u) == 0;
        a.flags = aligned ? kFlagVecOk : 0u;
        a.ep.scale = 1.0f;
    }
    void* params[] = {&args};
    e = cudaLaunchCooperativeKernel(fn, dim3(ctas, world), dim3(kFlashThreads), params, 0, stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return Refuse(e, "cooperative launch of the all-reduce kernel failed");
    }
    return cudaSuccess;
}
