// All-reduce of buffers in pinned host memory, with the host-to-device copy, the
// collective and the device-to-host copy overlapped chunk by chunk.
//
// Parity: none in the reference (its ops take device pointers only,
// src/ops/allreduce.cuh:563-565); a program whose data lives on the host pays the
// sum of the three phases there, here about one direction's copy time.
#pragma once

#include <cuda_runtime.h>

#include <vector>

#include "../comm/communicator.h"

namespace yali {

class HostPipeline {
   public:
    explicit HostPipeline(Communicator& comm) : comm_(comm) {}
    ~HostPipeline();
    HostPipeline(const HostPipeline&) = delete;
    HostPipeline& operator=(const HostPipeline&) = delete;

    // dst[i] = epilogue(sum over ranks of src) for every local rank i; src / dst are page-locked
    // host buffers of `count` elements.  The message moves in chunks of about `chunk_bytes` (0: about 32
    // chunks of 1-8 MiB)
    // through a ring of four symmetric staging buffers per direction (allocated from the
    // symmetric heap on first use: every process must make the same calls).  Work is queued
    // behind `user_streams[i]` (or the communicator's own stream), which also waits for the
    // last chunk; the call itself does not block.
    // `copies_only` leaves the collective out (dst = src through the device): the same copies on the
    // same streams, which is the ceiling the host link sets for this call.
    Result AllReduce(const void* const* src, void* const* dst, uint64_t count, Dtype dt, const OpOptions& opt,
                     uint64_t chunk_bytes, const cudaStream_t* user_streams, bool copies_only = false);

    // The staging ring lives in the symmetric heap: forget it when that heap is reset.
    void Invalidate() { slot_bytes_ = 0; }

   private:
    static constexpr int kSlots = 4;
    struct PerLocal {
        cudaStream_t h2d = nullptr, comp = nullptr, d2h = nullptr;
        cudaEvent_t start = nullptr;
        cudaEvent_t copied_in[kSlots] = {}, reduced[kSlots] = {}, copied_out[kSlots] = {};
    };
    Result Prepare(uint64_t chunk_bytes);

    Communicator& comm_;
    std::vector<PerLocal> loc_;
    uint64_t slot_bytes_ = 0;  // capacity of every staging buffer
    std::vector<void*> send_[kSlots], recv_[kSlots];  // [slot][local rank]
};

}  // namespace yali
