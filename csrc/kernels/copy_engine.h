// Host entry points of the kernels of the copy-engine all-reduce (copy_engine.cu).
#pragma once

#include <cuda_runtime.h>

#include "../comm/layout.h"

namespace yali {

constexpr int kCeReduceThreads = 512;
constexpr uint32_t kCeMaxChunks = 64;  // per rank and call; the progress word keeps 8 bits for the chunk count

struct alignas(16) CeReduceArgs {
    CommView cv;
    const void* in;                       // this rank's own data for the chunk
    void* out;                            // where the sums go (may equal `in`)
    const void* staged[kMaxRanks - 1];    // the peers' copies of the chunk, by SrcSlot(source, rank)
    uint64_t elems;
    uint32_t announce_chunk;  // one-shot: chunk index + 1, published to the peers as "read"; 0: nothing to publish
    uint32_t wait_pulled;     // one-shot in place: wait until every peer has read this chunk here before overwriting it
};

cudaError_t CeLaunchEnter(const CommView& cv, uint32_t plan_word, uint32_t flags, cudaStream_t s);
cudaError_t CeLaunchWaitEnter(const CommView& cv, uint32_t mask, cudaStream_t s);
cudaError_t CeLaunchDone(const CommView& cv, int peer, cudaStream_t s);
cudaError_t CeLaunchExit(const CommView& cv, uint32_t chunks, bool one_shot, uint32_t flags, cudaStream_t s);
cudaError_t CeLaunchReduce(const CeReduceArgs& a, Dtype dt, uint32_t ctas, cudaStream_t s);

}  // namespace yali
