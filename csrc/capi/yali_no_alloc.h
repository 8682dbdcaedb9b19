/* An all-reduce entry point that never allocates.
 *
 * This entry point has no counterpart in the reference library.
 *
 * Who needs it: some programs cannot obtain device memory at the moment they want to
 * reduce.  An inference server that handed all free HBM to its own pool at start-up
 * (every later cudaMalloc fails), a plug-in that runs inside somebody else's stream
 * capture, a hot path with a real-time budget that may not enter the driver's
 * allocator, or a host that forbids library-side allocations by policy.  The normal
 * way into this library (creating a communicator) allocates a symmetric heap; this
 * function does not.  It reserves its working memory at link time instead: a
 * file-scope __device__ array inside the library, which every GPU that loads the
 * library carries until the process exits (about 6.6 MB, see
 * YALI_NO_ALLOC_SCRATCH_BYTES).
 *
 * What it does: a one-shot sum all-reduce among `world` logical ranks whose buffers
 * all live on the CURRENT device (the multi-rank kernel of this library run as one
 * cooperative launch, ranks = blockIdx.y).  send[r] / recv[r] are rank r's input and
 * output of `count` elements of `dtype` (0 fp32, 1 fp16, 2 bf16); recv[r] may equal
 * send[r].  Every recv[r] receives the element-wise sum over the ranks, accumulated
 * in fp32 in rank order, so all ranks get bit-identical results.  The caller owns
 * all of send and recv; nothing else is touched except the library's scratch array.
 *
 * Limits: 2 <= world <= YALI_NO_ALLOC_MAX_WORLD and count * element size <=
 * YALI_NO_ALLOC_MAX_BYTES; anything larger is refused with cudaErrorInvalidValue and a
 * message from yaliNoAllocLastError().  No cudaMalloc, cudaFree, or allocating
 * library routine is called, on the first call or later.
 *
 * First call on a device: looks up the device address of the scratch array
 * (cudaGetSymbolAddress); that set-up is done once per device, with that device
 * current.  The flag words of the array are cleared on `stream` on that first call
 * and again whenever `world` differs from the previous call on the device.  Make the
 * first call before you start capturing a stream.
 *
 * Waits: ranks wait for one another inside the kernel with a two-second limit.  All ranks
 * run in one cooperative launch, so the limit cannot be reached in practice; should it
 * ever be (a GPU so loaded that co-resident CTAs starve for seconds), the call still
 * returns cudaSuccess, the outputs are incomplete and later calls on that device keep
 * failing the same way until a call with a different `world` clears the flag words.
 * This entry point has no status block to report through; use a communicator where that
 * matters.
 *
 * Alignment: any element-aligned pointers work, and ranks may differ (a rank whose
 * buffers are not 16-byte aligned is merely slower).
 *
 * Sharing: all calls on a device use the same scratch array, and the array keeps
 * what the last call left there.  Calls are safe one after another in one stream (or
 * otherwise ordered); two calls that overlap on the GPU race on the scratch and give
 * wrong sums.
 */
#ifndef YALI_B200_NO_ALLOC_H_
#define YALI_B200_NO_ALLOC_H_

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define YALI_NO_ALLOC_MAX_WORLD 4
#define YALI_NO_ALLOC_MAX_BYTES (256u * 1024u)                 /* largest message per rank */
#define YALI_NO_ALLOC_RANK_BYTES (128u * 1024u + 2u * 3u * YALI_NO_ALLOC_MAX_BYTES) /* flags + 2 halves x 3 sources */
#define YALI_NO_ALLOC_SCRATCH_BYTES (YALI_NO_ALLOC_MAX_WORLD * YALI_NO_ALLOC_RANK_BYTES)

cudaError_t yaliAllReduceLocalNoAlloc(const void* const* send, void* const* recv, int world, size_t count, int dtype,
                                      cudaStream_t stream);
/* Text of the last refusal or CUDA failure of the calling thread ("" when none). */
const char* yaliNoAllocLastError(void);

#ifdef __cplusplus
}
#endif
#endif
