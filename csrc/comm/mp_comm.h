/* C ABI of the multi-process layer: communicator bootstrap and CUDA-IPC export /
 * import of user buffers.
 *
 * Parity: yaliMPCommCreate / Destroy / Barrier / Broadcast, yaliGetLocalRankFromEnv
 * (src/comm/comm.h:76-113, comm.cu:28-216) and yaliIpcExport / Import / Close /
 * ExchangeBuffers / CloseAll / ExchangeRingBuffers / CloseRingBuffers
 * (src/comm/ipc.cuh:51-142, ipc.cu:27-407).  Same entry points; the control plane
 * behind them is the library's bootstrap (environment rendezvous over Unix
 * sockets, or MPI when built with YALI_MPI_SUPPORT) instead of raw MPI calls, and
 * the rings of the two-shot kernel live in the symmetric heap, so the ring
 * exchange is only needed by callers that manage their own rings.
 */
#ifndef YALI_B200_MP_COMM_H_
#define YALI_B200_MP_COMM_H_

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct YaliMPComm {
    int rank;
    int worldSize;
    int localRank;
    int localSize;
    int useMpi;                      /* non-zero when MPI carries the control plane */
    cudaIpcMemHandle_t* peerHandles; /* [worldSize] handles of the last yaliIpcExchangeBuffers */
    void** peerPtrs;                 /* [worldSize] opened pointers (own slot = local buffer) */
    cudaStream_t stream;
    void* bootstrap;                 /* opaque control-plane object */
    uint64_t uniqueId;               /* same value on every rank of the job */
} YaliMPComm;

YaliMPComm* yaliMPCommCreate(int* argc, char*** argv);
void yaliMPCommDestroy(YaliMPComm* comm);
void yaliMPCommBarrier(YaliMPComm* comm);
void yaliMPCommBroadcast(YaliMPComm* comm, void* data, size_t bytes);
/* out has worldSize*bytes bytes. Returns 0 on success. */
int yaliMPCommAllgather(YaliMPComm* comm, const void* in, void* out, size_t bytes);
int yaliGetLocalRankFromEnv(void);

typedef struct YaliIpcHandle {
    cudaIpcMemHandle_t handle;
    size_t size;
    size_t offset; /* of the exported pointer inside its allocation */
    int srcRank;
} YaliIpcHandle;

cudaError_t yaliIpcExport(void* devPtr, size_t size, YaliIpcHandle* handle);
cudaError_t yaliIpcImport(const YaliIpcHandle* handle, void** devPtr);
cudaError_t yaliIpcClose(void* importedPtr);
/* Collective: every rank exports localBuf; afterwards comm->peerPtrs[r] addresses rank r's buffer. 0 on success. */
int yaliIpcExchangeBuffers(YaliMPComm* comm, void* localBuf, size_t size);
void yaliIpcCloseAll(YaliMPComm* comm);

typedef struct YaliRingDesc {
    void* sequence;
    void* gating;
    void* data;
    size_t sequenceBytes;
    size_t gatingBytes;
    size_t dataBytes;
} YaliRingDesc;
/* Collective: exports numLanes rings; peerX[r * numLanes + lane] addresses rank r's lane (arrays malloc'd here). */
int yaliIpcExchangeRingBuffers(YaliMPComm* comm, const YaliRingDesc* localRings, int numLanes, void*** peerSequence,
                               void*** peerGating, void*** peerData);
void yaliIpcCloseRingBuffers(YaliMPComm* comm, int numLanes, void** peerSequence, void** peerGating, void** peerData);

#ifdef __cplusplus
}
#endif
#endif /* YALI_B200_MP_COMM_H_ */
