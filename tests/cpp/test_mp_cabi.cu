// The multi-process C ABI end to end, one process per rank (start with
// `python -m yali_b200.launch -np 2 build/bin/test_mp_cabi`): yaliMPCommCreate, broadcast and
// all-gather over the control plane, yaliIpcExchangeBuffers followed by a kernel that reads
// every peer's buffer through comm->peerPtrs, yaliIpcExchangeRingBuffers with four lanes
// (sequence / gating / data arrays of every rank written and read back through the
// imported pointers), the close functions and yaliMPCommDestroy.  The ranks meet at host
// barriers between the steps, so no kernel waits for another process and the test also
// runs with all ranks on one GPU.
//
// Reference counterpart: examples/02_multi_process/01_allreduce/multilane_mpi.cu:125-187
// drives the same entry points (src/comm/comm.h:76-113, src/comm/ipc.cuh:51-142) by hand.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "comm/mp_comm.h"

#define CK(x)                                                                                      \
    do {                                                                                           \
        cudaError_t e_ = (x);                                                                      \
        if (e_ != cudaSuccess) {                                                                   \
            std::printf("rank %d: %s failed: %s (line %d)\n", g_rank, #x, cudaGetErrorString(e_), __LINE__); \
            return 1;                                                                              \
        }                                                                                          \
    } while (0)

static int g_rank = -1;

struct PeerTable {
    const float* p[8];
};

// out[i] = sum over ranks of peers[r][i], in rank order.
__global__ void sum_peers(PeerTable t, int world, float* out, size_t n) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float s = 0.f;
        for (int r = 0; r < world; ++r) s += t.p[r][i];
        out[i] = s;
    }
}
__global__ void fill(float* p, size_t n, float base) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        p[i] = base + static_cast<float>(i % 251);
}
// Writes a word that names (writer, lane) into the writer's element of a peer's array.
__global__ void stamp(unsigned long long* peer_array, int writer, int lane) {
    peer_array[writer] = 0xabc00000ull + static_cast<unsigned long long>(writer) * 100 + lane;
}

int main(int argc, char** argv) {
    YaliMPComm* comm = yaliMPCommCreate(&argc, &argv);
    if (!comm) {
        std::printf("yaliMPCommCreate failed\n");
        return 1;
    }
    const int rank = comm->rank, W = comm->worldSize;
    g_rank = rank;
    int fails = 0;
    if (W < 2 || W > 8) {
        std::printf("needs 2..8 ranks, got %d\n", W);
        return 1;
    }
    if (comm->localRank != yaliGetLocalRankFromEnv()) ++fails;

    // ---- control plane: broadcast and all-gather
    unsigned long long token = rank == 0 ? 0x1234567890abcdefull : 0;
    yaliMPCommBroadcast(comm, &token, sizeof(token));
    if (token != 0x1234567890abcdefull) ++fails;
    std::vector<int> ranks(W, -1);
    const int mine = rank * 7 + 1;
    if (yaliMPCommAllgather(comm, &mine, ranks.data(), sizeof(int)) != 0) ++fails;
    for (int r = 0; r < W; ++r)
        if (ranks[r] != r * 7 + 1) ++fails;
    std::vector<unsigned long long> ids(W);
    yaliMPCommAllgather(comm, &comm->uniqueId, ids.data(), sizeof(unsigned long long));
    for (int r = 0; r < W; ++r)
        if (ids[r] != comm->uniqueId) ++fails;

    // ---- user buffers: export, exchange, read the peers' memory from a kernel
    const size_t n = 1 << 20;
    float *send = nullptr, *out = nullptr;
    CK(cudaMalloc(&send, n * sizeof(float)));
    CK(cudaMalloc(&out, n * sizeof(float)));
    fill<<<64, 256, 0, comm->stream>>>(send, n, 1000.0f * (rank + 1));
    CK(cudaStreamSynchronize(comm->stream));
    if (yaliIpcExchangeBuffers(comm, send, n * sizeof(float)) != 0) {
        std::printf("rank %d: yaliIpcExchangeBuffers failed\n", rank);
        return 1;
    }
    if (comm->peerPtrs[rank] != send) ++fails;
    PeerTable t;
    std::memset(&t, 0, sizeof(t));
    for (int r = 0; r < W; ++r) t.p[r] = static_cast<const float*>(comm->peerPtrs[r]);
    yaliMPCommBarrier(comm);  // every rank's buffer is filled and mapped
    sum_peers<<<128, 256, 0, comm->stream>>>(t, W, out, n);
    CK(cudaStreamSynchronize(comm->stream));
    yaliMPCommBarrier(comm);  // nobody unmaps while a peer still reads
    std::vector<float> host(n);
    CK(cudaMemcpy(host.data(), out, n * sizeof(float), cudaMemcpyDeviceToHost));
    size_t bad = 0;
    for (size_t i = 0; i < n; ++i) {
        float want = 0.f;
        for (int r = 0; r < W; ++r) want += 1000.0f * (r + 1) + static_cast<float>(i % 251);
        if (host[i] != want) ++bad;
    }
    if (bad) {
        std::printf("rank %d: %zu wrong sums through peerPtrs\n", rank, bad);
        ++fails;
    }
    // An interior pointer of the same allocation: the handle names the allocation, the offset is kept.
    YaliIpcHandle h;
    CK(yaliIpcExport(send + 4096, 1024, &h));
    if (h.offset != 4096 * sizeof(float)) ++fails;
    yaliIpcCloseAll(comm);
    for (int r = 0; r < W; ++r)
        if (comm->peerPtrs[r] != nullptr) ++fails;

    // ---- rings of a caller that manages its own: four lanes, three arrays each
    const int lanes = 4;
    std::vector<YaliRingDesc> rings(lanes);
    for (int l = 0; l < lanes; ++l) {
        rings[l].sequenceBytes = 64 * 1024;
        rings[l].gatingBytes = 64 * 1024;
        rings[l].dataBytes = 1 << 20;
        CK(cudaMalloc(&rings[l].sequence, rings[l].sequenceBytes));
        CK(cudaMalloc(&rings[l].gating, rings[l].gatingBytes));
        CK(cudaMalloc(&rings[l].data, rings[l].dataBytes));
        CK(cudaMemset(rings[l].sequence, 0, rings[l].sequenceBytes));
        CK(cudaMemset(rings[l].gating, 0, rings[l].gatingBytes));
        CK(cudaMemset(rings[l].data, 0, rings[l].dataBytes));
    }
    void **pseq = nullptr, **pgat = nullptr, **pdat = nullptr;
    if (yaliIpcExchangeRingBuffers(comm, rings.data(), lanes, &pseq, &pgat, &pdat) != 0) {
        std::printf("rank %d: yaliIpcExchangeRingBuffers failed\n", rank);
        return 1;
    }
    for (int l = 0; l < lanes; ++l)
        if (pseq[rank * lanes + l] != rings[l].sequence || pdat[rank * lanes + l] != rings[l].data) ++fails;
    yaliMPCommBarrier(comm);
    // Every rank stamps element [rank] of every rank's three arrays of every lane ...
    for (int r = 0; r < W; ++r)
        for (int l = 0; l < lanes; ++l) {
            stamp<<<1, 1, 0, comm->stream>>>(static_cast<unsigned long long*>(pseq[r * lanes + l]), rank, l);
            stamp<<<1, 1, 0, comm->stream>>>(static_cast<unsigned long long*>(pgat[r * lanes + l]), rank, l + 10);
            stamp<<<1, 1, 0, comm->stream>>>(static_cast<unsigned long long*>(pdat[r * lanes + l]), rank, l + 20);
        }
    CK(cudaStreamSynchronize(comm->stream));
    yaliMPCommBarrier(comm);
    // ... and finds all ranks' stamps in its own arrays.
    for (int l = 0; l < lanes; ++l) {
        unsigned long long got[3][8];
        CK(cudaMemcpy(got[0], rings[l].sequence, sizeof(unsigned long long) * W, cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(got[1], rings[l].gating, sizeof(unsigned long long) * W, cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(got[2], rings[l].data, sizeof(unsigned long long) * W, cudaMemcpyDeviceToHost));
        for (int k = 0; k < 3; ++k)
            for (int r = 0; r < W; ++r)
                if (got[k][r] != 0xabc00000ull + static_cast<unsigned long long>(r) * 100 + l + 10 * k) ++fails;
    }
    yaliMPCommBarrier(comm);
    yaliIpcCloseRingBuffers(comm, lanes, pseq, pgat, pdat);
    for (int l = 0; l < lanes; ++l) {
        cudaFree(rings[l].sequence);
        cudaFree(rings[l].gating);
        cudaFree(rings[l].data);
    }
    cudaFree(send);
    cudaFree(out);

    // ---- verdict: every rank must agree
    std::vector<int> all_fails(W, 0);
    yaliMPCommAllgather(comm, &fails, all_fails.data(), sizeof(int));
    int total = 0;
    for (int f : all_fails) total += f;
    if (rank == 0) std::printf("C ABI test on %d ranks: %s (%d failed checks)\n", W, total ? "FAILED" : "PASSED", total);
    yaliMPCommDestroy(comm);
    return total ? 1 : 0;
}
