// nccl_sweep: the NCCL baseline over a range of message sizes in ONE process group (one process
// per GPU), so that a size sweep does not pay NCCL's start-up once per size.  Timing is the code of
// benchmark_nccl_mpi: small messages as one CUDA-graph replay of all calls, large ones with one
// CUDA-event pair around the calls, max over ranks.  One JSON line per (dtype, size), in the row
// format of bench/sweep.py, so bench/report.py joins both.
//
//   python -m yali_b200.launch -np N build/bin/nccl_sweep [min_bytes=4096] [max_bytes=1073741824]
//          [dtypes=fp32] [graph_max_bytes=4194304]
//
// Parity: the reference sweeps NCCL by starting bench/benchmark_nccl once per size
// (scripts/sweep.py:576-621).
#include <cuda_runtime.h>
#include <nccl.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "comm/bootstrap.h"
#include "comm/topology.h"
#include "core/status.h"
#include "ops/buffer_ops.h"

using namespace yali;

#define CK(x)                                                                                \
    do {                                                                                     \
        cudaError_t e_ = (x);                                                                \
        if (e_ != cudaSuccess) {                                                             \
            std::fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            std::exit(1);                                                                    \
        }                                                                                    \
    } while (0)
#define NK(x)                                                                                \
    do {                                                                                     \
        ncclResult_t r_ = (x);                                                               \
        if (r_ != ncclSuccess) {                                                             \
            std::fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, ncclGetErrorString(r_)); \
            std::exit(1);                                                                    \
        }                                                                                    \
    } while (0)

int main(int argc, char** argv) {
    const size_t min_bytes = argc > 1 ? std::strtoull(argv[1], nullptr, 10) : 4096;
    const size_t max_bytes = argc > 2 ? std::strtoull(argv[2], nullptr, 10) : (1ull << 30);
    const std::string dtypes = argc > 3 ? argv[3] : "fp32";
    const size_t graph_max = argc > 4 ? std::strtoull(argv[4], nullptr, 10) : (4ull << 20);
    Result res;
    std::string err;
    std::unique_ptr<Bootstrap> bs = MakeEnvBootstrap(&res, &err);
    if (!bs) {
        std::fprintf(stderr, "bootstrap: %s\n", err.c_str());
        return 2;
    }
    const int W = bs->world(), rank = bs->rank();
    int ndev = 0;
    CK(cudaGetDeviceCount(&ndev));
    CK(cudaSetDevice(bs->local_rank() % ndev));
    ncclUniqueId id;
    if (rank == 0) NK(ncclGetUniqueId(&id));
    if (bs->broadcast(&id, sizeof(id), 0) != Result::Success) return 2;
    ncclComm_t comm;
    NK(ncclCommInitRank(&comm, W, id, rank));
    int version = 0;
    ncclGetVersion(&version);
    // Small messages rotate over buffers that together exceed the L2 (126 MB), as in bench/sweep.py.
    const size_t pool = std::max<size_t>(max_bytes, 320ull << 20);
    void *send, *recv;
    cudaStream_t st;
    CK(cudaMalloc(&send, pool));
    CK(cudaMalloc(&recv, pool));
    CK(cudaStreamCreate(&st));
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0));
    CK(cudaEventCreate(&e1));
    size_t pos = 0;
    while (pos <= dtypes.size()) {
        size_t comma = dtypes.find(',', pos);
        if (comma == std::string::npos) comma = dtypes.size();
        const std::string dname = dtypes.substr(pos, comma - pos);
        pos = comma + 1;
        Dtype dt;
        if (dname.empty() || !ParseDtype(dname.c_str(), &dt)) continue;
        const ncclDataType_t nd = dt == Dtype::FP32 ? ncclFloat : (dt == Dtype::FP16 ? ncclHalf : ncclBfloat16);
        CK(FillRandom(send, pool / DtypeSize(dt), dt, kDistUniformPm1, 1234 + rank, st));
        CK(cudaStreamSynchronize(st));
        for (size_t size = min_bytes; size <= max_bytes; size *= 2) {
            const size_t n = size / DtypeSize(dt);
            const size_t nbuf = size < (126ull << 20) ? std::max<size_t>(1, std::min<size_t>(256, (252ull << 20) / size)) : 1;
            const int iters = size <= (1u << 20) ? 200 : (size <= (64u << 20) ? 50 : 15);
            const int warm = size <= (16u << 20) ? 20 : 5;
            auto call = [&](int i) {
                const size_t off = (static_cast<size_t>(i) % nbuf) * size;
                NK(ncclAllReduce(static_cast<char*>(send) + off, static_cast<char*>(recv) + off, n, nd, ncclSum, comm, st));
            };
            for (int i = 0; i < warm; ++i) call(i);
            CK(cudaStreamSynchronize(st));
            bs->barrier();
            float ms = 0;
            const bool graph = size <= graph_max;
            if (graph) {
                cudaGraph_t g;
                cudaGraphExec_t ex;
                CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
                for (int i = 0; i < iters; ++i) call(warm + i);
                CK(cudaStreamEndCapture(st, &g));
                CK(cudaGraphInstantiate(&ex, g, 0));
                CK(cudaGraphLaunch(ex, st));
                CK(cudaStreamSynchronize(st));
                bs->barrier();
                CK(cudaEventRecord(e0, st));
                CK(cudaGraphLaunch(ex, st));
                CK(cudaEventRecord(e1, st));
                CK(cudaStreamSynchronize(st));
                cudaGraphExecDestroy(ex);
                cudaGraphDestroy(g);
            } else {
                CK(cudaEventRecord(e0, st));
                for (int i = 0; i < iters; ++i) call(warm + i);
                CK(cudaEventRecord(e1, st));
                CK(cudaStreamSynchronize(st));
            }
            CK(cudaEventElapsedTime(&ms, e0, e1));
            double us = ms * 1e3 / iters;
            std::vector<double> all(W);
            if (bs->allgather(&us, all.data(), sizeof(double)) != Result::Success) return 4;
            for (double v : all) us = std::max(us, v);
            if (rank == 0) {
                std::printf("{\"impl\":\"nccl\",\"world\":%d,\"dtype\":\"%s\",\"bytes\":%zu,\"variant\":\"nccl\",\"us\":%.2f,"
                            "\"busbw_gbps\":%.2f,\"timing\":\"%s\",\"nccl_version\":%d}\n",
                            W, dname.c_str(), size, us, size * BusBwFactor(W) / us / 1e3, graph ? "graph" : "events", version);
                std::fflush(stdout);
            }
        }
    }
    cudaFree(send);
    cudaFree(recv);
    ncclCommDestroy(comm);
    return 0;
}
