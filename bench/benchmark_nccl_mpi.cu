// benchmark_nccl_mpi: the NCCL baseline with one process per GPU.  The unique id is
// broadcast over this library's bootstrap (no MPI needed); arguments, timing and the
// result line are those of benchmark_yali_mpi.
//
// Parity: bench/benchmark_nccl_mpi.cu of the reference (MPI_Bcast of ncclUniqueId,
// one ncclAllReduce per iteration, max over ranks).
#include <cuda_runtime.h>
#include <nccl.h>

#include <chrono>

#include "bench_common.h"
#include "comm/bootstrap.h"
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
    bench::Args a = bench::Parse(argc, argv);
    if (a.help) {
        bench::Usage(argv[0], "NCCL baseline, one process per GPU (launch with python -m yali_b200.launch).");
        return 0;
    }
    Result res;
    std::string err;
    std::unique_ptr<Bootstrap> bs = MakeEnvBootstrap(&res, &err);
    if (!bs) {
        std::fprintf(stderr, "bootstrap: %s\n", err.c_str());
        return 2;
    }
    const int W = bs->world(), rank = bs->rank();
    a.gpus = W;
    int ndev = 0;
    CK(cudaGetDeviceCount(&ndev));
    CK(cudaSetDevice(bs->local_rank() % ndev));
    ncclUniqueId id;
    if (rank == 0) NK(ncclGetUniqueId(&id));
    if (bs->broadcast(&id, sizeof(id), 0) != Result::Success) return 2;
    ncclComm_t comm;
    NK(ncclCommInitRank(&comm, W, id, rank));
    const size_t bytes = a.elements * DtypeSize(a.dtype);
    const ncclDataType_t nd = a.dtype == Dtype::FP32 ? ncclFloat : (a.dtype == Dtype::FP16 ? ncclHalf : ncclBfloat16);
    void *send, *recv;
    cudaStream_t st;
    CK(cudaMalloc(&send, bytes ? bytes : 16));
    CK(cudaMalloc(&recv, bytes ? bytes : 16));
    CK(cudaStreamCreate(&st));
    CK(FillRandom(send, a.elements, a.dtype, kDistUniformPm1, 1234 + rank, st));
    CK(cudaStreamSynchronize(st));
    auto call = [&]() { NK(ncclAllReduce(send, recv, a.elements, nd, ncclSum, comm, st)); };
    for (int i = 0; i < a.warmup; ++i) call();
    CK(cudaStreamSynchronize(st));
    bs->barrier();
    std::vector<double> per(a.calls, 0.0);
    double total_us = 0;
    if (a.timing == bench::TimingMode::CudaEvents) {
        std::vector<cudaEvent_t> ev(a.calls + 1);
        for (auto& e : ev) CK(cudaEventCreate(&e));
        CK(cudaEventRecord(ev[0], st));
        for (int c = 0; c < a.calls; ++c) {
            call();
            CK(cudaEventRecord(ev[c + 1], st));
        }
        CK(cudaStreamSynchronize(st));
        float ms = 0;
        CK(cudaEventElapsedTime(&ms, ev[0], ev[a.calls]));
        total_us = ms * 1e3;
        for (int c = 0; c < a.calls; ++c) {
            CK(cudaEventElapsedTime(&ms, ev[c], ev[c + 1]));
            per[c] = ms * 1e3;
        }
        // Average from a second batch with one event pair (see benchmark_yali.cu).
        bs->barrier();
        cudaEvent_t b0, b1;
        CK(cudaEventCreate(&b0));
        CK(cudaEventCreate(&b1));
        CK(cudaEventRecord(b0, st));
        for (int c = 0; c < a.calls; ++c) call();
        CK(cudaEventRecord(b1, st));
        CK(cudaStreamSynchronize(st));
        CK(cudaEventElapsedTime(&ms, b0, b1));
        total_us = ms * 1e3;
    } else if (a.timing == bench::TimingMode::Graph) {
        // All calls in one CUDA graph: no host launch work between the kernels.  Two replays, the
        // second one is timed.
        cudaGraph_t graph;
        cudaGraphExec_t exec;
        CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        for (int c = 0; c < a.calls; ++c) call();
        CK(cudaStreamEndCapture(st, &graph));
        CK(cudaGraphInstantiate(&exec, graph, 0));
        cudaEvent_t g0, g1;
        CK(cudaEventCreate(&g0));
        CK(cudaEventCreate(&g1));
        CK(cudaGraphLaunch(exec, st));
        CK(cudaStreamSynchronize(st));
        CK(cudaEventRecord(g0, st));
        CK(cudaGraphLaunch(exec, st));
        CK(cudaEventRecord(g1, st));
        CK(cudaStreamSynchronize(st));
        float ms = 0;
        CK(cudaEventElapsedTime(&ms, g0, g1));
        total_us = ms * 1e3;
        cudaGraphExecDestroy(exec);
        cudaGraphDestroy(graph);
    } else {
        auto t0 = std::chrono::steady_clock::now();
        for (int c = 0; c < a.calls; ++c) {
            auto s0 = std::chrono::steady_clock::now();
            call();
            if (a.timing == bench::TimingMode::Latency) {
                CK(cudaStreamSynchronize(st));
                per[c] = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - s0).count();
            }
        }
        CK(cudaStreamSynchronize(st));
        total_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
    }
    bs->barrier();
    std::vector<double> mine(per);
    mine.push_back(total_us);
    std::vector<double> all(mine.size() * W);
    if (bs->allgather(mine.data(), all.data(), mine.size() * sizeof(double)) != Result::Success) return 4;
    for (size_t c = 0; c < mine.size(); ++c) {
        double m = 0;
        for (int r = 0; r < W; ++r) m = std::max(m, all[r * mine.size() + c]);
        if (c < per.size()) per[c] = m;
        else total_us = m;
    }
    int ok = 1;
    if (a.verify) ok = ValidateRandomResult(recv, a.elements, a.dtype, a.dtype, kDistUniformPm1, 1234, W, 1.0f, nullptr);
    if (rank == 0) {
        int ver = 0;
        ncclGetVersion(&ver);
        bench::Stats s = (a.timing == bench::TimingMode::Throughput || a.timing == bench::TimingMode::Graph)
                             ? bench::Stats()
                             : bench::Summarise(per);
        char extra[96];
        std::snprintf(extra, sizeof(extra), "\"nccl_version\":%d,\"processes\":%d", ver, W);
        bench::Report("NCCL", "AllReduce", a, W, total_us / a.calls, &s, extra);
        if (a.verify) std::printf("Correctness: %s\n", ok ? "PASSED" : "FAILED");
    }
    cudaFree(send);
    cudaFree(recv);
    ncclCommDestroy(comm);
    return ok ? 0 : 1;
}
