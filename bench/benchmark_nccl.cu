// benchmark_nccl: the NCCL baseline with the same arguments, timing loop and result
// line as benchmark_yali (arguments that do not apply are accepted and ignored).
// One process, one communicator per GPU, ncclAllReduce inside a group per call.
//
// Parity: bench/benchmark_nccl.cu of the reference (two GPUs; argv elements calls
// timing dtype).  Here the argument order is benchmark_yali's so that one sweep
// drives both, and any number of GPUs up to 8 is accepted.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <nccl.h>

#include <chrono>

#include "bench_common.h"
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
        bench::Usage(argv[0], "NCCL all-reduce baseline (mode, lanes and symmetric are ignored).");
        return 0;
    }
    const int W = a.gpus;
    const size_t bytes = a.elements * DtypeSize(a.dtype);
    const ncclDataType_t nd = a.dtype == Dtype::FP32 ? ncclFloat : (a.dtype == Dtype::FP16 ? ncclHalf : ncclBfloat16);
    std::vector<int> devs(W);
    for (int i = 0; i < W; ++i) devs[i] = i;
    std::vector<ncclComm_t> comms(W);
    NK(ncclCommInitAll(comms.data(), W, devs.data()));
    std::vector<void*> send(W), recv(W);
    std::vector<cudaStream_t> st(W);
    for (int i = 0; i < W; ++i) {
        CK(cudaSetDevice(i));
        CK(cudaMalloc(&send[i], bytes ? bytes : 16));
        CK(cudaMalloc(&recv[i], bytes ? bytes : 16));
        CK(cudaStreamCreate(&st[i]));
        CK(FillRandom(send[i], a.elements, a.dtype, kDistUniformPm1, 1234 + i, st[i]));
        CK(cudaStreamSynchronize(st[i]));
    }
    auto call = [&]() {
        NK(ncclGroupStart());
        for (int i = 0; i < W; ++i) NK(ncclAllReduce(send[i], recv[i], a.elements, nd, ncclSum, comms[i], st[i]));
        NK(ncclGroupEnd());
    };
    auto sync_all = [&]() {
        for (int i = 0; i < W; ++i) {
            CK(cudaSetDevice(i));
            CK(cudaStreamSynchronize(st[i]));
        }
    };
    int ver = 0;
    ncclGetVersion(&ver);
    std::printf("NCCL %d AllReduce Benchmark (%s) ranks=%d %zu elements (%.2f MB) calls=%d warmup=%d timing=%s\n", ver,
                DtypeName(a.dtype), W, a.elements, bytes / 1e6, a.calls, a.warmup, bench::TimingModeName(a.timing));
    for (int i = 0; i < a.warmup; ++i) call();
    sync_all();
    double avg_us = 0;
    bench::Stats per_call;
    if (a.timing == bench::TimingMode::CudaEvents) {
        std::vector<std::vector<cudaEvent_t>> ev(W, std::vector<cudaEvent_t>(a.calls + 1));
        for (int i = 0; i < W; ++i) {
            CK(cudaSetDevice(i));
            for (auto& e : ev[i]) CK(cudaEventCreate(&e));
            CK(cudaEventRecord(ev[i][0], st[i]));
        }
        for (int c = 0; c < a.calls; ++c) {
            call();
            for (int i = 0; i < W; ++i) {
                CK(cudaSetDevice(i));
                CK(cudaEventRecord(ev[i][c + 1], st[i]));
            }
        }
        sync_all();
        std::vector<double> per(a.calls, 0.0);
        double total = 0;
        for (int i = 0; i < W; ++i) {
            float ms = 0;
            CK(cudaEventElapsedTime(&ms, ev[i][0], ev[i][a.calls]));
            total = std::max(total, static_cast<double>(ms) * 1e3);
            for (int c = 0; c < a.calls; ++c) {
                CK(cudaEventElapsedTime(&ms, ev[i][c], ev[i][c + 1]));
                per[c] = std::max(per[c], static_cast<double>(ms) * 1e3);
            }
        }
        per_call = bench::Summarise(per);
        (void)total;
        // Average from a second batch with one event pair per rank (events between calls
        // keep consecutive launches from overlapping and would inflate the average).
        std::vector<cudaEvent_t> b0(W), b1(W);
        for (int i = 0; i < W; ++i) {
            CK(cudaSetDevice(i));
            CK(cudaEventCreate(&b0[i]));
            CK(cudaEventCreate(&b1[i]));
            CK(cudaEventRecord(b0[i], st[i]));
        }
        for (int c = 0; c < a.calls; ++c) call();
        for (int i = 0; i < W; ++i) {
            CK(cudaSetDevice(i));
            CK(cudaEventRecord(b1[i], st[i]));
        }
        sync_all();
        double batch = 0;
        for (int i = 0; i < W; ++i) {
            float ms = 0;
            CK(cudaEventElapsedTime(&ms, b0[i], b1[i]));
            batch = std::max(batch, static_cast<double>(ms) * 1e3);
        }
        avg_us = batch / a.calls;
    } else if (a.timing == bench::TimingMode::Throughput) {
        auto t0 = std::chrono::steady_clock::now();
        for (int c = 0; c < a.calls; ++c) call();
        sync_all();
        avg_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count() / a.calls;
    } else {
        std::vector<double> per(a.calls);
        auto t0 = std::chrono::steady_clock::now();
        for (int c = 0; c < a.calls; ++c) {
            auto s0 = std::chrono::steady_clock::now();
            call();
            sync_all();
            per[c] = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - s0).count();
        }
        avg_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count() / a.calls;
        per_call = bench::Summarise(per);
    }
    char extra[64];
    std::snprintf(extra, sizeof(extra), "\"nccl_version\":%d", ver);
    bench::Report("NCCL", "AllReduce", a, W, avg_us, &per_call, extra);
    int rc = 0;
    if (a.verify) {
        bool all_ok = true;
        for (int i = 0; i < W; ++i) {
            CK(cudaSetDevice(i));
            all_ok &= ValidateRandomResult(recv[i], a.elements, a.dtype, a.dtype, kDistUniformPm1, 1234, W, 1.0f, nullptr);
        }
        std::printf("Correctness: %s\n", all_ok ? "PASSED" : "FAILED");
        rc = all_ok ? 0 : 1;
    }
    for (int i = 0; i < W; ++i) {
        cudaSetDevice(i);
        cudaFree(send[i]);
        cudaFree(recv[i]);
        ncclCommDestroy(comms[i]);
    }
    return rc;
}
