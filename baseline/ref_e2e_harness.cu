// End-to-end harness around the UNMODIFIED reference: calls the reference's own
// public API (yali::Comm + yali::allreduce from its src/ops/allreduce.cuh) on two
// GPUs and, per step, copies both ranks' inputs from pinned host memory to the
// GPUs, runs the all-reduce and copies both results back.  Prints one line:
//   REF_E2E <dtype> <elements> <steps> <warmup> <avg_us_per_step> <kernel_only_avg_us>
// Only the timing loop is ours; no kernel, communicator or tuning of this
// repository is linked in.
#include <cuda_runtime.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "src/ops/allreduce.cuh"

#define CK(x)                                                                      \
    do {                                                                           \
        cudaError_t e_ = (x);                                                      \
        if (e_ != cudaSuccess) {                                                   \
            std::fprintf(stderr, "%s:%d %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            std::exit(1);                                                          \
        }                                                                          \
    } while (0)

int main(int argc, char** argv) {
    size_t elems = argc > 1 ? std::strtoull(argv[1], nullptr, 10) : 262144;
    int steps = argc > 2 ? std::atoi(argv[2]) : 20;
    int warmup = argc > 3 ? std::atoi(argv[3]) : 5;
    const size_t bytes = elems * sizeof(float);
    yali::Comm comm(0, 1);
    if (!comm.ok()) {
        std::fprintf(stderr, "reference Comm init failed\n");
        return 2;
    }
    float *send[2], *recv[2], *h_in[2], *h_out[2];
    cudaStream_t st[2];
    for (int g = 0; g < 2; ++g) {
        CK(cudaSetDevice(g));
        CK(cudaMalloc(&send[g], bytes));
        CK(cudaMalloc(&recv[g], bytes));
        CK(cudaMallocHost(&h_in[g], bytes));
        CK(cudaMallocHost(&h_out[g], bytes));
        for (size_t i = 0; i < elems; ++i) h_in[g][i] = static_cast<float>((i * 2654435761u + g) % 2001) / 1000.f - 1.f;
        CK(cudaStreamCreate(&st[g]));
    }
    auto step = [&](bool copies) {
        if (copies) {
            for (int g = 0; g < 2; ++g) {
                CK(cudaSetDevice(g));
                CK(cudaMemcpyAsync(send[g], h_in[g], bytes, cudaMemcpyHostToDevice, 0));
            }
        }
        CK(yali::allreduce(comm, send[0], recv[0], send[1], recv[1], elems));
        if (copies) {
            for (int g = 0; g < 2; ++g) {
                CK(cudaSetDevice(g));
                CK(cudaMemcpyAsync(h_out[g], recv[g], bytes, cudaMemcpyDeviceToHost, 0));
            }
            for (int g = 0; g < 2; ++g) {
                CK(cudaSetDevice(g));
                CK(cudaDeviceSynchronize());
            }
        }
    };
    double us[2];
    for (int pass = 0; pass < 2; ++pass) {
        const bool copies = pass == 0;
        for (int i = 0; i < warmup; ++i) step(copies);
        for (int g = 0; g < 2; ++g) {
            CK(cudaSetDevice(g));
            CK(cudaDeviceSynchronize());
        }
        auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < steps; ++i) step(copies);
        for (int g = 0; g < 2; ++g) {
            CK(cudaSetDevice(g));
            CK(cudaDeviceSynchronize());
        }
        auto t1 = std::chrono::steady_clock::now();
        us[pass] = std::chrono::duration<double, std::micro>(t1 - t0).count() / steps;
    }
    // correctness spot check
    double want = static_cast<double>(h_in[0][12345 % elems]) + h_in[1][12345 % elems];
    if (std::abs(h_out[0][12345 % elems] - want) > 1e-4) std::fprintf(stderr, "REF_E2E mismatch\n");
    std::printf("REF_E2E fp32 %zu %d %d %.3f %.3f\n", elems, steps, warmup, us[0], us[1]);
    return 0;
}
