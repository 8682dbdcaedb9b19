// Smallest single-process example: one host thread, two GPUs, yali::allreduce.
//
//   make examples && CUDA_VISIBLE_DEVICES=0,1 build/bin/example_simple
//
// Reference counterpart: examples/01_single_process/01_allreduce/simple.cu (same call, there
// only element 0 is checked; here every element is).
#include <cuda_runtime.h>

#include <cstdio>
#include <vector>

#include "ops/yali.h"

namespace {

constexpr size_t kElems = 1 << 20;

// Input and output of one GPU.  GPU g contributes g + 1 in every element.
struct GpuBuffers {
    int gpu = 0;
    float* in = nullptr;
    float* out = nullptr;

    bool Create(int g) {
        gpu = g;
        const std::vector<float> host(kElems, static_cast<float>(g + 1));
        return cudaSetDevice(g) == cudaSuccess && cudaMalloc(&in, kElems * sizeof(float)) == cudaSuccess &&
               cudaMalloc(&out, kElems * sizeof(float)) == cudaSuccess &&
               cudaMemcpy(in, host.data(), kElems * sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess;
    }
    // Number of elements of `out` that differ from `want`, and the first element for the printout.
    size_t Mismatches(float want, float* first) const {
        std::vector<float> host(kElems);
        cudaSetDevice(gpu);
        cudaMemcpy(host.data(), out, kElems * sizeof(float), cudaMemcpyDeviceToHost);
        *first = host[0];
        size_t bad = 0;
        for (float v : host) bad += v != want;
        return bad;
    }
    void Destroy() {
        cudaSetDevice(gpu);
        cudaFree(in);
        cudaFree(out);
    }
};

}  // namespace

int main() {
    yali::Comm comm(0, 1);  // maps each GPU's heap on the other, enables peer access
    if (!comm.ok()) {
        std::printf("communicator setup failed: %s\n", comm.error().c_str());
        return 1;
    }
    GpuBuffers a, b;
    if (!a.Create(0) || !b.Create(1)) {
        std::printf("allocation failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        return 1;
    }
    // out = a.in + b.in on both GPUs; returns when both have finished.
    const cudaError_t status = yali::allreduce(comm, a.in, a.out, b.in, b.out, kElems);
    if (status != cudaSuccess) {
        std::printf("allreduce failed: %s (%s)\n", cudaGetErrorString(status), comm.error().c_str());
        return 1;
    }
    float first_a = 0.f, first_b = 0.f;
    const size_t bad = a.Mismatches(3.0f, &first_a) + b.Mismatches(3.0f, &first_b);
    std::printf("GPU0[0]=%.1f, GPU1[0]=%.1f (expected: 3.0, 3.0); %zu of %zu elements wrong\n", first_a, first_b, bad,
                2 * kElems);
    a.Destroy();
    b.Destroy();
    return bad == 0 ? 0 : 1;
}
