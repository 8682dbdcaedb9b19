// Smallest single-process example: one host thread, two GPUs, yali::allreduce.
//
//   make examples && CUDA_VISIBLE_DEVICES=0,1 build/bin/example_simple
//
// Reference counterpart: examples/01_single_process/01_allreduce/simple.cu.
#include <cuda_runtime.h>

#include <cstdio>

#include "ops/yali.h"

int main() {
    yali::Comm comm(0, 1);  // maps each GPU's heap on the other, enables peer access
    if (!comm.ok()) {
        std::printf("communicator setup failed: %s\n", comm.error().c_str());
        return 1;
    }
    constexpr size_t N = 1 << 20;
    float *send0, *recv0, *send1, *recv1;
    cudaSetDevice(0);
    cudaMalloc(&send0, N * sizeof(float));
    cudaMalloc(&recv0, N * sizeof(float));
    cudaSetDevice(1);
    cudaMalloc(&send1, N * sizeof(float));
    cudaMalloc(&recv1, N * sizeof(float));
    const float one = 1.0f, two = 2.0f;
    cudaSetDevice(0);
    cudaMemset(send0, 0, N * sizeof(float));
    cudaMemcpy(send0, &one, sizeof(float), cudaMemcpyHostToDevice);
    cudaSetDevice(1);
    cudaMemset(send1, 0, N * sizeof(float));
    cudaMemcpy(send1, &two, sizeof(float), cudaMemcpyHostToDevice);

    cudaError_t err = yali::allreduce(comm, send0, recv0, send1, recv1, N);  // recv = send0 + send1 on both GPUs
    if (err != cudaSuccess) {
        std::printf("allreduce failed: %s\n", cudaGetErrorString(err));
        return 1;
    }
    float r0 = 0, r1 = 0;
    cudaSetDevice(0);
    cudaMemcpy(&r0, recv0, sizeof(float), cudaMemcpyDeviceToHost);
    cudaSetDevice(1);
    cudaMemcpy(&r1, recv1, sizeof(float), cudaMemcpyDeviceToHost);
    std::printf("GPU0[0]=%.1f, GPU1[0]=%.1f (expected: 3.0, 3.0)\n", r0, r1);
    cudaSetDevice(0);
    cudaFree(send0);
    cudaFree(recv0);
    cudaSetDevice(1);
    cudaFree(send1);
    cudaFree(recv1);
    return (r0 == 3.0f && r1 == 3.0f) ? 0 : 1;
}
