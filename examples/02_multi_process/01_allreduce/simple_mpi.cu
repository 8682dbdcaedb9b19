// Smallest multi-process example: one GPU per process, yali::MPIComm + yali::allreduce.
//
//   make examples && python -m yali_b200.launch -np 2 build/bin/example_simple_mpi
//   (torchrun or an MPI launcher work too: the rendezvous reads their environment)
//
// Reference counterpart: examples/02_multi_process/01_allreduce/simple_mpi.cu.
#include <cuda_runtime.h>

#include <cstdio>

#include "ops/yali.h"

int main(int argc, char** argv) {
    yali::MPIComm comm(&argc, &argv);
    if (!comm.ok()) {
        std::printf("communicator setup failed\n");
        return 1;
    }
    const int rank = comm.rank();
    constexpr size_t N = 1 << 20;
    float *send, *recv;
    cudaMalloc(&send, N * sizeof(float));
    cudaMalloc(&recv, N * sizeof(float));
    const float seed = static_cast<float>(rank + 1);
    cudaMemset(send, 0, N * sizeof(float));
    cudaMemcpy(send, &seed, sizeof(float), cudaMemcpyHostToDevice);
    if (rank == 0) std::printf("=== yali-b200 multi-process all-reduce, world size %d ===\n", comm.world_size());

    cudaError_t err = yali::allreduce(comm, send, recv, N);  // recv = sum over ranks
    if (err != cudaSuccess) {
        std::printf("rank %d: allreduce failed: %s\n", rank, cudaGetErrorString(err));
        return 1;
    }
    float result = 0;
    cudaMemcpy(&result, recv, sizeof(float), cudaMemcpyDeviceToHost);
    const float expected = 0.5f * comm.world_size() * (comm.world_size() + 1);
    std::printf("rank %d: recv[0]=%.1f (expected %.1f)\n", rank, result, expected);
    cudaFree(send);
    cudaFree(recv);
    return result == expected ? 0 : 1;
}
