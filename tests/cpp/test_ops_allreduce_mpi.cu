// Multi-process integration test of yali::MPIComm + yali::allreduce; start with
//   python -m yali_b200.launch -np 2 build/bin/test_ops_allreduce_mpi
// Each rank validates its result; rank 0 prints the verdict agreed by all ranks.
// Reference counterpart: tests/test_ops_allreduce_mpi.cu.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>

#include "ops/buffer_ops.h"
#include "ops/yali.h"

using namespace yali;

template <typename T>
static bool Run(MPIComm& comm, size_t n, Dtype dt, bool symmetric, bool stable) {
    T *send, *recv;
    if (symmetric) {
        send = static_cast<T*>(comm.alloc(n * sizeof(T)));
        recv = static_cast<T*>(comm.alloc(n * sizeof(T)));
        if (!send || !recv) return false;
    } else {
        cudaMalloc(&send, n * sizeof(T));
        cudaMalloc(&recv, n * sizeof(T));
    }
    FillRandom(send, n, dt, kDistUniformPm1, 1234 + comm.rank(), nullptr);
    cudaDeviceSynchronize();
    bool ok = allreduce(comm, send, recv, n, nullptr, stable) == cudaSuccess;
    ok = ok && ValidateRandomResult(recv, n, dt, dt, kDistUniformPm1, 1234, comm.world_size(), 1.0f, nullptr);
    if (!ok) std::printf("rank %d: case n=%zu dtype=%s symmetric=%d FAILED (%s)\n", comm.rank(), n, DtypeName(dt),
                         symmetric ? 1 : 0, comm.impl()->last_error().c_str());
    if (!symmetric) {
        cudaFree(send);
        cudaFree(recv);
    }
    return ok;
}

int main(int argc, char** argv) {
    CommOptions copt;
    copt.heap_bytes = 2ull << 30;  // room for the 128 MiB symmetric cases
    MPIComm comm(&argc, &argv, copt);
    if (!comm.ok()) return 2;
    int ok = 1;
    ok &= Run<float>(comm, 1024, Dtype::FP32, false, false);
    ok &= Run<float>(comm, 1 << 20, Dtype::FP32, false, false);
    ok &= Run<__half>(comm, 1 << 20, Dtype::FP16, false, true);
    ok &= Run<__nv_bfloat16>(comm, 1 << 20, Dtype::BF16, true, true);
    ok &= Run<float>(comm, 32u << 20, Dtype::FP32, true, true);          // 128 MiB, two-shot
    ok &= Run<__half>(comm, 64u << 20, Dtype::FP16, false, false);       // 128 MiB, staged
    ok &= Run<__nv_bfloat16>(comm, 64u << 20, Dtype::BF16, true, true);
    std::vector<int> all(comm.world_size());
    comm.impl()->bootstrap() ? (void)comm.impl()->bootstrap()->allgather(&ok, all.data(), sizeof(int)) : (void)(all[0] = ok);
    for (int v : all) ok &= v;
    comm.barrier();
    if (comm.rank() == 0) std::printf("test_ops_allreduce_mpi (%d ranks): %s\n", comm.world_size(), ok ? "PASSED" : "FAILED");
    return ok ? 0 : 1;
}
