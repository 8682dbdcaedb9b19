// Multi-process example on the C ABI alone: the program owns its buffers (cudaMalloc), maps
// every peer's input with yaliIpcExchangeBuffers and runs a kernel of its own that reads the
// peers' memory over NVLink, with host barriers (yaliMPCommBarrier) around the launch.
// This is the level the reference's multi-process example works at; most programs should
// use yali::MPIComm (simple_mpi.cu, multilane_mpi.cu), whose kernels synchronise on the
// device and need no host barrier per call.
// YALI_DTYPE / YALI_ELEMS / YALI_LANES select dtype, element count and lanes (CTA groups).
//
// Reference counterpart: examples/02_multi_process/01_allreduce/multilane_mpi.cu:69-187
// (environment knobs, yaliMPCommCreate, yaliIpcExchangeBuffers, barriers around the launch).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "comm/mp_comm.h"
#include "core/status.h"
#include "ops/buffer_ops.h"

using namespace yali;

struct Peers {
    const void* p[kMaxRanks];
};

template <typename T>
__device__ float load_f32(const T* p, size_t i);
template <>
__device__ float load_f32<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ float load_f32<__half>(const __half* p, size_t i) { return __half2float(p[i]); }
template <>
__device__ float load_f32<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
template <typename T>
__device__ T store_f32(float v);
template <>
__device__ float store_f32<float>(float v) { return v; }
template <>
__device__ __half store_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __nv_bfloat16 store_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Lane l (a group of CTAs) owns a contiguous part of the message; every rank reads all ranks'
// parts of its lanes and sums them in fp32 in rank order.
template <typename T>
__global__ void lanes_sum(Peers peers, int world, T* out, size_t n, int lanes, int ctas_per_lane) {
    const int lane = blockIdx.x % lanes, cta = blockIdx.x / lanes;
    const size_t per_lane = (n + lanes - 1) / lanes;
    const size_t lb = static_cast<size_t>(lane) * per_lane, le = lb + per_lane < n ? lb + per_lane : n;
    for (size_t i = lb + static_cast<size_t>(cta) * blockDim.x + threadIdx.x; i < le;
         i += static_cast<size_t>(ctas_per_lane) * blockDim.x) {
        float s = 0.f;
        for (int r = 0; r < world; ++r) s += load_f32<T>(static_cast<const T*>(peers.p[r]), i);
        out[i] = store_f32<T>(s);
    }
}

template <typename T>
static void launch(const Peers& peers, int world, void* out, size_t n, int lanes, cudaStream_t st) {
    const int ctas_per_lane = 8;
    lanes_sum<T><<<lanes * ctas_per_lane, 512, 0, st>>>(peers, world, static_cast<T*>(out), n, lanes, ctas_per_lane);
}

int main(int argc, char** argv) {
    YaliMPComm* comm = yaliMPCommCreate(&argc, &argv);
    if (!comm) return 1;
    const int rank = comm->rank, W = comm->worldSize;
    const size_t n = std::getenv("YALI_ELEMS") ? std::strtoull(std::getenv("YALI_ELEMS"), nullptr, 10) : (1u << 22);
    const int lanes = std::getenv("YALI_LANES") && std::atoi(std::getenv("YALI_LANES")) > 0
                          ? std::atoi(std::getenv("YALI_LANES"))
                          : 16;
    Dtype dt = Dtype::FP32;
    if (const char* e = std::getenv("YALI_DTYPE")) ParseDtype(e, &dt);
    const size_t bytes = n * DtypeSize(dt);
    void *send = nullptr, *recv = nullptr;
    if (cudaMalloc(&send, bytes) != cudaSuccess || cudaMalloc(&recv, bytes) != cudaSuccess) {
        std::printf("rank %d: cudaMalloc failed\n", rank);
        return 1;
    }
    FillRandom(send, n, dt, kDistUniformPm1, 1234 + rank, comm->stream);
    cudaStreamSynchronize(comm->stream);
    if (yaliIpcExchangeBuffers(comm, send, bytes) != 0) {
        std::printf("rank %d: buffer exchange failed\n", rank);
        return 1;
    }
    Peers peers;
    std::memset(&peers, 0, sizeof(peers));
    for (int r = 0; r < W; ++r) peers.p[r] = comm->peerPtrs[r];

    for (int it = 0; it < 4; ++it) {
        yaliMPCommBarrier(comm);  // every rank's input is final
        switch (dt) {
            case Dtype::FP32: launch<float>(peers, W, recv, n, lanes, comm->stream); break;
            case Dtype::FP16: launch<__half>(peers, W, recv, n, lanes, comm->stream); break;
            case Dtype::BF16: launch<__nv_bfloat16>(peers, W, recv, n, lanes, comm->stream); break;
        }
        yaliMPCommBarrier(comm);  // synchronises the stream, then the ranks: nobody rewrites an input a peer still reads
    }
    ValidateReport rep;
    const bool ok = ValidateRandomResult(recv, n, dt, dt, kDistUniformPm1, 1234, W, 1.0f, &rep);
    std::printf("rank %d: %s (%zu %s elements, %d lanes, max abs err %.3g)\n", rank, ok ? "OK" : "MISMATCH", n,
                DtypeName(dt), lanes, rep.max_abs_err);
    int mine = ok ? 1 : 0;
    std::vector<int> all(W, 0);
    yaliMPCommAllgather(comm, &mine, all.data(), sizeof(int));
    bool all_ok = true;
    for (int v : all) all_ok &= v != 0;
    yaliIpcCloseAll(comm);
    cudaFree(send);
    cudaFree(recv);
    if (rank == 0) std::printf("=== Example %s ===\n", all_ok ? "PASSED" : "FAILED");
    yaliMPCommDestroy(comm);
    return all_ok ? 0 : 1;
}
